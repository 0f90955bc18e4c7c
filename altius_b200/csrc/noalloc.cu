// altius_cuda_reduce_max_noalloc: whole-tensor maximum without any allocation.
//
// Who this is for: code that must not allocate device memory at the moment it
// needs the result -- a host callback or a real-time loop that cannot afford
// the implicit device synchronisation and the unbounded latency of cudaMalloc /
// cudaFree, a plug-in running inside a host whose memory pool is owned by
// someone else, or a section of a program that is being recorded into a CUDA
// graph, where allocation calls are not permitted. A session (altius_cuda_create)
// owns an arena and is the normal way to run a graph; this entry point is the
// escape hatch for the single reduction such callers tend to need (a global
// max, e.g. for a scale factor), with caller-owned input and output.
//
// The two-stage reduction needs a place for the per-block partial maxima. Here
// that place is a fixed array in the library's device image instead of arena
// memory, so:
//   * its size is fixed: kMaxPartials floats (64 KB). Every GPU that loads the
//     library carries those 64 KB until the process exits;
//   * it bounds the input: one partial per kElemsPerBlock elements, i.e. at most
//     kMaxPartials * kElemsPerBlock = 67,108,864 elements (256 MiB of f32).
//     Longer inputs are refused with AC_ERR_INVALID and a message;
//   * all calls on one GPU share it. Two calls whose kernels can overlap (different
//     streams, or different host threads on the same GPU) race on the partials
//     and may both return garbage: serialise them. The array keeps whatever the
//     previous call left; that is harmless because stage 1 overwrites every slot
//     that stage 2 of the same call reads, so nothing has to start from zero.
//
// Host code cannot use the array's name as a pointer: on the host the symbol is
// only a handle. The device address is looked up with cudaGetSymbolAddress, once
// per device, on the first call made while that device is current, and cached.
// That first call should happen before any stream capture begins (the lookup is
// not a stream operation); later calls only launch the two kernels.
#include <cuda_runtime.h>
#include <math_constants.h>

#include <mutex>
#include <string>

#include "../../include/altius_session_cuda.h"

namespace ac {
void set_thread_error(const std::string& msg);   // session.cu: feeds altius_cuda_last_error(NULL)
}

namespace {

constexpr int kThreads = 256;
constexpr int kElemsPerBlock = 4096;
constexpr int kMaxPartials = 16384;
constexpr int kMaxDevices = 64;

static __device__ __align__(256) float g_noalloc_partials[kMaxPartials];

__device__ __forceinline__ float block_max(float v, float* sm) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    v = threadIdx.x < kThreads / 32 ? sm[threadIdx.x] : -CUDART_INF_F;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  }
  return v;
}

// Stage 1: block b owns elements [b * kElemsPerBlock, (b + 1) * kElemsPerBlock) and writes
// exactly one partial, partials[b].
__global__ void __launch_bounds__(kThreads) noalloc_max_stage1(const float* __restrict__ x, int64_t n,
                                                               float* __restrict__ partials) {
  __shared__ float sm[kThreads / 32];
  const int64_t lo = (int64_t)blockIdx.x * kElemsPerBlock;
  const int64_t hi = lo + kElemsPerBlock < n ? lo + kElemsPerBlock : n;
  float acc = -CUDART_INF_F;
  for (int64_t i = lo + threadIdx.x; i < hi; i += kThreads) acc = fmaxf(__ldg(x + i), acc);
  acc = block_max(acc, sm);
  if (threadIdx.x == 0) partials[blockIdx.x] = acc;
}

// Stage 2: one block folds the `count` partials written by stage 1 of the same call.
__global__ void __launch_bounds__(kThreads) noalloc_max_stage2(const float* __restrict__ partials, int count,
                                                               float* __restrict__ out) {
  __shared__ float sm[kThreads / 32];
  float acc = -CUDART_INF_F;
  for (int i = threadIdx.x; i < count; i += kThreads) acc = fmaxf(partials[i], acc);
  acc = block_max(acc, sm);
  if (threadIdx.x == 0) out[0] = acc;
}

std::mutex g_setup_mutex;
float* g_scratch_ptr[kMaxDevices] = {nullptr};

}  // namespace

extern "C" int altius_cuda_reduce_max_noalloc(const float* d_x, int64_t n, float* d_out, void* stream) {
  if (!d_x || !d_out) {
    ac::set_thread_error("reduce_max_noalloc: null pointer");
    return AC_ERR_INVALID;
  }
  if (n <= 0) {
    ac::set_thread_error("reduce_max_noalloc: the maximum of an empty tensor is undefined");
    return AC_ERR_INVALID;
  }
  const int64_t max_elems = (int64_t)kMaxPartials * kElemsPerBlock;
  if (n > max_elems) {
    ac::set_thread_error("reduce_max_noalloc: " + std::to_string(n) + " elements exceed the fixed scratch (" +
                         std::to_string(max_elems) + " elements at most); use a session for larger tensors");
    return AC_ERR_INVALID;
  }
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    ac::set_thread_error(std::string("reduce_max_noalloc: no current device: ") +
                         (e != cudaSuccess ? cudaGetErrorString(e) : "ordinal out of range"));
    return AC_ERR_NO_DEVICE;
  }
  float* scratch = nullptr;
  {
    // Once per device, with that device current: resolve the array's device address.
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_scratch_ptr[dev]) {
      float* p = nullptr;
      e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_partials);
      if (e != cudaSuccess || !p) {
        ac::set_thread_error(std::string("reduce_max_noalloc: cudaGetSymbolAddress: ") + cudaGetErrorString(e));
        return AC_ERR_CUDA;
      }
      g_scratch_ptr[dev] = p;
    }
    scratch = g_scratch_ptr[dev];
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int blocks = (int)((n + kElemsPerBlock - 1) / kElemsPerBlock);
  noalloc_max_stage1<<<blocks, kThreads, 0, st>>>(d_x, n, scratch);
  noalloc_max_stage2<<<1, kThreads, 0, st>>>(scratch, blocks, d_out);
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    ac::set_thread_error(std::string("reduce_max_noalloc: launch: ") + cudaGetErrorString(e));
    return AC_ERR_CUDA;
  }
  return AC_OK;
}
