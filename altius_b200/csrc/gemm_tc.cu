// Tensor-core GEMM for sm_100a: tcgen05.mma (kind::tf32) with the accumulator
// in tensor memory, operands staged in shared memory by TMA, 3xTF32 split for
// fp32 fidelity.
//
//   C[b] = epilogue( A[b] (M x K, K contiguous) * B[b]^T (B stored N x K, K contiguous) )
//
// It replaces the cblas_sgemm the reference calls for MatMul / Gemm / Conv2d
// (crates/session_interpreter/src/gemm.rs:36-51, session.rs:621-794,
// conv2d.rs:145-209). Every fp32 operand x is split into x_hi = x rounded to
// TF32 (round to nearest) and x_lo = (x - x_hi) rounded to TF32; x - x_hi is
// exact in fp32. Each product is evaluated as a_lo*b_hi + a_hi*b_lo + a_hi*b_hi
// with fp32 accumulation in TMEM; the dropped a_lo*b_lo term and the rounding
// of x_lo are each below 2^-22 relative.
//
// One CTA computes one 128 x BN tile:
//   warp 4      TMA producer: one elected thread issues cp.async.bulk.tensor
//               loads (128B-swizzled boxes of 32 floats along K) into a ring of
//               stages, completion on an mbarrier per stage;
//   warps 0-3   splitters: rewrite the A tile as x_hi in place and write x_lo
//               beside it (the same for the B tile unless B is a constant whose
//               split was prepared at load time and arrives by TMA), then
//               the epilogue: tcgen05.ld of the accumulator, bias / activation
//               / residual, global stores;
//   warp 5      one thread issues the tcgen05.mma stream and tcgen05.commit.
// Every mbarrier wait is bounded: on expiry the kernel records a code in the
// error word, drains, frees its tensor memory and returns.
#include <cuda.h>

#include <mutex>

#include "kernels.h"
#include "ref_math.cuh"

namespace ac {
namespace {

constexpr int BM = 128;
constexpr int BK = 32;                       // floats: one 128-byte swizzle row
constexpr int kSplitThreads = 128;
constexpr int kThreads = 192;
constexpr uint32_t kWaitLimit = 1u << 24;    // polls before a wait gives up

enum TcMode { TC_3X_BLO_TMA = 0, TC_3X_SPLIT_B = 1, TC_1X = 2 };

struct TcEpilogue {
  int m, n;
  float* c; long long ldc, sc;
  float alpha, beta;
  const float* cin; long long ldcin, scin;
  const float* bias_n; const float* bias_m; float bias_scale;
  int act; float act_alpha, act_beta;
  const float* res; long long ldres, sres;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
// Bounded wait on the phase with the given parity. Returns false on expiry.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t i = 0; i < kWaitLimit; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(addr), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int x,
                                            int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tc_mma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_ld_32x32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]),
        "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]),
        "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]),
        "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor for a K-major tile whose rows are 128 bytes
// (32 floats), stored row after row with the 128-byte swizzle: 8-row groups are
// 1024 bytes apart (stride byte offset), the leading byte offset is unused.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);        // start address
  d |= (uint64_t)1 << 16;                        // leading byte offset (ignored for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset
  d |= (uint64_t)1 << 46;                        // descriptor version for this architecture
  d |= (uint64_t)2 << 61;                        // 128-byte swizzle
  return d;
}

__device__ __forceinline__ float round_tf32(float x) {
  uint32_t u;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
  return __uint_as_float(u);
}
// hi = rn_tf32(x), lo = rn_tf32(x - hi), for 4 packed floats.
__device__ __forceinline__ void tf32_split(float4 v, float4& hi, float4& lo) {
  hi.x = round_tf32(v.x); lo.x = round_tf32(__fsub_rn(v.x, hi.x));
  hi.y = round_tf32(v.y); lo.y = round_tf32(__fsub_rn(v.y, hi.y));
  hi.z = round_tf32(v.z); lo.z = round_tf32(__fsub_rn(v.z, hi.z));
  hi.w = round_tf32(v.w); lo.w = round_tf32(__fsub_rn(v.w, hi.w));
}

template <int BN>
struct TcSmem {
  static constexpr int kABytes = BM * BK * 4;
  static constexpr int kBBytes = BN * BK * 4;
  static constexpr int kStageBytes = 2 * kABytes + 2 * kBBytes;
  static constexpr int kStages = BN >= 256 ? 2 : (BN >= 128 ? 3 : 4);
  static constexpr int kDynBytes = kStages * kStageBytes + 1024 /*alignment*/ + 256 /*barriers*/;
};

template <int BN, int MODE>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
               const __grid_constant__ CUtensorMap tm_blo, TcEpilogue ep, int num_kb, int b_batched,
               int* err) {
  using L = TcSmem<BN>;
  constexpr int S = L::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S * L::kStageBytes);
  uint64_t* full = bars;            // TMA bytes landed
  uint64_t* ready = bars + S;       // remainders written
  uint64_t* empty = bars + 2 * S;   // MMAs that read the stage have completed
  uint64_t* accfull = bars + 3 * S; // accumulator complete
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * S + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BN, m0 = blockIdx.y * BM, bz = blockIdx.z;

  auto a_raw = [&](int s) { return smem + s * L::kStageBytes; };
  auto a_lo = [&](int s) { return smem + s * L::kStageBytes + L::kABytes; };
  auto b_raw = [&](int s) { return smem + s * L::kStageBytes + 2 * L::kABytes; };
  auto b_lo = [&](int s) { return smem + s * L::kStageBytes + 2 * L::kABytes + L::kBBytes; };

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&ready[s], kSplitThreads);
      mbar_init(&empty[s], 1);
    }
    mbar_init(accfull, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"((uint32_t)BN));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      const uint32_t bytes = L::kABytes + L::kBBytes + (MODE == TC_3X_BLO_TMA ? L::kBBytes : 0);
      const int bzb = b_batched ? bz : 0;
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % S;
        const uint32_t ph = (kb / S) & 1;
        if (!mbar_wait(&empty[s], ph ^ 1)) { atomicExch(err, 1); *abort_flag = 1; break; }
        mbar_arrive_expect_tx(&full[s], bytes);
        tma_load_3d(a_raw(s), &tm_a, &full[s], kb * BK, m0, bz);
        tma_load_3d(b_raw(s), &tm_b, &full[s], kb * BK, n0, bzb);
        if (MODE == TC_3X_BLO_TMA) tma_load_3d(b_lo(s), &tm_blo, &full[s], kb * BK, n0, bzb);
      }
    }
  } else if (warp == 5) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      // Instruction descriptor: fp32 accumulator, TF32 A and B, both K-major, N = BN, M = 128.
      const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(BN >> 3) << 17) |
                             ((uint32_t)(BM >> 4) << 24);
      bool ok = true;
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        const int s = kb % S;
        const uint32_t ph = (kb / S) & 1;
        ok = mbar_wait(MODE == TC_1X ? &full[s] : &ready[s], ph);
        if (!ok) { atomicExch(err, 2); *abort_flag = 1; break; }
        tc_fence_after();
        const uint64_t da = make_smem_desc(smem_u32(a_raw(s)));
        const uint64_t dal = make_smem_desc(smem_u32(a_lo(s)));
        const uint64_t db = make_smem_desc(smem_u32(b_raw(s)));
        const uint64_t dbl = make_smem_desc(smem_u32(b_lo(s)));
#pragma unroll
        for (int kk = 0; kk < BK / 8; ++kk) {
          const uint64_t off = (uint64_t)(kk * 32 >> 4);  // 8 floats = 32 bytes along K
          const uint32_t acc = (kb > 0 || kk > 0) ? 1u : 0u;
          if (MODE == TC_1X) {
            tc_mma_tf32(tmem_base, da + off, db + off, idesc, acc);
          } else {
            tc_mma_tf32(tmem_base, dal + off, db + off, idesc, acc);   // a_lo * b_hi
            tc_mma_tf32(tmem_base, da + off, dbl + off, idesc, 1u);    // a_hi * b_lo
            tc_mma_tf32(tmem_base, da + off, db + off, idesc, 1u);     // a_hi * b_hi
          }
        }
        tc_commit(&empty[s]);
      }
      tc_commit(accfull);
    }
  } else {
    // ---------------- splitters, then epilogue (warps 0-3) ----------------
    const int t = threadIdx.x;  // 0..127
    bool ok = true;
    if (MODE != TC_1X) {
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        const int s = kb % S;
        const uint32_t ph = (kb / S) & 1;
        ok = mbar_wait(&full[s], ph);
        if (!ok) { atomicExch(err, 3); *abort_flag = 1; break; }
        float4* src = reinterpret_cast<float4*>(a_raw(s));
        float4* dst = reinterpret_cast<float4*>(a_lo(s));
#pragma unroll
        for (int i = 0; i < L::kABytes / 16 / kSplitThreads; ++i) {
          float4 hi, lo;
          tf32_split(src[i * kSplitThreads + t], hi, lo);
          src[i * kSplitThreads + t] = hi;
          dst[i * kSplitThreads + t] = lo;
        }
        if (MODE == TC_3X_SPLIT_B) {
          float4* sb = reinterpret_cast<float4*>(b_raw(s));
          float4* dbp = reinterpret_cast<float4*>(b_lo(s));
#pragma unroll
          for (int i = 0; i < L::kBBytes / 16 / kSplitThreads; ++i) {
            float4 hi, lo;
            tf32_split(sb[i * kSplitThreads + t], hi, lo);
            sb[i * kSplitThreads + t] = hi;
            dbp[i * kSplitThreads + t] = lo;
          }
        }
        fence_proxy_async();
        mbar_arrive(&ready[s]);
      }
    }
    if (ok) ok = mbar_wait(accfull, 0);
    if (!ok) { atomicExch(err, 4); *abort_flag = 1; }
    tc_fence_after();
    if (ok && *abort_flag == 0) {
      const int row = m0 + warp * 32 + lane;
      float* c = ep.c + (long long)bz * ep.sc;
      const float* cin = ep.cin ? ep.cin + (long long)bz * ep.scin : nullptr;
      const float* res = ep.res ? ep.res + (long long)bz * ep.sres : nullptr;
      const bool vec_ok = (ep.ldc % 4) == 0 && ((reinterpret_cast<uintptr_t>(c) & 15) == 0);
      const float bm = (ep.bias_m && row < ep.m)
                           ? (ep.bias_scale == 1.f ? __ldg(ep.bias_m + row)
                                                   : __fmul_rn(ep.bias_scale, __ldg(ep.bias_m + row)))
                           : 0.f;
#pragma unroll 1
      for (int cc = 0; cc < BN / 32; ++cc) {
        const int col0 = n0 + cc * 32;
        if (col0 >= ep.n) break;                 // uniform across the warp
        uint32_t v[32];
        tc_ld_32x32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(cc * 32), v);
        if (row < ep.m) {
          float o[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int col = col0 + j;
            float x = __uint_as_float(v[j]);
            if (col < ep.n) {
              if (ep.alpha != 1.f) x = __fmul_rn(ep.alpha, x);
              if (cin && ep.beta != 0.f) {
                const float cv = __ldg(cin + (long long)row * ep.ldcin + col);
                x = __fadd_rn(ep.beta == 1.f ? cv : __fmul_rn(ep.beta, cv), x);
              }
              if (ep.bias_n) {
                const float bv = __ldg(ep.bias_n + col);
                x = __fadd_rn(x, ep.bias_scale == 1.f ? bv : __fmul_rn(ep.bias_scale, bv));
              }
              if (ep.bias_m) x = __fadd_rn(x, bm);
              x = apply_act(ep.act, x, ep.act_alpha, ep.act_beta);
              if (res) x = __fadd_rn(x, __ldg(res + (long long)row * ep.ldres + col));
            }
            o[j] = x;
          }
          float* crow = c + (long long)row * ep.ldc + col0;
          if (vec_ok && col0 + 32 <= ep.n) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              *reinterpret_cast<float4*>(crow + j) = make_float4(o[j], o[j + 1], o[j + 2], o[j + 3]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < ep.n) crow[j] = o[j];
          }
        }
      }
    }
    tc_fence_before();
  }

  // ---------------- teardown ----------------
  __syncthreads();
  if (*abort_flag != 0 && warp == 4 && lane == 0) {
    // Give copies that may still be in flight a bounded time to land before the
    // shared memory is released.
    for (int s = 0; s < S; ++s) {
      (void)mbar_wait(&full[s], 0);
      (void)mbar_wait(&full[s], 1);
    }
  }
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)BN));
  }
}

// hi / lo split of a whole tensor (constant operands, once at load).
__global__ void tf32_split_kernel(const float* __restrict__ x, float* __restrict__ hi,
                                  float* __restrict__ lo, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    const float v = __ldg(x + i);
    const float h = round_tf32(v);
    hi[i] = h;
    lo[i] = round_tf32(__fsub_rn(v, h));
  }
}

// ---- host side ---------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// 3-D map over a row-major [batch, rows, k] f32 tensor: box = 32 floats of K x box_rows rows.
bool make_map(CUtensorMap* map, const float* base, int64_t k, int64_t rows, int64_t batch, int64_t ld,
              int64_t batch_stride, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {(cuuint64_t)k, (cuuint64_t)rows, (cuuint64_t)std::max<int64_t>(batch, 1)};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 4,
                           (cuuint64_t)(batch > 1 && batch_stride > 0 ? batch_stride : rows * ld) * 4};
  cuuint32_t box[3] = {(cuuint32_t)BK, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN, int MODE>
cudaError_t launch_tc(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mbl,
                      const TcEpilogue& ep, int num_kb, int b_batched, int64_t batch, int* err,
                      cudaStream_t st) {
  using L = TcSmem<BN>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         L::kDynBytes);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  dim3 grid((unsigned)((ep.n + BN - 1) / BN), (unsigned)((ep.m + BM - 1) / BM), (unsigned)batch);
  gemm_tc_kernel<BN, MODE><<<grid, kThreads, L::kDynBytes, st>>>(ma, mb, mbl, ep, num_kb, b_batched, err);
  return cudaGetLastError();
}

}  // namespace

bool gemm_tc_supported(const GemmParams& q) {
  if (q.trans_a || !q.trans_b) return false;
  if (q.m <= 0 || q.n <= 0 || q.k <= 0 || q.batch <= 0 || q.batch > 65535) return false;
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (!al(q.a) || !al(q.b) || (q.lda % 4) || (q.ldb % 4)) return false;
  if (q.batch > 1 && ((q.stride_a % 4) || (q.stride_b % 4))) return false;
  if (q.batch > 1 && q.stride_a <= 0) return false;
  if (q.b_lo && (!al(q.b_lo))) return false;
  return encode_fn() != nullptr;
}

int gemm_tc_pick_bn(int64_t m, int64_t n, int64_t batch) {
  // Fewest waves over 148 SMs, weighted by the tile's cost; ties go to the wider tile.
  const int cands[3] = {256, 128, 64};
  int best = 256;
  double best_cost = 1e300;
  for (int bn : cands) {
    const int64_t tiles = ((m + BM - 1) / BM) * ((n + bn - 1) / bn) * batch;
    const double waves = (double)((tiles + 147) / 148);
    const double cost = waves * (bn + 40);   // + fixed per-tile overhead in the same unit
    if (cost < best_cost - 1e-9) { best_cost = cost; best = bn; }
  }
  return best;
}

cudaError_t launch_gemm_tc(const GemmParams& q, int mode, int* err_word, cudaStream_t st) {
  if (!gemm_tc_supported(q)) return cudaErrorInvalidValue;
  const int bn = gemm_tc_pick_bn(q.m, q.n, q.batch);
  CUtensorMap ma, mb, mbl;
  const int b_batched = (q.batch > 1 && q.stride_b > 0) ? 1 : 0;
  if (!make_map(&ma, q.a, q.k, q.m, q.batch, q.lda, q.stride_a, BM)) return cudaErrorInvalidValue;
  if (!make_map(&mb, q.b, q.k, q.n, b_batched ? q.batch : 1, q.ldb, q.stride_b, bn))
    return cudaErrorInvalidValue;
  int kmode = mode == 2 ? TC_1X : (q.b_lo ? TC_3X_BLO_TMA : TC_3X_SPLIT_B);
  if (kmode == TC_3X_BLO_TMA) {
    if (!make_map(&mbl, q.b_lo, q.k, q.n, b_batched ? q.batch : 1, q.ldb, q.stride_b, bn))
      return cudaErrorInvalidValue;
  } else {
    mbl = mb;
  }
  TcEpilogue ep;
  ep.m = (int)q.m; ep.n = (int)q.n;
  ep.c = q.c; ep.ldc = q.ldc; ep.sc = q.stride_c;
  ep.alpha = q.alpha; ep.beta = q.beta;
  ep.cin = q.beta != 0.f ? q.c_in : nullptr; ep.ldcin = q.ldc_in; ep.scin = q.stride_c_in;
  ep.bias_n = q.bias_n; ep.bias_m = q.bias_m; ep.bias_scale = q.bias_scale;
  ep.act = q.act; ep.act_alpha = q.act_alpha; ep.act_beta = q.act_beta;
  ep.res = q.residual; ep.ldres = q.ld_res; ep.sres = q.stride_res;
  const int num_kb = (int)((q.k + BK - 1) / BK);
#define AC_TC(BNV)                                                                                   \
  (kmode == TC_1X ? launch_tc<BNV, TC_1X>(ma, mb, mbl, ep, num_kb, b_batched, q.batch, err_word, st) \
   : kmode == TC_3X_BLO_TMA                                                                          \
       ? launch_tc<BNV, TC_3X_BLO_TMA>(ma, mb, mbl, ep, num_kb, b_batched, q.batch, err_word, st)    \
       : launch_tc<BNV, TC_3X_SPLIT_B>(ma, mb, mbl, ep, num_kb, b_batched, q.batch, err_word, st))
  if (bn == 256) return AC_TC(256);
  if (bn == 128) return AC_TC(128);
  return AC_TC(64);
#undef AC_TC
}

cudaError_t launch_tf32_split(const float* x, float* hi, float* lo, int64_t n, cudaStream_t st) {
  if (n == 0) return cudaSuccess;
  tf32_split_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(x, hi, lo, n);
  return cudaGetLastError();
}

}  // namespace ac
