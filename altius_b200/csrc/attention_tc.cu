// Fused multi-head attention core on the sm_100a tensor cores: one CTA per
// (image, head, block of 128 query rows),
//
//   S = (Q K^T) (* | /) scale ;  P = Softmax(S) ;  O = P V
//
// with both products issued as tcgen05.mma (kind::tf32, 3xTF32 split, fp32
// accumulators in tensor memory). It replaces the same operator chain as the
// CUDA-core kernel in attention.cu (Split / Reshape / Transpose / MatMul / Mul /
// Softmax / MatMul / Transpose / Reshape of crates/session_interpreter/src/
// session.rs:621-682, 990-1026, 1179-1278, 1488-1512) and reads Q, K, V in place
// from the [B, T, 3D] projection buffer.
//
// Shared memory holds every operand as K-major blocks of 16 floats per row with
// the 64-byte swizzle (the layout the GEMM kernel's TMA boxes have), each as a
// TF32-rounded `hi` copy and a `lo` copy of the remainder:
//   region KV : K [NS x 64] as 4 blocks; after S is complete it is overwritten by
//               V^T [64 x NS] as NS/16 blocks (V is transposed on the way in, so
//               that the second product also takes a K-major B operand);
//   region QP : Q [128 x 64] as 4 blocks; after S is complete it becomes a ring of
//               four P chunks [128 x 16].
// Tensor memory: S in columns [0, NS), O in columns [256, 320).
//
//   all 8 warps  stage Q and K (global -> registers -> split -> swizzled stores),
//                prefetch V into registers, and after S transpose-store V;
//   warp 4       one thread issues the MMAs and commits to mbarriers;
//   warps 0-3    one query row per thread (= tensor-memory lane): pass 1 row maximum
//                of the scaled scores, pass 2 e = exp(s - max) with the reference's
//                polynomial, running sum, e split into hi/lo and stored as the A
//                operand of the second product; finally O * (1 / sum) to global.
// P is fed unnormalised and O scaled by 1 / sum at the end (the reference
// normalises P first); the difference is a few ulp.
// Every mbarrier wait is bounded; on expiry the kernel records a code in the
// error word and runs to its end without touching the barrier again.
#include "kernels.h"
#include "ref_math.cuh"
#include "tc_common.cuh"

namespace ac {
namespace {

using namespace tc;

constexpr int HD = 64;                        // head dimension
constexpr int QM = 128;                       // query rows per CTA = tensor-memory lanes
constexpr int kAtThreads = 256;
constexpr int kSlots = 4;                     // P ring depth
constexpr int kSlotBytes = 2 * QM * 64;       // hi + lo of a [128 x 16] chunk
constexpr int kQBytes = 2 * 4 * QM * 64;      // hi + lo of Q as 4 blocks = the P ring
constexpr uint32_t kOCol = 256;               // first tensor-memory column of O
constexpr uint32_t kTmemCols = 512;

struct AttnTcDev {
  const float* q; const float* k; const float* v;
  long long row_stride, batch_stride;
  float* out; long long out_row_stride, out_batch_stride;
  int heads, tokens;
  const float* scale; int scale_mode;   // 0 none, 1 multiply, 2 divide
  int* err;
};

// Byte offset of 16-byte chunk `chunk` (0..3) of row `row` in a K-major block with
// 64-byte rows and the 64-byte swizzle: address bits 4-5 are XORed with bits 7-8.
__device__ __forceinline__ uint32_t sw64_off(int row, int chunk) {
  return (uint32_t)((row >> 3) * 512 + (row & 7) * 64 + ((chunk ^ ((row & 7) >> 1)) << 4));
}

__device__ __forceinline__ uint64_t desc_sw64(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);   // start address
  d |= (uint64_t)1 << 16;                   // leading byte offset (ignored for swizzled K-major)
  d |= (uint64_t)(512 >> 4) << 32;          // stride byte offset: 8 rows of 64 bytes
  d |= (uint64_t)1 << 46;                   // descriptor version for this architecture
  d |= (uint64_t)4 << 61;                   // 64-byte swizzle
  return d;
}

__device__ __forceinline__ void tc_ld_32x16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]),
        "=r"(v[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ float apply_scale(float s, float sc, int mode) {
  if (mode == 1) return __fmul_rn(s, sc);
  if (mode == 2) return __fdiv_rn(s, sc);
  return s;
}

__device__ __forceinline__ void store_split(uint8_t* hi_base, uint8_t* lo_base, uint32_t off, float4 v) {
  float4 hi, lo;
  tf32_split(v, hi, lo);
  *reinterpret_cast<float4*>(hi_base + off) = hi;
  *reinterpret_cast<float4*>(lo_base + off) = lo;
}

// NB = 16-column blocks of keys: NS = 16 * NB >= tokens.
template <int NB>
__global__ void __launch_bounds__(kAtThreads, 1) attention_tc_kernel(AttnTcDev p) {
  constexpr int NS = NB * 16;
  constexpr int kKBlock = NS * 64;            // bytes of one [NS x 16] block of K
  constexpr int kVBlock = HD * 64;            // bytes of one [64 x 16] block of V^T
  static_assert(8 * kKBlock == 2 * NB * kVBlock, "K and V^T share one region");
  extern __shared__ uint8_t at_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(at_smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* kv = smem;                          // 8 * kKBlock bytes
  uint8_t* qp = smem + 8 * kKBlock;            // kQBytes
  uint64_t* bars = reinterpret_cast<uint64_t*>(qp + kQBytes);
  uint64_t* s_full = bars;                     // S complete in tensor memory
  uint64_t* o_full = bars + 1;                 // O complete
  uint64_t* ready = bars + 2;                  // [kSlots] P chunk written by the 128 softmax threads
  uint64_t* freeb = ready + kSlots;            // [kSlots] P chunk consumed by its MMAs
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(freeb + kSlots);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int T = p.tokens;
  const int bh = blockIdx.y;
  const int b = bh / p.heads, h = bh % p.heads;
  const int q0 = blockIdx.x * QM;
  const long long base = (long long)b * p.batch_stride + (long long)h * HD;
  const float* qg = p.q + base;
  const float* kg = p.k + base;
  const float* vg = p.v + base;
  bool ok = true;

  if (tid == 0) {
    mbar_init(s_full, 1);
    mbar_init(o_full, 1);
    for (int i = 0; i < kSlots; ++i) {
      mbar_init(&ready[i], QM);
      mbar_init(&freeb[i], 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 4) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(kTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }

  // ---- stage Q [128 x 64] and K [NS x 64]: 16 threads per row, one float4 each ----
  {
    float4 qv[8], kvv[NB];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int idx = tid + kAtThreads * i, row = idx >> 4, c4 = idx & 15;
      qv[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (q0 + row < T) qv[i] = __ldg(reinterpret_cast<const float4*>(qg + (long long)(q0 + row) * p.row_stride + c4 * 4));
    }
#pragma unroll
    for (int i = 0; i < NB; ++i) {
      const int idx = tid + kAtThreads * i, row = idx >> 4, c4 = idx & 15;
      kvv[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (row < T) kvv[i] = __ldg(reinterpret_cast<const float4*>(kg + (long long)row * p.row_stride + c4 * 4));
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int idx = tid + kAtThreads * i, row = idx >> 4, c4 = idx & 15;
      uint8_t* blk = qp + (c4 >> 2) * (QM * 64);
      store_split(blk, blk + 4 * QM * 64, sw64_off(row, c4 & 3), qv[i]);
    }
#pragma unroll
    for (int i = 0; i < NB; ++i) {
      const int idx = tid + kAtThreads * i, row = idx >> 4, c4 = idx & 15;
      uint8_t* blk = kv + (c4 >> 2) * kKBlock;
      store_split(blk, blk + 4 * kKBlock, sw64_off(row, c4 & 3), kvv[i]);
    }
  }
  // ---- V into registers: thread (d, tg) takes tokens 16 i + 4 tg + {0..3} of column d,
  // the 16-byte chunk tg of row d in block i of V^T ----
  const int vd = tid & 63, vtg = tid >> 6;
  float vv[NB][4];
#pragma unroll
  for (int i = 0; i < NB; ++i)
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int t = 16 * i + 4 * vtg + u;
      vv[i][u] = (t < T) ? __ldg(vg + (long long)t * p.row_stride + vd) : 0.f;
    }

  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t idesc_s = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(NS >> 3) << 17) | ((uint32_t)(QM >> 4) << 24);
  const uint32_t idesc_o = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(QM >> 4) << 24);

  // ---- S = Q K^T: 4 blocks x 2 K-steps x 3 MMAs ----
  if (warp == 4 && lane == 0) {
#pragma unroll
    for (int blk = 0; blk < 4; ++blk)
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {
        const uint32_t qa = smem_u32(qp + blk * (QM * 64)) + kk * 32;
        const uint32_t ka = smem_u32(kv + blk * kKBlock) + kk * 32;
        const uint64_t a_hi = desc_sw64(qa), a_lo = desc_sw64(qa + 4 * QM * 64);
        const uint64_t b_hi = desc_sw64(ka), b_lo = desc_sw64(ka + 4 * kKBlock);
        tc_mma_tf32(tmem_base, a_lo, b_hi, idesc_s, (blk | kk) ? 1u : 0u);
        tc_mma_tf32(tmem_base, a_hi, b_lo, idesc_s, 1u);
        tc_mma_tf32(tmem_base, a_hi, b_hi, idesc_s, 1u);
      }
    tc_commit(s_full);
  }
  __syncwarp();
  if (!mbar_wait(s_full, 0)) { atomicExch(p.err, 11); ok = false; }
  tc_fence_after();

  // ---- K is consumed: store V^T (hi / lo) over it ----
#pragma unroll
  for (int i = 0; i < NB; ++i) {
    uint8_t* blk = kv + i * kVBlock;
    store_split(blk, blk + NB * kVBlock, sw64_off(vd, vtg), make_float4(vv[i][0], vv[i][1], vv[i][2], vv[i][3]));
  }
  fence_proxy_async();
  __syncthreads();

  if (warp < 4) {
    // ---------------- softmax: one row per thread ----------------
    const int row = warp * 32 + lane;
    const uint32_t trow = tmem_base + ((uint32_t)(warp * 32) << 16);
    const float sc = p.scale_mode ? __ldg(p.scale) : 1.f;
    const int mode = p.scale_mode;
    float m = CUDART_NAN_F;
#pragma unroll 1
    for (int c = 0; c < NB; ++c) {
      uint32_t v[16];
      tc_ld_32x16(trow + (uint32_t)(c * 16), v);
#pragma unroll
      for (int u = 0; u < 16; ++u)
        if (c * 16 + u < T) m = fmaxf(apply_scale(__uint_as_float(v[u]), sc, mode), m);
    }
    float sum = 0.f;
#pragma unroll 1
    for (int c = 0; c < NB; ++c) {
      const int slot = c % kSlots;
      if (ok && c >= kSlots && !mbar_wait(&freeb[slot], ((c / kSlots) - 1) & 1)) { atomicExch(p.err, 12); ok = false; }
      uint32_t v[16];
      tc_ld_32x16(trow + (uint32_t)(c * 16), v);
      float e[16];
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        e[u] = 0.f;
        if (c * 16 + u < T) {
          e[u] = exp_poly_softmax(__fsub_rn(apply_scale(__uint_as_float(v[u]), sc, mode), m));
          sum = __fadd_rn(sum, e[u]);
        }
      }
      uint8_t* sl = qp + slot * kSlotBytes;
#pragma unroll
      for (int j = 0; j < 4; ++j)
        store_split(sl, sl + QM * 64, sw64_off(row, j), make_float4(e[4 * j], e[4 * j + 1], e[4 * j + 2], e[4 * j + 3]));
      fence_proxy_async();
      if (ok) mbar_arrive(&ready[slot]);
    }
    // ---- O * (1 / sum) -> out[b, q0 + row, h * 64 ...] ----
    if (ok && !mbar_wait(o_full, 0)) { atomicExch(p.err, 13); ok = false; }
    tc_fence_after();
    const float recip = __fdiv_rn(1.f, sum);
    float* og = p.out + (long long)b * p.out_batch_stride + (long long)h * HD + (long long)(q0 + row) * p.out_row_stride;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      uint32_t o[32];
      tc_ld_32x32(trow + kOCol + (uint32_t)(half * 32), o);
      if (ok && q0 + row < T) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          *reinterpret_cast<float4*>(og + half * 32 + 4 * j) =
              make_float4(__fmul_rn(__uint_as_float(o[4 * j]), recip), __fmul_rn(__uint_as_float(o[4 * j + 1]), recip),
                          __fmul_rn(__uint_as_float(o[4 * j + 2]), recip), __fmul_rn(__uint_as_float(o[4 * j + 3]), recip));
      }
    }
  } else if (warp == 4 && lane == 0) {
    // ---------------- O = P V: per chunk 2 K-steps x 3 MMAs ----------------
#pragma unroll 1
    for (int c = 0; ok && c < NB; ++c) {
      const int slot = c % kSlots;
      if (!mbar_wait(&ready[slot], (c / kSlots) & 1)) { atomicExch(p.err, 14); ok = false; break; }
      tc_fence_after();
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {
        const uint32_t pa = smem_u32(qp + slot * kSlotBytes) + kk * 32;
        const uint32_t va = smem_u32(kv + c * kVBlock) + kk * 32;
        const uint64_t a_hi = desc_sw64(pa), a_lo = desc_sw64(pa + QM * 64);
        const uint64_t b_hi = desc_sw64(va), b_lo = desc_sw64(va + NB * kVBlock);
        tc_mma_tf32(tmem_base + kOCol, a_lo, b_hi, idesc_o, (c | kk) ? 1u : 0u);
        tc_mma_tf32(tmem_base + kOCol, a_hi, b_lo, idesc_o, 1u);
        tc_mma_tf32(tmem_base + kOCol, a_hi, b_hi, idesc_o, 1u);
      }
      tc_commit(&freeb[slot]);
    }
    if (ok) tc_commit(o_full);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols));
  }
}

template <int NB>
cudaError_t launch_nb(const AttnTcDev& d, int bh, cudaStream_t st) {
  constexpr int kDyn = NB * 8192 + kQBytes + 128 /*barriers*/ + 1024 /*alignment*/;
  static_assert(kDyn <= 227 * 1024, "shared memory per CTA");
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(attention_tc_kernel<NB>, cudaFuncAttributeMaxDynamicSharedMemorySize, kDyn);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  dim3 grid((d.tokens + QM - 1) / QM, bh);
  attention_tc_kernel<NB><<<grid, kAtThreads, kDyn, st>>>(d);
  return cudaGetLastError();
}

}  // namespace

bool attention_tc_supported(const AttentionParams& p) {
  auto al = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  return p.head_dim == HD && p.tokens > 64 && p.tokens <= 256 && p.batch >= 1 && p.heads >= 1 &&
         (long long)p.batch * p.heads <= 65535 && (p.row_stride % 4) == 0 && (p.batch_stride % 4) == 0 &&
         (p.out_row_stride % 4) == 0 && (p.out_batch_stride % 4) == 0 && al(p.q) && al(p.k) && al(p.v) &&
         al(p.out) && p.out != nullptr && p.err_word != nullptr;
}

cudaError_t launch_attention_tc(const AttentionParams& p, cudaStream_t st) {
  if (!attention_tc_supported(p)) return cudaErrorInvalidValue;
  AttnTcDev d;
  d.q = p.q; d.k = p.k; d.v = p.v;
  d.row_stride = p.row_stride; d.batch_stride = p.batch_stride;
  d.out = p.out; d.out_row_stride = p.out_row_stride; d.out_batch_stride = p.out_batch_stride;
  d.heads = p.heads; d.tokens = p.tokens;
  d.scale = p.scale; d.scale_mode = p.scale ? p.scale_mode : 0;
  d.err = p.err_word;
  const int bh = p.batch * p.heads;
  if (p.tokens <= 128) return launch_nb<8>(d, bh, st);
  if (p.tokens <= 208) return launch_nb<13>(d, bh, st);
  return launch_nb<16>(d, bh, st);
}

}  // namespace ac
