// Fused multi-head attention core on the sm_100a tensor cores: one CTA per
// (image, head, block of 128 query rows),
//
//   S = (Q K^T) (* | /) scale ;  P = Softmax(S) ;  O = P V
//
// with both products issued as tcgen05.mma with fp32 accumulators in tensor memory:
// Q K^T as 3xTF32 (kind::tf32), P V with fp16-split operands (kind::f16, two
// accumulators, see gemm_tc.cu) after a power-of-two scaling that makes the split
// safe: P = e * 2^13 with e <= 1, V times 2^s with s from the head's largest |v|.
// It replaces the same operator chain as the CUDA-core kernel in attention.cu
// (Split / Reshape / Transpose / MatMul / Mul / Softmax / MatMul / Transpose /
// Reshape of crates/session_interpreter/src/session.rs:621-682, 990-1026,
// 1179-1278, 1488-1512) and reads Q, K, V in place from the [B, T, 3D] projection
// buffer.
//
// Shared memory holds every operand as K-major tiles with 64-byte rows and the
// 64-byte swizzle (the layout the GEMM kernel's TMA boxes have), as a `hi` and a
// `lo` copy:
//   region KV : K [NS x 64] TF32 as 4 blocks of 16 floats; after S is complete it is
//               overwritten by V^T [64 x NS] fp16 as blocks of 32 keys (V is
//               transposed on the way in, so that the second product also takes a
//               K-major B operand);
//   region QP : Q [128 x 64] TF32 as 4 blocks; after S is complete it becomes a ring
//               of four P blocks [128 x 32 keys] fp16.
// Tensor memory: S in columns [0, NS), O in columns [256, 320) (hi * hi) and
// [320, 384) (cross terms, scaled by 2^11).
//
//   warps 0-7    stage Q and K (global -> registers -> split -> swizzled stores),
//                prefetch V into registers, and after S transpose-store V; then softmax,
//                two threads per query row (= tensor-memory lane), one per half of the
//                key columns: pass 1 row maximum of the scaled scores, pass 2
//                e = 2^((s - max) log2 e) by ex2.approx (2 ulp), running sum, e split
//                into hi/lo and stored as the A operand of the second product; maxima and
//                sums of the two halves meet in shared memory; finally O * (1 / sum) goes
//                to global through a shared-memory transpose (full 128-byte lines);
//   warp 8       allocates tensor memory; one thread issues the MMAs and commits to
//                mbarriers (the P chunks of the two halves alternate).
// P is fed unnormalised and O scaled by 1 / sum at the end (the reference
// normalises P first), and the exponential is the hardware's instead of the reference's
// degree-6 polynomial: differences of a few ulp, far below those of the split products.
// Every mbarrier wait is bounded; on expiry the kernel records a code in the
// error word and runs to its end without touching the barrier again.
#include <cstdio>
#include <cstdlib>
#include <type_traits>

#include "kernels.h"
#include "ref_math.cuh"
#include "tc_common.cuh"

namespace ac {
namespace {

using namespace tc;

constexpr int HD = 64;                        // head dimension
constexpr int QM = 128;                       // query rows per CTA = tensor-memory lanes
constexpr int kAtThreads = 256;              // warps 0-7: staging and softmax
constexpr int kAtLaunch = kAtThreads + 32;    // + warp 8: MMA issue, tensor-memory allocation
constexpr int kSlots = 4;                     // P ring depth
constexpr int kSlotBytes = 2 * QM * 64;       // hi + lo of a [128 x 32 keys] fp16 block of P
constexpr int kQBytes = 2 * 4 * QM * 64;      // hi + lo of Q as 4 blocks = the P ring
constexpr uint32_t kOCol = 256;               // first tensor-memory column of O
constexpr uint32_t kTmemCols = 512;

struct AttnTcDev {
  const float* q; const float* k; const float* v;
  long long row_stride, batch_stride;
  float* out; long long out_row_stride, out_batch_stride;   // out may be null when o16_hi / o16_lo are given
  uint2* o16_hi; uint2* o16_lo;   // the result as fp16 halves on the fixed scale (f16_split_fixed; same strides, in elements), or null
  int heads, tokens;
  const float* scale; int scale_mode;   // 0 none, 1 multiply, 2 divide
  int* err;
  long long* dbg;   // phase time stamps of CTA (0, 0) when not null (debug toggle)
};
__device__ long long g_attn_stamps[32];   // [0]: kernel entry; [1..8] first query tile, [11..18] second
#define AT_STAMP(i) do { if (p.dbg && blockIdx.x == 0 && blockIdx.y == 0 && tid == 0) p.dbg[(i) + stamp_base] = clock64(); } while (0)

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

// The load alone: several may be in flight before one tc_ld_wait().
__device__ __forceinline__ void tc_ld_32x16_issue(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]),
        "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

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

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Barrier of the two softmax warps that share tensor-memory lane quarter q (named barriers 1-4).
__device__ __forceinline__ void pair_sync(int q) {
  asm volatile("bar.sync %0, 64;" ::"r"(q + 1) : "memory");
}

__device__ __forceinline__ void store_split(uint8_t* hi_base, uint8_t* lo_base, uint32_t off, float4 v) {
  float4 hi, lo;
  tf32_split(v, hi, lo);
  *reinterpret_cast<float4*>(hi_base + off) = hi;
  *reinterpret_cast<float4*>(lo_base + off) = lo;
}

// V^T as fp16 hi / lo of v * sv, blocks of 32 keys (64-byte rows); an odd last block gets
// zeros in its second half. Thread (vd, vtg) holds keys 16 i + 4 vtg + {0..3} of column vd.
template <int NB>
__device__ __forceinline__ void store_vt(uint8_t* vt, const float (&vv)[NB][4], float sv, int vd, int vtg, int T) {
  constexpr int NBLK = (NB + 1) / 2;
  constexpr int kVBlock = HD * 64;
#pragma unroll
  for (int i = 0; i < 2 * NBLK; ++i) {
    const int t0 = 16 * i + 4 * vtg;
    float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < NB) {
      constexpr int kLast = NB - 1;
      const int ii = i < NB ? i : kLast;
      x = make_float4(t0 < T ? __fmul_rn(vv[ii][0], sv) : 0.f, t0 + 1 < T ? __fmul_rn(vv[ii][1], sv) : 0.f,
                      t0 + 2 < T ? __fmul_rn(vv[ii][2], sv) : 0.f, t0 + 3 < T ? __fmul_rn(vv[ii][3], sv) : 0.f);
    }
    uint2 hi, lo;
    f16_split(x, hi, lo);
    const uint32_t off = (uint32_t)((i >> 1) * kVBlock) + sw64_off8(vd, 4 * (i & 1) + vtg);
    *reinterpret_cast<uint2*>(vt + off) = hi;
    *reinterpret_cast<uint2*>(vt + NBLK * kVBlock + off) = lo;
  }
}

// sv = 2^(13 - floor(log2 max|v|)) from the eight warp maxima in xch: |v * sv| < 2^14. A zero,
// infinite or NaN maximum leaves V unscaled (the result is then zero, or not finite as in fp32).
__device__ __forceinline__ void scale_from_maxima(const float* xch, float& sv, float& inv_sv) {
  float vm = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) vm = fmaxf(vm, xch[w]);
  const int eb = (int)((__float_as_uint(vm) >> 23) & 0xFFu);
  if (eb > 0 && eb < 255) {
    const int f = min(max(267 - eb, 1), 253);
    sv = __uint_as_float((uint32_t)f << 23);
    inv_sv = __uint_as_float((uint32_t)(254 - f) << 23);
  }
}

// Barrier of the eight staging / softmax warps (named barrier 5).
__device__ __forceinline__ void group_sync() {
  asm volatile("bar.sync 5, 256;" ::: "memory");
}

// NB = 16-column blocks of keys: NS = 16 * NB >= tokens. RESIDENT: K and V^T have shared
// memory of their own, and one CTA walks all query tiles of its (image, head) with K and V
// staged once (grid.x = 1); otherwise V^T overwrites K and each query tile is a CTA of
// its own (grid.x = tiles).
template <int NB, int SMODE, bool RESIDENT>
__global__ void __launch_bounds__(kAtLaunch, 1) attention_tc_kernel(AttnTcDev p) {
  constexpr int NS = NB * 16;
  constexpr int kKBlock = NS * 64;            // bytes of one [NS x 16] block of K
  constexpr int kVBlock = HD * 64;            // bytes of one [64 x 32] fp16 block of V^T
  constexpr int NBLK = (NB + 1) / 2;          // 32-key blocks of V^T and P
  constexpr int NBLK0 = (NBLK + 1) / 2;       // blocks of the first column half
  extern __shared__ uint8_t at_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(at_smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* kv = smem;                                              // K: 8 * kKBlock bytes
  uint8_t* vt = RESIDENT ? smem + 8 * kKBlock : smem;              // V^T: 2 * NBLK * kVBlock bytes
  uint8_t* qp = vt + (RESIDENT ? 2 * NBLK * kVBlock : 8 * kKBlock);   // Q, then the P ring: kQBytes
  uint64_t* bars = reinterpret_cast<uint64_t*>(qp + kQBytes);
  uint64_t* s_full = bars;                     // S complete in tensor memory
  uint64_t* o_full = bars + 1;                 // O complete
  uint64_t* ready = bars + 2;                  // [kSlots] P block written by the 128 threads of a half
  uint64_t* freeb = ready + kSlots;            // [kSlots] P block consumed by its MMAs
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(freeb + kSlots);
  float* xch = reinterpret_cast<float*>(bars + 16);   // [2][128] row maxima, then row sums, of the two halves

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int T = p.tokens;
  const int bh = blockIdx.y;
  const int b = bh / p.heads, h = bh % p.heads;
  const int n_tiles = RESIDENT ? (T + QM - 1) / QM : 1;
  const long long base = (long long)b * p.batch_stride + (long long)h * HD;
  const float* qg = p.q + base;
  const float* kg = p.k + base;
  const float* vg = p.v + base;
  bool ok = true;
  unsigned seen_out = 0;   // range of what this thread wrote split (o16_hi)
  int stamp_base = 0;
  AT_STAMP(0);

  if (tid == 0) {
    mbar_init(s_full, 1);
    mbar_init(o_full, 1);
    for (int i = 0; i < kSlots; ++i) {
      mbar_init(&ready[i], QM);
      mbar_init(&freeb[i], 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 8) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(kTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }

  const uint32_t idesc_s = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(NS >> 3) << 17) | ((uint32_t)(QM >> 4) << 24);
  // Second product: fp16 operands (format 0), N = 64.
  const uint32_t idesc_o = (1u << 4) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(QM >> 4) << 24);
  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
  const int vd = tid & 63, vtg = (tid >> 6) & 3;   // V: thread (d, tg) takes keys 16 i + 4 tg + {0..3} of column d
  float sv = 1.f, inv_sv = 1.f;                // power-of-two scale of V and its inverse
  uint32_t tmem_base = 0;
  int uses0 = 0, uses1 = 0;                    // softmax: uses so far of this half's two ring slots
  uint32_t mma_par = 0;                        // MMA thread: bit s = parity of the next use of ring slot s
  float4 qnext[8];                             // the next query tile, fetched while this one finishes

  // One query tile. The first one also stages K and V (FIRST: compiled as its own copy, so
  // that V's registers are not carried through the later tiles).
  auto do_tile = [&](auto first_tag, const int tile) {
    constexpr bool FIRST = decltype(first_tag)::value;
    stamp_base = FIRST ? 0 : 10;
    float vv[FIRST ? NB : 1][4];
    const int q0 = (RESIDENT ? tile : (int)blockIdx.x) * QM;
    const uint32_t par = (uint32_t)(tile & 1);
    // ---- stage Q [128 x 64] (and, once, K [NS x 64] and V): 16 threads per row, one float4
    // each. Rows past the end are read from the last row (unconditional loads, all in
    // flight at once) and zeroed when stored. ----
    if (warp < 8) {
      if (!FIRST) group_sync();                // every warp is done with the P ring / output tiles in qp
      float4 qv[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int idx = tid + kAtThreads * i, row = idx >> 4, c4 = idx & 15;
        if (FIRST) qv[i] = __ldg(reinterpret_cast<const float4*>(qg + (long long)min(q0 + row, T - 1) * p.row_stride + c4 * 4));
        else qv[i] = qnext[i];
      }
      if constexpr (FIRST) {
        float4 kvv[NB];
#pragma unroll
        for (int i = 0; i < NB; ++i) {
          const int idx = tid + kAtThreads * i, row = idx >> 4, c4 = idx & 15;
          kvv[i] = __ldg(reinterpret_cast<const float4*>(kg + (long long)min(row, T - 1) * p.row_stride + c4 * 4));
        }
#pragma unroll
        for (int i = 0; i < NB; ++i) {
          const int idx = tid + kAtThreads * i, row = idx >> 4, c4 = idx & 15;
          uint8_t* blk = kv + (c4 >> 2) * kKBlock;
          store_split(blk, blk + 4 * kKBlock, sw64_off(row, c4 & 3), row < T ? kvv[i] : zero4);
        }
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int idx = tid + kAtThreads * i, row = idx >> 4, c4 = idx & 15;
        uint8_t* blk = qp + (c4 >> 2) * (QM * 64);
        store_split(blk, blk + 4 * QM * 64, sw64_off(row, c4 & 3), q0 + row < T ? qv[i] : zero4);
      }
      if constexpr (FIRST) {
        // V into registers; it is used after the barrier below, under the first product.
#pragma unroll
        for (int i = 0; i < NB; ++i)
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int t = 16 * i + 4 * vtg + u;
            vv[i][u] = __ldg(vg + (long long)min(t, T - 1) * p.row_stride + vd);   // masked when stored
          }
      }
    }
    AT_STAMP(1);
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    AT_STAMP(2);
    if (FIRST) tmem_base = *tmem_slot;

    // ---- S = Q K^T: 4 blocks x 2 K-steps x 3 TF32 MMAs ----
    if (warp == 8 && lane == 0) {
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
    if constexpr (FIRST) {
    if (warp < 8) {
      // Largest |v| of this head, for the power-of-two scale that puts V into the fp16 range.
      float vmax = 0.f;
#pragma unroll
      for (int i = 0; i < NB; ++i)
#pragma unroll
        for (int u = 0; u < 4; ++u) vmax = fmaxf(vmax, fabsf(vv[i][u]));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, o));
      if (lane == 0) xch[warp] = vmax;
      group_sync();
      scale_from_maxima(xch, sv, inv_sv);
      // V^T with memory of its own is stored under the first product; otherwise it
      // overwrites K and has to wait for S.
      if (RESIDENT) store_vt<NB>(vt, vv, sv, vd, vtg, T);
    }
    if (RESIDENT) {
      fence_proxy_async();
      __syncthreads();
    }
    }
    if (ok && !warp_mbar_wait(s_full, par, lane)) { atomicExch(p.err, 11); ok = false; }
    tc_fence_after();
    AT_STAMP(3);
    if constexpr (FIRST && !RESIDENT) {
      if (warp < 8) store_vt<NB>(vt, vv, sv, vd, vtg, T);
      fence_proxy_async();
      __syncthreads();
    }
    AT_STAMP(4);

    if (warp < 8) {
      // ---------------- softmax: two threads per row, one per column half ----------------
      const int q = warp & 3, hf = warp >> 2;    // tensor-memory lane quarter, column half
      const int row = q * 32 + lane;
      const int b_begin = hf ? NBLK0 : 0, b_count = hf ? NBLK - NBLK0 : NBLK0;
      const uint32_t trow = tmem_base + ((uint32_t)(q * 32) << 16);
      // Scores enter the exponential as t = acc * c1 with c1 = log2(e) (* | /) scale, so that
      // e = 2^(t - max t) is one FFMA and one ex2.approx per score (2 ulp; the CUDA-core kernel
      // keeps the reference's polynomial).
      const float kLog2e = 1.44269504088896341f;
      const float sc = SMODE ? __ldg(p.scale) : 1.f;
      const float c1 = SMODE == 1 ? __fmul_rn(sc, kLog2e) : (SMODE == 2 ? __fdiv_rn(kLog2e, sc) : kLog2e);
      float m = CUDART_NAN_F;
#pragma unroll 1
      for (int i = 0; i < b_count; ++i) {
        const int c0 = (b_begin + i) * 32;       // 32 columns per step; columns past NS read junk that is masked
        uint32_t v[2][16];
        tc_ld_32x16_issue(trow + (uint32_t)c0, v[0]);
        tc_ld_32x16_issue(trow + (uint32_t)(c0 + 16), v[1]);
        tc_ld_wait();
        // Columns past T (exact zeros up to NS, junk beyond) are kept out of the maximum
        // by a select, not a branch, so that the chains stay interleaved.
        float m0 = CUDART_NAN_F, m1 = CUDART_NAN_F;
#pragma unroll
        for (int u = 0; u < 16; ++u) {
          const float t0 = __fmul_rn(__uint_as_float(v[0][u]), c1), t1 = __fmul_rn(__uint_as_float(v[1][u]), c1);
          m0 = fmaxf(c0 + u < T ? t0 : CUDART_NAN_F, m0);
          m1 = fmaxf(c0 + 16 + u < T ? t1 : CUDART_NAN_F, m1);
        }
        m = fmaxf(fmaxf(m0, m1), m);
      }
      xch[hf * QM + row] = m;
      pair_sync(q);
      m = fmaxf(xch[QM + row], xch[row]);
      pair_sync(q);                              // both have read before the sums overwrite
      AT_STAMP(5);
      const float m13 = __fsub_rn(m, 13.f);      // P = e * 2^13 comes out of the exponential directly
      float sum = 0.f;                           // of e * 2^13; the factor cancels in O / sum
#pragma unroll 1
      for (int i = 0; i < b_count; ++i) {
        const int blk = b_begin + i;
        const int slot = 2 * hf + (i & 1);
        const int n = (i & 1) ? uses1 : uses0;   // this is use n of the slot over the whole kernel
        if (ok && n >= 1 && !warp_mbar_wait(&freeb[slot], (uint32_t)((n - 1) & 1), lane)) { atomicExch(p.err, 12); ok = false; }
        if (i & 1) ++uses1; else ++uses0;
        uint8_t* sl = qp + slot * kSlotBytes;
#pragma unroll
        for (int h16 = 0; h16 < 2; ++h16) {
          const int c0 = blk * 32 + h16 * 16;
          uint32_t v[16];
          tc_ld_32x16(trow + (uint32_t)c0, v);
          float e[16];
#pragma unroll
          for (int u = 0; u < 16; ++u) {
            const float ev = ex2_approx(fmaf(__uint_as_float(v[u]), c1, -m13));
            e[u] = c0 + u < T ? ev : 0.f;
          }
#pragma unroll
          for (int u = 0; u < 16; ++u) sum = __fadd_rn(sum, e[u]);   // + 0 for masked columns: exact
          // P as fp16 hi / lo (at most 2^13: in range, and far from the subnormals)
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            uint2 h0, l0, h1, l1;
            f16_split(make_float4(e[8 * j], e[8 * j + 1], e[8 * j + 2], e[8 * j + 3]), h0, l0);
            f16_split(make_float4(e[8 * j + 4], e[8 * j + 5], e[8 * j + 6], e[8 * j + 7]), h1, l1);
            const uint32_t off = sw64_off(row, 2 * h16 + j);
            *reinterpret_cast<uint4*>(sl + off) = make_uint4(h0.x, h0.y, h1.x, h1.y);
            *reinterpret_cast<uint4*>(sl + QM * 64 + off) = make_uint4(l0.x, l0.y, l1.x, l1.y);
          }
        }
        fence_proxy_async();
        if (ok) mbar_arrive(&ready[slot]);
      }
      if (tile + 1 < n_tiles) {                  // next query tile into registers, under the tail of this one
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int idx = tid + kAtThreads * i, r2 = idx >> 4, c4 = idx & 15;
          qnext[i] = __ldg(reinterpret_cast<const float4*>(qg + (long long)min(q0 + QM + r2, T - 1) * p.row_stride + c4 * 4));
        }
      }
      xch[hf * QM + row] = sum;
      pair_sync(q);
      sum = __fadd_rn(xch[row], xch[QM + row]);
      // ---- O = (D1 + D2 * 2^-11) * (1 / sum) / sv: this warp takes 32 of the 64
      // columns; through a 4 KB tile of the (now idle) P ring so that every 8 lanes write one
      // full 128-byte line ----
      AT_STAMP(6);
      if (ok && !warp_mbar_wait(o_full, par, lane)) { atomicExch(p.err, 13); ok = false; }
      tc_fence_after();
      AT_STAMP(7);
      const float recip = __fdiv_rn(1.f, sum);
      uint32_t o[32], o2[32];
      tc_ld_32x32(trow + kOCol + (uint32_t)(hf * 32), o);
      tc_ld_32x32(trow + kOCol + (uint32_t)(HD + hf * 32), o2);
      float4* stage = reinterpret_cast<float4*>(qp + warp * 4096);
      auto fin = [&](int j) {
        const float y = fmaf(__uint_as_float(o2[j]), kLoUnscale, __uint_as_float(o[j]));
        return __fmul_rn(__fmul_rn(y, recip), inv_sv);
      };
#pragma unroll
      for (int j = 0; j < 8; ++j)
        stage[lane * 8 + (j ^ (lane & 7))] = make_float4(fin(4 * j), fin(4 * j + 1), fin(4 * j + 2), fin(4 * j + 3));
      __syncwarp();
      const int c4 = lane & 7, rsub = lane >> 3;
      const long long obase = (long long)b * p.out_batch_stride + (long long)h * HD + hf * 32 + 4 * c4;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int rl = 4 * i + rsub, r = q0 + q * 32 + rl;
        if (ok && r < T) {
          const float4 y = stage[rl * 8 + (c4 ^ (rl & 7))];
          const long long o = obase + (long long)r * p.out_row_stride;
          if (p.out) *reinterpret_cast<float4*>(p.out + o) = y;
          if (p.o16_hi) {   // for the projection GEMM that takes this result as its pre-split A
            uint2 hh, ll;
            f16_split_fixed(y, hh, ll);
            p.o16_hi[o >> 2] = hh;
            p.o16_lo[o >> 2] = ll;
            seen_out |= split_seen_fixed(y);
          }
        }
      }
      tc_fence_before();                         // the tensor-memory loads above precede the next tile's MMAs
    } else if (lane == 0) {
      // ---------------- O = P V: per 32-key block 2 K-steps x 3 fp16 MMAs; the halves alternate ----------------
#pragma unroll 1
      for (int n = 0; ok && n < 2 * NBLK0; ++n) {
        const int hf = n & 1, i = n >> 1;
        const int blk = hf ? NBLK0 + i : i;
        if (blk >= NBLK) continue;
        const int slot = 2 * hf + (i & 1);
        if (!mbar_wait(&ready[slot], (mma_par >> slot) & 1u)) { atomicExch(p.err, 14); ok = false; break; }
        mma_par ^= 1u << slot;
        tc_fence_after();
        // One accumulator after the other: alternating between D1 and D2 with every MMA
        // slows the tensor pipe down.
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
          const uint32_t pa = smem_u32(qp + slot * kSlotBytes) + kk * 32;
          const uint32_t va = smem_u32(vt + blk * kVBlock) + kk * 32;
          tc_mma_f16(tmem_base + kOCol, desc_sw64(pa), desc_sw64(va), idesc_o, (n | kk) ? 1u : 0u);     // hi * hi -> D1
        }
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
          const uint32_t pa = smem_u32(qp + slot * kSlotBytes) + kk * 32;
          const uint32_t va = smem_u32(vt + blk * kVBlock) + kk * 32;
          const uint64_t a_hi = desc_sw64(pa), a_lo = desc_sw64(pa + QM * 64);
          const uint64_t b_hi = desc_sw64(va), b_lo = desc_sw64(va + NBLK * kVBlock);
          tc_mma_f16(tmem_base + kOCol + HD, a_lo, b_hi, idesc_o, (n | kk) ? 1u : 0u);   // lo' * hi -> D2
          tc_mma_f16(tmem_base + kOCol + HD, a_hi, b_lo, idesc_o, 1u);                   // hi * lo' -> D2
        }
        tc_commit(&freeb[slot]);
      }
      if (ok) tc_commit(o_full);
    }
    AT_STAMP(8);
  };
  do_tile(std::true_type{}, 0);
#pragma unroll 1
  for (int tile = 1; tile < n_tiles; ++tile) do_tile(std::false_type{}, tile);
  if (p.o16_hi && warp < 8) split_report_warp(seen_out, p.err);   // one head's rows: out of range, or all tiny
  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols));
  }
}

template <int NB, int SMODE>
cudaError_t launch_nb_mode(const AttnTcDev& d, int bh, cudaStream_t st) {
  constexpr int kExtra = 128 /*barriers*/ + 1024 /*row exchange*/ + 1024 /*alignment*/;
  constexpr int kDynResident = NB * 8192 + ((NB + 1) / 2) * 8192 + kQBytes + kExtra;
  constexpr int kDynOverlay = NB * 8192 + kQBytes + kExtra;
  constexpr bool kResident = kDynResident <= 227 * 1024;
  constexpr int kDyn = kResident ? kDynResident : kDynOverlay;
  static_assert(kDyn <= 227 * 1024, "shared memory per CTA");
  static unsigned long long attr_done = 0;
  cudaError_t e = ensure_dynamic_smem(attention_tc_kernel<NB, SMODE, kResident>, kDyn, &attr_done);
  if (e != cudaSuccess) return e;
  dim3 grid(kResident ? 1 : (d.tokens + QM - 1) / QM, bh);
  attention_tc_kernel<NB, SMODE, kResident><<<grid, kAtLaunch, kDyn, st>>>(d);
  return cudaGetLastError();
}

template <int NB>
cudaError_t launch_nb(const AttnTcDev& d, int bh, cudaStream_t st) {
  if (d.scale_mode == 1) return launch_nb_mode<NB, 1>(d, bh, st);
  if (d.scale_mode == 2) return launch_nb_mode<NB, 2>(d, bh, st);
  return launch_nb_mode<NB, 0>(d, bh, st);
}

}  // namespace

bool attention_tc_supported(const AttentionParams& p) {
  auto al = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  return p.head_dim == HD && p.tokens > 64 && p.tokens <= 256 && p.batch >= 1 && p.heads >= 1 &&
         (long long)p.batch * p.heads <= 65535 && (p.row_stride % 4) == 0 && (p.batch_stride % 4) == 0 &&
         (p.out_row_stride % 4) == 0 && (p.out_batch_stride % 4) == 0 && al(p.q) && al(p.k) && al(p.v) &&
         al(p.out) && (p.out != nullptr || (p.out16_hi && p.out16_lo)) && al(p.out16_hi) && al(p.out16_lo) &&
         p.err_word != nullptr;
}

cudaError_t launch_attention_tc(const AttentionParams& p, cudaStream_t st) {
  if (!attention_tc_supported(p)) return cudaErrorInvalidValue;
  AttnTcDev d;
  d.q = p.q; d.k = p.k; d.v = p.v;
  d.row_stride = p.row_stride; d.batch_stride = p.batch_stride;
  d.out = p.out; d.out_row_stride = p.out_row_stride; d.out_batch_stride = p.out_batch_stride;
  d.o16_hi = static_cast<uint2*>(p.out16_hi); d.o16_lo = static_cast<uint2*>(p.out16_lo);
  d.heads = p.heads; d.tokens = p.tokens;
  d.scale = p.scale; d.scale_mode = p.scale ? p.scale_mode : 0;
  d.err = p.err_word;
  d.dbg = nullptr;
  // Debug toggle: ALTIUS_CUDA_ATTN_STAMPS=1 prints the phase clocks of CTA (0, 0) after every launch.
  static const bool stamps = std::getenv("ALTIUS_CUDA_ATTN_STAMPS") != nullptr;
  if (stamps) cudaGetSymbolAddress(reinterpret_cast<void**>(&d.dbg), g_attn_stamps);
  const int bh = p.batch * p.heads;
  cudaError_t e = p.tokens <= 128 ? launch_nb<8>(d, bh, st) : p.tokens <= 208 ? launch_nb<13>(d, bh, st) : launch_nb<16>(d, bh, st);
  if (stamps && e == cudaSuccess) {
    long long h[32];
    cudaStreamSynchronize(st);
    cudaMemcpyFromSymbol(h, g_attn_stamps, sizeof(h));
    std::fprintf(stderr, "attention_tc stamps:");
    for (int i = 1; i <= 8; ++i) std::fprintf(stderr, " %lld", h[i] - h[0]);
    std::fprintf(stderr, " |");
    for (int i = 11; i <= 18; ++i) std::fprintf(stderr, " %lld", h[i] - h[0]);
    std::fprintf(stderr, "\n");
  }
  return e;
}

}  // namespace ac
