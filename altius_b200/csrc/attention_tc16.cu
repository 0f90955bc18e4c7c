// Fused multi-head attention core fed by TMA from fp16 operands: the same operator chain as
// attention_tc.cu (Split / head Reshape / Transpose / MatMul / Mul / Softmax / MatMul /
// Transpose / Reshape of crates/session_interpreter/src/session.rs:621-682, 990-1026,
// 1179-1278, 1488-1512), for the case where the projection GEMM in front has written its
// [B, T, 3D] result as two fp16 arrays on one fixed scale (f16_split_fixed: X = x * 2^8,
// hi = rn(X), lo = rn(X - hi)). With both halves on one scale every product is three
// kind::f16 MMAs into ONE fp32 accumulator (lo * hi, hi * lo, hi * hi), so the scores need
// 208 tensor-memory columns instead of 416 and two score buffers fit beside the output.
//
// Persistent: a CTA walks (image, head) units and their query tiles of 128 rows; an item is
// one (unit, tile).
//
//   warp 17       TMA producer: K and V of a unit (rows of 128 bytes, 128-byte swizzle) as soon
//                 as the previous unit's last product has read them, Q of the next item as soon
//                 as the current scores are complete: loads run under the softmax.
//   warp 16       allocates tensor memory; one thread issues the MMAs: the scores of item i + 1
//                 (into the other score buffer) before the P V products of item i, which it
//                 feeds block by block from a ring of P tiles.
//   warps 0-7     softmax group 0 (even items), warps 8-15 group 1 (odd items): two threads per
//                 query row, one per half of the key columns: pass 1 row maximum, pass 2
//                 e * 2^13 = 2^((s - max) log2 e + 13) by one FFMA and one ex2.approx, split into
//                 fp16 hi / lo (unscaled: P is at the top of fp16's range by construction) and
//                 stored as the A operand of P V; then O * (1 / sum) to global memory. While one
//                 group runs pass 2, the other finishes its output and runs pass 1 of the next
//                 item, so the tensor pipe and the exponentials of consecutive items overlap.
//
// Tensor memory: scores of even items in columns [0, 208), of odd items in [224, 432), the
// output accumulator in [448, 512). V is used as stored, keys x head_dim with head_dim
// contiguous: the B operand of P V is MN-major (128-byte swizzle, 8-key groups 1024 bytes
// apart). Every mbarrier wait is bounded; on expiry the kernel records a code in the error
// word and runs to its end without waiting again.
#include <cuda.h>

#include <cstdio>
#include <cstdlib>

#include "kernels.h"
#include "ref_math.cuh"
#include "tc_common.cuh"

namespace ac {
namespace {

using namespace tc;

constexpr int HD = 64;                        // head dimension
constexpr int QM = 128;                       // query rows per item = tensor-memory lanes
constexpr int kSoftWarps = 16;
constexpr int kMmaWarp = 16, kTmaWarp = 17;
constexpr int kLaunch = 18 * 32;
constexpr int kSlots = 4;                     // P ring depth
constexpr int kSlotBytes = 2 * QM * 64;       // hi + lo of a [128 x 32 keys] fp16 block of P
constexpr int kQHalfBytes = QM * 128;         // Q hi (or lo): 128 rows of 128 bytes
constexpr uint32_t kS1Col = 224, kOCol = 448, kTmemCols = 512;

struct Attn16Dev {
  float* out; long long out_row_stride, out_batch_stride;   // may be null when o16_hi / o16_lo are given
  uint2* o16_hi; uint2* o16_lo;   // the result as fp16 hi / lo halves on the fixed scale (f16_split_fixed), or null
  int heads, tokens, units;
  int q_col, k_col, v_col;        // first column of each operand in the [B, T, C] arrays
  const float* scale; int scale_mode;   // 0 none, 1 multiply, 2 divide
  int* err;
  long long* dbg;   // phase time stamps of CTA 0 when not null (debug toggle)
};
__device__ long long g_attn16_stamps[40];   // [0]: kernel entry; [1 + 6 item + k]: phase k of the item (first six items)
#define AT16_STAMP(k) do { if (p.dbg && blockIdx.x == 0 && (warp & 7) == 0 && lane == 0 && i < 6) p.dbg[1 + 6 * i + (k)] = clock64(); } while (0)

// K-major tile with rows of 128 bytes and the 128-byte swizzle: 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_k128(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;                   // leading byte offset (ignored for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;         // stride byte offset
  d |= (uint64_t)1 << 46;                   // descriptor version for this architecture
  d |= (uint64_t)2 << 61;                   // 128-byte swizzle
  return d;
}
// MN-major tile of 64 fp16 columns (one 128-byte swizzle atom wide): k-rows of 128 bytes, 8-row
// groups 1024 bytes apart (stride byte offset); a second atom along N does not exist here.
__device__ __forceinline__ uint64_t desc_mn128(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)(1024 >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// K-major tile with rows of 64 bytes and the 64-byte swizzle (the P ring).
__device__ __forceinline__ uint64_t desc_k64(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(512 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)4 << 61;
  return d;
}
__device__ __forceinline__ uint32_t sw64_off(int row, int chunk) {
  return (uint32_t)((row >> 3) * 512 + (row & 7) * 64 + ((chunk ^ ((row & 7) >> 1)) << 4));
}

__device__ __forceinline__ void ld16_issue(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]),
        "=r"(v[15])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Barrier of the two softmax warps of group g that share tensor-memory lane quarter q.
__device__ __forceinline__ void pair_sync(int g, int q) {
  asm volatile("bar.sync %0, 64;" ::"r"(1 + 4 * g + q) : "memory");
}

// NB = 16-key blocks: NS = 16 * NB >= tokens (NS <= 208: two score buffers fit tensor memory).
template <int NB, int SMODE>
__global__ void __launch_bounds__(kLaunch, 1)
attention_tc16_kernel(const __grid_constant__ CUtensorMap tm_q_hi, const __grid_constant__ CUtensorMap tm_q_lo,
                      const __grid_constant__ CUtensorMap tm_kv_hi, const __grid_constant__ CUtensorMap tm_kv_lo,
                      Attn16Dev p) {
  constexpr int NS = NB * 16;
  constexpr int kKvHalfBytes = NS * 128;      // K (or V) hi (or lo): NS rows of 128 bytes
  constexpr int NBLK = (NB + 1) / 2;          // 32-key blocks of P
  constexpr int NBLK0 = (NBLK + 1) / 2;       // blocks of the first column half
  static_assert(NS <= 208 && (kKvHalfBytes % 1024) == 0, "two score buffers; whole swizzle atoms");
  extern __shared__ uint8_t at16_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(at16_smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* k_hi = smem;                        // + kKvHalfBytes: K lo
  uint8_t* v_hi = k_hi + 2 * kKvHalfBytes;     // + kKvHalfBytes: V lo
  uint8_t* q_hi = v_hi + 2 * kKvHalfBytes;     // + kQHalfBytes: Q lo
  uint8_t* ring = q_hi + 2 * kQHalfBytes;      // kSlots P blocks
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring + kSlots * kSlotBytes);
  uint64_t* q_full = bars;                     // TMA: Q of an item has landed
  uint64_t* q_free = bars + 1;                 // the scores of an item are complete: Q may be overwritten
  uint64_t* k_full = bars + 2;
  uint64_t* k_free = bars + 3;                 // the scores of a unit's last item are complete
  uint64_t* v_full = bars + 4;
  uint64_t* v_free = bars + 5;                 // the last P V product of a unit is complete
  uint64_t* o_full = bars + 6;                 // the output accumulator of an item is complete
  uint64_t* o_free = bars + 7;                 // ... has been read by the 8 warps of its group
  uint64_t* s_full = bars + 8;                 // [2] scores complete in buffer j
  uint64_t* s_free = bars + 10;                // [2] buffer j read for the last time (8 warps)
  uint64_t* ready = bars + 12;                 // [kSlots] P block written by the 128 threads of a half
  uint64_t* freeb = ready + kSlots;            // [kSlots] P block consumed by its MMAs
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(freeb + kSlots);
  // The ring is shared by the two groups, and a parity wait is only right for a waiter at most
  // one phase ahead: a group starts pass 2 of item i only after the other group has written the
  // last P block of item i - 1 (8 warps arrive here per item).
  uint64_t* p2_turn = bars + 21;
  float* xch_all = reinterpret_cast<float*>(bars + 32);   // [2 groups][2 halves][128] row maxima, then row sums

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int T = p.tokens;
  const int n_tiles = (T + QM - 1) / QM;
  const int my_units = ((int)p.units - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
  const int n_items = my_units * n_tiles;
  bool ok = true;
  if (p.dbg && blockIdx.x == 0 && tid == 0) p.dbg[0] = clock64();

  if (tid == 0) {
    for (int i = 0; i < 7; ++i) mbar_init(&bars[i], 1);
    mbar_init(o_free, 8);
    mbar_init(p2_turn, 8);
    mbar_init(&s_full[0], 1); mbar_init(&s_full[1], 1);
    mbar_init(&s_free[0], 8); mbar_init(&s_free[1], 8);
    for (int i = 0; i < kSlots; ++i) {
      mbar_init(&ready[i], QM);
      mbar_init(&freeb[i], 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(kTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Use number of ring slot (hf, par) at its m-th use inside item i: every item uses it the
  // same number of times.
  auto uses_per_item = [&](int hf, int par) {
    const int bc = hf ? NBLK - NBLK0 : NBLK0;
    return par ? bc / 2 : (bc + 1) / 2;
  };

  if (warp == kTmaWarp) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      for (int u = 0; ok && u < my_units; ++u) {
        const int unit = (int)blockIdx.x + u * (int)gridDim.x;
        const int b = unit / p.heads, h = unit % p.heads;
        if (u >= 1 && !mbar_wait(k_free, (uint32_t)((u - 1) & 1))) { atomicExch(p.err, 31); ok = false; break; }
        mbar_arrive_expect_tx(k_full, 2 * kKvHalfBytes);
        tma_load_3d(k_hi, &tm_kv_hi, k_full, p.k_col + h * HD, 0, b);
        tma_load_3d(k_hi + kKvHalfBytes, &tm_kv_lo, k_full, p.k_col + h * HD, 0, b);
        for (int tile = 0; ok && tile < n_tiles; ++tile) {
          const int i = u * n_tiles + tile;
          if (i >= 1 && !mbar_wait(q_free, (uint32_t)((i - 1) & 1))) { atomicExch(p.err, 32); ok = false; break; }
          mbar_arrive_expect_tx(q_full, 2 * kQHalfBytes);
          tma_load_3d(q_hi, &tm_q_hi, q_full, p.q_col + h * HD, tile * QM, b);
          tma_load_3d(q_hi + kQHalfBytes, &tm_q_lo, q_full, p.q_col + h * HD, tile * QM, b);
          if (tile == 0) {
            if (u >= 1 && !mbar_wait(v_free, (uint32_t)((u - 1) & 1))) { atomicExch(p.err, 33); ok = false; break; }
            mbar_arrive_expect_tx(v_full, 2 * kKvHalfBytes);
            tma_load_3d(v_hi, &tm_kv_hi, v_full, p.v_col + h * HD, 0, b);
            tma_load_3d(v_hi + kKvHalfBytes, &tm_kv_lo, v_full, p.v_col + h * HD, 0, b);
          }
        }
      }
    }
  } else if (warp == kMmaWarp) {
    // ---------------- MMA issue ----------------
    if (lane == 0) {
      const uint32_t idesc_s = (1u << 4) | ((uint32_t)(NS >> 3) << 17) | ((uint32_t)(QM >> 4) << 24);
      const uint32_t idesc_o = (1u << 4) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(QM >> 4) << 24);   // B MN-major
      auto issue_s = [&](int i) {
        const int u = i / n_tiles, tile = i - u * n_tiles, j = i & 1;
        if (!mbar_wait(q_full, (uint32_t)(i & 1))) { atomicExch(p.err, 34); ok = false; return; }
        if (tile == 0 && !mbar_wait(k_full, (uint32_t)(u & 1))) { atomicExch(p.err, 35); ok = false; return; }
        if (i >= 2 && !mbar_wait(&s_free[j], (uint32_t)(((i >> 1) - 1) & 1))) { atomicExch(p.err, 36); ok = false; return; }
        tc_fence_after();
        const uint32_t d = tmem_base + (j ? kS1Col : 0u);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const uint32_t qa = smem_u32(q_hi) + kk * 32, ka = smem_u32(k_hi) + kk * 32;
          const uint64_t a_hi = desc_k128(qa), a_lo = desc_k128(qa + kQHalfBytes);
          const uint64_t b_hi = desc_k128(ka), b_lo = desc_k128(ka + kKvHalfBytes);
          tc_mma_f16(d, a_lo, b_hi, idesc_s, kk ? 1u : 0u);
          tc_mma_f16(d, a_hi, b_lo, idesc_s, 1u);
          tc_mma_f16(d, a_hi, b_hi, idesc_s, 1u);
        }
        tc_commit(&s_full[j]);
        tc_commit(q_free);
        if (tile == n_tiles - 1) tc_commit(k_free);
      };
      auto issue_pv = [&](int i) {
        const int u = i / n_tiles, tile = i - u * n_tiles;
        if (tile == 0 && !mbar_wait(v_full, (uint32_t)(u & 1))) { atomicExch(p.err, 37); ok = false; return; }
        if (i >= 1 && !mbar_wait(o_free, (uint32_t)((i - 1) & 1))) { atomicExch(p.err, 38); ok = false; return; }
        bool first = true;
#pragma unroll 1
        for (int n = 0; n < 2 * NBLK0; ++n) {
          const int hf = n & 1, ib = n >> 1;
          const int blk = hf ? NBLK0 + ib : ib;
          if (blk >= NBLK) continue;
          const int slot = 2 * hf + (ib & 1);
          const int use = i * uses_per_item(hf, ib & 1) + (ib >> 1);
          if (!mbar_wait(&ready[slot], (uint32_t)(use & 1))) { atomicExch(p.err, 39); ok = false; return; }
          tc_fence_after();
          const int ksteps = (blk == NBLK - 1 && (NB & 1)) ? 1 : 2;   // an odd last block holds 16 keys
          for (int kk = 0; kk < ksteps; ++kk) {
            const uint32_t pa = smem_u32(ring + slot * kSlotBytes) + kk * 32;
            const uint32_t va = smem_u32(v_hi) + (uint32_t)(blk * 32 + kk * 16) * 128u;
            const uint64_t a_hi = desc_k64(pa), a_lo = desc_k64(pa + QM * 64);
            const uint64_t b_hi = desc_mn128(va), b_lo = desc_mn128(va + kKvHalfBytes);
            tc_mma_f16(tmem_base + kOCol, a_lo, b_hi, idesc_o, first ? 0u : 1u);
            tc_mma_f16(tmem_base + kOCol, a_hi, b_lo, idesc_o, 1u);
            tc_mma_f16(tmem_base + kOCol, a_hi, b_hi, idesc_o, 1u);
            first = false;
          }
          tc_commit(&freeb[slot]);
        }
        tc_commit(o_full);
        if (tile == n_tiles - 1) tc_commit(v_free);
      };
      if (n_items > 0) issue_s(0);
      for (int i = 0; ok && i < n_items; ++i) {
        if (i + 1 < n_items) issue_s(i + 1);
        if (ok) issue_pv(i);
      }
      // The last commit of all: no arrival is still on its way to this CTA's barriers at exit.
      if (ok && my_units > 0 && !mbar_wait(v_free, (uint32_t)((my_units - 1) & 1))) atomicExch(p.err, 40);
    }
  } else {
    // ---------------- softmax groups: two threads per row, one per column half ----------------
    const int g = warp >> 3, wg = warp & 7;
    const int q = wg & 3, hf = wg >> 2;          // tensor-memory lane quarter, column half
    const int row = q * 32 + lane;
    const int b_begin = hf ? NBLK0 : 0, b_count = hf ? NBLK - NBLK0 : NBLK0;
    float* xch = xch_all + g * 2 * QM;
    const uint32_t trow = tmem_base + ((uint32_t)(q * 32) << 16);
    const uint32_t srow = trow + (g ? kS1Col : 0u);
    // Scores arrive as (q * 2^8) . (k * 2^8); they enter the exponential as t = acc * c1 with
    // c1 = 2^-16 * log2(e) (* | /) scale, so that e = 2^(t - max t) is one FFMA and one
    // ex2.approx per score (2 ulp; the CUDA-core kernel keeps the reference's polynomial).
    const float kLog2e = 1.44269504088896341f;
    const float sc = SMODE ? __ldg(p.scale) : 1.f;
    const float c1 = __fmul_rn(SMODE == 1 ? __fmul_rn(sc, kLog2e) : (SMODE == 2 ? __fdiv_rn(kLog2e, sc) : kLog2e),
                               kFixedUnscale * kFixedUnscale);
    unsigned seen_out = 0;
#pragma unroll 1
    for (int i = g; i < n_items; i += 2) {
      const int u = i / n_tiles, tile = i - u * n_tiles;
      const int unit = (int)blockIdx.x + u * (int)gridDim.x;
      const int b = unit / p.heads, h = unit % p.heads;
      const int q0 = tile * QM;
      if (ok && !warp_mbar_wait(&s_full[g], (uint32_t)((i >> 1) & 1), lane)) { atomicExch(p.err, 41); ok = false; }
      tc_fence_after();
      AT16_STAMP(0);
      // ---- pass 1: row maximum of the scaled scores ----
      float m = CUDART_NAN_F;
#pragma unroll 1
      for (int bi = 0; bi < b_count; ++bi) {
        const int c0 = (b_begin + bi) * 32;      // columns past NS read junk that is masked
        uint32_t v[2][16];
        ld16_issue(srow + (uint32_t)c0, v[0]);
        ld16_issue(srow + (uint32_t)(c0 + 16), v[1]);
        tc_wait_ld();
        float m0 = CUDART_NAN_F, m1 = CUDART_NAN_F;
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const float t0 = __fmul_rn(__uint_as_float(v[0][e]), c1), t1 = __fmul_rn(__uint_as_float(v[1][e]), c1);
          m0 = fmaxf(c0 + e < T ? t0 : CUDART_NAN_F, m0);
          m1 = fmaxf(c0 + 16 + e < T ? t1 : CUDART_NAN_F, m1);
        }
        m = fmaxf(fmaxf(m0, m1), m);
      }
      xch[hf * QM + row] = m;
      pair_sync(g, q);
      m = fmaxf(xch[QM + row], xch[row]);
      pair_sync(g, q);                           // both have read before the sums overwrite
      // ---- pass 2: P = e * 2^13 as fp16 hi / lo into the ring, running sum ----
      const float m13 = __fsub_rn(m, 13.f);
      float sum = 0.f;
      AT16_STAMP(1);
      if (ok && i >= 1 && !warp_mbar_wait(p2_turn, (uint32_t)((i - 1) & 1), lane)) { atomicExch(p.err, 44); ok = false; }
      AT16_STAMP(2);
#pragma unroll 1
      for (int bi = 0; bi < b_count; ++bi) {
        const int blk = b_begin + bi;
        const int slot = 2 * hf + (bi & 1);
        const int use = i * uses_per_item(hf, bi & 1) + (bi >> 1);
        if (ok && use >= 1 && !warp_mbar_wait(&freeb[slot], (uint32_t)((use - 1) & 1), lane)) { atomicExch(p.err, 42); ok = false; }
        uint8_t* sl = ring + slot * kSlotBytes;
#pragma unroll
        for (int h16 = 0; h16 < 2; ++h16) {
          const int c0 = blk * 32 + h16 * 16;
          uint32_t v[16];
          ld16_issue(srow + (uint32_t)c0, v);
          tc_wait_ld();
          float e[16];
#pragma unroll
          for (int x = 0; x < 16; ++x) {
            const float ev = ex2_approx(fmaf(__uint_as_float(v[x]), c1, -m13));
            e[x] = c0 + x < T ? ev : 0.f;
          }
#pragma unroll
          for (int x = 0; x < 16; ++x) sum = __fadd_rn(sum, e[x]);   // + 0 for masked columns: exact
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            uint2 h0, l0, h1, l1;
            f16_split_plain(make_float4(e[8 * j], e[8 * j + 1], e[8 * j + 2], e[8 * j + 3]), h0, l0);
            f16_split_plain(make_float4(e[8 * j + 4], e[8 * j + 5], e[8 * j + 6], e[8 * j + 7]), h1, l1);
            const uint32_t off = sw64_off(row, 2 * h16 + j);
            *reinterpret_cast<uint4*>(sl + off) = make_uint4(h0.x, h0.y, h1.x, h1.y);
            *reinterpret_cast<uint4*>(sl + QM * 64 + off) = make_uint4(l0.x, l0.y, l1.x, l1.y);
          }
        }
        fence_proxy_async();
        if (ok) mbar_arrive(&ready[slot]);
      }
      AT16_STAMP(3);
      // The score buffer has been read for the last time: the scores of item i + 2 may overwrite it.
      tc_fence_before();
      __syncwarp();
      if (ok && lane == 0) {
        mbar_arrive(&s_free[g]);
        mbar_arrive(p2_turn);
      }
      xch[hf * QM + row] = sum;
      pair_sync(g, q);
      sum = __fadd_rn(xch[row], xch[QM + row]);
      pair_sync(g, q);                           // the next item's maxima overwrite the sums
      // ---- O = acc * (1 / sum) * 2^-8: this thread's row, 32 of the 64 columns ----
      if (ok && !warp_mbar_wait(o_full, (uint32_t)(i & 1), lane)) { atomicExch(p.err, 43); ok = false; }
      tc_fence_after();
      AT16_STAMP(4);
      uint32_t o[32];
      tc_ld_32x32(trow + kOCol + (uint32_t)(hf * 32), o);
      tc_fence_before();
      __syncwarp();
      if (ok && lane == 0) mbar_arrive(o_free);
      const float recip = __fmul_rn(__fdiv_rn(1.f, sum), kFixedUnscale);
      const int r = q0 + row;
      if (ok && r < T) {
        const long long ob = (long long)b * p.out_batch_stride + (long long)r * p.out_row_stride + h * HD + hf * 32;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float4 y0 = make_float4(__fmul_rn(__uint_as_float(o[8 * j]), recip), __fmul_rn(__uint_as_float(o[8 * j + 1]), recip),
                                        __fmul_rn(__uint_as_float(o[8 * j + 2]), recip), __fmul_rn(__uint_as_float(o[8 * j + 3]), recip));
          const float4 y1 = make_float4(__fmul_rn(__uint_as_float(o[8 * j + 4]), recip), __fmul_rn(__uint_as_float(o[8 * j + 5]), recip),
                                        __fmul_rn(__uint_as_float(o[8 * j + 6]), recip), __fmul_rn(__uint_as_float(o[8 * j + 7]), recip));
          if (p.out) {
            *reinterpret_cast<float4*>(p.out + ob + 8 * j) = y0;
            *reinterpret_cast<float4*>(p.out + ob + 8 * j + 4) = y1;
          }
          if (p.o16_hi) {   // for the projection GEMM that takes this result as its pre-split A
            uint2 h0, l0, h1, l1;
            f16_split_fixed(y0, h0, l0);
            f16_split_fixed(y1, h1, l1);
            const long long o4 = (ob + 8 * j) >> 2;      // uint2 index; even: 16-byte aligned
            *reinterpret_cast<uint4*>(p.o16_hi + o4) = make_uint4(h0.x, h0.y, h1.x, h1.y);
            *reinterpret_cast<uint4*>(p.o16_lo + o4) = make_uint4(l0.x, l0.y, l1.x, l1.y);
            seen_out |= split_seen_fixed(y0) | split_seen_fixed(y1);
          }
        }
      }
      AT16_STAMP(5);
    }
    if (p.o16_hi) split_report_warp(seen_out, p.err);   // out of range, or all tiny
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols));
  }
}

// 3-D map over a row-major [batch, rows, cols] fp16 array: boxes of 64 columns (128 bytes, the
// 128-byte swizzle) x box_rows rows; rows past `rows` are zero-filled.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);
bool make_map16(CUtensorMap* map, const void* base, int64_t cols, int64_t rows, int64_t batch, int64_t ld,
                int64_t batch_stride, int box_rows) {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  if (!fn) return false;
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)batch_stride * 2};
  cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int NB, int SMODE>
cudaError_t launch16_nb_mode(const Attention16Params& p, const Attn16Dev& d, cudaStream_t st) {
  constexpr int NS = NB * 16;
  constexpr int kDyn = 4 * NS * 128 + 2 * kQHalfBytes + kSlots * kSlotBytes + 256 /*barriers*/ +
                       2 * 2 * QM * 4 /*row exchange*/ + 1024 /*alignment*/;
  static_assert(kDyn <= 227 * 1024, "shared memory per CTA");
  static unsigned long long attr_done = 0;
  cudaError_t e = ensure_dynamic_smem(attention_tc16_kernel<NB, SMODE>, kDyn, &attr_done);
  if (e != cudaSuccess) return e;
  CUtensorMap q_hi, q_lo, kv_hi, kv_lo;
  const int64_t bs = (int64_t)p.tokens * p.ld16;
  if (!make_map16(&q_hi, p.qkv16_hi, p.ld16, p.tokens, p.batch, p.ld16, bs, QM) ||
      !make_map16(&q_lo, p.qkv16_lo, p.ld16, p.tokens, p.batch, p.ld16, bs, QM) ||
      !make_map16(&kv_hi, p.qkv16_hi, p.ld16, p.tokens, p.batch, p.ld16, bs, NS) ||
      !make_map16(&kv_lo, p.qkv16_lo, p.ld16, p.tokens, p.batch, p.ld16, bs, NS))
    return cudaErrorInvalidValue;
  const int grid = std::min(d.units, device_sm_count());
  attention_tc16_kernel<NB, SMODE><<<grid, kLaunch, kDyn, st>>>(q_hi, q_lo, kv_hi, kv_lo, d);
  return cudaGetLastError();
}

template <int NB>
cudaError_t launch16_nb(const Attention16Params& p, const Attn16Dev& d, cudaStream_t st) {
  if (d.scale_mode == 1) return launch16_nb_mode<NB, 1>(p, d, st);
  if (d.scale_mode == 2) return launch16_nb_mode<NB, 2>(p, d, st);
  return launch16_nb_mode<NB, 0>(p, d, st);
}

}  // namespace

bool attention_tc16_shape_ok(int head_dim, int tokens, int64_t ld16, int64_t q_col, int64_t k_col, int64_t v_col,
                             int64_t out_row_stride, int64_t out_batch_stride) {
  return head_dim == HD && tokens > 64 && tokens <= 208 && ld16 > 0 && (ld16 % 8) == 0 && (q_col % 8) == 0 &&
         (k_col % 8) == 0 && (v_col % 8) == 0 && q_col >= 0 && k_col >= 0 && v_col >= 0 &&
         (out_row_stride % 8) == 0 && (out_batch_stride % 8) == 0;
}

bool attention_tc16_supported(const Attention16Params& p) {
  auto al = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  return attention_tc16_shape_ok(p.head_dim, p.tokens, p.ld16, p.q_col, p.k_col, p.v_col, p.out_row_stride,
                                 p.out_batch_stride) &&
         p.batch >= 1 && p.heads >= 1 && p.qkv16_hi && p.qkv16_lo && al(p.qkv16_hi) && al(p.qkv16_lo) &&
         al(p.out) && al(p.out16_hi) && al(p.out16_lo) && (p.out != nullptr || (p.out16_hi && p.out16_lo)) &&
         (p.out16_hi == nullptr) == (p.out16_lo == nullptr) && p.err_word != nullptr &&
         (int64_t)std::max(std::max(p.q_col, p.k_col), p.v_col) + (int64_t)p.heads * HD <= p.ld16;
}

cudaError_t launch_attention_tc16(const Attention16Params& p, cudaStream_t st) {
  if (!attention_tc16_supported(p)) return cudaErrorInvalidValue;
  Attn16Dev d;
  d.out = p.out; d.out_row_stride = p.out_row_stride; d.out_batch_stride = p.out_batch_stride;
  d.o16_hi = static_cast<uint2*>(p.out16_hi); d.o16_lo = static_cast<uint2*>(p.out16_lo);
  d.heads = p.heads; d.tokens = p.tokens; d.units = p.batch * p.heads;
  d.q_col = (int)p.q_col; d.k_col = (int)p.k_col; d.v_col = (int)p.v_col;
  d.scale = p.scale; d.scale_mode = p.scale ? p.scale_mode : 0;
  d.err = p.err_word;
  d.dbg = nullptr;
  // Debug toggle: ALTIUS_CUDA_ATTN_STAMPS=1 prints the phase clocks of CTA 0 after every launch
  // (per item: scores complete, pass 1 done, turn for pass 2, pass 2 done, output complete, written).
  static const bool stamps = std::getenv("ALTIUS_CUDA_ATTN_STAMPS") != nullptr;
  if (stamps) cudaGetSymbolAddress(reinterpret_cast<void**>(&d.dbg), g_attn16_stamps);
  const cudaError_t e = p.tokens <= 128 ? launch16_nb<8>(p, d, st) : launch16_nb<13>(p, d, st);
  if (stamps && e == cudaSuccess) {
    long long h[40];
    cudaStreamSynchronize(st);
    cudaMemcpyFromSymbol(h, g_attn16_stamps, sizeof(h));
    std::fprintf(stderr, "attention_tc16 stamps:");
    for (int i = 0; i < 6; ++i) {
      std::fprintf(stderr, " |");
      for (int k = 0; k < 6; ++k) std::fprintf(stderr, " %lld", h[1 + 6 * i + k] - h[0]);
    }
    std::fprintf(stderr, "\n");
  }
  return e;
}

}  // namespace ac
