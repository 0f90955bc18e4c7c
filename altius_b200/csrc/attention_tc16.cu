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
//   warp 17       TMA producer (rows of 128 bytes, 128-byte swizzle): K of a unit as soon as the
//                 previous unit's last scores are complete; V into one of two buffers, Q into
//                 one of two buffers: the loads of a unit run under the products of the one before.
//   warp 16       allocates tensor memory; one thread issues the MMAs: the scores of item i + 1
//                 (into the other score buffer) before the P V products of item i, which take
//                 their A operand, P, from tensor memory, stage by stage as it is written.
//   warps 0-7     softmax group 0 (even items), warps 8-15 group 1 (odd items): two threads per
//                 query row, one per half of the key columns: pass 1 row maximum, pass 2
//                 e * 2^13 = 2^((s - max) log2 e + 13) by one FFMA and one ex2.approx, split into
//                 fp16 hi / lo (unscaled: P is at the top of fp16's range by construction) and
//                 written with tcgen05.st over the scores it came from (16 score columns ->
//                 8 columns of hi, 8 of lo); then O * (1 / sum) to global memory. Nothing but
//                 the output accumulator is shared by the groups, so their passes overlap.
//
// Tensor memory: scores, then P, of even items in columns [0, 208), of odd items in [224, 432),
// the output accumulator in [448, 512). V is used as stored, keys x head_dim with head_dim
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
constexpr int kMmaWarp = 16, kTmaWarp = 17;
constexpr int kLaunch = 18 * 32;
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
__device__ long long g_attn16_stamps[80];   // [0]: kernel entry; [1 + 6 item + k]: phase k of the item (first six items); [40 + 6 item + k]: the MMA thread
#define AT16_MSTAMP(i, k) do { if (p.dbg && blockIdx.x == 0 && (i) < 6) p.dbg[40 + 6 * (i) + (k)] = clock64(); } while (0)
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

// The three partial products of one 16-key chunk (lo * hi, hi * lo, hi * hi) in one statement:
// tcgen05.mma with the A operand in tensor memory (row r of A in lane r, 16 fp16 values of K in
// 8 consecutive 32-bit columns, element 2c in the low half of column c).
__device__ __forceinline__ void tc_mma3_f16_ta(uint32_t d_tmem, uint32_t a_hi, uint32_t a_lo, uint64_t b_hi, uint64_t b_lo,
                                               uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, t;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "setp.eq.b32 t, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%2], %3, %5, p;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %4, %5, t;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %3, %5, t;\n\t}"
      ::"r"(d_tmem), "r"(a_hi), "r"(a_lo), "l"(b_hi), "l"(b_lo), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void st16_issue(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
        "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Barrier of the two softmax warps of group g that share tensor-memory lane quarter q.
__device__ __forceinline__ void pair_sync(int g, int q) {
  asm volatile("bar.sync %0, 64;" ::"r"(1 + 4 * g + q) : "memory");
}

// NB = 16-key chunks: NS = 16 * NB >= tokens (NS <= 208: two score buffers fit tensor memory).
// The first NB0 chunks belong to column half 0, the rest to half 1; a stage = two chunks of a
// half, published to the MMA thread by one arrival per warp.
template <int NB, int SMODE>
__global__ void __launch_bounds__(kLaunch, 1)
attention_tc16_kernel(const __grid_constant__ CUtensorMap tm_q_hi, const __grid_constant__ CUtensorMap tm_q_lo,
                         const __grid_constant__ CUtensorMap tm_kv_hi, const __grid_constant__ CUtensorMap tm_kv_lo,
                         Attn16Dev p) {
  constexpr int NS = NB * 16;
  constexpr int kKvHalfBytes = NS * 128;      // K (or V) hi (or lo): NS rows of 128 bytes
  constexpr int NB0 = (NB + 1) / 2;           // chunks of the first column half
  constexpr int kStages = (NB0 + 1) / 2;
  static_assert(NS <= 208 && (kKvHalfBytes % 1024) == 0 && kStages <= 4, "two score buffers; whole swizzle atoms");
  extern __shared__ uint8_t at16_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(at16_smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* k_hi = smem;                        // + kKvHalfBytes: K lo
  uint8_t* v_base = k_hi + 2 * kKvHalfBytes;   // two buffers of V hi, V lo
  uint8_t* q_base = v_base + 4 * kKvHalfBytes; // two buffers of Q hi, Q lo
  uint64_t* bars = reinterpret_cast<uint64_t*>(q_base + 4 * kQHalfBytes);
  uint64_t* q_full = bars;                     // [2] TMA: Q of an item has landed in buffer i & 1
  uint64_t* q_free = bars + 2;                 // [2] the scores of the item are complete
  uint64_t* k_full = bars + 4;
  uint64_t* k_free = bars + 5;                 // the scores of a unit's last item are complete
  uint64_t* v_full = bars + 6;                 // [2] V of a unit has landed in buffer u & 1
  uint64_t* v_free = bars + 8;                 // [2] the last P V product of the unit is complete
  // One barrier per group wherever a group waits: a parity wait is only right for a waiter at
  // most one phase ahead, and a group may be a whole item ahead of the other.
  uint64_t* o_full = bars + 10;                // [2] the output accumulator of an item of group g is complete
  uint64_t* o_free = bars + 12;                // [2] ... has been read by the 8 warps of the group
  uint64_t* s_full = bars + 14;                // [2] scores complete in buffer j
  uint64_t* s_free = bars + 16;                // [2] the products that read P from buffer j are complete
  uint64_t* ready = bars + 18;                 // [2 groups][2 halves][4 stages] P written (4 warps)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 34);
  float* xch_all = reinterpret_cast<float*>(bars + 40);   // [2 groups][2 halves][128] row maxima, then row sums

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int T = p.tokens;
  const int n_tiles = (T + QM - 1) / QM;
  const int my_units = ((int)p.units - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
  const int n_items = my_units * n_tiles;
  bool ok = true;
  if (p.dbg && blockIdx.x == 0 && tid == 0) p.dbg[0] = clock64();

  if (tid == 0) {
    for (int i = 0; i < 12; ++i) mbar_init(&bars[i], 1);
    for (int j = 0; j < 2; ++j) {
      mbar_init(&o_free[j], 8);
      mbar_init(&s_full[j], 1);
      mbar_init(&s_free[j], 1);
    }
    for (int i = 0; i < 16; ++i) mbar_init(&ready[i], 4);
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

  if (warp == kTmaWarp) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      auto load_q = [&](int i, int tile, int h, int b) {
        const int qb = i & 1;
        if (i >= 2 && !mbar_wait(&q_free[qb], (uint32_t)(((i >> 1) - 1) & 1))) { atomicExch(p.err, 32); ok = false; return; }
        uint8_t* dst = q_base + qb * 2 * kQHalfBytes;
        mbar_arrive_expect_tx(&q_full[qb], 2 * kQHalfBytes);
        tma_load_3d(dst, &tm_q_hi, &q_full[qb], p.q_col + h * HD, tile * QM, b);
        tma_load_3d(dst + kQHalfBytes, &tm_q_lo, &q_full[qb], p.q_col + h * HD, tile * QM, b);
      };
      for (int u = 0; ok && u < my_units; ++u) {
        const int unit = (int)blockIdx.x + u * (int)gridDim.x;
        const int b = unit / p.heads, h = unit % p.heads;
        const int vb = u & 1;
        load_q(u * n_tiles, 0, h, b);
        if (!ok) break;
        if (u >= 1 && !mbar_wait(k_free, (uint32_t)((u - 1) & 1))) { atomicExch(p.err, 31); ok = false; break; }
        mbar_arrive_expect_tx(k_full, 2 * kKvHalfBytes);
        tma_load_3d(k_hi, &tm_kv_hi, k_full, p.k_col + h * HD, 0, b);
        tma_load_3d(k_hi + kKvHalfBytes, &tm_kv_lo, k_full, p.k_col + h * HD, 0, b);
        if (u >= 2 && !mbar_wait(&v_free[vb], (uint32_t)(((u >> 1) - 1) & 1))) { atomicExch(p.err, 33); ok = false; break; }
        uint8_t* vdst = v_base + vb * 2 * kKvHalfBytes;
        mbar_arrive_expect_tx(&v_full[vb], 2 * kKvHalfBytes);
        tma_load_3d(vdst, &tm_kv_hi, &v_full[vb], p.v_col + h * HD, 0, b);
        tma_load_3d(vdst + kKvHalfBytes, &tm_kv_lo, &v_full[vb], p.v_col + h * HD, 0, b);
        for (int tile = 1; ok && tile < n_tiles; ++tile) load_q(u * n_tiles + tile, tile, h, b);
      }
    }
  } else if (warp == kMmaWarp) {
    // ---------------- MMA issue ----------------
    if (lane == 0) {
      const uint32_t idesc_s = (1u << 4) | ((uint32_t)(NS >> 3) << 17) | ((uint32_t)(QM >> 4) << 24);
      const uint32_t idesc_o = (1u << 4) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(QM >> 4) << 24);   // B MN-major
      auto issue_s = [&](int i) {
        const int u = i / n_tiles, tile = i - u * n_tiles, j = i & 1;
        AT16_MSTAMP(i, 0);
        if (!mbar_wait(&q_full[j], (uint32_t)((i >> 1) & 1))) { atomicExch(p.err, 34); ok = false; return; }
        if (tile == 0 && !mbar_wait(k_full, (uint32_t)(u & 1))) { atomicExch(p.err, 35); ok = false; return; }
        if (i >= 2 && !mbar_wait(&s_free[j], (uint32_t)(((i >> 1) - 1) & 1))) { atomicExch(p.err, 36); ok = false; return; }
        tc_fence_after();
        AT16_MSTAMP(i, 1);
        const uint32_t d = tmem_base + (j ? kS1Col : 0u);
        const uint32_t q_hi = smem_u32(q_base + j * 2 * kQHalfBytes);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const uint32_t qa = q_hi + kk * 32, ka = smem_u32(k_hi) + kk * 32;
          const uint64_t a_hi = desc_k128(qa), a_lo = desc_k128(qa + kQHalfBytes);
          const uint64_t b_hi = desc_k128(ka), b_lo = desc_k128(ka + kKvHalfBytes);
          tc_mma_f16(d, a_lo, b_hi, idesc_s, kk ? 1u : 0u);
          tc_mma_f16(d, a_hi, b_lo, idesc_s, 1u);
          tc_mma_f16(d, a_hi, b_hi, idesc_s, 1u);
        }
        tc_commit(&s_full[j]);
        tc_commit(&q_free[j]);
        if (tile == n_tiles - 1) tc_commit(k_free);
      };
      auto issue_pv = [&](int i) {
        const int u = i / n_tiles, tile = i - u * n_tiles, g = i & 1, vb = u & 1;
        AT16_MSTAMP(i, 2);
        if (tile == 0 && !mbar_wait(&v_full[vb], (uint32_t)((u >> 1) & 1))) { atomicExch(p.err, 37); ok = false; return; }
        if (i >= 1 && !mbar_wait(&o_free[g ^ 1], (uint32_t)(((i - 1) >> 1) & 1))) { atomicExch(p.err, 38); ok = false; return; }
        AT16_MSTAMP(i, 3);
        const uint32_t pcol = tmem_base + (g ? kS1Col : 0u);
        const uint64_t v_desc = desc_mn128(smem_u32(v_base + vb * 2 * kKvHalfBytes));   // + 128 per chunk of 16 keys (2048 bytes)
        // When the products are behind the softmax, all of P is there already: one test of each
        // half's last stage (stages complete in order) replaces the waits stage by stage.
        const uint32_t rpar = (uint32_t)((i >> 1) & 1);
        const bool all_there = mbar_test(&ready[(g * 2) * 4 + (NB0 + 1) / 2 - 1], rpar) &&
                               mbar_test(&ready[(g * 2 + 1) * 4 + (NB - NB0 + 1) / 2 - 1], rpar);
        if (all_there) tc_fence_after();
        bool first = true;
#pragma unroll 1
        for (int n = 0; n < 2 * kStages; ++n) {
          const int st = n >> 1, hf = n & 1;
          const int cnt = hf ? NB - NB0 : NB0;
          if (2 * st >= cnt) continue;
          if (!all_there) {
            if (!mbar_wait(&ready[(g * 2 + hf) * 4 + st], rpar)) { atomicExch(p.err, 39); ok = false; return; }
            tc_fence_after();
          }
          if (n == 0) AT16_MSTAMP(i, 4);
          const int c_end = 2 * st + 2 < cnt ? 2 * st + 2 : cnt;
          for (int c = 2 * st; c < c_end; ++c) {
            const int chunk = (hf ? NB0 : 0) + c;
            const uint32_t a_hi = pcol + (uint32_t)(16 * chunk), a_lo = a_hi + 8u;
            const uint64_t b_hi = v_desc + (uint64_t)(chunk * 128), b_lo = b_hi + (uint64_t)(kKvHalfBytes >> 4);
            tc_mma3_f16_ta(tmem_base + kOCol, a_hi, a_lo, b_hi, b_lo, idesc_o, first ? 0u : 1u);
            first = false;
          }
        }
        AT16_MSTAMP(i, 5);
        tc_commit(&o_full[g]);
        tc_commit(&s_free[g]);
        if (tile == n_tiles - 1) tc_commit(&v_free[vb]);
      };
      if (n_items > 0) issue_s(0);
      for (int i = 0; ok && i < n_items; ++i) {
        if (i + 1 < n_items) issue_s(i + 1);
        if (ok) issue_pv(i);
      }
      // The last commit of all: no arrival is still on its way to this CTA's barriers at exit.
      if (ok && my_units > 0 &&
          !mbar_wait(&v_free[(my_units - 1) & 1], (uint32_t)(((my_units - 1) >> 1) & 1)))
        atomicExch(p.err, 40);
    }
  } else {
    // ---------------- softmax groups: two threads per row, one per column half ----------------
    const int g = warp >> 3, wg = warp & 7;
    const int q = wg & 3, hf = wg >> 2;          // tensor-memory lane quarter, column half
    const int row = q * 32 + lane;
    const int c_begin = hf ? NB0 : 0, c_count = hf ? NB - NB0 : NB0;
    float* xch = xch_all + g * 2 * QM;
    const uint32_t trow = tmem_base + ((uint32_t)(q * 32) << 16);
    const uint32_t srow = trow + (g ? kS1Col : 0u);
    uint64_t* my_ready = ready + (g * 2 + hf) * 4;
    // Scores arrive as (q * 2^8) . (k * 2^8); they enter the exponential as t = acc * c1 with
    // c1 = 2^-16 * log2(e) (* | /) scale, so that e = 2^(t - max t) is one FFMA and one
    // ex2.approx per score (2 ulp; the CUDA-core kernel keeps the reference's polynomial).
    const float kLog2e = 1.44269504088896341f;
    const float sc = SMODE ? __ldg(p.scale) : 1.f;
    const float c1 = __fmul_rn(SMODE == 1 ? __fmul_rn(sc, kLog2e) : (SMODE == 2 ? __fdiv_rn(kLog2e, sc) : kLog2e),
                               kFixedUnscale * kFixedUnscale);
    float seen_max = 0.f;           // largest magnitude written as fixed-scale halves
#pragma unroll 1
    for (int i = g; i < n_items; i += 2) {
      const int u = i / n_tiles, tile = i - u * n_tiles;
      const int unit = (int)blockIdx.x + u * (int)gridDim.x;
      const int b = unit / p.heads, h = unit % p.heads;
      const int q0 = tile * QM;
      if (ok && !warp_mbar_wait(&s_full[g], (uint32_t)((i >> 1) & 1), lane)) { atomicExch(p.err, 41); ok = false; }
      tc_fence_after();
      AT16_STAMP(0);
      // ---- pass 1: row maximum of the scaled scores (a chunk past the half's last is masked or
      // belongs to the other half: neither changes the row maximum) ----
      float m = CUDART_NAN_F;
#pragma unroll 1
      for (int ci = 0; ci < c_count; ci += 2) {
        const int c0 = (c_begin + ci) * 16;
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
      // ---- pass 2: P = e * 2^13 as fp16 hi / lo over the scores it came from, running sum ----
      const float m13 = __fsub_rn(m, 13.f);
      float sum = 0.f;
      AT16_STAMP(1);
      AT16_STAMP(2);
#pragma unroll 1
      for (int ci = 0; ci < c_count; ++ci) {
        const int c0 = (c_begin + ci) * 16;
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
        uint32_t w[16];                          // columns 0-7: hi of keys 2c, 2c + 1; columns 8-15: lo
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint2 h2, l2;
          f16_split_plain(make_float4(e[4 * j], e[4 * j + 1], e[4 * j + 2], e[4 * j + 3]), h2, l2);
          w[2 * j] = h2.x; w[2 * j + 1] = h2.y;
          w[8 + 2 * j] = l2.x; w[8 + 2 * j + 1] = l2.y;
        }
        st16_issue(srow + (uint32_t)c0, w);
        if ((ci & 1) || ci == c_count - 1) {     // a stage is complete
          tc_wait_st();
          tc_fence_before();
          __syncwarp();
          if (ok && lane == 0) mbar_arrive(&my_ready[ci >> 1]);
        }
      }
      AT16_STAMP(3);
      xch[hf * QM + row] = sum;
      pair_sync(g, q);
      sum = __fadd_rn(xch[row], xch[QM + row]);
      pair_sync(g, q);                           // the next item's maxima overwrite the sums
      // ---- O = acc * (1 / sum) * 2^-8: this thread's row, 32 of the 64 columns ----
      if (ok && !warp_mbar_wait(&o_full[g], (uint32_t)((i >> 1) & 1), lane)) { atomicExch(p.err, 43); ok = false; }
      tc_fence_after();
      AT16_STAMP(4);
      uint32_t o[32];
      tc_ld_32x32(trow + kOCol + (uint32_t)(hf * 32), o);
      tc_fence_before();
      __syncwarp();
      if (ok && lane == 0) mbar_arrive(&o_free[g]);
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
            seen_max = split_track(split_track(seen_max, y0), y1);
          }
        }
      }
      AT16_STAMP(5);
    }
    if (p.o16_hi) split_report_warp(split_seen_fixed_of_max(seen_max), p.err);   // out of range, or all tiny
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
  constexpr int kDyn = 6 * NS * 128 /*K, two V*/ + 4 * kQHalfBytes /*two Q*/ + 320 /*barriers*/ +
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
  // Debug toggle: ALTIUS_CUDA_ATTN_STAMPS=1 prints the phase clocks of CTA 0 after every launch. Softmax
  // warp 0 of each group, per item: scores complete, pass 1 done (twice), pass 2 done, output complete,
  // written. MMA thread, per item: scores entered, their waits over, P V entered, its waits over, first
  // stage of P there, last product issued.
  static const bool stamps = std::getenv("ALTIUS_CUDA_ATTN_STAMPS") != nullptr;
  if (stamps) cudaGetSymbolAddress(reinterpret_cast<void**>(&d.dbg), g_attn16_stamps);
  const cudaError_t e = p.tokens <= 128 ? launch16_nb<8>(p, d, st) : launch16_nb<13>(p, d, st);
  if (stamps && e == cudaSuccess) {
    long long h[80];
    cudaStreamSynchronize(st);
    cudaMemcpyFromSymbol(h, g_attn16_stamps, sizeof(h));
    for (int base = 1; base <= 40; base += 39) {
      std::fprintf(stderr, base == 1 ? "attention_tc16 stamps:" : "attention_tc16 MMA thread:");
      for (int i = 0; i < 6; ++i) {
        std::fprintf(stderr, " |");
        for (int k = 0; k < 6; ++k) std::fprintf(stderr, " %lld", h[base + 6 * i + k] - h[0]);
      }
      std::fprintf(stderr, "\n");
    }
  }
  return e;
}

}  // namespace ac
