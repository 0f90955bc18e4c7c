// Tensor-core GEMM for sm_100a: tcgen05.mma with the accumulators in tensor memory,
// operands staged in shared memory by TMA, split operands for fp32 fidelity.
//
//   C[b] = epilogue( A[b] (M x K, K contiguous) * B[b]^T (B stored N x K, K contiguous) )
//
// B may also be given K x N (N contiguous: a convolution's input planes or column buffer with
// the filter matrix as A, the value operand of a batched product): its tiles are then MN-major
// in shared memory (3xTF32 only). Either operand may be shared by the whole batch (stride 0).
//
// It replaces the cblas_sgemm the reference calls for MatMul / Gemm / Conv2d
// (crates/session_interpreter/src/gemm.rs:36-51, session.rs:621-794,
// conv2d.rs:145-209). Two ways of getting fp32-level products out of narrow MMAs:
//   3xTF32   x_hi = x rounded to TF32, x_lo = (x - x_hi) rounded to TF32 (x - x_hi is exact
//            in fp32); a_lo*b_hi + a_hi*b_lo + a_hi*b_hi as three kind::tf32 MMAs into one
//            accumulator. The dropped a_lo*b_lo term and the rounding of x_lo are each below
//            2^-22 relative.
//   fp16 split (constant B)  x_hi = x rounded to fp16, x_lo = ((x - x_hi) * 2^11) rounded to
//            fp16 (the scaling keeps x_lo out of the fp16 subnormals); a_hi*b_hi into one
//            accumulator, a_lo*b_hi + a_hi*b_lo into a second one that the epilogue adds
//            scaled by 2^-11. Same 22 bits per operand, half the operand bytes and twice the
//            MMA rate. |x| must not exceed 65504: B is checked when it is split at load time,
//            A by the splitters, which leave kRangeCode in the error word (the host then
//            repeats the run on the 3xTF32 path).
//
// Persistent CTAs (one per SM) walk the 128 x BN output tiles:
//   warp 16     TMA producer: one elected thread issues cp.async.bulk.tensor loads (boxes of
//               64-byte rows, 64-byte swizzle; the fp32 rows of A in the fp16 mode: 128-byte
//               rows, no swizzle) into a ring of stages, completion on an mbarrier per stage;
//   warps 0-7   splitters (two groups on alternate stages). TF32: rewrite the A tile as x_hi
//               in place and write x_lo beside it (the same for the B tile unless B is a
//               constant whose split was prepared at load time and arrives by TMA). fp16: read
//               the fp32 rows of A into registers, meet at a named barrier, write the fp16
//               hi / lo tiles over them;
//   warp 17     one thread issues the tcgen05.mma stream and tcgen05.commit into an
//               accumulator set in tensor memory (two sets when they fit 512 columns);
//   warps 8-15  epilogue of the other set (two warps per tensor-memory lane quarter, half of
//               the tile's columns each): tcgen05.ld, a shared-memory transpose to
//               row-contiguous float4s, bias / activation / residual, full-line global stores.
// Tiles beyond the last whole round of the grid are cut along K into slices (one per
// otherwise idle SM) whose unreduced accumulators go to a workspace; a small second kernel
// adds them in slice order and applies the epilogue.
// Every mbarrier wait is bounded: on expiry the kernel records a code in the
// error word, drains, frees its tensor memory and returns.
#include <cuda.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <mutex>

#include "kernels.h"
#include "ref_math.cuh"
#include "tc_common.cuh"

namespace ac {
namespace {

using namespace tc;

constexpr int BM = 128;
constexpr int BK = 16;                       // floats of K per stage in the TF32 modes (64-byte rows)
constexpr int BK16 = 32;                     // floats of K per stage in the fp16 mode (64-byte rows of halves)
constexpr int kSplitGroups = 2;                 // groups of 4 warps taking alternate stages
constexpr int kSplitWarps = 4 * kSplitGroups;
constexpr int kSplitThreads = 128;             // threads working on one stage
constexpr int kEpiWarps = 8;                   // two per tensor-memory lane quarter, half of the columns each
constexpr int kTmaWarp = kSplitWarps + kEpiWarps, kMmaWarp = kTmaWarp + 1;
constexpr int kThreads = (kSplitWarps + kEpiWarps + 2) * 32;

// TC_F16X3: operands split into fp16 hi + fp16 (remainder * 2^11); hi*hi goes to one
// accumulator, the two cross terms (scaled by 2^11) to a second one.
// TC_3X_SPLIT_B_MN: as TC_3X_SPLIT_B with B given [K, N] (N contiguous), the form of a
// convolution's input and of the value operand of an attention product: its tiles are
// MN-major in shared memory (32 columns x 16 k-rows per TMA box, 128-byte swizzle with
// 32-byte atoms).
enum TcMode { TC_3X_BLO_TMA = 0, TC_3X_SPLIT_B = 1, TC_1X = 2, TC_F16X3 = 3, TC_3X_SPLIT_B_MN = 4 };

struct TcEpilogue {
  int m, n;
  float* c; long long ldc, sc;
  float alpha, beta;
  const float* cin; long long ldcin, scin;
  const float* bias_n; const float* bias_m; float bias_scale;
  int act; float act_alpha, act_beta;
  const float* res; long long ldres, sres;
  uint2* c16_hi; uint2* c16_lo; long long ldc16;   // result as fp16 hi / lo halves (4 per uint2; ldc16 in halves), or null
  int c16_fixed;            // the halves on the fixed scale (f16_split_fixed) instead of f16_split
  const float* acc_scale;   // device scalar the accumulators are multiplied by (B was scaled by its inverse), or null
  float acc_scale_const;    // times this power of two (the inverse of the fixed scale of a pre-split A; else 1)
  const float* b_row_scale; long long b_row_scale_stride; int k_total;   // [K, N] operand: row k of B[bz] is multiplied by
                                                                       // b_row_scale[bz * stride + k] while it is split, or null
  int* err;                 // error word: range of the split output
  int dbg;   // timing experiments only (0 in normal use)
};

// Shared-memory matrix descriptor for a K-major tile whose rows are 64 bytes
// (16 floats), stored row after row with the 64-byte swizzle: 8-row groups are
// 512 bytes apart (stride byte offset), the leading byte offset is unused.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);        // start address
  d |= (uint64_t)1 << 16;                        // leading byte offset (ignored for swizzled K-major)
  d |= (uint64_t)((8 * 64) >> 4) << 32;          // stride byte offset: 8 rows
  d |= (uint64_t)1 << 46;                        // descriptor version for this architecture
  d |= (uint64_t)4 << 61;                        // 64-byte swizzle
  return d;
}

// K-major tile whose rows are 128 bytes (64 halves) with the 128-byte swizzle: 8-row groups
// are 1024 bytes apart. A K-step of 16 halves advances the start address by 32 bytes.
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;                        // leading byte offset (ignored for swizzled K-major)
  d |= (uint64_t)((8 * 128) >> 4) << 32;         // stride byte offset: 8 rows
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;                        // 128-byte swizzle
  return d;
}

// Descriptor of an MN-major tile of 4-byte elements. The one layout the tensor core accepts
// for them is the 128-byte swizzle with 32-byte atoms: 32 columns (128 bytes) x 4 k-rows form
// a 512-byte atom in which the 32-byte quarter of a row is XORed with the row index; the
// next 4 k-rows of the same columns follow at the stride byte offset (512 bytes), the next 32
// columns `col_group_bytes` further on (the leading byte offset). TMA writes exactly this with
// CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B and a box of 32 columns x any number of k-rows.
__device__ __forceinline__ uint64_t make_smem_desc_mn(uint32_t saddr, uint32_t col_group_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)((col_group_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)(512 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)1 << 61;                        // 128-byte swizzle, 32-byte atoms
  return d;
}

// 32 accumulator columns of this warp's rows. D2OFF != 0: the fp16 mode's second
// accumulator (cross terms, scaled by 2^11) sits D2OFF columns further on.
// `sc`: power of two that undoes the scaling of a constant B (1 when there is none).
template <int D2OFF>
__device__ __forceinline__ void load_acc(uint32_t taddr, uint32_t (&v)[32], float sc) {
  tc_ld_32x32_nowait(taddr, v);
  if (D2OFF != 0) {
    uint32_t w[32];
    tc_ld_32x32_nowait(taddr + (uint32_t)D2OFF, w);
    tc_wait_ld();
#pragma unroll
    for (int j = 0; j < 32; ++j)
      v[j] = __float_as_uint(__fmul_rn(fmaf(__uint_as_float(w[j]), kLoUnscale, __uint_as_float(v[j])), sc));
  } else {
    tc_wait_ld();
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__fmul_rn(__uint_as_float(v[j]), sc));   // sc is a power of two
  }
}
__device__ __forceinline__ float acc_scale_of(const TcEpilogue& ep) {
  return ep.acc_scale ? __fmul_rn(__ldg(ep.acc_scale), ep.acc_scale_const) : ep.acc_scale_const;
}

// Epilogue of one warp's 32 rows. The accumulator chunk arrives with one thread
// per row (32 columns each); it goes through a 4 KB shared-memory tile so that
// each group of 8 lanes then owns one row's 128 contiguous bytes: global loads
// and stores are full lines. 16-byte chunks are XOR-swizzled by the row, which
// keeps both the row-wise writes and the transposed reads free of bank conflicts.
template <int BN, int D2OFF>
__device__ __noinline__ void epilogue_generic(const TcEpilogue& ep, float4* stage, uint32_t tmem_base,
                                              int warp, int lane, int m0, int n0, int bz, int cc0, int cc1) {
      const float sc = acc_scale_of(ep);
      float* c = ep.c + (long long)bz * ep.sc;
      const float* cin = (ep.cin && ep.beta != 0.f) ? ep.cin + (long long)bz * ep.scin : nullptr;
      const float* res = ep.res ? ep.res + (long long)bz * ep.sres : nullptr;
      const bool vec_ok = (ep.ldc % 4) == 0 && ((reinterpret_cast<uintptr_t>(c) & 15) == 0) &&
                          (!cin || ((ep.ldcin % 4) == 0 && (reinterpret_cast<uintptr_t>(cin) & 15) == 0)) &&
                          (!res || ((ep.ldres % 4) == 0 && (reinterpret_cast<uintptr_t>(res) & 15) == 0)) &&
                          (!ep.bias_n || (reinterpret_cast<uintptr_t>(ep.bias_n) & 15) == 0);
      const int c4 = lane & 7;             // float4 column within the 32-column chunk
      const int rsub = lane >> 3;          // row within a group of 4
#pragma unroll 1
      for (int cc = cc0; cc < cc1; ++cc) {
        const int col0 = n0 + cc * 32;
        if (col0 >= ep.n) break;           // uniform across the warp
        uint32_t v[32];
        load_acc<D2OFF>(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(cc * 32), v, sc);
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 8; ++j)
          stage[lane * 8 + (j ^ (lane & 7))] =
              make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                          __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
        __syncwarp();
        const int col = col0 + 4 * c4;
        float4 bn = make_float4(0.f, 0.f, 0.f, 0.f);
        if (ep.bias_n) {
          if (vec_ok && col + 3 < ep.n) bn = __ldg(reinterpret_cast<const float4*>(ep.bias_n + col));
          else {
            if (col < ep.n) bn.x = __ldg(ep.bias_n + col);
            if (col + 1 < ep.n) bn.y = __ldg(ep.bias_n + col + 1);
            if (col + 2 < ep.n) bn.z = __ldg(ep.bias_n + col + 2);
            if (col + 3 < ep.n) bn.w = __ldg(ep.bias_n + col + 3);
          }
          if (ep.bias_scale != 1.f) {
            bn.x = __fmul_rn(ep.bias_scale, bn.x); bn.y = __fmul_rn(ep.bias_scale, bn.y);
            bn.z = __fmul_rn(ep.bias_scale, bn.z); bn.w = __fmul_rn(ep.bias_scale, bn.w);
          }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int rl = 4 * i + rsub;                 // row within the warp's 32
          const int row = m0 + warp * 32 + rl;
          const float4 a = stage[rl * 8 + (c4 ^ (rl & 7))];
          if (row >= ep.m || col >= ep.n) continue;
          float x[4] = {a.x, a.y, a.z, a.w};
          const bool full4 = vec_ok && col + 3 < ep.n;
          float cv[4] = {0.f, 0.f, 0.f, 0.f}, rv[4] = {0.f, 0.f, 0.f, 0.f};
          if (cin) {
            if (full4) {
              const float4 t4 = __ldg(reinterpret_cast<const float4*>(cin + (long long)row * ep.ldcin + col));
              cv[0] = t4.x; cv[1] = t4.y; cv[2] = t4.z; cv[3] = t4.w;
            } else {
              for (int e = 0; e < 4; ++e)
                if (col + e < ep.n) cv[e] = __ldg(cin + (long long)row * ep.ldcin + col + e);
            }
          }
          if (res) {
            if (full4) {
              const float4 t4 = __ldg(reinterpret_cast<const float4*>(res + (long long)row * ep.ldres + col));
              rv[0] = t4.x; rv[1] = t4.y; rv[2] = t4.z; rv[3] = t4.w;
            } else {
              for (int e = 0; e < 4; ++e)
                if (col + e < ep.n) rv[e] = __ldg(res + (long long)row * ep.ldres + col + e);
            }
          }
          const float bm = ep.bias_m ? (ep.bias_scale == 1.f ? __ldg(ep.bias_m + row)
                                                             : __fmul_rn(ep.bias_scale, __ldg(ep.bias_m + row)))
                                     : 0.f;
          const float bnv[4] = {bn.x, bn.y, bn.z, bn.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float y = x[e];
            if (ep.alpha != 1.f) y = __fmul_rn(ep.alpha, y);
            if (cin) y = __fadd_rn(ep.beta == 1.f ? cv[e] : __fmul_rn(ep.beta, cv[e]), y);
            if (ep.bias_n) y = __fadd_rn(y, bnv[e]);
            if (ep.bias_m) y = __fadd_rn(y, bm);
            y = apply_act(ep.act, y, ep.act_alpha, ep.act_beta);
            if (res) y = __fadd_rn(y, rv[e]);
            x[e] = y;
          }
          float* dst = c + (long long)row * ep.ldc + col;
          if (full4) {
            *reinterpret_cast<float4*>(dst) = make_float4(x[0], x[1], x[2], x[3]);
          } else {
            for (int e = 0; e < 4; ++e)
              if (col + e < ep.n) dst[e] = x[e];
          }
        }
      }
    }

// Same data path for the common epilogues (alpha 1, no C input, one kind of bias,
// everything 16-byte aligned, N a multiple of 4), with the options fixed at
// compile time and the eight rows of a chunk processed as independent streams.
// BIAS: 0 none, 1 per column (MatMul + Add), 2 per row (a convolution's channels).
//
// `release()` hands the accumulator back to the MMA warp. It is called as soon as the
// warp's last chunk has left tensor memory, before that chunk's arithmetic and stores;
// it returns whether it did so, and so does this function (no chunk in range, or a
// sub-tile that is not the last: the caller releases).
template <int BN, int D2OFF, int ACT, int BIAS, bool HAS_RES, typename Release>
__device__ __forceinline__ bool epilogue_fast(const TcEpilogue& ep, float4* stage, uint32_t tmem_base,
                                              int warp, int lane, int m0, int n0, int bz, int cc0, int cc1,
                                              Release&& release) {
  bool released = false;
  const float sc = acc_scale_of(ep);
  float* c = ep.c + (long long)bz * ep.sc;
  const float* res = HAS_RES ? ep.res + (long long)bz * ep.sres : nullptr;
  const int c4 = lane & 7, rsub = lane >> 3;
  const int row_base = m0 + warp * 32 + rsub;
  float bm[8];
  if (BIAS == 2) {
#pragma unroll
    for (int i = 0; i < 8; ++i) bm[i] = row_base + 4 * i < ep.m ? __ldg(ep.bias_m + row_base + 4 * i) : 0.f;
  }
#pragma unroll 1
  for (int cc = cc0; cc < cc1; ++cc) {
    const int col0 = n0 + cc * 32;
    if (col0 >= ep.n) break;
    uint32_t v[32];
    load_acc<D2OFF>(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(cc * 32), v, sc);
    if (cc + 1 == cc1 || col0 + 32 >= ep.n) released = release();   // uniform across the warp
    __syncwarp();
#pragma unroll
    for (int j = 0; j < 8; ++j)
      stage[lane * 8 + (j ^ (lane & 7))] =
          make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                      __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
    __syncwarp();
    const int col = col0 + 4 * c4;
    const bool col_ok = col < ep.n;   // n % 4 == 0: the whole float4 is in range
    float4 bn = make_float4(0.f, 0.f, 0.f, 0.f);
    if (BIAS == 1 && col_ok) bn = __ldg(reinterpret_cast<const float4*>(ep.bias_n + col));
    float4 a[8], r[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int rl = 4 * i + rsub;
      a[i] = stage[rl * 8 + (c4 ^ (rl & 7))];
      if (HAS_RES) {
        const int row = row_base + 4 * i;
        r[i] = (col_ok && row < ep.m)
                   ? __ldg(reinterpret_cast<const float4*>(res + (long long)row * ep.ldres + col))
                   : make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float4 x = a[i];
      if (BIAS == 1) {
        x.x = __fadd_rn(x.x, bn.x); x.y = __fadd_rn(x.y, bn.y);
        x.z = __fadd_rn(x.z, bn.z); x.w = __fadd_rn(x.w, bn.w);
      }
      if (BIAS == 2) {
        x.x = __fadd_rn(x.x, bm[i]); x.y = __fadd_rn(x.y, bm[i]);
        x.z = __fadd_rn(x.z, bm[i]); x.w = __fadd_rn(x.w, bm[i]);
      }
      if (ACT == ACT_GELU) {
        const float2 lo = gelu_ref2(make_float2(x.x, x.y)), hi = gelu_ref2(make_float2(x.z, x.w));
        x = make_float4(lo.x, lo.y, hi.x, hi.y);
      } else if (ACT != ACT_NONE) {
        const float al = ep.act_alpha, be = ep.act_beta;   // HardSigmoid / HardSwish coefficients
        x.x = apply_act(ACT, x.x, al, be); x.y = apply_act(ACT, x.y, al, be);
        x.z = apply_act(ACT, x.z, al, be); x.w = apply_act(ACT, x.w, al, be);
      }
      if (HAS_RES) {
        x.x = __fadd_rn(x.x, r[i].x); x.y = __fadd_rn(x.y, r[i].y);
        x.z = __fadd_rn(x.z, r[i].z); x.w = __fadd_rn(x.w, r[i].w);
      }
      const int row = row_base + 4 * i;
      if (col_ok && row < ep.m) *reinterpret_cast<float4*>(c + (long long)row * ep.ldc + col) = x;
    }
  }
  return released;
}

// The epilogue of the pair kernel that takes A pre-split: sixteen warps, a warp per tensor-memory
// lane quarter and 64-column group, each with 4 KB of shared memory. Reading tensor memory
// while MMAs write it is slow, so a warp first takes its whole 32 x 64 part out -- the second
// 32-column chunk into its shared memory, the first into registers -- and hands tensor memory
// back to the MMA warp; bias, activation, residual, the stores and the fp16 split for a
// consuming kernel then run under the next tile's MMAs: the parked chunk first, then the one
// from the registers through the same 4 KB. Shared memory is written a row per lane and read
// eight lanes per row (the whole 128 bytes of a row of the chunk per instruction and row: the
// global loads and stores that follow are whole 128-byte lines, or 64 bytes of each fp16 half);
// the 16-byte slots of a row are XOR-swizzled by the row so that neither side has bank conflicts.
__device__ long long g_epi_stamps[8];   // debug aid: clock64 inside the epilogue of CTA 0, warp 0, tiles 0 and 1
__device__ __forceinline__ int epi_slot(int row, int j) { return j ^ (((row & 1) << 2) | ((row >> 1) & 3)); }

template <int D2OFF, int ACT, int BIAS, bool HAS_RES, typename Release>
__device__ __forceinline__ bool epilogue_parked(const TcEpilogue& ep, float4* buf, uint32_t tmem_base, int q,
                                                int lane, int m0, int n0, int bz, int cc0, unsigned& seen,
                                                Release&& release, int stamp = -1) {
  const float sc = acc_scale_of(ep);
  float* c = ep.c ? ep.c + (long long)bz * ep.sc : nullptr;
  const float* res = HAS_RES ? ep.res + (long long)bz * ep.sres : nullptr;
  const bool have0 = n0 + cc0 * 32 < ep.n, have1 = n0 + (cc0 + 1) * 32 < ep.n;   // uniform across the warp
  const uint32_t trow = tmem_base + ((uint32_t)(q * 32) << 16);
  auto to_buf = [&](const uint32_t (&v)[32]) {
#pragma unroll
    for (int j = 0; j < 8; ++j)
      buf[lane * 8 + epi_slot(lane, j)] = make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                                      __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
  };
  uint32_t v[32];
  __syncwarp();                                     // the previous tile's reads of the buffer are over
  if (D2OFF == 0 && have0 && have1 && !(ep.dbg & 128)) {
    // One accumulator, both chunks there. A load of tensor memory issued behind the parking
    // stores waited 2.7 K clocks where the first one took 0.4 K: the kept chunk and the first
    // half of the parked one are requested together, the second half before the first is parked.
    uint32_t w[16];
    tc_ld_32x32_nowait(trow + (uint32_t)(cc0 * 32), v);
    tc_ld_32x16_nowait(trow + (uint32_t)((cc0 + 1) * 32), w);
    tc_wait_ld();
    uint32_t w2[16];
    tc_ld_32x16_nowait(trow + (uint32_t)((cc0 + 1) * 32 + 16), w2);
#pragma unroll
    for (int j = 0; j < 4; ++j)
      buf[lane * 8 + epi_slot(lane, j)] =
          make_float4(__fmul_rn(__uint_as_float(w[4 * j]), sc), __fmul_rn(__uint_as_float(w[4 * j + 1]), sc),
                      __fmul_rn(__uint_as_float(w[4 * j + 2]), sc), __fmul_rn(__uint_as_float(w[4 * j + 3]), sc));
    tc_wait_ld();
#pragma unroll
    for (int j = 0; j < 4; ++j)
      buf[lane * 8 + epi_slot(lane, 4 + j)] =
          make_float4(__fmul_rn(__uint_as_float(w2[4 * j]), sc), __fmul_rn(__uint_as_float(w2[4 * j + 1]), sc),
                      __fmul_rn(__uint_as_float(w2[4 * j + 2]), sc), __fmul_rn(__uint_as_float(w2[4 * j + 3]), sc));
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__fmul_rn(__uint_as_float(v[j]), sc));   // sc is a power of two
  } else {
    if (have1) {
      load_acc<D2OFF>(trow + (uint32_t)((cc0 + 1) * 32), v, sc);
      to_buf(v);
    }
    if (have0) load_acc<D2OFF>(trow + (uint32_t)(cc0 * 32), v, sc);
  }
  const bool released = release();                  // includes a __syncwarp: the buffer is written
  if (stamp >= 0 && lane == 0) g_epi_stamps[stamp] = clock64();
  // Eight lanes per row: 128 contiguous bytes of fp32 (64 of each fp16 half) per row and
  // instruction, four rows per instruction, sixteen rows per pass.
  const int c8 = lane & 7, r4 = lane >> 3;
  float seen_max = 0.f;                             // largest magnitude written as fixed-scale halves
  auto from_buf = [&](const int chunk) {            // bias, activation, residual, stores of one 32-column chunk
    const int col = n0 + chunk * 32 + 4 * c8;
    const bool col_ok = col < ep.n;                 // n % 4 == 0: the whole float4 is in range
    float4 bn = make_float4(0.f, 0.f, 0.f, 0.f);
    if (BIAS == 1 && col_ok) bn = __ldg(reinterpret_cast<const float4*>(ep.bias_n + col));
#pragma unroll 1
    for (int pass = 0; pass < 2; ++pass) {
      const int row_base = m0 + q * 32 + 16 * pass + r4;
      float4 a[4], r[4];
      float bm[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int rl = 16 * pass + 4 * i + r4;
        a[i] = buf[rl * 8 + epi_slot(rl, c8)];
        const int row = row_base + 4 * i;
        if (BIAS == 2) bm[i] = row < ep.m ? __ldg(ep.bias_m + row) : 0.f;
        if (HAS_RES) {
          r[i] = (col_ok && row < ep.m)
                     ? __ldg(reinterpret_cast<const float4*>(res + (long long)row * ep.ldres + col))
                     : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float4 x = a[i];
        if (BIAS == 1) {
          x.x = __fadd_rn(x.x, bn.x); x.y = __fadd_rn(x.y, bn.y);
          x.z = __fadd_rn(x.z, bn.z); x.w = __fadd_rn(x.w, bn.w);
        }
        if (BIAS == 2) {
          x.x = __fadd_rn(x.x, bm[i]); x.y = __fadd_rn(x.y, bm[i]);
          x.z = __fadd_rn(x.z, bm[i]); x.w = __fadd_rn(x.w, bm[i]);
        }
        if (ACT == ACT_GELU) {
          const float2 lo = gelu_ref2(make_float2(x.x, x.y)), hi = gelu_ref2(make_float2(x.z, x.w));
          x = make_float4(lo.x, lo.y, hi.x, hi.y);
        } else if (ACT != ACT_NONE) {
          const float al = ep.act_alpha, be = ep.act_beta;
          x.x = apply_act(ACT, x.x, al, be); x.y = apply_act(ACT, x.y, al, be);
          x.z = apply_act(ACT, x.z, al, be); x.w = apply_act(ACT, x.w, al, be);
        }
        if (HAS_RES) {
          x.x = __fadd_rn(x.x, r[i].x); x.y = __fadd_rn(x.y, r[i].y);
          x.z = __fadd_rn(x.z, r[i].z); x.w = __fadd_rn(x.w, r[i].w);
        }
        const int row = row_base + 4 * i;
        if (col_ok && row < ep.m) {
          if (c) *reinterpret_cast<float4*>(c + (long long)row * ep.ldc + col) = x;
          if (ep.c16_hi) {   // the kernel that consumes this result takes it split (batch 1)
            uint2 h, l;
            if (ep.c16_fixed) { f16_split_fixed(x, h, l); seen_max = split_track(seen_max, x); }
            else { f16_split(x, h, l); seen |= split_seen(x); }
            const long long o = ((long long)row * ep.ldc16 + col) >> 2;
            ep.c16_hi[o] = h;
            ep.c16_lo[o] = l;
          }
        }
      }
    }
  };
  if (have1) {
    from_buf(cc0 + 1);
    __syncwarp();                                   // everybody has read the parked chunk
  }
  if (stamp >= 0 && lane == 0) g_epi_stamps[stamp + 1] = clock64();
  if (have0) {
    to_buf(v);
    __syncwarp();
    if (stamp >= 0 && lane == 0) g_epi_stamps[stamp + 2] = clock64();
    from_buf(cc0);
  }
  if (stamp >= 0 && lane == 0) g_epi_stamps[stamp + 3] = clock64();
  seen |= split_seen_fixed_of_max(seen_max);
  return released;
}

// Unreduced accumulator of a K-slice -> workspace tile [128][BN], same staging
// as the real epilogues so that the stores are full lines.
template <int BN, int D2OFF>
__device__ __forceinline__ void epilogue_raw(float* ws_tile, float4* stage, uint32_t tmem_base, int warp,
                                             int lane, int cc0, int cc1, float sc) {
  const int c4 = lane & 7, rsub = lane >> 3;
#pragma unroll 1
  for (int cc = cc0; cc < cc1; ++cc) {
    uint32_t v[32];
    load_acc<D2OFF>(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(cc * 32), v, sc);
    __syncwarp();
#pragma unroll
    for (int j = 0; j < 8; ++j)
      stage[lane * 8 + (j ^ (lane & 7))] =
          make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                      __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int rl = 4 * i + rsub;
      *reinterpret_cast<float4*>(ws_tile + (size_t)(warp * 32 + rl) * BN + cc * 32 + 4 * c4) =
          stage[rl * 8 + (c4 ^ (rl & 7))];
    }
  }
}

// The epilogue of four consecutive elements of row `row` from column `col0` on (n % 4 == 0 when
// the split result is written): what the tail fix-up applies to the summed K-slices.
__device__ __forceinline__ void fixup_apply(const TcEpilogue& ep, int row, int col0, int bz, float4 acc) {
  float* c = ep.c ? ep.c + (long long)bz * ep.sc : nullptr;
  const float* cin = (ep.cin && ep.beta != 0.f) ? ep.cin + (long long)bz * ep.scin : nullptr;
  const float* res = ep.res ? ep.res + (long long)bz * ep.sres : nullptr;
  const float x[4] = {acc.x, acc.y, acc.z, acc.w};
  float y4[4] = {0.f, 0.f, 0.f, 0.f};
  for (int e = 0; e < 4; ++e) {
    const int col = col0 + e;
    if (col >= ep.n) break;
    float y = x[e];
    if (ep.alpha != 1.f) y = __fmul_rn(ep.alpha, y);
    if (cin) {
      const float cv = __ldg(cin + (long long)row * ep.ldcin + col);
      y = __fadd_rn(ep.beta == 1.f ? cv : __fmul_rn(ep.beta, cv), y);
    }
    if (ep.bias_n) {
      const float bv = __ldg(ep.bias_n + col);
      y = __fadd_rn(y, ep.bias_scale == 1.f ? bv : __fmul_rn(ep.bias_scale, bv));
    }
    if (ep.bias_m) {
      const float bv = __ldg(ep.bias_m + row);
      y = __fadd_rn(y, ep.bias_scale == 1.f ? bv : __fmul_rn(ep.bias_scale, bv));
    }
    y = apply_act(ep.act, y, ep.act_alpha, ep.act_beta);
    if (res) y = __fadd_rn(y, __ldg(res + (long long)row * ep.ldres + col));
    if (c) c[(long long)row * ep.ldc + col] = y;
    y4[e] = y;
  }
  if (ep.c16_hi) {   // n is a multiple of 8 here: the whole float4 is in range
    uint2 h, l;
    const float4 yv = make_float4(y4[0], y4[1], y4[2], y4[3]);
    if (ep.c16_fixed) f16_split_fixed(yv, h, l); else f16_split(yv, h, l);
    const long long o = ((long long)row * ep.ldc16 + col0) >> 2;
    ep.c16_hi[o] = h;
    ep.c16_lo[o] = l;
    // A tile's few K-sliced elements say nothing about the tensor being tiny: overflow only.
    if ((ep.c16_fixed ? split_seen_fixed(yv) : split_seen(yv)) & 1u) atomicCAS(ep.err, 0, kRangeCode);
  }
}

// Adds the K-slices of the tail tiles in slice order and applies the epilogue.
__global__ void __launch_bounds__(256) gemm_tc_fixup_kernel(const float* __restrict__ ws, TcEpilogue ep, int bm,
                                                            int bn, int dp_tiles, int parts, int tiles_m,
                                                            int tiles_n) {
  const int tt = blockIdx.y;
  const int t = dp_tiles + tt;
  const int tn = t % tiles_n, tm = (t / tiles_n) % tiles_m, bz = t / (tiles_n * tiles_m);
  const int e4 = blockIdx.x * 256 + threadIdx.x;          // float4 index inside the tile
  if (e4 >= bm * bn / 4) return;
  const int rl = e4 / (bn / 4), cl = (e4 % (bn / 4)) * 4;
  const int row = tm * bm + rl, col0 = tn * bn + cl;
  if (row >= ep.m || col0 >= ep.n) return;
  const float* src = ws + (size_t)tt * parts * bm * bn + (size_t)rl * bn + cl;
  // Slices are added in slice order; their loads are issued eight at a time so that the
  // chain of additions does not also serialise the L2 round trips.
  float4 acc = __ldg(reinterpret_cast<const float4*>(src));
  auto add = [&](const float4& v) {
    acc.x = __fadd_rn(acc.x, v.x); acc.y = __fadd_rn(acc.y, v.y);
    acc.z = __fadd_rn(acc.z, v.z); acc.w = __fadd_rn(acc.w, v.w);
  };
  int p = 1;
  for (; p + 8 <= parts; p += 8) {
    float4 v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = __ldg(reinterpret_cast<const float4*>(src + (size_t)(p + j) * bm * bn));
#pragma unroll
    for (int j = 0; j < 8; ++j) add(v[j]);
  }
  for (; p < parts; ++p) add(__ldg(reinterpret_cast<const float4*>(src + (size_t)p * bm * bn)));
  fixup_apply(ep, row, col0, bz, acc);
}

// Shared-memory stage of the main loop. MT = 128-row sub-tiles per CTA tile.
// TF32 modes: A arrives by TMA where its hi copy lives (split in place), lo beside it.
// fp16 mode: A arrives as fp32 rows of 32 floats (no swizzle); the splitters read it into
// registers and write the fp16 hi / lo tiles over it (same size); B arrives as fp16 hi / lo
// by TMA.
template <int BN, int MT, int MODE>
struct TcSmem {
  static constexpr bool kF16 = MODE == TC_F16X3;
  static constexpr int kKb = kF16 ? BK16 : BK;                          // floats of K per stage
  static constexpr int kARaw = kF16 ? MT * BM * kKb * 4 : 0;
  static constexpr int kABytes = kF16 ? MT * BM * kKb * 2 : MT * BM * kKb * 4;   // one of A hi / lo
  static constexpr int kBBytes = kF16 ? BN * kKb * 2 : BN * kKb * 4;             // one of B hi / lo
  static constexpr int kOffAHi = 0;
  static constexpr bool k1X = MODE == TC_1X;                      // one copy of each operand, no lo tiles
  static constexpr int kOffALo = kABytes;
  static constexpr int kOffBHi = (k1X ? 1 : 2) * kABytes;         // fp16: kARaw == 2 * kABytes
  static constexpr int kOffBLo = kOffBHi + kBBytes;
  static constexpr int kStageBytes = k1X ? kABytes + kBBytes : 2 * kABytes + 2 * kBBytes;
  static_assert(!kF16 || kARaw == 2 * kABytes, "the fp16 tiles replace the fp32 rows in place");
  static constexpr int kTxBytes = (kF16 ? kARaw : kABytes) + kBBytes + ((kF16 || MODE == TC_3X_BLO_TMA) ? kBBytes : 0);
  static constexpr int kStages = (200 * 1024) / kStageBytes;      // TF32 and fp16: 4 / 6 / 8 (BN 256 / 128 / 64)
  static constexpr int kEpiBytes = kEpiWarps * 4096;              // one 4 KB transpose tile per epilogue warp
  static constexpr int kDynBytes = kStages * kStageBytes + kEpiBytes + 1024 /*alignment*/ + 512 /*barriers*/;
  static constexpr int kAccCols = (kF16 ? 2 : 1) * MT * BN;       // tensor-memory columns of one accumulator set
  static constexpr int kNumAcc = (2 * kAccCols <= 512) ? 2 : 1;   // sets: two when they fit (epilogue overlaps)
  static constexpr int kD2Off = kF16 ? MT * BN : 0;               // column offset of the cross-term accumulator
  static_assert(kDynBytes <= 227 * 1024, "shared memory per CTA");
  static_assert(kAccCols <= 512, "tensor memory");
};

// Work distribution of the persistent kernel. The first `dp_tiles` tiles (whole
// rounds of the grid) are taken round-robin, one whole tile at a time. The
// remaining `num_tiles - dp_tiles` tiles would leave most SMs idle for a full
// tile time, so each of them is cut along K into `tail_parts` slices, one slice
// per CTA; a slice's accumulator goes unreduced to a workspace slot (its CTA
// index) and a second small kernel adds the slices in a fixed order and applies
// the epilogue. tail_parts < 2: no slicing, dp_tiles == num_tiles.
struct TcSched {
  int num_tiles, dp_tiles, tail_parts, num_kb;
};
struct TcWork {
  int tile, k0, k1, raw;   // raw: workspace slot, or -1 for a whole tile with the real epilogue
};
__device__ __forceinline__ bool tc_get_work(const TcSched& sc, int w, TcWork* out) {
  const int c = blockIdx.x, g = gridDim.x;
  const int n_dp = sc.dp_tiles > c ? (sc.dp_tiles - c + g - 1) / g : 0;
  if (w < n_dp) {
    out->tile = c + w * g; out->k0 = 0; out->k1 = sc.num_kb; out->raw = -1;
    return true;
  }
  if (w == n_dp && sc.tail_parts >= 2 && c < (sc.num_tiles - sc.dp_tiles) * sc.tail_parts) {
    const int part = c % sc.tail_parts;
    out->tile = sc.dp_tiles + c / sc.tail_parts;
    out->k0 = (int)((long long)part * sc.num_kb / sc.tail_parts);
    out->k1 = (int)((long long)(part + 1) * sc.num_kb / sc.tail_parts);
    out->raw = c;
    return true;
  }
  return false;
}

// Persistent kernel: one CTA per SM walks tiles t = blockIdx.x, blockIdx.x +
// gridDim.x, ... The accumulator is double-buffered in tensor memory, so the
// epilogue of one tile overlaps the main loop of the next.
//   warps 0-7   splitters, two groups of four taking alternate K-blocks (hi/lo of the
//               A tile, and of B unless it arrives split)
//   warps 8-15  epilogue (warp w owns TMEM lanes 32*((w-8) % 4) .. +31 and half of the columns)
//   warp  16    TMA producer (one thread)
//   warp  17    MMA issuer (one thread); allocates and frees tensor memory
template <int BN, int MT, int MODE>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
               const __grid_constant__ CUtensorMap tm_blo, TcEpilogue ep, TcSched sc, int a_batched,
               int b_batched, int tiles_m, int tiles_n, float* workspace, int* err) {
  using L = TcSmem<BN, MT, MODE>;
  constexpr bool kBMN = MODE == TC_3X_SPLIT_B_MN;
  constexpr int S = L::kStages;
  constexpr int NACC = L::kNumAcc;      // accumulator sets in tensor memory
  constexpr int KB = L::kKb;            // floats of K per stage
  constexpr int D2 = L::kD2Off;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_smem = smem + S * L::kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + L::kEpiBytes);
  uint64_t* full = bars;               // TMA bytes landed
  uint64_t* ready = bars + S;          // hi/lo written
  uint64_t* empty = bars + 2 * S;      // MMAs that read the stage have completed
  uint64_t* acc_full = bars + 3 * S;   // [2] accumulator complete
  uint64_t* acc_empty = bars + 3 * S + 2;  // [2] accumulator drained by the epilogue
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * S + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t kTmemCols = NACC * L::kAccCols;   // 128, 256 or 512: a power of two

  auto a_raw = [&](int s) { return smem + s * L::kStageBytes; };
  auto a_hi = [&](int s) { return smem + s * L::kStageBytes + L::kOffAHi; };
  auto a_lo = [&](int s) { return smem + s * L::kStageBytes + L::kOffALo; };
  auto b_hi = [&](int s) { return smem + s * L::kStageBytes + L::kOffBHi; };
  auto b_lo = [&](int s) { return smem + s * L::kStageBytes + L::kOffBLo; };

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&ready[s], kSplitThreads);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], kEpiWarps);   // one arrival per epilogue warp
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
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
      const uint32_t bytes = L::kTxBytes;
      int it = 0;   // running K-block count over all of this CTA's tiles
      bool ok = true;
      TcWork wk;
      for (int w = 0; ok && tc_get_work(sc, w, &wk); ++w) {
        const int t = wk.tile;
        const int tn = t % tiles_n, tm = (t / tiles_n) % tiles_m, bz = t / (tiles_n * tiles_m);
        const int bzb = b_batched ? bz : 0, bza = a_batched ? bz : 0;
        for (int kb = wk.k0; kb < wk.k1; ++kb, ++it) {
          const int s = it % S;
          const uint32_t ph = (it / S) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1)) { atomicExch(err, 1); *abort_flag = 1; ok = false; break; }
          mbar_arrive_expect_tx(&full[s], bytes);
          tma_load_3d(a_raw(s), &tm_a, &full[s], kb * KB, tm * (MT * BM), bza);   // TF32 modes: a_raw == a_hi
          if (kBMN) {
            // [K, N] operand: one box per 32 columns (128 bytes) x KB k-rows.
#pragma unroll
            for (int j = 0; j < BN / 32; ++j)
              tma_load_3d(b_hi(s) + j * (KB * 128), &tm_b, &full[s], tn * BN + 32 * j, kb * KB, bzb);
          } else
          tma_load_3d(b_hi(s), &tm_b, &full[s], kb * KB, tn * BN, bzb);
          if (MODE == TC_3X_BLO_TMA || MODE == TC_F16X3)
            tma_load_3d(b_lo(s), &tm_blo, &full[s], kb * KB, tn * BN, bzb);
        }
      }
    }
  } else if (warp == kMmaWarp) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      // Instruction descriptor: fp32 accumulator, A and B both TF32 (format 2) or both
      // fp16 (format 0), both K-major, N = BN, M = 128.
      constexpr uint32_t kFmt = MODE == TC_F16X3 ? 0u : 2u;
      const uint32_t idesc = (1u << 4) | (kFmt << 7) | (kFmt << 10) | (kBMN ? 1u << 16 : 0u) |   // bit 16: B MN-major
                             ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      int it = 0, ti = 0;
      bool ok = true;
      TcWork wk;
      for (int w = 0; ok && tc_get_work(sc, w, &wk); ++w, ++ti) {
        const int ab = ti % NACC;
        // The epilogue must have drained this accumulator (NACC tiles ago).
        if (!mbar_wait(&acc_empty[ab], ((ti / NACC) & 1) ^ 1)) { atomicExch(err, 5); *abort_flag = 1; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(ab * L::kAccCols);
        for (int kb = wk.k0; kb < wk.k1; ++kb, ++it) {
          const int s = it % S;
          const uint32_t ph = (it / S) & 1;
          ok = mbar_wait(MODE == TC_1X ? &full[s] : &ready[s], ph);
          if (!ok) { atomicExch(err, 2); *abort_flag = 1; break; }
          tc_fence_after();
          const uint64_t db = kBMN ? make_smem_desc_mn(smem_u32(b_hi(s)), KB * 128) : make_smem_desc(smem_u32(b_hi(s)));
          const uint64_t dbl = kBMN ? make_smem_desc_mn(smem_u32(b_lo(s)), KB * 128) : make_smem_desc(smem_u32(b_lo(s)));
#pragma unroll
          for (int kk = 0; kk < 2; ++kk) {                  // two K-steps per 64-byte row
            const uint64_t off = (uint64_t)(kk * 32 >> 4);  // 8 floats or 16 halves = 32 bytes along K
            // MN-major B: the second group of 8 k-rows (two atoms of 4) lies 1 KB further on.
            const uint64_t boff = kBMN ? (uint64_t)(kk * 1024 >> 4) : off;
            const uint32_t acc = (kb > wk.k0 || kk > 0) ? 1u : 0u;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              const uint64_t da = make_smem_desc(smem_u32(a_hi(s) + mt * (BM * 64)));
              const uint64_t dal = make_smem_desc(smem_u32(a_lo(s) + mt * (BM * 64)));
              const uint32_t d = d_tmem + (uint32_t)(mt * BN);
              if (MODE == TC_F16X3) {
                // Issued further down, one accumulator after the other: alternating between the
                // two with every MMA costs 30 % of the tensor pipe's rate.
              } else if (MODE == TC_1X) {
                tc_mma_tf32(d, da + off, db + boff, idesc, acc);
              } else {
                tc_mma_tf32(d, dal + off, db + boff, idesc, acc);   // a_lo * b_hi
                tc_mma_tf32(d, da + off, dbl + boff, idesc, 1u);    // a_hi * b_lo
                tc_mma_tf32(d, da + off, db + boff, idesc, 1u);     // a_hi * b_hi
              }
            }
          }
          if (MODE == TC_F16X3) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              const uint64_t da = make_smem_desc(smem_u32(a_hi(s) + mt * (BM * 64)));
              const uint64_t dal = make_smem_desc(smem_u32(a_lo(s) + mt * (BM * 64)));
              const uint32_t d = d_tmem + (uint32_t)(mt * BN);
#pragma unroll
              for (int kk = 0; kk < 2; ++kk)                               // a_hi * b_hi -> D1
                tc_mma_f16(d, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), idesc, (kb > wk.k0 || kk > 0) ? 1u : 0u);
#pragma unroll
              for (int kk = 0; kk < 2; ++kk) {                             // cross terms (scaled by 2^11) -> D2
                tc_mma_f16(d + D2, dal + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), idesc, (kb > wk.k0 || kk > 0) ? 1u : 0u);
                tc_mma_f16(d + D2, da + (uint64_t)(kk * 2), dbl + (uint64_t)(kk * 2), idesc, 1u);
              }
            }
          }
          tc_commit(&empty[s]);
        }
        if (ok) tc_commit(&acc_full[ab]);
      }
    }
  } else if (warp < kSplitWarps) {
    // ---------------- splitters ----------------
    if (MODE != TC_1X) {
      const int t0 = threadIdx.x & (kSplitThreads - 1);
      const int group = threadIdx.x / kSplitThreads;   // takes the K-blocks with it % kSplitGroups == group
      int it = 0;
      bool ok = true;
      unsigned seen = 0;
      TcWork wk;
      for (int w = 0; ok && tc_get_work(sc, w, &wk); ++w) {
        for (int kb = wk.k0; kb < wk.k1; ++kb, ++it) {
          if (it % kSplitGroups != group) continue;
          const int s = it % S;
          const uint32_t ph = (it / S) & 1;
          ok = mbar_wait(&full[s], ph);
          if (MODE != TC_F16X3 && !ok) { atomicExch(err, 3); *abort_flag = 1; break; }
          if (MODE == TC_F16X3) {
            // fp32 rows of 32 floats -> fp16 hi / lo tiles; one float4 (4 consecutive k) per item.
            // The tiles take the place of the rows: everything is read first, the group's
            // 128 threads meet at a named barrier, then everything is written.
            const float4* raw = reinterpret_cast<const float4*>(a_raw(s));
            uint8_t* hi_t = a_hi(s);
            uint8_t* lo_t = a_lo(s);
            constexpr int kItems = L::kARaw / 16 / kSplitThreads;
            float4 x[kItems > 0 ? kItems : 1];
#pragma unroll
            for (int i = 0; i < kItems; ++i) x[i] = raw[i * kSplitThreads + t0];
            // The barrier also ORs the threads' wait results, so that the whole group leaves
            // together if the wait above expired for any of them.
            ok = !group_barrier_or(group + 1, kSplitThreads, !ok);
            if (!ok) { atomicExch(err, 3); *abort_flag = 1; break; }
#pragma unroll
            for (int i = 0; i < kItems; ++i) {
              const int item = i * kSplitThreads + t0;
              seen |= split_seen(x[i]);
              uint2 hi, lo;
              f16_split(x[i], hi, lo);
              const uint32_t off = sw64_off8(item >> 3, item & 7);
              *reinterpret_cast<uint2*>(hi_t + off) = hi;
              *reinterpret_cast<uint2*>(lo_t + off) = lo;
            }
          } else {
          float4* src = reinterpret_cast<float4*>(a_hi(s));
          float4* dst = reinterpret_cast<float4*>(a_lo(s));
#pragma unroll
          for (int i = 0; i < L::kABytes / 16 / kSplitThreads; ++i) {
            float4 hi, lo;
            tf32_split(src[i * kSplitThreads + t0], hi, lo);
            src[i * kSplitThreads + t0] = hi;
            dst[i * kSplitThreads + t0] = lo;
          }
          }
          if (MODE == TC_3X_SPLIT_B || MODE == TC_3X_SPLIT_B_MN) {   // elementwise: any tile layout
            float4* sb = reinterpret_cast<float4*>(b_hi(s));
            float4* dbp = reinterpret_cast<float4*>(b_lo(s));
            // A per-row factor of the [K, N] operand (the squeeze-excite gate of the input planes
            // of a pointwise convolution) is applied here, one fp32 multiply before the split:
            // the same bits as a separate broadcast Mul in front of the GEMM. In the MN-major
            // tile a float4 lies within one k-row: 128-byte rows, KB rows per 32-column box.
            const float* rs = (MODE == TC_3X_SPLIT_B_MN && ep.b_row_scale)
                                  ? ep.b_row_scale + (long long)(wk.tile / (tiles_n * tiles_m)) * ep.b_row_scale_stride
                                  : nullptr;
#pragma unroll
            for (int i = 0; i < L::kBBytes / 16 / kSplitThreads; ++i) {
              float4 hi, lo;
              float4 v = sb[i * kSplitThreads + t0];
              if (MODE == TC_3X_SPLIT_B_MN && rs) {
                const int k = kb * KB + ((i * kSplitThreads + t0) % (KB * 8)) / 8;
                const float f = k < ep.k_total ? __ldg(rs + k) : 1.f;
                v.x = __fmul_rn(v.x, f); v.y = __fmul_rn(v.y, f); v.z = __fmul_rn(v.z, f); v.w = __fmul_rn(v.w, f);
              }
              tf32_split(v, hi, lo);
              sb[i * kSplitThreads + t0] = hi;
              dbp[i * kSplitThreads + t0] = lo;
            }
          }
          fence_proxy_async();
          mbar_arrive(&ready[s]);
        }
      }
      // An element of A too large for fp16, or nothing but tiny ones: the result is not to be
      // used (the host re-runs on the TF32 path); a code from a timed-out wait takes precedence.
      if (MODE == TC_F16X3) split_report_warp(seen, err);
    }
  } else {
    // ---------------- epilogue ----------------
    const int e = warp - kSplitWarps, q = e & 3;   // TMEM lane quarter (kSplitWarps is a multiple of 4)
    const int cc0 = (e >> 2) * (BN / 64), cc1 = cc0 + BN / 64;   // this warp's 32-column chunks
    float4* stage = reinterpret_cast<float4*>(epi_smem + e * 4096);
    const bool simple = ep.alpha == 1.f && !(ep.cin && ep.beta != 0.f) && !(ep.bias_m && ep.bias_n) &&
                        ep.bias_scale == 1.f && (ep.ldc % 4) == 0 && (ep.n % 4) == 0 && (ep.sc % 4) == 0 &&
                        ((reinterpret_cast<uintptr_t>(ep.c) & 15) == 0) &&
                        (!ep.res || ((ep.ldres % 4) == 0 && (ep.sres % 4) == 0 &&
                                     (reinterpret_cast<uintptr_t>(ep.res) & 15) == 0)) &&
                        (!ep.bias_n || (reinterpret_cast<uintptr_t>(ep.bias_n) & 15) == 0);
    const int key = !simple ? -1 : ((ep.bias_n ? 1 : 0) | (ep.res ? 2 : 0) | (ep.act << 2) | (ep.bias_m ? 64 : 0));
    int ti = 0;
    TcWork wk;
    for (int w = 0; tc_get_work(sc, w, &wk); ++w, ++ti) {
      const int t = wk.tile;
      const int tn = t % tiles_n, tm = (t / tiles_n) % tiles_m, bz = t / (tiles_n * tiles_m);
      const int ab = ti % NACC;
      if (!mbar_wait(&acc_full[ab], (ti / NACC) & 1)) { atomicExch(err, 4); *abort_flag = 1; break; }
      tc_fence_after();
      // Every tcgen05.ld of this warp has completed (each is followed by wait::ld) when the
      // accumulator is handed back to the MMA warp.
      int mt = 0;
      bool released = false;
      auto do_release = [&]() {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[ab]);
      };
      auto release = [&]() -> bool {
        if (mt != MT - 1) return false;
        do_release();
        return true;
      };
#pragma unroll 1
      for (mt = 0; mt < MT; ++mt) {
      const uint32_t acc = tmem_base + (uint32_t)(ab * L::kAccCols + mt * BN);
      const int m0 = (tm * MT + mt) * BM, n0 = tn * BN;
      if (m0 >= ep.m) break;                     // uniform: the second sub-tile may lie past M
      if (wk.raw >= 0) {
        epilogue_raw<BN, D2>(workspace + ((size_t)wk.raw * MT + mt) * BM * BN, stage, acc, q, lane, cc0, cc1, acc_scale_of(ep));
      } else
      switch (key) {
        case 0: released = epilogue_fast<BN, D2, ACT_NONE, 0, false>(ep, stage, acc, q, lane, m0, n0, bz, cc0, cc1, release); break;
        case 1: released = epilogue_fast<BN, D2, ACT_NONE, 1, false>(ep, stage, acc, q, lane, m0, n0, bz, cc0, cc1, release); break;
        case 2: released = epilogue_fast<BN, D2, ACT_NONE, 0, true>(ep, stage, acc, q, lane, m0, n0, bz, cc0, cc1, release); break;
        case 3: released = epilogue_fast<BN, D2, ACT_NONE, 1, true>(ep, stage, acc, q, lane, m0, n0, bz, cc0, cc1, release); break;
        case (ACT_GELU << 2) | 1: released = epilogue_fast<BN, D2, ACT_GELU, 1, false>(ep, stage, acc, q, lane, m0, n0, bz, cc0, cc1, release); break;
        case (ACT_RELU << 2) | 1: released = epilogue_fast<BN, D2, ACT_RELU, 1, false>(ep, stage, acc, q, lane, m0, n0, bz, cc0, cc1, release); break;
        case 64: released = epilogue_fast<BN, D2, ACT_NONE, 2, false>(ep, stage, acc, q, lane, m0, n0, bz, cc0, cc1, release); break;
        case 64 | 2: released = epilogue_fast<BN, D2, ACT_NONE, 2, true>(ep, stage, acc, q, lane, m0, n0, bz, cc0, cc1, release); break;
        case 64 | (ACT_RELU << 2): released = epilogue_fast<BN, D2, ACT_RELU, 2, false>(ep, stage, acc, q, lane, m0, n0, bz, cc0, cc1, release); break;
        case 64 | (ACT_HARDSWISH << 2): released = epilogue_fast<BN, D2, ACT_HARDSWISH, 2, false>(ep, stage, acc, q, lane, m0, n0, bz, cc0, cc1, release); break;
        default: epilogue_generic<BN, D2>(ep, stage, acc, q, lane, m0, n0, bz, cc0, cc1); break;
      }
      }
      if (!released) do_release();
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0 && warp == kTmaWarp && lane == 0) {
    // Give copies that may still be in flight a bounded time to land before the
    // shared memory is released.
    for (int s = 0; s < S; ++s) {
      (void)mbar_wait(&full[s], 0);
      (void)mbar_wait(&full[s], 1);
    }
  }
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols));
  }
}

// ---- CTA pairs ---------------------------------------------------------------------------
// fp16-split GEMM on clusters of two CTAs (tcgen05 .cta_group::2): a pair owns a 256 x BN
// tile. Each CTA stages its own 128 rows of A and HALF of the B tile (BN / 2 rows): the
// tensor cores of the two SMs exchange the B halves, so every SM pulls 32 KB per stage
// instead of 48 KB -- the main loop is bound by exactly that feed. Per CTA: TMA producer and
// splitters as in the one-CTA kernel (local `full` barriers); the splitters of both CTAs
// arrive on the LEADER's (rank 0) `ready` barrier; one thread of the leader issues the MMAs
// for both SMs and commits to the `empty` / `acc_full` barriers of both CTAs; each CTA's
// epilogue warps drain its own 128 accumulator rows and arrive on the leader's `acc_empty`.
// Work is distributed over pairs exactly as over CTAs in the one-CTA kernel.
__device__ __forceinline__ bool pair_get_work(const TcSched& sc, int w, TcWork* out) {
  const int c = blockIdx.x >> 1, g = gridDim.x >> 1;
  const int n_dp = sc.dp_tiles > c ? (sc.dp_tiles - c + g - 1) / g : 0;
  if (w < n_dp) {
    out->tile = c + w * g; out->k0 = 0; out->k1 = sc.num_kb; out->raw = -1;
    return true;
  }
  if (w == n_dp && sc.tail_parts >= 2 && c < (sc.num_tiles - sc.dp_tiles) * sc.tail_parts) {
    const int part = c % sc.tail_parts;
    out->tile = sc.dp_tiles + c / sc.tail_parts;
    out->k0 = (int)((long long)part * sc.num_kb / sc.tail_parts);
    out->k1 = (int)((long long)(part + 1) * sc.num_kb / sc.tail_parts);
    out->raw = c;
    return true;
  }
  return false;
}

// PRE: A arrives already split (fp16 hi / lo arrays written by the kernel that produced it), so
// all four tiles of a stage come by TMA and no thread of the CTA touches them.
template <int BN, bool PRE = false>
struct PairSmem {
  // Without PRE a stage holds all four tiles for 32 halves of K (64-byte rows, 64-byte swizzle).
  // PRE: the ring's entries hold ONE operand's hi and lo tiles for 64 halves of K (rows of 128
  // bytes, 128-byte swizzle: TMA then asks L2 for whole 128-byte lines, which the L2 -> SM path
  // delivers about a fifth faster than twice as many 64-byte requests); the entries of a K-block
  // are A's and then B's.
  static constexpr int kKb = PRE ? 64 : BK16;
  static constexpr int kABytes = BM * kKb * 2;          // fp16 hi tile of A; the lo tile follows
  static constexpr int kBBytes = (BN / 2) * kKb * 2;    // this CTA's half of B: one of hi / lo
  static constexpr int kOffALo = kABytes;
  static constexpr int kOffBHi = 2 * kABytes;
  static constexpr int kOffBLo = kOffBHi + kBBytes;
  static_assert(!PRE || kABytes == kBBytes, "entries of one size");
  static constexpr int kStageBytes = PRE ? 2 * kABytes : 2 * kABytes + 2 * kBBytes;
  // TMA brings B only (A goes global -> registers -> tiles); PRE: a whole entry
  static constexpr int kTxBytes = PRE ? 2 * kABytes : 2 * kBBytes;
  // Epilogue memory: 4 KB per epilogue warp (PRE: sixteen of them; a parking place for half of
  // the warp's accumulator part, or the staging tile of the general epilogues).
  static constexpr int kEpiBytes = (PRE ? 16 : kEpiWarps) * 4096;
  static constexpr int kStages = (227 * 1024 - kEpiBytes - 1536) / kStageBytes;   // BN 256: 5 entries with PRE, else 6 stages
  static constexpr int kDynBytes = kStages * kStageBytes + kEpiBytes + 1024 /*alignment*/ + 512 /*barriers*/;
  // Without PRE: D1 and D2, one accumulator set. PRE: the operands are on fixed scales, the three
  // partial products share ONE accumulator, and two sets alternate between consecutive tiles, so
  // that a tile's epilogue runs under the next tile's MMAs.
  static constexpr int kTmemCols = 2 * BN;
  static_assert(kDynBytes <= 227 * 1024, "shared memory per CTA");
  static_assert(kTmemCols <= 512 && (kTmemCols & (kTmemCols - 1)) == 0, "tensor memory");
};

// Debug aid (ALTIUS_CUDA_TC_DBG bit 0x1000): clock64 stamps of a few events per CTA.
__device__ long long g_pair_stamps[160][24];
__device__ __forceinline__ void pair_stamp(int dbg, int slot) {
  if (dbg & 0x1000) g_pair_stamps[blockIdx.x][slot] = clock64();
}

// PRE runs 18 warps: sixteen epilogue warps (no thread has to touch the operand tiles), the TMA
// producer and the MMA issuer. Both CTAs' loads count their bytes on the leader's `ready`
// barriers, which is all the MMA thread waits for.
template <int BN, bool PRE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_tc_pair_kernel(const float* __restrict__ a_ptr, long long lda, int k_total,
                    const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_alo,
                    const __grid_constant__ CUtensorMap tm_b, const __grid_constant__ CUtensorMap tm_blo,
                    TcEpilogue ep, TcSched sc, int tiles_m, int tiles_n, float* workspace, int* err, int dbg) {
  using L = PairSmem<BN, PRE>;
  // Debug toggle: bits 16-19 of dbg, when set, use fewer stages of the ring.
  const int S = ((dbg >> 16) & 15) > 0 && ((dbg >> 16) & 15) < L::kStages ? ((dbg >> 16) & 15) : L::kStages;
  constexpr int KB = L::kKb;
  constexpr int D2 = PRE ? 0 : BN;       // column offset of the cross-term accumulator (none with PRE)
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int SM = L::kStages;
  uint8_t* epi_smem = smem + SM * L::kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + L::kEpiBytes);
  uint64_t* full = bars;                 // this CTA's TMA bytes landed
  uint64_t* ready = bars + SM;            // leader's: both CTAs' fp16 tiles written (2 x 4 warps arrive)
  uint64_t* empty = bars + 2 * SM;        // this CTA's: the pair's MMAs that read the stage have completed
  uint64_t* acc_full = bars + 3 * SM;     // [2] this CTA's: accumulator set complete (PRE uses both sets)
  uint64_t* acc_empty = bars + 3 * SM + 2;   // [2] leader's: set drained by the epilogue warps of the pair
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * SM + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();
  const bool leader = rank == 0;
  if (threadIdx.x == 0) pair_stamp(dbg, 0);

  auto pwait = [&](uint64_t* bar, uint32_t parity) { return mbar_wait(bar, parity); };
  auto a_raw = [&](int s) { return smem + s * L::kStageBytes; };    // fp16 hi tile of A
  auto a_lo = [&](int s) { return smem + s * L::kStageBytes + L::kOffALo; };
  auto b_hi = [&](int s) { return smem + s * L::kStageBytes + L::kOffBHi; };
  auto b_lo = [&](int s) { return smem + s * L::kStageBytes + L::kOffBLo; };

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&full[s], 1);
      // one arrival per splitter warp of the pair; PRE: the leader's producer, with the bytes of both CTAs
      mbar_init(&ready[s], PRE ? 1 : 2 * (kSplitThreads / 32));
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 2 * (PRE ? 16 : kEpiWarps));   // one arrival per epilogue warp of the pair
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kMmaWarp) {         // the same warp in both CTAs, the same shared-memory slot
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"((uint32_t)L::kTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::);
  }
  tc_fence_before();
  cluster_sync_all();                    // barriers of both CTAs initialised before any remote arrival
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) pair_stamp(dbg, 1);

  if (warp == kTmaWarp) {
    // ---------------- TMA producer (each CTA for itself) ----------------
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      TcWork wk;
      for (int w = 0; ok && pair_get_work(sc, w, &wk); ++w) {
        const int tn = wk.tile % tiles_n;
        const int m0 = ((wk.tile / tiles_n) % tiles_m) * (2 * BM) + (int)rank * BM;
        if (PRE) {
          // Two ring entries per K-block of 64 halves: this CTA's 128 rows of A (hi, lo; rows past
          // M are zero-filled), then its half of the B tile (hi, lo).
          for (int kb = wk.k0; ok && kb < wk.k1; ++kb) {
            for (int op = 0; op < 2; ++op, ++it) {
              const int s = it % S;
              const uint32_t ph = (it / S) & 1;
              if (!pwait(&empty[s], ph ^ 1)) { atomicExch(err, 1); *abort_flag = 1; ok = false; break; }
              const uint32_t rdy = map_to_cta(&ready[s], 0);       // the leader's barrier of this entry
              if (leader) mbar_arrive_expect_tx(&ready[s], 2 * L::kTxBytes);
              uint8_t* e = smem + s * L::kStageBytes;
              if (op == 0) {
                tma_load_3d_pair(e, &tm_a, rdy, kb * KB, m0, 0);
                tma_load_3d_pair(e + L::kABytes, &tm_alo, rdy, kb * KB, m0, 0);
              } else {
                tma_load_3d_pair(e, &tm_b, rdy, kb * KB, tn * BN + (int)rank * (BN / 2), 0);
                tma_load_3d_pair(e + L::kABytes, &tm_blo, rdy, kb * KB, tn * BN + (int)rank * (BN / 2), 0);
              }
            }
          }
          continue;
        }
        for (int kb = wk.k0; kb < wk.k1; ++kb, ++it) {
          const int s = it % S;
          const uint32_t ph = (it / S) & 1;
          if (!pwait(&empty[s], ph ^ 1)) { atomicExch(err, 1); *abort_flag = 1; ok = false; break; }
          mbar_arrive_expect_tx(&full[s], L::kTxBytes);
          tma_load_3d(b_hi(s), &tm_b, &full[s], kb * KB, tn * BN + (int)rank * (BN / 2), 0);
          tma_load_3d(b_lo(s), &tm_blo, &full[s], kb * KB, tn * BN + (int)rank * (BN / 2), 0);
        }
      }
    }
  } else if (warp == kMmaWarp) {
    // ---------------- MMA issuer (leader only) ----------------
    if (leader && lane == 0) {
      // fp32 accumulators, fp16 A and B (format 0), both K-major, N = BN, M = 256 over the pair.
      const uint32_t idesc = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
      int it = 0, ti = 0;
      bool ok = true;
      TcWork wk;
      for (int w = 0; ok && pair_get_work(sc, w, &wk); ++w, ++ti) {
        // The epilogue warps must have drained this accumulator set (PRE: the tile before last).
        const bool two_sets = PRE && !(dbg & 1024);
        const int set = two_sets ? (ti & 1) : 0, use = two_sets ? (ti >> 1) : ti;
        if (!mbar_wait(&acc_empty[set], (use & 1) ^ 1)) { atomicExch(err, 5); *abort_flag = 1; break; }
        tc_fence_after();
        const uint32_t d1 = tmem_base + (uint32_t)(set * BN);
        if (PRE) {
          for (int kb = wk.k0; kb < wk.k1; ++kb, it += 2) {
            const int sa = it % S, sb = (it + 1) % S;          // the K-block's A entry and B entry
            ok = pwait(&ready[sa], (it / S) & 1) && pwait(&ready[sb], ((it + 1) / S) & 1);
            if (!ok) { atomicExch(err, 2); *abort_flag = 1; break; }
            if (it == 0) pair_stamp(dbg, 2);
            tc_fence_after();
            const uint32_t ea = smem_u32(smem + sa * L::kStageBytes), eb = smem_u32(smem + sb * L::kStageBytes);
            const uint64_t da = make_smem_desc_sw128(ea), dal = make_smem_desc_sw128(ea + L::kABytes);
            const uint64_t db = make_smem_desc_sw128(eb), dbl = make_smem_desc_sw128(eb + L::kABytes);
            // Operands on fixed scales: the cross terms go into the same accumulator.
#pragma unroll
            for (int kk = 0; kk < KB / 16; ++kk) {          // K-steps of 16 halves (32 bytes of a row)
              const uint64_t off = (uint64_t)(kk * 2);
              tc_mma_f16_pair(d1, dal + off, db + off, idesc, (kb > wk.k0 || kk > 0) ? 1u : 0u);   // a_lo * b_hi
              tc_mma_f16_pair(d1, da + off, dbl + off, idesc, 1u);                                  // a_hi * b_lo
              tc_mma_f16_pair(d1, da + off, db + off, idesc, 1u);                                   // a_hi * b_hi
            }
            tc_commit_pair(smem_u32(&empty[sa]));          // both entries are free again in this CTA ...
            tc_commit_pair(map_to_cta(&empty[sa], 1));     // ... and in the peer
            tc_commit_pair(smem_u32(&empty[sb]));
            tc_commit_pair(map_to_cta(&empty[sb], 1));
          }
        } else
        for (int kb = wk.k0; kb < wk.k1; ++kb, ++it) {
          const int s = it % S;
          const uint32_t ph = (it / S) & 1;
          ok = pwait(&ready[s], ph);
          if (!ok) { atomicExch(err, 2); *abort_flag = 1; break; }
          if (it == 0) pair_stamp(dbg, 2);
          tc_fence_after();
          const uint64_t da = make_smem_desc(smem_u32(a_raw(s))), dal = make_smem_desc(smem_u32(a_lo(s)));
          const uint64_t db = make_smem_desc(smem_u32(b_hi(s))), dbl = make_smem_desc(smem_u32(b_lo(s)));
          {
            // One accumulator after the other within a stage: alternating between them with every
            // MMA cost 30 % of the tensor pipe's rate.
#pragma unroll
            for (int kk = 0; kk < KB / 16; ++kk)
              tc_mma_f16_pair(d1, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), idesc, (kb > wk.k0 || kk > 0) ? 1u : 0u);
#pragma unroll
            for (int kk = 0; kk < KB / 16; ++kk) {
              tc_mma_f16_pair(d1 + D2, dal + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), idesc, (kb > wk.k0 || kk > 0) ? 1u : 0u);
              tc_mma_f16_pair(d1 + D2, da + (uint64_t)(kk * 2), dbl + (uint64_t)(kk * 2), idesc, 1u);
            }
          }
          tc_commit_pair(smem_u32(&empty[s]));      // the stage is free again in this CTA ...
          tc_commit_pair(map_to_cta(&empty[s], 1)); // ... and in the peer
        }
        if (ok) {
          tc_commit_pair(smem_u32(&acc_full[set]));
          tc_commit_pair(map_to_cta(&acc_full[set], 1));
        }
        if (ti < 5) pair_stamp(dbg, 3 + ti);   // all MMAs of tile ti issued
      }
    }
  } else if (!PRE && warp < kSplitWarps) {
    // ---------------- splitters (each CTA its own A rows) ----------------
    // A does not pass through shared memory as fp32: each thread loads its eight float4
    // (row, four consecutive k) of the stage from global memory, splits them in registers and
    // writes the fp16 hi / lo tiles. The loads of a group's next stage are in flight while
    // it waits for that stage to be free.
    const int t0 = threadIdx.x & (kSplitThreads - 1);
    const int group = threadIdx.x / kSplitThreads;   // takes the K-blocks with it % kSplitGroups == group
    constexpr int kItems = BM * KB / 4 / kSplitThreads;   // 8
    int it = 0;
    bool ok = true;
    unsigned seen = 0;
    TcWork wk;
    for (int w = 0; ok && pair_get_work(sc, w, &wk); ++w) {
      const int t = wk.tile;
      const int tm = (t / tiles_n) % tiles_m;
      const int m0 = tm * (2 * BM) + (int)rank * BM;
      const float* a_tile = a_ptr + (long long)m0 * lda;   // one GEMM (batch 1)
      for (int kb = wk.k0; kb < wk.k1; ++kb, ++it) {
        if (it % kSplitGroups != group) continue;
        const int s = it % S;
        const uint32_t ph = (it / S) & 1;
        float4 x[kItems];
#pragma unroll
        for (int i = 0; i < kItems; ++i) {
          const int item = i * kSplitThreads + t0;
          const int r = item >> 3, kcol = kb * KB + (item & 7) * 4;
          x[i] = (m0 + r < ep.m && kcol < k_total)
                     ? __ldg(reinterpret_cast<const float4*>(a_tile + (long long)r * lda + kcol))
                     : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        ok = mbar_wait(&empty[s], ph ^ 1);          // the pair's MMAs on the previous use of the stage are done
        if (!ok) { atomicExch(err, 3); *abort_flag = 1; break; }
        uint8_t* hi_t = a_raw(s);
        uint8_t* lo_t = a_lo(s);
#pragma unroll
        for (int i = 0; i < kItems; ++i) {
          const int item = i * kSplitThreads + t0;
          seen |= split_seen(x[i]);
          uint2 hi, lo;
          f16_split(x[i], hi, lo);
          const uint32_t off = sw64_off8(item >> 3, item & 7);
          *reinterpret_cast<uint2*>(hi_t + off) = hi;
          *reinterpret_cast<uint2*>(lo_t + off) = lo;
        }
        fence_proxy_async();
        ok = mbar_wait(&full[s], ph);               // this CTA's half of B has landed too
        if (!ok) { atomicExch(err, 3); *abort_flag = 1; break; }
        __syncwarp();                               // one remote arrival per warp, not per thread
        if (lane == 0) mbar_arrive_cluster(map_to_cta(&ready[s], 0));
      }
    }
    split_report_warp(seen, err);
  } else if (!PRE || warp < 16) {
    // ---------------- epilogue (each CTA its own 128 rows) ----------------
    // PRE: warps 0-15, a warp per lane quarter and quarter of the columns on the common
    // epilogues (2 KB of staging each); the general and the K-slice epilogues are left to warps
    // 8-15 with 4 KB each (the same 32 KB), the others only hand the accumulator back.
    const int e = PRE ? warp : warp - kSplitWarps, q = e & 3;
    const int eo = PRE ? e - 8 : e;                                // index among the eight "old" warps
    const int cc0 = (eo >> 2) * (BN / 64), cc1 = cc0 + BN / 64;   // their 32-column chunks
    const int hc0 = (e >> 2) * (BN / 128);                        // PRE, common epilogues: 64 columns from chunk hc0
    // 4 KB of shared memory per epilogue warp: the parking place of the common epilogues, the
    // staging tile of the others.
    float4* stage = reinterpret_cast<float4*>(epi_smem + e * 4096);
    float4* park = stage;
    const bool simple = ep.alpha == 1.f && !(ep.cin && ep.beta != 0.f) && !(ep.bias_m && ep.bias_n) &&
                        ep.bias_scale == 1.f && (ep.ldc % 4) == 0 && (ep.n % 4) == 0 && (ep.sc % 4) == 0 &&
                        ((reinterpret_cast<uintptr_t>(ep.c) & 15) == 0) &&
                        (!ep.res || ((ep.ldres % 4) == 0 && (ep.sres % 4) == 0 &&
                                     (reinterpret_cast<uintptr_t>(ep.res) & 15) == 0)) &&
                        (!ep.bias_n || (reinterpret_cast<uintptr_t>(ep.bias_n) & 15) == 0);
    const int key = !simple ? -1 : ((ep.bias_n ? 1 : 0) | (ep.res ? 2 : 0) | (ep.act << 2) | (ep.bias_m ? 64 : 0));
    int ti = 0;
    unsigned seen_out = 0;   // what this warp has seen of the results it wrote split (ep.c16_hi)
    TcWork wk;
    for (int w = 0; pair_get_work(sc, w, &wk); ++w, ++ti) {
      const int t = wk.tile;
      const int tn = t % tiles_n, tm = (t / tiles_n) % tiles_m, bz = t / (tiles_n * tiles_m);
      const int m0 = tm * (2 * BM) + (int)rank * BM, n0 = tn * BN;
      const bool two_sets = PRE && !(dbg & 1024);
      const int set = two_sets ? (ti & 1) : 0, use = two_sets ? (ti >> 1) : ti;
      const uint32_t acc = tmem_base + (uint32_t)(set * BN);
      const uint32_t acc_empty_leader = map_to_cta(&acc_empty[set], 0);
      if (PRE && ep.res && key >= 0 && wk.raw < 0) {
        // While the tile's MMAs run: pull this warp's 32 x 64 block of the residual into L2 -- but
        // not ahead of the kernel's first operand tiles (a thousand prefetches per SM issued at
        // kernel entry delayed those by 5 K clocks): wait until the first K-block has been used.
        if (ti == 0) (void)mbar_wait(&empty[1], 0);
        const float* rp = ep.res + (long long)bz * ep.sres;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int row = m0 + q * 32 + (lane >> 1) + 16 * i, col = n0 + hc0 * 32 + (lane & 1) * 32;
          if (row < ep.m && col < ep.n)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(rp + (long long)row * ep.ldres + col));
        }
      }
      const bool wide = wk.raw >= 0 || key < 0 || (key & 64);
      if (!mbar_wait(&acc_full[set], use & 1)) { atomicExch(err, 4); *abort_flag = 1; break; }
      tc_fence_after();
      if (e == 0 && lane == 0 && ti < 3) pair_stamp(dbg, 8 + 2 * ti);     // accumulator of tile ti complete
      bool released = false;
      const int estamp = ((dbg & 0x1000) && blockIdx.x == 0 && e == 0 && ti < 2) ? 4 * ti : -1;
      auto release = [&]() -> bool {     // all of this warp's tcgen05.ld have completed
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(acc_empty_leader);
        return true;
      };
      if (PRE && BN == 256 && m0 < ep.m && !wide) {
        switch (key) {
          case 0: released = epilogue_parked<D2, ACT_NONE, 0, false>(ep, park, acc, q, lane, m0, n0, bz, hc0, seen_out, release, estamp); break;
          case 1: released = epilogue_parked<D2, ACT_NONE, 1, false>(ep, park, acc, q, lane, m0, n0, bz, hc0, seen_out, release, estamp); break;
          case 2: released = epilogue_parked<D2, ACT_NONE, 0, true>(ep, park, acc, q, lane, m0, n0, bz, hc0, seen_out, release, estamp); break;
          case 3: released = epilogue_parked<D2, ACT_NONE, 1, true>(ep, park, acc, q, lane, m0, n0, bz, hc0, seen_out, release, estamp); break;
          case (ACT_GELU << 2) | 1: released = epilogue_parked<D2, ACT_GELU, 1, false>(ep, park, acc, q, lane, m0, n0, bz, hc0, seen_out, release, estamp); break;
          case (ACT_RELU << 2) | 1: released = epilogue_parked<D2, ACT_RELU, 1, false>(ep, park, acc, q, lane, m0, n0, bz, hc0, seen_out, release, estamp); break;
          default:
            if (eo >= 0) epilogue_generic<BN, D2>(ep, stage, acc, q, lane, m0, n0, bz, cc0, cc1);
            break;
        }
      } else if (m0 < ep.m && eo >= 0) {
        if (wk.raw >= 0) {
          epilogue_raw<BN, D2>(workspace + ((size_t)wk.raw * 2 + rank) * BM * BN, stage, acc, q, lane, cc0, cc1, acc_scale_of(ep));
        } else
        switch (key) {
          case 0: released = epilogue_fast<BN, D2, ACT_NONE, 0, false>(ep, stage, acc, q, lane, m0, n0, bz, cc0, cc1, release); break;
          case 1: released = epilogue_fast<BN, D2, ACT_NONE, 1, false>(ep, stage, acc, q, lane, m0, n0, bz, cc0, cc1, release); break;
          case 2: released = epilogue_fast<BN, D2, ACT_NONE, 0, true>(ep, stage, acc, q, lane, m0, n0, bz, cc0, cc1, release); break;
          case 3: released = epilogue_fast<BN, D2, ACT_NONE, 1, true>(ep, stage, acc, q, lane, m0, n0, bz, cc0, cc1, release); break;
          case (ACT_GELU << 2) | 1: released = epilogue_fast<BN, D2, ACT_GELU, 1, false>(ep, stage, acc, q, lane, m0, n0, bz, cc0, cc1, release); break;
          case (ACT_RELU << 2) | 1: released = epilogue_fast<BN, D2, ACT_RELU, 1, false>(ep, stage, acc, q, lane, m0, n0, bz, cc0, cc1, release); break;
          case 64: released = epilogue_fast<BN, D2, ACT_NONE, 2, false>(ep, stage, acc, q, lane, m0, n0, bz, cc0, cc1, release); break;
          case 64 | 2: released = epilogue_fast<BN, D2, ACT_NONE, 2, true>(ep, stage, acc, q, lane, m0, n0, bz, cc0, cc1, release); break;
          case 64 | (ACT_RELU << 2): released = epilogue_fast<BN, D2, ACT_RELU, 2, false>(ep, stage, acc, q, lane, m0, n0, bz, cc0, cc1, release); break;
          case 64 | (ACT_HARDSWISH << 2): released = epilogue_fast<BN, D2, ACT_HARDSWISH, 2, false>(ep, stage, acc, q, lane, m0, n0, bz, cc0, cc1, release); break;
          default: epilogue_generic<BN, D2>(ep, stage, acc, q, lane, m0, n0, bz, cc0, cc1); break;
        }
      }
      if (!released) release();
      if (e == 0 && lane == 0 && ti < 3) pair_stamp(dbg, 9 + 2 * ti);     // this warp's part of tile ti stored
    }
    if (PRE && ep.c16_hi) split_report_warp(seen_out, err);
  }

  // ---------------- teardown ----------------
  if (threadIdx.x == 0) pair_stamp(dbg, 14);
  tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0 && warp == kTmaWarp && lane == 0) {
    for (int s = 0; s < S; ++s) {        // copies that may still be in flight: a bounded time to land
      (void)mbar_wait(PRE ? &ready[s] : &full[s], 0);
      (void)mbar_wait(PRE ? &ready[s] : &full[s], 1);
    }
  }
  cluster_sync_all();                    // no CTA leaves while its peer may still signal it or read its B half
  if (warp == kMmaWarp) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)L::kTmemCols));
  }
  if (threadIdx.x == 0) pair_stamp(dbg, 15);
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

// Largest magnitude of a [rows, k] operand as the bits of a non-negative float (finite values).
__global__ void absmax_kernel(const float* __restrict__ x, int64_t rows, int64_t k, int64_t ld, unsigned* out) {
  unsigned m = 0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < rows * k; i += (int64_t)gridDim.x * blockDim.x) {
    const unsigned ab = __float_as_uint(__ldg(x + (i / k) * ld + (i % k))) & 0x7FFFFFFFu;
    if (ab < 0x7F800000u) m = max(m, ab);
  }
  m = __reduce_max_sync(0xffffffffu, m);
  if ((threadIdx.x & 31) == 0 && m) atomicMax(out, m);
}

// Power of two 2^e that brings a largest magnitude `absmax_bits` into [2^13, 2^14); 1 for zero.
__device__ __forceinline__ float weight_scale(unsigned absmax_bits) {
  if (absmax_bits == 0) return 1.f;
  const int ex = (int)(absmax_bits >> 23) - 127;           // floor(log2(max)); subnormals read as -127
  int e = 13 - ex;
  e = e > 100 ? 100 : (e < -100 ? -100 : e);
  return __uint_as_float((unsigned)(e + 127) << 23);
}

// fp16 hi / lo split of a constant [rows, k] operand (row stride ld) into [rows, k8]
// halves, columns k .. k8-1 zero. With `absmax` the operand is first scaled by weight_scale
// (and *inv_scale receives the inverse). An element beyond fp16 leaves kRangeCode in *err.
// `plain`: lo = rn(v - hi) on the scale of hi (the operands of the single-accumulator kernel: a
// constant scaled to [2^13, 2^14), an activation on the fixed scale 2^8) instead of
// rn((v - hi) * 2^11).
__global__ void f16_split_kernel(const float* __restrict__ x, __half* __restrict__ hi, __half* __restrict__ lo,
                                 int64_t rows, int64_t k, int64_t ld, int64_t k8, int* err,
                                 const unsigned* __restrict__ absmax, float* inv_scale, int plain) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const float sc = absmax ? weight_scale(*absmax) : (plain ? kFixedScale : 1.f);
  if (i == 0 && inv_scale) *inv_scale = __fdiv_rn(1.f, sc);
  if (i >= rows * k8) return;
  const int64_t r = i / k8, c = i % k8;
  const float v = c < k ? __fmul_rn(__ldg(x + r * ld + c), sc) : 0.f;
  const __half h = __float2half_rn(v);
  hi[i] = h;
  const float rest = __fsub_rn(v, __half2float(h));
  lo[i] = __float2half_rn(plain ? rest : __fmul_rn(rest, kLoScale));
  if (beyond_half(v)) atomicCAS(err, 0, kRangeCode);
}

// The same split for an activation whose rows are a multiple of 8 floats, 16-byte aligned:
// eight elements per thread (two 16-byte loads, one 16-byte store to each of hi and lo).
__global__ void __launch_bounds__(256) f16_split_vec8_kernel(const float* __restrict__ x, uint4* __restrict__ hi,
                                                             uint4* __restrict__ lo, int64_t rows, int64_t k8th,
                                                             int64_t ld, int* err, int fixed) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  unsigned seen = 0;
  if (i < rows * k8th) {
    const int64_t r = i / k8th, c = i % k8th;
    const float4* src = reinterpret_cast<const float4*>(x + r * ld + c * 8);
    const float4 v0 = __ldg(src), v1 = __ldg(src + 1);
    uint2 h0, l0, h1, l1;
    if (fixed) {
      f16_split_fixed(v0, h0, l0);
      f16_split_fixed(v1, h1, l1);
      seen = split_seen_fixed(v0) | split_seen_fixed(v1);
    } else {
      f16_split(v0, h0, l0);
      f16_split(v1, h1, l1);
      seen = split_seen(v0) | split_seen(v1);
    }
    hi[i] = make_uint4(h0.x, h0.y, h1.x, h1.y);
    lo[i] = make_uint4(l0.x, l0.y, l1.x, l1.y);
  }
  // The block's 2048 elements: out of range, or non-zero values that are all tiny.
  const int over = __syncthreads_or(seen & 1u), big = __syncthreads_or(seen & 2u), tiny = __syncthreads_or(seen & 4u);
  if (threadIdx.x == 0 && (over || (tiny && !big))) atomicCAS(err, 0, kRangeCode);
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

// 3-D map over a row-major [batch, rows, k] tensor of f32 (elem_bytes 4) or fp16 (2):
// box = box_k elements of K x box_rows rows. `swizzle`: 0, 64 or 128 (the latter with 32-byte
// atoms, see make_smem_desc_mn); a swizzled box is exactly that many bytes wide. (For an operand given [K, N] the roles are swapped: "k" is N, the
// contiguous dimension, and the rows are the k-rows.)
bool make_map(CUtensorMap* map, const void* base, int elem_bytes, int64_t k, int64_t rows, int64_t batch,
              int64_t ld, int64_t batch_stride, int box_k, int box_rows, int swizzle) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {(cuuint64_t)k, (cuuint64_t)rows, (cuuint64_t)std::max<int64_t>(batch, 1)};
  cuuint64_t strides[2] = {(cuuint64_t)ld * elem_bytes,
                           (cuuint64_t)(batch > 1 && batch_stride > 0 ? batch_stride : rows * ld) * elem_bytes};
  cuuint32_t box[3] = {(cuuint32_t)box_k, (cuuint32_t)box_rows, 1};
  // 1128: the plain 128-byte swizzle (K-major tiles of 128-byte rows); 128: the same span with 32-byte atoms
  const bool sw128_plain = swizzle == 1128;
  if (sw128_plain) swizzle = 128;
  if (swizzle != 0 && box_k * elem_bytes != swizzle) return false;
  cuuint32_t estr[3] = {1, 1, 1};
  return fn(map, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3,
            const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            sw128_plain ? CU_TENSOR_MAP_SWIZZLE_128B
            : swizzle == 128 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B
                             : (swizzle == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE),
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    // Debug toggle: ALTIUS_CUDA_TC_SMS caps the persistent grid (scaling experiments).
    if (const char* e = std::getenv("ALTIUS_CUDA_TC_SMS")) {
      const int v = std::atoi(e);
      if (v > 0 && v < n) n = v;
    }
  }
  return n;
}

// Host-side schedule: whole rounds of the grid are data parallel; a last partial
// round of `tail` tiles is cut along K into `parts` slices when that keeps more
// SMs busy (see TcSched).
struct TcPlan {
  int grid, tiles_m, tiles_n;
  TcSched sc;
  size_t workspace_bytes;
};
// `workers`: CTAs (or CTA pairs) that walk the tiles; 0 = one per SM.
TcPlan make_plan(int64_t m, int64_t n, int64_t k, int64_t batch, int bn, int mt, int kb_floats, int workers = 0) {
  TcPlan pl{};
  const int sms = workers > 0 ? workers : sm_count();
  pl.tiles_n = (int)((n + bn - 1) / bn);
  pl.tiles_m = (int)((m + mt * BM - 1) / (mt * BM));
  const long long tiles = (long long)pl.tiles_n * pl.tiles_m * batch;
  const int num_kb = (int)((k + kb_floats - 1) / kb_floats);
  pl.sc.num_tiles = (int)tiles;
  pl.sc.num_kb = num_kb;
  pl.sc.dp_tiles = (int)tiles;
  pl.sc.tail_parts = 0;
  pl.grid = (int)std::min<long long>(tiles, sms);
  const int tail = (int)(tiles % sms);
  if (tail > 0) {
    const int parts = std::min(std::min(sms / tail, num_kb / 2), 32);   // at least two K-blocks per slice
    if (parts >= 2) {
      pl.sc.dp_tiles = (int)(tiles - tail);
      pl.sc.tail_parts = parts;
      pl.grid = std::max(pl.grid, tail * parts);
      pl.grid = std::min(pl.grid, sms);
      pl.workspace_bytes = (size_t)tail * parts * mt * BM * bn * sizeof(float);
    }
  }
  return pl;
}

template <int BN, int MT, int MODE>
cudaError_t launch_tc(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mbl,
                      const TcEpilogue& ep, const TcPlan& pl, int a_batched, int b_batched, float* workspace,
                      int* err, cudaStream_t st) {
  using L = TcSmem<BN, MT, MODE>;
  static unsigned long long attr_done = 0;
  if (cudaError_t e0 = ensure_dynamic_smem(gemm_tc_kernel<BN, MT, MODE>, L::kDynBytes, &attr_done)) return e0;
  gemm_tc_kernel<BN, MT, MODE><<<pl.grid, kThreads, L::kDynBytes, st>>>(ma, mb, mbl, ep, pl.sc, a_batched, b_batched,
                                                                    pl.tiles_m, pl.tiles_n, workspace, err);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess || pl.sc.tail_parts < 2) return e;
  const int tail = pl.sc.num_tiles - pl.sc.dp_tiles;
  dim3 grid((MT * BM * BN / 4 + 255) / 256, tail);
  gemm_tc_fixup_kernel<<<grid, 256, 0, st>>>(workspace, ep, MT * BM, BN, pl.sc.dp_tiles, pl.sc.tail_parts, pl.tiles_m,
                                             pl.tiles_n);
  return cudaGetLastError();
}

template <int BN, bool PRE>
cudaError_t launch_pair(const float* a, long long lda, int k, const CUtensorMap& ma, const CUtensorMap& mal,
                        const CUtensorMap& mb, const CUtensorMap& mbl, const TcEpilogue& ep, const TcPlan& pl,
                        float* workspace, int* err, cudaStream_t st) {
  using L = PairSmem<BN, PRE>;
  static unsigned long long attr_done = 0;
  if (cudaError_t e0 = ensure_dynamic_smem(gemm_tc_pair_kernel<BN, PRE>, L::kDynBytes, &attr_done)) return e0;
  // pl.grid counts pairs; the cluster shape (2, 1, 1) is a compile-time attribute of the kernel.
  static const int dbg = std::getenv("ALTIUS_CUDA_TC_DBG") ? std::atoi(std::getenv("ALTIUS_CUDA_TC_DBG")) : 0;
  gemm_tc_pair_kernel<BN, PRE><<<2 * pl.grid, kThreads, L::kDynBytes, st>>>(a, lda, k, ma, mal, mb, mbl, ep, pl.sc,
                                                                          pl.tiles_m, pl.tiles_n, workspace, err, dbg);
  if (dbg & 0x1000) {
    cudaStreamSynchronize(st);
    static long long h[160][24];
    cudaMemcpyFromSymbol(h, g_pair_stamps, sizeof(h));
    long long eh[8];
    cudaMemcpyFromSymbol(eh, g_epi_stamps, sizeof(eh));
    std::printf("epi stamps:");
    for (int i = 0; i < 8; ++i) std::printf(" %lld", eh[i] - h[0][0]);
    std::printf("\n");
    for (int c : {0, 1, 64, 65, 146, 147}) {
      if (c >= 2 * pl.grid) continue;
      std::printf("pair cta %3d:", c);
      for (int i = 1; i < 16; ++i) std::printf(" %lld", h[c][i] ? h[c][i] - h[c][0] : -1);
      std::printf("\n");
    }
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess || pl.sc.tail_parts < 2) return e;
  const int tail = pl.sc.num_tiles - pl.sc.dp_tiles;
  dim3 grid((2 * BM * BN / 4 + 255) / 256, tail);
  gemm_tc_fixup_kernel<<<grid, 256, 0, st>>>(workspace, ep, 2 * BM, BN, pl.sc.dp_tiles, pl.sc.tail_parts, pl.tiles_m,
                                             pl.tiles_n);
  return cudaGetLastError();
}

}  // namespace

bool gemm_tc_supported(const GemmParams& q) {
  // A is [M, K]; B is [N, K] (trans_b) or [K, N] (the MN-major mode, 3xTF32 only).
  if (q.trans_a) return false;
  if (q.m <= 0 || q.n <= 0 || q.k <= 0 || q.batch <= 0 || q.batch > 65535) return false;
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (!al(q.a) || !al(q.b) || (q.lda % 4) || (q.ldb % 4)) return false;
  if (q.batch > 1 && ((q.stride_a % 4) || (q.stride_b % 4))) return false;
  if (q.stride_a < 0 || q.stride_b < 0) return false;      // 0: the operand is shared by the batch
  if (q.b_lo && (!al(q.b_lo))) return false;
  return encode_fn() != nullptr;
}

namespace {
struct TcShape { int bn, mt; bool pair; };

// CTA pairs that can be resident at once for the pair kernel (0: clusters unavailable).
int pair_count() {
  static int n = -1;
  if (n < 0) {
    n = 0;
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
      (void)cudaGetLastError();
      n = sm_count() / 2;      // no device (a plan_only session): plan as for a B200
      return n;
    }
    {
      using L = PairSmem<256, false>;
      if (cudaFuncSetAttribute(gemm_tc_pair_kernel<256, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               L::kDynBytes) == cudaSuccess) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(sm_count() & ~1);
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = L::kDynBytes;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, gemm_tc_pair_kernel<256, false>, &cfg) == cudaSuccess && clusters > 0)
          n = std::min(clusters, sm_count() / 2);
      }
      (void)cudaGetLastError();
    }
  }
  return n;
}

// Tile shape by a cost model in SM clocks, fitted to measurements: TMA fills shared
// memory at about 28 bytes per clock per SM (8 TB/s over the chip, the L2 -> SM
// limit), and an MMA of 128 x BN x 32 bytes of K takes about (4096 + 32 BN) / 64 clocks
// (it is bound by fetching its operands from shared memory). A stage costs the larger
// of its MMA time and its operand bytes; rounds come from the same plan the launch uses
// (a K-sliced tail costs 1 / parts of a round); a shape that fills tensor memory with
// one accumulator set cannot hide its epilogue. variant: 0 TF32 with B arriving split,
// 1 TF32 with one B copy, 2 fp16 split.
// allow_pairs: 0 no CTA pairs, 1 pairs that stage A through registers, 2 pairs whose A arrives
// already split by TMA (each SM then pulls 32 KB per stage and no thread touches a tile).
TcShape pick_shape(int64_t m, int64_t n, int64_t k, int64_t batch, int variant, int allow_pairs) {
  static const TcShape cands[3] = {{256, 1, false}, {128, 1, false}, {64, 1, false}};
  // Debug toggle: ALTIUS_CUDA_TC_BN=64|128|256 forces the tile width.
  const char* ebn = std::getenv("ALTIUS_CUDA_TC_BN");
  const int fbn = ebn ? std::atoi(ebn) : 0;
  const int sms = sm_count();
  const bool f16 = variant == 2;
  const int kbf = f16 ? BK16 : BK;
  TcShape best = {256, 1, false};
  double best_cost = 1e300;
  for (int i = 0; i < 3; ++i) {
    const TcShape c = cands[i];
    if (fbn && c.bn != fbn) continue;
    const TcPlan pl = make_plan(m, n, k, batch, c.bn, c.mt, kbf);
    double rounds = (double)(pl.sc.dp_tiles / sms) + (pl.sc.dp_tiles % sms ? 1.0 : 0.0);
    if (pl.sc.tail_parts >= 2) rounds += 1.0 / pl.sc.tail_parts + 0.05;
    const double mma_clk = c.mt * 6.0 * (4096.0 + 32.0 * c.bn) / 64.0 * (variant == 1 ? 1.0 / 3.0 : 1.0);
    const double a_bytes = c.mt * BM * kbf * 4.0;
    const double b_bytes = f16 ? c.bn * kbf * 4.0 : c.bn * kbf * 4.0 * (variant == 0 ? 2 : 1);
    const double feed_clk = (a_bytes + b_bytes) / 28.0;
    const int acc_cols = (f16 ? 2 : 1) * c.mt * c.bn;
    const double epi_clk = 2 * acc_cols <= 512 ? 0.0 : c.mt * c.bn * (f16 ? 24.0 : 18.0);
    double cost = rounds * (pl.sc.num_kb * std::max(mma_clk, feed_clk) + epi_clk);
    if (pl.sc.num_tiles < sms) cost += 1.0;   // ties: prefer the shape with more tiles in flight
    if (cost < best_cost - 1e-9) { best_cost = cost; best = c; }
  }
  // CTA pairs (fp16 split, one GEMM, BN 256): 256 x 256 tiles, each SM pulls its A rows and
  // half of B (32 KB per stage), the pair's MMAs cost 128 clocks per SM; single accumulator set.
  const int pairs = allow_pairs ? pair_count() : 0;
  if (f16 && batch == 1 && (k % (allow_pairs == 2 ? 8 : 4)) == 0 && pairs > 0 && (!fbn || fbn == 256)) {
    const int pkb = kbf;
    const TcPlan pl = make_plan(m, n, k, batch, 256, 2, pkb, pairs);
    double rounds = (double)(pl.sc.dp_tiles / pairs) + (pl.sc.dp_tiles % pairs ? 1.0 : 0.0);
    if (pl.sc.tail_parts >= 2) rounds += 1.0 / pl.sc.tail_parts + 0.05;
    const double cost = rounds * (pl.sc.num_kb * (pkb / 32) * std::max(6.0 * 128.0, 32768.0 / 28.0) + 256 * 24.0);
    if (cost < best_cost - 1e-9) { best_cost = cost; best = {256, 2, true}; }
  }
  return best;
}
}  // namespace

bool gemm_tc_wants_presplit(int64_t m, int64_t n, int64_t k, int64_t batch) {
  return pick_shape(m, n, k, batch, 2, 2).pair;
}

size_t gemm_tc_workspace_bytes(int64_t m, int64_t n, int64_t k, int64_t batch, int variant, int allow_pairs) {
  const TcShape sh = pick_shape(m, n, k, batch, variant, allow_pairs);
  const int kbf = sh.pair && allow_pairs == 2 ? 64 : (variant == 2 ? BK16 : BK);   // pre-split A: K-blocks of 64 halves
  return make_plan(m, n, k, batch, sh.bn, sh.mt, kbf, sh.pair ? pair_count() : 0).workspace_bytes;
}

cudaError_t launch_gemm_tc(const GemmParams& q, int mode, int* err_word, cudaStream_t st) {
  if (!gemm_tc_supported(q)) return cudaErrorInvalidValue;
  // mode 0: fp16 split when B comes with one, else 3xTF32; 2: 1xTF32; 3: 3xTF32.
  if (!q.trans_b && mode == 2) return cudaErrorInvalidValue;   // the [K, N] form exists for 3xTF32 only
  const int kmode = !q.trans_b ? TC_3X_SPLIT_B_MN
                    : mode == 2 ? TC_1X
                    : (mode == 0 && q.b16_hi && q.b16_lo) ? TC_F16X3
                    : (q.b_lo ? TC_3X_BLO_TMA : TC_3X_SPLIT_B);
  const int variant = kmode == TC_F16X3 ? 2 : (kmode == TC_3X_BLO_TMA ? 0 : 1);
  const bool pre = q.allow_pairs == 2 && q.a16_hi && q.a16_lo;
  const TcShape sh = pick_shape(q.m, q.n, q.k, q.batch, variant, pre ? 2 : (q.allow_pairs == 1 ? 1 : 0));
  CUtensorMap mal;
  const int bn = sh.bn;
  CUtensorMap ma, mb, mbl;
  const int b_batched = (q.batch > 1 && q.stride_b > 0) ? 1 : 0;
  const int a_batched = (q.batch > 1 && q.stride_a > 0) ? 1 : 0;
  const int64_t a_batch = a_batched ? q.batch : 1;
  if (kmode == TC_F16X3) {
    if (b_batched || (q.ldb16 % 8) != 0) return cudaErrorInvalidValue;
    // A pair's CTAs each load their own 128 rows of A and half of the B tile.
    const int a_rows = sh.pair ? BM : sh.mt * BM, b_rows = sh.pair ? bn / 2 : bn;
    if (pre && (!sh.pair || !q.a16_fixed || !q.b16_plain)) return cudaErrorInvalidValue;   // the single-accumulator kernel's formats
    if (!pre && q.b16_plain) return cudaErrorInvalidValue;
    if (sh.pair && pre) {
      if ((q.lda16 % 8) != 0) return cudaErrorInvalidValue;
      if (!make_map(&ma, q.a16_hi, 2, q.k, q.m, 1, q.lda16, 0, 64, BM, 1128)) return cudaErrorInvalidValue;
      if (!make_map(&mal, q.a16_lo, 2, q.k, q.m, 1, q.lda16, 0, 64, BM, 1128)) return cudaErrorInvalidValue;
    } else {
      if (!make_map(&ma, q.a, 4, q.k, q.m, a_batch, q.lda, q.stride_a, BK16, a_rows, 0)) return cudaErrorInvalidValue;
      mal = ma;
    }
    const int bbox = (sh.pair && pre) ? 64 : BK16, bsw = (sh.pair && pre) ? 1128 : 64;   // pre: K-blocks of 64 halves
    if (!make_map(&mb, q.b16_hi, 2, q.k, q.n, 1, q.ldb16, 0, bbox, b_rows, bsw)) return cudaErrorInvalidValue;
    if (!make_map(&mbl, q.b16_lo, 2, q.k, q.n, 1, q.ldb16, 0, bbox, b_rows, bsw)) return cudaErrorInvalidValue;
  } else if (kmode == TC_3X_SPLIT_B_MN) {
    // B [K, N]: N is the contiguous dimension, boxes of 32 columns x BK k-rows.
    if (!make_map(&ma, q.a, 4, q.k, q.m, a_batch, q.lda, q.stride_a, BK, sh.mt * BM, 64)) return cudaErrorInvalidValue;
    if (!make_map(&mb, q.b, 4, q.n, q.k, b_batched ? q.batch : 1, q.ldb, q.stride_b, 32, BK, 128))
      return cudaErrorInvalidValue;
    mbl = mb;
  } else {
    if (!make_map(&ma, q.a, 4, q.k, q.m, a_batch, q.lda, q.stride_a, BK, sh.mt * BM, 64)) return cudaErrorInvalidValue;
    if (!make_map(&mb, q.b, 4, q.k, q.n, b_batched ? q.batch : 1, q.ldb, q.stride_b, BK, bn, 64))
      return cudaErrorInvalidValue;
    if (kmode == TC_3X_BLO_TMA) {
      if (!make_map(&mbl, q.b_lo, 4, q.k, q.n, b_batched ? q.batch : 1, q.ldb, q.stride_b, BK, bn, 64))
        return cudaErrorInvalidValue;
    } else {
      mbl = mb;
    }
  }
  TcEpilogue ep;
  ep.m = (int)q.m; ep.n = (int)q.n;
  ep.c = q.c; ep.ldc = q.ldc; ep.sc = q.stride_c;
  ep.alpha = q.alpha; ep.beta = q.beta;
  ep.cin = q.beta != 0.f ? q.c_in : nullptr; ep.ldcin = q.ldc_in; ep.scin = q.stride_c_in;
  ep.bias_n = q.bias_n; ep.bias_m = q.bias_m; ep.bias_scale = q.bias_scale;
  ep.act = q.act; ep.act_alpha = q.act_alpha; ep.act_beta = q.act_beta;
  ep.res = q.residual; ep.ldres = q.ld_res; ep.sres = q.stride_res;
  ep.c16_hi = static_cast<uint2*>(q.c16_hi); ep.c16_lo = static_cast<uint2*>(q.c16_lo); ep.ldc16 = q.ldc16;
  ep.c16_fixed = q.c16_fixed;
  ep.acc_scale = kmode == TC_F16X3 ? q.b16_inv_scale : nullptr;
  ep.acc_scale_const = (kmode == TC_F16X3 && pre) ? kFixedUnscale : 1.f;   // A arrives on the fixed scale
  ep.b_row_scale = q.b_row_scale; ep.b_row_scale_stride = q.b_row_scale_stride; ep.k_total = (int)q.k;
  if (q.b_row_scale && kmode != TC_3X_SPLIT_B_MN) return cudaErrorInvalidValue;   // exists for the [K, N] operand only
  ep.err = err_word;
  if (q.c16_hi) {
    // Only the pair kernel's common epilogues (and the tail fix-up) write the split result.
    if (!(sh.pair && pre) || !q.c16_lo || q.batch != 1 || (q.n % 8) != 0 || (q.ldc16 % 8) != 0 ||
        !gemm_tc_can_split_output(q.act, q.bias_n != nullptr, q.bias_m != nullptr, q.c_in && q.beta != 0.f, q.alpha, q.bias_scale) ||
        (q.c && ((q.ldc % 4) != 0 || (reinterpret_cast<uintptr_t>(q.c) & 15) != 0)) ||
        (q.residual && ((q.ld_res % 4) != 0 || (reinterpret_cast<uintptr_t>(q.residual) & 15) != 0)) ||
        (q.bias_n && (reinterpret_cast<uintptr_t>(q.bias_n) & 15) != 0))
      return cudaErrorInvalidValue;
  } else if (!q.c) {
    return cudaErrorInvalidValue;
  }
  ep.dbg = std::getenv("ALTIUS_CUDA_TC_DBG") ? std::atoi(std::getenv("ALTIUS_CUDA_TC_DBG")) : 0;
  TcPlan pl = make_plan(q.m, q.n, q.k, q.batch, bn, sh.mt, (sh.pair && pre) ? 64 : (kmode == TC_F16X3 ? BK16 : BK),
                        sh.pair ? pair_count() : 0);
  if (pl.sc.tail_parts >= 2 && (!q.workspace || q.workspace_bytes < pl.workspace_bytes)) {
    // No (or too small a) workspace: fall back to whole tiles only.
    pl.sc.dp_tiles = pl.sc.num_tiles;
    pl.sc.tail_parts = 0;
  }
  float* ws = q.workspace;
  if (sh.pair && pre) return launch_pair<256, true>(q.a, q.lda, (int)q.k, ma, mal, mb, mbl, ep, pl, ws, err_word, st);
  if (sh.pair) return launch_pair<256, false>(q.a, q.lda, (int)q.k, ma, ma, mb, mbl, ep, pl, ws, err_word, st);
#define AC_TC(BNV)                                                                                         \
  (kmode == TC_1X ? launch_tc<BNV, 1, TC_1X>(ma, mb, mbl, ep, pl, a_batched, b_batched, ws, err_word, st)     \
   : kmode == TC_F16X3                                                                                     \
       ? launch_tc<BNV, 1, TC_F16X3>(ma, mb, mbl, ep, pl, a_batched, b_batched, ws, err_word, st)           \
   : kmode == TC_3X_BLO_TMA                                                                                \
       ? launch_tc<BNV, 1, TC_3X_BLO_TMA>(ma, mb, mbl, ep, pl, a_batched, b_batched, ws, err_word, st)      \
   : kmode == TC_3X_SPLIT_B_MN                                                                             \
       ? launch_tc<BNV, 1, TC_3X_SPLIT_B_MN>(ma, mb, mbl, ep, pl, a_batched, b_batched, ws, err_word, st)   \
       : launch_tc<BNV, 1, TC_3X_SPLIT_B>(ma, mb, mbl, ep, pl, a_batched, b_batched, ws, err_word, st))
  if (bn == 256) return AC_TC(256);
  if (bn == 128) return AC_TC(128);
  return AC_TC(64);
#undef AC_TC
}

cudaError_t launch_f16_split(const float* x, void* hi, void* lo, int64_t rows, int64_t k, int64_t ld, int64_t k8,
                             int* err_word, float* inv_scale, unsigned* absmax_scratch, int plain, cudaStream_t st) {
  const int64_t n = rows * k8;
  if (n == 0) return cudaSuccess;
  if (inv_scale) {   // a constant operand: scaled by a power of two first
    if (!absmax_scratch) return cudaErrorInvalidValue;
    cudaError_t e = cudaMemsetAsync(absmax_scratch, 0, sizeof(unsigned), st);
    if (e != cudaSuccess) return e;
    const int64_t blocks = std::min<int64_t>((rows * k + 255) / 256, 1184);
    absmax_kernel<<<(unsigned)blocks, 256, 0, st>>>(x, rows, k, ld, absmax_scratch);
    f16_split_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(x, static_cast<__half*>(hi), static_cast<__half*>(lo),
                                                                 rows, k, ld, k8, err_word, absmax_scratch, inv_scale, plain);
    return cudaGetLastError();
  }
  if (k8 == k && (k % 8) == 0 && (ld % 4) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(hi) & 15) == 0 && (reinterpret_cast<uintptr_t>(lo) & 15) == 0) {
    const int64_t n8 = n / 8;
    f16_split_vec8_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, st>>>(x, static_cast<uint4*>(hi), static_cast<uint4*>(lo),
                                                                       rows, k / 8, ld, err_word, plain);
    return cudaGetLastError();
  }
  f16_split_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(x, static_cast<__half*>(hi), static_cast<__half*>(lo),
                                                               rows, k, ld, k8, err_word, nullptr, nullptr, plain);
  return cudaGetLastError();
}

bool gemm_tc_can_split_output(int act, bool bias_n, bool bias_m, bool c_in, float alpha, float bias_scale) {
  // The epilogues the pair kernel has compiled in with the split store (epilogue_parked's callers).
  return !bias_m && !c_in && alpha == 1.f && bias_scale == 1.f && (act == ACT_NONE || (bias_n && (act == ACT_GELU || act == ACT_RELU)));
}

cudaError_t launch_tf32_split(const float* x, float* hi, float* lo, int64_t n, cudaStream_t st) {
  if (n == 0) return cudaSuccess;
  tf32_split_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(x, hi, lo, n);
  return cudaGetLastError();
}

}  // namespace ac
