// Row kernels: reductions over the last axis. Softmax, LayerNormalization
// (with its elementwise producers folded in), ReduceMean / ReduceMax,
// GlobalAveragePool, whole-tensor ReduceMax.
//
// One warp owns one row; the row lives in registers between the reduction
// passes, so every element is read from HBM once and written once. Reductions
// are warp-shuffle trees. The per-element arithmetic restates the reference
// (crates/session_interpreter/src/session.rs and fast_math.rs); only the
// summation order differs (tree instead of 8-lane partial sums).
#include <cstdlib>

#include "kernels.h"
#include "ref_math.cuh"
#include "tc_common.cuh"

namespace ac {
namespace {

constexpr int kWarpsPerBlock = 8;
constexpr int kThreads = kWarpsPerBlock * 32;
constexpr unsigned kFull = 0xffffffffu;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(kFull, v, o));
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(kFull, v, o));
  return v;
}

template <int MODE>
__device__ __forceinline__ float pre_scale(float x, float s) {
  if (MODE == 1) return __fmul_rn(x, s);
  if (MODE == 2) return __fdiv_rn(x, s);
  return x;
}

// ---- Softmax -----------------------------------------------------------------
// compute_softmax, session.rs:990-1026 + fast_sum_exp, fast_math.rs:102-187:
// m = max(row) ignoring NaN; e = exp_poly(max(x - m, -88.37626)); out = e * (1 / sum e).
struct SoftmaxMask {
  const uint8_t* mask;   // [mask_rows, len] or null
  int64_t mask_rows;
  const float* other;    // value where the mask is false
};

template <int VPT, int MODE, bool MASK>
__global__ void __launch_bounds__(kThreads) softmax_warp(const float* __restrict__ x,
                                                         float* __restrict__ out, int64_t rows,
                                                         int len, const float* __restrict__ scale, SoftmaxMask mk) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * kWarpsPerBlock;
  const float s = MODE ? __ldg(scale) : 1.f;
  const float other = MASK ? __ldg(mk.other) : 0.f;
  for (int64_t row = warp; row < rows; row += nwarps) {
    const float* xr = x + row * len;
    const uint8_t* mr = MASK ? mk.mask + (row % mk.mask_rows) * len : nullptr;
    float v[VPT];
    float m = CUDART_NAN_F;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = lane + 32 * i;
      if (c < len) {
        v[i] = pre_scale<MODE>(__ldg(xr + c), s);
        if (MASK) v[i] = mr[c] ? v[i] : other;     // Where(mask, x, other): a selection, exact
        m = fmaxf(v[i], m);
      }
    }
    m = warp_max(m);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = lane + 32 * i;
      if (c < len) {
        v[i] = exp_poly_softmax(__fsub_rn(v[i], m));
        sum = __fadd_rn(sum, v[i]);
      }
    }
    sum = warp_sum(sum);
    const float recip = __fdiv_rn(1.f, sum);
    float* orow = out + row * len;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = lane + 32 * i;
      if (c < len) orow[c] = __fmul_rn(v[i], recip);
    }
  }
}

// Rows longer than the register path holds: three passes over the row by one
// warp (the re-reads hit L1/L2).
template <int MODE, bool MASK>
__global__ void __launch_bounds__(kThreads) softmax_long(const float* __restrict__ x,
                                                         float* __restrict__ out, int64_t rows,
                                                         int64_t len,
                                                         const float* __restrict__ scale, SoftmaxMask mk) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * kWarpsPerBlock;
  const float s = MODE ? __ldg(scale) : 1.f;
  const float other = MASK ? __ldg(mk.other) : 0.f;
  for (int64_t row = warp; row < rows; row += nwarps) {
    const float* xr = x + row * len;
    const uint8_t* mr = MASK ? mk.mask + (row % mk.mask_rows) * len : nullptr;
    float* orow = out + row * len;
    auto val = [&](int64_t c) {
      const float v = pre_scale<MODE>(xr[c], s);
      return MASK ? (mr[c] ? v : other) : v;
    };
    float m = CUDART_NAN_F;
    for (int64_t c = lane; c < len; c += 32) m = fmaxf(val(c), m);
    m = warp_max(m);
    float sum = 0.f;
    for (int64_t c = lane; c < len; c += 32) {
      const float e = exp_poly_softmax(__fsub_rn(val(c), m));
      orow[c] = e;
      sum = __fadd_rn(sum, e);
    }
    sum = warp_sum(sum);
    const float recip = __fdiv_rn(1.f, sum);
    for (int64_t c = lane; c < len; c += 32) orow[c] = __fmul_rn(orow[c], recip);
  }
}

template <int MODE, bool MASK>
cudaError_t softmax_dispatch(const float* x, float* out, int64_t rows, int64_t len,
                             const float* scale, SoftmaxMask mk, cudaStream_t st) {
  const int64_t blocks64 = (rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
  const unsigned blocks = (unsigned)(blocks64 > device_sm_count() * 64 ? device_sm_count() * 64 : blocks64);
  const int vpt = (int)((len + 31) / 32);
#define AC_SM(V)                                                                         \
  softmax_warp<V, MODE, MASK><<<blocks, kThreads, 0, st>>>(x, out, rows, (int)len, scale, mk)
  if (vpt <= 1) AC_SM(1);
  else if (vpt <= 2) AC_SM(2);
  else if (vpt <= 4) AC_SM(4);
  else if (vpt <= 7) AC_SM(7);
  else if (vpt <= 8) AC_SM(8);
  else if (vpt <= 12) AC_SM(12);
  else if (vpt <= 16) AC_SM(16);
  else if (vpt <= 24) AC_SM(24);
  else if (vpt <= 32) AC_SM(32);
  else softmax_long<MODE, MASK><<<blocks, kThreads, 0, st>>>(x, out, rows, len, scale, mk);
#undef AC_SM
  return cudaGetLastError();
}

// ---- LayerNormalization --------------------------------------------------------
// compute_layer_normalization, session.rs:1465-1482:
//   mean = sum(x) * (1/n); o = x - mean; inv = 1 / sqrt(fma(sum(o*o), 1/n, eps));
//   out = fma(o * inv, gamma, beta)
// with the elementwise producers of x (bias Add, Gelu, residual Add) evaluated in
// registers first.
struct LnDev {
  const float* x; const float* pre_bias; const float* residual; const float* gamma;
  const float* beta; float* sum_out; float* out; int64_t rows; int len; float eps; int gelu;
  uint2* hi; uint2* lo; int* err;    // fp16 split of the result (4 halves per uint2), or null
};

__device__ __forceinline__ float ln_prologue(const LnDev& p, float v, int col, float res) {
  if (p.pre_bias) v = __fadd_rn(v, __ldg(p.pre_bias + col));
  if (p.gelu) v = gelu_ref(v);
  if (p.residual) v = __fadd_rn(v, res);
  return v;
}

// Vector path: len % 4 == 0, all pointers 16-byte aligned. NV float4 per lane.
// Each warp walks rows warp, warp + nwarps, ...; the next row's loads are issued
// before the current row is reduced and stored, so reads and writes overlap
// instead of alternating in phases. FUSED = false compiles the producers out.
template <int NV, bool FUSED>
__device__ __forceinline__ void ln_load_row(const LnDev& p, int64_t row, int lane, int nvec, float4 (&v)[NV],
                                            float4 (&r)[NV]) {
  const float4* xr = reinterpret_cast<const float4*>(p.x + row * p.len);
  const float4* rr = (FUSED && p.residual) ? reinterpret_cast<const float4*>(p.residual + row * p.len) : nullptr;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = lane + 32 * i;
    if (c < nvec) {
      v[i] = __ldg(xr + c);
      if (FUSED && rr) r[i] = __ldg(rr + c);
    }
  }
}

// The fused variants are bound by arithmetic (the Gelu above all), not by memory: they keep
// only the current row in registers (no prefetch of the next one), which lets two or three
// blocks share an SM.
// SPLIT: the result is (also) written as fp16 hi / lo halves on the fixed scale (f16_split_fixed)
// for the GEMM that consumes it.
// RESX (1, 2): the residual operand is the chain's own input x, so it is taken from the row in
// registers, float4 by float4, instead of being loaded and held as a second row: fewer live
// registers, which buys a fourth block per SM (1) or the prefetch of the next row (2).
// PF: the next row of a warp is prefetched into registers under the current one (pays when a
// warp walks many rows; with few rows per warp the registers are worth more as a second pair
// of resident blocks).
template <int NV, bool FUSED, bool GELU, bool SPLIT, int RESX, bool PF = (!FUSED || RESX == 2)>
__global__ void __launch_bounds__(kThreads, FUSED ? (RESX == 1 ? 4 : 3) : (PF ? 2 : 4)) layer_norm_vec(LnDev p) {
  constexpr bool PREFETCH = PF;
  float seen_max = 0.f;           // largest magnitude written as fixed-scale halves
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * kWarpsPerBlock;
  const int nvec = p.len >> 2;
  const float inv_n = __fdiv_rn(1.f, (float)p.len);
  int64_t row = warp;
  if (row >= p.rows) return;      // whole warps only: `warp` is uniform across the lanes
  constexpr bool LOAD_RES = FUSED && RESX == 0;
  float4 v[NV], r[LOAD_RES ? NV : 1];
  float4 nv[PREFETCH ? NV : 1];
  if (LOAD_RES) ln_load_row<NV, true>(p, row, lane, nvec, v, reinterpret_cast<float4(&)[NV]>(r));
  else ln_load_row<NV, false>(p, row, lane, nvec, v, reinterpret_cast<float4(&)[NV]>(v));
  while (true) {
    const int64_t next = row + nwarps;
    const bool has_next = next < p.rows;
    if (PREFETCH && has_next)
      ln_load_row<NV, false>(p, next, lane, nvec, reinterpret_cast<float4(&)[NV]>(nv), reinterpret_cast<float4(&)[NV]>(nv));
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = lane + 32 * i;
      if (c < nvec) {
        if (FUSED) {
          // Same operations as ln_prologue, with the options tested per float4 (or at
          // compile time for the Gelu) instead of per element.
          const float4 orig = v[i];
          if (p.pre_bias) {
            const float4 bv = __ldg(reinterpret_cast<const float4*>(p.pre_bias) + c);
            v[i].x = __fadd_rn(v[i].x, bv.x); v[i].y = __fadd_rn(v[i].y, bv.y);
            v[i].z = __fadd_rn(v[i].z, bv.z); v[i].w = __fadd_rn(v[i].w, bv.w);
          }
          if (GELU) {
            const float2 lo = gelu_ref2(make_float2(v[i].x, v[i].y));
            const float2 hi = gelu_ref2(make_float2(v[i].z, v[i].w));
            v[i] = make_float4(lo.x, lo.y, hi.x, hi.y);
          }
          if (RESX != 0) {
            v[i].x = __fadd_rn(v[i].x, orig.x); v[i].y = __fadd_rn(v[i].y, orig.y);
            v[i].z = __fadd_rn(v[i].z, orig.z); v[i].w = __fadd_rn(v[i].w, orig.w);
          } else if (p.residual) {
            v[i].x = __fadd_rn(v[i].x, r[LOAD_RES ? i : 0].x); v[i].y = __fadd_rn(v[i].y, r[LOAD_RES ? i : 0].y);
            v[i].z = __fadd_rn(v[i].z, r[LOAD_RES ? i : 0].z); v[i].w = __fadd_rn(v[i].w, r[LOAD_RES ? i : 0].w);
          }
          if (p.sum_out) reinterpret_cast<float4*>(p.sum_out + row * p.len)[c] = v[i];
        }
        sum = __fadd_rn(sum, __fadd_rn(__fadd_rn(v[i].x, v[i].y), __fadd_rn(v[i].z, v[i].w)));
      }
    }
    const float mean = __fmul_rn(warp_sum(sum), inv_n);
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = lane + 32 * i;
      if (c < nvec) {
        v[i].x = __fsub_rn(v[i].x, mean);
        v[i].y = __fsub_rn(v[i].y, mean);
        v[i].z = __fsub_rn(v[i].z, mean);
        v[i].w = __fsub_rn(v[i].w, mean);
        sq = __fadd_rn(sq, __fadd_rn(__fadd_rn(__fmul_rn(v[i].x, v[i].x), __fmul_rn(v[i].y, v[i].y)),
                                     __fadd_rn(__fmul_rn(v[i].z, v[i].z), __fmul_rn(v[i].w, v[i].w))));
      }
    }
    const float var = fmaf(warp_sum(sq), inv_n, p.eps);
    const float inv = __fdiv_rn(1.f, __fsqrt_rn(var));
    float4* orow = reinterpret_cast<float4*>(p.out + row * p.len);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = lane + 32 * i;
      if (c < nvec) {
        const float4 g = __ldg(reinterpret_cast<const float4*>(p.gamma) + c);
        const float4 b = __ldg(reinterpret_cast<const float4*>(p.beta) + c);
        float4 o;
        o.x = fmaf(__fmul_rn(v[i].x, inv), g.x, b.x);
        o.y = fmaf(__fmul_rn(v[i].y, inv), g.y, b.y);
        o.z = fmaf(__fmul_rn(v[i].z, inv), g.z, b.z);
        o.w = fmaf(__fmul_rn(v[i].w, inv), g.w, b.w);
        if (!SPLIT || p.out) orow[c] = o;
        if (SPLIT) {
          uint2 h, l;
          tc::f16_split_fixed(o, h, l);
          p.hi[row * nvec + c] = h;
          p.lo[row * nvec + c] = l;
          seen_max = tc::split_track(seen_max, o);
        }
      }
    }
    if (!has_next) break;
    row = next;
    if (PREFETCH) {
#pragma unroll
      for (int i = 0; i < NV; ++i) v[i] = nv[PREFETCH ? i : 0];
    } else if (LOAD_RES) {
      ln_load_row<NV, true>(p, row, lane, nvec, v, reinterpret_cast<float4(&)[NV]>(r));
    } else {
      ln_load_row<NV, false>(p, row, lane, nvec, v, reinterpret_cast<float4(&)[NV]>(v));
    }
  }
  if (SPLIT) tc::split_report_warp(tc::split_seen_fixed_of_max(seen_max), p.err);
}

// Any length / alignment: one warp per row, values recomputed from global
// memory in each pass (served by L1/L2 after the first).
__global__ void __launch_bounds__(kThreads) layer_norm_generic(LnDev p) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * kWarpsPerBlock;
  const float inv_n = __fdiv_rn(1.f, (float)p.len);
  for (int64_t row = warp; row < p.rows; row += nwarps) {
    const float* xr = p.x + row * p.len;
    const float* rr = p.residual ? p.residual + row * p.len : nullptr;
    float sum = 0.f;
    for (int c = lane; c < p.len; c += 32) {
      const float v = ln_prologue(p, xr[c], c, rr ? rr[c] : 0.f);
      if (p.sum_out) p.sum_out[row * p.len + c] = v;
      sum = __fadd_rn(sum, v);
    }
    const float mean = __fmul_rn(warp_sum(sum), inv_n);
    float sq = 0.f;
    for (int c = lane; c < p.len; c += 32) {
      const float o = __fsub_rn(ln_prologue(p, xr[c], c, rr ? rr[c] : 0.f), mean);
      sq = __fadd_rn(sq, __fmul_rn(o, o));
    }
    const float var = fmaf(warp_sum(sq), inv_n, p.eps);
    const float inv = __fdiv_rn(1.f, __fsqrt_rn(var));
    for (int c = lane; c < p.len; c += 32) {
      const float o = __fsub_rn(ln_prologue(p, xr[c], c, rr ? rr[c] : 0.f), mean);
      p.out[row * p.len + c] = fmaf(__fmul_rn(o, inv), __ldg(p.gamma + c), __ldg(p.beta + c));
    }
  }
}

// ---- last-axis reductions ---------------------------------------------------------
// MODE 0: mean = fast_sum(row) * (1/n)  (compute_reduce_mean, session.rs:1328-1339)
// MODE 1: max over the row              (ONNX ReduceMax on the last axis)
// MODE 2: sum / n                       (compute_gavg_pool, session.rs:289-293)
template <int MODE>
__global__ void __launch_bounds__(kThreads) reduce_last(const float* __restrict__ x,
                                                        float* __restrict__ out, int64_t rows,
                                                        int64_t len) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * kWarpsPerBlock;
  const bool vec = (len % 4) == 0 && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
  for (int64_t row = warp; row < rows; row += nwarps) {
    const float* xr = x + row * len;
    float acc = MODE == 1 ? -CUDART_INF_F : 0.f;
    if (vec) {
      const float4* x4 = reinterpret_cast<const float4*>(xr);
      for (int64_t c = lane; c < (len >> 2); c += 32) {
        const float4 v = __ldg(x4 + c);
        if (MODE == 1) acc = fmaxf(fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)), acc);
        else acc = __fadd_rn(acc, __fadd_rn(__fadd_rn(v.x, v.y), __fadd_rn(v.z, v.w)));
      }
    } else {
      for (int64_t c = lane; c < len; c += 32) {
        const float v = __ldg(xr + c);
        acc = MODE == 1 ? fmaxf(v, acc) : __fadd_rn(acc, v);
      }
    }
    acc = MODE == 1 ? warp_max(acc) : warp_sum(acc);
    if (lane == 0) {
      if (MODE == 0) out[row] = __fmul_rn(acc, __fdiv_rn(1.0f, (float)len));
      else if (MODE == 1) out[row] = acc;
      else out[row] = __fdiv_rn(acc, (float)len);
    }
  }
}

// Rows of NV * 128 floats, 16-byte aligned: a warp takes two rows per step and issues all
// of their 2 * NV float4 loads before the first use. Same order of additions as reduce_last.
template <int MODE, int NV>
__global__ void __launch_bounds__(kThreads) reduce_last_vec(const float* __restrict__ x,
                                                            float* __restrict__ out, int64_t rows) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * kWarpsPerBlock;
  constexpr int len = NV * 128;
  const float inv_len = __fdiv_rn(1.0f, (float)len);
  for (int64_t row = 2 * warp; row < rows; row += 2 * nwarps) {
    const bool two = row + 1 < rows;
    const float4* x0 = reinterpret_cast<const float4*>(x + row * len);
    const float4* x1 = reinterpret_cast<const float4*>(x + (two ? row + 1 : row) * len);
    float4 a[NV], b[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) a[j] = __ldg(x0 + lane + 32 * j);
#pragma unroll
    for (int j = 0; j < NV; ++j) b[j] = __ldg(x1 + lane + 32 * j);
    float acc0 = MODE == 1 ? -CUDART_INF_F : 0.f, acc1 = acc0;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      if (MODE == 1) {
        acc0 = fmaxf(fmaxf(fmaxf(a[j].x, a[j].y), fmaxf(a[j].z, a[j].w)), acc0);
        acc1 = fmaxf(fmaxf(fmaxf(b[j].x, b[j].y), fmaxf(b[j].z, b[j].w)), acc1);
      } else {
        acc0 = __fadd_rn(acc0, __fadd_rn(__fadd_rn(a[j].x, a[j].y), __fadd_rn(a[j].z, a[j].w)));
        acc1 = __fadd_rn(acc1, __fadd_rn(__fadd_rn(b[j].x, b[j].y), __fadd_rn(b[j].z, b[j].w)));
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {      // the two rows' trees interleaved
      const float t0 = __shfl_xor_sync(0xffffffffu, acc0, o), t1 = __shfl_xor_sync(0xffffffffu, acc1, o);
      acc0 = MODE == 1 ? fmaxf(acc0, t0) : __fadd_rn(acc0, t0);
      acc1 = MODE == 1 ? fmaxf(acc1, t1) : __fadd_rn(acc1, t1);
    }
    if (lane < 2 && (lane == 0 || two)) {
      const float acc = lane == 0 ? acc0 : acc1;
      float r;
      if (MODE == 0) r = __fmul_rn(acc, inv_len);
      else if (MODE == 1) r = acc;
      else r = __fdiv_rn(acc, (float)len);
      out[row + lane] = r;
    }
  }
}

// ReduceMean and ReduceMax of the same rows in one pass over them (the two are siblings in
// the tensor-op micrograph): same loads, same order of additions as reduce_last_vec.
template <int NV>
__global__ void __launch_bounds__(kThreads) reduce_mean_max_vec(const float* __restrict__ x, float* __restrict__ mean_out,
                                                                float* __restrict__ max_out, int64_t rows) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * kWarpsPerBlock;
  constexpr int len = NV * 128;
  const float inv_len = __fdiv_rn(1.0f, (float)len);
  for (int64_t row = 2 * warp; row < rows; row += 2 * nwarps) {
    const bool two = row + 1 < rows;
    const float4* x0 = reinterpret_cast<const float4*>(x + row * len);
    const float4* x1 = reinterpret_cast<const float4*>(x + (two ? row + 1 : row) * len);
    float4 a[NV], b[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) a[j] = __ldg(x0 + lane + 32 * j);
#pragma unroll
    for (int j = 0; j < NV; ++j) b[j] = __ldg(x1 + lane + 32 * j);
    float s0 = 0.f, s1 = 0.f, m0 = -CUDART_INF_F, m1 = -CUDART_INF_F;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      m0 = fmaxf(fmaxf(fmaxf(a[j].x, a[j].y), fmaxf(a[j].z, a[j].w)), m0);
      m1 = fmaxf(fmaxf(fmaxf(b[j].x, b[j].y), fmaxf(b[j].z, b[j].w)), m1);
      s0 = __fadd_rn(s0, __fadd_rn(__fadd_rn(a[j].x, a[j].y), __fadd_rn(a[j].z, a[j].w)));
      s1 = __fadd_rn(s1, __fadd_rn(__fadd_rn(b[j].x, b[j].y), __fadd_rn(b[j].z, b[j].w)));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      s0 = __fadd_rn(s0, __shfl_xor_sync(0xffffffffu, s0, o));
      s1 = __fadd_rn(s1, __shfl_xor_sync(0xffffffffu, s1, o));
      m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, o));
      m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, o));
    }
    if (lane < 2 && (lane == 0 || two)) {
      mean_out[row + lane] = __fmul_rn(lane == 0 ? s0 : s1, inv_len);
      max_out[row + lane] = lane == 0 ? m0 : m1;
    }
  }
}

template <int MODE>
cudaError_t reduce_last_dispatch(const float* x, float* out, int64_t rows, int64_t len,
                                 cudaStream_t st) {
  if (rows == 0) return cudaSuccess;
  const int64_t blocks64 = (rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
  if ((len % 128) == 0 && len <= 1024 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    // One pair of rows per warp up to six blocks per SM (measured: a second pass of a
    // partly idle grid costs more than the extra blocks), a grid-stride walk beyond that.
    const int64_t want = (rows + 2 * kWarpsPerBlock - 1) / (2 * kWarpsPerBlock);
    const int64_t cap = (int64_t)device_sm_count() * 6;
    const unsigned vb = (unsigned)(want > cap ? cap : want);
    switch (len / 128) {
      case 1: reduce_last_vec<MODE, 1><<<vb, kThreads, 0, st>>>(x, out, rows); break;
      case 2: reduce_last_vec<MODE, 2><<<vb, kThreads, 0, st>>>(x, out, rows); break;
      case 3: reduce_last_vec<MODE, 3><<<vb, kThreads, 0, st>>>(x, out, rows); break;
      case 4: reduce_last_vec<MODE, 4><<<vb, kThreads, 0, st>>>(x, out, rows); break;
      case 5: reduce_last_vec<MODE, 5><<<vb, kThreads, 0, st>>>(x, out, rows); break;
      case 6: reduce_last_vec<MODE, 6><<<vb, kThreads, 0, st>>>(x, out, rows); break;
      case 7: reduce_last_vec<MODE, 7><<<vb, kThreads, 0, st>>>(x, out, rows); break;
      default: reduce_last_vec<MODE, 8><<<vb, kThreads, 0, st>>>(x, out, rows); break;
    }
    return cudaGetLastError();
  }
  const unsigned blocks = (unsigned)(blocks64 > device_sm_count() * 64 ? device_sm_count() * 64 : blocks64);
  reduce_last<MODE><<<blocks, kThreads, 0, st>>>(x, out, rows, len);
  return cudaGetLastError();
}

// ---- whole-tensor max (compute_reduce_max, session.rs:1292-1305) ---------------------
constexpr int kMaxAllBlocks = 1184;   // fixed bound on the partial maxima (sizes the scratch), not a grid rule

__global__ void __launch_bounds__(kThreads) max_all_stage(const float* __restrict__ x,
                                                          float* __restrict__ out, int64_t n) {
  __shared__ float sm[kWarpsPerBlock];
  float acc = -CUDART_INF_F;
  for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * kThreads)
    acc = fmaxf(__ldg(x + i), acc);
  acc = warp_max(acc);
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    acc = threadIdx.x < kWarpsPerBlock ? sm[threadIdx.x] : -CUDART_INF_F;
    acc = warp_max(acc);
    if (threadIdx.x == 0) out[blockIdx.x] = acc;
  }
}

}  // namespace

cudaError_t launch_softmax(const float* x, float* out, int64_t rows, int64_t len, int scale_mode,
                           const float* scale, const uint8_t* mask, int64_t mask_rows, const float* mask_else,
                           cudaStream_t st) {
  if (rows == 0 || len == 0) return cudaSuccess;
  if (mask) {
    if (mask_rows <= 0 || !mask_else) return cudaErrorInvalidValue;
    const SoftmaxMask mk{mask, mask_rows, mask_else};
    if (scale_mode == 1) return softmax_dispatch<1, true>(x, out, rows, len, scale, mk, st);
    if (scale_mode == 2) return softmax_dispatch<2, true>(x, out, rows, len, scale, mk, st);
    return softmax_dispatch<0, true>(x, out, rows, len, scale, mk, st);
  }
  const SoftmaxMask mk{nullptr, 1, nullptr};
  if (scale_mode == 1) return softmax_dispatch<1, false>(x, out, rows, len, scale, mk, st);
  if (scale_mode == 2) return softmax_dispatch<2, false>(x, out, rows, len, scale, mk, st);
  return softmax_dispatch<0, false>(x, out, rows, len, scale, mk, st);
}

cudaError_t launch_layer_norm(const LayerNormParams& q, cudaStream_t st) {
  if (q.rows == 0 || q.len == 0) return cudaSuccess;
  LnDev p{q.x, q.pre_bias, q.residual, q.gamma, q.beta, q.sum_out, q.out, q.rows, (int)q.len,
          q.eps, q.gelu, static_cast<uint2*>(q.out16_hi), static_cast<uint2*>(q.out16_lo), q.err_word};
  const bool split = q.out16_hi != nullptr;
  if (split && (!q.out16_lo || !q.err_word)) return cudaErrorInvalidValue;
  if (!split && !q.out) return cudaErrorInvalidValue;
  const int64_t blocks64 = (q.rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
  const unsigned blocks = (unsigned)(blocks64 > device_sm_count() * 64 ? device_sm_count() * 64 : blocks64);
  auto al = [](const void* ptr) { return ptr == nullptr || (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; };
  const bool vec = (q.len % 4) == 0 && q.len <= 32 * 4 * 8 && al(q.x) && al(q.residual) && al(q.pre_bias) &&
                   al(q.gamma) && al(q.beta) && al(q.sum_out) && al(q.out) && al(q.out16_hi) && al(q.out16_lo);
  if (split && !vec) return cudaErrorInvalidValue;   // the split output exists on the vector path only
  if (vec) {
    const int nv = (int)((q.len / 4 + 31) / 32);
    const bool fused = q.pre_bias || q.residual || q.gelu || q.sum_out;
    // Two blocks of 8 warps per SM: several rows per warp, so the prefetch of the next
    // row overlaps the stores of the current one.
    // The residual is the chain's own input (x + f(x)): variant 1 or 2 (debug toggle
    // ALTIUS_CUDA_LN_RESX=0|1|2 overrides the choice).
    static const int resx_env = std::getenv("ALTIUS_CUDA_LN_RESX") ? std::atoi(std::getenv("ALTIUS_CUDA_LN_RESX")) : -1;
    const int resx = (fused && q.residual && q.residual == q.x) ? (resx_env >= 0 ? resx_env : 1) : 0;
    // The plain kernel: with fewer than eight rows per warp at two blocks per SM, four blocks per
    // SM without the prefetch (debug toggle ALTIUS_CUDA_LN_PF=0|1 overrides the choice).
    static const int pf_env = std::getenv("ALTIUS_CUDA_LN_PF") ? std::atoi(std::getenv("ALTIUS_CUDA_LN_PF")) : -1;
    const bool few_rows = blocks64 < (int64_t)device_sm_count() * 2 * 8;
    const bool plain_pf = pf_env >= 0 ? pf_env != 0 : !few_rows;
    const int depth = fused ? (resx == 1 ? 4 : 3) : (plain_pf ? 2 : 4);    // blocks per SM
    const int64_t vcap = (int64_t)device_sm_count() * depth;
    const unsigned vblocks = blocks64 > vcap ? (unsigned)vcap : (unsigned)blocks64;
#define AC_LN2(NVV, SP)                                                                     \
  do {                                                                                     \
    if (fused && q.gelu && resx == 1) layer_norm_vec<NVV, true, true, SP, 1><<<vblocks, kThreads, 0, st>>>(p);  \
    else if (fused && q.gelu && resx == 2) layer_norm_vec<NVV, true, true, SP, 2><<<vblocks, kThreads, 0, st>>>(p);  \
    else if (fused && q.gelu) layer_norm_vec<NVV, true, true, SP, 0><<<vblocks, kThreads, 0, st>>>(p);  \
    else if (fused && resx) layer_norm_vec<NVV, true, false, SP, 1><<<vblocks, kThreads, 0, st>>>(p);   \
    else if (fused) layer_norm_vec<NVV, true, false, SP, 0><<<vblocks, kThreads, 0, st>>>(p);      \
    else if (plain_pf) layer_norm_vec<NVV, false, false, SP, 0, true><<<vblocks, kThreads, 0, st>>>(p);     \
    else layer_norm_vec<NVV, false, false, SP, 0, false><<<vblocks, kThreads, 0, st>>>(p);             \
  } while (0)
#define AC_LN(NVV)                                                                         \
  do {                                                                                     \
    if (split) AC_LN2(NVV, true);                                                          \
    else AC_LN2(NVV, false);                                                               \
  } while (0)
    if (nv <= 1) AC_LN(1);
    else if (nv <= 2) AC_LN(2);
    else if (nv <= 3) AC_LN(3);
    else if (nv <= 4) AC_LN(4);
    else if (nv <= 6) AC_LN(6);
    else AC_LN(8);
#undef AC_LN
#undef AC_LN2
  } else {
    layer_norm_generic<<<blocks, kThreads, 0, st>>>(p);
  }
  return cudaGetLastError();
}

cudaError_t launch_reduce_mean_last(const float* x, float* out, int64_t rows, int64_t len,
                                    cudaStream_t st) {
  return reduce_last_dispatch<0>(x, out, rows, len, st);
}
cudaError_t launch_reduce_max_last(const float* x, float* out, int64_t rows, int64_t len,
                                   cudaStream_t st) {
  return reduce_last_dispatch<1>(x, out, rows, len, st);
}
cudaError_t launch_reduce_mean_max_last(const float* x, float* mean_out, float* max_out, int64_t rows, int64_t len,
                                        cudaStream_t st) {
  if (rows == 0) return cudaSuccess;
  if ((len % 128) == 0 && len <= 1024 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    const int64_t want = (rows + 2 * kWarpsPerBlock - 1) / (2 * kWarpsPerBlock);
    const int64_t cap = (int64_t)device_sm_count() * 6;
    const unsigned vb = (unsigned)(want > cap ? cap : want);
    switch (len / 128) {
      case 1: reduce_mean_max_vec<1><<<vb, kThreads, 0, st>>>(x, mean_out, max_out, rows); break;
      case 2: reduce_mean_max_vec<2><<<vb, kThreads, 0, st>>>(x, mean_out, max_out, rows); break;
      case 3: reduce_mean_max_vec<3><<<vb, kThreads, 0, st>>>(x, mean_out, max_out, rows); break;
      case 4: reduce_mean_max_vec<4><<<vb, kThreads, 0, st>>>(x, mean_out, max_out, rows); break;
      case 5: reduce_mean_max_vec<5><<<vb, kThreads, 0, st>>>(x, mean_out, max_out, rows); break;
      case 6: reduce_mean_max_vec<6><<<vb, kThreads, 0, st>>>(x, mean_out, max_out, rows); break;
      case 7: reduce_mean_max_vec<7><<<vb, kThreads, 0, st>>>(x, mean_out, max_out, rows); break;
      default: reduce_mean_max_vec<8><<<vb, kThreads, 0, st>>>(x, mean_out, max_out, rows); break;
    }
    return cudaGetLastError();
  }
  cudaError_t e = reduce_last_dispatch<0>(x, mean_out, rows, len, st);
  return e != cudaSuccess ? e : reduce_last_dispatch<1>(x, max_out, rows, len, st);
}

cudaError_t launch_gavg_pool(const float* x, float* out, int64_t planes, int64_t hw,
                             cudaStream_t st) {
  return reduce_last_dispatch<2>(x, out, planes, hw, st);
}

int64_t reduce_max_all_scratch_elems(int64_t n) {
  const int64_t blocks = (n + kThreads - 1) / kThreads;
  return blocks < kMaxAllBlocks ? (blocks > 0 ? blocks : 1) : kMaxAllBlocks;
}

cudaError_t launch_reduce_max_all(const float* x, float* out, int64_t n, float* partials,
                                  cudaStream_t st) {
  if (n == 0) return cudaSuccess;
  const int64_t blocks = reduce_max_all_scratch_elems(n);
  max_all_stage<<<(unsigned)blocks, kThreads, 0, st>>>(x, partials, n);
  max_all_stage<<<1, kThreads, 0, st>>>(partials, out, blocks);
  return cudaGetLastError();
}

}  // namespace ac
