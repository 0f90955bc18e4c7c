// CUDA-core fp32 GEMM (explicit FMA accumulation) and the depthwise
// convolution stencil.
//
// The GEMM is the contraction path for shapes the tensor-core kernel does not
// take (tiny or oddly strided problems) and the fallback when gemm_mode forces
// it. It restates what the reference delegates to cblas_sgemm
// (crates/session_interpreter/src/gemm.rs:36-51, :95-110; MatMul / Gemm glue in
// session.rs:621-794; the per-(batch, group) GEMMs of conv2d.rs:145-209), with
// the bias / activation / residual consumers applied in the epilogue.
//
// Tiling: 128x128 output tile per 256-thread CTA, K step 16, each thread an
// 8x8 register block (two 4-wide halves 64 apart so shared-memory reads are
// conflict-free float4), operands staged through double-buffered shared memory
// with the next K step prefetched into registers during the math.
#include "kernels.h"
#include "ref_math.cuh"

namespace ac {
namespace {

constexpr int BM = 128, BN = 128, BK = 16, TM = 8, TN = 8, THREADS = 256;
constexpr int PAD = 4;

struct GemmDev {
  int m, n, k;
  const float* a; long long lda, sa; int ta;
  const float* b; long long ldb, sb; int tb;
  float* c; long long ldc, sc;
  float alpha, beta;
  const float* cin; long long ldcin, scin;
  const float* bias_n; const float* bias_m; float bias_scale;
  int act; float act_alpha, act_beta;
  const float* res; long long ldres, sres;
};

// Element (r, kk) of op(A): A[r, kk] (or A^T stored [K, M]).
__device__ __forceinline__ float load_a(const GemmDev& p, const float* a, int r, int kk) {
  if (r >= p.m || kk >= p.k) return 0.f;
  return p.ta ? __ldg(a + (long long)kk * p.lda + r) : __ldg(a + (long long)r * p.lda + kk);
}
__device__ __forceinline__ float load_b(const GemmDev& p, const float* b, int kk, int c) {
  if (c >= p.n || kk >= p.k) return 0.f;
  return p.tb ? __ldg(b + (long long)c * p.ldb + kk) : __ldg(b + (long long)kk * p.ldb + c);
}

// VEC: operands allow 128-bit loads along their contiguous dimension
// (alignment and leading dimensions checked on the host).
template <bool VEC>
__global__ void __launch_bounds__(THREADS) gemm_simt_kernel(GemmDev p) {
  __shared__ __align__(16) float As[2][BK][BM + PAD];
  __shared__ __align__(16) float Bs[2][BK][BN + PAD];
  const int bz = blockIdx.z;
  const float* a = p.a + (long long)bz * p.sa;
  const float* b = p.b + (long long)bz * p.sb;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;

  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  // Per-thread staging registers: 8 A values and 8 B values per K step.
  float ra[8], rb[8];

  auto fetch = [&](int k0) {
    // ---- A tile: BM x BK ----
    if (!p.ta) {
      // k contiguous: thread -> (row = tid / 4 + 64 * h, k4 = tid % 4)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int r = m0 + (tid >> 2) + 64 * h, kk = k0 + (tid & 3) * 4;
        if (VEC && r < p.m && kk + 3 < p.k) {
          const float4 v = __ldg(reinterpret_cast<const float4*>(a + (long long)r * p.lda + kk));
          ra[4 * h + 0] = v.x; ra[4 * h + 1] = v.y; ra[4 * h + 2] = v.z; ra[4 * h + 3] = v.w;
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) ra[4 * h + j] = load_a(p, a, r, kk + j);
        }
      }
    } else {
      // m contiguous: thread -> (k = tid / 32 + 8 * h, m4 = tid % 32)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int kk = k0 + (tid >> 5) + 8 * h, r = m0 + (tid & 31) * 4;
        if (VEC && kk < p.k && r + 3 < p.m) {
          const float4 v = __ldg(reinterpret_cast<const float4*>(a + (long long)kk * p.lda + r));
          ra[4 * h + 0] = v.x; ra[4 * h + 1] = v.y; ra[4 * h + 2] = v.z; ra[4 * h + 3] = v.w;
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) ra[4 * h + j] = load_a(p, a, r + j, kk);
        }
      }
    }
    // ---- B tile: BK x BN ----
    if (!p.tb) {
      // n contiguous: thread -> (k = tid / 32 + 8 * h, n4 = tid % 32)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int kk = k0 + (tid >> 5) + 8 * h, c = n0 + (tid & 31) * 4;
        if (VEC && kk < p.k && c + 3 < p.n) {
          const float4 v = __ldg(reinterpret_cast<const float4*>(b + (long long)kk * p.ldb + c));
          rb[4 * h + 0] = v.x; rb[4 * h + 1] = v.y; rb[4 * h + 2] = v.z; rb[4 * h + 3] = v.w;
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) rb[4 * h + j] = load_b(p, b, kk, c + j);
        }
      }
    } else {
      // k contiguous: thread -> (col = tid / 4 + 64 * h, k4 = tid % 4)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int c = n0 + (tid >> 2) + 64 * h, kk = k0 + (tid & 3) * 4;
        if (VEC && c < p.n && kk + 3 < p.k) {
          const float4 v = __ldg(reinterpret_cast<const float4*>(b + (long long)c * p.ldb + kk));
          rb[4 * h + 0] = v.x; rb[4 * h + 1] = v.y; rb[4 * h + 2] = v.z; rb[4 * h + 3] = v.w;
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) rb[4 * h + j] = load_b(p, b, kk + j, c);
        }
      }
    }
  };

  auto stash = [&](int buf) {
    if (!p.ta) {
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int j = 0; j < 4; ++j) As[buf][(tid & 3) * 4 + j][(tid >> 2) + 64 * h] = ra[4 * h + j];
    } else {
#pragma unroll
      for (int h = 0; h < 2; ++h)
        *reinterpret_cast<float4*>(&As[buf][(tid >> 5) + 8 * h][(tid & 31) * 4]) =
            make_float4(ra[4 * h], ra[4 * h + 1], ra[4 * h + 2], ra[4 * h + 3]);
    }
    if (!p.tb) {
#pragma unroll
      for (int h = 0; h < 2; ++h)
        *reinterpret_cast<float4*>(&Bs[buf][(tid >> 5) + 8 * h][(tid & 31) * 4]) =
            make_float4(rb[4 * h], rb[4 * h + 1], rb[4 * h + 2], rb[4 * h + 3]);
    } else {
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int j = 0; j < 4; ++j) Bs[buf][(tid & 3) * 4 + j][(tid >> 2) + 64 * h] = rb[4 * h + j];
    }
  };

  const int ktiles = (p.k + BK - 1) / BK;
  fetch(0);
  stash(0);
  __syncthreads();
  for (int kt = 0; kt < ktiles; ++kt) {
    const int buf = kt & 1;
    if (kt + 1 < ktiles) fetch((kt + 1) * BK);
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][kk][ty * 4]);
      const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][kk][ty * 4 + 64]);
      const float4 b0 = *reinterpret_cast<const float4*>(&Bs[buf][kk][tx * 4]);
      const float4 b1 = *reinterpret_cast<const float4*>(&Bs[buf][kk][tx * 4 + 64]);
      const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    if (kt + 1 < ktiles) {
      stash(buf ^ 1);
      __syncthreads();
    }
  }

  // ---- epilogue ----
  float* c = p.c + (long long)bz * p.sc;
  const float* cin = p.cin ? p.cin + (long long)bz * p.scin : nullptr;
  const float* res = p.res ? p.res + (long long)bz * p.sres : nullptr;
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int r = m0 + ty * 4 + (i & 3) + (i >> 2) * 64;
    if (r >= p.m) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int col = n0 + tx * 4 + (j & 3) + (j >> 2) * 64;
      if (col >= p.n) continue;
      float v = acc[i][j];
      if (p.alpha != 1.f) v = __fmul_rn(p.alpha, v);
      if (cin && p.beta != 0.f) {
        const float cv = __ldg(cin + (long long)r * p.ldcin + col);
        v = __fadd_rn(p.beta == 1.f ? cv : __fmul_rn(p.beta, cv), v);
      }
      if (p.bias_n) {
        const float bv = __ldg(p.bias_n + col);
        v = __fadd_rn(v, p.bias_scale == 1.f ? bv : __fmul_rn(p.bias_scale, bv));
      }
      if (p.bias_m) {
        const float bv = __ldg(p.bias_m + r);
        v = __fadd_rn(v, p.bias_scale == 1.f ? bv : __fmul_rn(p.bias_scale, bv));
      }
      v = apply_act(p.act, v, p.act_alpha, p.act_beta);
      if (res) v = __fadd_rn(v, __ldg(res + (long long)r * p.ldres + col));
      c[(long long)r * p.ldc + col] = v;
    }
  }
}

// Depthwise convolution (group == channels, one filter per channel). The
// reference computes it as 1 x k GEMMs over im2col columns
// (conv2d.rs:145-209); here each thread owns one output pixel and walks the
// taps with FMA, starting from 0 and adding the bias last (the reference's
// "bias + sum" and this "sum + bias" round identically).
__global__ void __launch_bounds__(256) depthwise_kernel(const float* __restrict__ x,
                                                        const float* __restrict__ w,
                                                        const float* __restrict__ bias,
                                                        float* __restrict__ out, ConvParams p,
                                                        long long total) {
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i >= total) return;
  const int ox = (int)(i % p.ow);
  const int oy = (int)((i / p.ow) % p.oh);
  const long long plane = i / ((long long)p.ow * p.oh);  // n * c + ch
  const int ch = (int)(plane % p.c);
  const float* in = x + plane * (long long)p.ih * p.iw;
  const float* wk = w + (long long)ch * p.kh * p.kw;
  const int y0 = oy * p.sh - p.pad_t, x0 = ox * p.sw - p.pad_l;
  float acc = 0.f;
  for (int fy = 0; fy < p.kh; ++fy) {
    const int iy = y0 + fy * p.dh;
    if (iy < 0 || iy >= p.ih) continue;
    for (int fx = 0; fx < p.kw; ++fx) {
      const int ix = x0 + fx * p.dw;
      if (ix < 0 || ix >= p.iw) continue;
      acc = fmaf(__ldg(wk + fy * p.kw + fx), __ldg(in + iy * p.iw + ix), acc);
    }
  }
  if (bias) acc = __fadd_rn(__ldg(bias + ch), acc);
  out[i] = apply_act(p.act, acc, p.act_alpha, p.act_beta);
}

// The same stencil for the shapes the CNNs have (square K x K filter, stride S, dilation 1),
// four consecutive output pixels of one row per thread: the filter taps sit in registers, an
// input row segment of 3 S + K values is loaded once per filter row and shared by the four
// pixels. Per output the taps are visited in the same order as above and out-of-range taps are
// skipped, so the results are bit-identical to the generic kernel.
template <int K, int S, int ACT>
__global__ void __launch_bounds__(256) depthwise_rows_kernel(const float* __restrict__ x,
                                                             const float* __restrict__ w,
                                                             const float* __restrict__ bias,
                                                             float* __restrict__ out, ConvParams p,
                                                             unsigned owg, unsigned items) {
  const unsigned item = blockIdx.x * 256u + threadIdx.x;
  if (item >= items) return;
  const unsigned xg = item % owg, t = item / owg;
  const unsigned oy = t % (unsigned)p.oh, plane = t / (unsigned)p.oh;   // plane = n * c + ch
  const int ch = (int)(plane % (unsigned)p.c);
  const float* in = x + (long long)plane * p.ih * p.iw;
  float wk[K * K];
#pragma unroll
  for (int i = 0; i < K * K; ++i) wk[i] = __ldg(w + ch * (K * K) + i);
  constexpr int SEG = 3 * S + K;
  const int ox0 = (int)xg * 4;
  const int y0 = (int)oy * S - p.pad_t, x0 = ox0 * S - p.pad_l;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int fy = 0; fy < K; ++fy) {
    const int iy = y0 + fy;
    if (iy < 0 || iy >= p.ih) continue;            // uniform per thread: all four pixels skip the row
    const float* row = in + iy * p.iw;
    float seg[SEG];
#pragma unroll
    for (int j = 0; j < SEG; ++j) {
      const int ix = x0 + j;
      seg[j] = (ix >= 0 && ix < p.iw) ? __ldg(row + ix) : 0.f;
    }
#pragma unroll
    for (int fx = 0; fx < K; ++fx)
#pragma unroll
      for (int o = 0; o < 4; ++o) {
        const int ix = x0 + o * S + fx;
        if (ix >= 0 && ix < p.iw) acc[o] = fmaf(wk[fy * K + fx], seg[o * S + fx], acc[o]);
      }
  }
  const float bv = bias ? __ldg(bias + ch) : 0.f;
  float* dst = out + ((long long)plane * p.oh + oy) * p.ow + ox0;
#pragma unroll
  for (int o = 0; o < 4; ++o) {
    if (ox0 + o >= p.ow) break;
    float v = acc[o];
    if (bias) v = __fadd_rn(bv, v);
    dst[o] = apply_act(ACT, v, p.act_alpha, p.act_beta);
  }
}

template <int K, int S>
bool launch_depthwise_rows(const ConvParams& p, const float* x, const float* w, const float* bias, float* out,
                           unsigned owg, unsigned items, cudaStream_t st) {
  const unsigned blocks = (items + 255u) / 256u;
  switch (p.act) {
    case ACT_NONE: depthwise_rows_kernel<K, S, ACT_NONE><<<blocks, 256, 0, st>>>(x, w, bias, out, p, owg, items); return true;
    case ACT_RELU: depthwise_rows_kernel<K, S, ACT_RELU><<<blocks, 256, 0, st>>>(x, w, bias, out, p, owg, items); return true;
    case ACT_HARDSWISH: depthwise_rows_kernel<K, S, ACT_HARDSWISH><<<blocks, 256, 0, st>>>(x, w, bias, out, p, owg, items); return true;
    default: return false;
  }
}

inline bool al16(const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; }

}  // namespace

cudaError_t launch_gemm_simt(const GemmParams& q, cudaStream_t st) {
  if (q.m == 0 || q.n == 0 || q.batch == 0) return cudaSuccess;
  if (q.batch > 65535 || (q.m + BM - 1) / BM > 65535) return cudaErrorInvalidValue;
  GemmDev p;
  p.m = (int)q.m; p.n = (int)q.n; p.k = (int)q.k;
  p.a = q.a; p.lda = q.lda; p.sa = q.stride_a; p.ta = q.trans_a;
  p.b = q.b; p.ldb = q.ldb; p.sb = q.stride_b; p.tb = q.trans_b;
  p.c = q.c; p.ldc = q.ldc; p.sc = q.stride_c;
  p.alpha = q.alpha; p.beta = q.beta;
  p.cin = q.beta != 0.f ? q.c_in : nullptr; p.ldcin = q.ldc_in; p.scin = q.stride_c_in;
  p.bias_n = q.bias_n; p.bias_m = q.bias_m; p.bias_scale = q.bias_scale;
  p.act = q.act; p.act_alpha = q.act_alpha; p.act_beta = q.act_beta;
  p.res = q.residual; p.ldres = q.ld_res; p.sres = q.stride_res;
  const bool vec = al16(q.a) && al16(q.b) && (q.lda % 4) == 0 && (q.ldb % 4) == 0 &&
                   (q.stride_a % 4) == 0 && (q.stride_b % 4) == 0;
  dim3 grid((unsigned)((q.n + BN - 1) / BN), (unsigned)((q.m + BM - 1) / BM), (unsigned)q.batch);
  if (vec) gemm_simt_kernel<true><<<grid, THREADS, 0, st>>>(p);
  else gemm_simt_kernel<false><<<grid, THREADS, 0, st>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_depthwise_conv(const ConvParams& p, const float* x, const float* w,
                                  const float* bias, float* out, cudaStream_t st) {
  const long long total = (long long)p.n * p.oc * p.oh * p.ow;
  if (total == 0) return cudaSuccess;
  const long long owg = (p.ow + 3) / 4, items = (long long)p.n * p.oc * p.oh * owg;
  if (p.kh == p.kw && p.sh == p.sw && p.dh == 1 && p.dw == 1 && items < (1ll << 31) &&
      (long long)p.ih * p.iw < (1ll << 31)) {
    bool done = false;
    if (p.kh == 3 && p.sh == 1) done = launch_depthwise_rows<3, 1>(p, x, w, bias, out, (unsigned)owg, (unsigned)items, st);
    else if (p.kh == 3 && p.sh == 2) done = launch_depthwise_rows<3, 2>(p, x, w, bias, out, (unsigned)owg, (unsigned)items, st);
    else if (p.kh == 5 && p.sh == 1) done = launch_depthwise_rows<5, 1>(p, x, w, bias, out, (unsigned)owg, (unsigned)items, st);
    else if (p.kh == 5 && p.sh == 2) done = launch_depthwise_rows<5, 2>(p, x, w, bias, out, (unsigned)owg, (unsigned)items, st);
    if (done) return cudaGetLastError();
  }
  depthwise_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(x, w, bias, out, p, total);
  return cudaGetLastError();
}

}  // namespace ac
