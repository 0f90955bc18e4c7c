// Elementwise kernels: NumPy-broadcast binary ops, unary activations, Greater,
// Where, Cast, BatchNormalization. All are HBM-bound streaming kernels:
// 128-bit loads/stores wherever alignment allows, several independent vectors
// in flight per thread, grids sized from the element count.
//
// Arithmetic follows the reference interpreter
// (crates/session_interpreter/src/session.rs): Add/Sub/Mul/Div are single IEEE
// operations (`op_bin_elemwise!`, :384-526) -- __fadd_rn/__fsub_rn/__fmul_rn/
// __fdiv_rn so nothing is contracted; the unary formulas are in ref_math.cuh.
#include "kernels.h"
#include "ref_math.cuh"

namespace ac {
namespace {

constexpr int kThreads = 256;

template <int OP>
__device__ __forceinline__ float bin_apply(float a, float b) {
  if (OP == BIN_ADD) return __fadd_rn(a, b);
  if (OP == BIN_SUB) return __fsub_rn(a, b);
  if (OP == BIN_MUL) return __fmul_rn(a, b);
  if (OP == BIN_DIV) return __fdiv_rn(a, b);
  return powf(a, b);  // compute_pow, session.rs:566-606
}

template <int OP>
__device__ __forceinline__ float4 bin_apply4(float4 a, float4 b) {
  return make_float4(bin_apply<OP>(a.x, b.x), bin_apply<OP>(a.y, b.y), bin_apply<OP>(a.z, b.z),
                     bin_apply<OP>(a.w, b.w));
}

// Same-shape operands, flat: 4 float4 per thread.
template <int OP>
__global__ void __launch_bounds__(kThreads) bin_flat_vec4(const float4* __restrict__ a,
                                                          const float4* __restrict__ b,
                                                          float4* __restrict__ o, int64_t nvec) {
  const int64_t base = ((int64_t)blockIdx.x * kThreads * 4) + threadIdx.x;
  float4 va[4], vb[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t idx = base + (int64_t)i * kThreads;
    if (idx < nvec) {
      va[i] = __ldg(a + idx);
      vb[i] = __ldg(b + idx);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t idx = base + (int64_t)i * kThreads;
    if (idx < nvec) o[idx] = bin_apply4<OP>(va[i], vb[i]);
  }
}

struct BcastDev {
  int rank;               // >= 1
  int64_t inner;          // dims[rank-1] (in elements)
  int64_t dims[kMaxRank]; // outer dims only are used for decomposition
  int64_t a_str[kMaxRank];
  int64_t b_str[kMaxRank];
};

// General broadcast kernel. Each thread produces VEC consecutive inner
// elements. A_IN / B_IN are the inner strides (0 or 1) known at compile time
// for the vector path; the scalar path reads them from the params.
template <int OP, int VEC, typename IDX>
__global__ void __launch_bounds__(kThreads) bin_bcast(const float* __restrict__ a,
                                                      const float* __restrict__ b,
                                                      float* __restrict__ o, BcastDev p,
                                                      IDX n_items) {
  const IDX item = (IDX)blockIdx.x * kThreads + threadIdx.x;
  if (item >= n_items) return;
  const IDX inner_items = (IDX)(p.inner / VEC);
  IDX outer = item / inner_items;
  const IDX in = (item - outer * inner_items) * VEC;
  const IDX oidx = outer * (IDX)p.inner + in;
  int64_t ao = 0, bo = 0;
#pragma unroll 1
  for (int d = p.rank - 2; d >= 0; --d) {
    const IDX dim = (IDX)p.dims[d];
    const IDX q = outer / dim;
    const IDX r = outer - q * dim;
    ao += (int64_t)r * p.a_str[d];
    bo += (int64_t)r * p.b_str[d];
    outer = q;
  }
  const int64_t sa = p.a_str[p.rank - 1], sb = p.b_str[p.rank - 1];
  if (VEC == 4) {
    float4 va, vb;
    if (sa == 1) va = __ldg(reinterpret_cast<const float4*>(a + ao + in));
    else { const float s = __ldg(a + ao); va = make_float4(s, s, s, s); }
    if (sb == 1) vb = __ldg(reinterpret_cast<const float4*>(b + bo + in));
    else { const float s = __ldg(b + bo); vb = make_float4(s, s, s, s); }
    *reinterpret_cast<float4*>(o + oidx) = bin_apply4<OP>(va, vb);
  } else {
    o[oidx] = bin_apply<OP>(__ldg(a + ao + (int64_t)in * sa), __ldg(b + bo + (int64_t)in * sb));
  }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <int OP>
cudaError_t binary_dispatch(const BinaryParams& p, const float* a, const float* b, float* out,
                            cudaStream_t st) {
  if (p.n == 0) return cudaSuccess;
  const int r = p.rank;
  // Flat same-shape fast path.
  if (r == 1 && p.a_str[0] == 1 && p.b_str[0] == 1 && (p.n % 4) == 0 && aligned16(a) &&
      aligned16(b) && aligned16(out)) {
    const int64_t nvec = p.n / 4;
    const int64_t blocks = (nvec + kThreads * 4 - 1) / (kThreads * 4);
    bin_flat_vec4<OP><<<(unsigned)blocks, kThreads, 0, st>>>(
        reinterpret_cast<const float4*>(a), reinterpret_cast<const float4*>(b),
        reinterpret_cast<float4*>(out), nvec);
    return cudaGetLastError();
  }
  BcastDev d;
  d.rank = r;
  d.inner = p.dims[r - 1];
  for (int i = 0; i < kMaxRank; ++i) {
    d.dims[i] = i < r ? p.dims[i] : 1;
    d.a_str[i] = i < r ? p.a_str[i] : 0;
    d.b_str[i] = i < r ? p.b_str[i] : 0;
  }
  const int64_t sa = p.a_str[r - 1], sb = p.b_str[r - 1];
  bool vec = (d.inner % 4) == 0 && (sa == 0 || sa == 1) && (sb == 0 || sb == 1) && aligned16(out) &&
             (sa == 0 || aligned16(a)) && (sb == 0 || aligned16(b));
  for (int i = 0; i < r - 1 && vec; ++i) {
    if (sa == 1 && (p.a_str[i] % 4) != 0) vec = false;
    if (sb == 1 && (p.b_str[i] % 4) != 0) vec = false;
  }
  const int64_t items = vec ? p.n / 4 : p.n;
  const int64_t blocks = (items + kThreads - 1) / kThreads;
  const bool small = p.n < (int64_t(1) << 31);
  if (vec) {
    if (small) bin_bcast<OP, 4, unsigned><<<(unsigned)blocks, kThreads, 0, st>>>(a, b, out, d, (unsigned)items);
    else bin_bcast<OP, 4, int64_t><<<(unsigned)blocks, kThreads, 0, st>>>(a, b, out, d, items);
  } else {
    if (small) bin_bcast<OP, 1, unsigned><<<(unsigned)blocks, kThreads, 0, st>>>(a, b, out, d, (unsigned)items);
    else bin_bcast<OP, 1, int64_t><<<(unsigned)blocks, kThreads, 0, st>>>(a, b, out, d, items);
  }
  return cudaGetLastError();
}

// ---- unary -----------------------------------------------------------------
template <int OP>
__device__ __forceinline__ float un_apply(float x, float alpha, float beta) {
  switch (OP) {
    case UN_RELU: return fmaxf(x, 0.f);                       // session.rs:801 x.max(0.0)
    case UN_SIGMOID: return sigmoid_ref(x);
    case UN_ERF: return erff(x);                              // un-vendored in the reference
    case UN_GELU: return gelu_ref(x);
    case UN_HARDSIGMOID: return hard_sigmoid_ref(x, alpha, beta);
    case UN_LEAKYRELU: return x < 0.f ? __fmul_rn(alpha, x) : x;  // session.rs:819
    case UN_SQRT: return __fsqrt_rn(x);
    case UN_TANH: return tanh_ref(x);
    case UN_HARDSWISH: return __fmul_rn(x, hard_sigmoid_ref(x, alpha, beta));
    case UN_SQUARE: return __fmul_rn(x, x);
    default: return x;
  }
}

template <int OP>
__global__ void __launch_bounds__(kThreads) unary_vec4(const float4* __restrict__ x,
                                                       float4* __restrict__ o, int64_t nvec,
                                                       float alpha, float beta) {
  const int64_t base = ((int64_t)blockIdx.x * kThreads * 4) + threadIdx.x;
  float4 v[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t idx = base + (int64_t)i * kThreads;
    if (idx < nvec) v[i] = __ldg(x + idx);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t idx = base + (int64_t)i * kThreads;
    if (idx >= nvec) continue;
    if (OP == UN_GELU) {   // two elements per instruction; same bits as gelu_ref
      const float2 lo = gelu_ref2(make_float2(v[i].x, v[i].y)), hi = gelu_ref2(make_float2(v[i].z, v[i].w));
      o[idx] = make_float4(lo.x, lo.y, hi.x, hi.y);
    } else {
      o[idx] = make_float4(un_apply<OP>(v[i].x, alpha, beta), un_apply<OP>(v[i].y, alpha, beta),
                           un_apply<OP>(v[i].z, alpha, beta), un_apply<OP>(v[i].w, alpha, beta));
    }
  }
}

template <int OP>
__global__ void __launch_bounds__(kThreads) unary_scalar(const float* __restrict__ x,
                                                         float* __restrict__ o, int64_t n,
                                                         float alpha, float beta) {
  const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (i < n) o[i] = un_apply<OP>(__ldg(x + i), alpha, beta);
}

template <int OP>
cudaError_t unary_dispatch(const float* x, float* out, int64_t n, float alpha, float beta,
                           cudaStream_t st) {
  if (n == 0) return cudaSuccess;
  if ((n % 4) == 0 && aligned16(x) && aligned16(out)) {
    const int64_t nvec = n / 4;
    const int64_t blocks = (nvec + kThreads * 4 - 1) / (kThreads * 4);
    unary_vec4<OP><<<(unsigned)blocks, kThreads, 0, st>>>(reinterpret_cast<const float4*>(x),
                                                          reinterpret_cast<float4*>(out), nvec,
                                                          alpha, beta);
  } else {
    const int64_t blocks = (n + kThreads - 1) / kThreads;
    unary_scalar<OP><<<(unsigned)blocks, kThreads, 0, st>>>(x, out, n, alpha, beta);
  }
  return cudaGetLastError();
}

__global__ void greater_scalar_kernel(const float* __restrict__ x, const float* __restrict__ y,
                                      uint8_t* __restrict__ o, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) o[i] = __ldg(x + i) > __ldg(y) ? 1 : 0;  // session.rs:547-556
}

__global__ void where_kernel(int mode, const uint8_t* __restrict__ cond, const float* __restrict__ x,
                             const float* __restrict__ y, float* __restrict__ o, int64_t n,
                             int64_t inner) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  if (mode == 0) o[i] = cond[i] ? __ldg(x) : __ldg(y + i);          // session.rs:947-956
  else o[i] = cond[i % inner] ? __ldg(x + i) : __ldg(y);            // session.rs:966-987
}

// General broadcast forms: one thread per output element, offsets by mixed-radix decomposition.
struct TernDev {
  int rank;
  int64_t dims[kMaxRank], c_str[kMaxRank], x_str[kMaxRank], y_str[kMaxRank];
};
__device__ __forceinline__ void tern_offsets(const TernDev& p, int64_t i, int64_t* co, int64_t* xo, int64_t* yo) {
  int64_t c = 0, x = 0, y = 0;
#pragma unroll 1
  for (int d = p.rank - 1; d >= 0; --d) {
    const int64_t q = i / p.dims[d], r = i - q * p.dims[d];
    c += r * p.c_str[d]; x += r * p.x_str[d]; y += r * p.y_str[d];
    i = q;
  }
  *co = c; *xo = x; *yo = y;
}
__global__ void greater_bcast_kernel(const float* __restrict__ x, const float* __restrict__ y,
                                     uint8_t* __restrict__ o, TernDev p, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int64_t co, xo, yo;
  tern_offsets(p, i, &co, &xo, &yo);
  o[i] = __ldg(x + xo) > __ldg(y + yo) ? 1 : 0;
}
__global__ void where_bcast_kernel(const uint8_t* __restrict__ cond, const float* __restrict__ x,
                                   const float* __restrict__ y, float* __restrict__ o, TernDev p, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int64_t co, xo, yo;
  tern_offsets(p, i, &co, &xo, &yo);
  o[i] = cond[co] ? __ldg(x + xo) : __ldg(y + yo);
}

template <typename TI, typename TO>
__global__ void cast_kernel(const TI* __restrict__ x, TO* __restrict__ o, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) o[i] = (TO)x[i];
}
template <typename TI>
__global__ void cast_to_bool_kernel(const TI* __restrict__ x, uint8_t* __restrict__ o, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) o[i] = x[i] != (TI)0 ? 1 : 0;
}
__global__ void cast_f32_bool_kernel(const float* __restrict__ x, uint8_t* __restrict__ o,
                                     int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) o[i] = x[i] != 0.0f ? 1 : 0;  // session.rs:1369-1374
}

// session.rs:1423-1426: ((x - mean) / sqrt(var + eps)) * scale + bias, no FMA.
__global__ void batch_norm_kernel(const float* __restrict__ x, const float* __restrict__ scale,
                                  const float* __restrict__ bias, const float* __restrict__ mean,
                                  const float* __restrict__ var, float* __restrict__ o, int64_t n,
                                  int64_t c, int64_t hw, float eps) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int64_t ch = (i / hw) % c;
  const float d = __fsqrt_rn(__fadd_rn(__ldg(var + ch), eps));
  const float v = __fdiv_rn(__fsub_rn(__ldg(x + i), __ldg(mean + ch)), d);
  o[i] = __fadd_rn(__fmul_rn(v, __ldg(scale + ch)), __ldg(bias + ch));
}

}  // namespace

cudaError_t launch_binary(const BinaryParams& p, const float* a, const float* b, float* out,
                          cudaStream_t st) {
  switch (p.op) {
    case BIN_ADD: return binary_dispatch<BIN_ADD>(p, a, b, out, st);
    case BIN_SUB: return binary_dispatch<BIN_SUB>(p, a, b, out, st);
    case BIN_MUL: return binary_dispatch<BIN_MUL>(p, a, b, out, st);
    case BIN_DIV: return binary_dispatch<BIN_DIV>(p, a, b, out, st);
    case BIN_POW: return binary_dispatch<BIN_POW>(p, a, b, out, st);
  }
  return cudaErrorInvalidValue;
}

cudaError_t launch_unary(int op, float alpha, float beta, const float* x, float* out, int64_t n,
                         cudaStream_t st) {
  switch (op) {
    case UN_RELU: return unary_dispatch<UN_RELU>(x, out, n, alpha, beta, st);
    case UN_SIGMOID: return unary_dispatch<UN_SIGMOID>(x, out, n, alpha, beta, st);
    case UN_ERF: return unary_dispatch<UN_ERF>(x, out, n, alpha, beta, st);
    case UN_GELU: return unary_dispatch<UN_GELU>(x, out, n, alpha, beta, st);
    case UN_HARDSIGMOID: return unary_dispatch<UN_HARDSIGMOID>(x, out, n, alpha, beta, st);
    case UN_LEAKYRELU: return unary_dispatch<UN_LEAKYRELU>(x, out, n, alpha, beta, st);
    case UN_SQRT: return unary_dispatch<UN_SQRT>(x, out, n, alpha, beta, st);
    case UN_TANH: return unary_dispatch<UN_TANH>(x, out, n, alpha, beta, st);
    case UN_HARDSWISH: return unary_dispatch<UN_HARDSWISH>(x, out, n, alpha, beta, st);
    case UN_SQUARE: return unary_dispatch<UN_SQUARE>(x, out, n, alpha, beta, st);
    case UN_COPY: return unary_dispatch<UN_COPY>(x, out, n, alpha, beta, st);
  }
  return cudaErrorInvalidValue;
}

cudaError_t launch_greater_scalar(const float* x, const float* y, uint8_t* out, int64_t n,
                                  cudaStream_t st) {
  if (n == 0) return cudaSuccess;
  greater_scalar_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(x, y, out, n);
  return cudaGetLastError();
}

cudaError_t launch_where(int mode, const uint8_t* cond, const float* x, const float* y, float* out,
                         int64_t n, int64_t inner, cudaStream_t st) {
  if (n == 0) return cudaSuccess;
  where_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(mode, cond, x, y, out, n,
                                                           inner > 0 ? inner : 1);
  return cudaGetLastError();
}

namespace {
TernDev tern_dev(const TernaryParams& p) {
  TernDev d;
  d.rank = p.rank;
  for (int i = 0; i < kMaxRank; ++i) {
    d.dims[i] = i < p.rank ? p.dims[i] : 1;
    d.c_str[i] = i < p.rank ? p.c_str[i] : 0;
    d.x_str[i] = i < p.rank ? p.x_str[i] : 0;
    d.y_str[i] = i < p.rank ? p.y_str[i] : 0;
  }
  return d;
}
}  // namespace

cudaError_t launch_greater_bcast(const TernaryParams& p, const float* x, const float* y, uint8_t* out, cudaStream_t st) {
  if (p.n == 0) return cudaSuccess;
  greater_bcast_kernel<<<(unsigned)((p.n + 255) / 256), 256, 0, st>>>(x, y, out, tern_dev(p), p.n);
  return cudaGetLastError();
}

cudaError_t launch_where_bcast(const TernaryParams& p, const uint8_t* cond, const float* x, const float* y, float* out,
                               cudaStream_t st) {
  if (p.n == 0) return cudaSuccess;
  where_bcast_kernel<<<(unsigned)((p.n + 255) / 256), 256, 0, st>>>(cond, x, y, out, tern_dev(p), p.n);
  return cudaGetLastError();
}

namespace {
template <typename TI>
cudaError_t cast_from(int to, const TI* x, void* out, int64_t n, unsigned blocks, cudaStream_t st) {
  switch (to) {
    case 0: cast_to_bool_kernel<TI><<<blocks, 256, 0, st>>>(x, (uint8_t*)out, n); break;
    case 1: cast_kernel<TI, float><<<blocks, 256, 0, st>>>(x, (float*)out, n); break;
    case 2: cast_kernel<TI, int32_t><<<blocks, 256, 0, st>>>(x, (int32_t*)out, n); break;
    case 3: cast_kernel<TI, int64_t><<<blocks, 256, 0, st>>>(x, (int64_t*)out, n); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}
}  // namespace

cudaError_t launch_cast(int from, int to, const void* x, void* out, int64_t n, cudaStream_t st) {
  if (n == 0) return cudaSuccess;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  // Beyond the four pairs of the reference (below): every other pair of bool / f32 / i32 / i64.
  const bool ref_pair = (from == 2 && to == 1) || (from == 3 && to == 2) || (from == 3 && to == 1) || (from == 1 && to == 0);
  if (!ref_pair) {
    switch (from) {
      case 0: return cast_from<uint8_t>(to, (const uint8_t*)x, out, n, blocks, st);
      case 1: return cast_from<float>(to, (const float*)x, out, n, blocks, st);
      case 2: return cast_from<int32_t>(to, (const int32_t*)x, out, n, blocks, st);
      case 3: return cast_from<int64_t>(to, (const int64_t*)x, out, n, blocks, st);
      default: return cudaErrorInvalidValue;
    }
  }
  // session.rs:1350-1378: i32->f32, i64->i32, i64->f32, f32->bool
  if (from == 2 && to == 1)
    cast_kernel<int32_t, float><<<blocks, 256, 0, st>>>((const int32_t*)x, (float*)out, n);
  else if (from == 3 && to == 2)
    cast_kernel<int64_t, int32_t><<<blocks, 256, 0, st>>>((const int64_t*)x, (int32_t*)out, n);
  else if (from == 3 && to == 1)
    cast_kernel<int64_t, float><<<blocks, 256, 0, st>>>((const int64_t*)x, (float*)out, n);
  else if (from == 1 && to == 0)
    cast_f32_bool_kernel<<<blocks, 256, 0, st>>>((const float*)x, (uint8_t*)out, n);
  else
    return cudaErrorInvalidValue;
  return cudaGetLastError();
}

cudaError_t launch_batch_norm(const float* x, const float* scale, const float* bias,
                              const float* mean, const float* var, float* out, int64_t n,
                              int64_t c, int64_t hw, float eps, cudaStream_t st) {
  const int64_t total = n * c * hw;
  if (total == 0) return cudaSuccess;
  batch_norm_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(x, scale, bias, mean, var,
                                                                    out, total, c, hw, eps);
  return cudaGetLastError();
}

}  // namespace ac
