// CPU oracle: a restatement of the altius reference interpreter's kernels.
//
// THIS IS TEST INFRASTRUCTURE. Nothing in the shipped CUDA path may link, load
// or call it; it exists so the parity tests and the benchmark's CPU-baseline
// leg have the reference's arithmetic to compare against.
//
// Every function names the reference source it follows (paths are relative to
// the altius repository root). Operation order, the places where the
// reference uses a fused multiply-add (Rust `mul_add`) and the places where it
// does not are kept; this file must be compiled with -ffp-contract=off and
// without -ffast-math so the compiler adds or removes no roundings.
//
// Parity status:
//  * elementwise formulas (binary ops, ReLU, HardSigmoid, LeakyReLU, Gelu,
//    Sigmoid, Tanh, the softmax exponential, LayerNorm's per-element step,
//    MaxPool) are bit-for-bit restatements of scalar Rust code.
//  * reductions (`fast_sum`, `fast_sum_squares`, `fast_sum_exp`) keep the
//    reference's 8-lane partial sums; the horizontal order of
//    `Simd::reduce_sum` is fixed here as a pairwise tree
//    ((0+1)+(2+3))+((4+5)+(6+7)); the reference leaves it to the compiler.
//  * sgemm: the reference calls BLIS `cblas_sgemm` (blis-src 0.2.2 through
//    cblas-sys 0.1.4), which is not vendored; its summation order is
//    unspecified. `or_sgemm` is an own blocked kernel with a documented order.
//    PARITY UNPINNED for contraction results beyond the reference tests'
//    tolerances.
//  * Erf: the reference calls fastapprox 0.3.1 `faster::erf`, not vendored and
//    tested only to 1e-1. `or_erf` uses libm erff. PARITY UNPINNED.
//  * The reference repository holds no golden output files for these kernels:
//    its tests are differential against ONNX Runtime (absent here). The pins
//    that do exist (IEEE operator identity for Add/Sub/Mul/Div, broadcast
//    shape cases, the MNIST topological order snapshot, one Add known-answer
//    vector) are checked in tests/.

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

#define OR_API extern "C" __attribute__((visibility("default")))

namespace {

inline float fma32(float a, float b, float c) { return __builtin_fmaf(a, b, c); }

inline float bits_to_f32(int32_t v) {
  float f;
  std::memcpy(&f, &v, 4);
  return f;
}
inline int32_t f32_to_bits(float f) {
  int32_t v;
  std::memcpy(&v, &f, 4);
  return v;
}

// Rust f32::max / f32::min: if one operand is NaN the other is returned.
inline float rust_max(float a, float b) { return std::fmax(a, b); }
inline float rust_min(float a, float b) { return std::fmin(a, b); }
// Rust f32::clamp: NaN stays NaN; otherwise plain comparisons.
inline float rust_clamp(float x, float lo, float hi) {
  if (x < lo) x = lo;
  if (x > hi) x = hi;
  return x;
}

// Horizontal sum of the 8 partial lanes (see header: order fixed here).
inline float hsum8(const float* l) {
  return ((l[0] + l[1]) + (l[2] + l[3])) + ((l[4] + l[5]) + (l[6] + l[7]));
}

// crates/session_interpreter/src/session.rs:1028-1040 `fast_sum`
float fast_sum(const float* x, size_t n) {
  float lanes[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  size_t i = 0;
  for (; i + 8 <= n; i += 8)
    for (int l = 0; l < 8; ++l) lanes[l] += x[i + l];
  float tail = 0.f;
  for (; i < n; ++i) tail += x[i];
  return hsum8(lanes) + tail;
}

// crates/session_interpreter/src/session.rs:1042-1055 `fast_sum_squares`
float fast_sum_squares(const float* x, size_t n) {
  float lanes[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  size_t i = 0;
  for (; i + 8 <= n; i += 8)
    for (int l = 0; l < 8; ++l) lanes[l] += x[i + l] * x[i + l];
  float tail = 0.f;
  for (; i < n; ++i) tail += x[i] * x[i];
  return hsum8(lanes) + tail;
}

// crates/session_interpreter/src/fast_math.rs:160-183 (scalar tail; the SIMD
// body :129-156 performs the same operations lane-wise).
inline float exp_poly_softmax(float v) {
  const float LOWER_RANGE_2 = -88.37626f;
  const float ROUNDING_BIAS = 12582912.0f;
  const float LOG2RECIPROCAL = 1.44269504088896341f;
  const float LOG2HIGH = -6.93145752e-1f;
  const float LOG2LOW = -1.42860677e-6f;
  const float POLY_0 = 0.0013780593872f;
  const float POLY_1 = 0.0083731245250f;
  const float POLY_2 = 0.0416695363820f;
  const float POLY_3 = 0.1666647195816f;
  const float POLY_4 = 0.4999998509884f;
  const float POLY_56 = 1.0000000000000f;
  const int32_t MAXIMUM_EXPONENT = 0x3F800000;
  v = rust_max(v, LOWER_RANGE_2);
  float biased = fma32(v, LOG2RECIPROCAL, ROUNDING_BIAS);
  float m = biased - ROUNDING_BIAS;
  v = fma32(m, LOG2HIGH, v);
  v = fma32(m, LOG2LOW, v);
  int32_t normal = (int32_t)((uint32_t)f32_to_bits(biased) << 23);
  normal = (int32_t)((uint32_t)normal + (uint32_t)MAXIMUM_EXPONENT);
  float p = POLY_0;
  p = fma32(p, v, POLY_1);
  p = fma32(p, v, POLY_2);
  p = fma32(p, v, POLY_3);
  p = fma32(p, v, POLY_4);
  p = fma32(p, v, POLY_56);
  p = fma32(p, v, POLY_56);
  return p * bits_to_f32(normal);
}

// crates/session_interpreter/src/fast_math.rs:102-187 `fast_sum_exp`
float fast_sum_exp(float* out, const float* in, size_t n) {
  // :127  fold(NAN, |m, v| v.max(m)) -- NaN-ignoring maximum.
  float mx = std::numeric_limits<float>::quiet_NaN();
  for (size_t i = 0; i < n; ++i) mx = rust_max(in[i], mx);
  float lanes[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  size_t i = 0;
  for (; i + 8 <= n; i += 8)
    for (int l = 0; l < 8; ++l) {
      float p = exp_poly_softmax(in[i + l] - mx);
      lanes[l] += p;
      out[i + l] = p;
    }
  float sum = hsum8(lanes);
  for (; i < n; ++i) {
    float p = exp_poly_softmax(in[i] - mx);
    sum += p;
    out[i] = p;
  }
  return sum;
}

// crates/session_interpreter/src/fast_math.rs:250-278 (scalar form of
// `fast_sigmoid`; the SIMD body :213-248 is the same lane-wise).
inline float sigmoid_one(float x) {
  const float LOWER_RANGE = -103.9720840454f;
  const float UPPER_RANGE = 88.7762626647950f;
  const float ROUNDING_BIAS = 12582912.0f;
  const float LOG2RECIPROCAL = 1.44269504088896341f;
  const float LOG2HIGH = -6.93145752e-1f;
  const float LOG2LOW = -1.42860677e-6f;
  const float POLY_0 = 0.0013780593872f;
  const float POLY_1 = 0.0083731245250f;
  const float POLY_2 = 0.0416695363820f;
  const float POLY_3 = 0.1666647195816f;
  const float POLY_4 = 0.4999998509884f;
  const float POLY_56 = 1.0000000000000f;
  const int32_t MINIMUM_EXPONENT = -1056964608;
  const int32_t MAXIMUM_EXPONENT = 0x3F800000;
  float v = rust_clamp(-x, LOWER_RANGE, UPPER_RANGE);
  float biased = fma32(v, LOG2RECIPROCAL, ROUNDING_BIAS);
  float m = biased - ROUNDING_BIAS;
  v = fma32(m, LOG2HIGH, v);
  v = fma32(m, LOG2LOW, v);
  int32_t overflow = (int32_t)((uint32_t)f32_to_bits(biased) << 23);
  int32_t normal = std::min(overflow, MAXIMUM_EXPONENT);
  normal = std::max(normal, MINIMUM_EXPONENT);
  overflow = (int32_t)((uint32_t)overflow - (uint32_t)normal);
  overflow = (int32_t)((uint32_t)overflow + (uint32_t)MAXIMUM_EXPONENT);
  normal = (int32_t)((uint32_t)normal + (uint32_t)MAXIMUM_EXPONENT);
  float p = POLY_0;
  p = fma32(p, v, POLY_1);
  p = fma32(p, v, POLY_2);
  p = fma32(p, v, POLY_3);
  p = fma32(p, v, POLY_4);
  p = fma32(p, v, POLY_56);
  v = v * bits_to_f32(overflow);
  p = fma32(p, v, bits_to_f32(overflow));
  p = p * bits_to_f32(normal);
  return 1.f / (1.f + p);
}

// Rational tanh shared by Gelu and Tanh.
// crates/session_interpreter/src/fast_math.rs:336-350 and
// crates/session_interpreter/src/session.rs:883-901.
inline float tanh_rational_clamped(float val /* already clamped to [-9, 9] */) {
  const float ALPHA_13 = -2.76076847742355e-16f;
  const float ALPHA_11 = 2.00018790482477e-13f;
  const float ALPHA_9 = -8.60467152213735e-11f;
  const float ALPHA_7 = 5.12229709037114e-08f;
  const float ALPHA_5 = 1.48572235717979e-05f;
  const float ALPHA_3 = 6.37261928875436e-04f;
  const float ALPHA_1 = 4.89352455891786e-03f;
  const float BETA_6 = 1.19825839466702e-06f;
  const float BETA_4 = 1.18534705686654e-04f;
  const float BETA_2 = 2.26843463243900e-03f;
  const float BETA_0 = 4.89352518554385e-03f;
  float s = val * val;
  float p = fma32(s, ALPHA_13, ALPHA_11);
  p = fma32(p, s, ALPHA_9);
  p = fma32(p, s, ALPHA_7);
  p = fma32(p, s, ALPHA_5);
  p = fma32(p, s, ALPHA_3);
  p = fma32(p, s, ALPHA_1);
  p = p * val;
  float q = fma32(s, BETA_6, BETA_4);
  q = fma32(q, s, BETA_2);
  q = fma32(q, s, BETA_0);
  return p / q;
}

// crates/session_interpreter/src/fast_math.rs:332-353 `fast_gelu` (scalar form)
inline float gelu_one(float i) {
  const float B = 0.7978845608028654f;
  const float C = 0.035677408136300125f;
  float val = i * (C * i * i + B);  // separate mul, mul, add: no FMA here
  val = rust_clamp(val, -9.f, 9.f);
  float o = tanh_rational_clamped(val);
  return (o + 1.f) * (i * 0.5f);
}

int num_threads_or(int n) {
#ifdef _OPENMP
  return n > 0 ? n : omp_get_max_threads();
#else
  (void)n;
  return 1;
#endif
}

inline float bin(int op, float a, float b) {
  switch (op) {
    case 0: return a + b;
    case 1: return a - b;
    case 2: return a * b;
    default: return a / b;
  }
}

// crates/session_interpreter/src/session.rs:446-507: recursive stride walk.
void bin_general(int op, const int64_t* as, const int64_t* bs, const int64_t* os,
                 const int64_t* shape, int rank, const float* a, const float* b, float* o) {
  if (rank == 1) {
    const int64_t len = shape[0], sa = as[0], sb = bs[0];
    for (int64_t i = 0; i < len; ++i) o[i] = bin(op, a[i * sa], b[i * sb]);
    return;
  }
  for (int64_t i = 0; i < shape[0]; ++i)
    bin_general(op, as + 1, bs + 1, os + 1, shape + 1, rank - 1, a + i * as[0], b + i * bs[0],
                o + i * os[0]);
}

// crates/core/src/tensor.rs:369-406 `strides_for_broadcasting`
bool strides_for_broadcasting(const int64_t* from, int from_rank, const int64_t* to, int to_rank,
                              int64_t* out) {
  if (to_rank < from_rank) return false;
  std::vector<int64_t> st(from_rank);
  for (int i = 0; i < from_rank; ++i) {
    int64_t s = 1;
    for (int j = i + 1; j < from_rank; ++j) s *= from[j];
    st[i] = s;
  }
  for (int i = 0; i < to_rank; ++i) out[i] = 0;
  for (int i = 0; i < from_rank; ++i) {
    const int fi = from_rank - 1 - i, ti = to_rank - 1 - i;
    if (to[ti] == from[fi]) out[ti] = st[fi];
    else if (from[fi] == 1) out[ti] = 0;
    else return false;
  }
  return true;
}

bool dims_equal(const int64_t* a, int ar, const int64_t* b, int br) {
  if (ar != br) return false;
  for (int i = 0; i < ar; ++i)
    if (a[i] != b[i]) return false;
  return true;
}
// crates/core/src/fixed_dim.rs:26-28 `is_scalar`
bool is_scalar(const int64_t* d, int r) { return r == 0 || (r == 1 && (d[0] == 0 || d[0] == 1)); }
int64_t numel(const int64_t* d, int r) {
  int64_t n = 1;
  for (int i = 0; i < r; ++i) n *= d[i];
  return n;
}

}  // namespace

// ---------------------------------------------------------------------------
// Binary elementwise with NumPy broadcasting.
// crates/session_interpreter/src/session.rs:384-526 `op_bin_elemwise!`
// op: 0 Add, 1 Sub, 2 Mul, 3 Div. Returns 0, or -1 when shapes do not broadcast.
OR_API int or_binary(int op, const float* a, const int64_t* adims, int arank, const float* b,
                     const int64_t* bdims, int brank, float* out, const int64_t* odims, int orank,
                     int threads) {
  const int64_t n = numel(odims, orank);
  if (dims_equal(adims, arank, bdims, brank)) {
    // :394-418 equal dims: 100000-element chunks, one task per chunk.
    const int64_t chunk = 100000;
    const int64_t nchunks = (n + chunk - 1) / chunk;
#pragma omp parallel for num_threads(num_threads_or(threads)) schedule(dynamic)
    for (int64_t c = 0; c < nchunks; ++c) {
      const int64_t lo = c * chunk, hi = std::min(n, lo + chunk);
      switch (op) {
        case 0: for (int64_t i = lo; i < hi; ++i) out[i] = a[i] + b[i]; break;
        case 1: for (int64_t i = lo; i < hi; ++i) out[i] = a[i] - b[i]; break;
        case 2: for (int64_t i = lo; i < hi; ++i) out[i] = a[i] * b[i]; break;
        default: for (int64_t i = lo; i < hi; ++i) out[i] = a[i] / b[i]; break;
      }
    }
    return 0;
  }
  if (is_scalar(bdims, brank)) {  // :420-429, single thread
    const float s = b[0];
    for (int64_t i = 0; i < n; ++i) out[i] = bin(op, a[i], s);
    return 0;
  }
  if (is_scalar(adims, arank)) {  // :431-440, single thread
    const float s = a[0];
    for (int64_t i = 0; i < n; ++i) out[i] = bin(op, s, b[i]);
    return 0;
  }
  // :445-524 general path, single thread. (`assert!(o_shape.len() > 1)` :521)
  if (orank < 1 || orank > 16) return -1;
  int64_t as[16], bs[16], os[16];
  if (!strides_for_broadcasting(adims, arank, odims, orank, as)) return -1;
  if (!strides_for_broadcasting(bdims, brank, odims, orank, bs)) return -1;
  for (int i = 0; i < orank; ++i) {
    int64_t s = 1;
    for (int j = i + 1; j < orank; ++j) s *= odims[j];
    os[i] = s;
  }
  bin_general(op, as, bs, os, odims, orank, a, b, out);
  return 0;
}

// crates/session_interpreter/src/session.rs:566-606 `compute_pow`
// mode 0: same shape; mode 1: scalar exponent (b[0]).
OR_API int or_pow(const float* a, const float* b, float* out, int64_t n, int mode) {
  if (mode == 0) {
    for (int64_t i = 0; i < n; ++i) out[i] = std::pow(a[i], b[i]);
  } else {
    const float e = b[0];
    if (e == 2.f) {
      for (int64_t i = 0; i < n; ++i) out[i] = a[i] * a[i];
    } else {
      for (int64_t i = 0; i < n; ++i) out[i] = std::pow(a[i], e);
    }
  }
  return 0;
}

// crates/session_interpreter/src/session.rs:608-619 `compute_sqrt`
OR_API void or_sqrt(const float* x, float* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = std::sqrt(x[i]);
}

// crates/session_interpreter/src/session.rs:796-803 `compute_relu`: x.max(0.0)
OR_API void or_relu(const float* x, float* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = rust_max(x[i], 0.0f);
}

// crates/session_interpreter/src/session.rs:805-812 `compute_hard_sigmoid`
OR_API void or_hard_sigmoid(const float* x, float* out, int64_t n, float alpha, float beta) {
  for (int64_t i = 0; i < n; ++i) out[i] = rust_clamp(fma32(alpha, x[i], beta), 0.f, 1.f);
}

// crates/session_interpreter/src/session.rs:814-821 `compute_leaky_relu`
OR_API void or_leaky_relu(const float* x, float* out, int64_t n, float alpha) {
  for (int64_t i = 0; i < n; ++i) out[i] = x[i] < 0.f ? alpha * x[i] : x[i];
}

// crates/session_interpreter/src/session.rs:823-838 `compute_gelu` (len/threads
// chunks, each through fast_gelu). The formula is per element, so chunking
// does not change results.
OR_API void or_gelu(const float* x, float* out, int64_t n, int threads) {
#pragma omp parallel for num_threads(num_threads_or(threads)) schedule(static)
  for (int64_t i = 0; i < n; ++i) out[i] = gelu_one(x[i]);
}

// crates/session_interpreter/src/session.rs:905-922 `compute_sigmoid`
OR_API void or_sigmoid(const float* x, float* out, int64_t n, int threads) {
  const int t = num_threads_or(threads);
  if (n / t > 512) {
#pragma omp parallel for num_threads(t) schedule(static)
    for (int64_t i = 0; i < n; ++i) out[i] = sigmoid_one(x[i]);
  } else {
    for (int64_t i = 0; i < n; ++i) out[i] = sigmoid_one(x[i]);
  }
}

// crates/session_interpreter/src/session.rs:924-931 `compute_erf`. The
// reference's arithmetic is in an un-vendored crate (see header): libm here.
OR_API void or_erf(const float* x, float* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = std::erf(x[i]);
}

// crates/session_interpreter/src/session.rs:933-938 + :840-903 `tanh`
OR_API void or_tanh(const float* x, float* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = tanh_rational_clamped(rust_clamp(x[i], -9.f, 9.f));
}

// crates/session_interpreter/src/session.rs:542-557 `compute_greater` (scalar rhs)
OR_API void or_greater_scalar(const float* x, float y, uint8_t* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = x[i] > y ? 1 : 0;
}

// crates/session_interpreter/src/session.rs:940-988 `compute_where`
// mode 0: cond and y same shape, x scalar. mode 1: x is [o0,o1,o2,o3], cond
// has o2*o3 elements (leading dims 1,1), y scalar.
OR_API void or_where(int mode, const uint8_t* cond, const float* x, const float* y, float* out,
                     int64_t n, int64_t inner) {
  if (mode == 0) {
    const float xs = x[0];
    for (int64_t i = 0; i < n; ++i) out[i] = cond[i] ? xs : y[i];
  } else {
    const float ys = y[0];
    for (int64_t i = 0; i < n; ++i) out[i] = cond[i % inner] ? x[i] : ys;
  }
}

// crates/session_interpreter/src/session.rs:990-1026 `compute_softmax`
// (last axis; row batches spread over threads; out = e * (1/sum)).
OR_API void or_softmax(const float* x, float* out, int64_t rows, int64_t axis_len, int threads) {
#pragma omp parallel for num_threads(num_threads_or(threads)) schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    float* o = out + r * axis_len;
    const float sum = fast_sum_exp(o, x + r * axis_len, (size_t)axis_len);
    const float recip = 1.f / sum;
    for (int64_t i = 0; i < axis_len; ++i) o[i] *= recip;
  }
}

// crates/session_interpreter/src/session.rs:1433-1486 `compute_layer_normalization`
OR_API void or_layer_norm(const float* x, const float* scale, const float* bias, float* out,
                          int64_t rows, int64_t axis_len, float eps, int threads) {
#pragma omp parallel for num_threads(num_threads_or(threads)) schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const float* in = x + r * axis_len;
    float* o = out + r * axis_len;
    const float inv_axis_len = 1.f / (float)axis_len;                      // :1468
    const float mean = fast_sum(in, (size_t)axis_len) * inv_axis_len;      // :1469
    for (int64_t i = 0; i < axis_len; ++i) o[i] = in[i] - mean;            // :1470-1472
    const float var = fma32(fast_sum_squares(o, (size_t)axis_len), inv_axis_len, eps);  // :1473-1474
    const float inv_mean = 1.f / std::sqrt(var);                           // :1475-1476
    for (int64_t i = 0; i < axis_len; ++i) o[i] = fma32(o[i] * inv_mean, scale[i], bias[i]);  // :1480
  }
}

// crates/session_interpreter/src/session.rs:1307-1340 `compute_reduce_mean`
// (rank 3, axis 2, keepdims; single thread)
OR_API void or_reduce_mean_last(const float* x, float* out, int64_t rows, int64_t axis_len) {
  const float r = 1.0f / (float)axis_len;
  for (int64_t i = 0; i < rows; ++i) out[i] = fast_sum(x + i * axis_len, (size_t)axis_len) * r;
}

// crates/session_interpreter/src/session.rs:1292-1305 `compute_reduce_max`
// (all axes, keepdims = 0 -> one scalar; max_by(partial_cmp) keeps the last of
// equal maxima, which is the same value).
OR_API void or_reduce_max_all(const float* x, float* out, int64_t n) {
  float m = x[0];
  for (int64_t i = 1; i < n; ++i)
    if (!(x[i] < m)) m = x[i];
  out[0] = m;
}

// EXTENSION (not in the reference, which asserts all-axes): ReduceMax over the
// last axis, per the ONNX operator definition. Parity is defined by ONNX
// semantics and is not pinned by the reference.
OR_API void or_reduce_max_last(const float* x, float* out, int64_t rows, int64_t axis_len) {
  for (int64_t r = 0; r < rows; ++r) {
    const float* p = x + r * axis_len;
    float m = p[0];
    for (int64_t i = 1; i < axis_len; ++i)
      if (!(p[i] < m)) m = p[i];
    out[r] = m;
  }
}

// crates/session_interpreter/src/session.rs:265-297 `compute_gavg_pool`
// (sequential left-to-right sum, then division by the area as f32)
OR_API void or_gavg_pool(const float* x, float* out, int64_t nc, int64_t hw) {
  for (int64_t i = 0; i < nc; ++i) {
    float sum = 0.f;
    const float* p = x + i * hw;
    for (int64_t j = 0; j < hw; ++j) sum += p[j];
    out[i] = sum / (float)hw;
  }
}

// compute_resize, crates/session_interpreter/src/session.rs:1057-1132: one scale
// (output_h / input_h) for both axes; "nearest" truncates dst / scale, anything else is the
// bilinear blend around max(dst / scale - 0.5, 0). The reference indexes without clamping in
// the nearest branch (it panics when the aspect ratio changes); indices are clamped here.
OR_API void or_resize(const float* x, float* out, int64_t outer, int64_t ih, int64_t iw, int64_t oh, int64_t ow,
                      int mode) {
  const float scale = (float)oh / (float)ih;
#pragma omp parallel for
  for (int64_t p = 0; p < outer; ++p) {
    const float* in = x + p * ih * iw;
    float* o = out + p * oh * ow;
    for (int64_t h = 0; h < oh; ++h) {
      for (int64_t w = 0; w < ow; ++w) {
        if (mode == 0) {
          const int64_t sy = std::min<int64_t>((int64_t)((float)h / scale), ih - 1);
          const int64_t sx = std::min<int64_t>((int64_t)((float)w / scale), iw - 1);
          o[h * ow + w] = in[sy * iw + sx];
        } else {
          const float yf = std::max((float)h / scale - 0.5f, 0.f);
          const float xf = std::max((float)w / scale - 0.5f, 0.f);
          const int64_t y = (int64_t)yf, xx = (int64_t)xf;
          const int64_t y0 = std::min(y, ih - 1), y1 = std::min(y + 1, ih - 1);
          const int64_t x0 = std::min(xx, iw - 1), x1 = std::min(xx + 1, iw - 1);
          const float v00 = in[y0 * iw + x0], v01 = in[y0 * iw + x1];
          const float v10 = in[y1 * iw + x0], v11 = in[y1 * iw + x1];
          const float hd = v00 + (v10 - v00) * (yf - (float)y);
          const float hw = v01 + (v11 - v01) * (yf - (float)y);
          o[h * ow + w] = hd + (hw - hd) * (xf - (float)xx);
        }
      }
    }
  }
}

// crates/session_interpreter/src/session.rs:325-382 `compute_max_pool`
OR_API void or_max_pool(const float* x, float* out, int64_t outer, int64_t ih, int64_t iw,
                        int64_t oh, int64_t ow, int64_t kh, int64_t kw, int64_t sh, int64_t sw,
                        int64_t pad_t, int64_t pad_l) {
  const float FMIN = std::numeric_limits<float>::lowest();  // f32::MIN
  for (int64_t o = 0; o < outer; ++o) {
    const float* in = x + o * ih * iw;
    float* ot = out + o * oh * ow;
    int64_t y = -pad_t;
    for (int64_t ay = 0; ay < oh; ++ay) {
      int64_t xx = -pad_l;
      const int64_t fy_min = std::max<int64_t>(-y, 0);
      const int64_t fy_max = std::min<int64_t>(kh, ih - y);
      for (int64_t ax = 0; ax < ow; ++ax) {
        float mx = FMIN;
        const int64_t fx_min = std::max<int64_t>(-xx, 0);
        const int64_t fx_max = std::min<int64_t>(kw, iw - xx);
        for (int64_t fy = fy_min; fy < fy_max; ++fy)
          for (int64_t fx = fx_min; fx < fx_max; ++fx)
            mx = rust_max(in[(y + fy) * iw + (xx + fx)], mx);
        ot[ay * ow + ax] = (mx == FMIN) ? 0.0f : mx;  // :374
        xx += sw;
      }
      y += sh;
    }
  }
}

// crates/session_interpreter/src/session.rs:1380-1431 `compute_batch_normalization`
OR_API void or_batch_norm(const float* x, const float* scale, const float* bias, const float* mean,
                          const float* var, float* out, int64_t n, int64_t c, int64_t hw,
                          float eps) {
  for (int64_t i = 0; i < n; ++i)
    for (int64_t ch = 0; ch < c; ++ch) {
      const int64_t off = (i * c + ch) * hw;
      for (int64_t j = 0; j < hw; ++j)
        out[off + j] = ((x[off + j] - mean[ch]) / std::sqrt(var[ch] + eps)) * scale[ch] + bias[ch];
    }
}

// ---------------------------------------------------------------------------
// sgemm. The reference calls cblas_sgemm (BLIS), crates/session_interpreter/
// src/gemm.rs:36-51 and :95-110. Own kernel, documented order: for every
// C[i][j] the products a[i][k]*b[k][j] are accumulated with FMA in ascending k
// into a zero-initialised accumulator per K-panel of 256; panels are added to
// C in ascending order; the first panel computes C = beta*C + alpha*acc, later
// ones C += alpha*acc.
namespace {
constexpr int KC = 256, MR = 6, NR = 32;

void sgemm_impl(bool ta, bool tb, int64_t M, int64_t K, int64_t N, float alpha, const float* A,
                int64_t lda, const float* B, int64_t ldb, float beta, float* C, int64_t ldc,
                int threads) {
  if (M <= 0 || N <= 0) return;
  if (K <= 0) {
    for (int64_t i = 0; i < M; ++i)
      for (int64_t j = 0; j < N; ++j) C[i * ldc + j] = beta * C[i * ldc + j];
    return;
  }
  const int64_t mblocks = (M + MR - 1) / MR;
#pragma omp parallel num_threads(num_threads_or(threads))
  {
    std::vector<float> bpack((size_t)KC * NR);
    std::vector<float> apack((size_t)KC * MR);
    // Threads split the N panels when M is small, else the M blocks.
    const int64_t nblocks = (N + NR - 1) / NR;
#pragma omp for collapse(2) schedule(static)
    for (int64_t jb = 0; jb < nblocks; ++jb)
      for (int64_t ibg = 0; ibg < (mblocks + 15) / 16; ++ibg) {
        const int64_t j0 = jb * NR, nr = std::min<int64_t>(NR, N - j0);
        for (int64_t k0 = 0; k0 < K; k0 += KC) {
          const int64_t kc = std::min<int64_t>(KC, K - k0);
          for (int64_t k = 0; k < kc; ++k) {
            float* bp = &bpack[(size_t)k * NR];
            for (int64_t j = 0; j < nr; ++j)
              bp[j] = tb ? B[(j0 + j) * ldb + (k0 + k)] : B[(k0 + k) * ldb + (j0 + j)];
            for (int64_t j = nr; j < NR; ++j) bp[j] = 0.f;
          }
          for (int64_t ib = ibg * 16; ib < std::min(mblocks, ibg * 16 + 16); ++ib) {
            const int64_t i0 = ib * MR, mr = std::min<int64_t>(MR, M - i0);
            for (int64_t k = 0; k < kc; ++k)
              for (int64_t i = 0; i < MR; ++i)
                apack[(size_t)k * MR + i] =
                    i < mr ? (ta ? A[(k0 + k) * lda + (i0 + i)] : A[(i0 + i) * lda + (k0 + k)])
                           : 0.f;
            float acc[MR][NR];
            for (int i = 0; i < MR; ++i)
              for (int j = 0; j < NR; ++j) acc[i][j] = 0.f;
            for (int64_t k = 0; k < kc; ++k) {
              const float* bp = &bpack[(size_t)k * NR];
              const float* ap = &apack[(size_t)k * MR];
              for (int i = 0; i < MR; ++i) {
                const float av = ap[i];
#pragma omp simd
                for (int j = 0; j < NR; ++j) acc[i][j] = fma32(av, bp[j], acc[i][j]);
              }
            }
            for (int64_t i = 0; i < mr; ++i)
              for (int64_t j = 0; j < nr; ++j) {
                float* c = &C[(i0 + i) * ldc + (j0 + j)];
                if (k0 == 0) *c = (beta == 0.f ? 0.f : beta * *c) + alpha * acc[i][j];
                else *c = *c + alpha * acc[i][j];
              }
          }
        }
      }
  }
}
}  // namespace

OR_API void or_sgemm(int trans_a, int trans_b, int64_t m, int64_t k, int64_t n, float alpha,
                     const float* a, int64_t lda, const float* b, int64_t ldb, float beta,
                     float* c, int64_t ldc, int threads) {
  sgemm_impl(trans_a != 0, trans_b != 0, m, k, n, alpha, a, lda, b, ldb, beta, c, ldc, threads);
}

// Batched loop of sgemm, as crates/session_interpreter/src/session.rs:641-672
// does for 3-D x 3-D and 4-D x 4-D MatMul (sequential over batches there; the
// batches are spread over threads here only when `threads` != 1, results are
// identical because each batch is independent).
OR_API void or_sgemm_batched(int64_t batch, int64_t m, int64_t k, int64_t n, const float* a,
                             const float* b, float* c, int threads) {
#pragma omp parallel for num_threads(num_threads_or(threads)) schedule(static)
  for (int64_t i = 0; i < batch; ++i)
    sgemm_impl(false, false, m, k, n, 1.f, a + i * m * k, k, b + i * k * n, n, 0.f, c + i * m * n,
               n, 1);
}

// ---------------------------------------------------------------------------
// Conv2d = bias pre-fill + im2col + per-(batch, group) sgemm with beta = 1.
// crates/session_interpreter/src/conv2d.rs:26-210, im2col :213-332.
// The reference offsets each im2col output row by `oh * output_h` (:232,
// :296); that equals `oh * output_w` for square outputs, the only case the
// reference tests. This restatement uses `oh * output_w`.
namespace {
void im2col_plane(int64_t ih_, int64_t iw_, int64_t oh_, int64_t ow_, int64_t sh, int64_t sw,
                  int64_t dh, int64_t dw, int64_t pad_t, int64_t pad_l, int64_t kh, int64_t kw,
                  const float* in, float* col) {
  const int64_t ohw = oh_ * ow_;
  for (int64_t fy = 0; fy < kh; ++fy)
    for (int64_t fx = 0; fx < kw; ++fx) {
      for (int64_t oh = 0; oh < oh_; ++oh) {
        float* c = col + oh * ow_;
        const int64_t ih = fy * dh + oh * sh;
        if (pad_t > ih || ih >= ih_ + pad_t) {
          for (int64_t i = 0; i < ow_; ++i) c[i] = 0.f;
          continue;
        }
        const int64_t base = (ih - pad_t) * iw_;
        for (int64_t ow = 0; ow < ow_; ++ow) {
          const int64_t iw = fx * dw + ow * sw;
          c[ow] = (iw < pad_l || iw >= iw_ + pad_l) ? 0.f : in[base + iw - pad_l];
        }
      }
      col += ohw;
    }
}
}  // namespace

OR_API void or_conv2d(const float* x, const float* w, const float* bias /* may be null */,
                      float* out, int64_t n, int64_t c, int64_t ih, int64_t iw, int64_t oc,
                      int64_t oh, int64_t ow, int64_t kh, int64_t kw, int64_t sh, int64_t sw,
                      int64_t dh, int64_t dw, int64_t pad_t, int64_t pad_l, int64_t group,
                      int threads) {
  const int64_t ohw = oh * ow, ihw = ih * iw;
  const int64_t icg = c / group, ocg = oc / group;
  // conv2d.rs:62-79 bias pre-fill (or zeros)
  for (int64_t b = 0; b < n; ++b)
    for (int64_t o = 0; o < oc; ++o) {
      const float v = bias ? bias[o] : 0.f;
      float* p = out + (b * oc + o) * ohw;
      for (int64_t i = 0; i < ohw; ++i) p[i] = v;
    }
  // conv2d.rs:81-143 im2col into col[n, c, kh, kw, oh, ow]
  std::vector<float> col((size_t)n * c * kh * kw * ohw);
#pragma omp parallel for num_threads(num_threads_or(threads)) schedule(static)
  for (int64_t p = 0; p < n * c; ++p)
    im2col_plane(ih, iw, oh, ow, sh, sw, dh, dw, pad_t, pad_l, kh, kw, x + p * ihw,
                 col.data() + (size_t)p * kh * kw * ohw);
  // conv2d.rs:145-209: one sgemm (ocg x k) * (k x ohw) per (batch, group), beta = 1
  const int64_t k = icg * kh * kw;
  if (group == 1) {
    for (int64_t b = 0; b < n; ++b)
      sgemm_impl(false, false, ocg, k, ohw, 1.f, w, k, col.data() + (size_t)b * k * ohw, ohw, 1.f,
                 out + b * oc * ohw, ohw, threads);
  } else {
#pragma omp parallel for num_threads(num_threads_or(threads)) schedule(static)
    for (int64_t bg = 0; bg < n * group; ++bg) {
      const int64_t g = bg % group;
      sgemm_impl(false, false, ocg, k, ohw, 1.f, w + g * ocg * k, k,
                 col.data() + (size_t)bg * k * ohw, ohw, 1.f, out + bg * ocg * ohw, ohw, 1);
    }
  }
}

// crates/session_interpreter/src/session.rs:1179-1278 `compute_transpose`
// (generic permutation of an f32 tensor; pure copy).
OR_API void or_transpose(const float* x, float* out, const int64_t* in_dims, const int64_t* perm,
                         int rank) {
  int64_t in_strides[16], out_dims[16], src_strides[16];
  for (int i = 0; i < rank; ++i) {
    int64_t s = 1;
    for (int j = i + 1; j < rank; ++j) s *= in_dims[j];
    in_strides[i] = s;
  }
  int64_t total = 1;
  for (int i = 0; i < rank; ++i) {
    out_dims[i] = in_dims[perm[i]];
    src_strides[i] = in_strides[perm[i]];
    total *= out_dims[i];
  }
  int64_t idx[16] = {0};
  int64_t src = 0;
  for (int64_t o = 0; o < total; ++o) {
    out[o] = x[src];
    for (int d = rank - 1; d >= 0; --d) {
      src += src_strides[d];
      if (++idx[d] < out_dims[d]) break;
      src -= src_strides[d] * idx[d];
      idx[d] = 0;
    }
  }
}

OR_API int or_max_threads() { return num_threads_or(0); }
