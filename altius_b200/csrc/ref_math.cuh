// Device versions of the reference interpreter's scalar formulas. Every
// multiply/add that the reference rounds separately uses __fmul_rn/__fadd_rn
// (never contracted); every Rust `mul_add` is an explicit fmaf. With that, the
// per-element results are bit-identical to the CPU formulas.
#pragma once
#include <cuda_runtime.h>
#include <math_constants.h>

namespace ac {

__device__ __forceinline__ float clampf_rust(float x, float lo, float hi) {
  // f32::clamp: NaN stays NaN.
  if (x < lo) x = lo;
  if (x > hi) x = hi;
  return x;
}

// Rational tanh on an input already clamped to [-9, 9].
// crates/session_interpreter/src/fast_math.rs:336-350, session.rs:883-901
__device__ __forceinline__ float tanh_rational(float v) {
  const float s = __fmul_rn(v, v);
  float p = fmaf(s, -2.76076847742355e-16f, 2.00018790482477e-13f);
  p = fmaf(p, s, -8.60467152213735e-11f);
  p = fmaf(p, s, 5.12229709037114e-08f);
  p = fmaf(p, s, 1.48572235717979e-05f);
  p = fmaf(p, s, 6.37261928875436e-04f);
  p = fmaf(p, s, 4.89352455891786e-03f);
  p = __fmul_rn(p, v);
  float q = fmaf(s, 1.19825839466702e-06f, 1.18534705686654e-04f);
  q = fmaf(q, s, 2.26843463243900e-03f);
  q = fmaf(q, s, 4.89352518554385e-03f);
  return __fdiv_rn(p, q);
}

// crates/session_interpreter/src/fast_math.rs:332-353 `fast_gelu`
__device__ __forceinline__ float gelu_ref(float x) {
  const float B = 0.7978845608028654f;
  const float C = 0.035677408136300125f;
  float v = __fmul_rn(x, __fadd_rn(__fmul_rn(__fmul_rn(C, x), x), B));
  v = clampf_rust(v, -9.f, 9.f);
  const float t = tanh_rational(v);
  return __fmul_rn(__fadd_rn(t, 1.f), __fmul_rn(x, 0.5f));
}

// `gelu_ref` on two elements at a time with the packed fp32 instructions of
// sm_100 (one issue slot per pair). Every packed operation rounds each half
// exactly as its scalar counterpart. The quotient p / q uses the reciprocal
// estimate and two FMA refinements: for q in [4.8e-3, 1.5] (the range of the
// denominator polynomial) and |p| above 2^-40 that sequence returns the
// correctly rounded quotient; a smaller |p| gives |t| < 2^-30, which the
// following t + 1 rounds away, so the result equals `gelu_ref` bit for bit.
__device__ __forceinline__ float2 gelu_ref2(float2 x) {
  const float2 kB = make_float2(0.7978845608028654f, 0.7978845608028654f);
  const float2 kC = make_float2(0.035677408136300125f, 0.035677408136300125f);
  const float2 one = make_float2(1.f, 1.f), half = make_float2(0.5f, 0.5f);
#define AC_F2(c) make_float2(c, c)
  // The sum is written as fma(., 1, B): a packed multiply feeding a packed add was seen to be
  // contracted into one fused operation, which rounds differently from the reference.
  float2 v = __fmul2_rn(x, __ffma2_rn(__fmul2_rn(__fmul2_rn(kC, x), x), one, kB));
  v.x = clampf_rust(v.x, -9.f, 9.f);
  v.y = clampf_rust(v.y, -9.f, 9.f);
  const float2 s = __fmul2_rn(v, v);
  float2 p = __ffma2_rn(s, AC_F2(-2.76076847742355e-16f), AC_F2(2.00018790482477e-13f));
  p = __ffma2_rn(p, s, AC_F2(-8.60467152213735e-11f));
  p = __ffma2_rn(p, s, AC_F2(5.12229709037114e-08f));
  p = __ffma2_rn(p, s, AC_F2(1.48572235717979e-05f));
  p = __ffma2_rn(p, s, AC_F2(6.37261928875436e-04f));
  p = __ffma2_rn(p, s, AC_F2(4.89352455891786e-03f));
  p = __fmul2_rn(p, v);
  float2 q = __ffma2_rn(s, AC_F2(1.19825839466702e-06f), AC_F2(1.18534705686654e-04f));
  q = __ffma2_rn(q, s, AC_F2(2.26843463243900e-03f));
  q = __ffma2_rn(q, s, AC_F2(4.89352518554385e-03f));
#undef AC_F2
  float2 r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r.x) : "f"(q.x));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r.y) : "f"(q.y));
  const float2 nq = make_float2(-q.x, -q.y);
  const float2 e = __ffma2_rn(nq, r, one);
  r = __ffma2_rn(r, e, r);
  float2 t = __fmul2_rn(p, r);
  t = __ffma2_rn(__ffma2_rn(nq, t, p), r, t);
  t = __ffma2_rn(__ffma2_rn(nq, t, p), r, t);
  return __fmul2_rn(__fadd2_rn(t, one), __fmul2_rn(x, half));
}

// crates/session_interpreter/src/session.rs:840-903 `tanh`
__device__ __forceinline__ float tanh_ref(float x) { return tanh_rational(clampf_rust(x, -9.f, 9.f)); }

// The softmax exponential: crates/session_interpreter/src/fast_math.rs:160-183.
// `v` is x - rowmax.
__device__ __forceinline__ float exp_poly_softmax(float v) {
  v = fmaxf(v, -88.37626f);
  const float biased = fmaf(v, 1.44269504088896341f, 12582912.0f);
  const float m = __fsub_rn(biased, 12582912.0f);
  v = fmaf(m, -6.93145752e-1f, v);
  v = fmaf(m, -1.42860677e-6f, v);
  const unsigned normal = (__float_as_uint(biased) << 23) + 0x3F800000u;
  float p = 0.0013780593872f;
  p = fmaf(p, v, 0.0083731245250f);
  p = fmaf(p, v, 0.0416695363820f);
  p = fmaf(p, v, 0.1666647195816f);
  p = fmaf(p, v, 0.4999998509884f);
  p = fmaf(p, v, 1.0f);
  p = fmaf(p, v, 1.0f);
  return __fmul_rn(p, __uint_as_float(normal));
}

// crates/session_interpreter/src/fast_math.rs:250-278 `fast_sigmoid`
__device__ __forceinline__ float sigmoid_ref(float x) {
  float v = clampf_rust(-x, -103.9720840454f, 88.7762626647950f);
  const float biased = fmaf(v, 1.44269504088896341f, 12582912.0f);
  const float m = __fsub_rn(biased, 12582912.0f);
  v = fmaf(m, -6.93145752e-1f, v);
  v = fmaf(m, -1.42860677e-6f, v);
  int overflow = (int)(__float_as_uint(biased) << 23);
  int normal = min(overflow, 0x3F800000);
  normal = max(normal, -1056964608);
  overflow = (int)((unsigned)overflow - (unsigned)normal + 0x3F800000u);
  normal = (int)((unsigned)normal + 0x3F800000u);
  float p = 0.0013780593872f;
  p = fmaf(p, v, 0.0083731245250f);
  p = fmaf(p, v, 0.0416695363820f);
  p = fmaf(p, v, 0.1666647195816f);
  p = fmaf(p, v, 0.4999998509884f);
  p = fmaf(p, v, 1.0f);
  v = __fmul_rn(v, __int_as_float(overflow));
  p = fmaf(p, v, __int_as_float(overflow));
  p = __fmul_rn(p, __int_as_float(normal));
  return __fdiv_rn(1.f, __fadd_rn(1.f, p));
}

// crates/session_interpreter/src/session.rs:810: alpha.mul_add(x, beta).clamp(0, 1)
__device__ __forceinline__ float hard_sigmoid_ref(float x, float alpha, float beta) {
  return clampf_rust(fmaf(alpha, x, beta), 0.f, 1.f);
}

// Activation codes shared with the GEMM / conv epilogues (enum Act in kernels.h).
__device__ __forceinline__ float apply_act(int act, float v, float alpha, float beta) {
  switch (act) {
    case 1: return fmaxf(v, 0.f);
    case 2: return hard_sigmoid_ref(v, alpha, beta);
    case 3: return __fmul_rn(v, hard_sigmoid_ref(v, alpha, beta));
    case 4: return gelu_ref(v);
    default: return v;
  }
}

}  // namespace ac
