// Launchers of the sm_100a kernels. Host code (the scheduler) sees only these
// declarations; each launcher enqueues on the given stream and returns the
// CUDA status of the launch.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace ac {

constexpr int kMaxRank = 8;

// Raises a kernel's dynamic shared-memory limit once per device (the attribute belongs to
// the device the call is made on; sessions on several devices may share one process).
// `done` is the caller's per-kernel record, one bit per device ordinal.
template <typename Kernel>
cudaError_t ensure_dynamic_smem(Kernel kernel, int bytes, unsigned long long* done) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  const unsigned long long bit = 1ull << (dev & 63);
  if (*done & bit) return cudaSuccess;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess) *done |= bit;
  return e;
}

// Number of SMs of the current device (grids are sized in multiples of it); cached per
// device ordinal. Falls back to 148 (B200) when the attribute cannot be read.
inline int device_sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) { (void)cudaGetLastError(); return 148; }
  int& n = cached[dev & 63];
  if (n <= 0 && (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)) {
    (void)cudaGetLastError();
    n = 148;
  }
  return n;
}

// ---- elementwise -----------------------------------------------------------
enum BinOp { BIN_ADD = 0, BIN_SUB, BIN_MUL, BIN_DIV, BIN_POW };

// Broadcast binary op over a collapsed iteration space: dims[rank-1] is the
// innermost extent; a_str / b_str are element strides (0 = broadcast).
struct BinaryParams {
  int op;
  int rank;
  int64_t dims[kMaxRank];
  int64_t a_str[kMaxRank];
  int64_t b_str[kMaxRank];
  int64_t n;  // total output elements
};
cudaError_t launch_binary(const BinaryParams& p, const float* a, const float* b, float* out,
                          cudaStream_t st);

enum UnaryOp {
  UN_RELU = 0, UN_SIGMOID, UN_ERF, UN_GELU, UN_HARDSIGMOID, UN_LEAKYRELU, UN_SQRT, UN_TANH,
  UN_HARDSWISH,  // x * HardSigmoid(x; alpha, beta): the HardSigmoid -> Mul pair folded
  UN_SQUARE,     // Pow(x, 2) special case of the reference: x * x
  UN_COPY
};
cudaError_t launch_unary(int op, float alpha, float beta, const float* x, float* out, int64_t n,
                         cudaStream_t st);
cudaError_t launch_greater_scalar(const float* x, const float* y_scalar, uint8_t* out, int64_t n,
                                  cudaStream_t st);
// mode 0: out = cond ? x[0] : y[i]; mode 1: out = cond[i % inner] ? x[i] : y[0]
cudaError_t launch_where(int mode, const uint8_t* cond, const float* x, const float* y, float* out,
                         int64_t n, int64_t inner, cudaStream_t st);
// NumPy-broadcast Greater and Where over a collapsed iteration space (as BinaryParams: dims and
// element strides per operand, 0 = broadcast): the general forms beyond the two patterns of
// the reference (ONNX semantics; comparisons and selections are exact).
struct TernaryParams {
  int rank;
  int64_t dims[kMaxRank];
  int64_t c_str[kMaxRank];
  int64_t x_str[kMaxRank];
  int64_t y_str[kMaxRank];
  int64_t n;
};
cudaError_t launch_greater_bcast(const TernaryParams& p, const float* x, const float* y, uint8_t* out, cudaStream_t st);
cudaError_t launch_where_bcast(const TernaryParams& p, const uint8_t* cond, const float* x, const float* y, float* out,
                               cudaStream_t st);
// from/to: 0 bool, 1 f32, 2 i32, 3 i64. Every pair (C conversion rules; to bool: x != 0).
cudaError_t launch_cast(int from, int to, const void* x, void* out, int64_t n, cudaStream_t st);
cudaError_t launch_batch_norm(const float* x, const float* scale, const float* bias,
                              const float* mean, const float* var, float* out, int64_t n,
                              int64_t c, int64_t hw, float eps, cudaStream_t st);

// ---- row kernels (reductions over the last axis) ----------------------------
// Softmax(x * scale) with the reference's polynomial exponential. `scale_mode`
// 0: none, 1: multiply by *scale, 2: divide by *scale (scalar read on device).
// With `mask` (bool, mask_rows x len, repeated over the rows) the scaled value is replaced by
// *mask_else where the mask is false before the softmax: the Where(mask, x, c) of a masked
// attention folded in (crates/session_interpreter/src/session.rs:958-987 computes that Where).
cudaError_t launch_softmax(const float* x, float* out, int64_t rows, int64_t len, int scale_mode,
                           const float* scale, const uint8_t* mask, int64_t mask_rows, const float* mask_else,
                           cudaStream_t st);

// v = x; if (pre_bias) v += pre_bias[col]; if (gelu) v = Gelu(v);
// if (residual) v = residual_first ? residual + v : v + residual;
// if (sum_out) sum_out = v;  out = LayerNorm(v) * gamma + beta.
struct LayerNormParams {
  const float* x;
  const float* pre_bias;   // [len] or null
  const float* residual;   // [rows, len] or null
  const float* gamma;
  const float* beta;
  float* sum_out;          // [rows, len] or null
  float* out;              // may be null when out16_hi / out16_lo are given
  void* out16_hi;          // the result split for the fp16-split GEMM that consumes it: [rows, len]
  void* out16_lo;          // halves each on the fixed scale: Y = y * 2^8, hi = rn_fp16(Y), lo = rn_fp16(Y - hi); or null
  int* err_word;           // receives kGemmRangeCode when the result does not fit that split
  int64_t rows;
  int64_t len;
  float eps;
  int gelu;
  int residual_first;
};
cudaError_t launch_layer_norm(const LayerNormParams& p, cudaStream_t st);

cudaError_t launch_reduce_mean_last(const float* x, float* out, int64_t rows, int64_t len,
                                    cudaStream_t st);
cudaError_t launch_reduce_max_last(const float* x, float* out, int64_t rows, int64_t len,
                                   cudaStream_t st);
// Both reductions of the same rows in one pass (sibling ReduceMean / ReduceMax nodes).
cudaError_t launch_reduce_mean_max_last(const float* x, float* mean_out, float* max_out, int64_t rows, int64_t len,
                                        cudaStream_t st);
// Whole-tensor maximum; `partials` is scratch of reduce_max_all_scratch_elems(n) floats.
int64_t reduce_max_all_scratch_elems(int64_t n);
cudaError_t launch_reduce_max_all(const float* x, float* out, int64_t n, float* partials,
                                  cudaStream_t st);
// out[i] = sum(x[i, 0:hw]) / hw
cudaError_t launch_gavg_pool(const float* x, float* out, int64_t planes, int64_t hw,
                             cudaStream_t st);

// ---- data movement ----------------------------------------------------------
cudaError_t launch_max_pool(const float* x, float* out, int64_t planes, int ih, int iw, int oh,
                            int ow, int kh, int kw, int sh, int sw, int pad_t, int pad_l,
                            cudaStream_t st);
// Generic strided gather: out (contiguous, dims[rank]) <- in at sum(idx[d] * in_str[d]) + in_off.
// Serves Transpose, Slice, Split, Gather, Concat pieces. elem_bytes 1, 4 or 8.
struct CopyParams {
  int rank;
  int64_t dims[kMaxRank];
  int64_t in_str[kMaxRank];
  int64_t out_str[kMaxRank];
  int64_t in_off;
  int64_t out_off;
  int64_t n;
  int elem_bytes;
};
cudaError_t launch_strided_copy(const CopyParams& p, const void* in, void* out, cudaStream_t st);
// Batched 2-D transpose: in [batch, r, c] -> out [batch, c, r] (f32).
cudaError_t launch_transpose2d(const float* in, float* out, int64_t batch, int r, int c,
                               cudaStream_t st);

// Resize of [planes, ih, iw] -> [planes, oh, ow] as the interpreter does it
// (crates/session_interpreter/src/session.rs:1057-1132): one scale oh / ih for both
// axes; mode 0 nearest (source index = trunc(dst / scale)), else bilinear around
// max(dst / scale - 0.5, 0). Source indices are clamped to the input.
cudaError_t launch_resize(const float* x, float* out, int64_t planes, int ih, int iw, int oh, int ow, int mode,
                          cudaStream_t st);

// ---- convolution ------------------------------------------------------------
enum Act { ACT_NONE = 0, ACT_RELU, ACT_HARDSIGMOID, ACT_HARDSWISH, ACT_GELU };
struct ConvParams {
  int n, c, ih, iw, oc, oh, ow, kh, kw, sh, sw, dh, dw, pad_t, pad_l, group;
  int act;
  float act_alpha, act_beta;
};
// col[n, c, kh, kw, oh, ow] <- x[n, c, ih, iw]
cudaError_t launch_im2col(const ConvParams& p, const float* x, float* col, cudaStream_t st);
// Non-overlapping patches (kernel == stride, no padding): rows[n * oh * ow, c * kh * kw] <- x,
// one row per patch with the (c, fy, fx) order of the weight's K axis. kw % 4 == 0.
cudaError_t launch_patchify(const ConvParams& p, const float* x, float* rows, cudaStream_t st);
// Depthwise (group == c == oc) stencil with bias and activation fused.
cudaError_t launch_depthwise_conv(const ConvParams& p, const float* x, const float* w,
                                  const float* bias, float* out, cudaStream_t st);

// ---- GEMM -------------------------------------------------------------------
// C[b] = act(alpha * op(A[b]) * op(B[b]) + beta * Cin[b] + bias) (+ residual)
// Row-major operands; trans_a: A stored [K, M]; trans_b: B stored [N, K].
struct GemmParams {
  int64_t m, n, k;
  int64_t batch;
  const float* a; int64_t lda; int64_t stride_a; int trans_a;
  const float* b; int64_t ldb; int64_t stride_b; int trans_b;
  const float* b_lo;        // tensor-core path only: when set, `b` holds the TF32-rounded values of
                            // B and `b_lo` the rounded remainders, same layout; or null
  const void* b16_hi;       // tensor-core path only: fp16 split of a constant B, [n, ldb16] halves each:
  const void* b16_lo;       // hi = rn_fp16(B), lo = rn_fp16((B - hi) * 2^11); or null
  int64_t ldb16;            // a multiple of 8
  const void* a16_hi;       // tensor-core path only: fp16 split of A written by its producer, [m, lda16]
  const void* a16_lo;       // halves each (same encoding as b16_hi / b16_lo); or null
  int64_t lda16;            // a multiple of 8
  float* c; int64_t ldc; int64_t stride_c;   // c may be null when c16_hi / c16_lo are given
  void* c16_hi;             // tensor-core pair kernel only: the result also (or only) as fp16 hi / lo
  void* c16_lo;             // halves [m, ldc16], for the GEMM that takes it as its pre-split A; or null
  int64_t ldc16;
  int c16_fixed;            // 0: hi / lo as f16_split (lo scaled by 2^11); 1: both on the fixed scale 2^8
                            // (f16_split_fixed): what the kernels that take their operands by TMA read
  int a16_fixed;            // a16_hi / a16_lo are on the fixed scale (required by the pair kernel that takes them)
  int b16_plain;            // b16_lo = rn(v - hi) on the scale of b16_hi (the same kernel's format for B)
  const float* b16_inv_scale;  // device scalar 2^-e when b16_hi / b16_lo hold B * 2^e; or null
  const float* b_row_scale;    // tensor-core path with B given [K, N] only: row k of B[batch] is multiplied by
  int64_t b_row_scale_stride;  // b_row_scale[batch * stride + k] (fp32, before the split); or null
  float alpha;
  float beta;               // applied to c_in (may alias c); 0: c_in not read
  const float* c_in; int64_t ldc_in; int64_t stride_c_in;
  const float* bias_n;      // [n] or null; added as bias_scale * bias_n[col]
  const float* bias_m;      // [m] or null; added as bias_scale * bias_m[row]
  float bias_scale;         // 1 unless a Gemm node carries beta != 1
  int act; float act_alpha, act_beta;
  const float* residual; int64_t ld_res; int64_t stride_res;  // added after act; or null
  int residual_first;       // residual + v instead of v + residual (same value, kept for clarity)
  float* workspace;         // tensor-core path: scratch for K-sliced tail tiles, or null
  size_t workspace_bytes;
  int allow_pairs;          // fp16 split on clusters of two CTAs (tcgen05 .cta_group::2): 0 no, 1 A staged
                            // through registers, 2 A taken pre-split from a16_hi / a16_lo by TMA
};
cudaError_t launch_gemm_simt(const GemmParams& p, cudaStream_t st);

// tcgen05 / TMEM / TMA path. Needs A row-major with K contiguous (trans_a == 0)
// and B stored [N, K] (trans_b == 1), 16-byte aligned bases and leading
// dimensions that are multiples of 4 floats. mode 0: the fp16 split (three fp16
// MMAs per product) when b16_hi / b16_lo are given, else 3xTF32; 2: 1xTF32; 3: 3xTF32.
// `err_word` (device memory) receives a non-zero code if a bounded wait expired, or
// kGemmRangeCode if an element of A does not fit the fp16 split (result unusable).
bool gemm_tc_supported(const GemmParams& p);
cudaError_t launch_gemm_tc(const GemmParams& p, int mode, int* err_word, cudaStream_t st);
// Scratch the tensor-core path wants for this problem (0 when its tiles fill whole rounds).
// variant: 0 TF32 with B arriving split, 1 TF32 with one copy of B, 2 fp16 split.
size_t gemm_tc_workspace_bytes(int64_t m, int64_t n, int64_t k, int64_t batch, int variant, int allow_pairs);
// True when the fp16-split GEMM of this shape runs on CTA pairs that want A pre-split
// (a16_hi / a16_lo): the producer of A, or a split kernel in front, then writes the halves.
bool gemm_tc_wants_presplit(int64_t m, int64_t n, int64_t k, int64_t batch);
constexpr int kGemmRangeCode = 21;
// fp16 split of a constant [rows, k] operand (row stride ld) into [rows, k8] halves
// (k8 >= k, a multiple of 8, padding zero); leaves kGemmRangeCode in *err_word when an
// element exceeds the fp16 range.
// `inv_scale` (constant operands): x is first multiplied by the power of two 2^e that brings its
// largest magnitude into [2^13, 2^14), so that neither half meets the fp16 subnormals however
// small the weights are; *inv_scale receives 2^-e for the GEMM's epilogue, `absmax_scratch` is
// one device word of scratch. Null for activations (no scaling).
// `plain` = 0: lo = rn((v - hi) * 2^11) (two accumulators in the GEMM); 1: lo = rn(v - hi) on the
// scale of hi, and an activation is first multiplied by the fixed scale 2^8 -- the operand
// formats of the single-accumulator pair kernel (GemmParams::a16_fixed, b16_plain).
cudaError_t launch_f16_split(const float* x, void* hi, void* lo, int64_t rows, int64_t k, int64_t ld, int64_t k8,
                             int* err_word, float* inv_scale, unsigned* absmax_scratch, int plain, cudaStream_t st);
// Whether the tensor-core pair kernel can write its result split (c16_hi / c16_lo) with this epilogue.
bool gemm_tc_can_split_output(int act, bool bias_n, bool bias_m, bool c_in, float alpha, float bias_scale);
// hi[i] = rn_tf32(x[i]); lo[i] = rn_tf32(x[i] - hi[i])
cudaError_t launch_tf32_split(const float* x, float* hi, float* lo, int64_t n, cudaStream_t st);

// ---- fused attention core ---------------------------------------------------------
// O[b, t, h*hd + d] = sum_j Softmax_j((Q K^T)[t, j] (*|/) scale) V[j, d], with
// Q/K/V[b, t, h*hd + d] at q/k/v + b*batch_stride + t*row_stride + h*hd + d.
struct AttentionParams {
  const float* q; const float* k; const float* v;
  int64_t row_stride, batch_stride;
  float* out; int64_t out_row_stride, out_batch_stride;
  int batch, heads, tokens, head_dim;
  const float* scale;   // device scalar or null
  int scale_mode;       // 1: multiply, 2: divide
  int use_tc;           // take the tcgen05 kernel when it supports the shape
  int* err_word;        // device word for the tcgen05 kernel's bounded waits (or null)
  void* out16_hi;       // tcgen05 kernel only: the result also (or, with out == null, only) split into
  void* out16_lo;       // fp16 hi / lo halves [B, T, H*hd] for the GEMM that consumes it; or null
};
bool attention_supported(const AttentionParams& p);
// Dispatches to the tcgen05 kernel (use_tc and attention_tc_supported) or the CUDA-core kernel.
cudaError_t launch_attention(const AttentionParams& p, cudaStream_t st);
// tcgen05 kernel: head_dim 64, 64 < tokens <= 256, 3xTF32 products.
bool attention_tc_supported(const AttentionParams& p);
cudaError_t launch_attention_tc(const AttentionParams& p, cudaStream_t st);

// tcgen05 kernel fed by TMA: Q, K and V are column ranges of one [B, T, ld16] projection that its
// GEMM wrote as two fp16 arrays on the fixed scale (GemmParams::c16_fixed); head_dim 64,
// 64 < tokens <= 208. Head h of an operand starts at column col + 64 h.
struct Attention16Params {
  const void* qkv16_hi; const void* qkv16_lo;
  int64_t ld16, q_col, k_col, v_col;
  float* out; int64_t out_row_stride, out_batch_stride;   // out may be null when out16_hi / out16_lo are given
  void* out16_hi; void* out16_lo;                         // the result as fp16 hi / lo halves (same strides), or null
  int batch, heads, tokens, head_dim;
  const float* scale; int scale_mode;                     // device scalar or null; 1: multiply, 2: divide
  int* err_word;
};
bool attention_tc16_shape_ok(int head_dim, int tokens, int64_t ld16, int64_t q_col, int64_t k_col, int64_t v_col,
                             int64_t out_row_stride, int64_t out_batch_stride);
bool attention_tc16_supported(const Attention16Params& p);
cudaError_t launch_attention_tc16(const Attention16Params& p, cudaStream_t st);

}  // namespace ac
