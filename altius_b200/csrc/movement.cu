// Data-movement kernels: MaxPool, generic strided copy (Transpose, Slice,
// Split, Gather, Concat pieces), batched 2-D transpose through shared memory,
// im2col. Pure copies are bit-exact by construction.
#include "kernels.h"

namespace ac {
namespace {

// compute_max_pool, crates/session_interpreter/src/session.rs:325-382:
// f32::MIN start value; a window that saw no element yields 0.0.
__global__ void max_pool_kernel(const float* __restrict__ x, float* __restrict__ out,
                                int64_t total, int ih, int iw, int oh, int ow, int kh, int kw,
                                int sh, int sw, int pad_t, int pad_l) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int ox = (int)(i % ow);
  const int oy = (int)((i / ow) % oh);
  const int64_t plane = i / ((int64_t)ow * oh);
  const float* in = x + plane * (int64_t)ih * iw;
  const int y0 = oy * sh - pad_t, x0 = ox * sw - pad_l;
  const float FMIN = -3.402823466e+38f;
  float m = FMIN;
  const int fy0 = max(-y0, 0), fy1 = min(kh, ih - y0);
  const int fx0 = max(-x0, 0), fx1 = min(kw, iw - x0);
  for (int fy = fy0; fy < fy1; ++fy)
    for (int fx = fx0; fx < fx1; ++fx) m = fmaxf(__ldg(in + (y0 + fy) * iw + (x0 + fx)), m);
  out[i] = (m == FMIN) ? 0.0f : m;
}

struct CopyDev {
  int rank;
  int64_t dims[kMaxRank];
  int64_t in_str[kMaxRank];
  int64_t out_str[kMaxRank];
};

// One item = VEC consecutive elements of the innermost dim (both strides 1 there).
template <typename T, typename IDX>
__global__ void __launch_bounds__(256) strided_copy_kernel(const T* __restrict__ in,
                                                           T* __restrict__ out, CopyDev p,
                                                           IDX n_items) {
  const IDX item = (IDX)blockIdx.x * 256 + threadIdx.x;
  if (item >= n_items) return;
  IDX rem = item;
  int64_t io = 0, oo = 0;
#pragma unroll 1
  for (int d = p.rank - 1; d >= 0; --d) {
    const IDX dim = (IDX)p.dims[d];
    const IDX q = rem / dim;
    const IDX r = rem - q * dim;
    io += (int64_t)r * p.in_str[d];
    oo += (int64_t)r * p.out_str[d];
    rem = q;
  }
  out[oo] = in[io];
}

// in [batch, R, C] -> out [batch, C, R], 32x32 tiles staged in shared memory
// (+1 padding: no bank conflicts), coalesced on both sides.
__global__ void __launch_bounds__(256) transpose2d_kernel(const float* __restrict__ in,
                                                          float* __restrict__ out, int R, int C) {
  __shared__ float tile[32][33];
  const int64_t b = blockIdx.z;
  const float* src = in + b * (int64_t)R * C;
  float* dst = out + b * (int64_t)R * C;
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    const int r = r0 + ty + j, c = c0 + tx;
    if (r < R && c < C) tile[ty + j][tx] = __ldg(src + (int64_t)r * C + c);
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    const int c = c0 + ty + j, r = r0 + tx;
    if (r < R && c < C) dst[(int64_t)c * R + r] = tile[tx][ty + j];
  }
}

// im2col, crates/session_interpreter/src/conv2d.rs:213-332:
// col[n, c, fy, fx, oh, ow] = x[n, c, fy*dh + oh*sh - pad_t, fx*dw + ow*sw - pad_l] or 0.
__global__ void __launch_bounds__(256) im2col_kernel(const float* __restrict__ x,
                                                     float* __restrict__ col, ConvParams p,
                                                     int64_t total) {
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= total) return;
  const int ow = (int)(i % p.ow);
  int64_t r = i / p.ow;
  const int oh = (int)(r % p.oh); r /= p.oh;
  const int fx = (int)(r % p.kw); r /= p.kw;
  const int fy = (int)(r % p.kh); r /= p.kh;  // r = n * c + ch
  const int iy = fy * p.dh + oh * p.sh - p.pad_t;
  const int ix = fx * p.dw + ow * p.sw - p.pad_l;
  float v = 0.f;
  if (iy >= 0 && iy < p.ih && ix >= 0 && ix < p.iw)
    v = __ldg(x + (r * p.ih + iy) * (int64_t)p.iw + ix);
  col[i] = v;
}

// Patch rows for a convolution whose windows do not overlap (kernel == stride, no
// padding): the im2col matrix transposed, rows[(n, oy, ox)][(c, fy, fx)], so that the
// convolution is one GEMM rows x W^T whose output is already [n, tokens, channels].
__global__ void __launch_bounds__(256) patchify_kernel(const float* __restrict__ x, float* __restrict__ rows,
                                                       ConvParams p, int64_t total4) {
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= total4) return;
  const int kw4 = p.kw / 4;
  const int fx4 = (int)(i % kw4);
  int64_t r = i / kw4;
  const int fy = (int)(r % p.kh); r /= p.kh;
  const int c = (int)(r % p.c); r /= p.c;
  const int ox = (int)(r % p.ow); r /= p.ow;
  const int oy = (int)(r % p.oh); r /= p.oh;   // r = image index
  const float* src = x + ((r * p.c + c) * p.ih + (oy * p.kh + fy)) * (int64_t)p.iw + ox * p.kw + fx4 * 4;
  reinterpret_cast<float4*>(rows)[i] = __ldg(reinterpret_cast<const float4*>(src));
}

// compute_resize, crates/session_interpreter/src/session.rs:1057-1132. Every operation is
// rounded separately, as the Rust expressions are.
__global__ void __launch_bounds__(256) resize_kernel(const float* __restrict__ x, float* __restrict__ out,
                                                     int64_t total, int ih, int iw, int oh, int ow, int mode) {
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= total) return;
  const int w = (int)(i % ow);
  const int h = (int)((i / ow) % oh);
  const int64_t plane = i / ((int64_t)ow * oh);
  const float* in = x + plane * (int64_t)ih * iw;
  const float scale = __fdiv_rn((float)oh, (float)ih);
  if (mode == 0) {
    const int sy = min((int)__fdiv_rn((float)h, scale), ih - 1);
    const int sx = min((int)__fdiv_rn((float)w, scale), iw - 1);
    out[i] = __ldg(in + (int64_t)sy * iw + sx);
    return;
  }
  const float yf = fmaxf(__fsub_rn(__fdiv_rn((float)h, scale), 0.5f), 0.f);
  const float xf = fmaxf(__fsub_rn(__fdiv_rn((float)w, scale), 0.5f), 0.f);
  const int y = (int)yf, xx = (int)xf;
  const int y0 = min(y, ih - 1), y1 = min(y + 1, ih - 1);
  const int x0 = min(xx, iw - 1), x1 = min(xx + 1, iw - 1);
  const float v00 = __ldg(in + (int64_t)y0 * iw + x0), v01 = __ldg(in + (int64_t)y0 * iw + x1);
  const float v10 = __ldg(in + (int64_t)y1 * iw + x0), v11 = __ldg(in + (int64_t)y1 * iw + x1);
  const float fy = __fsub_rn(yf, (float)y), fx = __fsub_rn(xf, (float)xx);
  const float hd = __fadd_rn(v00, __fmul_rn(__fsub_rn(v10, v00), fy));
  const float hw = __fadd_rn(v01, __fmul_rn(__fsub_rn(v11, v01), fy));
  out[i] = __fadd_rn(hd, __fmul_rn(__fsub_rn(hw, hd), fx));
}

}  // namespace

cudaError_t launch_resize(const float* x, float* out, int64_t planes, int ih, int iw, int oh, int ow, int mode,
                          cudaStream_t st) {
  const int64_t total = planes * oh * ow;
  if (total == 0) return cudaSuccess;
  resize_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(x, out, total, ih, iw, oh, ow, mode);
  return cudaGetLastError();
}

cudaError_t launch_patchify(const ConvParams& p, const float* x, float* rows, cudaStream_t st) {
  const int64_t total4 = (int64_t)p.n * p.oh * p.ow * p.c * p.kh * (p.kw / 4);
  if (total4 == 0) return cudaSuccess;
  patchify_kernel<<<(unsigned)((total4 + 255) / 256), 256, 0, st>>>(x, rows, p, total4);
  return cudaGetLastError();
}

cudaError_t launch_max_pool(const float* x, float* out, int64_t planes, int ih, int iw, int oh,
                            int ow, int kh, int kw, int sh, int sw, int pad_t, int pad_l,
                            cudaStream_t st) {
  const int64_t total = planes * oh * ow;
  if (total == 0) return cudaSuccess;
  max_pool_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(x, out, total, ih, iw, oh, ow,
                                                                  kh, kw, sh, sw, pad_t, pad_l);
  return cudaGetLastError();
}

cudaError_t launch_strided_copy(const CopyParams& q, const void* in, void* out, cudaStream_t st) {
  if (q.n == 0) return cudaSuccess;
  // Collapse the iteration space: drop extent-1 dims, merge dims that are
  // contiguous in both tensors.
  int64_t dims[kMaxRank], is[kMaxRank], os[kMaxRank];
  int r = 0;
  for (int d = 0; d < q.rank; ++d) {
    if (q.dims[d] == 1) continue;
    if (r > 0 && is[r - 1] == q.in_str[d] * q.dims[d] && os[r - 1] == q.out_str[d] * q.dims[d]) {
      dims[r - 1] *= q.dims[d];
      is[r - 1] = q.in_str[d];
      os[r - 1] = q.out_str[d];
    } else {
      dims[r] = q.dims[d]; is[r] = q.in_str[d]; os[r] = q.out_str[d]; ++r;
    }
  }
  if (r == 0) { dims[0] = 1; is[0] = 1; os[0] = 1; r = 1; }
  int eb = q.elem_bytes;
  const char* ip = static_cast<const char*>(in) + q.in_off * eb;
  char* op = static_cast<char*>(out) + q.out_off * eb;
  // Widen the element to 16 bytes when the innermost dim is contiguous on both
  // sides and everything stays aligned.
  if (eb == 4 && is[r - 1] == 1 && os[r - 1] == 1 && dims[r - 1] % 4 == 0 &&
      (reinterpret_cast<uintptr_t>(ip) & 15) == 0 && (reinterpret_cast<uintptr_t>(op) & 15) == 0) {
    bool ok = true;
    for (int d = 0; d < r - 1; ++d)
      if (is[d] % 4 != 0 || os[d] % 4 != 0) ok = false;
    if (ok) {
      dims[r - 1] /= 4;
      for (int d = 0; d < r - 1; ++d) { is[d] /= 4; os[d] /= 4; }
      eb = 16;
    }
  }
  CopyDev p;
  p.rank = r;
  int64_t n = 1;
  for (int d = 0; d < kMaxRank; ++d) {
    p.dims[d] = d < r ? dims[d] : 1;
    p.in_str[d] = d < r ? is[d] : 0;
    p.out_str[d] = d < r ? os[d] : 0;
    if (d < r) n *= dims[d];
  }
  const unsigned blocks = (unsigned)((n + 255) / 256);
  const bool small = n < (int64_t(1) << 31);
#define AC_COPY(T)                                                                              \
  do {                                                                                          \
    if (small) strided_copy_kernel<T, unsigned><<<blocks, 256, 0, st>>>((const T*)ip, (T*)op, p, (unsigned)n); \
    else strided_copy_kernel<T, int64_t><<<blocks, 256, 0, st>>>((const T*)ip, (T*)op, p, n);   \
  } while (0)
  if (eb == 16) AC_COPY(float4);
  else if (eb == 8) AC_COPY(int64_t);
  else if (eb == 4) AC_COPY(int32_t);
  else if (eb == 1) AC_COPY(uint8_t);
  else return cudaErrorInvalidValue;
#undef AC_COPY
  return cudaGetLastError();
}

cudaError_t launch_transpose2d(const float* in, float* out, int64_t batch, int r, int c,
                               cudaStream_t st) {
  if (batch == 0 || r == 0 || c == 0) return cudaSuccess;
  if (batch > 65535) return cudaErrorInvalidValue;
  dim3 grid((c + 31) / 32, (r + 31) / 32, (unsigned)batch);
  transpose2d_kernel<<<grid, 256, 0, st>>>(in, out, r, c);
  return cudaGetLastError();
}

cudaError_t launch_im2col(const ConvParams& p, const float* x, float* col, cudaStream_t st) {
  const int64_t total = (int64_t)p.n * p.c * p.kh * p.kw * p.oh * p.ow;
  if (total == 0) return cudaSuccess;
  im2col_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(x, col, p, total);
  return cudaGetLastError();
}

}  // namespace ac
