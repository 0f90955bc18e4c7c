// Fused multi-head attention core for one (image, head, block of 12*R query rows) per CTA:
//
//   S = (Q K^T) (* | /) scale ;  P = Softmax(S) ;  O = P V
//
// It replaces, in one launch, the chain the op graph spells out per layer
//   Split -> Reshape -> Transpose (x3) -> Transpose(K) -> MatMul -> Mul -> Softmax
//         -> MatMul -> Reshape -> Transpose -> Reshape
// (each a `compute_*` call in crates/session_interpreter/src/session.rs: split
// :1488-1512, transpose :1179-1278, mat_mul :621-682, mul :384-526, softmax
// :990-1026). Q, K and V are read in place from the [B, T, 3D] projection
// buffer (row stride and column offset instead of Split/Transpose copies), the
// T x T scores never leave shared memory, and O is written straight into the
// [B, T, D] layout the output projection reads.
//
// Arithmetic: both products are fp32 FMA chains in ascending k (the order of the
// oracle's sgemm for K <= 256); the scale is one separately rounded multiply or
// divide (the graph's Mul/Div node); the softmax is the reference's polynomial
// exponential with `e * (1 / sum)` (fast_math.rs:102-187, session.rs:1017-1021).
// Only the softmax row sum is reduced in a different order (warp tree).
#include "kernels.h"
#include "ref_math.cuh"

namespace ac {
namespace {

constexpr int HD = 64;        // head dimension this kernel is written for
constexpr int KPAD = HD + 4;  // K rows padded to 68 floats: conflict-free float4 reads down a column
constexpr int WARPS = 12;      // 12 warps x R rows each: three warps per scheduler hide FMA and LDS latency
constexpr int THREADS = WARPS * 32;
constexpr unsigned FULL = 0xffffffffu;

struct AttnDev {
  const float* q; const float* k; const float* v;
  long long row_stride;     // floats between consecutive tokens of q / k / v
  long long batch_stride;   // floats between images
  float* out; long long out_row_stride, out_batch_stride;
  int heads, tokens;
  const float* scale; int scale_mode;   // 0 none, 1 multiply, 2 divide
};

// NJ = ceil(tokens / 32) score columns per lane; R = query rows per thread (WARPS * R per CTA).
__device__ __forceinline__ void cp_async16(float* smem_dst, const float* gmem_src) {
  const unsigned d = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
}

template <int NJ, int R>
__global__ void __launch_bounds__(THREADS) attention_kernel(AttnDev p) {
  constexpr int TQ = WARPS * R;
  extern __shared__ __align__(16) float smem[];
  const int T = p.tokens;
  const int TP = ((T + 3) & ~3) + 4;          // score row pitch, a multiple of 4 floats
  float* Ks = smem;                           // [T][KPAD]
  float* Vs = Ks + (size_t)T * KPAD;          // [T][HD]
  float* Qs = Vs + (size_t)T * HD;            // [TQ][HD]
  float* Ss = Qs + TQ * HD;                   // [TQ][TP]

  const int bh = blockIdx.y;
  const int b = bh / p.heads, h = bh % p.heads;
  const int q0 = blockIdx.x * TQ;
  const long long base = (long long)b * p.batch_stride + (long long)h * HD;
  const float* qg = p.q + base;
  const float* kg = p.k + base;
  const float* vg = p.v + base;
  const int tid = threadIdx.x;

  // ---- stage K, V (all tokens of this head) and the Q tile with asynchronous 16-byte
  // copies (no register staging, all requests in flight at once). Group 0: Q and K,
  // needed by the first product; group 1: V, needed only by the second. ----
  for (int idx = tid; idx < TQ * (HD / 4); idx += THREADS) {
    const int row = idx / (HD / 4), c4 = idx % (HD / 4);
    float* dst = Qs + row * HD + c4 * 4;
    if (q0 + row < T) cp_async16(dst, qg + (long long)(q0 + row) * p.row_stride + c4 * 4);
    else *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  for (int idx = tid; idx < T * (HD / 4); idx += THREADS) {
    const int row = idx / (HD / 4), c4 = idx % (HD / 4);
    cp_async16(Ks + (size_t)row * KPAD + c4 * 4, kg + (long long)row * p.row_stride + c4 * 4);
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
  for (int idx = tid; idx < T * (HD / 4); idx += THREADS) {
    const int row = idx / (HD / 4), c4 = idx % (HD / 4);
    cp_async16(Vs + (size_t)row * HD + c4 * 4, vg + (long long)row * p.row_stride + c4 * 4);
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
  asm volatile("cp.async.wait_group 1;" ::: "memory");   // Q and K have landed
  __syncthreads();

  const int ty = tid >> 5, tx = tid & 31;   // ty: group of R query rows, tx: column lane
  // ---- S = Q K^T, then the scale ----
  {
    float acc[R][NJ];
#pragma unroll
    for (int i = 0; i < R; ++i)
#pragma unroll
      for (int j = 0; j < NJ; ++j) acc[i][j] = 0.f;
    int krow[NJ];
#pragma unroll
    for (int j = 0; j < NJ; ++j) krow[j] = min(tx + 32 * j, T - 1);   // clamped: extra columns are discarded
#pragma unroll 4
    for (int kk = 0; kk < HD; kk += 4) {
      float4 qv[R];
#pragma unroll
      for (int i = 0; i < R; ++i) qv[i] = *reinterpret_cast<const float4*>(Qs + (ty * R + i) * HD + kk);
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        const float4 kv = *reinterpret_cast<const float4*>(Ks + (size_t)krow[j] * KPAD + kk);
#pragma unroll
        for (int i = 0; i < R; ++i) {
          acc[i][j] = fmaf(qv[i].x, kv.x, acc[i][j]);
          acc[i][j] = fmaf(qv[i].y, kv.y, acc[i][j]);
          acc[i][j] = fmaf(qv[i].z, kv.z, acc[i][j]);
          acc[i][j] = fmaf(qv[i].w, kv.w, acc[i][j]);
        }
      }
    }
    const float sc = p.scale_mode ? __ldg(p.scale) : 1.f;
#pragma unroll
    for (int i = 0; i < R; ++i)
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        const int c = tx + 32 * j;
        if (c < T) {
          float s = acc[i][j];
          if (p.scale_mode == 1) s = __fmul_rn(s, sc);
          else if (p.scale_mode == 2) s = __fdiv_rn(s, sc);
          Ss[(ty * R + i) * TP + c] = s;
        }
      }
  }
  __syncthreads();

  // ---- row softmax: warp ty owns rows R*ty .. R*ty + R-1; the R rows advance in
  // lock step so that their shuffle chains overlap ----
  {
    float v[R][NJ];
    float m[R], sum[R];
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const float* srow = Ss + (ty * R + i) * TP;
      m[i] = CUDART_NAN_F;
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        const int c = tx + 32 * j;
        if (c < T) { v[i][j] = srow[c]; m[i] = fmaxf(v[i][j], m[i]); }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
      for (int i = 0; i < R; ++i) m[i] = fmaxf(m[i], __shfl_xor_sync(FULL, m[i], o));
#pragma unroll
    for (int i = 0; i < R; ++i) {
      sum[i] = 0.f;
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        const int c = tx + 32 * j;
        if (c < T) { v[i][j] = exp_poly_softmax(__fsub_rn(v[i][j], m[i])); sum[i] = __fadd_rn(sum[i], v[i][j]); }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
      for (int i = 0; i < R; ++i) sum[i] = __fadd_rn(sum[i], __shfl_xor_sync(FULL, sum[i], o));
#pragma unroll
    for (int i = 0; i < R; ++i) {
      float* srow = Ss + (ty * R + i) * TP;
      const float recip = __fdiv_rn(1.f, sum[i]);
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        const int c = tx + 32 * j;
        if (c < T) srow[c] = __fmul_rn(v[i][j], recip);
      }
      if (tx < TP - T) srow[T + tx] = 0.f;   // pad read by the float4 loop below
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");   // V has landed
  __syncthreads();

  // ---- O = P V: thread owns rows R*ty .. +R-1 and columns tx, tx + 32 ----
  {
    float acc[R][2];
#pragma unroll
    for (int i = 0; i < R; ++i) acc[i][0] = acc[i][1] = 0.f;
    const int t4 = T & ~3;
    for (int j = 0; j < t4; j += 4) {
      float4 pv[R];
#pragma unroll
      for (int i = 0; i < R; ++i) pv[i] = *reinterpret_cast<const float4*>(Ss + (ty * R + i) * TP + j);
      float v0[4], v1[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        v0[u] = Vs[(size_t)(j + u) * HD + tx];
        v1[u] = Vs[(size_t)(j + u) * HD + tx + 32];
      }
#pragma unroll
      for (int i = 0; i < R; ++i) {
        const float pp[4] = {pv[i].x, pv[i].y, pv[i].z, pv[i].w};
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          acc[i][0] = fmaf(pp[u], v0[u], acc[i][0]);
          acc[i][1] = fmaf(pp[u], v1[u], acc[i][1]);
        }
      }
    }
    for (int j = t4; j < T; ++j) {
      const float v0 = Vs[(size_t)j * HD + tx], v1 = Vs[(size_t)j * HD + tx + 32];
#pragma unroll
      for (int i = 0; i < R; ++i) {
        const float pp = Ss[(ty * R + i) * TP + j];
        acc[i][0] = fmaf(pp, v0, acc[i][0]);
        acc[i][1] = fmaf(pp, v1, acc[i][1]);
      }
    }
    float* og = p.out + (long long)b * p.out_batch_stride + (long long)h * HD;
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int r = q0 + ty * R + i;
      if (r < T) {
        og[(long long)r * p.out_row_stride + tx] = acc[i][0];
        og[(long long)r * p.out_row_stride + tx + 32] = acc[i][1];
      }
    }
  }
}

size_t attn_smem_bytes(int T, int R) {
  const int TP = ((T + 3) & ~3) + 4;
  return sizeof(float) * ((size_t)T * KPAD + (size_t)T * HD + WARPS * R * HD + (size_t)WARPS * R * TP);
}

// Query rows per thread: the tile height WARPS*R that minimises (tiles) x (work per tile),
// so that T = 197 takes three tiles of 72 rows rather than five of 48.
int pick_rows(int T) {
  const int nj = (T + 31) / 32;
  int best = 4;
  double best_cost = 1e300;
  for (int r : {2, 4, 6}) {
    const int tiles = (T + WARPS * r - 1) / (WARPS * r);
    const double cost = tiles * (16.0 * (r + 4 * nj) + (T / 4.0) * (r + 8) + 400.0);
    if (cost < best_cost) { best_cost = cost; best = r; }
  }
  return best;
}

template <int NJ, int R>
cudaError_t launch_nj(const AttnDev& d, int bh, cudaStream_t st) {
  static unsigned long long attr_done = 0;
  cudaError_t e = ensure_dynamic_smem(attention_kernel<NJ, R>, (int)attn_smem_bytes(NJ * 32, R), &attr_done);
  if (e != cudaSuccess) return e;
  dim3 grid((d.tokens + WARPS * R - 1) / (WARPS * R), bh);
  attention_kernel<NJ, R><<<grid, THREADS, attn_smem_bytes(d.tokens, R), st>>>(d);
  return cudaGetLastError();
}

template <int NJ>
cudaError_t launch_r(const AttnDev& d, int bh, int r, cudaStream_t st) {
  if (r == 6) return launch_nj<NJ, 6>(d, bh, st);
  if (r == 4) return launch_nj<NJ, 4>(d, bh, st);
  return launch_nj<NJ, 2>(d, bh, st);
}

}  // namespace

bool attention_supported(const AttentionParams& p) {
  auto al = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  return p.head_dim == HD && p.tokens >= 1 && p.tokens <= 256 && p.batch >= 1 && p.heads >= 1 &&
         (long long)p.batch * p.heads <= 65535 && (p.row_stride % 4) == 0 && (p.batch_stride % 4) == 0 &&
         al(p.q) && al(p.k) && al(p.v) && p.out != nullptr;
}

cudaError_t launch_attention(const AttentionParams& p, cudaStream_t st) {
  if (p.use_tc && attention_tc_supported(p)) return launch_attention_tc(p, st);
  if (p.out16_hi || !p.out) return cudaErrorInvalidValue;   // the split result exists in the tcgen05 kernel only
  if (!attention_supported(p)) return cudaErrorInvalidValue;
  AttnDev d;
  d.q = p.q; d.k = p.k; d.v = p.v;
  d.row_stride = p.row_stride; d.batch_stride = p.batch_stride;
  d.out = p.out; d.out_row_stride = p.out_row_stride; d.out_batch_stride = p.out_batch_stride;
  d.heads = p.heads; d.tokens = p.tokens;
  d.scale = p.scale; d.scale_mode = p.scale ? p.scale_mode : 0;
  const int bh = p.batch * p.heads;
  const int r = pick_rows(p.tokens);
  switch ((p.tokens + 31) / 32) {
    case 1: return launch_r<1>(d, bh, r, st);
    case 2: return launch_r<2>(d, bh, r, st);
    case 3: return launch_r<3>(d, bh, r, st);
    case 4: return launch_r<4>(d, bh, r, st);
    case 5: return launch_r<5>(d, bh, r, st);
    case 6: return launch_r<6>(d, bh, r, st);
    case 7: return launch_r<7>(d, bh, r, st);
    default: return launch_r<8>(d, bh, r, st);
  }
}

}  // namespace ac
