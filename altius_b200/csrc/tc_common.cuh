// Device-side primitives shared by the tcgen05 kernels (GEMM and attention):
// mbarrier with bounded waits, TMA tile loads, tcgen05 fences / commit / MMA /
// tensor-memory loads, and the TF32 hi/lo split. sm_100a only.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ac {
namespace tc {

constexpr uint32_t kWaitLimit = 1u << 21;    // polls before a wait gives up
// fp16 split: x = hi + lo * 2^-11 with lo kept scaled by 2^11 (out of the fp16 subnormals).
constexpr float kLoScale = 2048.f, kLoUnscale = 1.f / 2048.f;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
// Bounded wait on the phase with the given parity. Returns false on expiry.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t i = 0; i < kWaitLimit; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(addr), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}
// One non-blocking test of the phase with the given parity.
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// The same with the non-blocking test_wait: the thread keeps polling instead of being suspended
// by the hardware, which notices arrivals from another CTA of the cluster sooner.
__device__ __forceinline__ bool mbar_wait_spin(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t i = 0; i < (kWaitLimit << 4); ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(addr), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}
// A whole warp waits on an mbarrier phase: one lane polls (fewer probes of shared memory
// while the tensor core fetches its operands from it), the others get the result by shuffle.
__device__ __forceinline__ bool warp_mbar_wait(uint64_t* bar, uint32_t parity, int lane) {
  int done = 1;
  if (lane == 0) done = mbar_wait(bar, parity) ? 1 : 0;
  done = __shfl_sync(0xffffffffu, done, 0);
  return done != 0;
}

__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int x,
                                            int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
// The same load issued by either CTA of a pair with its completion counted on an mbarrier of
// the pair's leader (a shared::cluster address): the leader's MMA thread sees both CTAs' bytes
// on one barrier, without a relay.
__device__ __forceinline__ void tma_load_3d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x,
                                                 int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tc_mma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// fp16 operands (16 K-elements per instruction), fp32 accumulator.
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_ld_32x32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]),
        "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]),
        "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]),
        "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// The same load without the wait: several loads can be in flight before one tc_wait_ld().
__device__ __forceinline__ void tc_ld_32x32_nowait(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]),
        "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]),
        "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]),
        "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// Sixteen columns of the warp's 32 lanes, without the wait.
__device__ __forceinline__ void tc_ld_32x16_nowait(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]),
        "=r"(v[15])
      : "r"(taddr)
      : "memory");
}

// Round to nearest (ties away from zero) to TF32's 10 mantissa bits, on the
// integer ALU: cvt.rna.tf32.f32 gives the same bits but issues on the
// quarter-rate conversion pipe.
__device__ __forceinline__ float round_tf32(float x) {
  return __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xFFFFE000u);
}
// hi = rn_tf32(x), lo = rn_tf32(x - hi), for 4 packed floats.
__device__ __forceinline__ void tf32_split(float4 v, float4& hi, float4& lo) {
  hi.x = round_tf32(v.x); lo.x = round_tf32(__fsub_rn(v.x, hi.x));
  hi.y = round_tf32(v.y); lo.y = round_tf32(__fsub_rn(v.y, hi.y));
  hi.z = round_tf32(v.z); lo.z = round_tf32(__fsub_rn(v.z, hi.z));
  hi.w = round_tf32(v.w); lo.w = round_tf32(__fsub_rn(v.w, hi.w));
}


// hi = rn_fp16(x); lo = rn_fp16((x - hi) * 2^11); x - hi is exact in fp32.
__device__ __forceinline__ void f16_split(float4 x, uint2& hi, uint2& lo) {
  const __half2 h01 = __floats2half2_rn(x.x, x.y), h23 = __floats2half2_rn(x.z, x.w);
  const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
  const __half2 l01 = __floats2half2_rn(__fmul_rn(__fsub_rn(x.x, f01.x), kLoScale),
                                        __fmul_rn(__fsub_rn(x.y, f01.y), kLoScale));
  const __half2 l23 = __floats2half2_rn(__fmul_rn(__fsub_rn(x.z, f23.x), kLoScale),
                                        __fmul_rn(__fsub_rn(x.w, f23.y), kLoScale));
  hi.x = *reinterpret_cast<const uint32_t*>(&h01); hi.y = *reinterpret_cast<const uint32_t*>(&h23);
  lo.x = *reinterpret_cast<const uint32_t*>(&l01); lo.y = *reinterpret_cast<const uint32_t*>(&l23);
}

// ---- range of the fp16 split ------------------------------------------------------------
// Code left in the session's error word when an operand does not fit the fp16 split; the host
// then repeats the run on the 3xTF32 plan.
constexpr int kRangeCode = 21;
// |x| > 65504 (the largest fp16), infinities included, NaN excluded.
__device__ __forceinline__ unsigned beyond_half(float x) {
  const unsigned ab = __float_as_uint(x) & 0x7FFFFFFFu;
  return (ab - 0x477FE001u) <= (0x7F800000u - 0x477FE001u) ? 1u : 0u;
}
// What a thread has seen of the values it split: bit 0 an element beyond fp16, bit 1 an
// element of at least 2^-14 (the smallest normal fp16), bit 2 a non-zero element below it.
// Below 2^-14 `hi` is a subnormal and the scaled remainder has an absolute floor of 2^-36:
// harmless beside larger elements of the same rows, but a region whose non-zero elements are
// ALL that small would lose its relative precision, so it is reported like an overflow.
__device__ __forceinline__ unsigned split_seen(float x) {
  const unsigned ab = __float_as_uint(x) & 0x7FFFFFFFu;
  return beyond_half(x) | (ab >= 0x38800000u ? 2u : (ab != 0u ? 4u : 0u));
}
__device__ __forceinline__ unsigned split_seen(float4 v) {
  return split_seen(v.x) | split_seen(v.y) | split_seen(v.z) | split_seen(v.w);
}
// Verdict of a warp over everything its lanes have seen: out of range, or only tiny values.
__device__ __forceinline__ void split_report_warp(unsigned seen, int* err) {
  const unsigned all = __reduce_or_sync(0xffffffffu, seen);
  if (((all & 1u) || ((all & 4u) && !(all & 2u))) && (threadIdx.x & 31) == 0) atomicCAS(err, 0, kRangeCode);
}

// ---- the fixed-scale split (operands of the TMA-fed attention kernel) ---------------------
// X = x * 2^8; hi = rn_fp16(X); lo = rn_fp16(X - hi): both halves on ONE scale, so that the
// three partial products of a split GEMM can share an accumulator. X - hi is exact in fp32;
// lo is a normal fp16 (11 more bits of X) when |X| >= 2^-3 and has an absolute floor of 2^-25
// below that: full precision for |x| in [2^-11, 255], a loss relative to the largest element
// beside it of at most 2^-22 whenever a region holds one element of that size.
constexpr float kFixedScale = 256.f, kFixedUnscale = 1.f / 256.f;
__device__ __forceinline__ void f16_split_plain(float4 x, uint2& hi, uint2& lo) {
  const __half2 h01 = __floats2half2_rn(x.x, x.y), h23 = __floats2half2_rn(x.z, x.w);
  const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
  const __half2 l01 = __floats2half2_rn(__fsub_rn(x.x, f01.x), __fsub_rn(x.y, f01.y));
  const __half2 l23 = __floats2half2_rn(__fsub_rn(x.z, f23.x), __fsub_rn(x.w, f23.y));
  hi.x = *reinterpret_cast<const uint32_t*>(&h01); hi.y = *reinterpret_cast<const uint32_t*>(&h23);
  lo.x = *reinterpret_cast<const uint32_t*>(&l01); lo.y = *reinterpret_cast<const uint32_t*>(&l23);
}
__device__ __forceinline__ void f16_split_fixed(float4 x, uint2& hi, uint2& lo) {
  f16_split_plain(make_float4(__fmul_rn(x.x, kFixedScale), __fmul_rn(x.y, kFixedScale),
                              __fmul_rn(x.z, kFixedScale), __fmul_rn(x.w, kFixedScale)), hi, lo);
}
// As split_seen, for the fixed-scale split: bit 0 when x * 2^8 is beyond fp16, bit 1 an element
// with |x * 2^8| >= 2^-3, bit 2 a non-zero element below that.
__device__ __forceinline__ unsigned split_seen_fixed(float x) {
  const float X = __fmul_rn(x, kFixedScale);
  const unsigned ab = __float_as_uint(X) & 0x7FFFFFFFu;
  return beyond_half(X) | (ab >= 0x3E000000u ? 2u : (ab != 0u ? 4u : 0u));
}
// The same verdict from the largest magnitude a thread has seen (one FMNMX per element instead
// of the flag arithmetic; NaN is ignored by fmaxf as it is by beyond_half): beyond fp16 when
// |x| > 65504 / 2^8, at least 2^-3 after scaling when |x| >= 2^-11, else non-zero and tiny.
__device__ __forceinline__ float split_track(float m, float4 v) {
  return fmaxf(fmaxf(fmaxf(m, fabsf(v.x)), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
}
__device__ __forceinline__ unsigned split_seen_fixed_of_max(float m) {
  return (m > 255.875f ? 1u : 0u) | (m >= 0.00048828125f ? 2u : (m > 0.f ? 4u : 0u));
}
__device__ __forceinline__ unsigned split_seen_fixed(float4 v) {
  return split_seen_fixed(v.x) | split_seen_fixed(v.y) | split_seen_fixed(v.z) | split_seen_fixed(v.w);
}

// Byte offset of 8-byte chunk `c8` (4 halves) of row `row` in a K-major fp16 tile with
// 64-byte rows and the 64-byte swizzle (16-byte chunks XORed with bits 1-2 of the row).
__device__ __forceinline__ uint32_t sw64_off8(int row, int c8) {
  return (uint32_t)((row >> 3) * 512 + (row & 7) * 64 + (((c8 >> 1) ^ ((row & 7) >> 1)) << 4) + (c8 & 1) * 8);
}


// Named barrier `id` over `nthreads` threads that also returns the OR of their predicates.
__device__ __forceinline__ bool group_barrier_or(int id, int nthreads, bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %3, 0;\n\t"
      "barrier.cta.red.or.pred p, %1, %2, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r)
      : "r"(id), "r"(nthreads), "r"((uint32_t)pred)
      : "memory");
  return r != 0;
}

// ---- CTA pairs (clusters of two; tcgen05 .cta_group::2) ----------------------------------
__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// All threads of both CTAs.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(const void* local, uint32_t rank) {
  uint32_t a;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(smem_u32(local)), "r"(rank));
  return a;
}
// Arrive on an mbarrier given by its shared::cluster address (own or peer CTA). Default
// (CTA-scope release) semantics: what the arrival publishes is shared memory of the arriving
// CTA, written behind a fence.proxy.async and read by that CTA's own tensor core; a
// cluster-scope release here cost a memory-barrier stall per stage.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// MMA of a CTA pair: M = 256 (128 rows per CTA), B rows split between the two CTAs; issued by
// one thread of the leader CTA (rank 0). The eight zero words disable no output lane.
__device__ __forceinline__ void tc_mma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                uint32_t accumulate) {
  const uint32_t z = 0;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(z)
      : "memory");
}
// Completion of the pair's MMAs issued so far -> one arrival on the mbarrier at a
// shared::cluster address (own or peer CTA).
__device__ __forceinline__ void tc_commit_pair(uint32_t cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr)
               : "memory");
}

}  // namespace tc
}  // namespace ac
