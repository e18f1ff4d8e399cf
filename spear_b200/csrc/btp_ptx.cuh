// Inline-PTX wrappers used by the BTP kernels (sm_100a): mbarrier, TMA tiled and
// bulk copies, ldmatrix / movmatrix / mma.sync, fast exp2 / log2.
// Own replacement for what the reference takes from CUTLASS/CuTe
// (csrc/btp/btp_common.h:35-64).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace btp {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
// Makes freshly initialised barriers visible to the async (TMA) proxy.
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Raises the transaction count the current phase waits for, without arriving.
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// One probe of the barrier.  The thread may be suspended by the hardware for up to kTryWaitHintNs while the phase
// is incomplete (it is woken as soon as the phase completes), so that a warp whose data is still on its way
// does not fill the issue slots of its neighbours with polling.
#ifndef BTP_TRY_WAIT_HINT_NS
#define BTP_TRY_WAIT_HINT_NS 1000
#endif
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      "  .reg .pred p;\n"
      "  mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
      "  selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(static_cast<uint32_t>(BTP_TRY_WAIT_HINT_NS))
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after `limit_ns` of wall time and returns false.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, unsigned long long limit_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_timer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
    }
    if (global_timer_ns() - t0 > limit_ns) return false;
  }
}

// ---------------------------------------------------------------- thread-block clusters (distributed shared memory)
__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_cta_count() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
// Address, in the cluster-wide shared window, of the variable that sits at `addr` in the shared memory of CTA `rank`.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
// Barrier over all threads of the cluster (non-aligned forms: callable from divergent code).
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}
// Stores two floats into another CTA's shared memory and counts 8 bytes on an mbarrier of that CTA.
__device__ __forceinline__ void st_async_f32x2(uint32_t remote_addr, float a, float b, uint32_t remote_bar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v2.f32 [%0], {%1, %2}, [%3];" ::"r"(remote_addr),
               "f"(a), "f"(b), "r"(remote_bar)
               : "memory");
}
// Arrives on an mbarrier of another CTA of the cluster.
__device__ __forceinline__ void mbar_arrive_remote(uint32_t remote_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar) : "memory");
}
// Probe / bounded wait with cluster-scope acquire: the phase is completed by another CTA of the cluster.
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      "  .reg .pred p;\n"
      "  mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\n"
      "  selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(static_cast<uint32_t>(BTP_TRY_WAIT_HINT_NS))
      : "memory");
  return ok != 0;
}
// `abort_word`: shared-memory address of a word that a warp of the cluster sets when it has given up; the wait
// then gives up as well instead of sitting out its own limit (a chain of warps waiting for one another would
// otherwise take the limit once per link).
__device__ __forceinline__ bool mbar_wait_bounded_cluster(uint32_t bar, uint32_t parity, unsigned long long limit_ns,
                                                          uint32_t abort_word) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const unsigned long long t0 = global_timer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      if (mbar_try_wait_cluster(bar, parity)) return true;
    }
    uint32_t stop;
    asm volatile("ld.volatile.shared.u32 %0, [%1];" : "=r"(stop) : "r"(abort_word) : "memory");
    if (stop != 0 || global_timer_ns() - t0 > limit_ns) return false;
  }
}
// Plain store into the shared memory of a CTA of the cluster (address from map_to_cta).
__device__ __forceinline__ void st_cluster_u32(uint32_t remote_addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(remote_addr), "r"(v) : "memory");
}

// ---------------------------------------------------------------- programmatic dependent launch
// A kernel launched with the programmatic-stream-serialization attribute may start before the memory operations
// of the kernel before it in the stream are visible: it blocks in pdl_wait() until they are.  Without the launch
// attribute the instruction does nothing.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---------------------------------------------------------------- async-proxy fences / groups
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_group() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---------------------------------------------------------------- TMA (no multicast anywhere)
// 2-D tiled load global -> shared, completion on an mbarrier.  c0 = innermost coordinate.
// `map` is the generic address of a descriptor (kernel parameter, constant or global memory).
__device__ __forceinline__ void tma_load_2d(uint32_t dst, uint64_t map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  tma_load_2d(dst, reinterpret_cast<uint64_t>(map), c0, c1, bar);
}
// L2 eviction-priority policy for the stores below that take one.
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void tma_store_2d_hint(uint64_t map, int c0, int c1, uint32_t src, uint64_t policy) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group.L2::cache_hint [%0, {%1, %2}], [%3], %4;" ::"l"(map),
               "r"(c0), "r"(c1), "r"(src), "l"(policy)
               : "memory");
}
// 2-D tiled store shared -> global (bulk async-group).
__device__ __forceinline__ void tma_store_2d(uint64_t map, int c0, int c1, uint32_t src) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];" ::"l"(map), "r"(c0),
               "r"(c1), "r"(src)
               : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int c0, int c1, uint32_t src) {
  tma_store_2d(reinterpret_cast<uint64_t>(map), c0, c1, src);
}
// Untiled bulk load global -> shared (16-byte aligned addresses, size % 16 == 0).
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
// Untiled bulk store shared -> global (bulk async-group).
__device__ __forceinline__ void bulk_store(void* dst, uint32_t src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src), "r"(bytes)
               : "memory");
}
// 3-D tiled load / store (innermost coordinate first).
__device__ __forceinline__ void tma_load_3d(uint32_t dst, uint64_t map, int c0, int c1, int c2, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
  tma_load_3d(dst, reinterpret_cast<uint64_t>(map), c0, c1, c2, bar);
}
__device__ __forceinline__ void tma_store_3d(uint64_t map, int c0, int c1, int c2, uint32_t src) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3}], [%4];" ::"l"(map), "r"(c0),
               "r"(c1), "r"(c2), "r"(src)
               : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, int c0, int c1, int c2, uint32_t src) {
  tma_store_3d(reinterpret_cast<uint64_t>(map), c0, c1, c2, src);
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ---------------------------------------------------------------- warp matrix ops
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr)
               : "memory");
}
// Transposing forms: the four 8x8 matrices are stored with their COLUMNS along the 16-byte memory rows.
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr)
               : "memory");
}
__device__ __forceinline__ void stmatrix_x4_trans(uint32_t addr, uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3) {
  asm volatile("stmatrix.sync.aligned.m8n8.x4.trans.shared.b16 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(r0), "r"(r1),
               "r"(r2), "r"(r3)
               : "memory");
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}
// D(16x8,f32) = A(16x16,bf16,row) * B(16x8,bf16,col), zero accumulator in.
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}
// D(16x8,f32) = A(16x8,bf16,row) * B(8x8,bf16,col), zero accumulator in.
__device__ __forceinline__ void mma_1688(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
  asm(
      "mma.sync.aligned.m16n8k8.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(b0), "f"(0.0f));
}

// The same two products accumulating into d (d += A * B).
__device__ __forceinline__ void mma_16816_acc(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_1688_acc(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
  asm(
      "mma.sync.aligned.m16n8k8.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(b0));
}

// ---------------------------------------------------------------- scalar helpers
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float lg2(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// logistic function 1 / (1 + 2^(-z log2 e)): relative error of a few 2^-22 over the whole range, so that
// saturated gates (sigma ~ 1e-4) keep their relative accuracy; exactly 0 and 1 at the far ends.
__device__ __forceinline__ float sigmoid_fast(float z) { return rcp_approx(1.0f + ex2(z * -1.4426950408889634f)); }
// lo -> bits 0..15, hi -> bits 16..31, round to nearest even.
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}
__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
__device__ __forceinline__ float round_bf16(float v) { return bf16_lo(pack_bf16x2(v, 0.0f)); }
// Value that the tensor-core path effectively multiplies by when an Lmat entry `v` is fed as one bf16 term
// (SPLIT == false) or as two (hi + lo, SPLIT == true); the scalar halo code uses it so that a result does
// not depend on where the seams between warps fall.
template <bool SPLIT>
__device__ __forceinline__ float lmat_weight(float v) {
  const float hi = round_bf16(v);
  if constexpr (SPLIT) {
    return hi + round_bf16(v - hi);
  } else {
    return hi;
  }
}

// ---------------------------------------------------------------- the 16-bit activation type: bfloat16 or float16
// The kernels are written once; Act<F16> supplies what differs between the two 16-bit types - packing and
// unpacking of pairs, and the tensor-core instruction (the reference takes both, csrc/btp/_bindings.cu:29-31).
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}
__device__ __forceinline__ float f16_bits_to_float(unsigned short h) {
  float f;
  asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"(h));
  return f;
}
__device__ __forceinline__ void mma_16816_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}
__device__ __forceinline__ void mma_1688_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
  asm("mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(b0), "f"(0.0f));
}
__device__ __forceinline__ void mma_16816_acc_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                  uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_1688_acc_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
  asm("mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(b0));
}

template <bool F16>
struct Act {  // bfloat16
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) { return pack_bf16x2(lo, hi); }
  static __device__ __forceinline__ float lo(uint32_t v) { return bf16_lo(v); }
  static __device__ __forceinline__ float hi(uint32_t v) { return bf16_hi(v); }
  static __device__ __forceinline__ float scalar(unsigned short h) { return __uint_as_float(static_cast<uint32_t>(h) << 16); }
  static __device__ __forceinline__ void mma16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1) { mma_16816(d, a0, a1, a2, a3, b0, b1); }
  static __device__ __forceinline__ void mma8(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) { mma_1688(d, a0, a1, b0); }
  static __device__ __forceinline__ void mma16_acc(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                   uint32_t b0, uint32_t b1) { mma_16816_acc(d, a0, a1, a2, a3, b0, b1); }
  static __device__ __forceinline__ void mma8_acc(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) { mma_1688_acc(d, a0, a1, b0); }
};
template <>
struct Act<true> {  // float16
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) { return pack_f16x2(lo, hi); }
  static __device__ __forceinline__ float lo(uint32_t v) { return f16_bits_to_float(static_cast<unsigned short>(v & 0xffffu)); }
  static __device__ __forceinline__ float hi(uint32_t v) { return f16_bits_to_float(static_cast<unsigned short>(v >> 16)); }
  static __device__ __forceinline__ float scalar(unsigned short h) { return f16_bits_to_float(h); }
  static __device__ __forceinline__ void mma16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1) { mma_16816_f16(d, a0, a1, a2, a3, b0, b1); }
  static __device__ __forceinline__ void mma8(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) { mma_1688_f16(d, a0, a1, b0); }
  static __device__ __forceinline__ void mma16_acc(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                   uint32_t b0, uint32_t b1) { mma_16816_acc_f16(d, a0, a1, a2, a3, b0, b1); }
  static __device__ __forceinline__ void mma8_acc(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) { mma_1688_acc_f16(d, a0, a1, b0); }
};
// Value that the tensor-core path effectively multiplies by when `v` is fed as one 16-bit term or as two (hi + lo).
template <bool F16, bool SPLIT>
__device__ __forceinline__ float act_weight(float v) {
  const float hi = Act<F16>::lo(Act<F16>::pack(v, 0.0f));
  if constexpr (SPLIT) {
    return hi + Act<F16>::lo(Act<F16>::pack(v - hi, 0.0f));
  } else {
    return hi;
  }
}

__device__ __forceinline__ void st_shared_u32(uint32_t addr, uint32_t v) {
  asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}

}  // namespace btp
