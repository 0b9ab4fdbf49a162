// Asynchronous tile streaming: global -> shared memory bulk copies (the TMA engine's untiled
// cp.async.bulk) completed on mbarriers, for persistent kernels that walk a tensor tile by tile.
//
// Why: these kernels are bound by HBM bandwidth, and the bytes in flight that saturate it
// (about 45 KB per SM) should not depend on how many registers a thread needs or how many warps
// fit. A ring of S shared-memory stages with S-1 bulk copies in flight decouples the two: one
// elected thread issues a copy per tile, every thread waits on the stage's mbarrier, computes from
// shared memory and the stage is refilled after a CTA barrier.
//
// Rules encoded here:
//   * source and destination 16-byte aligned, byte counts multiples of 16 (callers check on the
//     host and take an element-wise kernel otherwise);
//   * no multicast, no cluster: every copy lands in the issuing CTA's own shared memory;
//   * every wait is bounded. When a wait runs out the thread bumps a device-side counter
//     (b200_wait_timeouts() on the host reads it) and the kernel stops streaming: the remaining
//     copies of the CTA are waited for, again with a bound, so that none is in flight when the CTA
//     exits. The GPU is never left spinning.
#pragma once

#include "common.cuh"

namespace b200 {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 16-byte load from a 32-bit shared-memory address (the form `[register + constant]` costs no
// address arithmetic when the constant is known at compile time).
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 r;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "r"(addr));
  return r;
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(arrivals) : "memory");
}

// Makes freshly initialised barriers visible to the asynchronous proxy (the copy engine).
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// One arrival that also announces `bytes` of copy traffic for the current phase.
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}

// Orders this thread's earlier generic-proxy accesses to shared memory before later
// asynchronous-proxy accesses (a stage that was read is about to be overwritten by a copy).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// Bulk copy of `bytes` (multiple of 16) from global to this CTA's shared memory; completion is
// signalled as transaction bytes on `bar`.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(smem_dst)),
      "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// The same copy with an L2 eviction-priority policy (createpolicy) attached.
__device__ __forceinline__ void bulk_load_hint(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar,
                                               uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::
          "r"(smem_u32(smem_dst)),
      "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}

// Bounded wait for the phase with the given parity. Returns false when the bound ran out.
// ~2M polls with back-off: far beyond any legitimate copy latency, well under a second.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t spin = 0; spin < (1u << 21); ++spin) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
    if (spin > 64) __nanosleep(32);
  }
  return false;
}

// Device-side count of waits that ran out, one per translation unit that streams tiles.
// (Each .cu file that includes this header gets its own counter and exports a reader.)
static __device__ unsigned int g_wait_timeouts = 0;

__device__ __forceinline__ void note_wait_timeout() { atomicAdd(&g_wait_timeouts, 1u); }

inline unsigned int read_wait_timeouts() {
  unsigned int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_wait_timeouts, sizeof(v)) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return v;
}

}  // namespace b200
