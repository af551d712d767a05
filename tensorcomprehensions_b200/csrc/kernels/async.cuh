// mbarrier / bulk-copy PTX helpers shared by the kernels that stage data with the async proxy.
// Every wait is bounded: after about two seconds it records a code in *dev_status (and in a
// CTA-wide abort flag so the other roles stop too) and returns false instead of spinning.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace tcb200 {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// One arrival per warp instead of 32: every lane's prior writes are ordered before the elected
// lane's (releasing) arrive by the warp barrier.  128 arrivals on one mbarrier are 128 serialised
// shared-memory atomics, which is what bounds pipelines with little work per hand-off.
__device__ __forceinline__ void mbar_arrive_warp(uint64_t* bar) {
  __syncwarp();
  if ((threadIdx.x & 31) == 0) mbar_arrive(bar);
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after `limit` SM cycles (default ~4e9, about two seconds), records `code` and
// returns false.  The SM cycle counter is used because it is cheap to read; a wait that succeeds within the
// first few thousand polls (every wait of a healthy pipeline) never reads a timer at all.
constexpr long long kWaitLimitCycles = 4000000000ll;
static __device__ __noinline__ bool mbar_wait_slow(uint64_t* bar, uint32_t parity, int code,
                                                   int* dev_status, volatile int* abort_flag,
                                                   long long limit = kWaitLimitCycles) {
  const long long t0 = clock64();
  for (;;) {
    for (int i = 0; i < 1024; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > limit) {
      *abort_flag = code;
      if (dev_status) atomicCAS(dev_status, 0, code);
      return false;
    }
  }
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int code,
                                          int* dev_status, volatile int* abort_flag) {
  for (int i = 0; i < 4096; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, code, dev_status, abort_flag);
}
// Same contract, for a role that waits long and can afford to react late: sleeps `ns` nanoseconds
// between polls so that its polling does not queue ahead of the shared-memory accesses of the
// warps that are on the critical path.
__device__ __forceinline__ bool mbar_wait_relaxed(uint64_t* bar, uint32_t parity, unsigned ns, int code,
                                                  int* dev_status, volatile int* abort_flag) {
  for (int i = 0; i < 4096; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    __nanosleep(ns);
  }
  return mbar_wait_slow(bar, parity, code, dev_status, abort_flag);
}

// ---- thread-block clusters -----------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// all threads of all CTAs of the cluster
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// One arrival per warp on the barrier at the same shared-memory offset in CTA `rank` of the cluster.
// Default semantics (release at CTA scope), as for a local arrival: the data the arrival publishes is
// consumed by the tensor core (async proxy) after the writer's own proxy / tcgen05 fences, not by
// generic loads of the other CTA.  A release at cluster scope was measured to cost ~1500 cycles per
// arrival in the split warps.
__device__ __forceinline__ void mbar_arrive_warp_remote(uint64_t* bar, uint32_t rank) {
  __syncwarp();
  if ((threadIdx.x & 31) == 0) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(bar)), "r"(rank));
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(remote) : "memory");
  }
}

// 1-D bulk copy global -> shared (both 16-byte aligned, size a multiple of 16), completion counted
// in bytes on an mbarrier.  No multicast.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

}  // namespace tcb200
