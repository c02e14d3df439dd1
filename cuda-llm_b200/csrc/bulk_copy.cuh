// Bulk asynchronous copies (the TMA engine without a tensor map) and the mbarrier that
// tracks them, in raw PTX for sm_100a.  One thread issues a copy of any 16-byte-multiple
// size from global to shared memory; the bytes land asynchronously and complete a
// transaction count on an mbarrier that the consumers poll.  No register ever holds the
// data in flight, so a single thread can keep tens of kilobytes in flight per CTA.
//
// Rules kept by every user in this library: source, destination and size are multiples
// of 16 bytes; copies never use cluster multicast; every wait is bounded.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace b2 {

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbarrier_init(uint64_t* bar, uint32_t arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(arrivals) : "memory");
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbarrier_expect_bytes(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* global_src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_addr(smem_dst)),
               "l"(global_src), "r"(bytes), "r"(smem_addr(bar))
               : "memory");
}
// One hardware-assisted wait: the thread is suspended until the barrier's phase with this parity has
// completed or about `hint_ns` nanoseconds have passed, whichever comes first; true = completed.
// (A polling loop around test_wait with a sleep wakes far later than the data arrives.)
__device__ __forceinline__ bool mbarrier_try_wait(uint64_t* bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t done;
  asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}"
               : "=r"(done)
               : "r"(smem_addr(bar)), "r"(parity), "r"(hint_ns)
               : "memory");
  return done != 0;
}
// Bounded wait: at most 2^15 suspensions of ~10 us each (a third of a second), then give up; the caller
// records the failure and carries on without touching the data.
__device__ __forceinline__ bool mbarrier_wait_bounded(uint64_t* bar, uint32_t parity) {
  for (int attempt = 0; attempt < (1 << 15); ++attempt)
    if (mbarrier_try_wait(bar, parity, 10000u)) return true;
  return false;
}

// Orders this thread's earlier generic-proxy accesses to shared memory before later async-proxy
// (bulk copy) accesses: needed before a buffer that threads have just read is refilled by a copy.
__device__ __forceinline__ void fence_before_bulk_copy() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

}  // namespace b2
