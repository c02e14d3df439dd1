// One-step exchange between the GPUs of a node, fused into the tail of a reduction kernel.
//
// The vocabulary-sharded reductions end with a tiny all-to-all: every GPU holds one 8-byte
// partial result per row (a packed (value, index) key for argmax, a (max, sum) pair for
// softmax) and every GPU needs all of them.  Instead of leaving the kernel, calling a
// collective library and launching a second kernel, the LAST CTA of the reduction kernel
//   1. copies this GPU's partials into slot `rank` of every peer's exchange buffer with plain
//      stores through NVLink peer mappings (coalesced, 8 bytes per row per peer),
//   2. publishes them: system-scope fence, then a release store of the call's epoch into
//      flag `rank` of every peer,
//   3. waits (bounded) until the flags of all peers in its OWN buffer show this epoch,
//   4. combines the world x rows partials, which by then sit in this GPU's own memory.
// Data always lands in the consumer's memory first; nothing here reads a peer's memory, and
// no multicast is involved.
//
// Exchange buffer (one per GPU, allocated by the caller, zero-filled once, mapped into every
// peer process with b2_ipc_export / b2_ipc_open):
//   [0]    uint32 epoch      calls completed on this GPU
//   [4]    uint32 done       rows finished in the running call (returns to 0)
//   [64]   uint32 flags[2][kMaxWorld]            epoch last published by each peer, per parity
//   [256]  uint64 slots[2][world][max_rows]      the partials, per parity
// Two parities: a GPU that has finished call n may already write call n+1 into its peers
// while a slower peer still reads call n; it cannot reach call n+2 before that peer has
// published call n+1, i.e. finished reading call n.
// Every GPU of the group must make the same sequence of calls on a buffer (a collective).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace b2 {

constexpr int kMaxWorld = 16;   // B2_P2P_MAX_WORLD
constexpr size_t kExchangeHeaderBytes = 256;

struct ExchangeArgs {
  unsigned char* buf[kMaxWorld];   // [rank] = this GPU's buffer, the others are peer mappings
  int world, rank;
  int64_t max_rows;
  unsigned long long timeout_ns;   // bound of step 3
  int* status;                     // device int32, may be null: bit 1 is OR-ed in when the wait ran out
};

__host__ __device__ inline size_t exchange_bytes(int world, int64_t max_rows) {
  return kExchangeHeaderBytes + size_t(2) * size_t(world) * size_t(max_rows) * 8;
}

__device__ __forceinline__ uint32_t* exchange_epoch(unsigned char* b) { return reinterpret_cast<uint32_t*>(b); }
__device__ __forceinline__ uint32_t* exchange_done(unsigned char* b) { return reinterpret_cast<uint32_t*>(b + 4); }
__device__ __forceinline__ uint32_t* exchange_flags(unsigned char* b, uint32_t parity) {
  return reinterpret_cast<uint32_t*>(b + 64) + parity * kMaxWorld;
}
__device__ __forceinline__ unsigned long long* exchange_slots(unsigned char* b, uint32_t parity, int from, int world,
                                                              int64_t max_rows) {
  return reinterpret_cast<unsigned long long*>(b + kExchangeHeaderBytes) + (int64_t(parity) * world + from) * max_rows;
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void store_release_system(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t load_acquire_system(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Where a row's finishing thread leaves this GPU's partial for the running call.
__device__ __forceinline__ unsigned long long* exchange_own_slot(const ExchangeArgs& xa) {
  unsigned char* own = xa.buf[xa.rank];
  const uint32_t parity = (*exchange_epoch(own) + 1u) & 1u;   // the epoch only changes at the very end of a call
  return exchange_slots(own, parity, xa.rank, xa.world, xa.max_rows);
}

// Called by a row's finishing thread after it has stored the row's partial into exchange_own_slot():
// true for exactly one thread per call, the one that finished the last row.
__device__ __forceinline__ bool exchange_row_done(const ExchangeArgs& xa, int64_t rows) {
  __threadfence();
  return atomicAdd(exchange_done(xa.buf[xa.rank]), 1u) == uint32_t(rows - 1);
}

// Steps 1-4, run by every thread of the CTA that finished the last row.  combine(row, partials_of_rank)
// is called for rows handed out thread by thread; partials_of_rank(g) returns GPU g's partial of that row.
template <typename Combine>
__device__ __forceinline__ void exchange_tail(const ExchangeArgs& xa, int64_t rows, Combine&& combine) {
  unsigned char* own = xa.buf[xa.rank];
  const int tid = threadIdx.x, threads = blockDim.x;
  __threadfence();   // the other CTAs' partials (ordered before their tickets) are visible to this CTA
  const uint32_t epoch = *exchange_epoch(own) + 1u, parity = epoch & 1u;
  const unsigned long long* mine = exchange_slots(own, parity, xa.rank, xa.world, xa.max_rows);
  // 1. this GPU's partials into slot `rank` of every peer
  for (int g = 0; g < xa.world; ++g) {
    if (g == xa.rank) continue;
    unsigned long long* theirs = exchange_slots(xa.buf[g], parity, xa.rank, xa.world, xa.max_rows);
    for (int64_t r = tid; r < rows; r += threads) theirs[r] = __ldcg(mine + r);
  }
  // 2. publish
  __threadfence_system();
  __syncthreads();
  if (tid < xa.world) store_release_system(exchange_flags(xa.buf[tid], parity) + xa.rank, epoch);
  // 3. bounded wait for every peer's flag in this GPU's own buffer
  int arrived = 1;
  if (tid < xa.world) {
    const uint32_t* flag = exchange_flags(own, parity) + tid;
    const unsigned long long start = global_timer_ns();
    while (load_acquire_system(flag) != epoch) {
      if (global_timer_ns() - start > xa.timeout_ns) { arrived = 0; break; }
      __nanosleep(64);
    }
  }
  arrived = __syncthreads_and(arrived);
  // 4. combine (meaningless after a timeout, but harmless: everything read is this GPU's own memory)
  for (int64_t r = tid; r < rows; r += threads) {
    combine(r, [&](int g) {
      // plain loads could be served by a stale line of this SM's L1; these go to L2
      return __ldcg(exchange_slots(own, parity, g, xa.world, xa.max_rows) + r);
    });
  }
  __syncthreads();
  if (tid == 0) {
    *exchange_done(own) = 0u;
    *exchange_epoch(own) = epoch;
    if (!arrived && xa.status != nullptr) atomicOr(xa.status, 2);
  }
}

}  // namespace b2
