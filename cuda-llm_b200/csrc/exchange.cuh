// One-step exchange between the GPUs of a node, fused into a reduction kernel.
//
// The vocabulary-sharded reductions end with a tiny all-to-all: every GPU holds one 8-byte
// partial result per row (a packed (value, index) key for argmax, a (max, sum) pair for
// softmax) and every GPU needs all of them.  Instead of leaving the kernel, calling a
// collective library and launching a second kernel, the reduction kernel does it itself:
//   1. The thread block that finishes a ROW stores that row's partial into slot `rank` of
//      every peer's exchange buffer right away, through NVLink peer mappings, while the
//      other rows are still being reduced.
//   2. A slot is 16 bytes: two 64-bit words, each carrying 32 bits of the partial and the
//      call's epoch.  A 64-bit store is delivered whole, so a word whose epoch matches
//      carries valid data: no fence, no separate flag and no second round trip are needed
//      (the scheme of low-latency collectives).  One NVLink crossing per row per peer.
//   3. The thread block that finishes the LAST row polls -- bounded -- the slots of all
//      peers in its OWN buffer (local memory), combines the world x rows partials and
//      writes the final results.
// Data always lands in the consumer's memory first; nothing here reads a peer's memory, and
// no multicast is involved.
//
// Exchange buffer (one per GPU, allocated by the caller, zero-filled once, mapped into every
// peer process with b2_ipc_export / b2_ipc_open):
//   [0]    uint32 epoch      calls completed on this GPU (a call's stamp is this + 1, never 0)
//   [4]    uint32 done       rows finished in the running call (returns to 0)
//   [256]  slots[2][world][max_rows], 16 bytes each, per parity of the epoch
// Two parities: a GPU that has finished call n may already write call n+1 into its peers
// while a slower peer still reads call n; it cannot reach call n+2 before that peer has
// sent call n+1, i.e. finished reading call n.  Stale slots carry an older epoch and are
// never taken for the current call's, so nothing is cleared between calls.
// Every GPU of the group must make the same sequence of calls on a buffer (a collective).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace b2 {

constexpr int kMaxWorld = 16;   // B2_P2P_MAX_WORLD
constexpr size_t kExchangeHeaderBytes = 256;
constexpr int kTraceStamps = 4;   // kernel start, tail start, all partials present, end; then one per peer

struct ExchangeArgs {
  unsigned char* buf[kMaxWorld];   // [rank] = this GPU's buffer, the others are peer mappings
  int world, rank;
  int64_t max_rows;
  unsigned long long timeout_ns;   // bound of step 3
  int* status;                     // device int32, may be null: bit 1 is OR-ed in when the wait ran out
  unsigned long long* trace;       // device uint64[kTraceStamps + world], may be null: %globaltimer stamps of the call
};

__host__ __device__ inline size_t exchange_bytes(int world, int64_t max_rows) {
  return kExchangeHeaderBytes + size_t(2) * size_t(world) * size_t(max_rows) * 16;
}

__device__ __forceinline__ uint32_t* exchange_epoch(unsigned char* b) { return reinterpret_cast<uint32_t*>(b); }
__device__ __forceinline__ uint32_t* exchange_done(unsigned char* b) { return reinterpret_cast<uint32_t*>(b + 4); }
__device__ __forceinline__ ulonglong2* exchange_slot(unsigned char* b, uint32_t parity, int from, int world, int64_t max_rows,
                                                     int64_t row) {
  return reinterpret_cast<ulonglong2*>(b + kExchangeHeaderBytes) + (int64_t(parity) * world + from) * max_rows + row;
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// One slot = one 16-byte store of two self-validating 64-bit words (low half | epoch, high half | epoch).
__device__ __forceinline__ void slot_store(ulonglong2* p, unsigned long long value, uint32_t epoch) {
  const unsigned long long stamp = static_cast<unsigned long long>(epoch) << 32;
  const unsigned long long w0 = (value & 0xffffffffull) | stamp, w1 = (value >> 32) | stamp;
  asm volatile("st.relaxed.sys.global.v2.u64 [%0], {%1, %2};" ::"l"(p), "l"(w0), "l"(w1) : "memory");
}
// true (and *value set) when both words of the slot carry this epoch
__device__ __forceinline__ bool slot_load(const ulonglong2* p, uint32_t epoch, unsigned long long* value) {
  unsigned long long w0, w1;
  asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];" : "=l"(w0), "=l"(w1) : "l"(p) : "memory");
  *value = (w0 & 0xffffffffull) | (w1 << 32);
  return uint32_t(w0 >> 32) == epoch && uint32_t(w1 >> 32) == epoch;
}
// Polls a slot of this GPU's own buffer until it carries the epoch, the time is up, or 2^26 polls have been made.
__device__ __forceinline__ bool slot_wait(const ulonglong2* p, uint32_t epoch, unsigned long long start,
                                          unsigned long long timeout_ns, unsigned long long* value) {
  for (int spin = 0; spin < (1 << 26); ++spin) {
    if (slot_load(p, epoch, value)) return true;
    if ((spin & 63) == 63 && global_timer_ns() - start > timeout_ns) return false;
  }
  return false;
}

// The epoch of the running call (the stored one only changes at the very end of a call).
__device__ __forceinline__ uint32_t exchange_call_epoch(const ExchangeArgs& xa) { return *exchange_epoch(xa.buf[xa.rank]) + 1u; }

// Step 1 for one row and one destination GPU (this GPU's own buffer included).
__device__ __forceinline__ void exchange_send(const ExchangeArgs& xa, uint32_t epoch, int to, int64_t row, unsigned long long partial) {
  slot_store(exchange_slot(xa.buf[to], epoch & 1u, xa.rank, xa.world, xa.max_rows, row), partial, epoch);
}

// Called by the thread that has stored a row's partial into this GPU's OWN slot: true for exactly one thread
// per call, the one that finished the last row.
// No fence orders the slot store before this count: the tail does not trust the count for the data, it polls its
// own slots like the peers' until each carries the call's epoch.
__device__ __forceinline__ bool exchange_row_done(const ExchangeArgs& xa, int64_t rows) {
  return atomicAdd(exchange_done(xa.buf[xa.rank]), 1u) == uint32_t(rows - 1);
}

__device__ __forceinline__ void exchange_trace_start(const ExchangeArgs& xa) {
  if (xa.trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0) xa.trace[0] = global_timer_ns();
}

// Step 3, run by every thread of the thread block that finished the last row.  combine(row, complete, partial_of)
// is called for rows handed out thread by thread; partial_of(g), g a compile-time-unrolled or runtime index below
// `world`, returns GPU g's partial of that row; `complete` is false when some GPU's partial had not arrived when the
// time ran out (the row's result must then be marked invalid, and the partials of the missing GPUs are undefined).
// `epoch` is the call's epoch as every thread block of the call read it (exchange_call_epoch at kernel start).
template <typename Combine>
__device__ __forceinline__ void exchange_tail(const ExchangeArgs& xa, int64_t rows, uint32_t epoch, Combine&& combine) {
  unsigned char* own = xa.buf[xa.rank];
  const int tid = threadIdx.x, threads = blockDim.x;
  const uint32_t parity = epoch & 1u;
  const unsigned long long start = global_timer_ns();
  if (xa.trace != nullptr) {
    if (tid == 0) xa.trace[1] = start;
    if (tid < xa.world) {   // when each GPU's first row was seen here
      unsigned long long ignored;
      slot_wait(exchange_slot(own, parity, tid, xa.world, xa.max_rows, 0), epoch, start, xa.timeout_ns, &ignored);
      xa.trace[kTraceStamps + tid] = global_timer_ns();
    }
  }
  int all_complete = 1;
  for (int64_t r = tid; r < rows; r += threads) {
    // all peers' slots of the row are asked for at once (the loads are independent: one trip to L2, not `world`),
    // again and again until every one carries the epoch or the time is up
    unsigned long long value[kMaxWorld];
    unsigned int missing = xa.world >= 32 ? 0xffffffffu : ((1u << xa.world) - 1u);
    for (int spin = 0; missing != 0u && spin < (1 << 26); ++spin) {
#pragma unroll
      for (int g = 0; g < kMaxWorld; ++g) {
        if (g < xa.world && (missing >> g & 1u) &&
            slot_load(exchange_slot(own, parity, g, xa.world, xa.max_rows, r), epoch, &value[g]))
          missing &= ~(1u << g);
      }
      if ((spin & 63) == 63 && global_timer_ns() - start > xa.timeout_ns) break;
    }
    const bool complete = missing == 0u;
    if (xa.trace != nullptr && r == rows - 1) xa.trace[2] = global_timer_ns();
    combine(r, complete, [&](int g) { return value[g]; });
    if (!complete) all_complete = 0;
  }
  all_complete = __syncthreads_and(all_complete);
  if (tid == 0) {
    *exchange_done(own) = 0u;
    *exchange_epoch(own) = epoch;
    if (!all_complete && xa.status != nullptr) atomicOr(xa.status, 2);
    if (xa.trace != nullptr) xa.trace[3] = global_timer_ns();
  }
}

}  // namespace b2
