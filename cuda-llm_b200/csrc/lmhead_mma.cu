// LM head fused with the greedy pick for MANY hidden rows (5 .. 64 per pass), on the 5th-generation
// tensor cores of sm_100a: logits = hidden x table^T as tcgen05.mma tiles with the arg-max taken in the
// epilogue, so that the [rows, vocab] logits tensor is never written (unless asked for) and never read.
//
// Replaces, for batches beyond the matrix-vector kernels of lmhead.cu, the reference's pair
// "cuda_lm_head / cuda_linear_out into a logits tensor, then cuda_argmax_last_row"
// (reference src/ops_cuda.cu:637-671,885; src/qwen3_cuda_model.cpp:1070-1071,1339).
//
// Shape of the work.  The table [vocab, H] fp16 (311 MB at 151936 x 1024) is read ONCE; with up to 64
// hidden rows the arithmetic (2 * 64 FLOP per table byte) is far below the tensor cores' rate, so the
// kernel is bound by HBM like the rest of this library and everything is arranged around the memory system:
//   D[128 table rows, N hidden rows] += A[128, 64] * B[N, 64]^T per 64-wide slab of H, both operands
//   K-major (the row-major tensors as they lie in memory), N = rows padded to 16 / 32 / 64.
//   warp 0      one lane claims work and issues the TMA tile copies (cp.async.bulk.tensor, 128-byte swizzle, no
//               multicast) into a ring of shared-memory stages, each completed through an mbarrier.  A stage holds
//               G = 4 consecutive slabs of 128 table rows, copied back to back: 512 contiguous bytes of every
//               row are asked for within a few hundred cycles (measured 62-68 us with one slab per stage, 60 us
//               with two, 56 us with four; the same ring fed by 16-byte cp.async copies from four warps: 69 us).
//               The hidden rows are copied once into shared memory that they keep for the whole kernel, or, when
//               N * H * 2 bytes do not fit beside two stages, their N x 64 tiles travel with every slab, from L2
//   warp 1      one lane issues tcgen05.mma (four K = 16 steps per slab) into one of two accumulators in
//               tensor memory, and tcgen05.commit to hand a stage back or an accumulator on
//   warps 2-5   read the finished accumulator with tcgen05.ld (one table row per thread, N columns), round
//               to fp16 as the stored logit would be, and keep per hidden row ONE 32-bit running best:
//               (order-preserving fp16 bits << 16 | 0xffff - first 32-row unit of the claim).  A thread's rows
//               only grow, so "strictly greater" keeps the lowest row among equal logits -- the reference's rule
//               (src/ops_cuda.cu:562); NaN and -inf never enter.  Logits are written only on request
//   at the end  the 128 threads' candidates meet in shared memory, one thread per hidden row folds them and
//               merges the block's winner into the packed (value, index) key of b2_argmax_keys with one
//               atomicMax; the last block (ticket) publishes ids / keys and re-zeroes the scratch.
// Work is claimed from a counter in units of 32 table rows: whole 128-row tiles while much is left, then three,
// two and one unit at a time, so that all thread blocks finish within one unit (64 KB) of each other.  (Equal
// static shares left the slowest SM 11 % behind the average: SMs do not get equal shares of the memory system.)
// Every wait on an mbarrier is bounded.  A wait that runs out (never expected) makes the whole thread block
// stop, frees its tensor memory, and poisons the call's keys so that every id of the call reads -1.
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_fp16.h>

#include <cfloat>
#include <climits>
#include <mutex>

#include "b2ops.h"
#include "bulk_copy.cuh"
#include "common.cuh"
#include "kernels.h"

namespace b2 {
namespace {

constexpr int kTileRows = 128;                 // table rows per tile = lanes of tensor memory
constexpr int kSlabK = 64;                     // fp16 elements per slab: 128 bytes, one swizzled row
constexpr int kUmmaK = 16;                     // K of one tcgen05.mma with 16-bit operands
constexpr int kEpilogueThreads = 128;
constexpr int kMmaThreads = 64 + kEpilogueThreads;   // warp 0 copies, warp 1 tensor cores, warps 2-5 epilogue
constexpr int kClaimSlots = 8;                 // claims travelling from the copy lane to the other roles
constexpr uint32_t kSlabBytes = kTileRows * kSlabK * 2;   // one slab of a tile: 16 KB
constexpr int kMaxStages = 12;
constexpr int kUnitRows = 32;                  // granularity of a thread block's share of the table
constexpr int kUnitsPerTile = kTileRows / kUnitRows;
constexpr unsigned long long kPoison = ~0ull;  // a key no real candidate can reach: "this call failed"
constexpr unsigned long long kSign = 0x8000000000000000ull;

// ---- raw sm_100a instructions -------------------------------------------------------------------------------

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          smem_addr(smem_dst)),
      "l"(map), "r"(x), "r"(y), "r"(smem_addr(bar))
      : "memory");
}
__device__ __forceinline__ void mbarrier_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(smem_result)), "r"(columns)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_free(uint32_t address, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns) : "memory");
}
__device__ __forceinline__ void tensor_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tensor_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// D (tensor memory) (+)= A (shared memory descriptor) * B (shared memory descriptor)
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate ? 1u : 0u)
      : "memory");
}
// the mbarrier gets one arrival once every tcgen05.mma issued so far by this thread has completed
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}
// 16 consecutive fp32 columns of this thread's lane of tensor memory
__device__ __forceinline__ void tmem_load_16(uint32_t address, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(address)
      : "memory");
}
__device__ __forceinline__ void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, swizzled in 1024-byte groups of
// eight rows: start address, leading offset 1 (unused with swizzling), 1024 bytes between row groups,
// descriptor version 1, layout "128-byte swizzle".
__device__ __forceinline__ uint64_t k_major_sw128_descriptor(const void* smem_tile) {
  const uint64_t start = (smem_addr(smem_tile) & 0x3ffffu) >> 4;
  return start | (1ull << 16) | (uint64_t(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// fp16 x fp16 -> fp32, both operands K-major, M = 128, N = n
__host__ __device__ constexpr uint32_t instruction_descriptor(int n) {
  return (1u << 4) | (uint32_t(n >> 3) << 17) | (uint32_t(kTileRows >> 4) << 24);
}

// One bounded wait of a role.  `stop` (shared memory) is raised by whichever role gives up first; the others see it
// at their next wait and leave their loops too.
__device__ __forceinline__ bool wait_or_stop(uint64_t* bar, uint32_t parity, volatile int* stop) {
  for (int attempt = 0; attempt < (1 << 14); ++attempt) {
    if (mbarrier_try_wait(bar, parity, 10000u)) return true;
    if (*stop != 0) return false;
  }
  *stop = 1;
  return false;
}

struct MmaArgs {
  int64_t vocab, index_base;
  int rows;              // hidden rows that exist (<= N)
  int slabs;             // H / 64
  int group;             // G: slabs per stage of the ring (a power of two, divides slabs)
  int stages;
  int units;             // ceil(vocab / 32): the table is dealt out in units of 32 rows
  __half* logits;        // may be null
  int64_t logits_stride;
  int32_t* out_ids;      // may be null
  int64_t* out_keys;     // may be null
  unsigned long long* keys;
  unsigned int* ticket;  // [0]: blocks that have finished; [1]: 32-row units claimed so far (both return to 0)
};

// order-preserving 16 bits of an fp16 value (neither NaN nor -inf reaches this)
__device__ __forceinline__ uint32_t ordered_half_bits(__half h) {
  const uint32_t b = __half_as_ushort(h);
  return (b & 0x8000u) ? (~b & 0xffffu) : (b | 0x8000u);
}
__device__ __forceinline__ float value_of_ordered_half_bits(uint32_t o) {
  const uint32_t b = (o & 0x8000u) ? (o & 0x7fffu) : (~o & 0xffffu);
  return __half2float(__ushort_as_half(static_cast<unsigned short>(b)));
}

// kResident: the hidden rows' slabs are copied into shared memory once (N * H * 2 bytes) and every stage of the ring
// holds table data only; otherwise each slab of a stage is followed by the slab's N x 64 hidden tile (from L2).
template <int N, bool kResident>
__global__ void __launch_bounds__(kMmaThreads, 1)
lm_head_mma_kernel(const __grid_constant__ CUtensorMap hidden_map, const __grid_constant__ CUtensorMap table_map128,
                   const __grid_constant__ CUtensorMap table_map32, const MmaArgs args) {
  constexpr uint32_t kHiddenTileBytes = N * kSlabK * 2;
  constexpr uint32_t kSlabStride = kSlabBytes + (kResident ? 0u : kHiddenTileBytes);   // one slab's share of a stage
  constexpr uint32_t kUnitBytes = kUnitRows * kSlabK * 2;                               // 4 KB
  constexpr uint32_t kAccumulatorColumns = 2 * N < 32 ? 32 : 2 * N;   // two accumulators; a power of two >= 32
  extern __shared__ unsigned char raw_smem[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~uintptr_t(1023));
  __shared__ __align__(8) uint64_t full_bar[kMaxStages], empty_bar[kMaxStages], acc_full_bar[2], acc_empty_bar[2], hidden_bar;
  __shared__ int2 claims[kClaimSlots];   // (first unit, units) of the block's n-th claim; units == 0: no more work
  __shared__ uint32_t tmem_base_slot;
  __shared__ int stop_flag;
  __shared__ int last_block;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int stages = args.stages, slabs = args.slabs, group = args.group;
  const uint32_t stage_bytes = uint32_t(group) * kSlabStride;
  volatile int* stop = &stop_flag;
  // shared memory: [resident hidden slabs] [ring of stages]
  unsigned char* resident = smem;
  unsigned char* ring = smem + (kResident ? size_t(slabs) * kHiddenTileBytes : 0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) { mbarrier_init(&full_bar[s], 1); mbarrier_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbarrier_init(&acc_full_bar[b], 1); mbarrier_init(&acc_empty_bar[b], kEpilogueThreads); }
    mbarrier_init(&hidden_bar, 1);
    stop_flag = 0;
  }
  if (warp == 1) tmem_alloc(&tmem_base_slot, kAccumulatorColumns);
  tensor_fence_before_sync();
  __syncthreads();
  tensor_fence_after_sync();
  const uint32_t tmem_base = tmem_base_slot;

  // running best of this thread's table rows per hidden row: (ordered fp16 bits << 16) | (0xffff - first unit of the
  // claim); 0 = none yet
  uint32_t best[N];
#pragma unroll
  for (int c = 0; c < N; ++c) best[c] = 0u;

  if (warp == 0) {
    // ---- claims and copies: the ring is refilled as soon as the tensor cores have read a stage
    if (lane == 0) {
      if (kResident) {
        mbarrier_expect_bytes(&hidden_bar, uint32_t(slabs) * kHiddenTileBytes);
        for (int slab = 0; slab < slabs; ++slab)
          tma_load_2d(resident + size_t(slab) * kHiddenTileBytes, &hidden_map, slab * kSlabK, 0, &hidden_bar);
      }
      unsigned int* work = args.ticket + 1;
      int stage = 0;
      uint32_t phase = 0;
      // Whole tiles while at least two units per block are left, then single units.  The NEXT claim is always
      // under way while this one is copied: the counter's answer takes a microsecond under load.
      auto claim_size = [&](int already_claimed) {
        return args.units - already_claimed >= 2 * int(gridDim.x) ? kUnitsPerTile : 1;
      };
      int next_want = claim_size(0);
      int next_first = int(atomicAdd(work, unsigned(next_want)));
      for (int seq = 0; *stop == 0; ++seq) {
        const int first = next_first, want = next_want;
        const int units = first >= args.units ? 0 : (args.units - first < want ? args.units - first : want);
        if (units != 0) {
          next_want = claim_size(first + want);
          next_first = int(atomicAdd(work, unsigned(next_want)));
        }
        if (!wait_or_stop(&empty_bar[stage], phase ^ 1u, stop)) break;   // the claim's slot is free long before
        claims[seq & (kClaimSlots - 1)] = make_int2(first, units);
        if (units == 0) {                                                 // tell the other roles, through one empty stage
          mbarrier_arrive(&full_bar[stage]);
          break;
        }
        bool ok = true;
        for (int slab0 = 0; slab0 < slabs; slab0 += group) {
          if (slab0 != 0 && !wait_or_stop(&empty_bar[stage], phase ^ 1u, stop)) { ok = false; break; }
          mbarrier_expect_bytes(&full_bar[stage], uint32_t(group) * (uint32_t(units) * kUnitBytes + (kResident ? 0u : kHiddenTileBytes)));
          for (int g = 0; g < group; ++g) {
            unsigned char* dst = ring + size_t(stage) * stage_bytes + size_t(g) * kSlabStride;
            if (units == kUnitsPerTile) {
              tma_load_2d(dst, &table_map128, (slab0 + g) * kSlabK, first * kUnitRows, &full_bar[stage]);
            } else {
              for (int u = 0; u < units; ++u)
                tma_load_2d(dst + size_t(u) * kUnitBytes, &table_map32, (slab0 + g) * kSlabK, (first + u) * kUnitRows, &full_bar[stage]);
            }
            if (!kResident) tma_load_2d(dst + kSlabBytes, &hidden_map, (slab0 + g) * kSlabK, 0, &full_bar[stage]);
          }
          if (++stage == stages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    // ---- tensor cores.  A claim of fewer than four units still runs as 128 rows: the rows past its end hold whatever
    // an earlier tile left in the stage, every accumulator row depends on its own table row only, and the epilogue
    // skips them.
    if (lane == 0) {
      constexpr uint32_t idesc = instruction_descriptor(N);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = !kResident || wait_or_stop(&hidden_bar, 0u, stop);
      for (int seq = 0; ok && *stop == 0; ++seq) {
        const int buf = seq & 1;
        if (!wait_or_stop(&acc_empty_bar[buf], ((seq >> 1) & 1u) ^ 1u, stop)) break;
        tensor_fence_after_sync();
        const uint32_t d_tmem = tmem_base + uint32_t(buf * N);
        bool finished = false;
        for (int slab0 = 0; slab0 < slabs; slab0 += group) {
          if (!wait_or_stop(&full_bar[stage], phase, stop)) { ok = false; break; }
          if (slab0 == 0 && claims[seq & (kClaimSlots - 1)].y == 0) { finished = true; break; }
          tensor_fence_after_sync();
          for (int g = 0; g < group; ++g) {
            const int slab = slab0 + g;
            const unsigned char* a = ring + size_t(stage) * stage_bytes + size_t(g) * kSlabStride;
            const unsigned char* b = kResident ? resident + size_t(slab) * kHiddenTileBytes : a + kSlabBytes;
            const uint64_t a_desc = k_major_sw128_descriptor(a), b_desc = k_major_sw128_descriptor(b);
#pragma unroll
            for (int k = 0; k < kSlabK / kUmmaK; ++k)   // 32 bytes further along the swizzled row per step
              umma_f16(d_tmem, a_desc + uint64_t(k * 2), b_desc + uint64_t(k * 2), idesc, slab > 0 || k > 0);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == stages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit(&acc_full_bar[buf]);     // an accumulator, or (finished) the news that there is none
        if (finished) break;
      }
    }
  } else {
    // ---- epilogue: thread = one table row of the tile = one lane of tensor memory
    const int quarter = warp & 3;                       // the 32 lanes this warp may read
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_address = uint32_t(quarter * 32) << 16;
    for (int seq = 0;; ++seq) {
      const int buf = seq & 1;
      if (*stop != 0 || !wait_or_stop(&acc_full_bar[buf], (seq >> 1) & 1u, stop)) break;
      const int2 claim = claims[seq & (kClaimSlots - 1)];
      if (claim.y == 0) break;
      tensor_fence_after_sync();
      const int64_t table_row = int64_t(claim.x) * kUnitRows + row_in_tile;
      const bool exists = row_in_tile < claim.y * kUnitRows && table_row < args.vocab;
      const uint32_t claim_tag = 0xffffu - uint32_t(claim.x);
      __half* logits_row = args.logits != nullptr && exists ? args.logits + table_row : nullptr;
#pragma unroll
      for (int c = 0; c < N / 16; ++c) {
        uint32_t acc[16];
        tmem_load_16(tmem_base + lane_address + uint32_t(buf * N + c * 16), acc);
        tmem_load_wait();
        if (c == N / 16 - 1) {                            // the tensor cores may overwrite this accumulator
          tensor_fence_before_sync();
          mbarrier_arrive(&acc_empty_bar[buf]);
        }
#pragma unroll
        for (int q = 0; q < 16; ++q) {
          const int r = c * 16 + q;
          const __half stored = __float2half(__uint_as_float(acc[q]));
          const uint32_t key = (ordered_half_bits(stored) << 16) | claim_tag;
          // NaN and -inf never win (the reference compares against a finite start value); equal logits keep the earlier row
          if (exists && __half2float(stored) > -INFINITY && key > best[r]) best[r] = key;
          if (logits_row != nullptr && r < args.rows) logits_row[int64_t(r) * args.logits_stride] = stored;
        }
      }
    }
  }

  // ---- every role has left its loop: nothing is in flight in a healthy run
  tensor_fence_before_sync();
  __syncthreads();
  tensor_fence_after_sync();
  const bool failed = stop_flag != 0;
  if (failed) {
    // copies that were requested may still be landing: they must not outlive this block's shared memory
    if (threadIdx.x == 0) {
      if (kResident) mbarrier_wait_bounded(&hidden_bar, 0u);
      for (int s = 0; s < stages; ++s) { mbarrier_wait_bounded(&full_bar[s], 0u); mbarrier_wait_bounded(&full_bar[s], 1u); }
    }
    __syncthreads();
  }
  if (warp == 1) tmem_free(tmem_base, kAccumulatorColumns);

  // ---- fold the 128 threads' candidates per hidden row (the ring's memory is free now)
  uint32_t* cand = reinterpret_cast<uint32_t*>(smem);
  if (warp >= 2) {
    const int t = (warp & 3) * 32 + lane;                 // the thread's row within a tile
#pragma unroll
    for (int c = 0; c < N; ++c) cand[c * kEpilogueThreads + t] = best[c];
  }
  __syncthreads();
  if (threadIdx.x < args.rows) {
    const int r = threadIdx.x;
    // Among equal values the lowest table row must win.  The rows of two claims never interleave, so the claim with
    // the lower first unit lies lower as a whole (larger key); within one claim the keys are equal and walking the
    // rows of the tile upwards, replacing only on a greater key, keeps the lowest row.
    uint32_t top = 0u;
    int top_row = 0;
    for (int t = 0; t < kEpilogueThreads; ++t) {
      const uint32_t k = cand[r * kEpilogueThreads + t];
      if (k > top) { top = k; top_row = t; }
    }
    if (failed) {
      atomicMax(args.keys + r, kPoison);
    } else if (top != 0u) {
      const int64_t row = int64_t(0xffffu - (top & 0xffffu)) * kUnitRows + top_row;
      const uint32_t b = __float_as_uint(value_of_ordered_half_bits(top >> 16));
      const uint32_t ordered = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
      atomicMax(args.keys + r, (static_cast<unsigned long long>(ordered) << 32) | (0xffffffffu - uint32_t(args.index_base + row)));
    }
    __threadfence();
  }
  __syncthreads();
  if (threadIdx.x == 0) last_block = atomicAdd(args.ticket, 1u) == gridDim.x - 1 ? 1 : 0;
  __syncthreads();
  if (!last_block || threadIdx.x >= args.rows) return;
  __threadfence();
  const int r = threadIdx.x;
  const unsigned long long key = atomicExch(args.keys + r, 0ull);
  if (key == kPoison) {
    if (args.out_keys != nullptr) args.out_keys[r] = LLONG_MIN;
    if (args.out_ids != nullptr) args.out_ids[r] = -1;
  } else {
    if (args.out_keys != nullptr) args.out_keys[r] = static_cast<int64_t>(key ^ kSign);
    if (args.out_ids != nullptr) args.out_ids[r] = key == 0ull ? 0 : int32_t(0xffffffffu - uint32_t(key & 0xffffffffull));
  }
  if (r == 0) { args.ticket[0] = 0u; args.ticket[1] = 0u; }
}

// ---- host side ----------------------------------------------------------------------------------------------

PFN_cuTensorMapEncodeTiled_v12000 tensor_map_encoder() {
  static std::once_flag once;
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult found;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &found) == cudaSuccess &&
        found == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
    else
      cudaGetLastError();
  });
  return fn;
}

// [rows, width] fp16 row-major tensor, copied in boxes of box_rows x 64 elements with the 128-byte swizzle;
// rows past the end read as zeros.
bool make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t width, int box_rows) {
  auto encode = tensor_map_encoder();
  if (encode == nullptr) return false;
  const cuuint64_t dims[2] = {cuuint64_t(width), cuuint64_t(rows)};
  const cuuint64_t strides[1] = {cuuint64_t(width) * 2};
  const cuuint32_t box[2] = {cuuint32_t(kSlabK), cuuint32_t(box_rows)};
  const cuuint32_t elem_strides[2] = {1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem_strides,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

constexpr size_t kSmemBudget = 227 * 1024 - 1024 - 2048;      // alignment slack, static shared memory

template <int N, bool kResident>
int launch_n(const CUtensorMap& hidden_map, const CUtensorMap& m128, const CUtensorMap& m32, MmaArgs args, cudaStream_t s) {
  const size_t resident_bytes = kResident ? size_t(args.slabs) * N * kSlabK * 2 : 0;
  const size_t stage_bytes = size_t(args.group) * (kSlabBytes + (kResident ? 0 : size_t(N) * kSlabK * 2));
  int stages = int((kSmemBudget - resident_bytes) / stage_bytes);
  if (stages > kMaxStages) stages = kMaxStages;
  args.stages = stages;
  size_t smem = resident_bytes + size_t(stages) * stage_bytes;
  const size_t fold = size_t(kEpilogueThreads) * N * 4;    // the final fold of the candidates reuses this memory
  if (smem < fold) smem = fold;
  smem += 1024;
  auto kernel = lm_head_mma_kernel<N, kResident>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess)
    return launch_status("lm_head_argmax (tensor cores, shared-memory attribute)");
  int grid = sm_count();
  const int tiles = (args.units + kUnitsPerTile - 1) / kUnitsPerTile;
  if (grid > tiles) grid = tiles;
  kernel<<<grid, kMmaThreads, smem, s>>>(hidden_map, m128, m32, args);
  return launch_status("lm_head_argmax (tensor cores)");
}

template <int N>
int launch_pick(const CUtensorMap& hidden_map, const CUtensorMap& m128, const CUtensorMap& m32, MmaArgs args, cudaStream_t s) {
  // four slabs per stage = 512 contiguous bytes per table row per stage, when the hidden size allows
  int group = 4;
  while (args.slabs % group != 0) group >>= 1;
  args.group = group;
  const size_t resident_bytes = size_t(args.slabs) * N * kSlabK * 2;
  const bool resident = resident_bytes + 2 * size_t(group) * kSlabBytes <= kSmemBudget;
  return resident ? launch_n<N, true>(hidden_map, m128, m32, args, s) : launch_n<N, false>(hidden_map, m128, m32, args, s);
}

}  // namespace

// True when the tensor-core kernel takes this call: fp16, a hidden size in whole 64-element slabs, 16-byte aligned
// tensors, and at most 65535 units of 32 table rows (2 M rows: the unit number travels in 16 bits).
bool lm_head_mma_supported(const void* hidden, const void* table, int64_t hidden_size, int64_t vocab) {
  return hidden_size % kSlabK == 0 && hidden_size >= kSlabK && hidden_size <= 16384 && aligned16(hidden) && aligned16(table) &&
         vocab <= int64_t(65535) * kUnitRows && tensor_map_encoder() != nullptr;
}

// One pass over the table for 2 to 64 hidden rows (fp16).  keys / ticket: the call's zeroed scratch (rows keys and
// rows tickets, of which two are used).
int launch_lm_head_mma(const void* hidden, const void* table, int64_t rows, int64_t hidden_size, int64_t vocab,
                       int64_t index_base, void* logits_out, int64_t logits_stride, int32_t* out_ids, int64_t* out_keys,
                       unsigned long long* keys, unsigned int* ticket, cudaStream_t s) {
  if (rows < 2 || rows > 64) { set_error("lm_head_argmax (tensor cores): 2 to 64 rows per pass"); return B2_ERR_INVALID; }
  const int n = rows <= 16 ? 16 : rows <= 32 ? 32 : 64;
  CUtensorMap hidden_map;
  CUtensorMap m128, m32;
  if (!make_map(&hidden_map, hidden, rows, hidden_size, n) || !make_map(&m128, table, vocab, hidden_size, 128) ||
      !make_map(&m32, table, vocab, hidden_size, 32)) {
    set_error("lm_head_argmax (tensor cores): cuTensorMapEncodeTiled refused the hidden rows");
    return B2_ERR_CUDA;
  }
  MmaArgs args{};
  args.vocab = vocab;
  args.index_base = index_base;
  args.rows = int(rows);
  args.slabs = int(hidden_size / kSlabK);
  args.units = int((vocab + kUnitRows - 1) / kUnitRows);
  args.logits = static_cast<__half*>(logits_out);
  args.logits_stride = logits_stride;
  args.out_ids = out_ids;
  args.out_keys = out_keys;
  args.keys = keys;
  args.ticket = ticket;
  switch (n) {
    case 16: return launch_pick<16>(hidden_map, m128, m32, args, s);
    case 32: return launch_pick<32>(hidden_map, m128, m32, args, s);
    default: return launch_pick<64>(hidden_map, m128, m32, args, s);
  }
}

}  // namespace b2
