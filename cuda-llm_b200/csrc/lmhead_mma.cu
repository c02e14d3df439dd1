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
// kernel is bound by HBM like the rest of this library and everything is arranged around keeping the
// copy engine busy:
//   D[128 table rows, N hidden rows] += A[128, 64] * B[N, 64]^T per 64-wide slab of H, both operands
//   K-major (the row-major tensors as they lie in memory), N = rows padded to 16 / 32 / 64.
//   warp 0      one lane issues the TMA tile copies (cp.async.bulk.tensor, 128-byte swizzle, no multicast):
//               a 128 x 64 tile of the table and the N x 64 tile of the hidden rows per slab, into a ring of
//               shared-memory stages, each completed through an mbarrier
//   warp 1      one lane issues tcgen05.mma (four K = 16 steps per slab) into one of two accumulators in
//               tensor memory, and tcgen05.commit to hand a stage back or an accumulator on
//   warps 2-5   read the finished accumulator with tcgen05.ld (one table row per thread, N columns), round
//               to fp16 as the stored logit would be, keep a running (best value, row) per hidden row in
//               registers -- rows only grow per thread, so "strictly greater" is the reference's rule
//               (src/ops_cuda.cu:562) -- and write the logits only when the caller wants them
//   at the end  the 128 threads' candidates meet in shared memory, one thread per hidden row folds them and
//               merges the block's winner into the packed (value, index) key of b2_argmax_keys with one
//               atomicMax; the last block (ticket) publishes ids / keys and re-zeroes the scratch.
// The hidden tile comes from L2 every slab (N * 128 bytes beside the table's 16 KB): no HBM traffic.
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
constexpr int kMmaThreads = 192;
constexpr int kEpilogueThreads = 128;
constexpr uint32_t kTableTileBytes = kTileRows * kSlabK * 2;   // 16 KB
constexpr int kMaxStages = 12;
constexpr unsigned long long kPoison = ~0ull;  // a key no real candidate can reach: "this call failed"
constexpr unsigned long long kSign = 0x8000000000000000ull;

__device__ __forceinline__ unsigned long long pack_candidate(float v, uint32_t global_index) {
  const uint32_t b = __float_as_uint(v);
  const uint32_t ordered = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
  return (static_cast<unsigned long long>(ordered) << 32) | (0xffffffffu - global_index);
}

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
// eight rows (what a TMA copy with 128-byte swizzle writes): start address, leading offset 1 (unused with
// swizzling), 1024 bytes between row groups, descriptor version 1, layout "128-byte swizzle".
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
  int stages;
  int tiles;             // ceil(vocab / 128)
  __half* logits;        // may be null
  int64_t logits_stride;
  int32_t* out_ids;      // may be null
  int64_t* out_keys;     // may be null
  unsigned long long* keys;
  unsigned int* ticket;
};

template <int N>
__global__ void __launch_bounds__(kMmaThreads, 1)
lm_head_mma_kernel(const __grid_constant__ CUtensorMap table_map, const __grid_constant__ CUtensorMap hidden_map,
                   const MmaArgs args) {
  constexpr uint32_t kHiddenTileBytes = N * kSlabK * 2;
  constexpr uint32_t kStageBytes = kTableTileBytes + kHiddenTileBytes;
  constexpr uint32_t kAccumulatorColumns = 2 * N < 32 ? 32 : 2 * N;   // two accumulators; a power of two >= 32
  extern __shared__ unsigned char raw_smem[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~uintptr_t(1023));
  __shared__ __align__(8) uint64_t full_bar[kMaxStages], empty_bar[kMaxStages], acc_full_bar[2], acc_empty_bar[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int stop_flag;
  __shared__ int last_block;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int stages = args.stages, slabs = args.slabs;
  volatile int* stop = &stop_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) { mbarrier_init(&full_bar[s], 1); mbarrier_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbarrier_init(&acc_full_bar[b], 1); mbarrier_init(&acc_empty_bar[b], kEpilogueThreads); }
    stop_flag = 0;
  }
  if (warp == 1) tmem_alloc(&tmem_base_slot, kAccumulatorColumns);
  tensor_fence_before_sync();
  __syncthreads();
  tensor_fence_after_sync();
  const uint32_t tmem_base = tmem_base_slot;

  // running best of this thread's table rows, per hidden row (epilogue threads only)
  float best_v[N];
  int best_i[N];
#pragma unroll
  for (int c = 0; c < N; ++c) { best_v[c] = -FLT_MAX; best_i[c] = INT_MAX; }

  if (warp == 0) {
    // ---- copies: the ring is refilled as soon as the tensor cores have read a stage
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int tile = blockIdx.x; tile < args.tiles && *stop == 0; tile += gridDim.x) {
        for (int slab = 0; slab < slabs; ++slab) {
          if (!wait_or_stop(&empty_bar[stage], phase ^ 1u, stop)) break;
          unsigned char* dst = smem + size_t(stage) * kStageBytes;
          mbarrier_expect_bytes(&full_bar[stage], kStageBytes);
          tma_load_2d(dst, &table_map, slab * kSlabK, tile * kTileRows, &full_bar[stage]);
          tma_load_2d(dst + kTableTileBytes, &hidden_map, slab * kSlabK, 0, &full_bar[stage]);
          if (++stage == stages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ---- tensor cores
    if (lane == 0) {
      constexpr uint32_t idesc = instruction_descriptor(N);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      for (int tile = blockIdx.x; tile < args.tiles && *stop == 0; tile += gridDim.x, ++local) {
        const int buf = local & 1;
        if (!wait_or_stop(&acc_empty_bar[buf], ((local >> 1) & 1u) ^ 1u, stop)) break;
        tensor_fence_after_sync();
        const uint32_t d_tmem = tmem_base + uint32_t(buf * N);
        bool ok = true;
        for (int slab = 0; slab < slabs; ++slab) {
          if (!wait_or_stop(&full_bar[stage], phase, stop)) { ok = false; break; }
          tensor_fence_after_sync();
          const unsigned char* a = smem + size_t(stage) * kStageBytes;
          const uint64_t a_desc = k_major_sw128_descriptor(a), b_desc = k_major_sw128_descriptor(a + kTableTileBytes);
#pragma unroll
          for (int k = 0; k < kSlabK / kUmmaK; ++k)   // 32 bytes further along the swizzled row per step
            umma_f16(d_tmem, a_desc + uint64_t(k * 2), b_desc + uint64_t(k * 2), idesc, slab > 0 || k > 0);
          umma_commit(&empty_bar[stage]);
          if (++stage == stages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit(&acc_full_bar[buf]);
      }
    }
  } else {
    // ---- epilogue: thread = one table row of the tile = one lane of tensor memory
    const int quarter = warp & 3;                       // the 32 lanes this warp may read
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_address = uint32_t(quarter * 32) << 16;
    int local = 0;
    for (int tile = blockIdx.x; tile < args.tiles; tile += gridDim.x, ++local) {
      const int buf = local & 1;
      if (*stop != 0 || !wait_or_stop(&acc_full_bar[buf], (local >> 1) & 1u, stop)) break;
      tensor_fence_after_sync();
      const int64_t table_row = int64_t(tile) * kTileRows + row_in_tile;
      const bool exists = table_row < args.vocab;
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
          const float v = __half2float(stored);
          if (exists && v > best_v[r]) { best_v[r] = v; best_i[r] = int(table_row); }
          if (args.logits != nullptr && exists && r < args.rows) args.logits[int64_t(r) * args.logits_stride + table_row] = stored;
        }
      }
    }
  }

  // ---- every role has left its loop: nothing is in flight in a healthy run
  tensor_fence_before_sync();
  __syncthreads();
  tensor_fence_after_sync();
  const bool failed = stop_flag != 0;
  if (failed && threadIdx.x == 0) {
    // copies that were requested may still be landing: they must not outlive this block's shared memory
    for (int s = 0; s < stages; ++s) { mbarrier_wait_bounded(&full_bar[s], 0u); mbarrier_wait_bounded(&full_bar[s], 1u); }
  }
  if (warp == 1) tmem_free(tmem_base, kAccumulatorColumns);

  // ---- fold the 128 threads' candidates per hidden row (the ring's memory is free now)
  float* cand_v = reinterpret_cast<float*>(smem);
  int* cand_i = reinterpret_cast<int*>(smem + size_t(kEpilogueThreads) * N * sizeof(float));
  if (warp >= 2) {
    const int t = (warp & 3) * 32 + lane;
#pragma unroll
    for (int c = 0; c < N; ++c) { cand_v[c * kEpilogueThreads + t] = best_v[c]; cand_i[c * kEpilogueThreads + t] = best_i[c]; }
  }
  __syncthreads();
  if (threadIdx.x < args.rows) {
    const int r = threadIdx.x;
    float bv = -FLT_MAX;
    int bi = INT_MAX;
    for (int t = 0; t < kEpilogueThreads; ++t) {
      const float v = cand_v[r * kEpilogueThreads + t];
      const int i = cand_i[r * kEpilogueThreads + t];
      if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
    if (failed) atomicMax(args.keys + r, kPoison);
    else if (bi != INT_MAX) atomicMax(args.keys + r, pack_candidate(bv, uint32_t(args.index_base + bi)));
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
  if (r == 0) *args.ticket = 0u;
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

template <int N>
int launch_n(const CUtensorMap& table_map, const CUtensorMap& hidden_map, MmaArgs args, cudaStream_t s) {
  constexpr size_t stage_bytes = kTableTileBytes + size_t(N) * kSlabK * 2;
  constexpr size_t budget = 227 * 1024 - 1024 - 2048;      // alignment slack, static shared memory
  int stages = int(budget / stage_bytes);
  if (stages > kMaxStages) stages = kMaxStages;
  args.stages = stages;
  const size_t smem = size_t(stages) * stage_bytes + 1024;
  auto kernel = lm_head_mma_kernel<N>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess)
    return launch_status("lm_head_argmax (tensor cores, shared-memory attribute)");
  int grid = sm_count();
  if (grid > args.tiles) grid = args.tiles;
  kernel<<<grid, kMmaThreads, smem, s>>>(table_map, hidden_map, args);
  return launch_status("lm_head_argmax (tensor cores)");
}

}  // namespace

// True when the tensor-core kernel takes this call: fp16, a hidden size in whole 64-element slabs, 16-byte aligned
// tensors, and tables small enough for 32-bit tile coordinates.
bool lm_head_mma_supported(const void* hidden, const void* table, int64_t hidden_size, int64_t vocab) {
  return hidden_size % kSlabK == 0 && hidden_size >= kSlabK && aligned16(hidden) && aligned16(table) &&
         vocab < (int64_t(1) << 31) - kTileRows && hidden_size < (int64_t(1) << 31) && tensor_map_encoder() != nullptr;
}

// One pass over the table for up to 64 hidden rows (fp16).  keys / ticket: the call's zeroed scratch (rows keys, one ticket).
int launch_lm_head_mma(const void* hidden, const void* table, int64_t rows, int64_t hidden_size, int64_t vocab,
                       int64_t index_base, void* logits_out, int64_t logits_stride, int32_t* out_ids, int64_t* out_keys,
                       unsigned long long* keys, unsigned int* ticket, cudaStream_t s) {
  if (rows <= 0 || rows > 64) { set_error("lm_head_argmax (tensor cores): 1 to 64 rows per pass"); return B2_ERR_INVALID; }
  const int n = rows <= 16 ? 16 : rows <= 32 ? 32 : 64;
  CUtensorMap table_map, hidden_map;
  if (!make_map(&table_map, table, vocab, hidden_size, kTileRows) || !make_map(&hidden_map, hidden, rows, hidden_size, n)) {
    set_error("lm_head_argmax (tensor cores): cuTensorMapEncodeTiled refused the tensors");
    return B2_ERR_CUDA;
  }
  MmaArgs args{};
  args.vocab = vocab;
  args.index_base = index_base;
  args.rows = int(rows);
  args.slabs = int(hidden_size / kSlabK);
  args.tiles = int((vocab + kTileRows - 1) / kTileRows);
  args.logits = static_cast<__half*>(logits_out);
  args.logits_stride = logits_stride;
  args.out_ids = out_ids;
  args.out_keys = out_keys;
  args.keys = keys;
  args.ticket = ticket;
  switch (n) {
    case 16: return launch_n<16>(table_map, hidden_map, args, s);
    case 32: return launch_n<32>(table_map, hidden_map, args, s);
    default: return launch_n<64>(table_map, hidden_map, args, s);
  }
}

}  // namespace b2
