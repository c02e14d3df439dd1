// The whole-row route of the sampler: one 64-bit key per token, a bitonic network over the whole row (keys in
// registers, 4096-key tiles, wider steps in global memory), the ordered sums and the pick -- and the sequence of
// launches that strings them together.  A header, because two translation units hold these kernels: sampler.cu
// launches them from the host (every row, and the head tile of the top-p route), sampler_fallback.cu launches its
// own copies from the device for the rows the top-p route hands back (device-side launches need relocatable
// device code, which costs registers in every kernel of its translation unit: the hot kernels stay out of it).
#pragma once
#include "common.cuh"
#include "b2ops.h"

#include <cfloat>

namespace b2 {
namespace {


constexpr int kTile = 4096;          // keys per thread block in the shared-memory sorting steps
constexpr int kSortThreads = 1024;   // small sorts in shared memory: many warps hide the dependent load-compare-store chain
constexpr int kChunk = 2048;         // tokens per step of the ordered sums
constexpr int kSelectThreads = 256;

// larger score -> larger key; among equal scores the lower index -> larger key
__device__ __forceinline__ unsigned long long sample_key(float score, uint32_t index) {
  const uint32_t b = __float_as_uint(score);
  const uint32_t ordered = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
  return (static_cast<unsigned long long>(ordered) << 32) | (0xffffffffu - index);
}
__device__ __forceinline__ float key_score(unsigned long long key) {
  const uint32_t o = uint32_t(key >> 32);
  return __uint_as_float((o & 0x80000000u) ? (o & 0x7fffffffu) : ~o);
}
__device__ __forceinline__ int32_t key_index(unsigned long long key) { return int32_t(0xffffffffu - uint32_t(key)); }

// The rows a kernel of the whole-row sort works on.  list == nullptr: every row, one per block of the grid's row
// dimension.  Otherwise the first *count entries of list (the rows that the top-p path could not settle), dealt over a
// row dimension of a few blocks.  Such launches are made from the device, and only when the list is not empty.
struct RowSet { const int* list; const int* count; };
__device__ __forceinline__ bool row_of(const RowSet& rs, int64_t it, int64_t grid_rows, int64_t* row) {
  if (rs.list == nullptr) { *row = it; return it < grid_rows; }
  if (it >= int64_t(*rs.count)) return false;
  *row = rs.list[it];
  return true;
}
constexpr int kListedRowBlocks = 16;   // at most this many blocks in the row dimension of a launch over a row list

// keys[r][i] for i < padded: the token's key, or 0 (below every real key) in the padding
template <typename T>
__global__ void __launch_bounds__(256)
sampler_keys_kernel(const T* logits, int64_t width, int64_t row_stride, int64_t padded, float temperature,
                    unsigned long long* keys, const RowSet rs) {
  dependent_launch_prologue();
  int64_t row;
  for (int64_t it = blockIdx.y; row_of(rs, it, gridDim.y, &row); it += gridDim.y) {
    const T* src = logits + row * row_stride;
    unsigned long long* dst = keys + row * padded;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < padded; i += int64_t(gridDim.x) * blockDim.x)
      dst[i] = i < width ? sample_key(__fdiv_rn(Elem<T>::load(src + i), temperature), uint32_t(i)) : 0ull;
  }
}

// ---- bitonic network, descending.  Element i and its partner i ^ j are put in descending order when
// (i & k) == 0 and in ascending order otherwise; after the step k == n the row is descending.
__device__ __forceinline__ void compare_exchange(unsigned long long& a, unsigned long long& b, bool descending) {
  if ((a < b) == descending) { const unsigned long long t = a; a = b; b = t; }
}

// All steps that stay inside a tile: k from k_first up to k_last with every j < kTile.  With k_first == 2
// this sorts the tile from scratch; with k_first == k_last it finishes a merge whose wide steps ran in
// global memory.
__global__ void __launch_bounds__(kSortThreads)
bitonic_tile_kernel(unsigned long long* keys, int64_t padded, int tile, int64_t k_first, int64_t k_last, const RowSet rs) {
  dependent_launch_prologue();
  extern __shared__ unsigned long long tile_keys[];
  int64_t row;
  for (int64_t it = blockIdx.y; row_of(rs, it, gridDim.y, &row); it += gridDim.y) {
  unsigned long long* base = keys + row * padded + int64_t(blockIdx.x) * tile;
  const int64_t global0 = int64_t(blockIdx.x) * tile;
  for (int i = threadIdx.x; i < tile; i += kSortThreads) tile_keys[i] = base[i];
  __syncthreads();
  for (int64_t k = k_first; k <= k_last; k <<= 1) {
    for (int j = int(k >> 1 < tile ? k >> 1 : tile >> 1); j > 0; j >>= 1) {
      for (int p = threadIdx.x; p < tile / 2; p += kSortThreads) {
        const int i = ((p & ~(j - 1)) << 1) | (p & (j - 1));   // the lower element of pair p
        const bool descending = ((global0 + i) & k) == 0;
        compare_exchange(tile_keys[i], tile_keys[i | j], descending);
      }
      __syncthreads();
    }
  }
  for (int i = threadIdx.x; i < tile; i += kSortThreads) base[i] = tile_keys[i];
  __syncthreads();   // the tile is reused for the block's next row
  }
}

// One step with j >= tile: partners sit in different tiles, so it runs in global memory (the keys of a
// few hundred rows fit the L2).
__global__ void __launch_bounds__(256)
bitonic_wide_kernel(unsigned long long* keys, int64_t padded, int64_t k, int64_t j, const RowSet rs) {
  dependent_launch_prologue();
  int64_t row;
  for (int64_t it = blockIdx.y; row_of(rs, it, gridDim.y, &row); it += gridDim.y) {
    unsigned long long* base = keys + row * padded;
    for (int64_t p = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; p < padded / 2; p += int64_t(gridDim.x) * blockDim.x) {
      const int64_t i = ((p & ~(j - 1)) << 1) | (p & (j - 1));
      unsigned long long a = base[i], b = base[i | j];
      const bool descending = (i & k) == 0;
      if ((a < b) == descending) { base[i] = b; base[i | j] = a; }
    }
  }
}

// ---- the same network for full 4096-key tiles, with the keys in registers.  The shared-memory kernel above
// moves every key through shared memory at every step (its bandwidth is what that kernel is bound by); here a
// thread keeps 16 keys in registers and a step costs shared memory only when the partner is in another warp:
//   layout B  thread t holds elements 16t .. 16t+15   steps j = 1..8 in registers, j = 16..256 by warp shuffles
//   layout S  thread t holds elements t, t+256, ...   steps j = 512..2048 in registers
// and two transposes through (swizzled) shared memory per phase that has steps of both kinds.
constexpr int kRegKeys = 16, kRegThreads = kTile / kRegKeys;   // 256 threads per 4096-key tile

__device__ __forceinline__ int swizzled(int e) { return e ^ ((e >> 4) & 15); }   // 64-bit accesses of either layout hit 16 banks pairs

__device__ __forceinline__ void steps_in_registers_b(unsigned long long (&key)[kRegKeys], int64_t first_global, int64_t k,
                                                     int j_from) {
#pragma unroll
  for (int j = 8; j >= 1; j >>= 1) {
    if (j > j_from) continue;
#pragma unroll
    for (int r = 0; r < kRegKeys; ++r)
      if ((r & j) == 0) compare_exchange(key[r], key[r | j], ((first_global + r) & k) == 0);
  }
}

__device__ __forceinline__ void steps_by_shuffle_b(unsigned long long (&key)[kRegKeys], int64_t first_global, int64_t k,
                                                   int j_from, int lane) {
  for (int j = j_from; j >= 16; j >>= 1) {
    const int m = j >> 4;
    const bool lower = (lane & m) == 0;
#pragma unroll
    for (int r = 0; r < kRegKeys; ++r) {
      const unsigned long long other = __shfl_xor_sync(0xffffffffu, key[r], m);
      const bool descending = ((first_global + r) & k) == 0;
      const bool keep_larger = lower == descending;
      key[r] = (key[r] < other) == keep_larger ? other : key[r];
    }
  }
}

// layout S: element of register r is r * 256 + t; steps j = 2048, 1024, 512 (those <= j_from)
__device__ __forceinline__ void steps_in_registers_s(unsigned long long (&key)[kRegKeys], int64_t tile_global, int t, int64_t k,
                                                     int j_from) {
#pragma unroll
  for (int m = 8; m >= 2; m >>= 1) {
    if (m * kRegThreads > j_from) continue;
#pragma unroll
    for (int r = 0; r < kRegKeys; ++r)
      if ((r & m) == 0) compare_exchange(key[r], key[r | m], ((tile_global + r * kRegThreads + t) & k) == 0);
  }
}

__device__ __forceinline__ void layout_b_to_s(unsigned long long (&key)[kRegKeys], unsigned long long* tile, int t) {
#pragma unroll
  for (int r = 0; r < kRegKeys; ++r) tile[swizzled(t * kRegKeys + r)] = key[r];
  __syncthreads();
#pragma unroll
  for (int r = 0; r < kRegKeys; ++r) key[r] = tile[swizzled(r * kRegThreads + t)];
  __syncthreads();
}
__device__ __forceinline__ void layout_s_to_b(unsigned long long (&key)[kRegKeys], unsigned long long* tile, int t) {
#pragma unroll
  for (int r = 0; r < kRegKeys; ++r) tile[swizzled(r * kRegThreads + t)] = key[r];
  __syncthreads();
#pragma unroll
  for (int r = 0; r < kRegKeys; ++r) key[r] = tile[swizzled(t * kRegKeys + r)];
  __syncthreads();
}

// k_first == 2: sorts every 4096-key tile from scratch (phases 2 .. 4096).  k_first == k_last > 4096: the steps
// j = 2048 .. 1 that finish a merge whose wide steps ran in global memory.
__global__ void __launch_bounds__(kRegThreads)
bitonic_tile_registers_kernel(unsigned long long* keys, int64_t padded, int64_t k_first, int64_t k_last, const RowSet rs) {
  dependent_launch_prologue();
  __shared__ unsigned long long tile[kTile];
  const int64_t tile_global = int64_t(blockIdx.x) * kTile;
  int64_t row;
  for (int64_t it = blockIdx.y; row_of(rs, it, gridDim.y, &row); it += gridDim.y) {
  unsigned long long* base = keys + row * padded + tile_global;
  const int t = threadIdx.x, lane = t & 31;
  const int64_t first_global = tile_global + int64_t(t) * kRegKeys;   // layout B: global index of register 0
  unsigned long long key[kRegKeys];
  // global memory is always read and written in layout S: a warp's 32 lanes touch 256 consecutive bytes
#pragma unroll
  for (int r = 0; r < kRegKeys; ++r) key[r] = base[r * kRegThreads + t];
  if (k_first > kTile) {
    steps_in_registers_s(key, tile_global, t, k_first, kTile / 2);
    layout_s_to_b(key, tile, t);
    steps_by_shuffle_b(key, first_global, k_first, 256, lane);
    steps_in_registers_b(key, first_global, k_first, 8);
  } else {
    layout_s_to_b(key, tile, t);
    for (int64_t k = k_first; k <= k_last; k <<= 1) {
      const int top = int(k >> 1);
      if (top >= 512) {
        layout_b_to_s(key, tile, t);
        steps_in_registers_s(key, tile_global, t, k, top);
        layout_s_to_b(key, tile, t);
      }
      if (top >= 16) steps_by_shuffle_b(key, first_global, k, top < 256 ? top : 256, lane);
      steps_in_registers_b(key, first_global, k, top < 8 ? top : 8);
    }
  }
  layout_b_to_s(key, tile, t);
#pragma unroll
  for (int r = 0; r < kRegKeys; ++r) base[r * kRegThreads + t] = key[r];
  }
}

// Two wide steps (j and j/2, both >= the tile) in one pass over global memory: the four elements that the two
// steps connect are loaded once.
__global__ void __launch_bounds__(256)
bitonic_wide_pair_kernel(unsigned long long* keys, int64_t padded, int64_t k, int64_t j, const RowSet rs) {
  dependent_launch_prologue();
  const int64_t h = j >> 1;
  int64_t row;
  for (int64_t it = blockIdx.y; row_of(rs, it, gridDim.y, &row); it += gridDim.y) {
  unsigned long long* base = keys + row * padded;
  for (int64_t q = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; q < padded / 4; q += int64_t(gridDim.x) * blockDim.x) {
    const int64_t i = ((q & ~(h - 1)) << 2) | (q & (h - 1));   // bits j and j/2 clear
    unsigned long long a0 = base[i], a1 = base[i + h], a2 = base[i + j], a3 = base[i + j + h];
    const bool descending = (i & k) == 0;
    compare_exchange(a0, a2, descending);
    compare_exchange(a1, a3, descending);
    compare_exchange(a0, a1, descending);
    compare_exchange(a2, a3, descending);
    base[i] = a0; base[i + h] = a1; base[i + j] = a2; base[i + j + h] = a3;
  }
  }
}

// Running sums of stage[0 .. n) in index order, one thread: sum_j = sum_(j-1) + stage[j], written back in place.
// The additions form one dependent chain (that is the reference's order); the loads and stores around them do not, so
// they go eight at a time: a loop that loads, adds and stores one element per turn waits for shared memory every turn.
// stage must be 16-byte aligned.
__device__ __forceinline__ float running_sums_in_order(float* stage, int n, float sum) {
  int j = 0;
  for (; j + 8 <= n; j += 8) {
    float4 a = *reinterpret_cast<const float4*>(stage + j), b = *reinterpret_cast<const float4*>(stage + j + 4);
    sum += a.x; a.x = sum; sum += a.y; a.y = sum; sum += a.z; a.z = sum; sum += a.w; a.w = sum;
    sum += b.x; b.x = sum; sum += b.y; b.y = sum; sum += b.z; b.z = sum; sum += b.w; b.w = sum;
    *reinterpret_cast<float4*>(stage + j) = a;
    *reinterpret_cast<float4*>(stage + j + 4) = b;
  }
  for (; j < n; ++j) { sum += stage[j]; stage[j] = sum; }
  return sum;
}

// ---- the ordered sums and the pick (reference src/ops_cuda.cu:587-617, same operations in the same order)
__device__ __forceinline__ unsigned long long sampler_hash(unsigned long long x) {
  x += 0x9e3779b97f4a7c15ULL;
  x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ULL;
  x = (x ^ (x >> 27)) * 0x94d049bb133111ebULL;
  return x ^ (x >> 31);
}

__global__ void __launch_bounds__(kSelectThreads)
sampler_pick_kernel(const unsigned long long* keys, int64_t width, int64_t padded, int top_k, float top_p,
                    unsigned long long seed, const unsigned long long* draw_offsets, float* running, int32_t* out_ids,
                    const RowSet rs) {
  dependent_launch_prologue();
  __shared__ float stage[kChunk];
  __shared__ float carry;
  __shared__ int found;
  int64_t row;
  for (int64_t it = blockIdx.x; row_of(rs, it, gridDim.x, &row); it += gridDim.x) {
  const unsigned long long* sorted = keys + row * padded;
  float* cum = running + row * padded;
  const int64_t limit = top_k == 0 ? width : (int64_t(top_k) < width ? int64_t(top_k) : width);
  const float maximum = key_score(sorted[0]);
  const int tid = threadIdx.x;

  // running sums cum[i] = e_0 + ... + e_i, added in order by one thread.  The terms come in descending order, so
  // once adding the smallest term seen so far no longer changes the fp32 sum, no later term can (rounding is
  // monotonic): from there on every running sum equals the current one, exactly as the serial walk would find,
  // and the rest of the row is filled in parallel.
  __shared__ int frozen;
  if (tid == 0) { carry = 0.0f; frozen = 0; }
  __syncthreads();
  for (int64_t base = 0; base < limit; base += kChunk) {
    const int n = int(limit - base < kChunk ? limit - base : kChunk);
    if (frozen) {
      const float settled = carry;
      for (int j = tid; j < n; j += kSelectThreads) cum[base + j] = settled;
      continue;                                   // `frozen` and `carry` no longer change: no barrier needed
    }
    for (int j = tid; j < n; j += kSelectThreads) stage[j] = expf(key_score(sorted[base + j]) - maximum);
    __syncthreads();
    if (tid == 0) {
      float sum = carry, term = 0.0f;
      for (int j = 0; j < n; ++j) { term = stage[j]; sum += term; stage[j] = sum; }
      carry = sum;
      if (sum + term == sum) frozen = 1;
    }
    __syncthreads();
    for (int j = tid; j < n; j += kSelectThreads) cum[base + j] = stage[j];
    __syncthreads();
  }
  const float total = carry;
  __syncthreads();   // everyone has read the total before thread 0 reuses `carry`

  // top-p: the shortest prefix whose normalised mass, added term by term, reaches top_p.  The same argument ends
  // the walk early: once the smallest quotient seen so far no longer moves the running mass, it stays below top_p
  // for good and the prefix is everything, as the serial walk would conclude after visiting every token.
  int64_t prefix = limit;
  if (top_p < 1.0f) {
    if (tid == 0) { carry = 0.0f; found = -1; frozen = 0; }
    __syncthreads();
    for (int64_t base = 0; base < limit; base += kChunk) {
      const int n = int(limit - base < kChunk ? limit - base : kChunk);
      for (int j = tid; j < n; j += kSelectThreads)
        stage[j] = __fdiv_rn(expf(key_score(sorted[base + j]) - maximum), total);
      __syncthreads();
      if (tid == 0) {
        float cumulative = carry, term = 0.0f;
        for (int j = 0; j < n; ++j) {
          term = stage[j];
          cumulative += term;
          if (cumulative >= top_p) { found = j; break; }
        }
        carry = cumulative;
        if (found < 0 && cumulative + term == cumulative) frozen = 1;
      }
      __syncthreads();
      if (found >= 0) { prefix = base + found + 1; break; }
      if (frozen) break;
    }
  }
  __syncthreads();

  const float prefix_total = cum[prefix - 1];
  const unsigned long long offset = draw_offsets != nullptr ? draw_offsets[row] : 0ull;
  const unsigned long long bits = sampler_hash(seed ^ (offset * 0xd1342543de82ef95ULL));
  const float u = (static_cast<float>((bits >> 11) & 0x1fffffffffffffULL) + 0.5f) / 9007199254740992.0f;
  const float target = u * prefix_total;
  // first i < prefix with target < cum[i]; the sums never decrease, so the lowest such i over all threads
  __shared__ unsigned long long best;
  if (tid == 0) best = static_cast<unsigned long long>(prefix - 1);
  __syncthreads();
  unsigned long long mine = static_cast<unsigned long long>(prefix - 1);
  for (int64_t i = tid; i < prefix; i += kSelectThreads)
    if (target < cum[i]) { mine = static_cast<unsigned long long>(i); break; }
  atomicMin(&best, mine);
  __syncthreads();
  if (tid == 0) out_ids[row] = key_index(sorted[best]);
  __syncthreads();   // the shared variables serve the block's next row
  }
}

// ---- the whole-row route as one sequence of launches, made from the host (every row) or from the device (the
// rows the top-p route handed back: launched by the kernel that lists them, and only if there are any, so that a
// call whose rows were all settled pays for one tiny kernel instead of two dozen idle ones)
struct ChainArgs {
  const void* logits;
  int dtype;
  int64_t width, row_stride, padded;
  float temperature;
  int top_k;
  float top_p;
  unsigned long long seed;
  const unsigned long long* draw_offsets;
  unsigned long long* keys;
  float* running;
  int32_t* out_ids;
};

#ifdef B2_DEVICE_CHAIN
#define B2_CHAIN_FN __host__ __device__
#else
#define B2_CHAIN_FN
#endif
#if defined(__CUDA_ARCH__) && defined(B2_DEVICE_CHAIN)
#define B2_CHAIN_LAUNCH(kernel, grid, block, smem, ...) kernel<<<grid, block, smem, cudaStreamTailLaunch>>>(__VA_ARGS__)
#else
#define B2_CHAIN_LAUNCH(kernel, grid, block, smem, ...) launch_kernel(kernel, grid, block, smem, s, __VA_ARGS__)
#endif

B2_CHAIN_FN inline void whole_row_chain(const ChainArgs& a, RowSet todo, unsigned row_blocks, cudaStream_t s) {
  (void)s;
  const int64_t padded = a.padded;
  // the whole-row sort has little per-block overhead: many small blocks
  const dim3 wide_grid(unsigned(padded / 256 < 1 ? 1 : (padded / 256 > 296 ? 296 : padded / 256)), row_blocks);
  if (a.dtype == B2_F32)
    B2_CHAIN_LAUNCH(sampler_keys_kernel<float>, wide_grid, dim3(256), 0, static_cast<const float*>(a.logits), a.width, a.row_stride,
                    padded, a.temperature, a.keys, todo);
  else
    B2_CHAIN_LAUNCH(sampler_keys_kernel<__half>, wide_grid, dim3(256), 0, static_cast<const __half*>(a.logits), a.width, a.row_stride,
                    padded, a.temperature, a.keys, todo);
  const int tile = int(padded < kTile ? padded : kTile);
  const dim3 tile_grid(unsigned(padded / tile), row_blocks);
  if (tile < kTile) {
    B2_CHAIN_LAUNCH(bitonic_tile_kernel, tile_grid, dim3(kSortThreads), size_t(tile) * 8, a.keys, padded, tile, 2, tile, todo);   // the whole row is one small tile
  } else {
    B2_CHAIN_LAUNCH(bitonic_tile_registers_kernel, tile_grid, dim3(kRegThreads), 0, a.keys, padded, int64_t(2), int64_t(kTile), todo);
    for (int64_t k = int64_t(kTile) * 2; k <= padded; k <<= 1) {
      int64_t j = k >> 1;
      for (; j >= 2 * kTile; j >>= 2) B2_CHAIN_LAUNCH(bitonic_wide_pair_kernel, wide_grid, dim3(256), 0, a.keys, padded, k, j, todo);   // steps j and j/2
      if (j >= kTile) B2_CHAIN_LAUNCH(bitonic_wide_kernel, wide_grid, dim3(256), 0, a.keys, padded, k, j, todo);                   // one step left over
      B2_CHAIN_LAUNCH(bitonic_tile_registers_kernel, tile_grid, dim3(kRegThreads), 0, a.keys, padded, k, k, todo);
    }
  }
  B2_CHAIN_LAUNCH(sampler_pick_kernel, dim3(row_blocks), dim3(kSelectThreads), 0, a.keys, a.width, padded, a.top_k, a.top_p, a.seed,
                  a.draw_offsets, a.running, a.out_ids, todo);
}

}  // namespace
}  // namespace b2
