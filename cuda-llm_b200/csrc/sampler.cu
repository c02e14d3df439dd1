// Temperature / top-k / top-p sampling over vocabulary-wide logits for sm_100a, many rows per call.
//
// Replaces the non-greedy route of the reference's CudaSampler (src/ops_cuda.cu:575-617,910-936):
// sampler_fill + a library radix sort of the whole vocabulary + sampler_select, which walks the sorted
// scores up to four times with ONE thread, one blocking call per row.  The result here is the same
// token, bit for bit, because the same arithmetic is done in the same order:
//   score_i = logit_i / temperature (IEEE division); tokens ordered by score descending, equal scores
//   by ascending index; e_i = expf(score_i - score_0); fp32 running sums in that order.
// What changes is how the order and the sums are produced:
//   keys     one 64-bit key per token, (order-preserving bits of the score) << 32 | ~index, so one
//            unsigned sort gives the reference's order including its tie rule
//   sort     when 0 < top_k <= 2048 only the k largest keys matter: a radix select over the L2-resident
//            keys finds the k-th largest key, a compaction gathers the survivors and one thread block
//            sorts them in shared memory; otherwise a bitonic network sorts the whole row (4096-key
//            tiles in shared memory, wider steps in global memory), all rows at once
//   select   one thread block per row: the exponentials of a 2048-token chunk are computed in
//            parallel, one thread adds them in order (the only serial part left) and records the
//            running sums; the top-p cut walks the same way and stops at the crossing; the final pick
//            is a parallel search in the recorded sums.
#include "common.cuh"
#include "kernels.h"
#include "b2ops.h"

#include <cfloat>

namespace b2 {
namespace {

constexpr int kTile = 4096;          // keys per thread block in the shared-memory sorting steps
constexpr int kSortThreads = 512;    // 8 keys per thread
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

// keys[r][i] for i < padded: the token's key, or 0 (below every real key) in the padding
template <typename T>
__global__ void __launch_bounds__(256)
sampler_keys_kernel(const T* logits, int64_t width, int64_t row_stride, int64_t padded, float temperature,
                    unsigned long long* keys) {
  const int64_t row = blockIdx.y;
  const T* src = logits + row * row_stride;
  unsigned long long* dst = keys + row * padded;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < padded; i += int64_t(gridDim.x) * blockDim.x)
    dst[i] = i < width ? sample_key(__fdiv_rn(Elem<T>::load(src + i), temperature), uint32_t(i)) : 0ull;
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
bitonic_tile_kernel(unsigned long long* keys, int64_t padded, int tile, int64_t k_first, int64_t k_last) {
  extern __shared__ unsigned long long tile_keys[];
  const int64_t row = blockIdx.y;
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
}

// One step with j >= tile: partners sit in different tiles, so it runs in global memory (the keys of a
// few hundred rows fit the L2).
__global__ void __launch_bounds__(256)
bitonic_wide_kernel(unsigned long long* keys, int64_t padded, int64_t k, int64_t j) {
  const int64_t row = blockIdx.y;
  unsigned long long* base = keys + row * padded;
  for (int64_t p = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; p < padded / 2; p += int64_t(gridDim.x) * blockDim.x) {
    const int64_t i = ((p & ~(j - 1)) << 1) | (p & (j - 1));
    unsigned long long a = base[i], b = base[i | j];
    const bool descending = (i & k) == 0;
    if ((a < b) == descending) { base[i] = b; base[i | j] = a; }
  }
}

// ---- small top_k: radix select of the k-th largest key over all 64 bits (six digits of 11, 11, 11, 11,
// 11 and 9 bits, most significant first).  Keys are unique (they carry the token index), so "every key
// >= the k-th largest" is exactly k keys and the tie rule needs no special case.
constexpr int kSelectBins = 2048;
constexpr int kSelectRounds = 6;
constexpr int kMaxSelectK = 2048;

struct SelectState {                 // per row, in the workspace
  unsigned long long prefix;         // the digits fixed so far, in place
  unsigned int remaining;            // how many of the wanted k still lie inside the open bin
  unsigned int taken;                // compaction cursor
};

__global__ void select_init_kernel(SelectState* state, int64_t rows, unsigned int k) {
  const int64_t r = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (r < rows) { state[r].prefix = 0ull; state[r].remaining = k; state[r].taken = 0u; }
}

// Histogram of one digit over the keys whose higher digits equal the prefix found so far.
__global__ void __launch_bounds__(256)
select_histogram_kernel(const unsigned long long* keys, int64_t width, int64_t padded, int shift, int bits,
                        unsigned long long mask_above, const SelectState* state, unsigned int* histograms) {
  __shared__ unsigned int local[kSelectBins];
  const int64_t row = blockIdx.y;
  const int bins = 1 << bits;
  for (int b = threadIdx.x; b < bins; b += blockDim.x) local[b] = 0u;
  __syncthreads();
  const unsigned long long prefix = state[row].prefix;
  const unsigned long long* src = keys + row * padded;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < width; i += int64_t(gridDim.x) * blockDim.x) {
    const unsigned long long key = src[i];
    if ((key & mask_above) == prefix) atomicAdd(&local[unsigned(key >> shift) & unsigned(bins - 1)], 1u);
  }
  __syncthreads();
  unsigned int* out = histograms + row * kSelectBins;
  for (int b = threadIdx.x; b < bins; b += blockDim.x)
    if (local[b] != 0u) atomicAdd(&out[b], local[b]);
}

// Walks the histogram from the top bin down until the wanted count is covered: fixes the next digit of the
// prefix, updates what is still wanted from inside that bin, and clears the histogram for the next round.
__global__ void __launch_bounds__(256)
select_scan_kernel(int shift, int bits, SelectState* state, unsigned int* histograms) {
  __shared__ unsigned int counts[kSelectBins];
  const int64_t row = blockIdx.x;
  const int bins = 1 << bits;
  unsigned int* hist = histograms + row * kSelectBins;
  for (int b = threadIdx.x; b < bins; b += blockDim.x) { counts[b] = hist[b]; hist[b] = 0u; }
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned int want = state[row].remaining;
    unsigned long long digit = 0;
    for (int b = bins - 1; b >= 0; --b) {
      if (counts[b] >= want) { digit = static_cast<unsigned long long>(b); break; }
      want -= counts[b];
    }
    state[row].prefix |= digit << shift;
    state[row].remaining = want;
  }
}

// After the last round state.prefix IS the k-th largest key: gather every key >= it (exactly k of them).
__global__ void __launch_bounds__(256)
select_compact_kernel(const unsigned long long* keys, int64_t width, int64_t padded, SelectState* state,
                      unsigned long long* survivors) {
  const int64_t row = blockIdx.y;
  const unsigned long long* src = keys + row * padded;
  const unsigned long long cut = state[row].prefix;
  unsigned long long* out = survivors + row * int64_t(kMaxSelectK);
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < width; i += int64_t(gridDim.x) * blockDim.x) {
    const unsigned long long key = src[i];
    if (key >= cut) {
      const unsigned int slot = atomicAdd(&state[row].taken, 1u);
      if (slot < unsigned(kMaxSelectK)) out[slot] = key;
    }
  }
}

// Sorts one row's survivors in shared memory, descending, into the front of the row's key area.
__global__ void __launch_bounds__(kSortThreads)
select_finish_kernel(unsigned long long* keys, int64_t padded, int top_k, const unsigned long long* survivors) {
  __shared__ unsigned long long buf[kMaxSelectK];
  const int64_t row = blockIdx.x;
  const unsigned long long* in = survivors + row * int64_t(kMaxSelectK);
  int n = 1;
  while (n < top_k) n <<= 1;
  for (int i = threadIdx.x; i < n; i += kSortThreads) buf[i] = i < top_k ? in[i] : 0ull;
  __syncthreads();
  for (int k = 2; k <= n; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int p = threadIdx.x; p < n / 2; p += kSortThreads) {
        const int i = ((p & ~(j - 1)) << 1) | (p & (j - 1));
        compare_exchange(buf[i], buf[i | j], (i & k) == 0);
      }
      __syncthreads();
    }
  }
  unsigned long long* dst = keys + row * padded;
  for (int i = threadIdx.x; i < top_k; i += kSortThreads) dst[i] = buf[i];
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
                    unsigned long long seed, const unsigned long long* draw_offsets, float* running, int32_t* out_ids) {
  __shared__ float stage[kChunk];
  __shared__ float carry;
  __shared__ int found;
  const int64_t row = blockIdx.x;
  const unsigned long long* sorted = keys + row * padded;
  float* cum = running + row * padded;
  const int64_t limit = top_k == 0 ? width : (int64_t(top_k) < width ? int64_t(top_k) : width);
  const float maximum = key_score(sorted[0]);
  const int tid = threadIdx.x;

  // running sums cum[i] = e_0 + ... + e_i, added in order by one thread
  if (tid == 0) carry = 0.0f;
  for (int64_t base = 0; base < limit; base += kChunk) {
    const int n = int(limit - base < kChunk ? limit - base : kChunk);
    for (int j = tid; j < n; j += kSelectThreads) stage[j] = expf(key_score(sorted[base + j]) - maximum);
    __syncthreads();
    if (tid == 0) {
      float sum = carry;
      for (int j = 0; j < n; ++j) { sum += stage[j]; stage[j] = sum; }
      carry = sum;
    }
    __syncthreads();
    for (int j = tid; j < n; j += kSelectThreads) cum[base + j] = stage[j];
    __syncthreads();
  }
  const float total = carry;
  __syncthreads();   // everyone has read the total before thread 0 reuses `carry`

  // top-p: the shortest prefix whose normalised mass, added term by term, reaches top_p
  int64_t prefix = limit;
  if (top_p < 1.0f) {
    if (tid == 0) { carry = 0.0f; found = -1; }
    __syncthreads();
    for (int64_t base = 0; base < limit; base += kChunk) {
      const int n = int(limit - base < kChunk ? limit - base : kChunk);
      for (int j = tid; j < n; j += kSelectThreads)
        stage[j] = __fdiv_rn(expf(key_score(sorted[base + j]) - maximum), total);
      __syncthreads();
      if (tid == 0) {
        float cumulative = carry;
        for (int j = 0; j < n; ++j) {
          cumulative += stage[j];
          if (cumulative >= top_p) { found = j; break; }
        }
        carry = cumulative;
      }
      __syncthreads();
      if (found >= 0) { prefix = base + found + 1; break; }
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
}

int64_t padded_width(int64_t width) {
  int64_t p = 1;
  while (p < width) p <<= 1;
  return p;
}

}  // namespace

// per row: padded keys (8 B each), padded running sums (4 B each), the survivors of the top-k select,
// a histogram and a select state
size_t sampler_workspace_bytes(int64_t rows, int64_t width) {
  const int64_t padded = padded_width(width);
  const size_t per_row = size_t(padded) * 12 + size_t(kMaxSelectK) * 8 + size_t(kSelectBins) * 4 + sizeof(SelectState);
  return (size_t(rows) * per_row + 255) / 256 * 256;
}

int launch_sample_rows(const void* logits, int64_t rows, int64_t width, int64_t row_stride, int dtype, float temperature,
                       int top_k, float top_p, unsigned long long seed, const unsigned long long* draw_offsets,
                       int32_t* out_ids, void* workspace, cudaStream_t s) {
  if (rows == 0) return B2_OK;
  const int64_t padded = padded_width(width);
  auto* keys = static_cast<unsigned long long*>(workspace);
  auto* survivors = keys + rows * padded;
  auto* state = reinterpret_cast<SelectState*>(survivors + rows * int64_t(kMaxSelectK));
  auto* running = reinterpret_cast<float*>(state + rows);
  auto* histograms = reinterpret_cast<unsigned int*>(running + rows * padded);

  const unsigned spread = unsigned(padded / 256 < 1 ? 1 : (padded / 256 > 296 ? 296 : padded / 256));
  const dim3 row_grid(spread, unsigned(rows));
  if (dtype == B2_F32)
    sampler_keys_kernel<float><<<row_grid, 256, 0, s>>>(static_cast<const float*>(logits), width, row_stride, padded,
                                                       temperature, keys);
  else
    sampler_keys_kernel<__half><<<row_grid, 256, 0, s>>>(static_cast<const __half*>(logits), width, row_stride, padded,
                                                        temperature, keys);

  if (top_k > 0 && top_k <= kMaxSelectK && width > kTile) {
    // only the k largest keys matter: find the k-th largest, gather the survivors, sort those
    if (cudaMemsetAsync(histograms, 0, size_t(rows) * kSelectBins * 4, s) != cudaSuccess) return launch_status("sample_rows");
    select_init_kernel<<<unsigned((rows + 255) / 256), 256, 0, s>>>(state, rows, unsigned(top_k));
    const int shifts[kSelectRounds] = {53, 42, 31, 20, 9, 0}, widths[kSelectRounds] = {11, 11, 11, 11, 11, 9};
    unsigned long long mask_above = 0ull;
    for (int round = 0; round < kSelectRounds; ++round) {
      select_histogram_kernel<<<row_grid, 256, 0, s>>>(keys, width, padded, shifts[round], widths[round], mask_above, state,
                                                      histograms);
      select_scan_kernel<<<unsigned(rows), 256, 0, s>>>(shifts[round], widths[round], state, histograms);
      mask_above |= ((1ull << widths[round]) - 1ull) << shifts[round];
    }
    select_compact_kernel<<<row_grid, 256, 0, s>>>(keys, width, padded, state, survivors);
    select_finish_kernel<<<unsigned(rows), kSortThreads, 0, s>>>(keys, padded, top_k, survivors);
  } else {
    const int tile = int(padded < kTile ? padded : kTile);
    const dim3 tile_grid(unsigned(padded / tile), unsigned(rows));
    const size_t smem = size_t(tile) * 8;
    bitonic_tile_kernel<<<tile_grid, kSortThreads, smem, s>>>(keys, padded, tile, 2, tile);
    for (int64_t k = int64_t(tile) * 2; k <= padded; k <<= 1) {
      for (int64_t j = k >> 1; j >= tile; j >>= 1) bitonic_wide_kernel<<<row_grid, 256, 0, s>>>(keys, padded, k, j);
      bitonic_tile_kernel<<<tile_grid, kSortThreads, smem, s>>>(keys, padded, tile, k, k);
    }
  }
  sampler_pick_kernel<<<unsigned(rows), kSelectThreads, 0, s>>>(keys, width, padded, top_k, top_p, seed, draw_offsets, running,
                                                                out_ids);
  return launch_status("sample_rows");
}

}  // namespace b2
