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
//   sort     when 0 < top_k <= 2048 only the k largest keys matter: a threshold taken from a sorted sample of
//            the row, ONE pass over the logits that gathers the few hundred tokens above it, and a one-block
//            sort of those (checked; a call whose sample misled it is redone by a radix select over all 64
//            key bits, one more launch that otherwise returns at once); otherwise a bitonic network sorts the whole row (keys in registers, 4096-key tiles,
//            wider steps in global memory)
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
                    unsigned long long* keys, const int* only_rows) {
  const int64_t row = blockIdx.y;
  if (only_rows != nullptr && only_rows[row] == 0) return;   // this row was settled without the whole-row sort
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
bitonic_tile_kernel(unsigned long long* keys, int64_t padded, int tile, int64_t k_first, int64_t k_last, const int* only_rows) {
  extern __shared__ unsigned long long tile_keys[];
  const int64_t row = blockIdx.y;
  if (only_rows != nullptr && only_rows[row] == 0) return;
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
bitonic_wide_kernel(unsigned long long* keys, int64_t padded, int64_t k, int64_t j, const int* only_rows) {
  const int64_t row = blockIdx.y;
  if (only_rows != nullptr && only_rows[row] == 0) return;
  unsigned long long* base = keys + row * padded;
  for (int64_t p = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; p < padded / 2; p += int64_t(gridDim.x) * blockDim.x) {
    const int64_t i = ((p & ~(j - 1)) << 1) | (p & (j - 1));
    unsigned long long a = base[i], b = base[i | j];
    const bool descending = (i & k) == 0;
    if ((a < b) == descending) { base[i] = b; base[i | j] = a; }
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
bitonic_tile_registers_kernel(unsigned long long* keys, int64_t padded, int64_t k_first, int64_t k_last, const int* only_rows) {
  __shared__ unsigned long long tile[kTile];
  const int64_t row = blockIdx.y, tile_global = int64_t(blockIdx.x) * kTile;
  if (only_rows != nullptr && only_rows[row] == 0) return;
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

// Two wide steps (j and j/2, both >= the tile) in one pass over global memory: the four elements that the two
// steps connect are loaded once.
__global__ void __launch_bounds__(256)
bitonic_wide_pair_kernel(unsigned long long* keys, int64_t padded, int64_t k, int64_t j, const int* only_rows) {
  const int64_t row = blockIdx.y, h = j >> 1;
  if (only_rows != nullptr && only_rows[row] == 0) return;
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

// ---- small top_k, exact fallback: radix select of the k-th largest key over all 64 bits (six digits of 11, 11,
// 11, 11, 11 and 9 bits, most significant first), one thread block per row, in ONE launch that returns at once
// unless the sampled-threshold path below raised its flag.  Keys are recomputed from the logits in every pass
// (no key array); they are unique (they carry the token index), so "every key >= the k-th largest" is exactly k
// keys and the tie rule needs no special case.  Seven passes over the row by one thread block: slow, and rare.
constexpr int kSelectBins = 2048;
constexpr int kSelectRounds = 6;
constexpr int kMaxSelectK = 2048;
constexpr int kExactThreads = 1024;

template <typename T>
__global__ void __launch_bounds__(kExactThreads)
topk_exact_kernel(const T* logits, int64_t width, int64_t row_stride, int64_t padded, float temperature, int top_k,
                  unsigned long long* keys, const int* only_if) {
  __shared__ unsigned int counts[kSelectBins];
  __shared__ unsigned long long survivors[kMaxSelectK];
  __shared__ unsigned long long prefix_s;
  __shared__ unsigned int remaining_s, taken_s;
  if (*only_if == 0) return;
  const int64_t row = blockIdx.x;
  const T* src = logits + row * row_stride;
  const int tid = threadIdx.x;
  if (tid == 0) { prefix_s = 0ull; remaining_s = unsigned(top_k); taken_s = 0u; }
  const int shifts[kSelectRounds] = {53, 42, 31, 20, 9, 0}, widths[kSelectRounds] = {11, 11, 11, 11, 11, 9};
  unsigned long long mask_above = 0ull;
  for (int round = 0; round < kSelectRounds; ++round) {
    const int shift = shifts[round], bins = 1 << widths[round];
    for (int b = tid; b < bins; b += kExactThreads) counts[b] = 0u;
    __syncthreads();
    const unsigned long long prefix = prefix_s;
    for (int64_t i = tid; i < width; i += kExactThreads) {
      const unsigned long long key = sample_key(__fdiv_rn(Elem<T>::load(src + i), temperature), uint32_t(i));
      if ((key & mask_above) == prefix) atomicAdd(&counts[unsigned(key >> shift) & unsigned(bins - 1)], 1u);
    }
    __syncthreads();
    if (tid == 0) {   // from the top bin down until the wanted count is covered: the next digit of the k-th largest key
      unsigned int want = remaining_s;
      unsigned long long digit = 0;
      for (int b = bins - 1; b >= 0; --b) {
        if (counts[b] >= want) { digit = static_cast<unsigned long long>(b); break; }
        want -= counts[b];
      }
      prefix_s = prefix | (digit << shift);
      remaining_s = want;
    }
    mask_above |= ((1ull << widths[round]) - 1ull) << shift;
    __syncthreads();
  }
  // prefix_s IS the k-th largest key: gather every key >= it (exactly top_k of them), sort, keep
  const unsigned long long cut = prefix_s;
  for (int64_t i = tid; i < width; i += kExactThreads) {
    const unsigned long long key = sample_key(__fdiv_rn(Elem<T>::load(src + i), temperature), uint32_t(i));
    if (key >= cut) {
      const unsigned int slot = atomicAdd(&taken_s, 1u);
      if (slot < unsigned(kMaxSelectK)) survivors[slot] = key;
    }
  }
  __syncthreads();
  int n = 2;
  while (n < top_k) n <<= 1;
  for (int i = tid; i < n; i += kExactThreads) if (i >= top_k) survivors[i] = 0ull;
  __syncthreads();
  for (int k = 2; k <= n; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int p = tid; p < n / 2; p += kExactThreads) {
        const int i = ((p & ~(j - 1)) << 1) | (p & (j - 1));
        compare_exchange(survivors[i], survivors[i | j], (i & k) == 0);
      }
      __syncthreads();
    }
  }
  unsigned long long* dst = keys + row * padded;
  for (int i = tid; i < top_k; i += kExactThreads) dst[i] = survivors[i];
}

// ---- small top_k, the usual case: ONE pass over the logits and no key array.
//   splitter  a thread block per row sorts 2048 evenly spaced logits of the row and takes, as threshold, the
//             sample whose rank makes "about 6 x top_k, and with near certainty at least top_k" tokens of the
//             whole row lie above it, lowered by 2^-12 of its magnitude
//   gather    the one pass: every token whose logit is at or above the threshold has its exact score computed and
//             its key appended to the row's candidate list (a few hundred of 150k tokens)
//   finish    one thread block checks the count, sorts the candidates and keeps the top_k largest
// The result is exact or the call is redone: when a row ends with fewer than top_k or more than kCandidates
// candidates (unlucky sample, long runs of equal logits), or when logits / temperature could overflow or lose
// precision near the threshold (then equal scores may hide behind different logits), a flag is raised and the
// radix select over all 64 key bits above redoes every row; that kernel is launched in any case and returns at
// once when the flag is down.  The margin covers the tokens whose score can equal the top_k-th score although
// their logit is smaller: scores are logits / temperature, a monotonic map with a relative rounding error of
// 2^-24.  A NaN logit also sends the call to the exact select (whose key order ranks NaNs as the reference's sort does).
constexpr int kCandidates = 8192;
constexpr int kSplitSamples = 2048;

struct CutState {            // per row
  float threshold;           // candidates are the tokens whose logit is >= this
  unsigned int taken;        // compaction cursor
};

__device__ __forceinline__ uint32_t ordered_bits(float x) {
  const uint32_t b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float from_ordered_bits(uint32_t o) {
  return __uint_as_float((o & 0x80000000u) ? (o & 0x7fffffffu) : ~o);
}

// f(value, index) for every element of a row, 16-byte loads when the row allows, blocks of the grid's x dimension
// striding over the row
template <typename T, typename F>
__device__ __forceinline__ void for_each_logit(const T* src, int64_t width, F&& f) {
  constexpr int N = Elem<T>::kPerVec;
  const int64_t first = int64_t(blockIdx.x) * blockDim.x + threadIdx.x, stride = int64_t(gridDim.x) * blockDim.x;
  if (aligned16(src)) {
    const int64_t nvec = width / N;
    const uint4* vp = reinterpret_cast<const uint4*>(src);
    for (int64_t v = first; v < nvec; v += stride) {
      float e[N];
      Elem<T>::unpack(ld_stream(vp + v), e);
#pragma unroll
      for (int q = 0; q < N; ++q) f(e[q], v * N + q);
    }
    for (int64_t i = nvec * N + first; i < width; i += stride) f(Elem<T>::load(src + i), i);
  } else {
    for (int64_t i = first; i < width; i += stride) f(Elem<T>::load(src + i), i);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
topk_splitter_kernel(const T* logits, int64_t width, int64_t row_stride, unsigned int top_k, int safe, CutState* cut,
                     int* overflow, int overflow_stride) {   // the flag of row r is overflow[r * overflow_stride]: stride 0 = one flag per call
  __shared__ uint32_t sample[kSplitSamples];
  const int64_t row = blockIdx.x;
  overflow += row * overflow_stride;
  const T* src = logits + row * row_stride;
  for (int s = threadIdx.x; s < kSplitSamples; s += 256) {
    const float x = Elem<T>::load(src + (int64_t(s) * width) / kSplitSamples);   // width > kSplitSamples: distinct tokens
    sample[s] = x == x ? ordered_bits(x) : 0u;                                     // a NaN never ranks
  }
  __syncthreads();
  for (int k = 2; k <= kSplitSamples; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int p = threadIdx.x; p < kSplitSamples / 2; p += 256) {
        const int i = ((p & ~(j - 1)) << 1) | (p & (j - 1));
        const uint32_t a = sample[i], b = sample[i | j];
        if ((a < b) == ((i & k) == 0)) { sample[i] = b; sample[i | j] = a; }
      }
      __syncthreads();
    }
  }
  if (threadIdx.x != 0) return;
  // expected rank of the top_k-th token among the samples, plus three standard deviations and two
  const float expected = float(top_k) * float(kSplitSamples) / float(width);
  int rank = int(ceilf(expected + 3.0f * sqrtf(expected))) + 2;
  bool ok = safe != 0 && rank < kSplitSamples;
  float threshold = -INFINITY;
  if (ok) {
    const float at_rank = from_ordered_bits(sample[rank]);
    const unsigned int exponent = (__float_as_uint(at_rank) >> 23) & 0xffu;
    ok = exponent >= 28u && exponent <= 226u;            // 2^-99 .. 2^99: the division stays exact to rounding
    threshold = at_rank - 0.000244140625f * fabsf(at_rank);   // 2^-12 of the magnitude: 4096 rounding errors of the division
  }
  if (!ok) atomicExch(overflow, 1);
  cut[row].threshold = threshold;
  cut[row].taken = 0u;
}

template <typename T>
__global__ void __launch_bounds__(256)
topk_gather_kernel(const T* logits, int64_t width, int64_t row_stride, float temperature, CutState* cut,
                   unsigned long long* candidates, const int* overflow, int overflow_stride) {
  const int64_t row = blockIdx.y;
  overflow += row * overflow_stride;
  if (*overflow != 0) return;                      // the row (or the call) is being redone by the exact path anyway
  const float threshold = cut[row].threshold;
  unsigned long long* out = candidates + row * int64_t(kCandidates);
  bool strange = false;
  for_each_logit<T>(logits + row * row_stride, width, [&](float x, int64_t i) {
    if (x >= threshold) {
      const unsigned int slot = atomicAdd(&cut[row].taken, 1u);
      if (slot < unsigned(kCandidates)) out[slot] = sample_key(__fdiv_rn(x, temperature), uint32_t(i));
    }
    strange |= x != x;
  });
  if (strange) atomicExch(const_cast<int*>(overflow), 1);
}

// Sorts one row's candidates in shared memory, descending, and leaves the top_k largest at the front of the
// row's key area; too few or too many candidates raise *overflow (the exact fallback then overwrites every row).
__global__ void __launch_bounds__(kSortThreads)
topk_finish_kernel(unsigned long long* keys, int64_t padded, int top_k, const CutState* cut,
                   const unsigned long long* candidates, int* overflow) {
  extern __shared__ unsigned long long buf[];
  const int64_t row = blockIdx.x;
  const unsigned int count = cut[row].taken;
  if (*overflow != 0) return;
  if (count < unsigned(top_k) || count > unsigned(kCandidates)) {
    if (threadIdx.x == 0) atomicExch(overflow, 1);
    return;
  }
  const unsigned long long* in = candidates + row * int64_t(kCandidates);
  int n = 2;
  while (n < int(count)) n <<= 1;
  for (int i = threadIdx.x; i < n; i += kSortThreads) buf[i] = unsigned(i) < count ? in[i] : 0ull;
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
                    unsigned long long seed, const unsigned long long* draw_offsets, float* running, int32_t* out_ids,
                    const int* only_rows) {
  __shared__ float stage[kChunk];
  __shared__ float carry;
  __shared__ int found;
  const int64_t row = blockIdx.x;
  if (only_rows != nullptr && only_rows[row] == 0) return;
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
}

// ---- top_p < 1 over the whole vocabulary without sorting it.
// The reference sorts all scores and walks them with one thread (src/ops_cuda.cu:575-617): `total` is the fp32 sum
// of every exponential in descending order, then the top-p prefix and the pick walk the head of that order.  Only
// the HEAD needs the order.  For the rest, the running sum S = M * 2^(k-23) (M a 24-bit integer) is already large
// against every term e that is left, and S + e rounds to (M + round(e / 2^(k-23))) * 2^(k-23) -- an integer increment
// that does not depend on M -- unless e / 2^(k-23) falls exactly on a half (a tie: the parity of M decides) or the
// sum reaches the next power of two (the grid of the rounding doubles).  Integer increments commute, so away from
// those two events the ORDER of the terms does not matter, only their multiset:
//   head    the few thousand largest logits, found as in the top-k path (sampled threshold, one pass), sorted in
//           one thread block, summed in order by one thread with the running sums kept: S_head, and its power of
//           two k
//   tail    one pass over the other logits: every term's increment for k and for k + 1 is added into one of 2048
//           buckets by score (a monotonic map, so the buckets partition the descending order into consecutive
//           runs); ties are flagged per bucket
//   finish  one thread walks the buckets: M += bucket sum.  A bucket with a tie, or in which M would pass 2^24, is
//           the only place where the order matters: its terms (tens) are gathered, sorted and added one by one in
//           fp32.  That yields `total` bit for bit.  The top-p walk and the pick then run over the head exactly as
//           the reference's single thread does.
// A row that breaks an assumption (fewer than 64 or more than 8192 head candidates, a NaN, the sum growing by more
// than one power of two in the tail, a bucket of more than 2048 terms, a prefix that does not end inside the head)
// raises its flag and is redone by the whole-row sort; those kernels are launched in any case and return at once for
// the rows whose flag is down.
constexpr int kTailBuckets = 2048;
constexpr unsigned int kHeadTarget = 2000;     // the splitter's threshold then leaves about 3000 head candidates of 150k tokens
constexpr int kMinHead = 64;

struct HeadState {          // per row
  float sum;                // S_head
  float max_score;          // score of the first token of the order
  float low_score;          // score of the last head token
  int count;
};

// increment of a term e under a sum whose unit in the last place is 2^(k-23), and whether it is a tie
__device__ __forceinline__ void term_increment(float e, int k, unsigned int& r, bool& tie) {
  const uint32_t b = __float_as_uint(e);
  const uint32_t field = b >> 23;                                   // e > 0: no sign bit
  const uint32_t m = field != 0u ? ((b & 0x7fffffu) | 0x800000u) : (b & 0x7fffffu);
  const int d = k - (field != 0u ? int(field) - 127 : -126);      // e = m * 2^(E-23), increment = m / 2^d
  if (d >= 25 || m == 0u) { r = 0u; tie = false; return; }
  if (d < 1) { r = 0xffffffffu; tie = true; return; }                // a term as large as the sum: never in a tail
  r = (m + (1u << (d - 1))) >> d;
  tie = (m & ((1u << d) - 1u)) == (1u << (d - 1));
}
__device__ __forceinline__ int exponent_of(float s) { return int((__float_as_uint(s) >> 23) & 0xffu) - 127; }

__device__ __forceinline__ int tail_bucket(float score, float low_score, float scale) {
  const float t = (low_score - score) * scale;                      // >= 0 for every tail term; monotonic in the score
  const int b = t >= float(kTailBuckets - 1) ? kTailBuckets - 1 : int(t);
  return b < 0 ? 0 : b;
}
// buckets per unit of score: the tail terms that can still move the sum lie within (k - 26) * ln 2 of the maximum
__device__ __forceinline__ float tail_scale(const HeadState& h) {
  const float lowest = h.max_score + float(exponent_of(h.sum) - 26) * 0.6931471805599453f;
  const float span = h.low_score - lowest;
  return span > 1e-6f ? float(kTailBuckets) / span : 0.0f;
}

// head: sort the row's candidates (all of them), leave them at the front of the row's key area, and add their
// exponentials in order, keeping every running sum
__global__ void __launch_bounds__(kSortThreads)
topp_head_kernel(unsigned long long* keys, int64_t padded, const CutState* cut, const unsigned long long* candidates,
                 float* running, unsigned int* tails, HeadState* heads, int* row_flags) {
  extern __shared__ unsigned long long buf[];
  __shared__ float stage[kChunk];
  __shared__ float carry;
  const int64_t row = blockIdx.x;
  const int tid = threadIdx.x;
  // the tail pass adds into these: they start at zero
  unsigned int* tail = tails + row * int64_t(3 * kTailBuckets);
  for (int i = tid; i < 3 * kTailBuckets; i += kSortThreads) tail[i] = 0u;
  if (row_flags[row] != 0) return;
  const unsigned int count = cut[row].taken;
  if (count < unsigned(kMinHead) || count > unsigned(kCandidates)) {
    if (tid == 0) row_flags[row] = 1;
    return;
  }
  const unsigned long long* in = candidates + row * int64_t(kCandidates);
  int n = 2;
  while (n < int(count)) n <<= 1;
  for (int i = tid; i < n; i += kSortThreads) buf[i] = unsigned(i) < count ? in[i] : 0ull;
  __syncthreads();
  for (int k = 2; k <= n; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int p = tid; p < n / 2; p += kSortThreads) {
        const int i = ((p & ~(j - 1)) << 1) | (p & (j - 1));
        compare_exchange(buf[i], buf[i | j], (i & k) == 0);
      }
      __syncthreads();
    }
  }
  unsigned long long* dst = keys + row * padded;
  for (int i = tid; i < int(count); i += kSortThreads) dst[i] = buf[i];
  const float maximum = key_score(buf[0]);
  float* cum = running + row * padded;
  if (tid == 0) carry = 0.0f;
  __syncthreads();
  for (int base = 0; base < int(count); base += kChunk) {
    const int m = int(count) - base < kChunk ? int(count) - base : kChunk;
    for (int j = tid; j < m; j += kSortThreads) stage[j] = expf(key_score(buf[base + j]) - maximum);
    __syncthreads();
    if (tid == 0) {
      float sum = carry;
      for (int j = 0; j < m; ++j) { sum += stage[j]; stage[j] = sum; }
      carry = sum;
    }
    __syncthreads();
    for (int j = tid; j < m; j += kSortThreads) cum[base + j] = stage[j];
    __syncthreads();
  }
  if (tid == 0) heads[row] = HeadState{carry, maximum, key_score(buf[count - 1]), int(count)};
}

// tail: increments of every term below the head, per bucket, for the head's power of two and the next one.
// Per bucket three words: sum of increments under k, under k + 1, and (terms << 2 | tie under k + 1 << 1 | tie under k).
template <typename T>
__global__ void __launch_bounds__(256)
topp_tail_kernel(const T* logits, int64_t width, int64_t row_stride, float temperature, const CutState* cut,
                 const HeadState* heads, unsigned int* tails, int* row_flags) {
  __shared__ unsigned int local[3 * kTailBuckets];
  const int64_t row = blockIdx.y;
  if (row_flags[row] != 0) return;
  for (int i = threadIdx.x; i < 3 * kTailBuckets; i += 256) local[i] = 0u;
  __syncthreads();
  const HeadState h = heads[row];
  const float threshold = cut[row].threshold, scale = tail_scale(h);
  const int k = exponent_of(h.sum);
  bool broken = false;
  for_each_logit<T>(logits + row * row_stride, width, [&](float x, int64_t) {
    if (x >= threshold) return;                                   // a head token (a NaN would have raised the row's flag)
    const float score = __fdiv_rn(x, temperature);
    const float e = expf(score - h.max_score);
    unsigned int r0, r1;
    bool t0, t1;
    term_increment(e, k, r0, t0);
    term_increment(e, k + 1, r1, t1);
    if (r0 == 0xffffffffu) { broken = true; return; }
    if ((r0 | r1) == 0u && !t0 && !t1) return;                    // cannot move the sum under either power of two
    const int b = tail_bucket(score, h.low_score, scale);
    if (r0 != 0u) atomicAdd(&local[b], r0);
    if (r1 != 0u) atomicAdd(&local[kTailBuckets + b], r1);
    atomicAdd(&local[2 * kTailBuckets + b], 4u);
    if (t0 || t1) atomicOr(&local[2 * kTailBuckets + b], (t0 ? 1u : 0u) | (t1 ? 2u : 0u));
  });
  if (broken) row_flags[row] = 1;
  __syncthreads();
  unsigned int* tail = tails + row * int64_t(3 * kTailBuckets);
  for (int i = threadIdx.x; i < 2 * kTailBuckets; i += 256)
    if (local[i] != 0u) atomicAdd(&tail[i], local[i]);
  for (int i = 2 * kTailBuckets + threadIdx.x; i < 3 * kTailBuckets; i += 256) {
    const unsigned int v = local[i];
    if (v != 0u) { atomicAdd(&tail[i], v & ~3u); if (v & 3u) atomicOr(&tail[i], v & 3u); }
  }
}

// finish: the walk over the buckets (exact where the order matters), then the reference's top-p walk and pick over the head
template <typename T>
__global__ void __launch_bounds__(kSortThreads)
topp_finish_kernel(const T* logits, int64_t width, int64_t row_stride, float temperature, const CutState* cut,
                   const unsigned long long* keys, int64_t padded, const float* running, const unsigned int* tails,
                   const HeadState* heads, float top_p, unsigned long long seed, const unsigned long long* draw_offsets,
                   int32_t* out_ids, int* row_flags) {
  __shared__ unsigned long long bucket_keys[kTailBuckets];
  __shared__ float stage[kChunk];
  __shared__ float carry;
  __shared__ unsigned int walk_m;
  __shared__ int walk_k, walk_bucket, found, give_up;
  __shared__ unsigned int gathered;
  const int64_t row = blockIdx.x;
  if (row_flags[row] != 0) return;
  const int tid = threadIdx.x;
  const HeadState h = heads[row];
  const unsigned int* tail = tails + row * int64_t(3 * kTailBuckets);
  const float threshold = cut[row].threshold, scale = tail_scale(h);
  const int k0 = exponent_of(h.sum);
  const T* src = logits + row * row_stride;
  if (tid == 0) {
    walk_m = (__float_as_uint(h.sum) & 0x7fffffu) | 0x800000u;
    walk_k = k0;
    walk_bucket = 0;
    give_up = 0;
  }
  __syncthreads();
  for (;;) {
    if (tid == 0) {
      unsigned int m = walk_m;
      int k = walk_k, b = walk_bucket;
      for (; b < kTailBuckets; ++b) {
        const unsigned int info = tail[2 * kTailBuckets + b];
        if (info == 0u) continue;
        if (k > k0 + 1) { give_up = 1; break; }
        const unsigned int r = k == k0 ? tail[b] : tail[kTailBuckets + b];
        const bool tie = (info & (k == k0 ? 1u : 2u)) != 0u;
        if (tie || static_cast<unsigned long long>(m) + r > (1ull << 24)) break;   // the order inside this bucket matters
        m += r;
        if (m == (1u << 24)) { m = 1u << 23; ++k; }
      }
      walk_m = m; walk_k = k; walk_bucket = b;
      gathered = 0u;
    }
    __syncthreads();
    if (give_up != 0) { if (tid == 0) row_flags[row] = 1; return; }
    const int b = walk_bucket;
    if (b >= kTailBuckets) break;
    // gather the terms of bucket b that can move the sum, sort them into the reference's order, add them one by one
    for (int64_t i = tid; i < width; i += kSortThreads) {
      const float x = Elem<T>::load(src + i);
      if (x >= threshold) continue;
      const float score = __fdiv_rn(x, temperature);
      if (tail_bucket(score, h.low_score, scale) != b) continue;
      const float e = expf(score - h.max_score);
      unsigned int r0, r1;
      bool t0, t1;
      term_increment(e, k0, r0, t0);
      term_increment(e, k0 + 1, r1, t1);
      if ((r0 | r1) == 0u && !t0 && !t1) continue;
      const unsigned int slot = atomicAdd(&gathered, 1u);
      if (slot < unsigned(kTailBuckets)) bucket_keys[slot] = sample_key(score, uint32_t(i));
    }
    __syncthreads();
    const unsigned int count = gathered;
    if (count > unsigned(kTailBuckets)) { if (tid == 0) row_flags[row] = 1; return; }
    int n = 2;
    while (n < int(count)) n <<= 1;
    for (int i = int(count) + tid; i < n; i += kSortThreads) bucket_keys[i] = 0ull;
    __syncthreads();
    for (int k = 2; k <= n; k <<= 1) {
      for (int j = k >> 1; j > 0; j >>= 1) {
        for (int p = tid; p < n / 2; p += kSortThreads) {
          const int i = ((p & ~(j - 1)) << 1) | (p & (j - 1));
          compare_exchange(bucket_keys[i], bucket_keys[i | j], (i & k) == 0);
        }
        __syncthreads();
      }
    }
    if (tid == 0) {
      float sum = __uint_as_float((uint32_t(walk_k + 127) << 23) | (walk_m & 0x7fffffu));
      for (unsigned int i = 0; i < count; ++i) sum += expf(key_score(bucket_keys[i]) - h.max_score);
      walk_m = (__float_as_uint(sum) & 0x7fffffu) | 0x800000u;
      walk_k = exponent_of(sum);
      walk_bucket = b + 1;
    }
    __syncthreads();
  }
  const float total = __uint_as_float((uint32_t(walk_k + 127) << 23) | (walk_m & 0x7fffffu));

  // the reference's top-p walk (src/ops_cuda.cu:596-603) over the head; it must end strictly above the head's lowest score
  const unsigned long long* sorted = keys + row * padded;
  const float* cum = running + row * padded;
  const int limit = h.count;
  if (tid == 0) { carry = 0.0f; found = -1; }
  __syncthreads();
  int prefix = -1;
  for (int base = 0; base < limit; base += kChunk) {
    const int m = limit - base < kChunk ? limit - base : kChunk;
    for (int j = tid; j < m; j += kSortThreads) stage[j] = __fdiv_rn(expf(key_score(sorted[base + j]) - h.max_score), total);
    __syncthreads();
    if (tid == 0) {
      float cumulative = carry;
      for (int j = 0; j < m; ++j) {
        cumulative += stage[j];
        if (cumulative >= top_p) { found = j; break; }
      }
      carry = cumulative;
    }
    __syncthreads();
    if (found >= 0) { prefix = base + found + 1; break; }
  }
  if (prefix < 0 || !(key_score(sorted[prefix - 1]) > h.low_score)) {   // not settled inside the head: the whole-row path decides
    if (tid == 0) row_flags[row] = 1;
    return;
  }
  const float prefix_total = cum[prefix - 1];
  const unsigned long long offset = draw_offsets != nullptr ? draw_offsets[row] : 0ull;
  const unsigned long long bits = sampler_hash(seed ^ (offset * 0xd1342543de82ef95ULL));
  const float u = (static_cast<float>((bits >> 11) & 0x1fffffffffffffULL) + 0.5f) / 9007199254740992.0f;
  const float target = u * prefix_total;
  __shared__ unsigned long long best;
  if (tid == 0) best = static_cast<unsigned long long>(prefix - 1);
  __syncthreads();
  unsigned long long mine = static_cast<unsigned long long>(prefix - 1);
  for (int i = tid; i < prefix; i += kSortThreads)
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

// per row: padded keys (8 B each), padded running sums (4 B each), the candidates of the top-k / top-p paths, the
// tail buckets of the top-p path and three small records; one flag for the whole call
size_t sampler_workspace_bytes(int64_t rows, int64_t width) {
  const int64_t padded = padded_width(width);
  const size_t per_row = size_t(padded) * 12 + size_t(kCandidates) * 8 + size_t(3 * kTailBuckets) * 4 + sizeof(CutState) +
                         sizeof(HeadState) + sizeof(int);
  return (size_t(rows) * per_row + 16 + 255) / 256 * 256;
}

int launch_sample_rows(const void* logits, int64_t rows, int64_t width, int64_t row_stride, int dtype, float temperature,
                       int top_k, float top_p, unsigned long long seed, const unsigned long long* draw_offsets,
                       int32_t* out_ids, void* workspace, cudaStream_t s) {
  if (rows == 0) return B2_OK;
  const int64_t padded = padded_width(width);
  auto* keys = static_cast<unsigned long long*>(workspace);
  auto* candidates = keys + rows * padded;                                   // kCandidates per row
  auto* running = reinterpret_cast<float*>(candidates + rows * int64_t(kCandidates));
  auto* tails = reinterpret_cast<unsigned int*>(running + rows * padded);
  auto* heads = reinterpret_cast<HeadState*>(tails + rows * int64_t(3 * kTailBuckets));
  auto* cut = reinterpret_cast<CutState*>(heads + rows);
  int* row_flags = reinterpret_cast<int*>(cut + rows);
  int* overflow = row_flags + rows;
  // thread blocks per row for a pass over the logits: enough to fill the GPU over all rows and no more
  int64_t spread64 = (int64_t(sm_count()) * 8 + rows - 1) / rows;
  if (spread64 > padded / 1024) spread64 = padded / 1024;
  if (spread64 < 1) spread64 = 1;
  const dim3 row_grid = dim3(unsigned(spread64), unsigned(rows), 1);
  // logits / temperature stays a normal number near a threshold only for a moderate temperature (and a moderate
  // logit there, which the splitter kernel checks)
  const int safe = temperature >= 9.5367431640625e-07f && temperature <= 1048576.0f;   // 2^-20 .. 2^20
  const int* only_rows = nullptr;   // the rows the whole-row sort below has to do (null: all of them)

  if (top_k > 0 && top_k <= kMaxSelectK && width > kTile) {
    // only the k largest keys matter: a sampled threshold, one pass over the logits, a small sort: five launches and
    // a four-byte clear
    if (cudaMemsetAsync(overflow, 0, sizeof(int), s) != cudaSuccess) return launch_status("sample_rows");
    // the opt-in is a per-device attribute: set on every call, as the other kernels with large shared memory do
    if (cudaFuncSetAttribute(topk_finish_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kCandidates * 8) != cudaSuccess) {
      cudaGetLastError();
      set_error("sample_rows: cannot reserve shared memory");
      return B2_ERR_CUDA;
    }
    if (dtype == B2_F32) {
      const float* x = static_cast<const float*>(logits);
      topk_splitter_kernel<float><<<unsigned(rows), 256, 0, s>>>(x, width, row_stride, unsigned(top_k), safe, cut, overflow, 0);
      topk_gather_kernel<float><<<row_grid, 256, 0, s>>>(x, width, row_stride, temperature, cut, candidates, overflow, 0);
    } else {
      const __half* x = static_cast<const __half*>(logits);
      topk_splitter_kernel<__half><<<unsigned(rows), 256, 0, s>>>(x, width, row_stride, unsigned(top_k), safe, cut, overflow, 0);
      topk_gather_kernel<__half><<<row_grid, 256, 0, s>>>(x, width, row_stride, temperature, cut, candidates, overflow, 0);
    }
    topk_finish_kernel<<<unsigned(rows), kSortThreads, kCandidates * 8, s>>>(keys, padded, top_k, cut, candidates, overflow);
    // ... unless that could not be trusted: then (and only then) the radix select over all 64 key bits redoes every row
    if (dtype == B2_F32)
      topk_exact_kernel<float><<<unsigned(rows), kExactThreads, 0, s>>>(static_cast<const float*>(logits), width, row_stride, padded,
                                                                        temperature, top_k, keys, overflow);
    else
      topk_exact_kernel<__half><<<unsigned(rows), kExactThreads, 0, s>>>(static_cast<const __half*>(logits), width, row_stride,
                                                                         padded, temperature, top_k, keys, overflow);
  } else {
    if (top_k == 0 && top_p < 1.0f && width >= 4 * kCandidates) {
      // top-p over the whole vocabulary: head sorted, tail summed by buckets; rows that do not fit that scheme raise
      // their flag and are the only ones the whole-row sort below still works on
      if (cudaMemsetAsync(row_flags, 0, size_t(rows) * sizeof(int), s) != cudaSuccess) return launch_status("sample_rows");
      if (cudaFuncSetAttribute(topp_head_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kCandidates * 8) != cudaSuccess) {
        cudaGetLastError();
        set_error("sample_rows: cannot reserve shared memory");
        return B2_ERR_CUDA;
      }
      if (dtype == B2_F32) {
        const float* x = static_cast<const float*>(logits);
        topk_splitter_kernel<float><<<unsigned(rows), 256, 0, s>>>(x, width, row_stride, kHeadTarget, safe, cut, row_flags, 1);
        topk_gather_kernel<float><<<row_grid, 256, 0, s>>>(x, width, row_stride, temperature, cut, candidates, row_flags, 1);
        topp_head_kernel<<<unsigned(rows), kSortThreads, kCandidates * 8, s>>>(keys, padded, cut, candidates, running, tails, heads, row_flags);
        topp_tail_kernel<float><<<row_grid, 256, 0, s>>>(x, width, row_stride, temperature, cut, heads, tails, row_flags);
        topp_finish_kernel<float><<<unsigned(rows), kSortThreads, 0, s>>>(x, width, row_stride, temperature, cut, keys, padded, running,
                                                                          tails, heads, top_p, seed, draw_offsets, out_ids, row_flags);
      } else {
        const __half* x = static_cast<const __half*>(logits);
        topk_splitter_kernel<__half><<<unsigned(rows), 256, 0, s>>>(x, width, row_stride, kHeadTarget, safe, cut, row_flags, 1);
        topk_gather_kernel<__half><<<row_grid, 256, 0, s>>>(x, width, row_stride, temperature, cut, candidates, row_flags, 1);
        topp_head_kernel<<<unsigned(rows), kSortThreads, kCandidates * 8, s>>>(keys, padded, cut, candidates, running, tails, heads, row_flags);
        topp_tail_kernel<__half><<<row_grid, 256, 0, s>>>(x, width, row_stride, temperature, cut, heads, tails, row_flags);
        topp_finish_kernel<__half><<<unsigned(rows), kSortThreads, 0, s>>>(x, width, row_stride, temperature, cut, keys, padded, running,
                                                                           tails, heads, top_p, seed, draw_offsets, out_ids, row_flags);
      }
      only_rows = row_flags;
    }
    // the whole-row sort has little per-block overhead: many small blocks
    const dim3 wide_grid(unsigned(padded / 256 < 1 ? 1 : (padded / 256 > 296 ? 296 : padded / 256)), unsigned(rows));
    if (dtype == B2_F32)
      sampler_keys_kernel<float><<<wide_grid, 256, 0, s>>>(static_cast<const float*>(logits), width, row_stride, padded,
                                                            temperature, keys, only_rows);
    else
      sampler_keys_kernel<__half><<<wide_grid, 256, 0, s>>>(static_cast<const __half*>(logits), width, row_stride, padded,
                                                           temperature, keys, only_rows);
    const int tile = int(padded < kTile ? padded : kTile);
    const dim3 tile_grid(unsigned(padded / tile), unsigned(rows));
    if (tile < kTile) {
      bitonic_tile_kernel<<<tile_grid, kSortThreads, size_t(tile) * 8, s>>>(keys, padded, tile, 2, tile, only_rows);   // the whole row is one small tile
    } else {
      bitonic_tile_registers_kernel<<<tile_grid, kRegThreads, 0, s>>>(keys, padded, 2, kTile, only_rows);
      for (int64_t k = int64_t(kTile) * 2; k <= padded; k <<= 1) {
        int64_t j = k >> 1;
        for (; j >= 2 * kTile; j >>= 2) bitonic_wide_pair_kernel<<<wide_grid, 256, 0, s>>>(keys, padded, k, j, only_rows);   // steps j and j/2
        if (j >= kTile) bitonic_wide_kernel<<<wide_grid, 256, 0, s>>>(keys, padded, k, j, only_rows);              // one step left over
        bitonic_tile_registers_kernel<<<tile_grid, kRegThreads, 0, s>>>(keys, padded, k, k, only_rows);
      }
    }
  }
  sampler_pick_kernel<<<unsigned(rows), kSelectThreads, 0, s>>>(keys, width, padded, top_k, top_p, seed, draw_offsets, running,
                                                                out_ids, only_rows);
  return launch_status("sample_rows");
}

}  // namespace b2
