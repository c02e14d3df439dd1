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
//   sort     when 0 < top_k <= 2048 only the k largest keys matter: a threshold taken from a sample of
//            the row, ONE pass over the logits that gathers the few hundred tokens above it, and a one-block
//            sort of those (checked; a call whose sample misled it is redone by a radix select over all 64
//            key bits, one more launch that otherwise returns at once); otherwise a bitonic network sorts the whole row (keys in registers, 4096-key tiles,
//            wider steps in global memory)
//   select   one thread block per row: the exponentials of a 2048-token chunk are computed in
//            parallel, one thread adds them in order (the only serial part left) and records the
//            running sums; the top-p cut walks the same way and stops at the crossing; the final pick
//            is a parallel search in the recorded sums.
#include "sampler_rows.cuh"
#include "kernels.h"

namespace b2 {
namespace {

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
  dependent_launch_prologue();
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
//   splitter  a thread block per row looks at 8192 logits of the row (256 evenly spaced runs of 32) and takes, as threshold, the
//             sample whose rank makes "a few times top_k, and with near certainty at least top_k" tokens of the
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
constexpr int kSplitSamples = 8192;   // evenly spaced logits per row from which the threshold is taken

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

constexpr int kSplitThreads = 1024;
constexpr int kSamplesPerThread = kSplitSamples / kSplitThreads;
constexpr int kSplitLowestBit = 12;   // the threshold is lowered by 2^-12 of its magnitude anyway: the low bits stay zero (a lower bound)
// The sample of rank `rank` (0 = largest) is found without sorting the samples: its 32 ordered bits are decided one
// at a time from the top by counting the samples at or above a candidate (the lowest twelve bits are left zero:
// that only lowers the threshold a little further).  Every thread keeps its samples in registers.  (A radix select with 256-bin histograms took three times as long: most samples share their leading
// digits, and matching a warp's votes per bin costs more than the eight comparisons of a count.)
template <typename T>
__global__ void __launch_bounds__(kSplitThreads)
topk_splitter_kernel(const T* logits, int64_t width, int64_t row_stride, unsigned int top_k, int safe, CutState* cut,
                     int* overflow, int overflow_stride) {   // the flag of row r is overflow[r * overflow_stride]: stride 0 = one flag per call
  // top_k == 0: no count to reach; the threshold is to leave as many candidates as fit one kTile-key tile with near
  // certainty (the top-p path's head)
  dependent_launch_prologue();
  __shared__ unsigned int counts[2][kSplitThreads / 32];
  const int64_t row = blockIdx.x;
  overflow += row * overflow_stride;
  const T* src = logits + row * row_stride;
  // as many samples as there are tokens to take them from two apart, at most kSplitSamples
  int samples = kSplitSamples;
  while (samples > kSplitThreads && int64_t(samples) * 2 > width) samples >>= 1;
  const int run_shift = 31 - __clz(samples >> 5);    // log2 of the number of 32-token runs
  uint32_t mine[kSamplesPerThread];
#pragma unroll
  for (int q = 0; q < kSamplesPerThread; ++q) {
    const int sidx = threadIdx.x + q * kSplitThreads;
    const bool present = sidx < samples;
    const int at = present ? sidx : 0;                 // every load is issued (none sits behind a branch): all in flight at once
    // runs of 32 neighbouring tokens, the runs evenly spaced: one 128-byte line per run instead of one sector
    // per sample (samples every 18 tokens would touch every sector of the row: a whole extra pass over the logits);
    // the number of runs is a power of two: a shift, not a 64-bit division per sample
    const float x = Elem<T>::load(src + ((int64_t(at >> 5) * width) >> run_shift) + (at & 31));
    mine[q] = present && x == x ? ordered_bits(x) : 0u;                          // a NaN never ranks
  }
  // expected rank of the top_k-th token among the samples, plus four standard deviations and two
  const float expected = float(top_k) * float(samples) / float(width);
  int rank = int(ceilf(expected + 4.0f * sqrtf(expected))) + 2;
  if (top_k == 0u) {
    // the number of tokens above the sample of rank r is about width * r / samples, with a relative spread of
    // 1 / sqrt(r): the largest r whose count stays within the tile at five and a half spreads (closed form of
    // r + 5.5 sqrt(r) <= tile * samples / width)
    const float budget = float(kTile) * float(samples) / float(width);
    const float root = 0.5f * (sqrtf(30.25f + 4.0f * budget) - 5.5f);
    rank = int(root * root) - 1;
    if (rank < 2) rank = 2;
  }
  bool ok = safe != 0 && rank < samples;
  // the key with exactly `need` samples at or above it, bit by bit from the top: a candidate keeps its bit when
  // at least `need` samples are at or above it (32 counts of 8 comparisons per thread, one barrier each)
  const unsigned int need = unsigned(ok ? rank : 0) + 1u;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t prefix_found = 0u;
  for (int bit = 31; bit >= kSplitLowestBit; --bit) {
    const uint32_t candidate = prefix_found | (1u << bit);
    unsigned int above = 0u;
#pragma unroll
    for (int q = 0; q < kSamplesPerThread; ++q) above += mine[q] >= candidate ? 1u : 0u;   // absent samples and NaNs are 0: never counted
    above = __reduce_add_sync(0xffffffffu, above);
    // one slot per warp (32 warps adding to one address would queue), two sets of slots in turn: a warp can be
    // one barrier ahead of the slowest reader, never two
    if (lane == 0) counts[bit & 1][warp] = above;
    __syncthreads();
    const unsigned int all = __reduce_add_sync(0xffffffffu, lane < kSplitThreads / 32 ? counts[bit & 1][lane] : 0u);
    if (all >= need) prefix_found = candidate;                // every thread takes the same decision
  }
  if (threadIdx.x != 0) return;
  float threshold = -INFINITY;
  if (ok) {
    const float at_rank = from_ordered_bits(prefix_found);
    const unsigned int exponent = (__float_as_uint(at_rank) >> 23) & 0xffu;
    ok = exponent >= 28u && exponent <= 226u;            // 2^-99 .. 2^99: the division stays exact to rounding
    threshold = at_rank - 0.000244140625f * fabsf(at_rank);   // 2^-12 of the magnitude: 4096 rounding errors of the division
  }
  if (!ok) atomicExch(overflow, 1);
  cut[row].threshold = threshold;
  cut[row].taken = 0u;
}

template <typename T>
__global__ void __launch_bounds__(256, 8)
topk_gather_kernel(const T* logits, int64_t width, int64_t row_stride, float temperature, CutState* cut,
                   unsigned long long* candidates, const int* overflow, int overflow_stride) {
  dependent_launch_prologue();
  const int64_t row = blockIdx.y;
  overflow += row * overflow_stride;
  if (*overflow != 0) return;                      // the row (or the call) is being redone by the exact path anyway
  // Candidates are rare (tenths of a percent to two percent of the tokens), so the pass only STAGES them: a turn
  // reads 16 tokens per thread, counts its candidates, a warp takes room for all of its own with one shared-memory
  // atomic (per-candidate atomics queue on one address), and each candidate's raw (logit, index) pair goes to the
  // staging area.  Scores and keys are computed afterwards, densely, and the block appends to the row's list
  // with ONE global atomic.  What does not fit the staging area goes out directly.
  constexpr int N = Elem<T>::kPerVec, kVecs = 16 / N, kLocal = 2048;   // 16 tokens per thread and turn
  __shared__ float2 staged[kLocal];                // (logit, index bits)
  __shared__ unsigned int local_count, base_slot;
  if (threadIdx.x == 0) local_count = 0u;
  __syncthreads();
  const float threshold = cut[row].threshold;
  unsigned long long* out = candidates + row * int64_t(kCandidates);
  const T* src = logits + row * row_stride;
  const int lane = threadIdx.x & 31;
  bool strange = false;
  auto place = [&](float x, int64_t i, unsigned int slot) {
    if (slot < unsigned(kLocal)) {
      staged[slot] = make_float2(x, __uint_as_float(uint32_t(i)));
    } else {
      const unsigned int direct = atomicAdd(&cut[row].taken, 1u);
      if (direct < unsigned(kCandidates)) out[direct] = sample_key(__fdiv_rn(x, temperature), uint32_t(i));
    }
  };
  // room for `count` candidates of this lane: returns the lane's first slot (every lane of the warp calls this)
  auto reserve = [&](unsigned int count) {
    unsigned int before = count;
#pragma unroll
    for (int offset = 1; offset < 32; offset <<= 1) {
      const unsigned int up = __shfl_up_sync(0xffffffffu, before, offset);
      if (lane >= offset) before += up;
    }
    const unsigned int total = __shfl_sync(0xffffffffu, before, 31);
    unsigned int base = 0u;
    if (total != 0u) {
      if (lane == 0) base = atomicAdd(&local_count, total);
      base = __shfl_sync(0xffffffffu, base, 0);
    }
    return base + before - count;
  };
  const int64_t first = int64_t(blockIdx.x) * 256 + threadIdx.x, stride = int64_t(gridDim.x) * 256;
  if (aligned16(src)) {
    const int64_t nvec = width / N;
    const uint4* vp = reinterpret_cast<const uint4*>(src);
    const int64_t turns = (nvec + stride * kVecs - 1) / (stride * kVecs);   // the same for every thread: the shuffles need whole warps
    for (int64_t turn = 0; turn < turns; ++turn) {
      const int64_t v0 = first + turn * stride * kVecs;
      uint4 r[kVecs];
#pragma unroll
      for (int q = 0; q < kVecs; ++q) r[q] = v0 + q * stride < nvec ? ld_stream(vp + v0 + q * stride) : make_uint4(0u, 0u, 0u, 0u);
      float e[kVecs][N];
      unsigned int hits = 0u, count = 0u;
#pragma unroll
      for (int q = 0; q < kVecs; ++q) {
        Elem<T>::unpack(r[q], e[q]);
        const bool in = v0 + q * stride < nvec;
#pragma unroll
        for (int z = 0; z < N; ++z) {
          const bool hit = in && e[q][z] >= threshold;
          strange |= in && e[q][z] != e[q][z];
          if (hit) { hits |= 1u << (q * N + z); ++count; }
        }
      }
      if (__any_sync(0xffffffffu, count != 0u)) {
        unsigned int slot = reserve(count);
#pragma unroll
        for (int q = 0; q < kVecs; ++q) {
#pragma unroll
          for (int z = 0; z < N; ++z)
            if (hits >> (q * N + z) & 1u) place(e[q][z], (v0 + q * stride) * N + z, slot++);
        }
      }
    }
    const int64_t rest_turns = (width - nvec * N + stride - 1) / stride;
    for (int64_t turn = 0; turn < rest_turns; ++turn) {
      const int64_t i = nvec * N + first + turn * stride;
      const float x = i < width ? Elem<T>::load(src + i) : -INFINITY;
      const bool hit = i < width && x >= threshold;
      strange |= x != x;
      if (__any_sync(0xffffffffu, hit)) {
        const unsigned int slot = reserve(hit ? 1u : 0u);
        if (hit) place(x, i, slot);
      }
    }
  } else {
    const int64_t turns = (width + stride - 1) / stride;
    for (int64_t turn = 0; turn < turns; ++turn) {
      const int64_t i = first + turn * stride;
      const float x = i < width ? Elem<T>::load(src + i) : -INFINITY;
      const bool hit = i < width && x >= threshold;
      strange |= x != x;
      if (__any_sync(0xffffffffu, hit)) {
        const unsigned int slot = reserve(hit ? 1u : 0u);
        if (hit) place(x, i, slot);
      }
    }
  }
  __syncthreads();
  const unsigned int kept = local_count < unsigned(kLocal) ? local_count : unsigned(kLocal);
  if (threadIdx.x == 0) base_slot = kept != 0u ? atomicAdd(&cut[row].taken, kept) : 0u;
  __syncthreads();
  for (unsigned int i = threadIdx.x; i < kept; i += blockDim.x) {
    const float2 c = staged[i];
    if (base_slot + i < unsigned(kCandidates)) out[base_slot + i] = sample_key(__fdiv_rn(c.x, temperature), __float_as_uint(c.y));
  }
  if (strange) atomicExch(const_cast<int*>(overflow), 1);
}

// Sorts one row's candidates in shared memory, descending, and leaves the top_k largest at the front of the
// row's key area; too few or too many candidates raise *overflow (the exact fallback then overwrites every row).
__global__ void __launch_bounds__(kSortThreads)
topk_finish_kernel(unsigned long long* keys, int64_t padded, int top_k, const CutState* cut,
                   const unsigned long long* candidates, int* overflow) {
  dependent_launch_prologue();
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
// A row that breaks an assumption (fewer than 64 or more than 4096 head candidates, a NaN, the sum growing by more
// than one power of two in the tail, a bucket of more than 2048 terms, a prefix that does not end inside the head)
// raises its flag and is redone by the whole-row sort, over exactly those rows: launched from the device by the
// kernel that lists them, and only when there are any (sampler_fallback.cu).
constexpr int kTailBuckets = 2048;
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
// the same for two sums at once: units 2^(k-23) and 2^(k-22)
__device__ __forceinline__ void term_increments(float e, int k, unsigned int& r0, bool& t0, unsigned int& r1, bool& t1) {
  const uint32_t b = __float_as_uint(e);
  const uint32_t field = b >> 23;
  const uint32_t m = field != 0u ? ((b & 0x7fffffu) | 0x800000u) : (b & 0x7fffffu);
  const int d = k - (field != 0u ? int(field) - 127 : -126);
  r0 = r1 = 0u;
  t0 = t1 = false;
  if (d >= 25 || m == 0u) return;
  if (d < 1) { r0 = 0xffffffffu; t0 = true; return; }
  const uint32_t half = 1u << (d - 1);
  r0 = (m + half) >> d;
  t0 = (m & (2u * half - 1u)) == half;
  if (d == 24) return;                                   // under the doubled unit the term is below a quarter: nothing
  r1 = (m + 2u * half) >> (d + 1);
  t1 = (m & (4u * half - 1u)) == 2u * half;
}
__device__ __forceinline__ int exponent_of(float s) { return int((__float_as_uint(s) >> 23) & 0xffu) - 127; }

__device__ __forceinline__ int tail_bucket(float score, float low_score, float scale) {
  const float t = (low_score - score) * scale;                      // >= 0 for every tail term; monotonic in the score
  const int b = t >= float(kTailBuckets - 1) ? kTailBuckets - 1 : int(t);
  return b < 0 ? 0 : b;
}
// buckets per unit of score: the tail terms that can still move the sum lie within (k - 24) * ln 2 of the maximum
__device__ __forceinline__ float tail_scale(const HeadState& h) {
  const float lowest = h.max_score + float(exponent_of(h.sum) - 24) * 0.6931471805599453f - 0.01f;
  const float span = h.low_score - lowest;
  return span > 1e-6f ? float(kTailBuckets) / span : 0.0f;
}

// ---- fp32 running sums in index order, by the whole thread block.
// vals[0 .. n) holds non-negative terms in descending order; on return vals[i] = fl(... fl(fl(vals[0] + vals[1]) +
// vals[2]) ... + vals[i]), bit for bit what one thread adding them in order computes -- the reference's order -- and
// *total the last of them.  The same observation as for the tail: while the sum S = M * 2^(k-23) stays inside one
// power of two, adding a term moves M by round(term / 2^(k-23)), whatever M is, except when the quotient falls on a
// half (then the parity of M decides: a tie) -- so inside one power of two the sums are a prefix sum of integers,
// corrected at the few ties, which one thread walks in order.  The first terms (large against the sum: ties are
// the rule there) and every term that carries the sum into the next power of two are added in fp32 by one thread.
// kThreads * kPer >= n; every thread of the block calls this.  More than kMaxTies ties inside one power of two: the
// rest is added serially (always correct, never seen on real rows).
constexpr int kSerialFirst = 64, kMaxTies = 64;
constexpr unsigned int kIncrementCap = 1u << 26;   // sums of increments saturate here: beyond 2^24 they only say "crossed"
__device__ __forceinline__ unsigned int add_capped(unsigned int a, unsigned int b) {
  const unsigned int c = a + b;                    // both <= the cap: no wrap
  return c < kIncrementCap ? c : kIncrementCap;
}
struct TieRecord { int index; unsigned int before, increment; };

template <int kThreads, int kPer>
__device__ void ordered_sums_block(float* vals, int n, float* total) {
  constexpr int kWarps = kThreads / 32;
  __shared__ unsigned int warp_sums[kWarps];
  __shared__ float seg_sum;
  __shared__ int seg_start, tie_count, event_count, cross, serial_rest;
  __shared__ TieRecord ties[kMaxTies];
  __shared__ int events[kMaxTies];
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  if (t == 0) {
    float s = 0.0f;
    const int first = n < kSerialFirst ? n : kSerialFirst;
    for (int i = 0; i < first; ++i) { s += vals[i]; vals[i] = s; }
    seg_sum = s;
    seg_start = first;
    serial_rest = (s > 0.0f && s <= 3.0e38f) ? 0 : 1;   // nothing to decompose in a zero, infinite or NaN sum
    if (serial_rest != 0) {
      for (int i = first; i < n; ++i) { s += vals[i]; vals[i] = s; }
      seg_sum = s;
      seg_start = n;
    }
  }
  __syncthreads();
  for (;;) {
    const int i0 = seg_start;
    if (i0 >= n) break;
    const float S = seg_sum;
    const unsigned int M = (__float_as_uint(S) & 0x7fffffu) | 0x800000u;
    const int k = exponent_of(S);
    if (t == 0) { tie_count = 0; event_count = 0; cross = n; }
    // this thread's terms: kPer consecutive ones
    unsigned int inc[kPer], tie_mask = 0u, mine = 0u;
#pragma unroll
    for (int q = 0; q < kPer; ++q) {
      const int j = t * kPer + q;
      inc[q] = 0u;
      if (j >= i0 && j < n) {
        bool tie;
        term_increment(vals[j], k, inc[q], tie);
        if (inc[q] > kIncrementCap) inc[q] = kIncrementCap;
        if (tie) tie_mask |= 1u << q;
      }
      mine = add_capped(mine, inc[q]);
    }
    // exclusive scan of the threads' sums over the block
    unsigned int scan = mine;
#pragma unroll
    for (int offset = 1; offset < 32; offset <<= 1) {
      const unsigned int up = __shfl_up_sync(0xffffffffu, scan, offset);
      if (lane >= offset) scan = add_capped(scan, up);
    }
    if (lane == 31) warp_sums[warp] = scan;
    __syncthreads();                                  // also: tie_count, event_count, cross are reset
    unsigned int before = scan - mine;                // exclusive within the warp (no cap was hit unless scan is at the cap: then "crossed" anyway)
    if (scan >= kIncrementCap) before = kIncrementCap;
    for (int w = 0; w < warp; ++w) before = add_capped(before, warp_sums[w]);
    unsigned int pref[kPer];                          // increments up to and including the term
#pragma unroll
    for (int q = 0; q < kPer; ++q) {
      if (tie_mask >> q & 1u) {
        const int slot = atomicAdd(&tie_count, 1);
        if (slot < kMaxTies) ties[slot] = TieRecord{t * kPer + q, before, inc[q]};
      }
      before = add_capped(before, inc[q]);
      pref[q] = before;
    }
    __syncthreads();
    if (t == 0) {
      const int count = tie_count;
      if (count > kMaxTies) {
        serial_rest = 1;
      } else {
        for (int a = 1; a < count; ++a) {             // by index: the order in which the sum meets them
          const TieRecord x = ties[a];
          int b = a - 1;
          for (; b >= 0 && ties[b].index > x.index; --b) ties[b + 1] = ties[b];
          ties[b + 1] = x;
        }
        unsigned int corrected = 0u;
        int found = 0;
        for (int a = 0; a < count; ++a) {
          const unsigned int m_before = M + ties[a].before - corrected, q = ties[a].increment - 1u;
          if (m_before + q >= (1u << 24)) break;      // at or beyond the next power of two: the serial step below takes over
          if (((m_before + q) & 1u) == 0u) { ++corrected; events[found++] = ties[a].index; }   // half-way rounds to the even side: down
        }
        event_count = found;
      }
    }
    __syncthreads();
    if (serial_rest != 0) {
      if (t == 0) {
        float s = S;
        for (int i = i0; i < n; ++i) { s += vals[i]; vals[i] = s; }
        seg_sum = s;
        seg_start = n;
      }
      __syncthreads();
      break;
    }
    const int found = event_count;
    unsigned int sums[kPer];
#pragma unroll
    for (int q = 0; q < kPer; ++q) {
      const int j = t * kPer + q;
      unsigned int corrected = 0u;
      for (int a = 0; a < found; ++a) corrected += events[a] <= j ? 1u : 0u;
      sums[q] = add_capped(M, pref[q]) - corrected;
      if (j >= i0 && j < n && sums[q] >= (1u << 24)) { atomicMin(&cross, j); break; }   // later ones are larger still
    }
    __syncthreads();
    const int c = cross;
#pragma unroll
    for (int q = 0; q < kPer; ++q) {
      const int j = t * kPer + q;
      if (j >= i0 && j < c) vals[j] = __uint_as_float((uint32_t(k + 127) << 23) | (sums[q] & 0x7fffffu));
    }
    __syncthreads();
    if (t == 0) {
      const float last = c > i0 ? vals[c - 1] : S;
      if (c < n) {
        const float s = last + vals[c];             // the term that reaches the next power of two: one fp32 addition
        vals[c] = s;
        seg_sum = s;
        seg_start = c + 1;
      } else {
        seg_sum = last;
        seg_start = n;
      }
    }
    __syncthreads();
  }
  if (t == 0) *total = seg_sum;
  __syncthreads();
}

// The running sums alone, one row of at most kTile terms per thread block (b2_ordered_sums).
__global__ void __launch_bounds__(kRegThreads)
ordered_sums_kernel(const float* terms, int64_t n, float* sums) {
  dependent_launch_prologue();
  __shared__ __align__(16) float vals[kTile];
  __shared__ float total;
  const float* src = terms + int64_t(blockIdx.x) * n;
  for (int j = threadIdx.x; j < kTile; j += kRegThreads) vals[j] = j < n ? src[j] : 0.0f;
  __syncthreads();
  ordered_sums_block<kRegThreads, kRegKeys>(vals, int(n), &total);
  float* dst = sums + int64_t(blockIdx.x) * n;
  for (int j = threadIdx.x; j < n; j += kRegThreads) dst[j] = vals[j];
}

// head: the row's candidates (at most one 4096-key tile of them) are sorted in registers (the network of the whole-row
// sort's tile kernel), written to the front of the row's key area for the finish kernel, and their exponentials
// are summed in the reference's order (ordered_sums_block above), every running sum kept.  One kernel: the keys go from the candidate list
// through registers and shared memory to the sums without a round trip through global memory in between.
__global__ void __launch_bounds__(kRegThreads)
topp_head_kernel(unsigned long long* keys, int64_t padded, const CutState* cut, const unsigned long long* candidates,
                 unsigned int* tails, float* running, HeadState* heads, int* row_flags) {
  dependent_launch_prologue();
  __shared__ unsigned long long tile[kTile];
  __shared__ float carry;
  const int64_t row = blockIdx.x;
  const int t = threadIdx.x, lane = t & 31;
  // the tail pass adds into these: they start at zero
  unsigned int* tail = tails + row * int64_t(3 * kTailBuckets);
  for (int i = t; i < 3 * kTailBuckets; i += kRegThreads) tail[i] = 0u;
  if (row_flags[row] != 0) return;
  const unsigned int taken = cut[row].taken;
  if (taken < unsigned(kMinHead) || taken > unsigned(kTile)) {
    if (t == 0) row_flags[row] = 1;
    return;
  }
  const int count = int(taken);
  const unsigned long long* in = candidates + row * int64_t(kCandidates);
  unsigned long long key[kRegKeys];
#pragma unroll
  for (int r = 0; r < kRegKeys; ++r) key[r] = r * kRegThreads + t < count ? in[r * kRegThreads + t] : 0ull;   // layout S
  const int64_t first_global = int64_t(t) * kRegKeys;
  layout_s_to_b(key, tile, t);
  for (int64_t k = 2; k <= kTile; k <<= 1) {
    const int top = int(k >> 1);
    if (top >= 512) {
      layout_b_to_s(key, tile, t);
      steps_in_registers_s(key, 0, t, k, top);
      layout_s_to_b(key, tile, t);
    }
    if (top >= 16) steps_by_shuffle_b(key, first_global, k, top < 256 ? top : 256, lane);
    steps_in_registers_b(key, first_global, k, top < 8 ? top : 8);
  }
  layout_b_to_s(key, tile, t);
  __syncthreads();                                   // the transposes are done with the tile
  unsigned long long* dst = keys + row * padded;
#pragma unroll
  for (int r = 0; r < kRegKeys; ++r) dst[r * kRegThreads + t] = key[r];   // in order (layout S), for the finish kernel
  // the exponentials, in order, in the shared memory the sort no longer needs; then their running sums by the block
  __shared__ float bounds[2];                        // score of the first and of the last head token
  float* vals = reinterpret_cast<float*>(tile);
  if (t == 0) bounds[0] = key_score(key[0]);
#pragma unroll
  for (int r = 0; r < kRegKeys; ++r)
    if (r * kRegThreads + t == count - 1) bounds[1] = key_score(key[r]);
  __syncthreads();
  const float maximum = bounds[0];
#pragma unroll
  for (int r = 0; r < kRegKeys; ++r) {
    const int j = r * kRegThreads + t;
    vals[j] = j < count ? expf(key_score(key[r]) - maximum) : 0.0f;
  }
  __syncthreads();
  ordered_sums_block<kRegThreads, kRegKeys>(vals, count, &carry);
  float* cum = running + row * padded;
  for (int j = t; j < count; j += kRegThreads) cum[j] = vals[j];
  if (t == 0) heads[row] = HeadState{carry, maximum, bounds[1], count};
}

// tail: increments of every term below the head, per bucket, for the head's power of two and the next one.
// Per bucket one 64-bit word (increments under k + 1 << 32 | increments under k) and one word of tie flags
// (bit 0: a tie under k, bit 1: under k + 1).  A term of more than 4096 units does not belong in a tail (the sums of
// up to 2^18 of them must stay below 2^32): the row is handed to the whole-row sort.
constexpr unsigned int kMaxTailIncrement = 4096;   // times at most kMaxToppWidth terms: a bucket's sum fits 30 bits
constexpr int64_t kMaxToppWidth = int64_t(1) << 18;

template <typename T>
__global__ void __launch_bounds__(256, 6)
topp_tail_kernel(const T* logits, int64_t width, int64_t row_stride, float temperature, const CutState* cut,
                 const HeadState* heads, unsigned int* tails, int* row_flags) {
  dependent_launch_prologue();
  constexpr int N = Elem<T>::kPerVec, kVecs = 16 / N;          // 16 elements per thread and turn
  constexpr int kQueue = 256 * 16;
  // 32-bit words: shared memory adds those natively.  A thread block's sums stay below 2^29 (at most 2^18 tokens of
  // at most 2^11 units under the doubled unit), so the two tie flags ride in bits 30 and 31 of local1
  __shared__ unsigned int local0[kTailBuckets], local1[kTailBuckets];
  __shared__ float queue[kQueue];
  __shared__ unsigned int queued;
  const int64_t row = blockIdx.y;
  if (row_flags[row] != 0) return;
  for (int i = threadIdx.x; i < kTailBuckets; i += 256) { local0[i] = 0u; local1[i] = 0u; }
  if (threadIdx.x == 0) queued = 0u;
  __syncthreads();
  const HeadState h = heads[row];
  const float threshold = cut[row].threshold, scale = tail_scale(h);
  const int k = exponent_of(h.sum);
  // a hair below the score at which the increments vanish (e < 2^(k-24) adds less than half a unit; the margin
  // covers the roundings of the subtraction and of expf, and the exact test is made on e itself)
  const float lowest = h.max_score + float(k - 24) * 0.6931471805599453f - 0.01f;
  // Only a quarter of the tokens lie between that point and the head, scattered over every warp: a warp that took the
  // slow path (division, exponential, increments, atomics) whenever one lane needs it would take it always.  So a
  // turn first only SELECTS, with one comparison per token against a cut-off in logit units (a little below
  // lowest * temperature: the exact test follows), and queues the selected logits; then all threads work the queue.
  const float cut_logit = lowest * temperature - 1e-5f * fabsf(lowest * temperature) - 1e-30f;
  bool broken = false;
  const T* src = logits + row * row_stride;
  const int lane = threadIdx.x & 31;
  auto select = [&](float x) {
    const bool take = x < threshold && x >= cut_logit;
    const unsigned int votes = __ballot_sync(0xffffffffu, take);
    if (votes == 0u) return;
    unsigned int base = 0u;
    if (lane == 0) base = atomicAdd(&queued, unsigned(__popc(votes)));
    base = __shfl_sync(0xffffffffu, base, 0);
    if (take) queue[base + __popc(votes & ((1u << lane) - 1u))] = x;
  };
  auto work_queue = [&]() {
    __syncthreads();
    const unsigned int n = queued;
    for (unsigned int q = threadIdx.x; q < n; q += 256) {
      const float score = temperature == 1.0f ? queue[q] : __fdiv_rn(queue[q], temperature);
      if (score < lowest) continue;
      const float e = expf(score - h.max_score);
      unsigned int r0, r1;
      bool t0, t1;
      term_increments(e, k, r0, t0, r1, t1);
      if (r0 > kMaxTailIncrement) { broken = true; continue; }
      if ((r0 | r1) == 0u && !t0 && !t1) continue;                 // cannot move the sum under either power of two
      const int b = tail_bucket(score, h.low_score, scale);
      if (r0 != 0u) atomicAdd(&local0[b], r0);
      if (r1 != 0u) atomicAdd(&local1[b], r1);
      if (t0 || t1) atomicOr(&local1[b], (t0 ? 1u << 30 : 0u) | (t1 ? 1u << 31 : 0u));
    }
    __syncthreads();
    if (threadIdx.x == 0) queued = 0u;
    __syncthreads();
  };
  const int64_t first = int64_t(blockIdx.x) * 256 + threadIdx.x, stride = int64_t(gridDim.x) * 256;
  if (aligned16(src)) {
    const int64_t nvec = width / N;
    const uint4* vp = reinterpret_cast<const uint4*>(src);
    // every thread of the block takes the same number of turns (the ballots and barriers need them all)
    const int64_t turns = (nvec + stride * kVecs - 1) / (stride * kVecs);
    for (int64_t turn = 0; turn < turns; ++turn) {
      const int64_t v0 = first + turn * stride * kVecs;
      uint4 r[kVecs];
#pragma unroll
      for (int q = 0; q < kVecs; ++q) r[q] = v0 + q * stride < nvec ? ld_stream(vp + v0 + q * stride) : make_uint4(0u, 0u, 0u, 0u);
      // count this thread's 16 tokens first; the warp then takes room in the queue with ONE atomic (a ballot and
      // an atomic per token cost more instructions than the comparison they serve)
      float e[kVecs][N];
      unsigned int hits = 0u, count = 0u;
#pragma unroll
      for (int q = 0; q < kVecs; ++q) {
        Elem<T>::unpack(r[q], e[q]);
        const bool in = v0 + q * stride < nvec;
#pragma unroll
        for (int z = 0; z < N; ++z)
          if (in && e[q][z] < threshold && e[q][z] >= cut_logit) { hits |= 1u << (q * N + z); ++count; }
      }
      if (__any_sync(0xffffffffu, count != 0u)) {
        unsigned int before = count;
#pragma unroll
        for (int offset = 1; offset < 32; offset <<= 1) {
          const unsigned int up = __shfl_up_sync(0xffffffffu, before, offset);
          if (lane >= offset) before += up;
        }
        const unsigned int total = __shfl_sync(0xffffffffu, before, 31);
        unsigned int base = 0u;
        if (lane == 0) base = atomicAdd(&queued, total);
        unsigned int slot = __shfl_sync(0xffffffffu, base, 0) + before - count;
#pragma unroll
        for (int q = 0; q < kVecs; ++q) {
#pragma unroll
          for (int z = 0; z < N; ++z)
            if (hits >> (q * N + z) & 1u) queue[slot++] = e[q][z];
        }
      }
      work_queue();
    }
    const int64_t tail_turns = (width - nvec * N + stride - 1) / stride;
    for (int64_t turn = 0; turn < tail_turns; ++turn) {
      const int64_t i = nvec * N + first + turn * stride;
      select(i < width ? Elem<T>::load(src + i) : INFINITY);
    }
  } else {
    const int64_t turns = (width + stride * 16 - 1) / (stride * 16);
    for (int64_t turn = 0; turn < turns; ++turn) {
      for (int q = 0; q < 16; ++q) {
        const int64_t i = first + (turn * 16 + q) * stride;
        select(i < width ? Elem<T>::load(src + i) : INFINITY);
      }
      work_queue();
    }
  }
  work_queue();
  if (broken) row_flags[row] = 2;           // (the values only tell the reasons apart for a reader of the flags)
  // global layout per row: [0, 2 kTailBuckets) the 64-bit sums, [2 kTailBuckets, 3 kTailBuckets) the tie flags
  unsigned int* tail = tails + row * int64_t(3 * kTailBuckets);
  unsigned long long* sums = reinterpret_cast<unsigned long long*>(tail);
  for (int i = threadIdx.x; i < kTailBuckets; i += 256) {
    const unsigned int ties = local1[i] >> 30;
    const unsigned long long both = (static_cast<unsigned long long>(local1[i] & 0x3fffffffu) << 32) | local0[i];
    if (both != 0ull) atomicAdd(&sums[i], both);
    if (ties != 0u) atomicOr(&tail[2 * kTailBuckets + i], ties);
  }
}

// finish: the walk over the buckets (exact where the order matters), then the reference's top-p walk and pick over the head
template <typename T>
__global__ void __launch_bounds__(kSortThreads)
topp_finish_kernel(const T* logits, int64_t width, int64_t row_stride, float temperature, const CutState* cut,
                   const unsigned long long* keys, int64_t padded, const float* running, const unsigned int* tails,
                   const HeadState* heads, float top_p, unsigned long long seed, const unsigned long long* draw_offsets,
                   int32_t* out_ids, int* row_flags) {
  dependent_launch_prologue();
  constexpr int kGroup = 64, kGroups = kTailBuckets / kGroup;   // the walk first steps over groups of 64 buckets
  __shared__ __align__(16) unsigned long long bucket_keys[kTailBuckets];
  __shared__ unsigned long long sums[kTailBuckets];          // (increments under k0 + 1) << 32 | (increments under k0)
  __shared__ unsigned int ties[kTailBuckets];
  __shared__ unsigned long long group_sums[kGroups];
  __shared__ unsigned int group_ties[kGroups];
  __shared__ float carry;
  __shared__ unsigned int walk_m;
  __shared__ int walk_k, walk_bucket, found, give_up;
  __shared__ unsigned int gathered;
  const int64_t row = blockIdx.x;
  if (row_flags[row] != 0) return;
  const int tid = threadIdx.x;
  const HeadState h = heads[row];
  {
    const unsigned int* tail = tails + row * int64_t(3 * kTailBuckets);
    const unsigned long long* tail_sums = reinterpret_cast<const unsigned long long*>(tail);
    for (int i = tid; i < kTailBuckets; i += kSortThreads) { sums[i] = tail_sums[i]; ties[i] = tail[2 * kTailBuckets + i]; }
  }
  __syncthreads();
  if (tid < kGroups) {
    unsigned long long total = 0ull;
    unsigned int any = 0u;
    for (int i = 0; i < kGroup; ++i) { total += sums[tid * kGroup + i]; any |= ties[tid * kGroup + i]; }
    group_sums[tid] = total;      // each half stays below 2^32: at most 2^18 terms of at most 4096 units
    group_ties[tid] = any;
  }
  const float threshold = cut[row].threshold, scale = tail_scale(h);
  const int k0 = exponent_of(h.sum);
  const float lowest = h.max_score + float(k0 - 24) * 0.6931471805599453f - 0.01f;   // as in the tail pass
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
      while (b < kTailBuckets) {
        if (k > k0 + 1) { give_up = 1; break; }
        const int shift = k == k0 ? 0 : 32;
        const unsigned int tie_bit = k == k0 ? 1u : 2u;
        if ((b & (kGroup - 1)) == 0) {        // a whole group at once when nothing in it needs the order
          const int g = b / kGroup;
          const unsigned long long r = (group_sums[g] >> shift) & 0xffffffffull;
          if ((group_ties[g] & tie_bit) == 0u && m + r < (1ull << 24)) { m += unsigned(r); b += kGroup; continue; }
        }
        const unsigned long long r = (sums[b] >> shift) & 0xffffffffull;
        if ((ties[b] & tie_bit) != 0u || m + r > (1ull << 24)) break;   // the order inside this bucket matters
        m += unsigned(r);
        if (m == (1u << 24)) { m = 1u << 23; ++k; }
        ++b;
      }
      walk_m = m; walk_k = k; walk_bucket = b;
      gathered = 0u;
    }
    __syncthreads();
    if (give_up != 0) { if (tid == 0) row_flags[row] = 3; return; }
    const int b = walk_bucket;
    if (b >= kTailBuckets) break;
    // gather the terms of bucket b that can move the sum, sort them into the reference's order, add them one by one
    // the bucket's range in logit units, a little wide (the exact test follows): most tokens leave after two comparisons
    const float score_hi = h.low_score - float(b) / scale, score_lo = h.low_score - float(b + 1) / scale;
    const float slack = 1e-5f * (fabsf(score_hi) + fabsf(score_lo)) + 2.0f / scale * 1e-3f;
    const float logit_a = (score_hi + slack) * temperature, logit_b = (score_lo - slack) * temperature;
    const float logit_hi = fmaxf(logit_a, logit_b) + 1e-5f * fabsf(fmaxf(logit_a, logit_b)) + 1e-30f;
    const float logit_lo = fminf(logit_a, logit_b) - 1e-5f * fabsf(fminf(logit_a, logit_b)) - 1e-30f;
    const bool last_bucket = b == kTailBuckets - 1;   // it also takes everything below its range
    auto consider = [&](float x, int64_t i) {
      if (x >= threshold || x > logit_hi || (x < logit_lo && !last_bucket)) return;
      const float score = temperature == 1.0f ? x : __fdiv_rn(x, temperature);
      if (score < lowest || tail_bucket(score, h.low_score, scale) != b) return;
      const float e = expf(score - h.max_score);
      unsigned int r0, r1;
      bool t0, t1;
      term_increments(e, k0, r0, t0, r1, t1);
      if ((r0 | r1) == 0u && !t0 && !t1) return;
      const unsigned int slot = atomicAdd(&gathered, 1u);
      if (slot < unsigned(kTailBuckets)) bucket_keys[slot] = sample_key(score, uint32_t(i));
    };
    {
      constexpr int N = Elem<T>::kPerVec;
      if (aligned16(src)) {
        const int64_t nvec = width / N;
        const uint4* vp = reinterpret_cast<const uint4*>(src);
        for (int64_t v0 = tid; v0 < nvec; v0 += int64_t(kSortThreads) * 8) {   // eight loads in flight per thread
          uint4 r[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) if (v0 + q * kSortThreads < nvec) r[q] = ld_stream(vp + v0 + q * kSortThreads);
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const int64_t v = v0 + q * kSortThreads;
            if (v < nvec) {
              float e[N];
              Elem<T>::unpack(r[q], e);
#pragma unroll
              for (int z = 0; z < N; ++z) consider(e[z], v * N + z);
            }
          }
        }
        for (int64_t i = nvec * N + tid; i < width; i += kSortThreads) consider(Elem<T>::load(src + i), i);
      } else {
        for (int64_t i = tid; i < width; i += kSortThreads) consider(Elem<T>::load(src + i), i);
      }
    }
    __syncthreads();
    const unsigned int count = gathered;
    if (count > unsigned(kTailBuckets)) { if (tid == 0) row_flags[row] = 4; return; }
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
  float* stage = reinterpret_cast<float*>(bucket_keys);   // the gathered keys are no longer needed: kTile floats fit their place
  __syncthreads();

  // the reference's top-p walk (src/ops_cuda.cu:596-603) over the head; it must end strictly above the head's lowest score
  const unsigned long long* sorted = keys + row * padded;
  const float* cum = running + row * padded;
  const int limit = h.count;
  // the masses in order, their running sums by the whole block (ordered_sums_block: the serial walk's additions, bit
  // for bit), then the first index at which the running mass reaches top_p
  for (int j = tid; j < kTile; j += kSortThreads)
    stage[j] = j < limit ? __fdiv_rn(expf(key_score(sorted[j]) - h.max_score), total) : 0.0f;
  if (tid == 0) found = limit;
  __syncthreads();
  ordered_sums_block<kSortThreads, kTile / kSortThreads>(stage, limit, &carry);
  for (int j = tid; j < limit; j += kSortThreads)
    if (stage[j] >= top_p) { atomicMin(&found, j); break; }   // the sums never decrease: a thread's first hit is its lowest
  __syncthreads();
  const int prefix = found < limit ? found + 1 : -1;
  if (prefix < 0 || !(key_score(sorted[prefix - 1]) > h.low_score)) {   // not settled inside the head: the whole-row path decides
    if (tid == 0) row_flags[row] = 5;
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
int launch_ordered_sums(const float* terms, int64_t rows, int64_t n, float* sums, cudaStream_t s) {
  if (rows == 0 || n == 0) return B2_OK;
  launch_kernel(ordered_sums_kernel, dim3(unsigned(rows)), dim3(kRegThreads), 0, s, terms, n, sums);
  return launch_status("ordered_sums");
}

size_t sampler_workspace_bytes(int64_t rows, int64_t width) {
  const int64_t padded = padded_width(width);
  const size_t per_row = size_t(padded) * 12 + size_t(kCandidates) * 8 + size_t(3 * kTailBuckets) * 4 + sizeof(CutState) +
                         sizeof(HeadState) + 2 * sizeof(int);
  return (size_t(rows) * per_row + 32 + 255) / 256 * 256;
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
  // thread blocks per row for a pass over the logits: as many as run at once over all rows (asked of the occupancy
  // calculator per kernel), so the pass is one wave and no block waits for a slot
  auto row_grid_of = [&](auto kernel) {
    int resident = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, kernel, 256, 0) != cudaSuccess || resident < 1) {
      cudaGetLastError();
      resident = 4;
    }
    int64_t spread = int64_t(sm_count()) * resident / rows;
    if (spread > padded / 1024) spread = padded / 1024;
    if (spread < 1) spread = 1;
    return dim3(unsigned(spread), unsigned(rows), 1);
  };
  // logits / temperature stays a normal number near a threshold only for a moderate temperature (and a moderate
  // logit there, which the splitter kernel checks)
  const int safe = temperature >= 9.5367431640625e-07f && temperature <= 1048576.0f;   // 2^-20 .. 2^20
  const ChainArgs chain{logits, dtype, width, row_stride, padded, temperature, top_k, top_p, seed, draw_offsets, keys, running, out_ids};

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
      launch_kernel(topk_splitter_kernel<float>, dim3(unsigned(rows)), dim3(kSplitThreads), 0, s, x, width, row_stride, unsigned(top_k), safe, cut, overflow, 0);
      launch_kernel(topk_gather_kernel<float>, dim3(row_grid_of(topk_gather_kernel<float>)), dim3(256), 0, s, x, width, row_stride, temperature, cut, candidates, overflow, 0);
    } else {
      const __half* x = static_cast<const __half*>(logits);
      launch_kernel(topk_splitter_kernel<__half>, dim3(unsigned(rows)), dim3(kSplitThreads), 0, s, x, width, row_stride, unsigned(top_k), safe, cut, overflow, 0);
      launch_kernel(topk_gather_kernel<__half>, dim3(row_grid_of(topk_gather_kernel<__half>)), dim3(256), 0, s, x, width, row_stride, temperature, cut, candidates, overflow, 0);
    }
    launch_kernel(topk_finish_kernel, dim3(unsigned(rows)), dim3(kSortThreads), kCandidates * 8, s, keys, padded, top_k, cut, candidates, overflow);
    // ... unless that could not be trusted: then (and only then) the radix select over all 64 key bits redoes every row
    if (dtype == B2_F32)
      launch_kernel(topk_exact_kernel<float>, dim3(unsigned(rows)), dim3(kExactThreads), 0, s, static_cast<const float*>(logits), width, row_stride, padded,
                                                                        temperature, top_k, keys, overflow);
    else
      launch_kernel(topk_exact_kernel<__half>, dim3(unsigned(rows)), dim3(kExactThreads), 0, s, static_cast<const __half*>(logits), width, row_stride,
                                                                         padded, temperature, top_k, keys, overflow);
  } else {
    if (top_k == 0 && top_p < 1.0f && width >= 4 * kCandidates && width <= kMaxToppWidth) {
      // top-p over the whole vocabulary: head sorted, tail summed by buckets; rows that do not fit that scheme raise
      // their flag and are the only ones the whole-row sort below still works on
      if (cudaMemsetAsync(row_flags, 0, size_t(rows) * sizeof(int), s) != cudaSuccess) return launch_status("sample_rows");
      if (dtype == B2_F32) {
        const float* x = static_cast<const float*>(logits);
        launch_kernel(topk_splitter_kernel<float>, dim3(unsigned(rows)), dim3(kSplitThreads), 0, s, x, width, row_stride, 0u, safe, cut, row_flags, 1);
        launch_kernel(topk_gather_kernel<float>, dim3(row_grid_of(topk_gather_kernel<float>)), dim3(256), 0, s, x, width, row_stride, temperature, cut, candidates, row_flags, 1);
        launch_kernel(topp_head_kernel, dim3(unsigned(rows)), dim3(kRegThreads), 0, s, keys, padded, cut, candidates, tails, running, heads, row_flags);
        launch_kernel(topp_tail_kernel<float>, dim3(row_grid_of(topp_tail_kernel<float>)), dim3(256), 0, s, x, width, row_stride, temperature, cut, heads, tails, row_flags);
        launch_kernel(topp_finish_kernel<float>, dim3(unsigned(rows)), dim3(kSortThreads), 0, s, x, width, row_stride, temperature, cut, keys, padded, running,
                                                                          tails, heads, top_p, seed, draw_offsets, out_ids, row_flags);
      } else {
        const __half* x = static_cast<const __half*>(logits);
        launch_kernel(topk_splitter_kernel<__half>, dim3(unsigned(rows)), dim3(kSplitThreads), 0, s, x, width, row_stride, 0u, safe, cut, row_flags, 1);
        launch_kernel(topk_gather_kernel<__half>, dim3(row_grid_of(topk_gather_kernel<__half>)), dim3(256), 0, s, x, width, row_stride, temperature, cut, candidates, row_flags, 1);
        launch_kernel(topp_head_kernel, dim3(unsigned(rows)), dim3(kRegThreads), 0, s, keys, padded, cut, candidates, tails, running, heads, row_flags);
        launch_kernel(topp_tail_kernel<__half>, dim3(row_grid_of(topp_tail_kernel<__half>)), dim3(256), 0, s, x, width, row_stride, temperature, cut, heads, tails, row_flags);
        launch_kernel(topp_finish_kernel<__half>, dim3(unsigned(rows)), dim3(kSortThreads), 0, s, x, width, row_stride, temperature, cut, keys, padded, running,
                                                                           tails, heads, top_p, seed, draw_offsets, out_ids, row_flags);
      }
      // the rows whose flag is up go through the whole-row route, launched from the device if there are any
      return launch_sampler_rows_fallback(row_flags, rows, overflow + 4, overflow + 1, logits, dtype, width, row_stride, padded, temperature,
                                          top_k, top_p, seed, draw_offsets, keys, running, out_ids, s);
    }
    whole_row_chain(chain, RowSet{nullptr, nullptr}, unsigned(rows), s);
    return launch_status("sample_rows");
  }
  launch_kernel(sampler_pick_kernel, dim3(unsigned(rows)), dim3(kSelectThreads), 0, s, keys, width, padded, top_k, top_p, seed, draw_offsets, running,
                out_ids, RowSet{nullptr, nullptr});
  return launch_status("sample_rows");
}

}  // namespace b2
