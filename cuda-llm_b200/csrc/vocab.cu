// Vocabulary-wide row reductions for sm_100a: argmax and softmax over logits
// [rows, width] with width ~ 150k.
//
// argmax   one pass over HBM.  A row is split over several CTAs so that few rows
//          still fill the machine; each CTA folds its slice to one packed
//          (value, index) key and merges it with a 64-bit atomicMax; the last CTA
//          of a row (atomic ticket) publishes the result and re-zeroes the scratch.
// softmax  fast mode keeps a whole row on chip: a thread-block cluster of up to 8
//          CTAs holds it in distributed shared memory, exchanges the slice maxima
//          and sums through DSMEM, and writes the probabilities, so HBM sees one
//          read and one write.  Rows too long for that, and the vocabulary-sharded
//          multi-GPU form, use a statistics pass plus an apply pass.
//          Deterministic mode adds the exponentials in index order in fp32.
//
// Replaces reference kernels argmax_partial<T> + argmax_final (src/ops_cuda.cu:562-563,
// with two cudaMalloc, two cudaFree and a blocking copy per call, :711) and softk<T>
// (src/ops_cuda.cu:132: one thread per row, strided access).
#include "common.cuh"
#include "bulk_copy.cuh"
#include "exchange.cuh"
#include "kernels.h"
#include "b2ops.h"

#include <cfloat>
#include <climits>
#include <cooperative_groups.h>
#include <mutex>

namespace cg = cooperative_groups;

namespace b2 {
namespace {

// Calls f(value, i) for i in [0, n) of p[], every thread in ascending i.
// kVec: p is 16-byte aligned; 16-byte loads, four in flight per thread.
template <typename T, bool kVec, typename F>
__device__ __forceinline__ void scan_range(const T* p, int64_t n, F&& f) {
  constexpr int N = Elem<T>::kPerVec;
  if (kVec) {
    const int64_t nvec = n / N, step = blockDim.x;
    const uint4* vp = reinterpret_cast<const uint4*>(p);
    for (int64_t v0 = threadIdx.x; v0 < nvec; v0 += step * 4) {
      uint4 r[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) if (v0 + k * step < nvec) r[k] = ld_stream(vp + v0 + k * step);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int64_t v = v0 + k * step;
        if (v < nvec) {
          float e[N];
          Elem<T>::unpack(r[k], e);
#pragma unroll
          for (int q = 0; q < N; ++q) f(e[q], v * N + q);
        }
      }
    }
    for (int64_t i = nvec * N + threadIdx.x; i < n; i += step) f(Elem<T>::load(p + i), i);
  } else {
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) f(Elem<T>::load(p + i), i);
  }
}

// ===========================================================================
// argmax
// ===========================================================================

constexpr int kArgThreads = 256;
constexpr int kNoIndex = INT_MAX;
constexpr int64_t kMinChunk = 2048;

// The reference's replacement rule (src/ops_cuda.cu:562): larger value, or equal value
// and lower index.  (-FLT_MAX, kNoIndex) is "nothing seen" and never beats anything.
__device__ __forceinline__ bool beats(float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); }

// unsigned key whose order is (value ascending, index descending); 0 = nothing seen
__device__ __forceinline__ unsigned long long pack_key(float v, uint32_t global_index) {
  const uint32_t b = __float_as_uint(v);
  const uint32_t ordered = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
  return (static_cast<unsigned long long>(ordered) << 32) | (0xffffffffu - global_index);
}
constexpr unsigned long long kSignBit = 0x8000000000000000ull;

template <typename T, bool kVec>
__global__ void __launch_bounds__(kArgThreads)
argmax_rows_kernel(const T* logits, int64_t width, int64_t row_stride, int64_t chunk, int chunks,
                   int64_t index_base, int32_t* out_ids, int64_t* out_keys, unsigned long long* keys,
                   unsigned int* tickets) {
  __shared__ float warp_v[kArgThreads / kWarpSize];
  __shared__ int warp_i[kArgThreads / kWarpSize];
  const int64_t row = blockIdx.x / chunks;
  const int c = int(blockIdx.x - row * chunks);
  const int64_t lo = int64_t(c) * chunk;
  const int64_t n = width - lo < chunk ? width - lo : chunk;

  float bv = -FLT_MAX;
  int bi = kNoIndex;
  // ascending indices within a thread: strictly-greater alone keeps the lowest index
  scan_range<T, kVec>(logits + row * row_stride + lo, n, [&](float v, int64_t i) {
    if (v > bv) { bv = v; bi = int(lo + i); }
  });

#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    const float ov = __shfl_down_sync(0xffffffffu, bv, offset);
    const int oi = __shfl_down_sync(0xffffffffu, bi, offset);
    if (beats(ov, oi, bv, bi)) { bv = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { warp_v[warp] = bv; warp_i[warp] = bi; }
  __syncthreads();
  if (threadIdx.x != 0) return;
  for (int k = 1; k < kArgThreads / kWarpSize; ++k)
    if (beats(warp_v[k], warp_i[k], bv, bi)) { bv = warp_v[k]; bi = warp_i[k]; }

  unsigned long long key = bi == kNoIndex ? 0ull : pack_key(bv, uint32_t(index_base + bi));
  if (chunks > 1) {
    if (key != 0ull) atomicMax(keys + row, key);
    __threadfence();
    if (atomicAdd(tickets + row, 1u) != unsigned(chunks - 1)) return;
    __threadfence();
    key = atomicExch(keys + row, 0ull);  // read the merged key and leave the scratch zeroed
    tickets[row] = 0u;
  }
  if (out_keys != nullptr) out_keys[row] = static_cast<int64_t>(key ^ kSignBit);
  if (out_ids != nullptr) out_ids[row] = key == 0ull ? 0 : int32_t(0xffffffffu - uint32_t(key & 0xffffffffull));
}

// Vocabulary-sharded form with the exchange fused into the kernel: the same fold of this GPU's columns to
// one key per row; the thread block that finishes a row sends its key to every peer at once (the stores
// cross NVLink while the other rows are still being read), and the thread block that finishes the last
// row waits (bounded) for the peers' keys and writes the global winners' indices.
__device__ __forceinline__ int32_t winner_index(unsigned long long best) {   // 0 = no shard saw a candidate: index 0, like the reference
  return best == 0ull ? 0 : int32_t(0xffffffffu - uint32_t(best & 0xffffffffull));
}
constexpr int32_t kInvalidIndex = -1;   // written for rows whose exchange did not complete in time

// (the register cap keeps the occupancy of the plain kernel: what the rarely run tail needs beyond it spills)
template <typename T, bool kVec, int kBlock>
__global__ void __launch_bounds__(kBlock, kBlock >= 1024 ? 2 : 8)
argmax_rows_exchange_kernel(const T* logits, int64_t rows, int64_t width, int64_t row_stride, int64_t chunk, int chunks,
                            int64_t index_base, int32_t* out_ids, unsigned long long* keys, unsigned int* tickets,
                            const __grid_constant__ ExchangeArgs xa) {
  __shared__ float warp_v[kBlock / kWarpSize];
  __shared__ int warp_i[kBlock / kWarpSize];
  __shared__ unsigned long long row_key;
  __shared__ uint32_t call_epoch;
  __shared__ int state;   // 0: this row is not finished yet, 1: finished (send its key), 2: and it was the last row
  exchange_trace_start(xa);
  // the call's epoch, fetched under the scan of the row (the stored value changes only at the very end of a call,
  // when every thread block has long read it)
  uint32_t epoch = 0u;
  if (threadIdx.x == 0) epoch = exchange_call_epoch(xa);
  const int64_t row = blockIdx.x / chunks;
  const int c = int(blockIdx.x - row * chunks);
  const int64_t lo = int64_t(c) * chunk;
  const int64_t n = width - lo < chunk ? width - lo : chunk;

  float bv = -FLT_MAX;
  int bi = kNoIndex;
  scan_range<T, kVec>(logits + row * row_stride + lo, n, [&](float v, int64_t i) {
    if (v > bv) { bv = v; bi = int(lo + i); }
  });
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    const float ov = __shfl_down_sync(0xffffffffu, bv, offset);
    const int oi = __shfl_down_sync(0xffffffffu, bi, offset);
    if (beats(ov, oi, bv, bi)) { bv = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { warp_v[warp] = bv; warp_i[warp] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int k = 1; k < kBlock / kWarpSize; ++k)
      if (beats(warp_v[k], warp_i[k], bv, bi)) { bv = warp_v[k]; bi = warp_i[k]; }
    unsigned long long key = bi == kNoIndex ? 0ull : pack_key(bv, uint32_t(index_base + bi));
    bool row_finished = true;
    if (chunks > 1) {
      if (key != 0ull) atomicMax(keys + row, key);
      __threadfence();
      row_finished = atomicAdd(tickets + row, 1u) == unsigned(chunks - 1);
      if (row_finished) {
        __threadfence();
        key = atomicExch(keys + row, 0ull);  // read the merged key and leave the scratch zeroed
        tickets[row] = 0u;
      }
    }
    row_key = key;
    call_epoch = epoch;
    state = row_finished ? 1 : 0;
  }
  __syncthreads();
  if (state == 0) return;
  // the row's key leaves for the peers first (threads 1 .. world-1: one peer each) while thread 0 stores this GPU's
  // own slot and counts the row
  if (threadIdx.x > 0 && threadIdx.x < xa.world) exchange_send(xa, call_epoch, (xa.rank + threadIdx.x) % xa.world, row, row_key);
  if (threadIdx.x == 0) {
    exchange_send(xa, epoch, xa.rank, row, row_key);
    if (exchange_row_done(xa, rows)) state = 2;
  }
  __syncthreads();
  if (state != 2) return;
  exchange_tail(xa, rows, call_epoch, [&](int64_t r, bool complete, auto partial_of) {
    unsigned long long best = 0ull;
#pragma unroll
    for (int g = 0; g < kMaxWorld; ++g)
      if (g < xa.world) { const unsigned long long k = partial_of(g); best = k > best ? k : best; }
    out_ids[r] = complete ? winner_index(best) : kInvalidIndex;
  });
}

// The exchange alone, for keys that another kernel produced (the vocabulary-parallel LM head): one thread block
// sends this GPU's keys to every GPU's exchange buffer and runs the same wait-and-combine as above.
__global__ void __launch_bounds__(kArgThreads)
argmax_keys_exchange_kernel(const int64_t* keys, int64_t rows, int32_t* out_ids, const __grid_constant__ ExchangeArgs xa) {
  exchange_trace_start(xa);
  const uint32_t epoch = exchange_call_epoch(xa);
  for (int64_t r = threadIdx.x; r < rows; r += blockDim.x) {
    const unsigned long long key = static_cast<unsigned long long>(keys[r]) ^ kSignBit;
    for (int g = 0; g < xa.world; ++g) exchange_send(xa, epoch, (xa.rank + g) % xa.world, r, key);
  }
  __syncthreads();   // nobody rewrites the stored epoch (end of the tail) before every thread has read it
  exchange_tail(xa, rows, epoch, [&](int64_t r, bool complete, auto partial_of) {
    unsigned long long best = 0ull;
#pragma unroll
    for (int g = 0; g < kMaxWorld; ++g)
      if (g < xa.world) { const unsigned long long k = partial_of(g); best = k > best ? k : best; }
    out_ids[r] = complete ? winner_index(best) : kInvalidIndex;
  });
}

__global__ void argmax_decode_kernel(const int64_t* keys, int64_t rows, int32_t* out_ids) {
  const int64_t r = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  const unsigned long long key = static_cast<unsigned long long>(keys[r]) ^ kSignBit;
  out_ids[r] = key == 0ull ? 0 : int32_t(0xffffffffu - uint32_t(key & 0xffffffffull));
}

// ===========================================================================
// softmax
// ===========================================================================

constexpr int kSoftThreads = 512;
constexpr size_t kClusterSliceBytes = 100 * 1024;  // two CTAs of a cluster fit one SM's shared memory

// exp(x - m) in the fast paths is 2^(x*log2(e) - m*log2(e)): one fused multiply-add and one
// hardware exponential (ex2.approx, 2^-22 relative).  The rounding of m*log2(e) is a factor
// common to every element of the row, so it cancels in the normalisation.
constexpr float kLog2e = 1.4426950408889634f;
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Running (max, sum of exp(x - max)) of a stream of values, updated one small group at a time:
// one rescale per group instead of one per element.  Works on t = x*log2(e).
template <int COUNT>
__device__ __forceinline__ void online_update(float& m, float& m2, float& s, const float* x) {
  float t[COUNT];
  float gx = x[0];
#pragma unroll
  for (int q = 1; q < COUNT; ++q) gx = fmaxf(gx, x[q]);
#pragma unroll
  for (int q = 0; q < COUNT; ++q) t[q] = x[q] * kLog2e;
  m = fmaxf(m, gx);                                     // the maximum itself, in the units of x
  const float gm = gx * kLog2e;                         // rounding is monotonic: this is max(t[])
  if (gm > m2) { s *= fast_exp2(m2 - gm); m2 = gm; }   // first group: s = 0 * 2^(-inf) = 0
  if (m2 != -INFINITY) {                                // a run of leading -inf (masked) entries adds nothing
#pragma unroll
    for (int q = 0; q < COUNT; ++q) s += fast_exp2(t[q] - m2);
  }
}

// ---- fast mode: one cluster per row, the row stays in distributed shared memory.
//   load    kBulk: one thread issues bulk asynchronous copies (TMA) for the CTA's whole slice, so
//           all of it is in flight at once and no register holds it; otherwise 16-byte thread loads
//   pass A  running max over the slice in shared memory; slice max pushed into every CTA of the cluster
//   pass B  in place: e = 2^(x*log2e - max*log2e), running sum; slice sum pushed likewise
//   pass C  shared memory -> HBM: e * (1/sum), 16-byte stores
// Values cross CTAs by remote shared-memory stores (DSMEM) followed by a cluster barrier, so
// nothing reads a neighbour's memory after the last barrier and CTAs retire independently.
// `status` (may be null): bit 0 is raised if the bulk-copy wait ran out; outputs are then invalid.
constexpr int kMaxClusterRanks = 16;
constexpr int kDeviceSlots = 64;
constexpr uint32_t kBulkChunk = 16 * 1024;

template <typename T, bool kVec, bool kBulk>
__global__ void __launch_bounds__(kSoftThreads, 2)
softmax_cluster_kernel(const T* x, T* out, int64_t width, int64_t slice, int* status) {
  constexpr int N = Elem<T>::kPerVec;
  extern __shared__ __align__(128) float vals[];
  __shared__ float scratch[32];
  __shared__ float peer_max[kMaxClusterRanks], peer_sum[kMaxClusterRanks];   // written by the other CTAs
  __shared__ __align__(8) uint64_t load_barrier;

  cg::cluster_group cluster = cg::this_cluster();
  const unsigned rank = cluster.block_rank(), ranks = cluster.num_blocks();
  const int64_t row = blockIdx.x / ranks;
  const int64_t lo = int64_t(rank) * slice;
  const int n = int(lo >= width ? 0 : (width - lo < slice ? width - lo : slice));
  const T* src = x + row * width + lo;
  T* dst = out + row * width + lo;
  const int step = blockDim.x, tid = threadIdx.x;
  const int n4 = n >> 2;                       // whole float4 groups of the slice in shared memory
  float4* vals4 = reinterpret_cast<float4*>(vals);

  // ---- load
  if (kBulk) {
    if (tid == 0) {
      mbarrier_init(&load_barrier, 1);
      const uint32_t bytes = uint32_t(n4) * 16u;            // the 16-byte multiple; a tail of < 4 floats is loaded below
      mbarrier_expect_bytes(&load_barrier, bytes);
      for (uint32_t off = 0; off < bytes; off += kBulkChunk)
        bulk_load(reinterpret_cast<char*>(vals) + off, reinterpret_cast<const char*>(src) + off,
                  bytes - off < kBulkChunk ? bytes - off : kBulkChunk, &load_barrier);
    }
    for (int i = (n4 << 2) + tid; i < n; i += step) vals[i] = Elem<T>::load(src + i);
  } else if (kVec) {
    const int nvec = n / N;
    const uint4* vp = reinterpret_cast<const uint4*>(src);
    for (int v0 = tid; v0 < nvec; v0 += step * 4) {
      uint4 r[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) if (v0 + k * step < nvec) r[k] = ld_stream(vp + v0 + k * step);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int v = v0 + k * step;
        if (v < nvec) {
          float e[N];
          Elem<T>::unpack(r[k], e);
#pragma unroll
          for (int q = 0; q < N; q += 4) vals4[(v * N + q) >> 2] = make_float4(e[q], e[q + 1], e[q + 2], e[q + 3]);
        }
      }
    }
    for (int i = nvec * N + tid; i < n; i += step) vals[i] = Elem<T>::load(src + i);
  } else {
    for (int i = tid; i < n; i += step) vals[i] = Elem<T>::load(src + i);
  }
  // every CTA of the cluster is running (and this CTA's barrier is initialised) before anyone
  // polls or writes into a neighbour's shared memory
  cluster.sync();
  bool load_ok = true;
  if (kBulk) {
    load_ok = mbarrier_wait_bounded(&load_barrier, 0);
    if (!load_ok && tid == 0 && status != nullptr) atomicOr(status, 1);
  }

  // ---- pass A
  float m0 = -INFINITY, m1 = -INFINITY;
  for (int g = tid; g < n4; g += step) {
    const float4 t = vals4[g];
    m0 = fmaxf(m0, fmaxf(t.x, t.y));
    m1 = fmaxf(m1, fmaxf(t.z, t.w));
  }
  for (int i = (n4 << 2) + tid; i < n; i += step) m0 = fmaxf(m0, vals[i]);
  const float slice_max = block_max(fmaxf(m0, m1), scratch);
  if (tid < int(ranks)) *cluster.map_shared_rank(&peer_max[rank], tid) = slice_max;
  cluster.sync();
  float row_max = -INFINITY;
  for (unsigned r = 0; r < ranks; ++r) row_max = fmaxf(row_max, peer_max[r]);
  const float neg_m2 = -row_max * kLog2e;

  // ---- pass B
  float s0 = 0.0f, s1 = 0.0f;
  for (int g = tid; g < n4; g += step) {
    float4 t = vals4[g];
    t.x = fast_exp2(fmaf(t.x, kLog2e, neg_m2)); t.y = fast_exp2(fmaf(t.y, kLog2e, neg_m2));
    t.z = fast_exp2(fmaf(t.z, kLog2e, neg_m2)); t.w = fast_exp2(fmaf(t.w, kLog2e, neg_m2));
    vals4[g] = t;
    s0 += t.x + t.y;
    s1 += t.z + t.w;
  }
  for (int i = (n4 << 2) + tid; i < n; i += step) { const float e = fast_exp2(fmaf(vals[i], kLog2e, neg_m2)); vals[i] = e; s0 += e; }
  const float slice_sum = block_sum(s0 + s1, scratch);
  if (tid < int(ranks)) *cluster.map_shared_rank(&peer_sum[rank], tid) = slice_sum;
  cluster.sync();
  float row_sum = 0.0f;
  for (unsigned r = 0; r < ranks; ++r) row_sum += peer_sum[r];   // rank order: the same sum on every CTA of the row
  const float inv_sum = 1.0f / row_sum;

  // ---- pass C
  if (kVec) {
    const int nvec = n / N;
    for (int v = tid; v < nvec; v += step) {
      float o[N];
#pragma unroll
      for (int q = 0; q < N; q += 4) {
        const float4 t = vals4[(v * N + q) >> 2];
        o[q] = t.x * inv_sum; o[q + 1] = t.y * inv_sum; o[q + 2] = t.z * inv_sum; o[q + 3] = t.w * inv_sum;
      }
      st_stream(reinterpret_cast<uint4*>(dst) + v, Elem<T>::pack(o));
    }
    for (int i = nvec * N + tid; i < n; i += step) Elem<T>::store(dst + i, vals[i] * inv_sum);
  } else {
    for (int i = tid; i < n; i += step) Elem<T>::store(dst + i, vals[i] * inv_sum);
  }
  // a copy that had not landed when the first wait gave up must not outlive this CTA's shared memory
  if (kBulk && !load_ok) mbarrier_wait_bounded(&load_barrier, 0);
}

// ---- fast mode, register-resident form: the same three steps, but every thread keeps its K
// 16-byte vectors of the row in registers from the load to the store.  All loads of the slice
// are in flight at once (K per thread), nothing passes through shared memory, and the loops are
// fully unrolled: ~6 instructions per element.  Used whenever the slice fits K <= 12 vectors
// per thread; the shared-memory kernel above takes the rest.
// Every CTA exponentiates against its OWN slice maximum and the slices are merged afterwards
// (out = e * 2^(m_slice - m_row) / sum), so one exchange and one cluster barrier carry both statistics.
template <typename T, int K>
__global__ void __launch_bounds__(kSoftThreads, 2)
softmax_cluster_reg_kernel(const T* x, T* out, int64_t width, int64_t slice) {
  constexpr int N = Elem<T>::kPerVec;
  __shared__ float scratch[32];
  __shared__ float peer_max[kMaxClusterRanks], peer_sum[kMaxClusterRanks];   // written by the other CTAs

  cg::cluster_group cluster = cg::this_cluster();
  const unsigned rank = cluster.block_rank(), ranks = cluster.num_blocks();
  const int64_t row = blockIdx.x / ranks;
  const int64_t lo = int64_t(rank) * slice;
  const int nvec = int(lo >= width ? 0 : (width - lo < slice ? width - lo : slice)) / N;
  const uint4* src = reinterpret_cast<const uint4*>(x + row * width + lo);
  uint4* dst = reinterpret_cast<uint4*>(out + row * width + lo);
  const int tid = threadIdx.x;

  uint4 raw[K];
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int v = tid + k * kSoftThreads;
    if (v < nvec) raw[k] = ld_stream(src + v);
  }
  cluster.sync();   // every CTA of the cluster is running before anyone writes into a neighbour's shared memory

  float e[K][N];
  float m0 = -INFINITY, m1 = -INFINITY;
#pragma unroll
  for (int k = 0; k < K; ++k) {
    if (tid + k * kSoftThreads < nvec) {
      Elem<T>::unpack(raw[k], e[k]);
    } else {
#pragma unroll
      for (int q = 0; q < N; ++q) e[k][q] = -INFINITY;   // contributes exp(-inf) = 0
    }
#pragma unroll
    for (int q = 0; q < N; q += 2) { m0 = fmaxf(m0, e[k][q]); m1 = fmaxf(m1, e[k][q + 1]); }
  }
  const float slice_max = block_max(fmaxf(m0, m1), scratch);
  // an all -inf slice exponentiates against 0 (every e becomes 0) and is left out of the merge
  const float neg_m2 = slice_max == -INFINITY ? 0.0f : -slice_max * kLog2e;

  float s0 = 0.0f, s1 = 0.0f;
#pragma unroll
  for (int k = 0; k < K; ++k) {
#pragma unroll
    for (int q = 0; q < N; q += 2) {
      e[k][q] = fast_exp2(fmaf(e[k][q], kLog2e, neg_m2));
      e[k][q + 1] = fast_exp2(fmaf(e[k][q + 1], kLog2e, neg_m2));
      s0 += e[k][q];
      s1 += e[k][q + 1];
    }
  }
  const float slice_sum = block_sum(s0 + s1, scratch);
  if (tid < int(ranks)) {
    *cluster.map_shared_rank(&peer_max[rank], tid) = slice_max;
    *cluster.map_shared_rank(&peer_sum[rank], tid) = slice_sum;
  }
  cluster.sync();
  float row_max = -INFINITY;
  for (unsigned r = 0; r < ranks; ++r) row_max = fmaxf(row_max, peer_max[r]);
  const float row_m2 = row_max * kLog2e;
  float row_sum = 0.0f;                                           // rank order: the same sum on every CTA of the row
  for (unsigned r = 0; r < ranks; ++r)
    if (peer_max[r] != -INFINITY) row_sum += peer_sum[r] * fast_exp2(fmaf(peer_max[r], kLog2e, -row_m2));
  // a row of nothing but -inf divides 0 by 0, as the reference does
  const float scale = slice_max == -INFINITY ? (row_max == -INFINITY ? __int_as_float(0x7fc00000) : 0.0f)
                                             : fast_exp2(fmaf(slice_max, kLog2e, -row_m2)) / row_sum;
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int v = tid + k * kSoftThreads;
    if (v < nvec) {
#pragma unroll
      for (int q = 0; q < N; ++q) e[k][q] *= scale;
      st_stream(dst + v, Elem<T>::pack(e[k]));
    }
  }
}

// ---- fast mode, streaming form of the register kernel.  The register kernel alone leaves HBM idle
// while a cluster is between its read burst and its write burst, and its cluster barriers carry a
// memory fence that waits for the stores in flight.  Here the grid is persistent (as many clusters as
// fit the GPU at once, each walking rows c, c + clusters, ...), and per row a CTA does:
//   wait for its stage (filled by the copy engine while the previous row was being finished)
//   -> registers -> per-warp max, exp against the warp's own max, per-warp sum
//   -> ONE __syncthreads (stage free: request the next row; warp statistics visible)
//   -> threads 0..ranks-1 fold the warps' statistics and send them to every CTA of the cluster with an
//      asynchronous remote store that completes a transaction count on the receiver's mbarrier
//   -> wait for the own mbarrier (all slices' statistics have landed) -> scale, store.
// No cluster barrier and no fence inside the loop, so stores of one row drain under the next row's work.
// Statistic buffers and their mbarriers alternate with the row's parity: a fast CTA may send row r+1
// while a slow one still reads row r, and cannot get further ahead (it needs the slow CTA's row r+1).
// `status`: bit 0 is raised if a bounded wait ran out; the outputs of that call are invalid.
__device__ __forceinline__ uint32_t cluster_address_of(const void* local_shared, uint32_t target_rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_addr(local_shared)), "r"(target_rank));
  return remote;
}
// 8-byte store into another CTA's shared memory that also counts 8 bytes on that CTA's mbarrier
__device__ __forceinline__ void remote_store_and_signal(uint32_t remote_data, uint64_t value, uint32_t remote_barrier) {
  asm volatile("st.async.shared::cluster.mbarrier::complete_tx::bytes.b64 [%0], %1, [%2];" ::"r"(remote_data), "l"(value),
               "r"(remote_barrier)
               : "memory");
}
// as mbarrier_wait_bounded, for data that other CTAs of the cluster wrote (acquire at cluster scope)
__device__ __forceinline__ bool mbarrier_wait_bounded_cluster(uint64_t* bar, uint32_t parity) {
  for (int attempt = 0; attempt < (1 << 15); ++attempt) {
    uint32_t done;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(done)
        : "r"(smem_addr(bar)), "r"(parity), "r"(10000u)
        : "memory");
    if (done != 0) return true;
  }
  return false;
}

template <typename T, int K>
__global__ void __launch_bounds__(kSoftThreads, 2)
softmax_cluster_stream_kernel(const T* x, T* out, int64_t rows, int64_t width, int64_t slice, int* status) {
  constexpr int N = Elem<T>::kPerVec;
  constexpr int kWarps = kSoftThreads / kWarpSize;
  extern __shared__ __align__(128) unsigned char stage_bytes_[];
  __shared__ float2 warp_stats[2][kWarps];                        // (max, sum) of each warp's elements
  __shared__ __align__(8) float2 peer_stats[2][kMaxClusterRanks];   // (max, sum) of each slice; written by the other CTAs
  __shared__ __align__(8) uint64_t stage_barrier, stats_barrier[2];

  cg::cluster_group cluster = cg::this_cluster();
  const unsigned rank = cluster.block_rank(), ranks = cluster.num_blocks();
  const int64_t clusters = gridDim.x / ranks;
  const int64_t lo = int64_t(rank) * slice;
  const int nvec = int(lo >= width ? 0 : (width - lo < slice ? width - lo : slice)) / N;
  const uint32_t bytes = uint32_t(nvec) * 16u;
  const uint4* stage = reinterpret_cast<const uint4*>(stage_bytes_);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  auto request = [&](int64_t row) {   // thread 0 only
    mbarrier_expect_bytes(&stage_barrier, bytes);
    const char* src = reinterpret_cast<const char*>(x + row * width + lo);
    for (uint32_t off = 0; off < bytes; off += kBulkChunk)
      bulk_load(stage_bytes_ + off, src + off, bytes - off < kBulkChunk ? bytes - off : kBulkChunk, &stage_barrier);
  };

  int64_t row = blockIdx.x / ranks;
  if (tid == 0) {
    mbarrier_init(&stage_barrier, 1);
    mbarrier_init(&stats_barrier[0], 1);
    mbarrier_init(&stats_barrier[1], 1);
    mbarrier_expect_bytes(&stats_barrier[0], ranks * 8u);   // the first row's statistics: 8 bytes from each CTA
    if (row < rows && bytes != 0u) request(row);
  }
  __syncthreads();
  cluster.sync();   // every CTA's barriers exist before anyone stores into a neighbour's shared memory

  bool healthy = true;
  for (int it = 0; row < rows; ++it, row += clusters) {
    const int par = it & 1;
    // A wait that runs out (never expected) makes this thread stop waiting for anything: it finishes the loop on
    // whatever is in memory, in step with the others (every barrier and shuffle below is still reached by all),
    // and the status word says that this call's outputs are invalid.
    if (healthy && bytes != 0u && !mbarrier_wait_bounded(&stage_barrier, uint32_t(par))) healthy = false;
    uint4 raw[K];
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int v = tid + k * kSoftThreads;
      if (v < nvec) raw[k] = stage[v];
    }
    float e[K][N];
    float m0 = -INFINITY, m1 = -INFINITY;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      if (tid + k * kSoftThreads < nvec) {
        Elem<T>::unpack(raw[k], e[k]);
      } else {
#pragma unroll
        for (int q = 0; q < N; ++q) e[k][q] = -INFINITY;   // contributes exp(-inf) = 0
      }
#pragma unroll
      for (int q = 0; q < N; q += 2) { m0 = fmaxf(m0, e[k][q]); m1 = fmaxf(m1, e[k][q + 1]); }
    }
    const float warp_m = warp_max(fmaxf(m0, m1));
    // a warp of nothing but -inf exponentiates against 0 (every e becomes 0) and is left out of the merges
    const float neg_m2 = warp_m == -INFINITY ? 0.0f : -warp_m * kLog2e;
    float s0 = 0.0f, s1 = 0.0f;
#pragma unroll
    for (int k = 0; k < K; ++k) {
#pragma unroll
      for (int q = 0; q < N; q += 2) {
        e[k][q] = fast_exp2(fmaf(e[k][q], kLog2e, neg_m2));
        e[k][q + 1] = fast_exp2(fmaf(e[k][q + 1], kLog2e, neg_m2));
        s0 += e[k][q];
        s1 += e[k][q + 1];
      }
    }
    const float warp_s = warp_sum(s0 + s1);
    if (lane == 0) warp_stats[par][warp] = make_float2(warp_m, warp_s);
    __syncthreads();   // the stage has been read by everyone; the warps' statistics are visible

    const int64_t next = row + clusters;
    if (tid == 0 && next < rows) {
      if (bytes != 0u && healthy) { fence_before_bulk_copy(); request(next); }
      // the next row's statistics: that barrier's previous phase was consumed by every thread before the
      // __syncthreads above
      mbarrier_expect_bytes(&stats_barrier[par ^ 1], ranks * 8u);
    }
    // Every warp folds the warps' statistics, one per lane, with shuffle trees (fixed order: the same bits in
    // every warp); a serial walk by a few threads would sit on the critical path of the whole cluster.
    const float2 mine = lane < kWarps ? warp_stats[par][lane] : make_float2(-INFINITY, 0.0f);
    const float slice_m = warp_max(mine.x);
    const float slice_s =
        warp_sum(mine.x == -INFINITY ? 0.0f : mine.y * fast_exp2(fmaf(mine.x, kLog2e, -slice_m * kLog2e)));
    if (tid < int(ranks)) {
      const uint64_t packed = (uint64_t(__float_as_uint(slice_s)) << 32) | uint64_t(__float_as_uint(slice_m));
      remote_store_and_signal(cluster_address_of(&peer_stats[par][rank], unsigned(tid)), packed,
                              cluster_address_of(&stats_barrier[par], unsigned(tid)));
    }
    if (healthy && !mbarrier_wait_bounded_cluster(&stats_barrier[par], uint32_t(it >> 1) & 1u)) healthy = false;
    // the same fold over the slices of the row: lane r holds slice r (same tree on every CTA of the row)
    const float2 theirs = lane < int(ranks) ? peer_stats[par][lane] : make_float2(-INFINITY, 0.0f);
    const float row_m = warp_max(theirs.x);
    const float row_m2 = row_m * kLog2e;
    const float row_sum = warp_sum(theirs.x == -INFINITY ? 0.0f : theirs.y * fast_exp2(fmaf(theirs.x, kLog2e, -row_m2)));
    // a row of nothing but -inf divides 0 by 0, as the reference does
    const float scale = warp_m == -INFINITY ? (row_m == -INFINITY ? __int_as_float(0x7fc00000) : 0.0f)
                                            : fast_exp2(fmaf(warp_m, kLog2e, -row_m2)) / row_sum;
    uint4* dst = reinterpret_cast<uint4*>(out + row * width + lo);
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int v = tid + k * kSoftThreads;
      if (v < nvec) {
#pragma unroll
        for (int q = 0; q < N; ++q) e[k][q] *= scale;
        st_stream(dst + v, Elem<T>::pack(e[k]));
      }
    }
  }
  if (!healthy) {
    // Flag it, and give a copy that may still be in flight one more bounded chance to land: it must not
    // outlive this CTA's shared memory.
    if (status != nullptr) atomicOr(status, 1);
    if (bytes != 0u) { mbarrier_wait_bounded(&stage_barrier, 0u); mbarrier_wait_bounded(&stage_barrier, 1u); }
  }
  // nobody leaves while a neighbour may still store into its shared memory (only matters after a failure:
  // in a healthy run every CTA has received all statistics of its last row by now)
  cluster.sync();
}

// ---- row statistics (max, sum of exp(x - max)), one CTA per row, one pass, online rescaling
template <typename T, bool kVec>
__global__ void __launch_bounds__(kSoftThreads)
softmax_stats_kernel(const T* x, int64_t width, float* row_max, float* row_sum) {
  constexpr int N = Elem<T>::kPerVec;
  __shared__ float scratch[32];
  const int64_t row = blockIdx.x;
  const T* src = x + row * width;
  const int64_t step = blockDim.x;
  float m = -INFINITY, m2 = -INFINITY, s = 0.0f;   // max of x, max of x*log2(e), sum of 2^(x*log2(e) - m2)
  if (kVec) {
    const int64_t nvec = width / N;
    const uint4* vp = reinterpret_cast<const uint4*>(src);
    for (int64_t v0 = threadIdx.x; v0 < nvec; v0 += step * 4) {
      uint4 r[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) if (v0 + k * step < nvec) r[k] = ld_stream(vp + v0 + k * step);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (v0 + k * step < nvec) {
          float e[N];
          Elem<T>::unpack(r[k], e);
          online_update<N>(m, m2, s, e);
        }
      }
    }
    for (int64_t i = nvec * N + threadIdx.x; i < width; i += step) { const float e = Elem<T>::load(src + i); online_update<1>(m, m2, s, &e); }
  } else {
    for (int64_t i = threadIdx.x; i < width; i += step) { const float e = Elem<T>::load(src + i); online_update<1>(m, m2, s, &e); }
  }
  const float big = block_max(m, scratch);       // max of x over the row; big*log2(e) is the max of t
  s = m2 == -INFINITY ? 0.0f : s * fast_exp2(m2 - big * kLog2e);
  s = block_sum(s, scratch);
  if (threadIdx.x == 0) { row_max[row] = big; row_sum[row] = s; }
}

// Vocabulary-sharded row statistics with the exchange fused into the kernel: (max, sum) of this GPU's
// columns per row, sent to every peer as soon as the row is done; the thread block that finishes the last
// row waits (bounded) for the peers' pairs and writes the statistics of the WHOLE row, ready for
// softmax_apply_kernel.
template <typename T, bool kVec>
__global__ void __launch_bounds__(kSoftThreads, 3)   // the tail's registers beyond the cap spill; the row loop's do not
softmax_stats_exchange_kernel(const T* x, int64_t rows, int64_t width, float* global_max, float* global_sum,
                              const __grid_constant__ ExchangeArgs xa) {
  constexpr int N = Elem<T>::kPerVec;
  __shared__ float scratch[32];
  __shared__ int run_tail;
  __shared__ uint32_t call_epoch;
  exchange_trace_start(xa);
  if (threadIdx.x == 0) call_epoch = exchange_call_epoch(xa);   // fetched under the scan of the row; published by the barriers of the reductions below
  const int64_t row = blockIdx.x;
  const T* src = x + row * width;
  const int64_t step = blockDim.x;
  float m = -INFINITY, m2 = -INFINITY, s = 0.0f;
  if (kVec) {
    const int64_t nvec = width / N;
    const uint4* vp = reinterpret_cast<const uint4*>(src);
    for (int64_t v0 = threadIdx.x; v0 < nvec; v0 += step * 4) {
      uint4 r[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) if (v0 + k * step < nvec) r[k] = ld_stream(vp + v0 + k * step);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (v0 + k * step < nvec) {
          float e[N];
          Elem<T>::unpack(r[k], e);
          online_update<N>(m, m2, s, e);
        }
      }
    }
    for (int64_t i = nvec * N + threadIdx.x; i < width; i += step) { const float e = Elem<T>::load(src + i); online_update<1>(m, m2, s, &e); }
  } else {
    for (int64_t i = threadIdx.x; i < width; i += step) { const float e = Elem<T>::load(src + i); online_update<1>(m, m2, s, &e); }
  }
  const float big = block_max(m, scratch);
  s = m2 == -INFINITY ? 0.0f : s * fast_exp2(m2 - big * kLog2e);
  s = block_sum(s, scratch);
  // every thread holds the row's (max, sum): thread 0 stores this GPU's own slot and takes the ticket, threads
  // 1 .. world-1 send the pair to one peer each
  const unsigned long long pair = (static_cast<unsigned long long>(__float_as_uint(s)) << 32) | __float_as_uint(big);
  // (block_max / block_sum above end with barriers: call_epoch is visible to every thread)
  if (threadIdx.x > 0 && threadIdx.x < xa.world) exchange_send(xa, call_epoch, (xa.rank + threadIdx.x) % xa.world, row, pair);
  if (threadIdx.x == 0) {
    exchange_send(xa, call_epoch, xa.rank, row, pair);
    run_tail = exchange_row_done(xa, rows) ? 1 : 0;
  }
  __syncthreads();
  if (!run_tail) return;
  exchange_tail(xa, rows, call_epoch, [&](int64_t r, bool complete, auto partial_of) {
    float top = -INFINITY;
#pragma unroll
    for (int g = 0; g < kMaxWorld; ++g)
      if (g < xa.world) top = fmaxf(top, __uint_as_float(uint32_t(partial_of(g))));
    const float top2 = top * kLog2e;
    float total = 0.0f;                             // rank order: the same sum on every GPU
#pragma unroll
    for (int g = 0; g < kMaxWorld; ++g) {
      if (g < xa.world) {
        const unsigned long long p = partial_of(g);
        const float pm = __uint_as_float(uint32_t(p)), ps = __uint_as_float(uint32_t(p >> 32));
        if (pm != -INFINITY) total += ps * fast_exp2(fmaf(pm, kLog2e, -top2));
      }
    }
    const float invalid = __int_as_float(0x7fc00000);   // a row whose exchange did not complete in time: NaN statistics
    global_max[r] = complete ? top : invalid;
    global_sum[r] = complete ? total : invalid;
  });
}

__global__ void softmax_rebase_kernel(const float* row_max, const float* global_max, float* row_sum, int64_t rows) {
  const int64_t r = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  // the same 2^(m*log2e - M*log2e) form as the kernels on either side of the exchange
  if (r < rows) row_sum[r] = row_max[r] == -INFINITY ? 0.0f : row_sum[r] * fast_exp2(row_max[r] * kLog2e - global_max[r] * kLog2e);
}

// ---- out = exp(x - max[r]) / sum[r]; blockIdx = row * tiles + tile
constexpr int kApplyThreads = 256, kApplyVecs = 4;
template <typename T, bool kVec>
__global__ void __launch_bounds__(kApplyThreads)
softmax_apply_kernel(const T* x, T* out, int64_t width, int tiles, int64_t tile_elems, const float* row_max,
                     const float* row_sum) {
  constexpr int N = Elem<T>::kPerVec;
  const int64_t row = blockIdx.x / tiles;
  const int64_t lo = int64_t(blockIdx.x - row * tiles) * tile_elems;
  const int64_t n = width - lo < tile_elems ? width - lo : tile_elems;
  const float neg_m2 = -row_max[row] * kLog2e, inv_z = 1.0f / row_sum[row];
  const T* src = x + row * width + lo;
  T* dst = out + row * width + lo;
  if (kVec) {
    const int64_t nvec = n / N;
    uint4 raw[kApplyVecs];
#pragma unroll
    for (int k = 0; k < kApplyVecs; ++k) {
      const int64_t v = threadIdx.x + k * kApplyThreads;
      if (v < nvec) raw[k] = ld_stream(reinterpret_cast<const uint4*>(src) + v);
    }
#pragma unroll
    for (int k = 0; k < kApplyVecs; ++k) {
      const int64_t v = threadIdx.x + k * kApplyThreads;
      if (v < nvec) {
        float e[N];
        Elem<T>::unpack(raw[k], e);
#pragma unroll
        for (int q = 0; q < N; ++q) e[q] = fast_exp2(fmaf(e[q], kLog2e, neg_m2)) * inv_z;
        st_stream(reinterpret_cast<uint4*>(dst) + v, Elem<T>::pack(e));
      }
    }
    for (int64_t i = nvec * N + threadIdx.x; i < n; i += kApplyThreads)
      Elem<T>::store(dst + i, fast_exp2(fmaf(Elem<T>::load(src + i), kLog2e, neg_m2)) * inv_z);
  } else {
    for (int64_t i = threadIdx.x; i < n; i += kApplyThreads)
      Elem<T>::store(dst + i, fast_exp2(fmaf(Elem<T>::load(src + i), kLog2e, neg_m2)) * inv_z);
  }
}

// ---- deterministic mode: the reference's order (src/ops_cuda.cu:132; src/ops_cpu.cpp:13).
// max by fmaxf from -FLT_MAX; e_j = expf(x_j - max) stored rounded; fp32 running sum of
// the unrounded e_j in index order; out_j = round(float(stored e_j) / sum).
constexpr int kOrdThreads = 256, kOrdChunk = 2048;
template <typename T>
__global__ void __launch_bounds__(kOrdThreads) softmax_ordered_kernel(const T* x, T* out, int64_t width) {
  __shared__ float stage[kOrdChunk];
  __shared__ float scratch[32];
  __shared__ float total;
  const T* src = x + int64_t(blockIdx.x) * width;
  T* dst = out + int64_t(blockIdx.x) * width;
  float m = -FLT_MAX;
  for (int64_t i = threadIdx.x; i < width; i += kOrdThreads) m = fmaxf(m, Elem<T>::load(src + i));
  m = block_max(m, scratch);
  float sum = 0.0f;  // meaningful in thread 0 only
  for (int64_t base = 0; base < width; base += kOrdChunk) {
    const int n = int(width - base < kOrdChunk ? width - base : kOrdChunk);
    for (int j = threadIdx.x; j < n; j += kOrdThreads) {
      const float e = expf(Elem<T>::load(src + base + j) - m);
      Elem<T>::store(dst + base + j, e);
      stage[j] = e;
    }
    __syncthreads();
    if (threadIdx.x == 0)
      for (int j = 0; j < n; ++j) sum += stage[j];
    __syncthreads();
  }
  if (threadIdx.x == 0) total = sum;
  __syncthreads();
  const float z = total;
  // every thread re-reads exactly the elements it stored itself
  for (int64_t i = threadIdx.x; i < width; i += kOrdThreads) Elem<T>::store(dst + i, __fdiv_rn(Elem<T>::load(dst + i), z));
}

template <typename T> bool rows_vector_ok(const void* p, int64_t row_stride) {
  return aligned16(p) && (row_stride * int64_t(sizeof(T))) % 16 == 0;
}

// ---------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------

template <typename T>
int launch_argmax_typed(const void* logits_, int64_t rows, int64_t width, int64_t row_stride, int64_t index_base,
                        int32_t* out_ids, int64_t* out_keys, void* workspace, cudaStream_t s) {
  if (rows == 0) return B2_OK;
  const T* logits = static_cast<const T*>(logits_);
  constexpr int N = Elem<T>::kPerVec;
  const int64_t target = int64_t(sm_count()) * 8;
  int64_t chunks = target / rows;
  const int64_t most = (width + kMinChunk - 1) / kMinChunk;
  if (chunks > most) chunks = most;
  if (chunks < 1) chunks = 1;
  int64_t chunk = (width + chunks - 1) / chunks;
  chunk = (chunk + 4 * N - 1) / (4 * N) * (4 * N);  // chunk starts stay 16-byte aligned
  chunks = (width + chunk - 1) / chunk;
  auto* keys = static_cast<unsigned long long*>(workspace);
  auto* tickets = reinterpret_cast<unsigned int*>(keys + rows);
  const unsigned grid = unsigned(rows * chunks);
  if (rows_vector_ok<T>(logits, row_stride))
    argmax_rows_kernel<T, true><<<grid, kArgThreads, 0, s>>>(logits, width, row_stride, chunk, int(chunks), index_base,
                                                            out_ids, out_keys, keys, tickets);
  else
    argmax_rows_kernel<T, false><<<grid, kArgThreads, 0, s>>>(logits, width, row_stride, chunk, int(chunks), index_base,
                                                             out_ids, out_keys, keys, tickets);
  return launch_status("argmax_rows");
}

template <typename T, bool kVec, bool kBulk>
int launch_softmax_cluster(const T* x, T* out, int64_t rows, int64_t width, int ranks, int64_t slice, int* status,
                           cudaStream_t s) {
  auto kernel = softmax_cluster_kernel<T, kVec, kBulk>;
  const size_t smem = size_t(slice) * sizeof(float);
  if (smem > 48 * 1024 &&
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) {
    cudaGetLastError();
    return B2_ERR_UNSUPPORTED;
  }
  if (ranks > 8 && cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) {
    cudaGetLastError();
    return B2_ERR_UNSUPPORTED;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(rows * ranks));
  cfg.blockDim = dim3(slice <= 4096 ? 128 : kSoftThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = unsigned(ranks);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, kernel, x, out, width, slice, status) != cudaSuccess) {
    cudaGetLastError();  // the two-pass path takes over
    return B2_ERR_UNSUPPORTED;
  }
  return B2_OK;
}

template <typename T, int K>
int launch_softmax_reg(const T* x, T* out, int64_t rows, int64_t width, int ranks, int64_t slice, cudaStream_t s) {
  auto kernel = softmax_cluster_reg_kernel<T, K>;
  if (ranks > 8 && cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) {
    cudaGetLastError();
    return B2_ERR_UNSUPPORTED;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(rows * ranks));
  cfg.blockDim = dim3(kSoftThreads);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = unsigned(ranks);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, kernel, x, out, width, slice) != cudaSuccess) {
    cudaGetLastError();
    return B2_ERR_UNSUPPORTED;
  }
  return B2_OK;
}

// Persistent launch of the streaming kernel: as many clusters as the GPU holds at once (asked of the
// occupancy calculator once per device and cluster size), each walking several rows.
template <typename T, int K>
int launch_softmax_stream(const T* x, T* out, int64_t rows, int64_t width, int ranks, int64_t slice, int* status,
                          cudaStream_t s) {
  auto kernel = softmax_cluster_stream_kernel<T, K>;
  const size_t smem = size_t(K) * kSoftThreads * 16;
  static std::mutex mutex;
  static int resident[kDeviceSlots][kMaxClusterRanks + 1] = {};   // 0 = not asked yet, -1 = cannot launch
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kDeviceSlots) { cudaGetLastError(); return B2_ERR_UNSUPPORTED; }
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(kSoftThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = unsigned(ranks);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int clusters;
  {
    std::lock_guard<std::mutex> lock(mutex);
    if (resident[device][ranks] == 0) {
      int n = 0;
      cfg.gridDim = dim3(unsigned(ranks) * 64u);
      const bool ok = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) == cudaSuccess &&
                      (ranks <= 8 || cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess) &&
                      cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) == cudaSuccess && n > 0;
      if (!ok) cudaGetLastError();
      resident[device][ranks] = ok ? n : -1;
    }
    clusters = resident[device][ranks];
  }
  if (clusters <= 0) return B2_ERR_UNSUPPORTED;
  if (int64_t(clusters) > rows) clusters = int(rows);
  cfg.gridDim = dim3(unsigned(clusters) * unsigned(ranks));
  if (cudaLaunchKernelEx(&cfg, kernel, x, out, rows, width, slice, status) != cudaSuccess) {
    cudaGetLastError();
    return B2_ERR_UNSUPPORTED;
  }
  return B2_OK;
}

// K vectors of N elements per thread stay in registers: at most 48 floats (64 registers at two CTAs per SM).
template <typename T, int K>
int launch_softmax_reg_if_fits(const T* x, T* out, int64_t rows, int64_t width, int ranks, int64_t slice, int* status,
                               cudaStream_t s) {
  if constexpr (K * Elem<T>::kPerVec <= 48) {
    // several rows per cluster: stream them; otherwise one cluster per row is all there is to do
    if (rows * ranks > int64_t(sm_count()) * 2 &&
        launch_softmax_stream<T, K>(x, out, rows, width, ranks, slice, status, s) == B2_OK)
      return B2_OK;
    return launch_softmax_reg<T, K>(x, out, rows, width, ranks, slice, s);
  } else {
    return B2_ERR_UNSUPPORTED;
  }
}

template <typename T>
int launch_softmax_reg_any(const T* x, T* out, int64_t rows, int64_t width, int ranks, int64_t slice, int* status,
                           cudaStream_t s) {
  const int64_t vecs = slice / Elem<T>::kPerVec, per_thread = (vecs + kSoftThreads - 1) / kSoftThreads;
  if (per_thread <= 1) return launch_softmax_reg_if_fits<T, 1>(x, out, rows, width, ranks, slice, status, s);
  if (per_thread <= 2) return launch_softmax_reg_if_fits<T, 2>(x, out, rows, width, ranks, slice, status, s);
  if (per_thread <= 3) return launch_softmax_reg_if_fits<T, 3>(x, out, rows, width, ranks, slice, status, s);
  if (per_thread <= 4) return launch_softmax_reg_if_fits<T, 4>(x, out, rows, width, ranks, slice, status, s);
  if (per_thread <= 5) return launch_softmax_reg_if_fits<T, 5>(x, out, rows, width, ranks, slice, status, s);
  if (per_thread <= 6) return launch_softmax_reg_if_fits<T, 6>(x, out, rows, width, ranks, slice, status, s);
  if (per_thread <= 7) return launch_softmax_reg_if_fits<T, 7>(x, out, rows, width, ranks, slice, status, s);
  if (per_thread <= 8) return launch_softmax_reg_if_fits<T, 8>(x, out, rows, width, ranks, slice, status, s);
  if (per_thread <= 9) return launch_softmax_reg_if_fits<T, 9>(x, out, rows, width, ranks, slice, status, s);
  if (per_thread <= 10) return launch_softmax_reg_if_fits<T, 10>(x, out, rows, width, ranks, slice, status, s);
  if (per_thread <= 11) return launch_softmax_reg_if_fits<T, 11>(x, out, rows, width, ranks, slice, status, s);
  if (per_thread <= 12) return launch_softmax_reg_if_fits<T, 12>(x, out, rows, width, ranks, slice, status, s);
  return B2_ERR_UNSUPPORTED;
}

template <typename T>
int launch_stats_typed(const void* x, int64_t rows, int64_t width, float* row_max, float* row_sum, cudaStream_t s) {
  if (rows == 0) return B2_OK;
  if (rows_vector_ok<T>(x, width))
    softmax_stats_kernel<T, true><<<unsigned(rows), kSoftThreads, 0, s>>>(static_cast<const T*>(x), width, row_max, row_sum);
  else
    softmax_stats_kernel<T, false><<<unsigned(rows), kSoftThreads, 0, s>>>(static_cast<const T*>(x), width, row_max, row_sum);
  return launch_status("softmax_stats");
}

template <typename T>
int launch_apply_typed(const void* x, void* out, int64_t rows, int64_t width, const float* row_max,
                       const float* row_sum, cudaStream_t s) {
  if (rows == 0 || width == 0) return B2_OK;
  constexpr int N = Elem<T>::kPerVec;
  const int64_t tile_elems = int64_t(kApplyThreads) * kApplyVecs * N;
  const int64_t tiles = (width + tile_elems - 1) / tile_elems;
  const unsigned grid = unsigned(rows * tiles);
  if (rows_vector_ok<T>(x, width) && aligned16(out))
    softmax_apply_kernel<T, true><<<grid, kApplyThreads, 0, s>>>(static_cast<const T*>(x), static_cast<T*>(out), width,
                                                                int(tiles), tile_elems, row_max, row_sum);
  else
    softmax_apply_kernel<T, false><<<grid, kApplyThreads, 0, s>>>(static_cast<const T*>(x), static_cast<T*>(out), width,
                                                                 int(tiles), tile_elems, row_max, row_sum);
  return launch_status("softmax_apply");
}

template <typename T>
int launch_softmax_typed(const void* x_, void* out_, int64_t rows, int64_t width, int mode, void* workspace,
                         cudaStream_t s) {
  if (rows == 0 || width == 0) return B2_OK;
  const T* x = static_cast<const T*>(x_);
  T* out = static_cast<T*>(out_);
  constexpr int N = Elem<T>::kPerVec;
  if (mode == B2_DETERMINISTIC) {
    softmax_ordered_kernel<T><<<unsigned(rows), kOrdThreads, 0, s>>>(x, out, width);
    return launch_status("softmax (deterministic)");
  }
  // smallest cluster whose slices fit, then widened (up to 8) while rows alone cannot fill the SMs
  constexpr int max_ranks = 8;   // the portable cluster size; 9 measured 2 % faster and 10 or more far slower
  int ranks = 1;
  while (ranks < max_ranks && size_t((width + ranks - 1) / ranks) * sizeof(float) > kClusterSliceBytes) ranks <<= 1;
  while (ranks < max_ranks && rows * ranks < int64_t(sm_count()) * 2 && width / (ranks * 2) >= 1024) ranks <<= 1;
  int64_t slice = (width + ranks - 1) / ranks;
  slice = (slice + N - 1) / N * N;
  if (size_t(slice) * sizeof(float) <= kClusterSliceBytes) {
    const bool vec = rows_vector_ok<T>(x, width) && aligned16(out);
    // status word: the last 16 bytes of the workspace (after the 2*rows floats of the two-pass path)
    int* status = reinterpret_cast<int*>(static_cast<char*>(workspace) + softmax_workspace_bytes(rows) - 16);
    int rc;
    if (vec && width % N == 0 && launch_softmax_reg_any<T>(x, out, rows, width, ranks, slice, status, s) == B2_OK) return B2_OK;
    if (vec && sizeof(T) == 4 && slice % 4 == 0)   // fp32 rows: shared memory holds the input's own bytes -> bulk copy
      rc = launch_softmax_cluster<T, true, true>(x, out, rows, width, ranks, slice, status, s);
    else
      rc = vec ? launch_softmax_cluster<T, true, false>(x, out, rows, width, ranks, slice, status, s)
               : launch_softmax_cluster<T, false, false>(x, out, rows, width, ranks, slice, status, s);
    if (rc == B2_OK) return B2_OK;
  }
  float* row_max = static_cast<float*>(workspace);
  float* row_sum = row_max + rows;
  const int rc = launch_stats_typed<T>(x, rows, width, row_max, row_sum, s);
  if (rc != B2_OK) return rc;
  return launch_apply_typed<T>(x, out, rows, width, row_max, row_sum, s);
}

template <typename T>
int launch_argmax_exchange_typed(const void* logits_, int64_t rows, int64_t width, int64_t row_stride, int64_t index_base,
                                 int32_t* out_ids, void* workspace, const ExchangeArgs& xa, cudaStream_t s) {
  const T* logits = static_cast<const T*>(logits_);
  constexpr int N = Elem<T>::kPerVec;
  auto* keys = static_cast<unsigned long long*>(workspace);
  auto* tickets = reinterpret_cast<unsigned int*>(keys + rows);
  const bool vec = rows_vector_ok<T>(logits, row_stride);
  // A shard of the vocabulary is short (19 k columns at eight GPUs): with enough rows to occupy the GPU, one
  // 1024-thread block per row fetches the whole row in one or two rounds of loads and needs no key merge, no
  // ticket and no fence -- the three dependent trips to L2 that otherwise end every block cost more than the row.
  if (rows >= sm_count() / 2 && width <= int64_t(1024) * 16 * N) {
    if (vec)
      argmax_rows_exchange_kernel<T, true, 1024><<<unsigned(rows), 1024, 0, s>>>(logits, rows, width, row_stride, width, 1, index_base,
                                                                               out_ids, keys, tickets, xa);
    else
      argmax_rows_exchange_kernel<T, false, 1024><<<unsigned(rows), 1024, 0, s>>>(logits, rows, width, row_stride, width, 1,
                                                                                index_base, out_ids, keys, tickets, xa);
    return launch_status("argmax_rows_sharded");
  }
  const int64_t target = int64_t(sm_count()) * 8;
  int64_t chunks = target / rows;
  const int64_t most = (width + kMinChunk - 1) / kMinChunk;
  if (chunks > most) chunks = most;
  if (chunks < 1) chunks = 1;
  int64_t chunk = (width + chunks - 1) / chunks;
  chunk = (chunk + 4 * N - 1) / (4 * N) * (4 * N);  // chunk starts stay 16-byte aligned
  chunks = (width + chunk - 1) / chunk;
  const unsigned grid = unsigned(rows * chunks);
  if (vec)
    argmax_rows_exchange_kernel<T, true, kArgThreads><<<grid, kArgThreads, 0, s>>>(logits, rows, width, row_stride, chunk, int(chunks),
                                                                                  index_base, out_ids, keys, tickets, xa);
  else
    argmax_rows_exchange_kernel<T, false, kArgThreads><<<grid, kArgThreads, 0, s>>>(logits, rows, width, row_stride, chunk,
                                                                                   int(chunks), index_base, out_ids, keys, tickets, xa);
  return launch_status("argmax_rows_sharded");
}

template <typename T>
int launch_stats_exchange_typed(const void* x, int64_t rows, int64_t width, float* global_max, float* global_sum,
                                const ExchangeArgs& xa, cudaStream_t s) {
  if (rows_vector_ok<T>(x, width))
    softmax_stats_exchange_kernel<T, true><<<unsigned(rows), kSoftThreads, 0, s>>>(static_cast<const T*>(x), rows, width,
                                                                                  global_max, global_sum, xa);
  else
    softmax_stats_exchange_kernel<T, false><<<unsigned(rows), kSoftThreads, 0, s>>>(static_cast<const T*>(x), rows, width,
                                                                                   global_max, global_sum, xa);
  return launch_status("softmax_stats_sharded");
}

}  // namespace

size_t argmax_workspace_bytes(int64_t rows) {
  const size_t raw = size_t(rows) * (sizeof(unsigned long long) + sizeof(unsigned int));
  return (raw + 15) / 16 * 16;
}

int launch_argmax(const void* logits, int64_t rows, int64_t width, int64_t row_stride, int dtype, int64_t index_base,
                  int32_t* out_ids, int64_t* out_keys, void* workspace, cudaStream_t s) {
  return dtype == B2_F32
             ? launch_argmax_typed<float>(logits, rows, width, row_stride, index_base, out_ids, out_keys, workspace, s)
             : launch_argmax_typed<__half>(logits, rows, width, row_stride, index_base, out_ids, out_keys, workspace, s);
}

int launch_argmax_decode(const int64_t* keys, int64_t rows, int32_t* out_ids, cudaStream_t s) {
  if (rows == 0) return B2_OK;
  argmax_decode_kernel<<<unsigned((rows + 255) / 256), 256, 0, s>>>(keys, rows, out_ids);
  return launch_status("argmax_decode_keys");
}

// 2*rows floats of row statistics for the two-pass path, then one 16-byte slot whose first int32 is a status word
size_t softmax_workspace_bytes(int64_t rows) { return (size_t(rows) * 2 * sizeof(float) + 15) / 16 * 16 + 16; }

int launch_softmax(const void* x, void* out, int64_t rows, int64_t width, int dtype, int mode, void* workspace,
                   cudaStream_t s) {
  return dtype == B2_F32 ? launch_softmax_typed<float>(x, out, rows, width, mode, workspace, s)
                         : launch_softmax_typed<__half>(x, out, rows, width, mode, workspace, s);
}

int launch_softmax_stats(const void* x, int64_t rows, int64_t width, int dtype, float* row_max, float* row_sum,
                         cudaStream_t s) {
  return dtype == B2_F32 ? launch_stats_typed<float>(x, rows, width, row_max, row_sum, s)
                         : launch_stats_typed<__half>(x, rows, width, row_max, row_sum, s);
}

int launch_softmax_rebase(const float* row_max, const float* global_max, float* row_sum, int64_t rows, cudaStream_t s) {
  if (rows == 0) return B2_OK;
  softmax_rebase_kernel<<<unsigned((rows + 255) / 256), 256, 0, s>>>(row_max, global_max, row_sum, rows);
  return launch_status("softmax_rebase");
}

int launch_softmax_apply(const void* x, void* out, int64_t rows, int64_t width, int dtype, const float* row_max,
                         const float* row_sum, cudaStream_t s) {
  return dtype == B2_F32 ? launch_apply_typed<float>(x, out, rows, width, row_max, row_sum, s)
                         : launch_apply_typed<__half>(x, out, rows, width, row_max, row_sum, s);
}

int launch_argmax_exchange(const void* logits, int64_t rows, int64_t width, int64_t row_stride, int dtype,
                           int64_t index_base, int32_t* out_ids, void* workspace, const ExchangeArgs& xa, cudaStream_t s) {
  if (rows == 0) return B2_OK;
  return dtype == B2_F32
             ? launch_argmax_exchange_typed<float>(logits, rows, width, row_stride, index_base, out_ids, workspace, xa, s)
             : launch_argmax_exchange_typed<__half>(logits, rows, width, row_stride, index_base, out_ids, workspace, xa, s);
}

int launch_argmax_keys_exchange(const int64_t* keys, int64_t rows, int32_t* out_ids, const ExchangeArgs& xa, cudaStream_t s) {
  if (rows == 0) return B2_OK;
  argmax_keys_exchange_kernel<<<1, kArgThreads, 0, s>>>(keys, rows, out_ids, xa);
  return launch_status("argmax_keys_exchange");
}

int launch_softmax_stats_exchange(const void* x, int64_t rows, int64_t width, int dtype, float* global_max,
                                  float* global_sum, const ExchangeArgs& xa, cudaStream_t s) {
  if (rows == 0) return B2_OK;
  return dtype == B2_F32 ? launch_stats_exchange_typed<float>(x, rows, width, global_max, global_sum, xa, s)
                         : launch_stats_exchange_typed<__half>(x, rows, width, global_max, global_sum, xa, s);
}

}  // namespace b2

// ---------------------------------------------------------------------------
// Argmax without a caller workspace and without any allocation.
//
// For hosts that must not call cudaMalloc after start-up (all device memory already
// belongs to their own pool) and plug-ins that receive tensors but no allocator.  The
// scratch the argmax kernel needs (one 64-bit key and one 32-bit ticket per row) is a
// fixed array in the library image.  In host code the array's NAME is only a handle:
// the address a kernel can use comes from cudaGetSymbolAddress, asked once per device
// with that device current.
// ---------------------------------------------------------------------------
namespace b2 {
namespace {

constexpr size_t kStaticScratchBytes = size_t(B2_ARGMAX_STATIC_MAX_ROWS) * 12;
static __device__ __align__(256) unsigned char g_argmax_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_static_mutex;
void* g_static_scratch_address[kMaxDevices] = {};

// Device address of the scratch array on the current device, or nullptr (error recorded).
void* static_scratch_for_current_device() {
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess || device < 0 || device >= kMaxDevices) {
    set_error("b2_argmax_rows_static: cannot identify the current device: %s", cudaGetErrorString(e));
    cudaGetLastError();
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (g_static_scratch_address[device] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_argmax_static_scratch);
    if (e != cudaSuccess || p == nullptr) {
      set_error("b2_argmax_rows_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      cudaGetLastError();
      return nullptr;
    }
    g_static_scratch_address[device] = p;
  }
  return g_static_scratch_address[device];
}

}  // namespace
}  // namespace b2

extern "C" int b2_argmax_rows_static(const void* logits, int64_t rows, int64_t width, int64_t row_stride, int dtype,
                                     int32_t* out_ids, b2_stream stream) {
  using namespace b2;
  const char* op = "b2_argmax_rows_static";
  if (dtype != B2_F32 && dtype != B2_F16) { set_error("%s: dtype must be B2_F32 or B2_F16", op); return B2_ERR_INVALID; }
  if (rows < 0 || width <= 0 || width > 0x7fffffffll || row_stride < width) {
    set_error("%s: rows must be >= 0, 0 < width < 2^31 and row_stride >= width", op);
    return B2_ERR_INVALID;
  }
  if (rows > B2_ARGMAX_STATIC_MAX_ROWS) {
    set_error("%s: %lld rows exceed the built-in scratch of %d rows; use b2_argmax_rows with a workspace", op,
              static_cast<long long>(rows), B2_ARGMAX_STATIC_MAX_ROWS);
    return B2_ERR_TOO_LARGE;
  }
  if (rows == 0) return B2_OK;
  if (logits == nullptr || out_ids == nullptr) { set_error("%s: null pointer", op); return B2_ERR_INVALID; }
  void* scratch = static_scratch_for_current_device();
  if (scratch == nullptr) return B2_ERR_CUDA;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // the array keeps whatever the previous call left: clear the part this call uses, in stream order
  if (cudaMemsetAsync(scratch, 0, argmax_workspace_bytes(rows), s) != cudaSuccess) return launch_status(op);
  return launch_argmax(logits, rows, width, row_stride, dtype, 0, out_ids, nullptr, scratch, s);
}

