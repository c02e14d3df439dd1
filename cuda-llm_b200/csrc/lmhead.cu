// Decode-size LM head fused with the greedy pick: logits = hidden x table^T for a handful of
// rows, and each row's arg-max, in ONE pass over the tied embedding table.
//
// Replaces, for decode batches, the reference's pair "cuda_lm_head / cuda_linear_out into a
// [rows, vocab] logits tensor, then cuda_argmax_last_row" (reference include/llm/ops_cuda.h:154,157;
// src/ops_cuda.cu:885; src/qwen3_cuda_model.cpp:1070-1071,1339).  With one to four rows the product
// is bound by reading the table once (151936 x 1024 fp16 = 311 MB), not by arithmetic, so this is
// streaming work for the CUDA cores like the rest of this library: no tensor cores, no library GEMM.
// Writing the logits is optional; the pick never reads them back.
//
// Arithmetic.  fp32 accumulation of fp16 or fp32 storage; the logit is rounded to the storage type
// before it is compared (the reference picks from the stored logits).  The pick follows the
// reference's rule (src/ops_cuda.cu:562-563): largest value, ties to the lowest index, NaN never wins,
// nothing comparable -> 0.  B2_DETERMINISTIC adds the products one by one in ascending k with a
// separately rounded multiply, the order of the reference's CPU `linear` (src/ops_cpu.cpp:9) and,
// for fp16 storage (where the product of two halves is exact in fp32), also of its
// `linear_f16_reference` kernel (src/ops_cuda.cu:101-111).  B2_FAST splits k over the lanes of a
// warp in a fixed order (run-to-run bit-identical).
#include <cfloat>
#include <climits>

#include "b2ops.h"
#include "common.cuh"
#include "kernels.h"

namespace b2 {
namespace {

constexpr int kLmThreads = 256;
constexpr int kLmWarps = kLmThreads / kWarpSize;
constexpr int kLmNone = INT_MAX;
constexpr int64_t kMmaMinRows = 3;   // fp16 batches from this size on go to the tensor-core kernel (lmhead_mma.cu)
constexpr unsigned long long kLmSignBit = 0x8000000000000000ull;

__device__ __forceinline__ bool lm_beats(float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); }

// the packed key of b2_argmax_keys: unsigned order == (value ascending, index descending); 0 = nothing seen
__device__ __forceinline__ unsigned long long lm_pack_key(float v, uint32_t global_index) {
  const uint32_t b = __float_as_uint(v);
  const uint32_t ordered = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
  return (static_cast<unsigned long long>(ordered) << 32) | (0xffffffffu - global_index);
}

template <typename T> __device__ __forceinline__ float round_to_storage(float v);
template <> __device__ __forceinline__ float round_to_storage<float>(float v) { return v; }
template <> __device__ __forceinline__ float round_to_storage<__half>(float v) { return __half2float(__float2half(v)); }

// Sums M values held by every lane over the 32 lanes with M-1 + log2(32/M) shuffles instead of 5*M:
// at each of the first log2(M) steps a lane hands half of its values to its partner and keeps the
// other half.  Afterwards v[0] of lane l is the total of value number l >> (5 - log2 M).
template <int M>
__device__ __forceinline__ void reduce_transpose(float (&v)[M], int lane) {
  int offset = 16;
#pragma unroll
  for (int m = M; m > 1; m >>= 1) {
    const int half = m >> 1;
    const bool upper = (lane & offset) != 0;
#pragma unroll
    for (int i = 0; i < half; ++i) {
      const float send = upper ? v[i] : v[i + half];
      const float keep = upper ? v[i + half] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, offset);
    }
    offset >>= 1;
  }
#pragma unroll
  for (; offset > 0; offset >>= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], offset);
}

template <int M> struct Log2;
template <> struct Log2<1> { static constexpr int value = 0; };
template <> struct Log2<2> { static constexpr int value = 1; };
template <> struct Log2<4> { static constexpr int value = 2; };
template <> struct Log2<8> { static constexpr int value = 3; };
template <> struct Log2<16> { static constexpr int value = 4; };

// Folds the thread block's candidates (slots[warp][slot], `slots_per_row` slots for each of R rows,
// slot = jj * R + r) into the call-wide keys, and lets the last block to arrive publish the result
// and leave the scratch zeroed for the next call.  Only the first `valid` of the R rows exist.
template <int R>
__device__ __forceinline__ void lm_publish(const float (*slot_v)[16], const int (*slot_i)[16], int warps, int slots_per_row,
                                           int64_t index_base, int32_t* out_ids, int64_t* out_keys,
                                           unsigned long long* keys, unsigned int* ticket, int valid = R) {
  __shared__ int last_block;
  if (threadIdx.x < valid) {
    const int r = threadIdx.x;
    float bv = -FLT_MAX;
    int bi = kLmNone;
    for (int w = 0; w < warps; ++w)
      for (int jj = 0; jj < slots_per_row; ++jj) {
        const float v = slot_v[w][jj * R + r];
        const int i = slot_i[w][jj * R + r];
        if (lm_beats(v, i, bv, bi)) { bv = v; bi = i; }
      }
    if (bi != kLmNone) atomicMax(keys + r, lm_pack_key(bv, uint32_t(index_base + bi)));
    __threadfence();
  }
  __syncthreads();
  if (threadIdx.x == 0) last_block = atomicAdd(ticket, 1u) == gridDim.x - 1 ? 1 : 0;
  __syncthreads();
  if (!last_block || threadIdx.x >= valid) return;
  __threadfence();
  const int r = threadIdx.x;
  const unsigned long long key = atomicExch(keys + r, 0ull);
  if (out_keys != nullptr) out_keys[r] = static_cast<int64_t>(key ^ kLmSignBit);
  if (out_ids != nullptr) out_ids[r] = key == 0ull ? 0 : int32_t(0xffffffffu - uint32_t(key & 0xffffffffull));
  if (r == 0) *ticket = 0u;
}

// ---------------------------------------------------------------------------
// Fast kernel.  Persistent grid; a warp takes J table rows at a time (warp g of W takes rows
// (g + i*W)*J .. +J-1, so at any moment the whole GPU reads one contiguous stretch of the table).
// Lane l owns the 16-byte vectors l, l+32, ... of a table row; the matching elements of the R hidden
// rows sit in its registers as fp32 for the whole kernel, so the only traffic in the loop is the
// table itself: KV 16-byte streaming loads per lane per table row, J*KV of them in flight.
// H = KV * 32 * (elements per vector) exactly.
// ---------------------------------------------------------------------------
template <typename T, int KV, int R, int J, bool kAhead>
__global__ void __launch_bounds__(kLmThreads, 1)
lm_head_argmax_kernel(const T* __restrict__ hidden, const T* __restrict__ table, int64_t vocab, int64_t index_base,
                      T* __restrict__ logits_out, int64_t logits_stride, int32_t* out_ids, int64_t* out_keys,
                      unsigned long long* keys, unsigned int* ticket) {
  constexpr int N = Elem<T>::kPerVec;
  constexpr int H = KV * kWarpSize * N;
  constexpr int M = J * R;                       // sums a warp produces per step
  constexpr int kGroup = kWarpSize >> Log2<M>::value;  // lanes that end up holding the same sum
  __shared__ float slot_v[kLmWarps][16];
  __shared__ int slot_i[kLmWarps][16];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  float h[R][KV * N];
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int k = 0; k < KV; ++k)
      Elem<T>::unpack(ld_reuse(hidden + int64_t(r) * H + (k * kWarpSize + lane) * N), &h[r][k * N]);

  const int my = lane >> (5 - Log2<M>::value);   // which of the M sums this lane holds after the reduction
  const int my_jj = my / R, my_r = my - my_jj * R;
  float bv = -FLT_MAX;
  int bi = kLmNone;

  const int64_t total_warps = int64_t(gridDim.x) * kLmWarps;
  auto load_rows = [&](int64_t p, uint4 (&dst)[J][KV]) {
#pragma unroll
    for (int jj = 0; jj < J; ++jj) {
      int64_t j = p * J + jj;
      if (j >= vocab) j = vocab - 1;             // a ragged last step re-reads a row; its sum is dropped below
      const T* row = table + j * H;
#pragma unroll
      for (int k = 0; k < KV; ++k) dst[jj][k] = ld_stream(row + (k * kWarpSize + lane) * N);
    }
  };
  int64_t p = int64_t(blockIdx.x) * kLmWarps + warp;
  uint4 w[J][KV];
  if (p * J < vocab) load_rows(p, w);
  for (; p * J < vocab; p += total_warps) {
    // the next step's rows are requested before this step's arithmetic (where the registers allow it)
    const int64_t pn = p + total_warps;
    uint4 nx[J][KV];
    if constexpr (kAhead) { if (pn * J < vocab) load_rows(pn, nx); }
    float acc[M];
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = 0.0f;
#pragma unroll
    for (int jj = 0; jj < J; ++jj)
#pragma unroll
      for (int k = 0; k < KV; ++k) {
        float f[N];
        Elem<T>::unpack(w[jj][k], f);
#pragma unroll
        for (int q = 0; q < N; ++q)
#pragma unroll
          for (int r = 0; r < R; ++r) acc[jj * R + r] = fmaf(f[q], h[r][k * N + q], acc[jj * R + r]);
      }
    reduce_transpose<M>(acc, lane);
    const int64_t j = p * J + my_jj;
    if (j < vocab) {
      const float v = round_to_storage<T>(acc[0]);
      if (logits_out != nullptr && (lane & (kGroup - 1)) == 0) Elem<T>::store(logits_out + my_r * logits_stride + j, v);
      if (v > bv) { bv = v; bi = int(j); }       // a lane's rows ascend: strictly-greater keeps the lowest index
    }
    if constexpr (kAhead) {
#pragma unroll
      for (int jj = 0; jj < J; ++jj)
#pragma unroll
        for (int k = 0; k < KV; ++k) w[jj][k] = nx[jj][k];
    } else {
      if (pn * J < vocab) load_rows(pn, w);
    }
  }
  if ((lane & (kGroup - 1)) == 0) { slot_v[warp][my] = bv; slot_i[warp][my] = bi; }
  __syncthreads();
  lm_publish<R>(slot_v, slot_i, kLmWarps, J, index_base, out_ids, out_keys, keys, ticket);
}

// ---------------------------------------------------------------------------
// Fast kernel for two to four hidden rows (and for hidden sizes the register-resident kernel is not
// built for).  With more than one hidden row the registers that held them are needed for table
// data in flight, so the hidden rows move to shared memory as fp32 and a warp takes J = 4 table rows
// per step: every 32 bytes a lane reads from shared memory (8 hidden values of one row) meet 4 table
// vectors, which keeps shared-memory traffic at R/2 times the table's (2x for four rows).  K is walked
// in chunks of 32 lanes x 4 vectors; the J x 4 streaming loads of a chunk are issued back to back: for fp32
// right before the chunk's arithmetic (three thread blocks of four warps per SM, ~100 KB of the table in
// flight per SM), for fp16, which carries twice the arithmetic per byte, one chunk ahead (two blocks per
// SM).  Packed fp32x2 multiply-adds; hidden rows laid out in two planes so shared-memory reads are free
// of bank conflicts.  Measured and dropped: staging the table through shared memory with bulk copies
// (cp.async.bulk + mbarrier rings, 16 KB in flight per warp at no register cost) was slower (62.8 us
// against 58.4 for four fp16 rows): the kernel is bound by its own instruction stream there (2 FMAs per
// byte), not by copy latency, and the extra shared-memory reads cost more than the registers they freed.
// H is a multiple of the chunk (1024 fp16 / 512 fp32 elements).
// ---------------------------------------------------------------------------
constexpr int kLmSmemThreads = 128;
constexpr int kLmSmemWarps = kLmSmemThreads / kWarpSize;
constexpr int kLmChunkVecs = 4;

template <typename T, int R, int J, bool kAhead>
__global__ void __launch_bounds__(kLmSmemThreads, kAhead ? 2 : 3)
lm_head_argmax_smem_kernel(const T* __restrict__ hidden, const T* __restrict__ table, int64_t vocab, int H, int64_t index_base,
                           T* __restrict__ logits_out, int64_t logits_stride, int32_t* out_ids, int64_t* out_keys,
                           unsigned long long* keys, unsigned int* ticket, int valid) {
  constexpr int N = Elem<T>::kPerVec;
  constexpr int KC = kLmChunkVecs;
  constexpr int kChunk = kWarpSize * KC * N;
  constexpr int M = J * R;
  constexpr int kGroup = kWarpSize >> Log2<M>::value;
  extern __shared__ __align__(16) float hs[];    // [R][H]
  __shared__ float slot_v[kLmSmemWarps][16];
  __shared__ int slot_i[kLmSmemWarps][16];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  // Layout of a hidden row in shared memory: the first four floats of every 16-byte table vector in one plane,
  // the next four (fp16 vectors hold eight) in a second plane H/2 floats further on, so that the lanes of a warp
  // read consecutive 16-byte pieces of a plane: no bank conflicts (eight floats per lane side by side would put
  // lanes i and i+4 on the same banks).
  constexpr int P = N / 4;
  const int plane = H / P, vecs_per_row = H / N;
  for (int i = threadIdx.x; i < R * vecs_per_row; i += kLmSmemThreads) {
    const int r = i / vecs_per_row, v = i - r * vecs_per_row;
    float f[N];
    if (r < valid) {                             // three rows ride in the four-row kernel: the fourth is zeros
      Elem<T>::unpack(ld_reuse(hidden + int64_t(i) * N), f);
    } else {
#pragma unroll
      for (int q = 0; q < N; ++q) f[q] = 0.0f;
    }
#pragma unroll
    for (int q = 0; q < P; ++q)
      *reinterpret_cast<float4*>(hs + r * H + q * plane + v * 4) = make_float4(f[4 * q], f[4 * q + 1], f[4 * q + 2], f[4 * q + 3]);
  }
  __syncthreads();

  const int my = lane >> (5 - Log2<M>::value);
  const int my_jj = my / R, my_r = my - my_jj * R;
  float bv = -FLT_MAX;
  int bi = kLmNone;
  const int chunks = H / kChunk;
  const int64_t total_warps = int64_t(gridDim.x) * kLmSmemWarps;
  // one chunk of J table rows: J x KC streaming loads, all issued back to back
  auto load_chunk = [&](int64_t p, int c, uint4 (&dst)[J][KC]) {
#pragma unroll
    for (int jj = 0; jj < J; ++jj) {
      int64_t j = p * J + jj;
      if (j >= vocab) j = vocab - 1;             // a ragged last step re-reads a row; its sums are dropped below
      const T* row = table + j * H + c * kChunk + lane * N;
#pragma unroll
      for (int k = 0; k < KC; ++k) dst[jj][k] = ld_stream(row + k * kWarpSize * N);
    }
  };
  int64_t p = int64_t(blockIdx.x) * kLmSmemWarps + warp;
  uint4 w[J][KC];
  if constexpr (kAhead) { if (p * J < vocab) load_chunk(p, 0, w); }
  for (; p * J < vocab; p += total_warps) {
    // packed fp32x2 arithmetic (one instruction per two multiply-adds): even and odd k accumulate apart
    float2 acc2[M];
#pragma unroll
    for (int m = 0; m < M; ++m) acc2[m] = make_float2(0.0f, 0.0f);
    for (int c = 0; c < chunks; ++c) {
      // kAhead: the chunk after this one (of these rows, or the first of the next rows) is requested before this
      // chunk's arithmetic, so the copy latency and the arithmetic overlap inside one warp
      uint4 nx[J][KC];
      if constexpr (kAhead) {
        const bool last = c + 1 == chunks;
        const int64_t pn = last ? p + total_warps : p;
        if (pn * J < vocab) load_chunk(pn, last ? 0 : c + 1, nx);
      } else {
        load_chunk(p, c, w);
      }
#pragma unroll
      for (int k = 0; k < KC; ++k) {
        float2 f[J][N / 2];
#pragma unroll
        for (int jj = 0; jj < J; ++jj) Elem<T>::unpack2(w[jj][k], f[jj]);
        const float* hk = hs + ((c * KC + k) * kWarpSize + lane) * 4;
        float2 hr[R][N / 2];
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
          for (int q = 0; q < P; ++q) {
            const float4 t = *reinterpret_cast<const float4*>(hk + r * H + q * plane);
            hr[r][2 * q] = make_float2(t.x, t.y);
            hr[r][2 * q + 1] = make_float2(t.z, t.w);
          }
        // q outermost: consecutive multiply-adds go to J * R different accumulators, none waits for the one before
#pragma unroll
        for (int q = 0; q < N / 2; ++q)
#pragma unroll
          for (int jj = 0; jj < J; ++jj)
#pragma unroll
            for (int r = 0; r < R; ++r) acc2[jj * R + r] = __ffma2_rn(f[jj][q], hr[r][q], acc2[jj * R + r]);
      }
      if constexpr (kAhead) {
#pragma unroll
        for (int jj = 0; jj < J; ++jj)
#pragma unroll
          for (int k = 0; k < KC; ++k) w[jj][k] = nx[jj][k];
      }
    }
    float acc[M];
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = acc2[m].x + acc2[m].y;
    reduce_transpose<M>(acc, lane);
    const int64_t j = p * J + my_jj;
    if (j < vocab && my_r < valid) {
      const float v = round_to_storage<T>(acc[0]);
      if (logits_out != nullptr && (lane & (kGroup - 1)) == 0) Elem<T>::store(logits_out + my_r * logits_stride + j, v);
      if (v > bv) { bv = v; bi = int(j); }
    }
  }
  if ((lane & (kGroup - 1)) == 0) { slot_v[warp][my] = bv; slot_i[warp][my] = bi; }
  __syncthreads();
  lm_publish<R>(slot_v, slot_i, kLmSmemWarps, J, index_base, out_ids, out_keys, keys, ticket, valid);
}

// ---------------------------------------------------------------------------
// Ordered kernel (B2_DETERMINISTIC, and every shape the fast kernel is not built for): one thread
// per table row walks k upwards, `acc = rn(acc + rn(x * w))`; the hidden rows sit in shared memory
// as fp32 (every lane reads the same word: a broadcast).  Each thread reads its own row in 16-byte
// pieces; the 128-byte lines it touches stay in L1 until it has walked through them.
// ---------------------------------------------------------------------------
constexpr int kOrdLmThreads = 128;

template <typename T, int R, bool kVec>
__global__ void __launch_bounds__(kOrdLmThreads)
lm_head_ordered_kernel(const T* __restrict__ hidden, const T* __restrict__ table, int64_t vocab, int H, int64_t index_base,
                       T* __restrict__ logits_out, int64_t logits_stride, int32_t* out_ids, int64_t* out_keys,
                       unsigned long long* keys, unsigned int* ticket) {
  constexpr int N = Elem<T>::kPerVec;
  extern __shared__ float hs[];                  // [R][H]
  __shared__ float slot_v[kOrdLmThreads / kWarpSize][16];
  __shared__ int slot_i[kOrdLmThreads / kWarpSize][16];
  for (int i = threadIdx.x; i < R * H; i += kOrdLmThreads) hs[i] = Elem<T>::load(hidden + i);
  __syncthreads();

  const int64_t j = int64_t(blockIdx.x) * kOrdLmThreads + threadIdx.x;
  float acc[R];
#pragma unroll
  for (int r = 0; r < R; ++r) acc[r] = 0.0f;
  if (j < vocab) {
    const T* row = table + j * H;
    if (kVec) {
      for (int k = 0; k < H; k += N) {
        float f[N];
        Elem<T>::unpack(__ldg(reinterpret_cast<const uint4*>(row + k)), f);
#pragma unroll
        for (int q = 0; q < N; ++q)
#pragma unroll
          for (int r = 0; r < R; ++r) acc[r] = __fadd_rn(acc[r], __fmul_rn(hs[r * H + k + q], f[q]));
      }
    } else {
      for (int k = 0; k < H; ++k) {
        const float f = Elem<T>::load(row + k);
#pragma unroll
        for (int r = 0; r < R; ++r) acc[r] = __fadd_rn(acc[r], __fmul_rn(hs[r * H + k], f));
      }
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int r = 0; r < R; ++r) {
    float bv = -FLT_MAX;
    int bi = kLmNone;
    if (j < vocab) {
      const float v = round_to_storage<T>(acc[r]);
      if (logits_out != nullptr) Elem<T>::store(logits_out + r * logits_stride + j, v);
      if (v > bv) { bv = v; bi = int(j); }
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
      const float ov = __shfl_down_sync(0xffffffffu, bv, offset);
      const int oi = __shfl_down_sync(0xffffffffu, bi, offset);
      if (lm_beats(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) { slot_v[warp][r] = bv; slot_i[warp][r] = bi; }
  }
  __syncthreads();
  lm_publish<R>(slot_v, slot_i, kOrdLmThreads / kWarpSize, 1, index_base, out_ids, out_keys, keys, ticket);
}

// The ordered kernel with coalesced reads: a warp owns 32 table rows (one per lane, as above) and walks k in
// tiles of 128 bytes per row.  The tile is fetched cooperatively - eight lanes read one row's 128 bytes, four
// rows per load instruction - into a shared-memory tile whose rows are 144 bytes apart (no bank conflicts on
// the way in or out), then every lane reads its own row back and adds its products in ascending k exactly as
// before.  Same arithmetic, same bits; the per-lane 16-byte reads at a 2 KB stride (32 cache lines per load
// instruction) are gone.  H is a multiple of the tile (64 fp16 / 32 fp32 elements), pointers 16-byte aligned.
constexpr int kOrdTileVecs = 8;                    // 16-byte vectors per row per tile
constexpr int kOrdTileStride = kOrdTileVecs + 1;   // row stride in vectors: 144 bytes

template <typename T, int R>
__global__ void __launch_bounds__(kOrdLmThreads)
lm_head_ordered_tiled_kernel(const T* __restrict__ hidden, const T* __restrict__ table, int64_t vocab, int H, int64_t index_base,
                             T* __restrict__ logits_out, int64_t logits_stride, int32_t* out_ids, int64_t* out_keys,
                             unsigned long long* keys, unsigned int* ticket) {
  constexpr int N = Elem<T>::kPerVec;
  constexpr int kTile = kOrdTileVecs * N;          // elements of k per tile
  constexpr int kWarps = kOrdLmThreads / kWarpSize;
  extern __shared__ __align__(16) unsigned char ord_smem[];
  uint4* tiles = reinterpret_cast<uint4*>(ord_smem);                                        // [warps][32][kOrdTileStride]
  float* hs = reinterpret_cast<float*>(ord_smem + size_t(kWarps) * kWarpSize * kOrdTileStride * 16);   // [R][H]
  __shared__ float slot_v[kWarps][16];
  __shared__ int slot_i[kWarps][16];
  for (int i = threadIdx.x; i < R * H; i += kOrdLmThreads) hs[i] = Elem<T>::load(hidden + i);
  __syncthreads();

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint4* tile = tiles + warp * kWarpSize * kOrdTileStride;
  const int64_t first = (int64_t(blockIdx.x) * kWarps + warp) * kWarpSize;   // this warp's first table row
  const int64_t j = first + lane;
  // the row and the 16-byte column this lane fetches in step i of a tile: vector i*32 + lane of the 32 x 8 tile
  const int fetch_col = lane & (kOrdTileVecs - 1), fetch_row0 = lane / kOrdTileVecs;
  float acc[R];
#pragma unroll
  for (int r = 0; r < R; ++r) acc[r] = 0.0f;
  if (first < vocab) {
    for (int k0 = 0; k0 < H; k0 += kTile) {
      uint4 v[kOrdTileVecs];
#pragma unroll
      for (int i = 0; i < kOrdTileVecs; ++i) {
        int64_t row = first + fetch_row0 + i * (kWarpSize / kOrdTileVecs);
        if (row >= vocab) row = vocab - 1;           // rows past the end re-read the last row; their sums are dropped
        v[i] = __ldg(reinterpret_cast<const uint4*>(table + row * H + k0 + fetch_col * N));
      }
      __syncwarp();                                  // the previous tile has been read by every lane
#pragma unroll
      for (int i = 0; i < kOrdTileVecs; ++i)
        tile[(fetch_row0 + i * (kWarpSize / kOrdTileVecs)) * kOrdTileStride + fetch_col] = v[i];
      __syncwarp();
#pragma unroll
      for (int c = 0; c < kOrdTileVecs; ++c) {
        float f[N];
        Elem<T>::unpack(tile[lane * kOrdTileStride + c], f);
#pragma unroll
        for (int q = 0; q < N; ++q)
#pragma unroll
          for (int r = 0; r < R; ++r) acc[r] = __fadd_rn(acc[r], __fmul_rn(hs[r * H + k0 + c * N + q], f[q]));
      }
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    float bv = -FLT_MAX;
    int bi = kLmNone;
    if (j < vocab) {
      const float v = round_to_storage<T>(acc[r]);
      if (logits_out != nullptr) Elem<T>::store(logits_out + r * logits_stride + j, v);
      if (v > bv) { bv = v; bi = int(j); }
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
      const float ov = __shfl_down_sync(0xffffffffu, bv, offset);
      const int oi = __shfl_down_sync(0xffffffffu, bi, offset);
      if (lm_beats(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) { slot_v[warp][r] = bv; slot_i[warp][r] = bi; }
  }
  __syncthreads();
  lm_publish<R>(slot_v, slot_i, kWarps, 1, index_base, out_ids, out_keys, keys, ticket);
}

// ---------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------

template <typename T, int KV, int R, int J, bool kAhead>
int launch_fast(const T* hidden, const T* table, int64_t vocab, int64_t index_base, T* logits_out, int64_t logits_stride,
                int32_t* out_ids, int64_t* out_keys, unsigned long long* keys, unsigned int* ticket, cudaStream_t s) {
  auto kernel = lm_head_argmax_kernel<T, KV, R, J, kAhead>;
  static int per_sm = 0;                         // resident thread blocks per SM (same on every B200)
  if (per_sm == 0) {
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, kLmThreads, 0) != cudaSuccess || n < 1) n = 1;
    per_sm = n > 4 ? 4 : n;
  }
  int64_t blocks = int64_t(sm_count()) * per_sm;
  const int64_t needed = (vocab + int64_t(J) * kLmWarps - 1) / (int64_t(J) * kLmWarps);
  if (blocks > needed) blocks = needed;
  kernel<<<unsigned(blocks), kLmThreads, 0, s>>>(hidden, table, vocab, index_base, logits_out, logits_stride, out_ids,
                                                 out_keys, keys, ticket);
  return launch_status("lm_head_argmax");
}

template <typename T, int R>
int launch_smem(const T* hidden, const T* table, int64_t vocab, int64_t H, int64_t index_base, T* logits_out,
                int64_t logits_stride, int32_t* out_ids, int64_t* out_keys, unsigned long long* keys, unsigned int* ticket,
                int valid, cudaStream_t s) {
  constexpr int J = 4;
  // fp16 rows carry twice the arithmetic per byte: there the next chunk is requested ahead of the arithmetic
  // fp16 rows carry twice the arithmetic per byte: there the next chunk is requested ahead of the arithmetic
  // (measured on 4 x 1024 by 151936 x 1024: 58.4 us against 60.2; fp32 is at the copy rate either way)
  auto kernel = lm_head_argmax_smem_kernel<T, R, J, (Elem<T>::kPerVec == 8 && R >= 2)>;
  const size_t smem = size_t(R) * size_t(H) * sizeof(float);
  if (smem > 48 * 1024 &&
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess)
    return launch_status("lm_head_argmax (shared-memory attribute)");
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kLmSmemThreads, smem) != cudaSuccess || per_sm < 1) per_sm = 1;
  int64_t blocks = int64_t(sm_count()) * per_sm;
  const int64_t needed = (vocab + int64_t(J) * kLmSmemWarps - 1) / (int64_t(J) * kLmSmemWarps);
  if (blocks > needed) blocks = needed;
  kernel<<<unsigned(blocks), kLmSmemThreads, smem, s>>>(hidden, table, vocab, int(H), index_base, logits_out, logits_stride,
                                                       out_ids, out_keys, keys, ticket, valid);
  return launch_status("lm_head_argmax");
}

// hidden rows the shared-memory kernel takes in one pass (R * H fp32 values within 64 KB), 0 = shape not built
template <typename T> int smem_rows_per_pass(int64_t H) {
  if (H % (kWarpSize * kLmChunkVecs * Elem<T>::kPerVec) != 0) return 0;
  return H <= 4096 ? 4 : H <= 8192 ? 2 : 1;
}

template <typename T, int R>
int launch_ordered(const T* hidden, const T* table, int64_t vocab, int64_t H, int64_t index_base, T* logits_out,
                   int64_t logits_stride, int32_t* out_ids, int64_t* out_keys, unsigned long long* keys,
                   unsigned int* ticket, cudaStream_t s) {
  const size_t smem = size_t(R) * size_t(H) * sizeof(float);
  const unsigned blocks = unsigned((vocab + kOrdLmThreads - 1) / kOrdLmThreads);
  const bool vec = aligned16(table) && H % Elem<T>::kPerVec == 0;
  if (vec && H % (kOrdTileVecs * Elem<T>::kPerVec) == 0) {
    auto kernel = lm_head_ordered_tiled_kernel<T, R>;
    const size_t tiled = smem + size_t(kOrdLmThreads) * kOrdTileStride * 16;
    if (tiled > 48 * 1024 &&
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(tiled)) != cudaSuccess)
      return launch_status("lm_head_argmax (shared-memory attribute)");
    kernel<<<blocks, kOrdLmThreads, tiled, s>>>(hidden, table, vocab, int(H), index_base, logits_out, logits_stride, out_ids,
                                                out_keys, keys, ticket);
    return launch_status("lm_head_argmax (ordered)");
  }
  if (vec)
    lm_head_ordered_kernel<T, R, true><<<blocks, kOrdLmThreads, smem, s>>>(hidden, table, vocab, int(H), index_base, logits_out,
                                                                          logits_stride, out_ids, out_keys, keys, ticket);
  else
    lm_head_ordered_kernel<T, R, false><<<blocks, kOrdLmThreads, smem, s>>>(hidden, table, vocab, int(H), index_base,
                                                                           logits_out, logits_stride, out_ids, out_keys, keys,
                                                                           ticket);
  return launch_status("lm_head_argmax (ordered)");
}

// 1 where the register-resident kernel is built for this hidden size (it then serves single rows), else 0.
// Only hidden size 1024: at 2048 and 4096 a lane would keep 64-128 hidden values and a whole table row's vectors in
// registers, one block per SM, and measured slower than the shared-memory kernel (fp16 2048: 105 us against 93).
template <typename T> int fast_rows_per_pass(int64_t H) { return H == 1024 ? 1 : 0; }

template <typename T>
int launch_typed(const void* hidden_, const void* table_, int64_t rows, int64_t H, int64_t vocab, int mode,
                 int64_t index_base, void* logits_, int64_t logits_stride, int32_t* out_ids, int64_t* out_keys,
                 void* workspace, cudaStream_t s) {
  constexpr int N = Elem<T>::kPerVec;
  const T* hidden = static_cast<const T*>(hidden_);
  const T* table = static_cast<const T*>(table_);
  T* logits = static_cast<T*>(logits_);
  auto* keys = static_cast<unsigned long long*>(workspace);
  auto* tickets = reinterpret_cast<unsigned int*>(keys + rows);
  const bool aligned = aligned16(hidden) && aligned16(table);
  const int reg_cap = mode == B2_FAST && aligned ? fast_rows_per_pass<T>(H) : 0;    // register-resident kernel: one row
  const int smem_cap = mode == B2_FAST && aligned ? smem_rows_per_pass<T>(H) : 0;
  const int ord_cap = H <= 2048 ? 4 : H <= 4096 ? 2 : 1;   // ordered kernel: R * H floats of shared memory, <= 32 KB
  for (int64_t r0 = 0; r0 < rows;) {
    const int64_t left = rows - r0;
    const bool use_reg = reg_cap > 0 && (left == 1 || smem_cap == 0);
    const bool use_smem = !use_reg && smem_cap > 0;
    const int cap = use_reg ? 1 : use_smem ? smem_cap : ord_cap;
    int R = left >= 4 ? 4 : left >= 2 ? 2 : 1;   // rows this pass takes
    if (use_smem && left == 3 && cap >= 4) R = 3;  // three rows ride in the four-row kernel
    if (R > cap) R = cap;
    const T* hp = hidden + r0 * H;
    T* lp = logits ? logits + r0 * logits_stride : nullptr;
    int32_t* ip = out_ids ? out_ids + r0 : nullptr;
    int64_t* kp = out_keys ? out_keys + r0 : nullptr;
    int rc;
    if (sizeof(T) == 2 && mode == B2_FAST && left >= kMmaMinRows && lm_head_mma_supported(hp, table, H, vocab)) {
      // more rows than the matrix-vector kernels take in one pass: tensor cores, up to 64 rows per pass over the table
      const int64_t take = left < 64 ? left : 64;
      rc = launch_lm_head_mma(hp, table, take, H, vocab, index_base, lp, logits_stride, ip, kp, keys + r0, tickets + r0, s);
      if (rc != B2_OK) return rc;
      r0 += take;
      continue;
    }
#define B2_LM_FAST(KV, RR, JJ, AH) \
  rc = launch_fast<T, KV, RR, JJ, AH>(hp, table, vocab, index_base, lp, logits_stride, ip, kp, keys + r0, tickets + r0, s)
#define B2_LM_SMEM(RR) \
  rc = launch_smem<T, RR>(hp, table, vocab, H, index_base, lp, logits_stride, ip, kp, keys + r0, tickets + r0, R, s)
#define B2_LM_ORD(RR) \
  rc = launch_ordered<T, RR>(hp, table, vocab, H, index_base, lp, logits_stride, ip, kp, keys + r0, tickets + r0, s)
    if (use_reg) {
      constexpr int KV1 = 1024 / (kWarpSize * N);
      B2_LM_FAST(KV1, 1, (N == 8 ? 2 : 1), true);
    } else if (use_smem) {
      if (R >= 3) B2_LM_SMEM(4);
      else if (R == 2) B2_LM_SMEM(2);
      else B2_LM_SMEM(1);
    } else {
      if (R == 4) B2_LM_ORD(4);
      else if (R == 2) B2_LM_ORD(2);
      else B2_LM_ORD(1);
    }
#undef B2_LM_FAST
#undef B2_LM_SMEM
#undef B2_LM_ORD
    if (rc != B2_OK) return rc;
    r0 += R;
  }
  return B2_OK;
}

}  // namespace

int launch_lm_head_argmax(const void* hidden, const void* table, int64_t rows, int64_t hidden_size, int64_t vocab,
                          int dtype, int mode, int64_t index_base, void* logits_out, int64_t logits_stride,
                          int32_t* out_ids, int64_t* out_keys, void* workspace, cudaStream_t s) {
  if (rows == 0) return B2_OK;
  return dtype == B2_F32 ? launch_typed<float>(hidden, table, rows, hidden_size, vocab, mode, index_base, logits_out,
                                               logits_stride, out_ids, out_keys, workspace, s)
                         : launch_typed<__half>(hidden, table, rows, hidden_size, vocab, mode, index_base, logits_out,
                                                logits_stride, out_ids, out_keys, workspace, s);
}

}  // namespace b2
