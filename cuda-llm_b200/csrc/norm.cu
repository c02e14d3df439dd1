// RMSNorm family for sm_100a: hidden-state norm, per-head QK-norm (rows = tokens*heads)
// and the fused residual-add + norm.  HBM-bound: every input byte is read once and
// every output byte written once, in 16-byte coalesced accesses; a row lives in
// registers between the sum-of-squares reduction and the scaling.
//
// Replaces reference kernels rmsk<T> and add_rms_normk<T> (src/ops_cuda.cu:77-99,112-131),
// which let a single thread walk the row with a dependent fp64 add chain.
#include "common.cuh"
#include "kernels.h"
#include "b2ops.h"


namespace b2 {
namespace {

constexpr int kRowThreads = 256;   // CTA size of the register-resident kernel
constexpr int kMaxVpt = 16;        // 16-byte vectors held per thread, at most

// ---------------------------------------------------------------------------
// Fast mode, the common case.  `tpr` threads (a power of two <= 256) share a row;
// a CTA of 256 threads covers 256/tpr rows.  Thread k of a row owns vectors
// k, k+tpr, k+2*tpr, ... (VPT of them), so a warp's loads are contiguous.
// Partial sums are fp32; lanes combine by xor-shuffle, warps through shared
// memory in warp order, so the result does not change from run to run.
// ---------------------------------------------------------------------------
template <typename T, int VPT, bool kAdd>
__global__ void __launch_bounds__(kRowThreads)
rms_norm_rows_kernel(const T* x, const T* rhs, const T* __restrict__ w, T* residual, T* out,
                     int64_t rows, int vecs_per_row, int tpr_shift, float hidden_f, float eps) {
  constexpr int N = Elem<T>::kPerVec;
  __shared__ float warp_part[kRowThreads / kWarpSize];
  dependent_launch_prologue();

  const int tpr = 1 << tpr_shift;
  const int lane_in_row = threadIdx.x & (tpr - 1);
  const int local_row = threadIdx.x >> tpr_shift;
  const int64_t row = int64_t(blockIdx.x) * (kRowThreads >> tpr_shift) + local_row;
  const bool row_ok = row < rows;
  const size_t row_off = size_t(row_ok ? row : 0) * size_t(vecs_per_row);
  const uint4* xv = reinterpret_cast<const uint4*>(x) + row_off;
  const uint4* rv = reinterpret_cast<const uint4*>(rhs) + row_off;
  const uint4* wv = reinterpret_cast<const uint4*>(w);

  // issue every load of the row before touching any of them
  uint4 raw_x[VPT], raw_r[VPT], raw_w[VPT];
  bool ok[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = lane_in_row + (i << tpr_shift);
    ok[i] = row_ok && v < vecs_per_row;
    if (ok[i]) {
      raw_x[i] = ld_stream(xv + v);
      if (kAdd) raw_r[i] = ld_stream(rv + v);
    }
  }
#pragma unroll
  for (int i = 0; i < VPT; ++i)
    if (ok[i]) raw_w[i] = ld_reuse(wv + lane_in_row + (i << tpr_shift));

  float val[VPT][N];
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    if (ok[i]) {
      Elem<T>::unpack(raw_x[i], val[i]);
      if (kAdd) {
        float other[N];
        Elem<T>::unpack(raw_r[i], other);
#pragma unroll
        for (int e = 0; e < N; ++e) val[i][e] = val[i][e] + other[e];
        // the residual stream is the rounded sum; the norm below keeps the fp32 sum
        st_stream(reinterpret_cast<uint4*>(residual) + row_off + lane_in_row + (i << tpr_shift),
                  Elem<T>::pack(val[i]));
      }
#pragma unroll
      for (int e = 0; e < N; ++e) ss = fmaf(val[i][e], val[i][e], ss);
    }
  }

  if (tpr <= kWarpSize) {
    ss = group_sum(ss, tpr);
  } else {
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = ss;
    __syncthreads();
    const int warps_per_row = tpr >> 5, first = local_row * warps_per_row;
    float total = 0.0f;
    for (int k = 0; k < warps_per_row; ++k) total += warp_part[first + k];
    ss = total;
  }
  // same expression as the CPU operator: 1/sqrt(sum/H + eps), IEEE sqrt and divide
  const float inv = 1.0f / sqrtf(ss / hidden_f + eps);

#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    if (ok[i]) {
      float wf[N], o[N];
      Elem<T>::unpack(raw_w[i], wf);
#pragma unroll
      for (int e = 0; e < N; ++e) o[e] = __fmul_rn(__fmul_rn(val[i][e], inv), wf[e]);
      st_stream(reinterpret_cast<uint4*>(out) + row_off + lane_in_row + (i << tpr_shift), Elem<T>::pack(o));
    }
  }
}

// ---------------------------------------------------------------------------
// Fast mode for shapes the vector kernel cannot take (row length not a multiple
// of the vector width, unaligned views, very long rows).  One CTA per row, scalar
// coalesced access.  The fp32 row is staged in shared memory when it fits
// (kStage); otherwise the second pass re-reads global memory (the rounded
// residual for the fused form, which also keeps in-place use safe).
// ---------------------------------------------------------------------------
template <typename T, bool kAdd, bool kStage>
__global__ void __launch_bounds__(kRowThreads)
rms_norm_generic_kernel(const T* x, const T* rhs, const T* __restrict__ w, T* residual, T* out,
                        int64_t rows, int64_t hidden, float eps) {
  extern __shared__ float staged[];
  __shared__ float scratch[32];
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * hidden;
    const T* rr = rhs + row * hidden;
    T* res = residual + row * hidden;
    T* o = out + row * hidden;
    float ss = 0.0f;
    for (int64_t j = threadIdx.x; j < hidden; j += kRowThreads) {
      float v = Elem<T>::load(xr + j);
      if (kAdd) { v = v + Elem<T>::load(rr + j); Elem<T>::store(res + j, v); }
      if (kStage) staged[j] = v;
      ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / float(hidden) + eps);
    for (int64_t j = threadIdx.x; j < hidden; j += kRowThreads) {
      const float v = kStage ? staged[j] : Elem<T>::load(kAdd ? res + j : xr + j);
      Elem<T>::store(o + j, __fmul_rn(__fmul_rn(v, inv), Elem<T>::load(w + j)));
    }
    __syncthreads();  // staged[] is rewritten by the next row
  }
}

// ---------------------------------------------------------------------------
// Deterministic mode: the arithmetic of the reference kernels, bit for bit.
// sum = fp64 running sum of double(v)*double(v) in index order (the product of two
// fp32 values is exact in fp64, so fused or unfused multiply-add give the same
// bits); inv = float(1.0 / sqrt(sum/H + eps)) in fp64; out = rn(rn(x*inv)*w).
// The fused form stores round(v), sums the unrounded v and normalises the
// re-read rounded residual (src/ops_cuda.cu:84-97).
// All 32 lanes of a warp load a chunk of the row (coalesced) into shared memory,
// lane 0 walks the chunk; one warp per row.
// ---------------------------------------------------------------------------
constexpr int kOrderedWarps = 4, kOrderedChunk = 1024;

template <typename T, bool kAdd>
__global__ void __launch_bounds__(kOrderedWarps* kWarpSize)
rms_norm_ordered_kernel(const T* x, const T* rhs, const T* __restrict__ w, T* residual, T* out,
                        int64_t rows, int64_t hidden, float eps) {
  __shared__ float stage[kOrderedWarps][kOrderedChunk];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = int64_t(blockIdx.x) * kOrderedWarps + warp;
  if (row >= rows) return;  // whole warp leaves together; no CTA-wide barrier is used below
  const T* xr = x + row * hidden;
  const T* rr = rhs + row * hidden;
  T* res = residual + row * hidden;
  T* o = out + row * hidden;

  double sum = 0.0;
  for (int64_t base = 0; base < hidden; base += kOrderedChunk) {
    const int n = int(hidden - base < kOrderedChunk ? hidden - base : kOrderedChunk);
    for (int j = lane; j < n; j += kWarpSize) {
      float v = Elem<T>::load(xr + base + j);
      if (kAdd) { v = v + Elem<T>::load(rr + base + j); Elem<T>::store(res + base + j, v); }
      stage[warp][j] = v;
    }
    __syncwarp();
    if (lane == 0)
      for (int j = 0; j < n; ++j) { const double d = double(stage[warp][j]); sum += d * d; }
    __syncwarp();
  }
  sum = __shfl_sync(0xffffffffu, sum, 0);
  const float inv = float(1.0 / sqrt(sum / double(hidden) + double(eps)));
  for (int64_t j = lane; j < hidden; j += kWarpSize) {
    // each lane re-reads exactly the residual elements it stored itself
    const float v = Elem<T>::load(kAdd ? res + j : xr + j);
    Elem<T>::store(o + j, __fmul_rn(__fmul_rn(v, inv), Elem<T>::load(w + j)));
  }
}

// ---------------------------------------------------------------------------
// dispatch
// ---------------------------------------------------------------------------

// Vectors per thread: 1 while the whole problem is smaller than a few waves of
// threads (latency matters, use every thread), otherwise `big` to raise the bytes
// in flight per thread; always large enough that a row fits 256 threads.
int pick_vpt(int64_t rows, int vecs_per_row, int big) {
  int vpt = 1;
  const int64_t threads_at_1 = rows * int64_t(vecs_per_row);
  if (threads_at_1 >= int64_t(sm_count()) * 2048 * 2) vpt = big;
  while (vpt > 1 && vecs_per_row < vpt) vpt >>= 1;          // never more vectors than the row has
  while (vpt < kMaxVpt && vecs_per_row > kRowThreads * vpt) vpt <<= 1;
  return vpt;
}

template <typename T, bool kAdd, int VPT>
void launch_rows_vpt(const T* x, const T* rhs, const T* w, T* residual, T* out, int64_t rows, int vecs,
                     int64_t hidden, float eps, cudaStream_t s) {
  int tpr = next_pow2((vecs + VPT - 1) / VPT);
  if (tpr > kRowThreads) tpr = kRowThreads;
  int shift = 0;
  while ((1 << shift) < tpr) ++shift;
  const int rows_per_cta = kRowThreads >> shift;
  const unsigned grid = unsigned((rows + rows_per_cta - 1) / rows_per_cta);
  launch_kernel(rms_norm_rows_kernel<T, VPT, kAdd>, dim3(grid), dim3(kRowThreads), 0, s, x, rhs, w, residual, out, rows, vecs,
                shift, float(hidden), eps);
}

template <typename T, bool kAdd>
int launch_typed(const void* x_, const void* rhs_, const void* w_, void* residual_, void* out_, int64_t rows,
                 int64_t hidden, float eps, int mode, cudaStream_t s) {
  if (rows == 0 || hidden == 0) return B2_OK;
  const T* x = static_cast<const T*>(x_);
  const T* rhs = static_cast<const T*>(kAdd ? rhs_ : x_);
  const T* w = static_cast<const T*>(w_);
  T* residual = static_cast<T*>(kAdd ? residual_ : out_);
  T* out = static_cast<T*>(out_);
  constexpr int N = Elem<T>::kPerVec;

  if (mode == B2_DETERMINISTIC) {
    const unsigned grid = unsigned((rows + kOrderedWarps - 1) / kOrderedWarps);
    rms_norm_ordered_kernel<T, kAdd><<<grid, kOrderedWarps * kWarpSize, 0, s>>>(x, rhs, w, residual, out, rows,
                                                                               hidden, eps);
    return launch_status(kAdd ? "add_rms_norm (deterministic)" : "rms_norm (deterministic)");
  }

  const bool vec_ok = hidden % N == 0 && hidden / N <= int64_t(kRowThreads) * kMaxVpt && aligned16(x) &&
                      aligned16(rhs) && aligned16(w) && aligned16(residual) && aligned16(out);
  if (vec_ok) {
    const int vecs = int(hidden / N);
    switch (pick_vpt(rows, vecs, kAdd ? 2 : 4)) {
      case 1: launch_rows_vpt<T, kAdd, 1>(x, rhs, w, residual, out, rows, vecs, hidden, eps, s); break;
      case 2: launch_rows_vpt<T, kAdd, 2>(x, rhs, w, residual, out, rows, vecs, hidden, eps, s); break;
      case 4: launch_rows_vpt<T, kAdd, 4>(x, rhs, w, residual, out, rows, vecs, hidden, eps, s); break;
      case 8: launch_rows_vpt<T, kAdd, 8>(x, rhs, w, residual, out, rows, vecs, hidden, eps, s); break;
      default: launch_rows_vpt<T, kAdd, 16>(x, rhs, w, residual, out, rows, vecs, hidden, eps, s); break;
    }
    return launch_status(kAdd ? "add_rms_norm" : "rms_norm");
  }

  const unsigned grid = unsigned(rows < int64_t(sm_count()) * 8 ? rows : int64_t(sm_count()) * 8);
  const size_t stage_bytes = size_t(hidden) * sizeof(float);
  if (stage_bytes <= 200 * 1024) {
    auto kernel = rms_norm_generic_kernel<T, kAdd, true>;
    if (stage_bytes > 48 * 1024 &&
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(stage_bytes)) != cudaSuccess)
      return launch_status("rms_norm (generic) shared-memory opt-in");
    kernel<<<grid, kRowThreads, stage_bytes, s>>>(x, rhs, w, residual, out, rows, hidden, eps);
  } else {
    rms_norm_generic_kernel<T, kAdd, false><<<grid, kRowThreads, 0, s>>>(x, rhs, w, residual, out, rows, hidden, eps);
  }
  return launch_status(kAdd ? "add_rms_norm (generic)" : "rms_norm (generic)");
}

}  // namespace

int launch_rms_norm(const void* x, const void* w, void* out, int64_t rows, int64_t hidden, float eps, int dtype,
                    int mode, cudaStream_t s) {
  return dtype == B2_F32 ? launch_typed<float, false>(x, nullptr, w, nullptr, out, rows, hidden, eps, mode, s)
                         : launch_typed<__half, false>(x, nullptr, w, nullptr, out, rows, hidden, eps, mode, s);
}

int launch_add_rms_norm(const void* lhs, const void* rhs, const void* w, void* residual, void* normalized,
                        int64_t rows, int64_t hidden, float eps, int dtype, int mode, cudaStream_t s) {
  return dtype == B2_F32
             ? launch_typed<float, true>(lhs, rhs, w, residual, normalized, rows, hidden, eps, mode, s)
             : launch_typed<__half, true>(lhs, rhs, w, residual, normalized, rows, hidden, eps, mode, s);
}

}  // namespace b2
