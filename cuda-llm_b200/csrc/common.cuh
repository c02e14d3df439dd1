// Shared device helpers for the sm_100a tensor-op kernels: 16-byte vector access
// with streaming cache hints, fp16/fp32 packing, and fixed-order reductions.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b2 {

constexpr int kWarpSize = 32;
constexpr int kSmCount = 148;  // B200; the launch helpers query the device and fall back to this

// ---- element traits ---------------------------------------------------------

template <typename T> struct Elem;
template <> struct Elem<float> {
  static constexpr int kPerVec = 4;  // elements in one 16-byte vector
  static __device__ __forceinline__ float load(const float* p) { return *p; }
  static __device__ __forceinline__ void store(float* p, float v) { *p = v; }
  static __device__ __forceinline__ void unpack(const uint4& v, float* f) {
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
  }
  static __device__ __forceinline__ uint4 pack(const float* f) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  }
  // the same vector as kPerVec/2 pairs, for the packed fp32x2 arithmetic of sm_100
  static __device__ __forceinline__ void unpack2(const uint4& v, float2* f) {
    f[0] = make_float2(__uint_as_float(v.x), __uint_as_float(v.y));
    f[1] = make_float2(__uint_as_float(v.z), __uint_as_float(v.w));
  }
  static __device__ __forceinline__ uint4 pack2(const float2* f) {
    return make_uint4(__float_as_uint(f[0].x), __float_as_uint(f[0].y), __float_as_uint(f[1].x), __float_as_uint(f[1].y));
  }
};
template <> struct Elem<__half> {
  static constexpr int kPerVec = 8;
  static __device__ __forceinline__ float load(const __half* p) { return __half2float(*p); }
  // __float2half rounds to nearest even, the rounding of every reference kernel store
  static __device__ __forceinline__ void store(__half* p, float v) { *p = __float2half(v); }
  static __device__ __forceinline__ void unpack(const uint4& v, float* f) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 t = __half22float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
  }
  static __device__ __forceinline__ uint4 pack(const float* f) {
    uint4 v;
    __half2* h = reinterpret_cast<__half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    return v;
  }
  static __device__ __forceinline__ void unpack2(const uint4& v, float2* f) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) f[i] = __half22float2(h[i]);
  }
  static __device__ __forceinline__ uint4 pack2(const float2* f) {
    uint4 v;
    __half2* h = reinterpret_cast<__half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __float22half2_rn(f[i]);
    return v;
  }
};

// ---- 16-byte global access ---------------------------------------------------
// Activations are read once and written once: "cs" (cache-streaming) marks the
// lines evict-first so they do not push reusable data (weights, sin/cos tables)
// out of L2.  These are ordinary coherent accesses, so in-place use is safe.

__device__ __forceinline__ uint4 ld_stream(const void* p) { return __ldcs(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ void st_stream(void* p, const uint4& v) { __stcs(reinterpret_cast<uint4*>(p), v); }
// small, reused, never written by the same kernel (norm weights)
__device__ __forceinline__ uint4 ld_reuse(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }

__host__ __device__ __forceinline__ bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- reductions with a fixed order (run-to-run bit-identical) -----------------

// Sum over an aligned group of `width` lanes (power of two, <= 32); all 32 lanes call.
__device__ __forceinline__ float group_sum(float v, int width) {
  for (int offset = width >> 1; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
  return v;
}
__device__ __forceinline__ float warp_sum(float v) { return group_sum(v, kWarpSize); }
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, offset));
  return v;
}

// Whole-CTA reductions through a 32-float scratch array; every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from an earlier call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = 0.0f;
  for (int k = 0; k < warps; ++k) total += scratch[k];
  return total;
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = scratch[0];
  for (int k = 1; k < warps; ++k) total = fmaxf(total, scratch[k]);
  return total;
}

// ---- programmatic dependent launch -----------------------------------------------
// A kernel launched with the "programmatic stream serialization" attribute may start while the kernel before it on
// the stream is still running; griddepcontrol.wait then blocks until that kernel has completed and its writes are
// visible, and griddepcontrol.launch_dependents lets the NEXT kernel's blocks be scheduled early in the same way.
// Kernels of a decode step last a few microseconds, about as long as the gap between two launches: with both
// instructions at the top of a kernel the gap is spent under the previous kernel.  Without the launch attribute
// both instructions do nothing.
// A translation unit whose kernels are launched from the device defines B2_NO_DEPENDENT_LAUNCH: those kernels take
// no part in this (a grid that early-launched dependents wait on must not need new blocks scheduled to finish,
// and a grid with child grids does).
__device__ __forceinline__ void dependent_launch_prologue() {
#ifndef B2_NO_DEPENDENT_LAUNCH
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#endif
}

// ---- host-side launch helpers -------------------------------------------------

bool programmatic_launch_enabled();   // the calling thread's b2_set_programmatic_launch switch

// kernel<<<grid, block, smem, s>>>(args...), with the programmatic-serialization attribute when the switch is on
template <typename... Params, typename... Args>
inline void launch_kernel(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
  if (!programmatic_launch_enabled()) {
    kernel<<<grid, block, smem, s>>>(args...);
    return;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(args)...);   // errors are picked up by launch_status()
}

int sm_count();                       // SMs of the current device (cached per device)
void set_error(const char* fmt, ...);  // records the calling thread's last error message
int launch_status(const char* what);   // cudaGetLastError -> B2_OK / B2_ERR_CUDA (+ message)

inline int ceil_div_i64(int64_t a, int64_t b) { return int((a + b - 1) / b); }
inline int next_pow2(int v) { int p = 1; while (p < v) p <<= 1; return p; }

}  // namespace b2
