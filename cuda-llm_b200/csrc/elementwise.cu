// Streaming elementwise operators for sm_100a: residual add and SwiGLU.
// Pure bandwidth: two 16-byte loads and one 16-byte store per lane per step, four or eight
// steps in flight per thread, one tile per thread block.  (A persistent grid that strides
// over the tiles was measured 15 % slower on 5 GB inputs: blocks dispatched in order walk
// DRAM pages in order, a grid-stride loop of a thousand resident blocks does not.)
//
// Replaces reference kernels addk<T> and siluk<T> (src/ops_cuda.cu:76,100), which
// move one element per thread with 2- or 4-byte accesses.
#include "common.cuh"
#include "kernels.h"
#include "b2ops.h"

namespace b2 {
namespace {

constexpr int kThreads = 256;
constexpr int kCtasPerSm = 8;   // grid cap of the scalar (unaligned) kernel

struct AddOp {
  __device__ __forceinline__ float operator()(float a, float b) const { return a + b; }
};
// silu(g) * u with the full-accuracy exponential and IEEE division: the reference's formula
struct SwigluExact {
  __device__ __forceinline__ float operator()(float g, float u) const {
    return __fmul_rn(__fdiv_rn(g, 1.0f + expf(-g)), u);
  }
};
// hardware exponential and reciprocal-based division (about 2 ulp of fp32 each):
// three orders of magnitude below an fp16 ulp, so used for fp16 storage only
struct SwigluHalfStorage {
  __device__ __forceinline__ float operator()(float g, float u) const {
    return __fdividef(g, 1.0f + __expf(-g)) * u;
  }
};

// n_vec full vectors, then `tail` (< kPerVec) trailing scalars handled by the first threads of block 0.
// kUnroll: independent 16-byte loads per input per thread; one tile of kThreads * kUnroll vectors per block
// (blocks beyond the 2^31 - 1 grid limit are folded into a stride, which only inputs above 17 TB would need).
template <typename T, typename Op, int kUnroll>
__global__ void __launch_bounds__(kThreads)
binary_stream_kernel(const T* a, const T* b, T* out, int64_t n_vec, int tail, Op op) {
  constexpr int N = Elem<T>::kPerVec;
  dependent_launch_prologue();
  const uint4* av = reinterpret_cast<const uint4*>(a);
  const uint4* bv = reinterpret_cast<const uint4*>(b);
  uint4* ov = reinterpret_cast<uint4*>(out);
  const int64_t tile = int64_t(kThreads) * kUnroll;
  const int64_t tiles = (n_vec + tile - 1) / tile;
  for (int64_t t = blockIdx.x; t < tiles; t += gridDim.x) {
    const int64_t base = t * tile + threadIdx.x;
    uint4 ra[kUnroll], rb[kUnroll];
#pragma unroll
    for (int k = 0; k < kUnroll; ++k) {
      const int64_t i = base + int64_t(k) * kThreads;
      if (i < n_vec) { ra[k] = ld_stream(av + i); rb[k] = ld_stream(bv + i); }
    }
#pragma unroll
    for (int k = 0; k < kUnroll; ++k) {
      const int64_t i = base + int64_t(k) * kThreads;
      if (i < n_vec) {
        float fa[N], fb[N];
        Elem<T>::unpack(ra[k], fa);
        Elem<T>::unpack(rb[k], fb);
#pragma unroll
        for (int e = 0; e < N; ++e) fa[e] = op(fa[e], fb[e]);
        st_stream(ov + i, Elem<T>::pack(fa));
      }
    }
  }
  if (blockIdx.x == 0 && int(threadIdx.x) < tail) {
    const int64_t i = n_vec * N + threadIdx.x;
    Elem<T>::store(out + i, op(Elem<T>::load(a + i), Elem<T>::load(b + i)));
  }
}

// any alignment: one element per thread per step
template <typename T, typename Op>
__global__ void __launch_bounds__(kThreads)
binary_scalar_kernel(const T* a, const T* b, T* out, int64_t n, Op op) {
  for (int64_t i = int64_t(blockIdx.x) * kThreads + threadIdx.x; i < n; i += int64_t(gridDim.x) * kThreads)
    Elem<T>::store(out + i, op(Elem<T>::load(a + i), Elem<T>::load(b + i)));
}

template <typename T, typename Op, int kUnroll>
int launch_binary(const void* a_, const void* b_, void* out_, int64_t n, Op op, cudaStream_t s, const char* what) {
  if (n == 0) return B2_OK;
  const T* a = static_cast<const T*>(a_);
  const T* b = static_cast<const T*>(b_);
  T* out = static_cast<T*>(out_);
  constexpr int N = Elem<T>::kPerVec;
  if (aligned16(a) && aligned16(b) && aligned16(out)) {
    const int64_t n_vec = n / N;
    const int64_t tiles = (n_vec + int64_t(kThreads) * kUnroll - 1) / (int64_t(kThreads) * kUnroll);
    const unsigned grid = unsigned(tiles < 1 ? 1 : (tiles < 0x7fffffffll ? tiles : 0x7fffffffll));
    launch_kernel(binary_stream_kernel<T, Op, kUnroll>, dim3(grid), dim3(kThreads), 0, s, a, b, out, n_vec, int(n % N), op);
  } else {
    const int64_t blocks = (n + kThreads - 1) / kThreads, cap = int64_t(sm_count()) * kCtasPerSm;
    binary_scalar_kernel<T, Op><<<unsigned(blocks < cap ? blocks : cap), kThreads, 0, s>>>(a, b, out, n, op);
  }
  return launch_status(what);
}

}  // namespace

int launch_add(const void* a, const void* b, void* out, int64_t n, int dtype, cudaStream_t s) {
  return dtype == B2_F32 ? launch_binary<float, AddOp, 8>(a, b, out, n, AddOp{}, s, "add")
                         : launch_binary<__half, AddOp, 8>(a, b, out, n, AddOp{}, s, "add");
}

int launch_swiglu(const void* g, const void* u, void* out, int64_t n, int dtype, int mode, cudaStream_t s) {
  if (dtype == B2_F32) return launch_binary<float, SwigluExact, 4>(g, u, out, n, SwigluExact{}, s, "swiglu");
  if (mode == B2_DETERMINISTIC) return launch_binary<__half, SwigluExact, 4>(g, u, out, n, SwigluExact{}, s, "swiglu");
  return launch_binary<__half, SwigluHalfStorage, 4>(g, u, out, n, SwigluHalfStorage{}, s, "swiglu");
}

}  // namespace b2
