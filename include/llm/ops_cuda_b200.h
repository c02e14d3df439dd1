// Additions of this library to the operator API of include/llm/ops_cuda.h: nothing here has a
// counterpart in the reference.  Include llm/ops_cuda.h first (it brings llm::Tensor); this header
// deliberately includes no other llm header, so it can also sit on top of the reference's own
// llm/ops_cuda.h when the reference's layer code is linked against these operators.
#pragma once
#include <cuda_runtime_api.h>

namespace llm {

// Fast: parallel fp32 partial sums.  Deterministic: the summation order of the reference's
// kernels (fp64 index-order sum for the RMSNorm family, fp32 index-order sum for softmax,
// all-fp32 RoPE angles), for bit-level regressions.  Thread-local, set through the RAII guard,
// in the idiom of the reference's CudaLinearModeGuard (:18-38).
enum class CudaReductionMode { kFast, kDeterministic };
class CudaReductionModeGuard {
 public:
  explicit CudaReductionModeGuard(CudaReductionMode mode);
  ~CudaReductionModeGuard();
  CudaReductionModeGuard(const CudaReductionModeGuard&) = delete;
  CudaReductionModeGuard& operator=(const CudaReductionModeGuard&) = delete;
 private:
  CudaReductionMode previous_;
};
CudaReductionMode cuda_reduction_mode();

// ---- additions of this library (no reference counterpart)
// cuda_argmax_rows_out and cuda_lm_head_argmax_out keep a small device scratch (keys and tickets, 12 bytes per
// row) per calling thread and device.  The first call of a thread on a device, and any call with more rows than
// every earlier one, allocates and clears it and waits for the device: make that call before any stream capture.
// The scratch is shared by every stream the thread drives, so one thread's calls on different streams must not
// overlap on the GPU; different threads never share it.
// Row-wise argmax of [R,V] logits into a CUDA/I32 [R] tensor, on `stream`, with no host round trip.
// (The reference reaches rows other than the last only through CudaSampler::sample_row, one blocking
// call per row, src/ops_cuda.cu:961-971.)
void cuda_argmax_rows_out(const Tensor& logits_cuda, Tensor& ids_i32, cudaStream_t stream = 0);
// Fused per-head RMSNorm + RoPE of q [T,Hq,D] and k [T,Hk,D] with one CUDA/I32 position per token:
// one launch for the four the reference's layer makes (src/qwen3_layer_cuda.cu:289-292).
void cuda_qk_norm_rope_out(const Tensor& q, const Tensor& k, const Tensor& q_weight, const Tensor& k_weight,
                           const Tensor& positions_device, float eps, float theta, Tensor& q_out, Tensor& k_out,
                           cudaStream_t stream = 0);

// Decode-size LM head fused with the greedy pick: ids[r] = argmax_j sum_k hidden[r,k] * embedding[j,k], one pass
// over the tied embedding, the logits never read back; `logits` (optional, [rows, vocab], same dtype) also receives
// what cuda_lm_head would return.  One launch for the reference's cuda_lm_head / cuda_linear_out followed by
// cuda_argmax_last_row (src/ops_cuda.cu:885; src/qwen3_cuda_model.cpp:1070-1071,1339).  Arguments are checked as
// cuda_lm_head checks them.  Three or more fp16 rows run on the tensor cores, up to 64 rows per pass over the embedding.
void cuda_lm_head_argmax_out(const Tensor& hidden_states_cuda, const Tensor& tied_embedding_cuda, Tensor& ids_i32,
                             Tensor* logits = nullptr, cudaStream_t stream = 0);

}  // namespace llm
