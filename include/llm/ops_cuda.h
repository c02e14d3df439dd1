// The in-scope operator functions of the reference's include/llm/ops_cuda.h, with the
// reference's signatures, argument rules and exception types, implemented on the sm_100a
// kernels behind the C ABI (b2ops.h).  Line numbers below are the reference's.
//
// Rules shared by all of them (reference src/ops_cuda.cu:62-73): inputs must be contiguous
// CUDA tensors of dtype F32 or F16, all of one dtype; `*_out` outputs must match the input's
// device, dtype, contiguity and shape exactly; violations throw std::invalid_argument with the
// operator's name as prefix; CUDA failures throw std::runtime_error.  `stream = 0` is the
// calling thread's default stream (the library is built with per-thread default streams, as the
// reference is).  The `*_out` forms allocate nothing and never synchronise.
#pragma once
#include "tensor.h"

#include <cstddef>
#include <cstdint>
#include <cuda_runtime_api.h>
#include <vector>

namespace llm {

// ---- sampling (:46-74).  temperature == 0 is greedy; otherwise scores = logits / temperature, the top_k
// highest (all when 0), of those the shortest prefix with softmax mass >= top_p, one seeded draw.  Every
// call returns one token to the host (blocking), like the reference; the token is the reference's.
struct SamplingConfig {
  float temperature = 0.0f;
  int32_t top_k = 0;
  float top_p = 1.0f;
  uint64_t seed = 0;
};

class CudaSampler {
 public:
  explicit CudaSampler(size_t max_vocab);
  ~CudaSampler();
  CudaSampler(const CudaSampler&) = delete;
  CudaSampler& operator=(const CudaSampler&) = delete;
  int32_t sample_last_row(const Tensor& logits_cuda, const SamplingConfig& config, uint64_t draw_offset);
  int32_t sample_row(const Tensor& logits_bv, size_t batch_index, const SamplingConfig& config, uint64_t draw_offset);
  int32_t sample_last_token_of_batch(const Tensor& logits_bsv, size_t batch_index, const SamplingConfig& config,
                                     uint64_t draw_offset);
 private:
  int32_t sample_row_offset(const Tensor& logits, size_t row_offset, const SamplingConfig& config, uint64_t draw_offset);
  void* workspace_ = nullptr;   // device scratch for one row of max_vocab_ logits, allocated once
  size_t max_vocab_ = 0;
};

// ---- allocating forms (:77-82)
Tensor cuda_rms_norm(const Tensor& input, const Tensor& weight, float eps);
Tensor cuda_add(const Tensor& lhs, const Tensor& rhs);
Tensor cuda_swiglu(const Tensor& gate, const Tensor& up);
Tensor cuda_rope(const Tensor& input, const std::vector<int32_t>& positions, float theta);          // [T,H,D], T positions
Tensor cuda_rope_batched(const Tensor& input, const std::vector<int32_t>& positions, float theta);  // [B,S,H,D], S positions
Tensor cuda_softmax_last_dim(const Tensor& input);

// ---- caller-provided outputs (:113-131)
void cuda_rms_norm_out(const Tensor& input, const Tensor& weight, float eps, Tensor& output,
                       cudaStream_t stream = 0);
void cuda_add_out(const Tensor& lhs, const Tensor& rhs, Tensor& output, cudaStream_t stream = 0);
void cuda_add_rms_norm_out(const Tensor& lhs, const Tensor& rhs, const Tensor& weight, float eps,
                           Tensor& residual, Tensor& normalized, cudaStream_t stream = 0);
void cuda_swiglu_out(const Tensor& gate, const Tensor& up, Tensor& output, cudaStream_t stream = 0);
// positions_device: CUDA/F32-typed buffer holding at least S int32 values (:123-125)
void cuda_rope_batched_out(const Tensor& input, const Tensor& positions_device, float theta, Tensor& output);
// positions_device: CUDA/I32 [rows], one position per row of input [rows,H,D] (:126-131).  The reference
// restricts these two to F16, H in {16, 8} and D = 128; any F32/F16 input with an even D is accepted here.
void cuda_rope_batched_positions_out(const Tensor& input, const Tensor& positions_device, float theta,
                                     Tensor& output);
void cuda_rope_token_positions_out(const Tensor& input, const Tensor& positions_device, float theta,
                                   Tensor& output, cudaStream_t stream = 0);

// ---- embedding gather and argmax (:148-156)
// token_ids_device: caller scratch, CUDA/F32-typed, numel >= token_ids.size(); ids are bounds-checked on the host.
void cuda_embedding_lookup_out(const Tensor& embedding_weight, const std::vector<int32_t>& token_ids,
                               Tensor& token_ids_device, Tensor& output);
// token_ids_device: CUDA/F32-typed rank-1 tensor holding int32 bits.  An id outside the table is not
// dereferenced (the reference does not check): its output row is zero.
void cuda_embedding_lookup_device_ids_out(const Tensor& embedding_weight, const Tensor& token_ids_device,
                                          Tensor& output);
int32_t cuda_argmax_last_row(const Tensor& logits_cuda);
Tensor cuda_embedding_lookup(const Tensor& embedding_weight_cuda, const std::vector<int32_t>& token_ids);

}  // namespace llm

// the additions of this library (reduction-mode switch, row-wise argmax, fused QK-norm + RoPE)
#include "ops_cuda_b200.h"
