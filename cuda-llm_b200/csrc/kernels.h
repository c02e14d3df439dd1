// Host-side launchers of the sm_100a kernels.  Arguments are already validated by
// the C ABI layer (capi.cu); each returns B2_OK or B2_ERR_CUDA.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace b2 {

// norm.cu
int launch_rms_norm(const void* x, const void* w, void* out, int64_t rows, int64_t hidden, float eps,
                    int dtype, int mode, cudaStream_t s);
int launch_add_rms_norm(const void* lhs, const void* rhs, const void* w, void* residual, void* normalized,
                        int64_t rows, int64_t hidden, float eps, int dtype, int mode, cudaStream_t s);
// elementwise.cu
int launch_add(const void* a, const void* b, void* out, int64_t n, int dtype, cudaStream_t s);
int launch_swiglu(const void* g, const void* u, void* out, int64_t n, int dtype, int mode, cudaStream_t s);
// rope.cu: x is [tokens, heads, head_dim]; position of token t is positions[pos_period ? t % pos_period : t]
int launch_rope(const void* x, const int32_t* positions, void* out, int64_t tokens, int64_t heads,
                int64_t head_dim, int64_t pos_period, float theta, int dtype, int mode, int32_t* status, cudaStream_t s);
int launch_qk_norm_rope(const void* q, const void* k, const void* qw, const void* kw, const int32_t* positions,
                        void* q_out, void* k_out, int64_t tokens, int64_t q_heads, int64_t k_heads,
                        int64_t head_dim, float eps, float theta, int dtype, int32_t* status, cudaStream_t s);
int rope_bulk_timeouts(unsigned int* out);   // blocking read of a device counter
int launch_qk_norm_rope_paged(const void* q, const void* k, const void* v, const void* qw, const void* kw,
                              const int32_t* positions, void* q_out, void* storage, const int32_t* block_tables,
                              const int32_t* slot_positions, int64_t tokens, int64_t q_heads, int64_t k_heads,
                              int64_t head_dim, float eps, float theta, int64_t tokens_per_table, int64_t max_blocks,
                              int64_t layer, int64_t total_blocks, int64_t block_size, int dtype, int32_t* status,
                              cudaStream_t s);
// gather.cu
int launch_gather(const void* table, const int32_t* ids, void* out, int64_t count, int64_t hidden,
                  int64_t vocab, int dtype, int32_t* status, cudaStream_t s);
// vocab.cu
size_t argmax_workspace_bytes(int64_t rows);
int launch_argmax(const void* logits, int64_t rows, int64_t width, int64_t row_stride, int dtype,
                  int64_t index_base, int32_t* out_ids, int64_t* out_keys, void* workspace, cudaStream_t s);
int launch_argmax_decode(const int64_t* keys, int64_t rows, int32_t* out_ids, cudaStream_t s);
size_t softmax_workspace_bytes(int64_t rows);
int launch_softmax(const void* x, void* out, int64_t rows, int64_t width, int dtype, int mode, void* workspace,
                   cudaStream_t s);
int launch_softmax_stats(const void* x, int64_t rows, int64_t width, int dtype, float* row_max, float* row_sum,
                         cudaStream_t s);
int launch_softmax_rebase(const float* row_max, const float* global_max, float* row_sum, int64_t rows,
                          cudaStream_t s);
int launch_softmax_apply(const void* x, void* out, int64_t rows, int64_t width, int dtype, const float* row_max,
                         const float* row_sum, cudaStream_t s);

// lmhead.cu: logits = hidden x table^T for a few rows, fused with the row arg-max (one pass over the table)
int launch_lm_head_argmax(const void* hidden, const void* table, int64_t rows, int64_t hidden_size, int64_t vocab,
                          int dtype, int mode, int64_t index_base, void* logits_out, int64_t logits_stride,
                          int32_t* out_ids, int64_t* out_keys, void* workspace, cudaStream_t s);

// lmhead_mma.cu: the same product on the tensor cores (tcgen05), fp16, up to 64 hidden rows per pass over the table
bool lm_head_mma_supported(const void* hidden, const void* table, int64_t hidden_size, int64_t vocab);
int launch_lm_head_mma(const void* hidden, const void* table, int64_t rows, int64_t hidden_size, int64_t vocab,
                       int64_t index_base, void* logits_out, int64_t logits_stride, int32_t* out_ids, int64_t* out_keys,
                       unsigned long long* keys, unsigned int* ticket, cudaStream_t s);

// kvmove.cu: mode 0 = decode batch (one block table and one position per token), 1 = packed prefill (token t at
// slot t of one block table), 2 = single decode (*positions is the cache length after the append)
int launch_paged_kv_write(int mode, const void* key, const void* value, void* storage, const int32_t* block_tables,
                          const int32_t* positions, int64_t tokens, int64_t max_blocks, int64_t layer, int64_t total_blocks,
                          int64_t block_size, int64_t row_bytes, int32_t* status, cudaStream_t s);
int launch_select_last_valid(const void* padded, const int32_t* valid_lengths, void* out, int64_t batch, int64_t seq,
                             int64_t row_bytes, int32_t* status, cudaStream_t s);
// sampler.cu
size_t sampler_workspace_bytes(int64_t rows, int64_t width);
int launch_sample_rows(const void* logits, int64_t rows, int64_t width, int64_t row_stride, int dtype, float temperature,
                       int top_k, float top_p, unsigned long long seed, const unsigned long long* draw_offsets,
                       int32_t* out_ids, void* workspace, cudaStream_t s);
int launch_ordered_sums(const float* terms, int64_t rows, int64_t n, float* sums, cudaStream_t s);
// sampler_fallback.cu: lists the rows whose flag is up and, from the device and only if there are any, launches the
// whole-row route over them
int launch_sampler_rows_fallback(const int* row_flags, int64_t rows, int* list, int* count, const void* logits, int dtype,
                                 int64_t width, int64_t row_stride, int64_t padded, float temperature, int top_k, float top_p,
                                 unsigned long long seed, const unsigned long long* draw_offsets, unsigned long long* keys,
                                 float* running, int32_t* out_ids, cudaStream_t s);
// vocab.cu, vocabulary-sharded forms with the inter-GPU exchange fused into the kernel (exchange.cuh)
struct ExchangeArgs;
int launch_argmax_exchange(const void* logits, int64_t rows, int64_t width, int64_t row_stride, int dtype,
                           int64_t index_base, int32_t* out_ids, void* workspace, const ExchangeArgs& xa, cudaStream_t s);
int launch_argmax_keys_exchange(const int64_t* keys, int64_t rows, int32_t* out_ids, const ExchangeArgs& xa, cudaStream_t s);
int launch_softmax_stats_exchange(const void* x, int64_t rows, int64_t width, int dtype, float* global_max,
                                  float* global_sum, const ExchangeArgs& xa, cudaStream_t s);

}  // namespace b2
