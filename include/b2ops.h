/*
 * b2ops — C ABI of the B200 (sm_100a) tensor-op library.
 *
 * Drop-in boundary for the memory-bound operators of cuda-llm's op library.  The
 * reference has no FFI of its own: its operator API is the C++ header
 * include/llm/ops_cuda.h.  Each entry point below is the raw-pointer form of one
 * kernel family behind that header and names the reference interface it replaces
 * (paths are relative to the reference tree).  The C++ functions with the
 * reference's own signatures (include/llm/ops_cuda.h in this repository) validate
 * their llm::Tensor arguments and forward here.
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer unless a parameter says "host".
 *   - Tensors are dense and row-major.  dtype: B2_F32 or B2_F16 storage; all
 *     arithmetic is fp32 (fp64 where the deterministic mode needs it).
 *   - Entry points never allocate, never synchronise and never copy to the host;
 *     scratch memory is passed in by the caller, so those calls may be recorded
 *     into a CUDA graph.  (b2_alloc/b2_free are the exceptions and say so.)
 *   - `stream` is a cudaStream_t.  NULL means the calling thread's default stream
 *     (the library is built with per-thread default streams, like the reference:
 *     its CMakeLists.txt:9).
 *   - Return value: B2_OK, or a negative b2_status.  b2_last_error() gives the
 *     message of the calling thread's most recent failure.  Nothing throws.
 *   - Outputs may alias inputs element-for-element (in-place use), as the
 *     reference's callers do (src/qwen3_layer_cuda.cu:323, :703-704).
 *   - mode: B2_FAST uses parallel fp32 partial sums.  B2_DETERMINISTIC reproduces
 *     the summation order of the reference's kernels (fp64 running sum in index
 *     order for the RMSNorm family, fp32 running sum in index order for softmax,
 *     all-fp32 angles for RoPE) so that bit-level regressions can still be run.
 */
#ifndef B2OPS_H_
#define B2OPS_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define B2_API
#else
#define B2_API __attribute__((visibility("default")))
#endif

typedef enum { B2_F32 = 0, B2_F16 = 1 } b2_dtype;
typedef enum { B2_FAST = 0, B2_DETERMINISTIC = 1 } b2_mode;
typedef enum {
  B2_OK = 0,
  B2_ERR_INVALID = -1,     /* bad argument: null pointer, size, dtype, eps, theta */
  B2_ERR_CUDA = -2,        /* the CUDA runtime refused the launch or the call */
  B2_ERR_UNSUPPORTED = -3, /* valid request that this build has no kernel for */
  B2_ERR_TOO_LARGE = -4    /* beyond a documented fixed capacity */
} b2_status;

typedef void* b2_stream; /* cudaStream_t */

B2_API int b2_version(void);
B2_API const char* b2_last_error(void);
B2_API const char* b2_status_string(int status);

/* ---- RMSNorm family ------------------------------------------------------ */

/* out[r,:] = (x[r,:] * inv_r) * weight, inv_r = 1/sqrt(mean(x[r,:]^2) + eps).
 * Covers the hidden-state norm and the per-head QK-norm (rows = tokens*heads,
 * hidden = head_dim).  eps must be > 0.
 * Replaces cuda_rms_norm / cuda_rms_norm_out and kernel rmsk<T>
 * (include/llm/ops_cuda.h:77,113-114; src/ops_cuda.cu:112-131,672-673). */
B2_API int b2_rms_norm(const void* x, const void* weight, void* out, int64_t rows, int64_t hidden,
                       float eps, int dtype, int mode, b2_stream stream);

/* v = lhs + rhs; residual = round(v); normalized = RMSNorm(v) * weight.
 * B2_FAST normalises the unrounded fp32 sum kept in registers; B2_DETERMINISTIC
 * re-reads the rounded residual exactly as the reference kernel does.
 * Replaces cuda_add_rms_norm_out and kernel add_rms_normk<T>
 * (include/llm/ops_cuda.h:117-120; src/ops_cuda.cu:77-99,675-703). */
B2_API int b2_add_rms_norm(const void* lhs, const void* rhs, const void* weight, void* residual,
                           void* normalized, int64_t rows, int64_t hidden, float eps, int dtype,
                           int mode, b2_stream stream);

/* ---- streaming elementwise ----------------------------------------------- */

/* out = a + b.  Replaces cuda_add / cuda_add_out and kernel addk<T>
 * (include/llm/ops_cuda.h:78,115-116; src/ops_cuda.cu:76,674,704). */
B2_API int b2_add(const void* a, const void* b, void* out, int64_t count, int dtype, b2_stream stream);

/* out = (gate / (1 + exp(-gate))) * up.  mode B2_DETERMINISTIC uses the
 * full-accuracy expf and IEEE division for both dtypes (the reference's formula);
 * B2_FAST uses the hardware exponential for fp16 storage only, which stays inside
 * half an fp16 ulp.  Replaces cuda_swiglu / cuda_swiglu_out and kernel siluk<T>
 * (include/llm/ops_cuda.h:79,121-122; src/ops_cuda.cu:100,705-706). */
B2_API int b2_swiglu(const void* gate, const void* up, void* out, int64_t count, int dtype, int mode,
                     b2_stream stream);

/* ---- launch pacing ------------------------------------------------------------ */

/* Programmatic dependent launch for the calling thread's later calls (off by default).  When on, the short
 * operators of a decode step (RMSNorm family, add, SwiGLU, RoPE family, paged-KV writes, gather) are launched
 * with the "programmatic stream serialization" attribute: each may be scheduled while the kernel before it on
 * the stream is still running and waits, on the device, for that kernel's completion before it touches memory.
 * Results are unchanged; what shrinks is the idle gap between two launches, which at one to a few dozen token
 * rows is as long as the kernels themselves.  The same launches are valid inside stream capture.  No reference
 * counterpart (the reference launches every kernel fully serialised). */
B2_API void b2_set_programmatic_launch(int enabled);
B2_API int b2_get_programmatic_launch(void);

/* ---- rotary embedding (NeoX rotate-half) ----------------------------------- */

/* x, out: [tokens, heads, head_dim]; positions: int32[tokens], one per token row.
 * Pairs (i, i + head_dim/2) are rotated by angle positions[t] * theta^(-2i/head_dim).
 * head_dim must be even, theta > 0.
 * status (here and in the two entry points below): NULL, or a device (or mapped host) int32 into which
 * bit 0 is OR-ed if one of the kernel's bounded waits on an on-chip bulk copy ran out -- never expected;
 * the call still returns normally, but some tokens of its output were not written.
 * Replaces cuda_rope (after its host->device copy of the positions),
 * cuda_rope_batched_positions_out and cuda_rope_token_positions_out, kernels ropek<T>
 * and rope_decode_batched_kernel<T> (include/llm/ops_cuda.h:80,126-131;
 * src/ops_cuda.cu:133,135,707,972-990,1083-1102). */
B2_API int b2_rope(const void* x, const int32_t* positions, void* out, int64_t tokens, int64_t heads,
                   int64_t head_dim, float theta, int dtype, int mode, int32_t* status, b2_stream stream);

/* x, out: [batch, seq, heads, head_dim]; positions: int32[seq], shared by every
 * batch entry.  Replaces cuda_rope_batched / cuda_rope_batched_out and kernel
 * rope_batched_kernel<T> (include/llm/ops_cuda.h:81,123-125; src/ops_cuda.cu:134,708-709). */
B2_API int b2_rope_batched(const void* x, const int32_t* positions, void* out, int64_t batch,
                           int64_t seq, int64_t heads, int64_t head_dim, float theta, int dtype,
                           int mode, int32_t* status, b2_stream stream);

/* Fused per-head RMSNorm + RoPE for the query and key projections of one layer:
 * q [tokens, q_heads, head_dim] with q_weight[head_dim], k [tokens, k_heads,
 * head_dim] with k_weight[head_dim], positions int32[tokens].  k (with k_weight,
 * k_out) may be NULL when k_heads == 0.  One pass over HBM instead of the four
 * the reference makes (cuda_rms_norm_out x2 then cuda_rope_token_positions_out x2,
 * src/qwen3_layer_cuda.cu:289-292,867-872); the normalised value stays in fp32
 * registers between the two steps.  Fast mode only. */
B2_API int b2_qk_norm_rope(const void* q, const void* k, const void* q_weight, const void* k_weight,
                           const int32_t* positions, void* q_out, void* k_out, int64_t tokens,
                           int64_t q_heads, int64_t k_heads, int64_t head_dim, float eps, float theta,
                           int dtype, int32_t* status, b2_stream stream);

/* Health check for the kernels that stage rows through on-chip bulk copies: every wait on such a
 * copy is bounded, and *count (host memory) receives how many waits have run out on the current
 * device since the library was loaded.  0 in a healthy run; anything else means outputs of some
 * earlier b2_rope / b2_qk_norm_rope call are invalid (the status argument of those calls says which).  Blocking (it copies a device counter to
 * the host).  No reference counterpart. */
B2_API int b2_bulk_copy_timeouts(uint32_t* count);

/* ---- embedding-row gather --------------------------------------------------- */

/* out[t,:] = table[ids[t],:], bit-exact.  An id outside [0, vocab) never reaches
 * memory: its row is written as zeros and, when `status` is not NULL, bit 0 of
 * *status is set (the caller zeroes *status beforehand).
 * Replaces cuda_embedding_lookup, cuda_embedding_lookup_out (after its host-side
 * bounds check and host->device copy of the ids), cuda_embedding_lookup_device_ids_out
 * and kernel embeddingk<T> (include/llm/ops_cuda.h:148-156; src/ops_cuda.cu:564,872-884). */
B2_API int b2_embedding_gather(const void* table, const int32_t* ids, void* out, int64_t count,
                               int64_t hidden, int64_t vocab, int dtype, int32_t* status,
                               b2_stream stream);

/* ---- vocabulary-wide reductions -------------------------------------------- */

/* Row argmax with the reference's rule: largest value, ties to the lowest index;
 * NaN, -inf and -FLT_MAX never win; a row with no winner gives 0.
 * logits: rows x width, consecutive rows `row_stride` elements apart.
 * workspace: b2_argmax_workspace_bytes(rows) bytes, zero-filled once before its
 * first use (b2_argmax_workspace_init); every call leaves it zero-filled again, so
 * it can be reused by later calls on the same stream.  Calls that share a
 * workspace must not overlap on the device.
 * Replaces cuda_argmax_last_row, argmax_row_impl and the temperature == 0 route of
 * CudaSampler, kernels argmax_partial<T> + argmax_final
 * (include/llm/ops_cuda.h:154; src/ops_cuda.cu:562-563,711,871,903-909). */
B2_API size_t b2_argmax_workspace_bytes(int64_t rows);
B2_API int b2_argmax_workspace_init(void* workspace, int64_t rows, b2_stream stream);
B2_API int b2_argmax_rows(const void* logits, int64_t rows, int64_t width, int64_t row_stride, int dtype,
                          int32_t* out_ids, void* workspace, b2_stream stream);

/* Row argmax for callers that cannot allocate device memory and have no scratch buffer to
 * hand over: same inputs, outputs and result as b2_argmax_rows, but the scratch lives in a
 * fixed array inside the library image instead of a caller workspace.  Meant for a host
 * that gave all device memory to its own pool at start-up and treats any later cudaMalloc
 * as an error (it may fail, and it stalls the device), or a plug-in that is handed tensors
 * by its host application but no allocator.  This entry point has no counterpart in the
 * reference, whose argmax allocates and frees two buffers on every call
 * (src/ops_cuda.cu:711).
 *   - rows must be <= B2_ARGMAX_STATIC_MAX_ROWS; more returns B2_ERR_TOO_LARGE.
 *   - The array (B2_ARGMAX_STATIC_MAX_ROWS * 12 bytes) is held on every GPU that loads the
 *     library, until the process exits.
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress); make that first call outside any stream capture.  No call
 *     uses cudaMalloc, cudaFree or any allocating routine.  The address is remembered per
 *     device for the life of the process: do not use this entry point across a
 *     cudaDeviceReset (or any other teardown of the device's primary context).
 *   - All calls on a device share the one array: the part a call uses is cleared on its
 *     stream first, and two calls whose kernels overlap on the GPU (different streams
 *     without ordering) race on it.  Order them, or use b2_argmax_rows with one workspace each. */
#define B2_ARGMAX_STATIC_MAX_ROWS 4096
B2_API int b2_argmax_rows_static(const void* logits, int64_t rows, int64_t width, int64_t row_stride,
                                 int dtype, int32_t* out_ids, b2_stream stream);

/* Vocabulary-sharded form: this GPU holds columns [index_base, index_base + width)
 * of every row.  keys[r] = packed (value, index_base + local index) such that the
 * signed 64-bit MAX over all shards' keys is the key of the global winner (one
 * ncclAllReduce(ncclInt64, ncclMax) of `rows` elements).  b2_argmax_decode_keys
 * turns reduced keys into int32 indices.  No reference counterpart: the reference
 * is single-GPU. */
B2_API int b2_argmax_keys(const void* logits, int64_t rows, int64_t width, int64_t row_stride, int dtype,
                          int64_t index_base, int64_t* keys, void* workspace, b2_stream stream);
B2_API int b2_argmax_decode_keys(const int64_t* keys, int64_t rows, int32_t* out_ids, b2_stream stream);

/* LM head fused with the greedy pick: logits[r, j] = sum_k hidden[r, k] * table[j, k] and, per row, the
 * arg-max over j, in one pass over the table; the pick never reads the logits back from memory.
 * Any row count is accepted.  One or two rows (and every fp32 call) are a matrix-vector product, bound by
 * reading the table once: they run on the CUDA cores like the other streaming operators (fp32: every 4 rows,
 * 2 above hidden size 4096, cost one more pass over the table).  Three or more fp16 rows in B2_FAST go to the
 * tensor cores (tcgen05.mma, accumulators in tensor memory, the arg-max in the epilogue): up to 64 rows per
 * pass over the table, still at the table's read rate.
 * hidden: rows x hidden_size; table: vocab x hidden_size (the tied embedding); same dtype.
 * logits_out: NULL, or rows x vocab of that dtype, consecutive rows `logits_stride` elements apart.
 * out_ids: NULL or int32[rows]; out_keys: NULL or int64[rows] packed as by b2_argmax_keys with
 * index_base added to every index (a vocabulary-sharded table: reduce the keys with a signed MAX,
 * then b2_argmax_decode_keys).  At least one of the three outputs must be given.
 * The logit is rounded to the storage type before it is compared, and the pick follows
 * b2_argmax_rows' rule.  B2_DETERMINISTIC adds the products in ascending k with separately
 * rounded multiplies (the reference's CPU `linear`, and for fp16 its linear_f16_reference kernel);
 * B2_FAST splits k over a warp in a fixed order, or leaves the order to the tensor cores (fp32
 * accumulation; run-to-run identical).  B2_FAST needs 16-byte aligned pointers and a hidden size that is a
 * multiple of 1024 (fp16 on the CUDA cores), 512 (fp32) or 64 (fp16 on the tensor cores) elements; other
 * shapes (hidden_size up to 8192) take the ordered kernel in both modes.
 * Should a bounded wait inside the tensor-core kernel ever run out (a copy that never lands), every id of the
 * call reads -1 (keys: INT64_MIN) instead of a result.
 * workspace: as for b2_argmax_rows (b2_argmax_workspace_bytes(rows), zero-filled once).
 * Replaces cuda_lm_head / cuda_linear_out followed by cuda_argmax_last_row
 * (include/llm/ops_cuda.h:154,157; src/ops_cuda.cu:637-671,885,101-111; src/qwen3_cuda_model.cpp:1070-1071,
 * 1339); CPU twin lm_head = linear (include/llm/ops.h:12; src/ops_cpu.cpp:9,17). */
B2_API int b2_lm_head_argmax(const void* hidden, const void* table, int64_t rows, int64_t hidden_size,
                             int64_t vocab, int dtype, int mode, int64_t index_base, void* logits_out,
                             int64_t logits_stride, int32_t* out_ids, int64_t* out_keys, void* workspace,
                             b2_stream stream);

/* Row softmax over the last dimension: out = exp(x - max) / sum.
 * B2_FAST keeps each row on chip (a thread-block cluster holds it in distributed
 * shared memory) when it fits, otherwise makes two passes; B2_DETERMINISTIC adds the
 * exponentials in index order in fp32, like ops_cpu and the reference kernel.
 * workspace: b2_softmax_workspace_bytes(rows) bytes.  Its last 16 bytes begin with an int32
 * status word that the kernel only ever ORs into: bit 0 = a bounded wait for an on-chip bulk
 * copy ran out and the outputs of that call are invalid.  Zero it once; the rest is scratch.
 * Replaces cuda_softmax_last_dim and kernel softk<T>
 * (include/llm/ops_cuda.h:82; src/ops_cuda.cu:132,710). */
B2_API size_t b2_softmax_workspace_bytes(int64_t rows);
B2_API int b2_softmax_rows(const void* x, void* out, int64_t rows, int64_t width, int dtype, int mode,
                           void* workspace, b2_stream stream);

/* Vocabulary-sharded softmax, three steps around two small all-reduces:
 *   b2_softmax_stats     row_max[r] = max of the local columns,
 *                        row_sum[r] = sum exp(x - row_max[r]) over the local columns
 *   (all-reduce MAX of a copy of row_max -> global_max)
 *   b2_softmax_rebase    row_sum[r] *= exp(row_max[r] - global_max[r])
 *   (all-reduce SUM of row_sum -> global_sum)
 *   b2_softmax_apply     out = exp(x - global_max[r]) / global_sum[r]
 * No reference counterpart: the reference is single-GPU. */
B2_API int b2_softmax_stats(const void* x, int64_t rows, int64_t width, int dtype, float* row_max,
                            float* row_sum, b2_stream stream);
B2_API int b2_softmax_rebase(const float* row_max, const float* global_max, float* row_sum, int64_t rows,
                             b2_stream stream);
B2_API int b2_softmax_apply(const void* x, void* out, int64_t rows, int64_t width, int dtype,
                            const float* row_max, const float* row_sum, b2_stream stream);

/* ---- row moves around the paged KV cache and the padded-prefill logits ------------- */

/* The KV pool is the reference's PagedKvCachePool storage: [layers, total_blocks, 2, block_size,
 * kv_heads, head_dim], plane 0 = keys, plane 1 = values (include/llm/paged_kv_cache_pool.h).
 * key, value: [tokens, kv_heads, head_dim]; every token's key row and value row are copied, bit for
 * bit, to the slot its position selects through a block table:
 *   b2_paged_kv_write_decode_batch  token b -> position positions[b] of block_tables[b, 0..max_blocks)
 *   b2_paged_kv_write_decode        the one token -> position *cache_length - 1 of block_table
 *                                   (nothing is written when *cache_length == 0)
 *   b2_paged_kv_prefill_copy        token t -> position t of block_table
 * A block id outside [0, total_blocks), a negative position or one past the table never reaches
 * memory: that row is skipped and bit 0 of *status (device int32, may be NULL) is raised.
 * Replace cuda_paged_kv_write_decode_batch / cuda_paged_kv_write_decode (include/llm/ops_cuda.h:178-186;
 * src/paged_attention_cuda.cu:219-262,639-716) and cuda_paged_kv_prefill_copy_packed
 * (src/ops_cuda.cu:1104-1160), after their checks of the pool object. */
B2_API int b2_paged_kv_write_decode_batch(const void* key, const void* value, void* storage,
                                          const int32_t* block_tables, const int32_t* positions, int64_t batch,
                                          int64_t max_blocks, int64_t layer, int64_t layers, int64_t total_blocks,
                                          int64_t block_size, int64_t kv_heads, int64_t head_dim, int dtype,
                                          int32_t* status, b2_stream stream);
B2_API int b2_paged_kv_write_decode(const void* key, const void* value, void* storage, const int32_t* block_table,
                                    const int32_t* cache_length, int64_t max_blocks, int64_t layer, int64_t layers,
                                    int64_t total_blocks, int64_t block_size, int64_t kv_heads, int64_t head_dim,
                                    int dtype, int32_t* status, b2_stream stream);
B2_API int b2_paged_kv_prefill_copy(const void* key, const void* value, void* storage, const int32_t* block_table,
                                    int64_t tokens, int64_t max_blocks, int64_t layer, int64_t layers,
                                    int64_t total_blocks, int64_t block_size, int64_t kv_heads, int64_t head_dim,
                                    int dtype, int32_t* status, b2_stream stream);

/* The attention prologue of a layer in ONE launch: per-head RMSNorm + RoPE of q and k as b2_qk_norm_rope,
 * with the rotated keys written straight into their slots of the paged KV pool and the value rows copied
 * beside them (plane 1) -- instead of cuda_rms_norm x2, cuda_rope_* x2 and cuda_paged_kv_write_decode_batch
 * (src/qwen3_layer_cuda.cu:390-403) or cuda_paged_kv_prefill_copy_packed (:860-880).  The keys never make
 * the round trip through a [tokens, kv_heads, head_dim] buffer.
 *   q [tokens, q_heads, head_dim], k and v [tokens, kv_heads, head_dim], positions int32[tokens] (rotary);
 *   token t uses row t / tokens_per_table of block_tables [.., max_blocks] and cache position
 *   slot_positions[t], or t % tokens_per_table when slot_positions is NULL
 *   (decode batch: tokens_per_table = 1, slot_positions = positions; one packed sequence: tokens_per_table =
 *   tokens, slot_positions = NULL).
 * Results are bit-identical to b2_qk_norm_rope followed by b2_paged_kv_write_*.  Bad block ids or positions:
 * that token's K/V are skipped and bit 0 of *status is raised; bit 1 says that a bounded wait on a bulk copy ran
 * out (never expected) and some tokens were not written.  Returns B2_ERR_UNSUPPORTED for head sizes or
 * alignments that only the scalar kernels take (use the separate calls then).  Fast mode only. */
B2_API int b2_qk_norm_rope_paged(const void* q, const void* k, const void* v, const void* q_weight,
                                 const void* k_weight, const int32_t* positions, void* q_out, void* storage,
                                 const int32_t* block_tables, const int32_t* slot_positions, int64_t tokens,
                                 int64_t q_heads, int64_t kv_heads, int64_t head_dim, float eps, float theta,
                                 int64_t tokens_per_table, int64_t max_blocks, int64_t layer, int64_t layers,
                                 int64_t total_blocks, int64_t block_size, int dtype, int32_t* status,
                                 b2_stream stream);

/* out[b, :] = padded[b, valid_lengths[b] - 1, :] for padded [batch, seq, width]: the logits of each
 * prompt's last real token, gathered in one launch.  valid_lengths: device int32[batch]; a length outside
 * [1, seq] zero-fills that row and raises bit 0 of *status (device int32, may be NULL).
 * Replaces the CUDA branch of select_last_valid_logits (src/qwen3_padded_prefill.cpp:118-148: one blocking
 * device-to-device copy per prompt), after its host-side checks. */
B2_API int b2_select_last_valid_rows(const void* padded, const int32_t* valid_lengths, void* out, int64_t batch,
                                     int64_t seq, int64_t width, int dtype, int32_t* status, b2_stream stream);

/* ---- temperature / top-k / top-p sampling ------------------------------------------ */

/* One token per row of logits [rows, width] (rows `row_stride` elements apart), chosen exactly as the
 * reference's CudaSampler chooses it: scores = logits / temperature; tokens ordered by score descending,
 * equal scores by ascending id; the first top_k of them (all when top_k == 0); of those the shortest
 * prefix whose softmax mass reaches top_p (all when top_p == 1); then one draw u(seed, draw_offsets[r]) in
 * (0,1) picks by cumulative mass.  Sums are fp32 and added in that order, so the token is the reference's
 * bit for bit.  temperature == 0 is the row argmax (top_k, top_p and the draw are ignored).
 * temperature must be finite and >= 0; with temperature > 0: 0 <= top_k <= width, 0 < top_p <= 1 and at most
 * B2_SAMPLER_MAX_ROWS rows per call (more: B2_ERR_TOO_LARGE before anything is launched).
 * draw_offsets: device uint64[rows], or NULL for offset 0 on every row.
 * workspace: b2_sampler_workspace_bytes(rows, width) bytes of scratch, no initialisation needed; calls
 * that share it must not overlap on the device.
 * Three routes, all exact: 0 < top_k <= 2048 makes one pass over the logits (a sampled threshold, checked);
 * top_k == 0 with top_p < 1 and 32768 <= width <= 262144 sorts only the row's largest ~2800 tokens and adds
 * the rest of the softmax sum from per-bucket integer increments (rows with a flat distribution, whose top-p
 * prefix does not end among those tokens, are redone by the third route); everything else sorts the whole row.
 * Replaces CudaSampler::sample_row / sample_last_row / sample_last_token_of_batch, kernels sampler_fill and
 * sampler_select and the library sort between them (include/llm/ops_cuda.h:46-74;
 * src/ops_cuda.cu:575-617,886-971), which handle one row per blocking call. */
#define B2_SAMPLER_MAX_ROWS 65535
B2_API size_t b2_sampler_workspace_bytes(int64_t rows, int64_t width);
B2_API int b2_sample_rows(const void* logits, int64_t rows, int64_t width, int64_t row_stride, int dtype,
                          float temperature, int32_t top_k, float top_p, uint64_t seed, const uint64_t* draw_offsets,
                          int32_t* out_ids, void* workspace, b2_stream stream);

/* sums[r, i] = fl(... fl(fl(terms[r, 0] + terms[r, 1]) + terms[r, 2]) ... + terms[r, i]): the fp32 running sums of
 * each row's terms added one after the other in index order -- what the single thread of the reference's
 * sampler_select computes (src/ops_cuda.cu:587-603), bit for bit -- by a whole thread block: inside one power
 * of two of the sum the additions are a prefix sum of integer increments, corrected at the ties.
 * terms: device fp32 [rows, n], non-negative, each row in descending order (the order the sampler meets them);
 * n <= B2_ORDERED_SUMS_MAX.  sums may alias terms. */
#define B2_ORDERED_SUMS_MAX 4096
B2_API int b2_ordered_sums(const float* terms, int64_t rows, int64_t n, float* sums, b2_stream stream);

/* ---- vocabulary-sharded reductions with the exchange fused into the kernel ------ */

/* One process per GPU, all GPUs on one NVLink node.  Instead of reduce kernel -> collective
 * library -> finishing kernel, the reduction kernel does the exchange itself: the thread
 * block that finishes a row stores that row's 8-byte partial result straight into every
 * peer's exchange buffer (peer-mapped device memory) while the other rows are still being
 * reduced -- as two 64-bit words that each carry the call's epoch, so a word that shows the
 * epoch is valid data and no fence or separate flag crosses NVLink -- and the thread block
 * that finishes the last row waits -- bounded -- for the peers' words in its own buffer and
 * writes the final row results.  One launch per GPU and no host round trip.  No reference
 * counterpart: the reference is single-GPU.
 *
 * Set-up, once per group of GPUs:
 *   1. every process: buffer = b2_alloc(b2_p2p_exchange_bytes(world, max_rows));
 *      b2_p2p_exchange_init(buffer, world, max_rows, stream)
 *   2. b2_ipc_export(buffer, handle): 64 bytes to hand to the other processes by any host
 *      channel (the Python side uses torch.distributed.all_gather_object)
 *   3. b2_ipc_open(peer_handle, &peer_pointer) for every other rank; fill b2_p2p_exchange with
 *      buffers[r] = rank r's buffer as addressable from THIS process (own pointer at [rank])
 *   4. a host barrier, so that every buffer is initialised before the first call.
 * Every rank must then make the same sequence of fused calls (they are collectives); calls
 * on one buffer must not overlap on a GPU.  timeout_ms bounds the wait for the peers (0 means
 * 2000): when it runs out the kernel still ends normally, ORs 2 into *status, and the rows
 * whose partials were incomplete are marked in the output itself (index -1; NaN statistics);
 * every rank then re-initialises its buffer before further use.
 * trace: NULL, or device uint64[4 + world] that receives the nanosecond timer of this GPU at the
 * kernel's start, at the start of the wait, when all partials were present and at the end, then
 * when each GPU's first row was seen (a measuring aid; costs nothing when NULL).
 * Tear-down: b2_ipc_close(peer_pointer) for each opened handle, then b2_free(buffer). */
#define B2_P2P_MAX_WORLD 16
typedef struct {
  void* buffers[B2_P2P_MAX_WORLD];
  int32_t world, rank;
  int64_t max_rows;
  uint32_t timeout_ms;
  uint64_t* trace;
} b2_p2p_exchange;
B2_API size_t b2_p2p_exchange_bytes(int world, int64_t max_rows);
B2_API int b2_p2p_exchange_init(void* buffer, int world, int64_t max_rows, b2_stream stream);
B2_API int b2_ipc_export(const void* device_ptr, unsigned char handle[64]);
B2_API int b2_ipc_open(const unsigned char handle[64], void** device_ptr);
B2_API int b2_ipc_close(void* device_ptr);

/* Global row argmax of logits whose columns [index_base, index_base + width) live on this
 * GPU: out_ids[r] on EVERY rank = index of the largest value of row r over all ranks' columns,
 * ties to the lowest index (the rule of b2_argmax_rows).  workspace as for b2_argmax_rows;
 * status: device int32 or NULL.  Replaces b2_argmax_keys + ncclAllReduce + b2_argmax_decode_keys. */
B2_API int b2_argmax_rows_sharded(const void* logits, int64_t rows, int64_t width, int64_t row_stride, int dtype,
                                  int64_t index_base, int32_t* out_ids, void* workspace,
                                  const b2_p2p_exchange* exchange, int32_t* status, b2_stream stream);

/* The exchange of b2_argmax_rows_sharded alone, for keys another kernel produced (b2_argmax_keys, or
 * b2_lm_head_argmax over this GPU's rows of a vocabulary-split embedding): this GPU's `rows` packed keys go to
 * every peer, and out_ids[r] receives the index of the largest key of all GPUs for row r.  One small launch in
 * place of ncclAllReduce(MAX) + b2_argmax_decode_keys; same buffers, same calling rules (a collective: every GPU
 * makes the same sequence of calls on the exchange) and the same bounded wait as b2_argmax_rows_sharded.
 * No reference counterpart: the reference is single-GPU. */
B2_API int b2_argmax_keys_exchange(const int64_t* keys, int64_t rows, int32_t* out_ids,
                                   const b2_p2p_exchange* exchange, int32_t* status, b2_stream stream);

/* Row statistics of the WHOLE row from this GPU's columns: global_max[r] = max over all ranks,
 * global_sum[r] = sum over all ranks of exp(x - global_max[r]); follow with
 * b2_softmax_apply(x, out, rows, width, dtype, global_max, global_sum).
 * Replaces b2_softmax_stats + two all-reduces + b2_softmax_rebase. */
B2_API int b2_softmax_stats_sharded(const void* x, int64_t rows, int64_t width, int dtype, float* global_max,
                                    float* global_sum, const b2_p2p_exchange* exchange, int32_t* status,
                                    b2_stream stream);

/* ---- device memory with the reference's allocation counters ----------------- */

/* cudaMalloc / cudaFree plus the counters of the reference's CudaAllocationStats
 * (include/llm/tensor.h:9-19; src/tensor_cuda.cu:12-54).  These two DO allocate and
 * b2_free synchronises like cudaFree. */
typedef struct {
  uint64_t malloc_calls, free_calls, allocated_bytes_total, freed_bytes_total, live_bytes, peak_live_bytes;
} b2_alloc_stats;
B2_API void* b2_alloc(size_t bytes);
B2_API int b2_free(void* ptr);
B2_API void b2_get_alloc_stats(b2_alloc_stats* out);
B2_API void b2_reset_alloc_stats(void);

#ifdef __cplusplus
}
#endif
#endif /* B2OPS_H_ */
