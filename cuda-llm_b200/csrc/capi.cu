// The C ABI (include/b2ops.h): argument validation, error reporting and dispatch to
// the kernel launchers.  Nothing here allocates, synchronises or copies to the host,
// except b2_alloc / b2_free.
#include "b2ops.h"
#include "common.cuh"
#include "exchange.cuh"
#include "kernels.h"

#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <unordered_map>

namespace b2 {

namespace {
thread_local char g_error[512] = "";
thread_local bool g_programmatic_launch = false;
}

bool programmatic_launch_enabled() { return g_programmatic_launch; }

void set_error(const char* fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, args);
  va_end(args);
}

int launch_status(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return B2_OK;
  set_error("%s: CUDA error: %s", what, cudaGetErrorString(e));
  return B2_ERR_CUDA;
}

int sm_count() {
  static thread_local int cached_device = -1, cached = kSmCount;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) { cudaGetLastError(); return kSmCount; }
  if (device != cached_device) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) == cudaSuccess && n > 0) cached = n;
    else { cudaGetLastError(); cached = kSmCount; }
    cached_device = device;
  }
  return cached;
}

namespace {

int invalid(const char* op, const char* why) {
  set_error("%s: %s", op, why);
  return B2_ERR_INVALID;
}
bool dtype_ok(int dtype) { return dtype == B2_F32 || dtype == B2_F16; }
bool mode_ok(int mode) { return mode == B2_FAST || mode == B2_DETERMINISTIC; }
cudaStream_t as_stream(b2_stream s) { return static_cast<cudaStream_t>(s); }
// products of validated, non-negative sizes must stay addressable
bool fits(int64_t a, int64_t b) { return a == 0 || b <= (int64_t(1) << 46) / a; }

#define B2_REQUIRE(cond, op, why) do { if (!(cond)) return invalid(op, why); } while (0)

std::mutex g_alloc_mutex;
b2_alloc_stats g_alloc_stats = {0, 0, 0, 0, 0, 0};
std::unordered_map<void*, size_t> g_alloc_sizes;

}  // namespace
}  // namespace b2

using namespace b2;

extern "C" {

int b2_version(void) { return 100; }
const char* b2_last_error(void) { return g_error; }
const char* b2_status_string(int status) {
  switch (status) {
    case B2_OK: return "ok";
    case B2_ERR_INVALID: return "invalid argument";
    case B2_ERR_CUDA: return "CUDA error";
    case B2_ERR_UNSUPPORTED: return "unsupported";
    case B2_ERR_TOO_LARGE: return "beyond a fixed capacity";
    default: return "unknown status";
  }
}

int b2_rms_norm(const void* x, const void* weight, void* out, int64_t rows, int64_t hidden, float eps, int dtype,
                int mode, b2_stream stream) {
  const char* op = "b2_rms_norm";
  B2_REQUIRE(dtype_ok(dtype), op, "dtype must be B2_F32 or B2_F16");
  B2_REQUIRE(mode_ok(mode), op, "mode must be B2_FAST or B2_DETERMINISTIC");
  B2_REQUIRE(rows >= 0 && hidden > 0 && fits(rows, hidden), op, "rows must be >= 0 and hidden > 0");
  B2_REQUIRE(eps > 0.0f, op, "eps must be positive");
  B2_REQUIRE(rows == 0 || (x && weight && out), op, "null pointer");
  return launch_rms_norm(x, weight, out, rows, hidden, eps, dtype, mode, as_stream(stream));
}

int b2_add_rms_norm(const void* lhs, const void* rhs, const void* weight, void* residual, void* normalized,
                    int64_t rows, int64_t hidden, float eps, int dtype, int mode, b2_stream stream) {
  const char* op = "b2_add_rms_norm";
  B2_REQUIRE(dtype_ok(dtype), op, "dtype must be B2_F32 or B2_F16");
  B2_REQUIRE(mode_ok(mode), op, "mode must be B2_FAST or B2_DETERMINISTIC");
  B2_REQUIRE(rows >= 0 && hidden > 0 && fits(rows, hidden), op, "rows must be >= 0 and hidden > 0");
  B2_REQUIRE(eps > 0.0f, op, "eps must be positive");
  B2_REQUIRE(rows == 0 || (lhs && rhs && weight && residual && normalized), op, "null pointer");
  B2_REQUIRE(rows == 0 || residual != normalized, op, "residual and normalized must be distinct buffers");
  return launch_add_rms_norm(lhs, rhs, weight, residual, normalized, rows, hidden, eps, dtype, mode,
                             as_stream(stream));
}

int b2_add(const void* a, const void* b, void* out, int64_t count, int dtype, b2_stream stream) {
  const char* op = "b2_add";
  B2_REQUIRE(dtype_ok(dtype), op, "dtype must be B2_F32 or B2_F16");
  B2_REQUIRE(count >= 0 && count <= (int64_t(1) << 46), op, "count out of range");
  B2_REQUIRE(count == 0 || (a && b && out), op, "null pointer");
  return launch_add(a, b, out, count, dtype, as_stream(stream));
}

int b2_swiglu(const void* gate, const void* up, void* out, int64_t count, int dtype, int mode, b2_stream stream) {
  const char* op = "b2_swiglu";
  B2_REQUIRE(dtype_ok(dtype), op, "dtype must be B2_F32 or B2_F16");
  B2_REQUIRE(mode_ok(mode), op, "mode must be B2_FAST or B2_DETERMINISTIC");
  B2_REQUIRE(count >= 0 && count <= (int64_t(1) << 46), op, "count out of range");
  B2_REQUIRE(count == 0 || (gate && up && out), op, "null pointer");
  return launch_swiglu(gate, up, out, count, dtype, mode, as_stream(stream));
}

int b2_rope(const void* x, const int32_t* positions, void* out, int64_t tokens, int64_t heads, int64_t head_dim,
            float theta, int dtype, int mode, int32_t* status, b2_stream stream) {
  const char* op = "b2_rope";
  B2_REQUIRE(dtype_ok(dtype), op, "dtype must be B2_F32 or B2_F16");
  B2_REQUIRE(mode_ok(mode), op, "mode must be B2_FAST or B2_DETERMINISTIC");
  B2_REQUIRE(tokens >= 0 && heads > 0 && head_dim > 0 && fits(tokens, heads * head_dim) && heads * head_dim < (1 << 30),
             op, "tokens must be >= 0, heads and head_dim > 0");
  B2_REQUIRE(head_dim % 2 == 0, op, "head_dim must be even");
  B2_REQUIRE(theta > 0.0f, op, "theta must be positive");
  B2_REQUIRE(tokens == 0 || (x && positions && out), op, "null pointer");
  return launch_rope(x, positions, out, tokens, heads, head_dim, 0, theta, dtype, mode, status, as_stream(stream));
}

int b2_rope_batched(const void* x, const int32_t* positions, void* out, int64_t batch, int64_t seq, int64_t heads,
                    int64_t head_dim, float theta, int dtype, int mode, int32_t* status, b2_stream stream) {
  const char* op = "b2_rope_batched";
  B2_REQUIRE(dtype_ok(dtype), op, "dtype must be B2_F32 or B2_F16");
  B2_REQUIRE(mode_ok(mode), op, "mode must be B2_FAST or B2_DETERMINISTIC");
  B2_REQUIRE(batch >= 0 && seq > 0 && heads > 0 && head_dim > 0 && fits(batch, seq) &&
                 fits(batch * seq, heads * head_dim) && heads * head_dim < (1 << 30),
             op, "batch must be >= 0, seq, heads and head_dim > 0");
  B2_REQUIRE(head_dim % 2 == 0, op, "head_dim must be even");
  B2_REQUIRE(theta > 0.0f, op, "theta must be positive");
  B2_REQUIRE(batch == 0 || (x && positions && out), op, "null pointer");
  return launch_rope(x, positions, out, batch * seq, heads, head_dim, seq, theta, dtype, mode, status, as_stream(stream));
}

int b2_qk_norm_rope(const void* q, const void* k, const void* q_weight, const void* k_weight,
                    const int32_t* positions, void* q_out, void* k_out, int64_t tokens, int64_t q_heads,
                    int64_t k_heads, int64_t head_dim, float eps, float theta, int dtype, int32_t* status,
                    b2_stream stream) {
  const char* op = "b2_qk_norm_rope";
  B2_REQUIRE(dtype_ok(dtype), op, "dtype must be B2_F32 or B2_F16");
  B2_REQUIRE(tokens >= 0 && q_heads > 0 && k_heads >= 0 && head_dim > 0 &&
                 fits(tokens, (q_heads + k_heads) * head_dim) && (q_heads + k_heads) * head_dim < (1 << 30),
             op, "tokens and k_heads must be >= 0, q_heads and head_dim > 0");
  B2_REQUIRE(head_dim % 2 == 0, op, "head_dim must be even");
  B2_REQUIRE(eps > 0.0f, op, "eps must be positive");
  B2_REQUIRE(theta > 0.0f, op, "theta must be positive");
  B2_REQUIRE(tokens == 0 || (q && q_weight && q_out && positions), op, "null pointer");
  B2_REQUIRE(tokens == 0 || k_heads == 0 || (k && k_weight && k_out), op, "null key pointer with k_heads > 0");
  return launch_qk_norm_rope(q, k, q_weight, k_weight, positions, q_out, k_out, tokens, q_heads, k_heads, head_dim,
                             eps, theta, dtype, status, as_stream(stream));
}

int b2_embedding_gather(const void* table, const int32_t* ids, void* out, int64_t count, int64_t hidden,
                        int64_t vocab, int dtype, int32_t* status, b2_stream stream) {
  const char* op = "b2_embedding_gather";
  B2_REQUIRE(dtype_ok(dtype), op, "dtype must be B2_F32 or B2_F16");
  B2_REQUIRE(count >= 0 && hidden > 0 && vocab > 0 && fits(count, hidden) && fits(vocab, hidden), op,
             "count must be >= 0, hidden and vocab > 0");
  B2_REQUIRE(count == 0 || (table && ids && out), op, "null pointer");
  return launch_gather(table, ids, out, count, hidden, vocab, dtype, status, as_stream(stream));
}

void b2_set_programmatic_launch(int enabled) { g_programmatic_launch = enabled != 0; }
int b2_get_programmatic_launch(void) { return g_programmatic_launch ? 1 : 0; }

int b2_bulk_copy_timeouts(uint32_t* count) {
  if (count == nullptr) return invalid("b2_bulk_copy_timeouts", "null pointer");
  unsigned int n = 0;
  const int rc = rope_bulk_timeouts(&n);
  *count = n;
  return rc;
}

size_t b2_argmax_workspace_bytes(int64_t rows) { return rows > 0 ? argmax_workspace_bytes(rows) : 0; }

int b2_argmax_workspace_init(void* workspace, int64_t rows, b2_stream stream) {
  const char* op = "b2_argmax_workspace_init";
  B2_REQUIRE(rows >= 0, op, "rows must be >= 0");
  if (rows == 0) return B2_OK;
  B2_REQUIRE(workspace != nullptr, op, "null pointer");
  if (cudaMemsetAsync(workspace, 0, argmax_workspace_bytes(rows), as_stream(stream)) != cudaSuccess)
    return launch_status(op);
  return B2_OK;
}

static int argmax_checks(const char* op, const void* logits, int64_t rows, int64_t width, int64_t row_stride,
                         int dtype, int64_t index_base, const void* out, const void* workspace) {
  B2_REQUIRE(dtype_ok(dtype), op, "dtype must be B2_F32 or B2_F16");
  B2_REQUIRE(rows >= 0 && width > 0 && row_stride >= width && fits(rows, row_stride) && rows < (1 << 24), op,
             "rows must be >= 0, width > 0 and row_stride >= width");
  B2_REQUIRE(index_base >= 0 && index_base + width <= 0xffffffffll, op, "global indices must fit 32 bits");
  B2_REQUIRE(rows == 0 || (logits && out && workspace), op, "null pointer");
  return B2_OK;
}

int b2_argmax_rows(const void* logits, int64_t rows, int64_t width, int64_t row_stride, int dtype, int32_t* out_ids,
                   void* workspace, b2_stream stream) {
  const int rc = argmax_checks("b2_argmax_rows", logits, rows, width, row_stride, dtype, 0, out_ids, workspace);
  if (rc != B2_OK) return rc;
  B2_REQUIRE(width <= 0x7fffffffll, "b2_argmax_rows", "width must fit int32");
  return launch_argmax(logits, rows, width, row_stride, dtype, 0, out_ids, nullptr, workspace, as_stream(stream));
}

int b2_argmax_keys(const void* logits, int64_t rows, int64_t width, int64_t row_stride, int dtype, int64_t index_base,
                   int64_t* keys, void* workspace, b2_stream stream) {
  const int rc = argmax_checks("b2_argmax_keys", logits, rows, width, row_stride, dtype, index_base, keys, workspace);
  if (rc != B2_OK) return rc;
  B2_REQUIRE(width <= 0x7fffffffll, "b2_argmax_keys", "width must fit int32");
  return launch_argmax(logits, rows, width, row_stride, dtype, index_base, nullptr, keys, workspace, as_stream(stream));
}

int b2_argmax_decode_keys(const int64_t* keys, int64_t rows, int32_t* out_ids, b2_stream stream) {
  const char* op = "b2_argmax_decode_keys";
  B2_REQUIRE(rows >= 0, op, "rows must be >= 0");
  B2_REQUIRE(rows == 0 || (keys && out_ids), op, "null pointer");
  return launch_argmax_decode(keys, rows, out_ids, as_stream(stream));
}

int b2_lm_head_argmax(const void* hidden, const void* table, int64_t rows, int64_t hidden_size, int64_t vocab, int dtype,
                      int mode, int64_t index_base, void* logits_out, int64_t logits_stride, int32_t* out_ids,
                      int64_t* out_keys, void* workspace, b2_stream stream) {
  const char* op = "b2_lm_head_argmax";
  B2_REQUIRE(dtype_ok(dtype), op, "dtype must be B2_F32 or B2_F16");
  B2_REQUIRE(mode_ok(mode), op, "mode must be B2_FAST or B2_DETERMINISTIC");
  B2_REQUIRE(rows >= 0 && rows < (1 << 24), op, "rows must be >= 0");
  B2_REQUIRE(hidden_size > 0 && vocab > 0 && vocab <= 0x7fffffffll && fits(vocab, hidden_size), op,
             "hidden_size and vocab must be > 0 and vocab must fit int32");
  B2_REQUIRE(hidden_size <= 8192, op, "hidden_size must be <= 8192");
  B2_REQUIRE(index_base >= 0 && index_base + vocab <= 0xffffffffll, op, "global indices must fit 32 bits");
  B2_REQUIRE(logits_out == nullptr || (logits_stride >= vocab && fits(rows > 0 ? rows : 1, logits_stride)), op,
             "logits_stride must be >= vocab");
  B2_REQUIRE(logits_out || out_ids || out_keys, op, "no output given");
  B2_REQUIRE(rows == 0 || (hidden && table && workspace), op, "null pointer");
  return launch_lm_head_argmax(hidden, table, rows, hidden_size, vocab, dtype, mode, index_base, logits_out, logits_stride,
                               out_ids, out_keys, workspace, as_stream(stream));
}

size_t b2_softmax_workspace_bytes(int64_t rows) { return rows > 0 ? softmax_workspace_bytes(rows) : 0; }

int b2_softmax_rows(const void* x, void* out, int64_t rows, int64_t width, int dtype, int mode, void* workspace,
                    b2_stream stream) {
  const char* op = "b2_softmax_rows";
  B2_REQUIRE(dtype_ok(dtype), op, "dtype must be B2_F32 or B2_F16");
  B2_REQUIRE(mode_ok(mode), op, "mode must be B2_FAST or B2_DETERMINISTIC");
  B2_REQUIRE(rows >= 0 && width > 0 && fits(rows, width) && rows < (1 << 24), op, "rows must be >= 0 and width > 0");
  B2_REQUIRE(rows == 0 || (x && out && workspace), op, "null pointer");
  return launch_softmax(x, out, rows, width, dtype, mode, workspace, as_stream(stream));
}

int b2_softmax_stats(const void* x, int64_t rows, int64_t width, int dtype, float* row_max, float* row_sum,
                     b2_stream stream) {
  const char* op = "b2_softmax_stats";
  B2_REQUIRE(dtype_ok(dtype), op, "dtype must be B2_F32 or B2_F16");
  B2_REQUIRE(rows >= 0 && width > 0 && fits(rows, width), op, "rows must be >= 0 and width > 0");
  B2_REQUIRE(rows == 0 || (x && row_max && row_sum), op, "null pointer");
  return launch_softmax_stats(x, rows, width, dtype, row_max, row_sum, as_stream(stream));
}

int b2_softmax_rebase(const float* row_max, const float* global_max, float* row_sum, int64_t rows, b2_stream stream) {
  const char* op = "b2_softmax_rebase";
  B2_REQUIRE(rows >= 0, op, "rows must be >= 0");
  B2_REQUIRE(rows == 0 || (row_max && global_max && row_sum), op, "null pointer");
  return launch_softmax_rebase(row_max, global_max, row_sum, rows, as_stream(stream));
}

int b2_softmax_apply(const void* x, void* out, int64_t rows, int64_t width, int dtype, const float* row_max,
                     const float* row_sum, b2_stream stream) {
  const char* op = "b2_softmax_apply";
  B2_REQUIRE(dtype_ok(dtype), op, "dtype must be B2_F32 or B2_F16");
  B2_REQUIRE(rows >= 0 && width > 0 && fits(rows, width), op, "rows must be >= 0 and width > 0");
  B2_REQUIRE(rows == 0 || (x && out && row_max && row_sum), op, "null pointer");
  return launch_softmax_apply(x, out, rows, width, dtype, row_max, row_sum, as_stream(stream));
}

static int pool_checks(const char* op, const void* key, const void* value, const void* storage, const int32_t* table,
                       const int32_t* positions, int64_t tokens, int64_t max_blocks, int64_t layer, int64_t layers,
                       int64_t total_blocks, int64_t block_size, int64_t kv_heads, int64_t head_dim, int dtype) {
  B2_REQUIRE(dtype_ok(dtype), op, "dtype must be B2_F32 or B2_F16");
  B2_REQUIRE(tokens >= 0 && max_blocks > 0 && layers > 0 && total_blocks > 0 && block_size > 0 && kv_heads > 0 && head_dim > 0,
             op, "sizes must be positive");
  B2_REQUIRE(layer >= 0 && layer < layers, op, "layer out of range");
  B2_REQUIRE(fits(kv_heads, head_dim) && fits(tokens, kv_heads * head_dim) && fits(layers * total_blocks * 2, block_size) &&
                 fits(layers * total_blocks * 2 * block_size, kv_heads * head_dim),
             op, "sizes out of range");
  B2_REQUIRE(tokens == 0 || (key && value && storage && table && positions), op, "null pointer");
  return B2_OK;
}

int b2_paged_kv_write_decode_batch(const void* key, const void* value, void* storage, const int32_t* block_tables,
                                   const int32_t* positions, int64_t batch, int64_t max_blocks, int64_t layer, int64_t layers,
                                   int64_t total_blocks, int64_t block_size, int64_t kv_heads, int64_t head_dim, int dtype,
                                   int32_t* status, b2_stream stream) {
  const int rc = pool_checks("b2_paged_kv_write_decode_batch", key, value, storage, block_tables, positions, batch, max_blocks,
                             layer, layers, total_blocks, block_size, kv_heads, head_dim, dtype);
  if (rc != B2_OK) return rc;
  return launch_paged_kv_write(0, key, value, storage, block_tables, positions, batch, max_blocks, layer, total_blocks,
                               block_size, kv_heads * head_dim * (dtype == B2_F32 ? 4 : 2), status, as_stream(stream));
}

int b2_paged_kv_write_decode(const void* key, const void* value, void* storage, const int32_t* block_table,
                             const int32_t* cache_length, int64_t max_blocks, int64_t layer, int64_t layers,
                             int64_t total_blocks, int64_t block_size, int64_t kv_heads, int64_t head_dim, int dtype,
                             int32_t* status, b2_stream stream) {
  const int rc = pool_checks("b2_paged_kv_write_decode", key, value, storage, block_table, cache_length, 1, max_blocks, layer,
                             layers, total_blocks, block_size, kv_heads, head_dim, dtype);
  if (rc != B2_OK) return rc;
  return launch_paged_kv_write(2, key, value, storage, block_table, cache_length, 1, max_blocks, layer, total_blocks, block_size,
                               kv_heads * head_dim * (dtype == B2_F32 ? 4 : 2), status, as_stream(stream));
}

int b2_paged_kv_prefill_copy(const void* key, const void* value, void* storage, const int32_t* block_table, int64_t tokens,
                             int64_t max_blocks, int64_t layer, int64_t layers, int64_t total_blocks, int64_t block_size,
                             int64_t kv_heads, int64_t head_dim, int dtype, int32_t* status, b2_stream stream) {
  const int rc = pool_checks("b2_paged_kv_prefill_copy", key, value, storage, block_table, block_table, tokens, max_blocks, layer,
                             layers, total_blocks, block_size, kv_heads, head_dim, dtype);
  if (rc != B2_OK) return rc;
  return launch_paged_kv_write(1, key, value, storage, block_table, nullptr, tokens, max_blocks, layer, total_blocks, block_size,
                               kv_heads * head_dim * (dtype == B2_F32 ? 4 : 2), status, as_stream(stream));
}

int b2_qk_norm_rope_paged(const void* q, const void* k, const void* v, const void* q_weight, const void* k_weight,
                          const int32_t* positions, void* q_out, void* storage, const int32_t* block_tables,
                          const int32_t* slot_positions, int64_t tokens, int64_t q_heads, int64_t kv_heads, int64_t head_dim,
                          float eps, float theta, int64_t tokens_per_table, int64_t max_blocks, int64_t layer, int64_t layers,
                          int64_t total_blocks, int64_t block_size, int dtype, int32_t* status, b2_stream stream) {
  const char* op = "b2_qk_norm_rope_paged";
  const int rc = pool_checks(op, k, v, storage, block_tables, positions, tokens, max_blocks, layer, layers, total_blocks,
                             block_size, kv_heads, head_dim, dtype);
  if (rc != B2_OK) return rc;
  B2_REQUIRE(q_heads > 0 && fits(tokens, (q_heads + kv_heads) * head_dim) && (q_heads + kv_heads) * head_dim < (1 << 30), op,
             "q_heads must be > 0");
  B2_REQUIRE(head_dim % 2 == 0, op, "head_dim must be even");
  B2_REQUIRE(eps > 0.0f && theta > 0.0f, op, "eps and theta must be positive");
  B2_REQUIRE(tokens_per_table >= 1, op, "tokens_per_table must be >= 1");
  B2_REQUIRE(tokens == 0 || (q && q_weight && k_weight && q_out), op, "null pointer");
  return launch_qk_norm_rope_paged(q, k, v, q_weight, k_weight, positions, q_out, storage, block_tables, slot_positions, tokens,
                                   q_heads, kv_heads, head_dim, eps, theta, tokens_per_table, max_blocks, layer, total_blocks,
                                   block_size, dtype, status, as_stream(stream));
}

int b2_select_last_valid_rows(const void* padded, const int32_t* valid_lengths, void* out, int64_t batch, int64_t seq,
                              int64_t width, int dtype, int32_t* status, b2_stream stream) {
  const char* op = "b2_select_last_valid_rows";
  B2_REQUIRE(dtype_ok(dtype), op, "dtype must be B2_F32 or B2_F16");
  B2_REQUIRE(batch >= 0 && seq > 0 && width > 0 && fits(batch, seq) && fits(batch * seq, width), op,
             "batch must be >= 0, seq and width > 0");
  B2_REQUIRE(batch == 0 || (padded && valid_lengths && out), op, "null pointer");
  return launch_select_last_valid(padded, valid_lengths, out, batch, seq, width * (dtype == B2_F32 ? 4 : 2), status,
                                  as_stream(stream));
}

size_t b2_sampler_workspace_bytes(int64_t rows, int64_t width) {
  if (rows <= 0 || width <= 0 || width > 0x7fffffffll) return 0;
  const size_t sampling = sampler_workspace_bytes(rows, width), greedy = argmax_workspace_bytes(rows);
  return sampling > greedy ? sampling : greedy;
}

int b2_sample_rows(const void* logits, int64_t rows, int64_t width, int64_t row_stride, int dtype, float temperature,
                   int32_t top_k, float top_p, uint64_t seed, const uint64_t* draw_offsets, int32_t* out_ids,
                   void* workspace, b2_stream stream) {
  const char* op = "b2_sample_rows";
  const int rc = argmax_checks(op, logits, rows, width, row_stride, dtype, 0, out_ids, workspace);
  if (rc != B2_OK) return rc;
  B2_REQUIRE(width <= 0x7fffffffll, op, "width must fit int32");
  B2_REQUIRE(std::isfinite(temperature) && temperature >= 0.0f, op, "temperature must be finite and >= 0");
  if (rows == 0) return B2_OK;
  if (temperature == 0.0f) {
    // greedy: the argmax kernel, whose scratch must start zeroed
    if (cudaMemsetAsync(workspace, 0, argmax_workspace_bytes(rows), as_stream(stream)) != cudaSuccess) return launch_status(op);
    return launch_argmax(logits, rows, width, row_stride, dtype, 0, out_ids, nullptr, workspace, as_stream(stream));
  }
  B2_REQUIRE(top_k >= 0 && int64_t(top_k) <= width, op, "top_k must be in [0, width]");
  B2_REQUIRE(std::isfinite(top_p) && top_p > 0.0f && top_p <= 1.0f, op, "top_p must be finite in (0, 1]");
  if (rows > B2_SAMPLER_MAX_ROWS) {   // the row index is the grid's second dimension
    set_error("%s: %lld rows exceed the %d rows of one call (temperature > 0); split the batch", op,
              static_cast<long long>(rows), B2_SAMPLER_MAX_ROWS);
    return B2_ERR_TOO_LARGE;
  }
  return launch_sample_rows(logits, rows, width, row_stride, dtype, temperature, top_k, top_p, seed,
                            reinterpret_cast<const unsigned long long*>(draw_offsets), out_ids, workspace, as_stream(stream));
}

int b2_ordered_sums(const float* terms, int64_t rows, int64_t n, float* sums, b2_stream stream) {
  const char* op = "b2_ordered_sums";
  B2_REQUIRE(rows >= 0 && n >= 0, op, "negative size");
  B2_REQUIRE(n <= B2_ORDERED_SUMS_MAX, op, "at most B2_ORDERED_SUMS_MAX terms per row");
  B2_REQUIRE(rows <= 0x7fffffffll, op, "too many rows");
  if (rows == 0 || n == 0) return B2_OK;
  B2_REQUIRE(terms != nullptr && sums != nullptr, op, "null pointer");
  return launch_ordered_sums(terms, rows, n, sums, as_stream(stream));
}

size_t b2_p2p_exchange_bytes(int world, int64_t max_rows) {
  return world >= 1 && world <= B2_P2P_MAX_WORLD && max_rows > 0 && max_rows < (1 << 24) ? exchange_bytes(world, max_rows) : 0;
}

int b2_p2p_exchange_init(void* buffer, int world, int64_t max_rows, b2_stream stream) {
  const char* op = "b2_p2p_exchange_init";
  B2_REQUIRE(buffer != nullptr, op, "null pointer");
  B2_REQUIRE(b2_p2p_exchange_bytes(world, max_rows) != 0, op, "need 1 <= world <= B2_P2P_MAX_WORLD and 0 < max_rows < 2^24");
  if (cudaMemsetAsync(buffer, 0, exchange_bytes(world, max_rows), as_stream(stream)) != cudaSuccess) return launch_status(op);
  return B2_OK;
}

int b2_ipc_export(const void* device_ptr, unsigned char handle[64]) {
  const char* op = "b2_ipc_export";
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the C ABI carries IPC handles as 64 bytes");
  B2_REQUIRE(device_ptr != nullptr && handle != nullptr, op, "null pointer");
  cudaIpcMemHandle_t h;
  const cudaError_t e = cudaIpcGetMemHandle(&h, const_cast<void*>(device_ptr));
  if (e != cudaSuccess) { set_error("%s: CUDA error: %s", op, cudaGetErrorString(e)); cudaGetLastError(); return B2_ERR_CUDA; }
  memcpy(handle, &h, 64);
  return B2_OK;
}

int b2_ipc_open(const unsigned char handle[64], void** device_ptr) {
  const char* op = "b2_ipc_open";
  B2_REQUIRE(handle != nullptr && device_ptr != nullptr, op, "null pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  void* p = nullptr;
  const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) { set_error("%s: CUDA error: %s", op, cudaGetErrorString(e)); cudaGetLastError(); return B2_ERR_CUDA; }
  *device_ptr = p;
  return B2_OK;
}

int b2_ipc_close(void* device_ptr) {
  if (device_ptr == nullptr) return B2_OK;
  const cudaError_t e = cudaIpcCloseMemHandle(device_ptr);
  if (e != cudaSuccess) { set_error("b2_ipc_close: CUDA error: %s", cudaGetErrorString(e)); cudaGetLastError(); return B2_ERR_CUDA; }
  return B2_OK;
}

static int exchange_checks(const char* op, const b2_p2p_exchange* x, int64_t rows, int32_t* status, ExchangeArgs* out) {
  B2_REQUIRE(x != nullptr, op, "null exchange descriptor");
  B2_REQUIRE(x->world >= 1 && x->world <= B2_P2P_MAX_WORLD && x->rank >= 0 && x->rank < x->world, op,
             "need 1 <= world <= B2_P2P_MAX_WORLD and 0 <= rank < world");
  B2_REQUIRE(x->max_rows > 0 && x->max_rows < (1 << 24), op, "max_rows out of range");
  if (rows > x->max_rows) { set_error("%s: %lld rows exceed the exchange buffer's max_rows %lld", op, (long long)rows, (long long)x->max_rows); return B2_ERR_TOO_LARGE; }
  for (int g = 0; g < x->world; ++g) {
    B2_REQUIRE(x->buffers[g] != nullptr, op, "null exchange buffer");
    out->buf[g] = static_cast<unsigned char*>(x->buffers[g]);
  }
  for (int g = x->world; g < kMaxWorld; ++g) out->buf[g] = nullptr;
  out->world = x->world;
  out->rank = x->rank;
  out->max_rows = x->max_rows;
  out->timeout_ns = static_cast<unsigned long long>(x->timeout_ms ? x->timeout_ms : 2000u) * 1000000ull;
  out->status = status;
  out->trace = reinterpret_cast<unsigned long long*>(x->trace);
  return B2_OK;
}

int b2_argmax_rows_sharded(const void* logits, int64_t rows, int64_t width, int64_t row_stride, int dtype,
                           int64_t index_base, int32_t* out_ids, void* workspace, const b2_p2p_exchange* exchange,
                           int32_t* status, b2_stream stream) {
  const char* op = "b2_argmax_rows_sharded";
  int rc = argmax_checks(op, logits, rows, width, row_stride, dtype, index_base, out_ids, workspace);
  if (rc != B2_OK) return rc;
  B2_REQUIRE(width <= 0x7fffffffll, op, "width must fit int32");
  ExchangeArgs xa;
  rc = exchange_checks(op, exchange, rows, status, &xa);
  if (rc != B2_OK) return rc;
  return launch_argmax_exchange(logits, rows, width, row_stride, dtype, index_base, out_ids, workspace, xa, as_stream(stream));
}

int b2_argmax_keys_exchange(const int64_t* keys, int64_t rows, int32_t* out_ids, const b2_p2p_exchange* exchange,
                            int32_t* status, b2_stream stream) {
  const char* op = "b2_argmax_keys_exchange";
  B2_REQUIRE(rows >= 0 && rows < (1 << 24), op, "rows must be >= 0");
  B2_REQUIRE(rows == 0 || (keys && out_ids), op, "null pointer");
  ExchangeArgs xa;
  const int rc = exchange_checks(op, exchange, rows, status, &xa);
  if (rc != B2_OK) return rc;
  return launch_argmax_keys_exchange(keys, rows, out_ids, xa, as_stream(stream));
}

int b2_softmax_stats_sharded(const void* x, int64_t rows, int64_t width, int dtype, float* global_max, float* global_sum,
                             const b2_p2p_exchange* exchange, int32_t* status, b2_stream stream) {
  const char* op = "b2_softmax_stats_sharded";
  B2_REQUIRE(dtype_ok(dtype), op, "dtype must be B2_F32 or B2_F16");
  B2_REQUIRE(rows >= 0 && width > 0 && fits(rows, width) && rows < (1 << 24), op, "rows must be >= 0 and width > 0");
  B2_REQUIRE(rows == 0 || (x && global_max && global_sum), op, "null pointer");
  ExchangeArgs xa;
  const int rc = exchange_checks(op, exchange, rows, status, &xa);
  if (rc != B2_OK) return rc;
  return launch_softmax_stats_exchange(x, rows, width, dtype, global_max, global_sum, xa, as_stream(stream));
}

void* b2_alloc(size_t bytes) {
  void* p = nullptr;
  const cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) {
    set_error("b2_alloc: CUDA error: %s", cudaGetErrorString(e));
    cudaGetLastError();
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_alloc_mutex);
  g_alloc_sizes[p] = bytes;
  ++g_alloc_stats.malloc_calls;
  g_alloc_stats.allocated_bytes_total += bytes;
  g_alloc_stats.live_bytes += bytes;
  if (g_alloc_stats.live_bytes > g_alloc_stats.peak_live_bytes) g_alloc_stats.peak_live_bytes = g_alloc_stats.live_bytes;
  return p;
}

int b2_free(void* ptr) {
  if (ptr == nullptr) return B2_OK;
  const cudaError_t e = cudaFree(ptr);
  if (e != cudaSuccess) {
    set_error("b2_free: CUDA error: %s", cudaGetErrorString(e));
    return B2_ERR_CUDA;
  }
  std::lock_guard<std::mutex> lock(g_alloc_mutex);
  const auto it = g_alloc_sizes.find(ptr);
  if (it != g_alloc_sizes.end()) {
    ++g_alloc_stats.free_calls;
    g_alloc_stats.freed_bytes_total += it->second;
    g_alloc_stats.live_bytes -= it->second;
    g_alloc_sizes.erase(it);
  }
  return B2_OK;
}

void b2_get_alloc_stats(b2_alloc_stats* out) {
  if (out == nullptr) return;
  std::lock_guard<std::mutex> lock(g_alloc_mutex);
  *out = g_alloc_stats;
}

// Allocations that are live at the reset are the baseline of the new measurement
// window: the peak restarts from the current live bytes (reference src/tensor_cuda.cu:16-25).
void b2_reset_alloc_stats(void) {
  std::lock_guard<std::mutex> lock(g_alloc_mutex);
  g_alloc_stats.malloc_calls = g_alloc_stats.free_calls = 0;
  g_alloc_stats.allocated_bytes_total = g_alloc_stats.freed_bytes_total = 0;
  g_alloc_stats.peak_live_bytes = g_alloc_stats.live_bytes;
}

}  // extern "C"
