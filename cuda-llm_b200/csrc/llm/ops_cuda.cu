// namespace llm operator functions with the reference's signatures (include/llm/ops_cuda.h),
// forwarding to the sm_100a kernels through the C ABI.  Each function applies the argument rules
// of its reference counterpart (src/ops_cuda.cu, lines cited per function) and throws the same
// exception types; no arithmetic happens here.
#include "llm/ops_cuda.h"
#include "llm/ops_cuda_b200.h"
#include "llm/cuda_check.h"
#include "b2ops.h"

#include <cmath>
#include <map>
#include <stdexcept>
#include <string>

namespace llm {
namespace {

thread_local CudaReductionMode g_reduction_mode = CudaReductionMode::kFast;

int mode_code() { return g_reduction_mode == CudaReductionMode::kDeterministic ? B2_DETERMINISTIC : B2_FAST; }
int dtype_code(const Tensor& t) { return t.dtype() == DType::F32 ? B2_F32 : B2_F16; }
[[noreturn]] void reject(const std::string& op, const std::string& why) { throw std::invalid_argument(op + ": " + why); }

// reference src/ops_cuda.cu:62 (req)
void require_input(const Tensor& t, const char* op) {
  if (t.device() != DeviceType::CUDA || !t.is_contiguous()) reject(op, "requires contiguous CUDA tensor");
  if (t.dtype() != DType::F32 && t.dtype() != DType::F16) reject(op, "supports only F32/F16");
}
// reference src/ops_cuda.cu:64-65 (same_dtype)
void require_same_dtype(const Tensor& a, const Tensor& b, const char* op) {
  if (a.dtype() != b.dtype())
    reject(op, std::string("all input dtypes must match; actual ") + dtype_name(a.dtype()) + " and " + dtype_name(b.dtype()));
}
// reference src/ops_cuda.cu:66-73 (output_req)
void require_output(const Tensor& out, const std::vector<int64_t>& shape, DType dtype, const char* op) {
  if (out.device() != DeviceType::CUDA || out.dtype() != dtype || !out.is_contiguous() || out.shape() != shape)
    reject(op, std::string("output must be CUDA/") + dtype_name(dtype) + "/contiguous shape with the expected dimensions");
}
// A C ABI failure after the shim's own checks is a CUDA problem (or a bug): runtime_error, like CUDA_CHECK.
void check(int status) {
  if (status == B2_OK) return;
  if (status == B2_ERR_INVALID) throw std::invalid_argument(b2_last_error());
  throw std::runtime_error(std::string("CUDA error: ") + b2_last_error());
}

// Device scratch of the calling thread on the current device: argmax keys/tickets (kept zeroed by the
// kernel), softmax row statistics, one int32 result slot and a positions staging area.  Allocated once
// and grown on demand with plain cudaMalloc, like the reference's DeviceBuffer (src/ops_cuda.cu:565):
// not part of the Tensor allocation counters.
// A first or growing call frees, allocates, clears and then waits for the whole device: the clear runs on
// the thread's default stream, which a caller's non-blocking stream is not ordered after, so the kernel
// that follows on that stream must not start before it has landed.  Such a call is therefore illegal
// inside a stream capture (warm the operator up first).  One scratch per (thread, device, purpose): two
// streams driven by ONE thread share the argmax keys and tickets, so their calls must not overlap.
struct Scratch {
  void* ptr = nullptr;
  size_t bytes = 0;
  void* get(size_t need, bool zero) {
    if (need > bytes) {
      if (ptr) CUDA_CHECK(cudaFree(ptr));
      ptr = nullptr;
      const size_t grown = need < 4096 ? 4096 : need * 2;
      CUDA_CHECK(cudaMalloc(&ptr, grown));
      bytes = grown;
      if (zero) {
        CUDA_CHECK(cudaMemset(ptr, 0, grown));
        CUDA_CHECK(cudaDeviceSynchronize());
      }
    }
    return ptr;
  }
};
Scratch& scratch(const char* purpose) {
  thread_local std::map<std::pair<int, std::string>, Scratch> table;   // leaked at thread exit on purpose
  int device = 0;
  CUDA_CHECK(cudaGetDevice(&device));
  return table[{device, purpose}];
}


}  // namespace

CudaReductionModeGuard::CudaReductionModeGuard(CudaReductionMode mode) : previous_(g_reduction_mode) { g_reduction_mode = mode; }
CudaReductionModeGuard::~CudaReductionModeGuard() { g_reduction_mode = previous_; }
CudaReductionMode cuda_reduction_mode() { return g_reduction_mode; }

// ---------------------------------------------------------------- RMSNorm family

// reference src/ops_cuda.cu:672
void cuda_rms_norm_out(const Tensor& x, const Tensor& w, float eps, Tensor& out, cudaStream_t stream) {
  const char* op = "cuda_rms_norm";
  require_input(x, op); require_input(w, op); require_same_dtype(x, w, op);
  if (w.shape().size() != 1) reject(op, "unexpected rank");
  if (x.shape().empty() || x.shape().back() != w.shape()[0] || !(eps > 0)) reject(op, "incompatible shape/epsilon");
  require_output(out, x.shape(), x.dtype(), op);
  const int64_t hidden = x.shape().back();
  if (hidden == 0 || x.numel() == 0) throw std::runtime_error("CUDA error: cuda_rms_norm launch with an empty grid");
  check(b2_rms_norm(x.data(), w.data(), out.data(), int64_t(x.numel()) / hidden, hidden, eps, dtype_code(x), mode_code(), stream));
}

// reference src/ops_cuda.cu:673
Tensor cuda_rms_norm(const Tensor& x, const Tensor& w, float eps) {
  const char* op = "cuda_rms_norm";
  require_input(x, op); require_input(w, op); require_same_dtype(x, w, op);
  if (w.shape().size() != 1) reject(op, "unexpected rank");
  if (x.shape().empty() || x.shape().back() != w.shape()[0] || !(eps > 0)) reject(op, "incompatible shape/epsilon");
  Tensor out(x.dtype(), x.shape(), DeviceType::CUDA);
  cuda_rms_norm_out(x, w, eps, out);
  return out;
}

// reference src/ops_cuda.cu:675-703
void cuda_add_rms_norm_out(const Tensor& lhs, const Tensor& rhs, const Tensor& w, float eps, Tensor& residual,
                           Tensor& normalized, cudaStream_t stream) {
  const char* op = "cuda_add_rms_norm";
  require_input(lhs, op); require_input(rhs, op); require_input(w, op);
  require_same_dtype(lhs, rhs, op); require_same_dtype(lhs, w, op);
  if (w.shape().size() != 1) reject(op, "unexpected rank");
  if (lhs.shape() != rhs.shape() || lhs.shape().empty() || lhs.shape().back() != w.shape()[0] || !(eps > 0.0f))
    reject(op, "incompatible shapes/epsilon");
  require_output(residual, lhs.shape(), lhs.dtype(), op);
  require_output(normalized, lhs.shape(), lhs.dtype(), op);
  const int64_t hidden = lhs.shape().back();
  if (hidden == 0 || lhs.numel() == 0) throw std::runtime_error("CUDA error: cuda_add_rms_norm launch with an empty grid");
  check(b2_add_rms_norm(lhs.data(), rhs.data(), w.data(), residual.data(), normalized.data(), int64_t(lhs.numel()) / hidden,
                        hidden, eps, dtype_code(lhs), mode_code(), stream));
}

// ---------------------------------------------------------------- elementwise

// reference src/ops_cuda.cu:674
void cuda_add_out(const Tensor& a, const Tensor& b, Tensor& out, cudaStream_t stream) {
  const char* op = "cuda_add";
  require_input(a, op); require_input(b, op); require_same_dtype(a, b, op);
  if (a.shape() != b.shape()) reject(op, "shapes must match");
  require_output(out, a.shape(), a.dtype(), op);
  check(b2_add(a.data(), b.data(), out.data(), int64_t(a.numel()), dtype_code(a), stream));
}
// reference src/ops_cuda.cu:704
Tensor cuda_add(const Tensor& a, const Tensor& b) {
  const char* op = "cuda_add";
  require_input(a, op); require_input(b, op); require_same_dtype(a, b, op);
  if (a.shape() != b.shape()) reject(op, "shapes must match");
  Tensor out(a.dtype(), a.shape(), DeviceType::CUDA);
  cuda_add_out(a, b, out);
  return out;
}

// reference src/ops_cuda.cu:705
void cuda_swiglu_out(const Tensor& gate, const Tensor& up, Tensor& out, cudaStream_t stream) {
  const char* op = "cuda_swiglu";
  require_input(gate, op); require_input(up, op); require_same_dtype(gate, up, op);
  if (gate.shape() != up.shape()) reject(op, "shapes must match");
  require_output(out, gate.shape(), gate.dtype(), op);
  check(b2_swiglu(gate.data(), up.data(), out.data(), int64_t(gate.numel()), dtype_code(gate), mode_code(), stream));
}
// reference src/ops_cuda.cu:706
Tensor cuda_swiglu(const Tensor& gate, const Tensor& up) {
  const char* op = "cuda_swiglu";
  require_input(gate, op); require_input(up, op); require_same_dtype(gate, up, op);
  if (gate.shape() != up.shape()) reject(op, "shapes must match");
  Tensor out(gate.dtype(), gate.shape(), DeviceType::CUDA);
  cuda_swiglu_out(gate, up, out);
  return out;
}

// ---------------------------------------------------------------- rotary embedding

namespace {
// The rotary-embedding kernels bound their waits on on-chip copies and say so in a status word if one ever runs out.
// The reference would have surfaced such a failure as a CUDA error at the caller's next call; so does this: the word
// is one pinned, device-visible int32 per thread and device, read by the host (no synchronisation) at the start of
// every rotary-embedding call, and a set bit becomes the runtime_error of that call.  The first call of a thread on a
// device allocates the word: make it outside any stream capture.
int32_t* rope_status_word() {
  thread_local std::map<int, int32_t*> words;   // leaked at thread exit on purpose
  int device = 0;
  CUDA_CHECK(cudaGetDevice(&device));
  int32_t*& word = words[device];
  if (word == nullptr) {
    CUDA_CHECK(cudaHostAlloc(reinterpret_cast<void**>(&word), sizeof(int32_t), cudaHostAllocMapped | cudaHostAllocPortable));
    *word = 0;
  }
  return word;
}
int32_t* checked_rope_status(const char* op) {
  int32_t* word = rope_status_word();
  if (*static_cast<volatile int32_t*>(word) != 0) {
    *word = 0;
    throw std::runtime_error(std::string("CUDA error: ") + op +
                             ": an earlier rotary-embedding launch gave up waiting for an on-chip copy; its output is incomplete");
  }
  return word;
}
// host positions -> the thread's device staging area (the reference allocates and frees a buffer
// per call, src/ops_cuda.cu:707; the copy is blocking in both)
const int32_t* stage_positions(const std::vector<int32_t>& positions) {
  void* p = scratch("positions").get(positions.size() * sizeof(int32_t), false);
  CUDA_CHECK(cudaMemcpy(p, positions.data(), positions.size() * sizeof(int32_t), cudaMemcpyHostToDevice));
  return static_cast<const int32_t*>(p);
}
}  // namespace

// reference src/ops_cuda.cu:707
Tensor cuda_rope(const Tensor& x, const std::vector<int32_t>& positions, float theta) {
  const char* op = "cuda_rope";
  require_input(x, op);
  if (x.shape().size() != 3) reject(op, "unexpected rank");
  const auto& s = x.shape();
  if (s[0] == 0 || s[1] == 0 || s[2] == 0 || s[2] % 2 || positions.empty() || positions.size() != size_t(s[0]) || !(theta > 0))
    reject(op, "invalid or empty shape/positions/theta");
  Tensor out(x.dtype(), s, DeviceType::CUDA);
  check(b2_rope(x.data(), stage_positions(positions), out.data(), s[0], s[1], s[2], theta, dtype_code(x), mode_code(),
                checked_rope_status(op), 0));
  return out;
}

// reference src/ops_cuda.cu:708
Tensor cuda_rope_batched(const Tensor& x, const std::vector<int32_t>& positions, float theta) {
  const char* op = "cuda_rope_batched";
  require_input(x, op);
  if (x.shape().size() != 4) reject(op, "unexpected rank");
  const auto& s = x.shape();
  if (s[0] == 0 || s[1] == 0 || s[2] == 0 || s[3] == 0 || s[3] % 2 || positions.size() != size_t(s[1]) || !(theta > 0))
    reject(op, "invalid shape/positions/theta");
  Tensor out(x.dtype(), s, DeviceType::CUDA);
  check(b2_rope_batched(x.data(), stage_positions(positions), out.data(), s[0], s[1], s[2], s[3], theta, dtype_code(x),
                        mode_code(), checked_rope_status(op), 0));
  return out;
}

// reference src/ops_cuda.cu:709
void cuda_rope_batched_out(const Tensor& x, const Tensor& positions_device, float theta, Tensor& out) {
  const char* op = "cuda_rope_batched";
  require_input(x, op);
  if (x.shape().size() != 4) reject(op, "unexpected rank");
  const auto& s = x.shape();
  if (s[0] == 0 || s[1] == 0 || s[2] == 0 || s[3] == 0 || s[3] % 2 || !(theta > 0)) reject(op, "invalid shape/theta");
  if (positions_device.device() != DeviceType::CUDA || positions_device.dtype() != DType::F32 ||
      !positions_device.is_contiguous() || positions_device.numel() < size_t(s[1]))
    reject(op, "positions buffer must be CUDA/F32/contiguous and large enough");
  require_output(out, s, x.dtype(), op);
  check(b2_rope_batched(x.data(), static_cast<const int32_t*>(positions_device.data()), out.data(), s[0], s[1], s[2], s[3],
                        theta, dtype_code(x), mode_code(), checked_rope_status(op), 0));
}

namespace {
// shared by the two one-position-per-row entry points (reference src/ops_cuda.cu:972-990,1083-1102)
void rope_rows(const char* op, const Tensor& x, const Tensor& positions, float theta, Tensor& out, cudaStream_t stream) {
  require_input(x, op);
  if (x.shape().size() != 3 || x.shape()[0] <= 0 || x.shape()[1] <= 0 || x.shape()[2] <= 0 || x.shape()[2] % 2 ||
      positions.device() != DeviceType::CUDA || positions.dtype() != DType::I32 || !positions.is_contiguous() ||
      positions.shape() != std::vector<int64_t>{x.shape()[0]} || !(theta > 0.0f))
    reject(op, "expected CUDA F32/F16 [T,H,D] with even D and CUDA/I32 positions [T]");
  require_output(out, x.shape(), x.dtype(), op);
  check(b2_rope(x.data(), static_cast<const int32_t*>(positions.data()), out.data(), x.shape()[0], x.shape()[1],
                x.shape()[2], theta, dtype_code(x), mode_code(), checked_rope_status(op), stream));
}
}  // namespace

void cuda_rope_batched_positions_out(const Tensor& x, const Tensor& positions_device, float theta, Tensor& out) {
  rope_rows("cuda_rope_batched_positions", x, positions_device, theta, out, 0);
}
void cuda_rope_token_positions_out(const Tensor& x, const Tensor& positions_device, float theta, Tensor& out,
                                   cudaStream_t stream) {
  rope_rows("cuda_rope_token_positions", x, positions_device, theta, out, stream);
}

void cuda_qk_norm_rope_out(const Tensor& q, const Tensor& k, const Tensor& qw, const Tensor& kw, const Tensor& positions,
                           float eps, float theta, Tensor& q_out, Tensor& k_out, cudaStream_t stream) {
  const char* op = "cuda_qk_norm_rope";
  require_input(q, op); require_input(k, op); require_input(qw, op); require_input(kw, op);
  require_same_dtype(q, k, op); require_same_dtype(q, qw, op); require_same_dtype(q, kw, op);
  if (q.shape().size() != 3 || k.shape().size() != 3 || q.shape()[0] != k.shape()[0] || q.shape()[2] != k.shape()[2] ||
      q.shape()[0] <= 0 || q.shape()[1] <= 0 || k.shape()[1] <= 0 || q.shape()[2] <= 0 || q.shape()[2] % 2 ||
      qw.shape() != std::vector<int64_t>{q.shape()[2]} || kw.shape() != qw.shape() || !(eps > 0) || !(theta > 0))
    reject(op, "expected q [T,Hq,D], k [T,Hk,D] with even D, weights [D], eps > 0, theta > 0");
  if (positions.device() != DeviceType::CUDA || positions.dtype() != DType::I32 || !positions.is_contiguous() ||
      positions.shape() != std::vector<int64_t>{q.shape()[0]})
    reject(op, "positions must be CUDA/I32 [T]");
  require_output(q_out, q.shape(), q.dtype(), op);
  require_output(k_out, k.shape(), k.dtype(), op);
  check(b2_qk_norm_rope(q.data(), k.data(), qw.data(), kw.data(), static_cast<const int32_t*>(positions.data()), q_out.data(),
                        k_out.data(), q.shape()[0], q.shape()[1], k.shape()[1], q.shape()[2], eps, theta, dtype_code(q),
                        checked_rope_status(op), stream));
}

// ---------------------------------------------------------------- softmax

// reference src/ops_cuda.cu:710
Tensor cuda_softmax_last_dim(const Tensor& x) {
  const char* op = "cuda_softmax_last_dim";
  require_input(x, op);
  if (x.shape().empty() || x.shape().back() <= 0) reject(op, "invalid last dimension");
  Tensor out(x.dtype(), x.shape(), DeviceType::CUDA);
  const int64_t width = x.shape().back(), rows = int64_t(x.numel()) / width;
  if (rows == 0) throw std::runtime_error("CUDA error: cuda_softmax_last_dim launch with an empty grid");
  void* ws = scratch("softmax").get(b2_softmax_workspace_bytes(rows), true);
  check(b2_softmax_rows(x.data(), out.data(), rows, width, dtype_code(x), mode_code(), ws, 0));
  return out;
}

// ---------------------------------------------------------------- embedding gather

namespace {
void gather_weight_rules(const Tensor& w, const char* op) {
  require_input(w, op);
  if (w.shape().size() != 2) reject(op, "unexpected rank");
}
}  // namespace

// reference src/ops_cuda.cu:872
void cuda_embedding_lookup_out(const Tensor& w, const std::vector<int32_t>& ids, Tensor& ids_device, Tensor& out) {
  const char* op = "cuda_embedding_lookup";
  gather_weight_rules(w, op);
  if (ids.empty()) reject(op, "token_ids must be non-empty");
  const int64_t vocab = w.shape()[0], hidden = w.shape()[1];
  if (vocab <= 0 || hidden <= 0) reject(op, "weight shape must be positive");
  for (int32_t id : ids)
    if (id < 0 || int64_t(id) >= vocab) reject(op, "token id out of range");
  if (ids_device.device() != DeviceType::CUDA || ids_device.dtype() != DType::F32 || !ids_device.is_contiguous() ||
      ids_device.numel() < ids.size())
    reject(op, "token storage must be CUDA/F32/contiguous");
  require_output(out, {int64_t(ids.size()), hidden}, w.dtype(), op);
  CUDA_CHECK(cudaMemcpy(ids_device.data(), ids.data(), ids.size() * sizeof(int32_t), cudaMemcpyHostToDevice));
  check(b2_embedding_gather(w.data(), static_cast<const int32_t*>(ids_device.data()), out.data(), int64_t(ids.size()), hidden,
                            vocab, dtype_code(w), nullptr, 0));
}

// reference src/ops_cuda.cu:873-884
void cuda_embedding_lookup_device_ids_out(const Tensor& w, const Tensor& ids, Tensor& out) {
  const char* op = "cuda_embedding_lookup_device_ids";
  gather_weight_rules(w, op);
  if (ids.device() != DeviceType::CUDA || ids.dtype() != DType::F32 || !ids.is_contiguous() || ids.shape().size() != 1 ||
      ids.shape()[0] <= 0)
    reject(op, "ids must be CUDA/F32/contiguous rank-1");
  const int64_t vocab = w.shape()[0], hidden = w.shape()[1];
  if (vocab <= 0 || hidden <= 0) reject(op, "weight shape must be positive");
  require_output(out, {ids.shape()[0], hidden}, w.dtype(), op);
  check(b2_embedding_gather(w.data(), static_cast<const int32_t*>(ids.data()), out.data(), ids.shape()[0], hidden, vocab,
                            dtype_code(w), nullptr, 0));
}

// reference src/ops_cuda.cu:885
Tensor cuda_embedding_lookup(const Tensor& w, const std::vector<int32_t>& ids) {
  const char* op = "cuda_embedding_lookup";
  gather_weight_rules(w, op);
  if (ids.empty()) reject(op, "token_ids must be non-empty");
  if (w.shape()[0] <= 0 || w.shape()[1] <= 0) reject(op, "weight shape must be positive");
  Tensor ids_device(DType::F32, {int64_t(ids.size())}, DeviceType::CUDA);
  Tensor out(w.dtype(), {int64_t(ids.size()), w.shape()[1]}, DeviceType::CUDA);
  cuda_embedding_lookup_out(w, ids, ids_device, out);
  return out;
}

// ---------------------------------------------------------------- argmax

namespace {
void logits_rules(const Tensor& logits, const char* op) {
  if (logits.device() != DeviceType::CUDA || !logits.is_contiguous()) reject(op, "requires contiguous CUDA tensor");
  if (logits.dtype() != DType::F32 && logits.dtype() != DType::F16) reject(op, "supports only F32/F16");
  if (logits.shape().size() != 2) reject(op, "unexpected rank");
  if (logits.shape()[0] <= 0 || logits.shape()[1] <= 0) reject(op, "shape dimensions must be > 0");
}
}  // namespace

// reference src/ops_cuda.cu:871 + :711 (argmax_row_impl).  One kernel, no allocation; the only blocking
// step is the 4-byte copy of the result, which the return type requires.
int32_t cuda_argmax_last_row(const Tensor& logits) {
  const char* op = "cuda_argmax_last_row";
  logits_rules(logits, op);
  const int64_t rows = logits.shape()[0], width = logits.shape()[1];
  char* ws = static_cast<char*>(scratch("argmax").get(b2_argmax_workspace_bytes(1) + 16, true));
  int32_t* result = reinterpret_cast<int32_t*>(ws + b2_argmax_workspace_bytes(1));
  const char* last_row = static_cast<const char*>(logits.data()) + size_t(rows - 1) * size_t(width) * dtype_size(logits.dtype());
  check(b2_argmax_rows(last_row, 1, width, width, dtype_code(logits), result, ws, 0));
  int32_t host = 0;
  CUDA_CHECK(cudaMemcpyAsync(&host, result, sizeof(host), cudaMemcpyDeviceToHost, 0));
  CUDA_CHECK(cudaStreamSynchronize(0));
  return host;
}

void cuda_argmax_rows_out(const Tensor& logits, Tensor& ids, cudaStream_t stream) {
  const char* op = "cuda_argmax_rows";
  logits_rules(logits, op);
  const int64_t rows = logits.shape()[0], width = logits.shape()[1];
  if (ids.device() != DeviceType::CUDA || ids.dtype() != DType::I32 || !ids.is_contiguous() ||
      ids.shape() != std::vector<int64_t>{rows})
    reject(op, "output must be CUDA/I32 [rows]");
  void* ws = scratch("argmax_rows").get(b2_argmax_workspace_bytes(rows), true);
  check(b2_argmax_rows(logits.data(), rows, width, width, dtype_code(logits), static_cast<int32_t*>(ids.data()), ws, stream));
}

// Argument rules of the reference's cuda_lm_head (src/ops_cuda.cu:885), then one fused launch.
void cuda_lm_head_argmax_out(const Tensor& hidden, const Tensor& embedding, Tensor& ids, Tensor* logits, cudaStream_t stream) {
  const char* op = "cuda_lm_head";
  if (hidden.device() != DeviceType::CUDA || embedding.device() != DeviceType::CUDA)
    reject(op, "hidden and tied embedding must be CUDA");
  if (hidden.shape().size() != 2 || embedding.shape().size() != 2) reject(op, "hidden and embedding must be rank-2");
  if (hidden.shape().back() != embedding.shape()[1]) reject(op, "hidden_size mismatch");
  if (hidden.dtype() != embedding.dtype()) reject(op, "all input dtypes must match");
  if (hidden.dtype() != DType::F32 && hidden.dtype() != DType::F16) reject(op, "supports only F32/F16");
  if (!hidden.is_contiguous() || !embedding.is_contiguous()) reject(op, "requires contiguous CUDA tensor");
  const int64_t rows = hidden.shape()[0], hsz = hidden.shape()[1], vocab = embedding.shape()[0];
  if (rows <= 0 || hsz <= 0 || vocab <= 0) reject(op, "shape dimensions must be > 0");
  if (ids.device() != DeviceType::CUDA || ids.dtype() != DType::I32 || !ids.is_contiguous() ||
      ids.shape() != std::vector<int64_t>{rows})
    reject(op, "ids must be CUDA/I32 [rows]");
  if (logits != nullptr && (logits->device() != DeviceType::CUDA || logits->dtype() != hidden.dtype() || !logits->is_contiguous() ||
                            logits->shape() != std::vector<int64_t>{rows, vocab}))
    reject(op, "logits must be CUDA [rows, vocab] of the inputs' dtype");
  void* ws = scratch("argmax_rows").get(b2_argmax_workspace_bytes(rows), true);
  check(b2_lm_head_argmax(hidden.data(), embedding.data(), rows, hsz, vocab, dtype_code(hidden), mode_code(), 0,
                          logits ? logits->data() : nullptr, vocab, static_cast<int32_t*>(ids.data()), nullptr, ws, stream));
}

// ---------------------------------------------------------------- sampler

// reference src/ops_cuda.cu:886-890.  The workspace (keys, running sums, one result slot, one draw offset)
// is a plain device allocation made once, like the reference's SamplerWorkspace buffers.
CudaSampler::CudaSampler(size_t max_vocab) : max_vocab_(max_vocab) {
  if (max_vocab == 0) throw std::invalid_argument("CudaSampler: max_vocab must be > 0");
  const size_t bytes = b2_sampler_workspace_bytes(1, int64_t(max_vocab));
  if (bytes == 0) throw std::invalid_argument("CudaSampler: max_vocab out of range");
  CUDA_CHECK(cudaMalloc(&workspace_, bytes + 16));
}
CudaSampler::~CudaSampler() { cudaFree(workspace_); }

// reference src/ops_cuda.cu:891-937
int32_t CudaSampler::sample_row_offset(const Tensor& logits, size_t row_offset, const SamplingConfig& config,
                                       uint64_t draw_offset) {
  const char* op = "CudaSampler::sample_last_row";
  if (logits.device() != DeviceType::CUDA || !logits.is_contiguous()) reject(op, "requires contiguous CUDA tensor");
  if (logits.dtype() != DType::F32 && logits.dtype() != DType::F16) reject(op, "supports F32/F16 only");
  if ((logits.shape().size() != 2 && logits.shape().size() != 3) || logits.shape().back() == 0)
    reject(op, "requires non-empty rank-2 or rank-3 logits");
  const size_t vocab = static_cast<size_t>(logits.shape().back());
  if (vocab > max_vocab_) reject(op, "vocab exceeds sampler capacity");
  if (!std::isfinite(config.temperature) || config.temperature < 0.0f) reject(op, "temperature must be finite and >= 0");
  if (config.temperature != 0.0f) {
    if (config.top_k < 0 || static_cast<size_t>(config.top_k) > vocab) reject(op, "top_k must be in [0,vocab]");
    if (!std::isfinite(config.top_p) || config.top_p <= 0.0f || config.top_p > 1.0f) reject(op, "top_p must be finite in (0,1]");
  }
  const size_t bytes = b2_sampler_workspace_bytes(1, int64_t(max_vocab_));
  char* tail = static_cast<char*>(workspace_) + bytes;                 // [0,8): the draw offset, [8,12): the result
  uint64_t* offset_device = reinterpret_cast<uint64_t*>(tail);
  int32_t* result_device = reinterpret_cast<int32_t*>(tail + 8);
  CUDA_CHECK(cudaMemcpyAsync(offset_device, &draw_offset, sizeof(draw_offset), cudaMemcpyHostToDevice, 0));
  const char* row = static_cast<const char*>(logits.data()) + row_offset * dtype_size(logits.dtype());
  check(b2_sample_rows(row, 1, int64_t(vocab), int64_t(vocab), dtype_code(logits), config.temperature, config.top_k,
                       config.temperature != 0.0f ? config.top_p : 1.0f, config.seed, offset_device, result_device,
                       workspace_, 0));
  int32_t host = 0;
  CUDA_CHECK(cudaMemcpyAsync(&host, result_device, sizeof(host), cudaMemcpyDeviceToHost, 0));
  CUDA_CHECK(cudaStreamSynchronize(0));
  return host;
}

// reference src/ops_cuda.cu:938-944
int32_t CudaSampler::sample_last_row(const Tensor& logits, const SamplingConfig& config, uint64_t draw_offset) {
  if (logits.shape().size() != 2 || logits.shape()[0] == 0)
    reject("CudaSampler::sample_last_row", "requires non-empty rank-2 logits");
  return sample_row_offset(logits, (static_cast<size_t>(logits.shape()[0]) - 1) * static_cast<size_t>(logits.shape()[1]),
                           config, draw_offset);
}

// reference src/ops_cuda.cu:945-960
int32_t CudaSampler::sample_last_token_of_batch(const Tensor& logits, size_t batch_index, const SamplingConfig& config,
                                                uint64_t draw_offset) {
  const char* op = "CudaSampler::sample_last_token_of_batch";
  if (logits.device() != DeviceType::CUDA || !logits.is_contiguous()) reject(op, "requires contiguous CUDA tensor");
  if (logits.dtype() != DType::F32 && logits.dtype() != DType::F16) reject(op, "supports F32/F16 only");
  if (logits.shape().size() != 3 || logits.numel() == 0) reject(op, "requires non-empty rank-3 logits");
  if (batch_index >= static_cast<size_t>(logits.shape()[0])) throw std::out_of_range(std::string(op) + ": batch_index out of range");
  const size_t seq = static_cast<size_t>(logits.shape()[1]), vocab = static_cast<size_t>(logits.shape()[2]);
  return sample_row_offset(logits, (batch_index * seq + seq - 1) * vocab, config, draw_offset);
}

// reference src/ops_cuda.cu:961-971
int32_t CudaSampler::sample_row(const Tensor& logits, size_t batch_index, const SamplingConfig& config, uint64_t draw_offset) {
  const char* op = "CudaSampler::sample_row";
  if (logits.shape().size() != 2 || logits.numel() == 0) reject(op, "requires non-empty rank-2 logits");
  if (batch_index >= static_cast<size_t>(logits.shape()[0])) throw std::out_of_range(std::string(op) + ": batch_index out of range");
  return sample_row_offset(logits, batch_index * static_cast<size_t>(logits.shape()[1]), config, draw_offset);
}

}  // namespace llm
