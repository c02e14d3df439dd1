// extern "C" doors into the reference's own, unmodified CPU operators
// (reference include/llm/ops.h:7-12, src/ops_cpu.cpp).  TEST INFRASTRUCTURE ONLY:
// built by oracle/Makefile from the reference sources where they lie, used by the
// tests to validate oracle.c and by the bench's reference arm as the CPU baseline.
#include "llm/ops.h"

#include <chrono>
#include <cstring>
#include <exception>
#include <thread>
#include <vector>

#define REF_API extern "C" __attribute__((visibility("default")))

namespace {
llm::Tensor wrap(const float* p, std::vector<int64_t> shape) {
  llm::Tensor t(llm::DType::F32, std::move(shape));
  std::memcpy(t.data(), p, t.nbytes());
  return t;
}
void unwrap(const llm::Tensor& t, float* out) { std::memcpy(out, t.data(), t.nbytes()); }
template <class F> int guarded(F&& f) {
  try { f(); return 0; } catch (const std::out_of_range&) { return -2; }
  catch (const std::invalid_argument&) { return -1; } catch (const std::exception&) { return -3; }
}
}  // namespace

REF_API int ref_rms_norm(const float* x, const float* w, float eps, int64_t rows, int64_t hidden, float* out) {
  return guarded([&] { unwrap(llm::rms_norm(wrap(x, {rows, hidden}), wrap(w, {hidden}), eps), out); });
}
REF_API int ref_add(const float* a, const float* b, int64_t n, float* out) {
  return guarded([&] { unwrap(llm::add(wrap(a, {n}), wrap(b, {n})), out); });
}
REF_API int ref_swiglu(const float* gate, const float* up, int64_t n, float* out) {
  return guarded([&] { unwrap(llm::swiglu(wrap(gate, {n}), wrap(up, {n})), out); });
}
REF_API int ref_rope(const float* x, const int32_t* positions, float theta, int64_t tokens, int64_t heads,
                     int64_t head_dim, float* out) {
  return guarded([&] {
    std::vector<int32_t> p(positions, positions + tokens);
    unwrap(llm::rope(wrap(x, {tokens, heads, head_dim}), p, theta), out);
  });
}
REF_API int ref_softmax(const float* x, int64_t rows, int64_t width, float* out) {
  return guarded([&] { unwrap(llm::softmax_last_dim(wrap(x, {rows, width})), out); });
}
REF_API int ref_embedding_lookup(const float* table, int64_t vocab, int64_t hidden, const int32_t* ids,
                                 int64_t count, float* out) {
  return guarded([&] {
    std::vector<int32_t> v(ids, ids + count);
    unwrap(llm::embedding_lookup(wrap(table, {vocab, hidden}), v), out);
  });
}
REF_API int ref_lm_head(const float* hidden, const float* table, int64_t rows, int64_t in, int64_t vocab, float* out) {
  return guarded([&] { unwrap(llm::lm_head(wrap(hidden, {rows, in}), wrap(table, {vocab, in})), out); });
}
REF_API float ref_decode_f16(uint16_t h) { return llm::decode_f16(h); }
REF_API uint16_t ref_encode_f16(float x) { return llm::encode_f16(x); }

// add followed by rms_norm: how the reference's CPU layer expresses the fused op
// (reference src/qwen3_layer.cpp:48-49).
REF_API int ref_add_rms_norm(const float* lhs, const float* rhs, const float* w, float eps, int64_t rows,
                             int64_t hidden, float* residual, float* normalized) {
  return guarded([&] {
    llm::Tensor r = llm::add(wrap(lhs, {rows, hidden}), wrap(rhs, {rows, hidden}));
    unwrap(r, residual);
    unwrap(llm::rms_norm(r, wrap(w, {hidden}), eps), normalized);
  });
}

// Timed form of the above for the CPU baseline: rows are split into contiguous
// slices, one std::thread per slice, every slice calling the unmodified reference
// functions.  Returns elapsed seconds (negative on error).
REF_API double ref_time_add_rms_norm(const float* lhs, const float* rhs, const float* w, float eps,
                                     int64_t rows, int64_t hidden, float* residual, float* normalized,
                                     int threads) {
  if (threads < 1) threads = 1;
  if (threads > rows) threads = int(rows);
  std::vector<int> status(size_t(threads), 0);
  const auto t0 = std::chrono::steady_clock::now();
  std::vector<std::thread> pool;
  for (int k = 0; k < threads; ++k) {
    const int64_t lo = rows * k / threads, hi = rows * (k + 1) / threads;
    pool.emplace_back([&, k, lo, hi] {
      status[size_t(k)] = ref_add_rms_norm(lhs + lo * hidden, rhs + lo * hidden, w, eps, hi - lo, hidden,
                                           residual + lo * hidden, normalized + lo * hidden);
    });
  }
  for (auto& t : pool) t.join();
  const double dt = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
  for (int s : status) if (s) return -1.0;
  return dt;
}
REF_API int ref_hardware_threads() { return int(std::thread::hardware_concurrency()); }
