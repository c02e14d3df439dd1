// GPU checks of the namespace llm operator functions against the CPU oracle (oracle/oracle.c).
// The cases follow the reference's own operator tests: tests/test_ops_cuda.cpp:111-151,196-206,
// tests/test_argmax_cuda.cpp:42-57, tests/test_embedding_lm_head_cuda.cpp:19-24,
// tests/test_tensor_cuda.cpp:10-12 and tests/test_cuda_allocation_stats.cpp:22-52 (same inputs, same
// tolerances, same rejections), and add the `*_out`, in-place, view and mode paths that the
// reference only exercises through its model-level tests.
#include "llm/cuda_check.h"
#include "llm/ops_cuda.h"

#include <cmath>
#include <cstring>
#include <functional>
#include <iostream>
#include <stdexcept>
#include <string>
#include <vector>

using namespace llm;

extern "C" {   // the CPU oracle (test infrastructure)
void orc_cpu_rms_norm(const float*, const float*, float, int64_t, int64_t, float*);
void orc_cpu_add(const float*, const float*, int64_t, float*);
void orc_cpu_swiglu(const float*, const float*, int64_t, float*);
int orc_cpu_rope(const float*, const int32_t*, float, int64_t, int64_t, int64_t, float*);
void orc_cpu_softmax(const float*, int64_t, int64_t, float*);
int orc_cpu_embedding_lookup(const float*, int64_t, int64_t, const int32_t*, int64_t, float*);
void orc_cpu_linear(const float*, const float*, int64_t, int64_t, int64_t, float*);
int32_t orc_argmax_row_f32(const float*, int64_t);
uint16_t orc_f32_to_f16_rn(float);
void orc_dev_add_rms_norm(const void*, const void*, const void*, float, int64_t, int64_t, void*, void*, int);
}

static void fail(const std::string& m) { throw std::runtime_error("test_ops_cuda_b200: " + m); }
static void expect_throw(const std::string& name, const std::function<void()>& fn) {
  try { fn(); } catch (const std::exception& e) { std::cout << "rejected " << name << ": " << e.what() << "\n"; return; }
  fail(name + " was accepted");
}
static std::vector<float> values(const Tensor& t) {
  Tensor h = t.device() == DeviceType::CUDA ? t.to(DeviceType::CPU) : t;
  std::vector<float> v(h.numel());
  for (size_t i = 0; i < v.size(); ++i) v[i] = h.get_f32(i);
  return v;
}
// fp16 tensor holding round-to-nearest-even conversions of `src` (the host encoder truncates, so it is not used)
static Tensor half_of(const Tensor& src) {
  Tensor h(DType::F16, src.shape());
  for (size_t i = 0; i < src.numel(); ++i) h.data_f16()[i] = orc_f32_to_f16_rn(src.get_f32(i));
  return h;
}
static Tensor widen(const Tensor& h) {
  Tensor f(DType::F32, h.shape());
  for (size_t i = 0; i < h.numel(); ++i) f.set_f32(i, h.get_f32(i));
  return f;
}
static void metric(const std::string& name, const Tensor& actual, const std::vector<float>& expected, float tol) {
  const std::vector<float> got = values(actual);
  if (got.size() != expected.size()) fail(name + " size mismatch");
  float worst = 0;
  for (size_t i = 0; i < got.size(); ++i) {
    if (!std::isfinite(got[i]) || !std::isfinite(expected[i])) fail(name + " non-finite value");
    worst = std::max(worst, std::fabs(got[i] - expected[i]));
  }
  std::cout << name << " dtype=" << dtype_name(actual.dtype()) << " max_abs_error=" << worst << " tolerance=" << tol << "\n";
  if (worst > tol) fail(name + " numeric threshold failed");
}
static Tensor cuda(const Tensor& t) { return t.to(DeviceType::CUDA); }

static void operators_against_oracle() {
  Tensor x = Tensor::from_f32({3, 4}, {1, -2, 3, 0, .5f, 2, -1, 4, -3, 1, 2, -.5f});
  Tensor w = Tensor::from_f32({4}, {1, .5f, 2, -1});
  Tensor x16 = half_of(x), w16 = half_of(w), xf = widen(x16), wf = widen(w16);
  std::vector<float> want(12), want16(12);

  orc_cpu_rms_norm(x.data_f32(), w.data_f32(), 1e-5f, 3, 4, want.data());
  orc_cpu_rms_norm(xf.data_f32(), wf.data_f32(), 1e-5f, 3, 4, want16.data());
  metric("cuda_rms_norm_f32", cuda_rms_norm(cuda(x), cuda(w), 1e-5f), want, 1e-4f);
  metric("cuda_rms_norm_f16", cuda_rms_norm(cuda(x16), cuda(w16), 1e-5f), want16, 5e-3f);
  {
    CudaReductionModeGuard guard(CudaReductionMode::kDeterministic);
    metric("cuda_rms_norm_f32 deterministic", cuda_rms_norm(cuda(x), cuda(w), 1e-5f), want, 1e-4f);
    if (cuda_reduction_mode() != CudaReductionMode::kDeterministic) fail("mode guard");
  }
  if (cuda_reduction_mode() != CudaReductionMode::kFast) fail("mode guard restore");

  orc_cpu_add(x.data_f32(), x.data_f32(), 12, want.data());
  orc_cpu_add(xf.data_f32(), xf.data_f32(), 12, want16.data());
  metric("cuda_add_f32", cuda_add(cuda(x), cuda(x)), want, 1e-4f);
  metric("cuda_add_f16", cuda_add(cuda(x16), cuda(x16)), want16, 5e-3f);
  orc_cpu_swiglu(x.data_f32(), x.data_f32(), 12, want.data());
  orc_cpu_swiglu(xf.data_f32(), xf.data_f32(), 12, want16.data());
  metric("cuda_swiglu_f32", cuda_swiglu(cuda(x), cuda(x)), want, 1e-4f);
  metric("cuda_swiglu_f16", cuda_swiglu(cuda(x16), cuda(x16)), want16, 5e-3f);

  // *_out forms: caller storage, output aliasing an input (reference src/qwen3_layer_cuda.cu:323), views
  Tensor gate = cuda(x), up = cuda(x);
  cuda_swiglu_out(gate, up, gate);
  metric("cuda_swiglu_out in place", gate, want, 1e-4f);
  Tensor big = cuda(Tensor::from_f32({4, 4}, {9, 9, 9, 9, 1, -2, 3, 0, .5f, 2, -1, 4, -3, 1, 2, -.5f}));
  Tensor view = big.slice_first_dim(1, 3), out(DType::F32, {3, 4}, DeviceType::CUDA);
  orc_cpu_rms_norm(x.data_f32(), w.data_f32(), 1e-5f, 3, 4, want.data());
  cuda_rms_norm_out(view, cuda(w), 1e-5f, out);
  metric("cuda_rms_norm_out on a row slice", out, want, 1e-4f);

  // fused add + norm: two outputs; deterministic mode is bit-exact against the device-order restatement
  Tensor res(DType::F16, {3, 4}, DeviceType::CUDA), nrm(DType::F16, {3, 4}, DeviceType::CUDA);
  std::vector<float> sum(12), normed(12);
  orc_cpu_add(xf.data_f32(), xf.data_f32(), 12, sum.data());
  orc_cpu_rms_norm(sum.data(), wf.data_f32(), 1e-5f, 3, 4, normed.data());
  cuda_add_rms_norm_out(cuda(x16), cuda(x16), cuda(w16), 1e-5f, res, nrm);
  metric("cuda_add_rms_norm_out residual f16", res, sum, 5e-3f);
  metric("cuda_add_rms_norm_out normalized f16", nrm, normed, 5e-3f);
  {
    CudaReductionModeGuard guard(CudaReductionMode::kDeterministic);
    cuda_add_rms_norm_out(cuda(x16), cuda(x16), cuda(w16), 1e-5f, res, nrm);
    std::vector<uint16_t> want_res(12), want_nrm(12);
    orc_dev_add_rms_norm(x16.data(), x16.data(), w16.data(), 1e-5f, 3, 4, want_res.data(), want_nrm.data(), 1);
    Tensor hres = res.to(DeviceType::CPU), hnrm = nrm.to(DeviceType::CPU);
    if (std::memcmp(hres.data(), want_res.data(), 24) || std::memcmp(hnrm.data(), want_nrm.data(), 24))
      fail("deterministic add_rms_norm is not bit-exact");
    std::cout << "cuda_add_rms_norm_out deterministic: bit-exact\n";
  }

  Tensor rope_x = Tensor::from_f32({2, 1, 4}, {1, 2, 3, 4, 2, -1, .5f, 3});
  std::vector<int32_t> positions{0, 1};
  std::vector<float> rope_want(8);
  orc_cpu_rope(rope_x.data_f32(), positions.data(), 10000, 2, 1, 4, rope_want.data());
  metric("cuda_rope_f32", cuda_rope(cuda(rope_x), positions, 10000), rope_want, 1e-4f);
  Tensor rope16 = half_of(rope_x), ropef = widen(rope16);
  orc_cpu_rope(ropef.data_f32(), positions.data(), 10000, 2, 1, 4, rope_want.data());
  metric("cuda_rope_f16", cuda_rope(cuda(rope16), positions, 10000), rope_want, 5e-3f);

  // the device-position entry points on a Qwen3-shaped tensor: [T,16,128] rows, one position per row
  const int64_t T = 5, H = 16, D = 128;
  Tensor q(DType::F32, {T, H, D});
  for (size_t i = 0; i < q.numel(); ++i) q.set_f32(i, std::sin(0.37f * float(i)) * 2.0f);
  std::vector<int32_t> pos{0, 3, 17, 511, 4096};
  std::vector<float> q_want(q.numel());
  Tensor q16 = half_of(q), q16f = widen(q16);
  orc_cpu_rope(q16f.data_f32(), pos.data(), 1e6f, T, H, D, q_want.data());
  Tensor pos_dev(DType::I32, {T});
  std::memcpy(pos_dev.data_i32(), pos.data(), sizeof(int32_t) * size_t(T));
  Tensor pos_cuda = pos_dev.to(DeviceType::CUDA), q_cuda = cuda(q16), q_out(DType::F16, {T, H, D}, DeviceType::CUDA);
  cuda_rope_token_positions_out(q_cuda, pos_cuda, 1e6f, q_out);
  metric("cuda_rope_token_positions_out f16", q_out, q_want, 5e-3f);
  cuda_rope_batched_positions_out(q_cuda, pos_cuda, 1e6f, q_cuda);   // in place (src/qwen3_layer_cuda.cu:800-801)
  metric("cuda_rope_batched_positions_out in place", q_cuda, q_want, 5e-3f);
  // batched: [B=1,S=T,H,D] with S shared positions carried in an F32-typed buffer (src/ops_cuda.cu:709)
  Tensor pos_f32(DType::F32, {8});
  std::memcpy(pos_f32.data(), pos.data(), sizeof(int32_t) * size_t(T));
  Tensor b_out(DType::F16, {1, T, H, D}, DeviceType::CUDA);
  cuda_rope_batched_out(cuda(q16).reshape({1, T, H, D}), pos_f32.to(DeviceType::CUDA), 1e6f, b_out);
  metric("cuda_rope_batched_out f16", b_out, q_want, 5e-3f);
  metric("cuda_rope_batched f16", cuda_rope_batched(cuda(q16).reshape({1, T, H, D}), pos, 1e6f), q_want, 5e-3f);

  // fused QK-norm + RoPE against the oracle chain rms_norm -> rope
  Tensor kk = q.slice_first_dim(0, T).reshape({T, H, D}), gq(DType::F32, {D});
  for (size_t i = 0; i < size_t(D); ++i) gq.set_f32(i, 0.5f + float(i) / float(D));
  std::vector<float> qn(q.numel()), qr(q.numel());
  orc_cpu_rms_norm(q.data_f32(), gq.data_f32(), 1e-6f, T * H, D, qn.data());
  orc_cpu_rope(qn.data(), pos.data(), 1e6f, T, H, D, qr.data());
  Tensor fq(DType::F32, {T, H, D}, DeviceType::CUDA), fk(DType::F32, {T, H, D}, DeviceType::CUDA);
  cuda_qk_norm_rope_out(cuda(q), cuda(kk), cuda(gq), cuda(gq), pos_cuda, 1e-6f, 1e6f, fq, fk);
  metric("cuda_qk_norm_rope_out q f32", fq, qr, 1e-4f);
  metric("cuda_qk_norm_rope_out k f32", fk, qr, 1e-4f);

  Tensor sm = Tensor::from_f32({2, 4}, {1000, 1001, -1000, -999, 1, 2, 3, 4});
  std::vector<float> sm_want(8);
  orc_cpu_softmax(sm.data_f32(), 2, 4, sm_want.data());
  metric("cuda_softmax_last_dim_f32", cuda_softmax_last_dim(cuda(sm)), sm_want, 1e-4f);
  Tensor sm16 = half_of(sm), sm16f = widen(sm16);
  orc_cpu_softmax(sm16f.data_f32(), 2, 4, sm_want.data());
  Tensor sm16_out = cuda_softmax_last_dim(cuda(sm16));
  metric("cuda_softmax_last_dim_f16", sm16_out, sm_want, 5e-3f);
  const std::vector<float> probs = values(sm16_out);
  for (int row = 0; row < 2; ++row)
    if (std::fabs(probs[row * 4] + probs[row * 4 + 1] + probs[row * 4 + 2] + probs[row * 4 + 3] - 1.0f) > 5e-3f) fail("softmax row sum");

  expect_throw("cuda_rms_norm dtype mismatch", [&] { cuda_rms_norm(cuda(x), cuda(w16), 1e-5f); });
  expect_throw("cuda_rms_norm epsilon", [&] { cuda_rms_norm(cuda(x), cuda(w), 0); });
  expect_throw("cuda_rms_norm shape", [&] { cuda_rms_norm(cuda(x), Tensor(DType::F32, {5}, DeviceType::CUDA), 1e-5f); });
  expect_throw("cuda_rms_norm CPU input", [&] { cuda_rms_norm(x, w, 1e-5f); });
  expect_throw("cuda_add shape", [&] { cuda_add(cuda(x), cuda(w)); });
  expect_throw("cuda_add_out wrong output", [&] { Tensor o(DType::F32, {4, 3}, DeviceType::CUDA); cuda_add_out(cuda(x), cuda(x), o); });
  expect_throw("cuda_rope invalid theta", [&] { cuda_rope(cuda(rope_x), positions, 0); });
  expect_throw("cuda_rope positions mismatch", [&] { cuda_rope(cuda(rope_x), {0}, 10000); });
  expect_throw("cuda_rope_token_positions F32-typed positions", [&] { cuda_rope_token_positions_out(q_cuda, pos_f32.to(DeviceType::CUDA), 1e6f, q_out); });
  for (int i = 0; i < 100; ++i) { auto tmp = cuda_rope(cuda(rope_x), positions, 10000); CUDA_CHECK(cudaDeviceSynchronize()); }
}

static void argmax_cases() {
  auto expect = [](const std::string& name, const Tensor& logits, int32_t want) {
    const int32_t got = cuda_argmax_last_row(cuda(logits));
    std::cout << name << " dtype=" << dtype_name(logits.dtype()) << " argmax=" << got << " expected=" << want << "\n";
    if (got != want) fail(name);
  };
  expect("f32_normal", Tensor::from_f32({2, 5}, {-1, 2, 3, 4, 5, 1, 9, 2, 8, 3}), 1);
  expect("f16_normal", half_of(Tensor::from_f32({2, 5}, {-1, 2, 3, 4, 5, 1, 9, 2, 8, 3})), 1);
  expect("f32_tie_min_id", Tensor::from_f32({1, 6}, {4, 7, 7, 1, 7, 2}), 1);
  expect("f16_negative", half_of(Tensor::from_f32({1, 4}, {-1, -2, -3, -4})), 0);
  std::vector<float> two_rows(2 * 151936, -10.0f);
  two_rows[11] = 100.0f; two_rows[151936 + 12345] = 101.0f;
  expect("f32_large_vocab", Tensor::from_f32({2, 151936}, two_rows), 12345);
  std::vector<float> large(151936, -10.0f);
  large[11] = 100.0f; large[12345] = 101.0f; large[151935] = 101.0f;
  expect("f16_large_vocab_tie", half_of(Tensor::from_f32({1, 151936}, large)), 12345);
  // every row at once, on the device
  Tensor many = Tensor::from_f32({2, 151936}, two_rows);
  Tensor ids(DType::I32, {2}, DeviceType::CUDA);
  cuda_argmax_rows_out(cuda(many), ids);
  Tensor host_ids = ids.to(DeviceType::CPU);
  if (host_ids.data_i32()[0] != orc_argmax_row_f32(two_rows.data(), 151936) || host_ids.data_i32()[1] != 12345) fail("cuda_argmax_rows_out");
  expect_throw("argmax CPU input", [&] { cuda_argmax_last_row(Tensor::from_f32({1, 2}, {1, 2})); });
  expect_throw("argmax rank mismatch", [&] { cuda_argmax_last_row(Tensor(DType::F32, {2, 2, 1}, DeviceType::CUDA)); });
  expect_throw("argmax BF16 input", [&] { cuda_argmax_last_row(Tensor(DType::BF16, {1, 2}, DeviceType::CUDA)); });
  expect_throw("argmax zero shape", [&] { cuda_argmax_last_row(Tensor(DType::F32, {0, 2}, DeviceType::CUDA)); });
  expect_throw("argmax empty shape", [&] { cuda_argmax_last_row(Tensor(DType::F32, {}, DeviceType::CUDA)); });
}

// Decode-size LM head + greedy pick against the CPU operator lm_head = linear (reference src/ops_cpu.cpp:9,17;
// known answer of reference tests/test_ops_cpu.cpp:14) followed by the arg-max rule.
static void lm_head_argmax_cases() {
  Tensor w = Tensor::from_f32({3, 2}, {1, 2, 3, 4, 5, 6}), x = Tensor::from_f32({1, 2}, {2, 3});
  Tensor ids(DType::I32, {1}, DeviceType::CUDA), logits(DType::F32, {1, 3}, DeviceType::CUDA);
  cuda_lm_head_argmax_out(cuda(x), cuda(w), ids, &logits);
  metric("cuda_lm_head_argmax logits [1,2]x[3,2]", logits, {8, 18, 28}, 0);
  if (ids.to(DeviceType::CPU).data_i32()[0] != 2) fail("cuda_lm_head_argmax known answer");
  const int rows = 3, hidden = 1024, vocab = 777;
  std::vector<float> h(size_t(rows) * hidden), t(size_t(vocab) * hidden), want(size_t(rows) * vocab);
  uint32_t state = 12345u;
  auto next = [&] { state = state * 1664525u + 1013904223u; return float(int32_t(state >> 8) % 2001 - 1000) / 1000.0f; };
  for (auto& v : h) v = next();
  for (auto& v : t) v = 0.02f * next();
  for (const bool f16 : {false, true}) {
    Tensor ht = Tensor::from_f32({rows, hidden}, h), tt = Tensor::from_f32({vocab, hidden}, t);
    if (f16) { ht = half_of(ht); tt = half_of(tt); }
    const Tensor hw = f16 ? widen(ht) : ht, tw = f16 ? widen(tt) : tt;
    orc_cpu_linear(hw.data_f32(), tw.data_f32(), rows, hidden, vocab, want.data());
    Tensor out_ids(DType::I32, {rows}, DeviceType::CUDA), out_logits(ht.dtype(), {rows, vocab}, DeviceType::CUDA);
    {
      CudaReductionModeGuard ordered(CudaReductionMode::kDeterministic);
      cuda_lm_head_argmax_out(cuda(ht), cuda(tt), out_ids, &out_logits);
    }
    metric(std::string("cuda_lm_head_argmax deterministic ") + (f16 ? "f16" : "f32"), out_logits, want, f16 ? 2e-3f : 0.0f);
    Tensor got = out_ids.to(DeviceType::CPU);
    Tensor stored = f16 ? widen(out_logits.to(DeviceType::CPU)) : out_logits.to(DeviceType::CPU);
    for (int r = 0; r < rows; ++r)
      if (got.data_i32()[r] != orc_argmax_row_f32(stored.data_f32() + size_t(r) * vocab, vocab)) fail("cuda_lm_head_argmax ids");
    Tensor fast_ids(DType::I32, {rows}, DeviceType::CUDA);
    cuda_lm_head_argmax_out(cuda(ht), cuda(tt), fast_ids, &out_logits);
    metric(std::string("cuda_lm_head_argmax fast ") + (f16 ? "f16" : "f32"), out_logits, want, f16 ? 2e-3f : 1e-5f);
  }
  expect_throw("lm_head CPU input", [&] { cuda_lm_head_argmax_out(x, cuda(w), ids); });
  expect_throw("lm_head hidden_size mismatch", [&] { cuda_lm_head_argmax_out(cuda(Tensor::from_f32({1, 3}, {1, 2, 3})), cuda(w), ids); });
  expect_throw("lm_head dtype mismatch", [&] { cuda_lm_head_argmax_out(cuda(half_of(x)), cuda(w), ids); });
  expect_throw("lm_head rank", [&] { cuda_lm_head_argmax_out(cuda(Tensor::from_f32({2}, {2, 3})), cuda(w), ids); });
  Tensor two(DType::I32, {2}, DeviceType::CUDA);
  expect_throw("lm_head ids shape", [&] { cuda_lm_head_argmax_out(cuda(x), cuda(w), two); });
}

static void embedding_cases() {
  const int vocab = 7, hidden = 4;
  Tensor ew = Tensor::from_f32({vocab, hidden}, {.01f, .02f, .03f, .04f, .10f, .20f, .30f, .40f, -.10f, -.20f, -.30f, -.40f, .50f, .60f,
                                                 .70f, .80f, -.50f, -.60f, -.70f, -.80f, .90f, .80f, .70f, .60f, -.90f, -.80f, -.70f, -.60f});
  std::vector<int32_t> ids{0, 3, 6, 2};
  std::vector<float> want(16);
  orc_cpu_embedding_lookup(ew.data_f32(), vocab, hidden, ids.data(), 4, want.data());
  Tensor ew_cuda = cuda(ew);
  metric("cuda_embedding_lookup_f32", cuda_embedding_lookup(ew_cuda, ids), want, 0);          // exact
  Tensor ew16 = half_of(ew), ew16f = widen(ew16);
  orc_cpu_embedding_lookup(ew16f.data_f32(), vocab, hidden, ids.data(), 4, want.data());
  metric("cuda_embedding_lookup_f16", cuda_embedding_lookup(cuda(ew16), ids), want, 0);
  // device-id form: ids travel in an F32-typed tensor (src/ops_cuda.cu:875)
  Tensor ids_f32(DType::F32, {4});
  std::memcpy(ids_f32.data(), ids.data(), 16);
  Tensor out(DType::F16, {4, hidden}, DeviceType::CUDA);
  cuda_embedding_lookup_device_ids_out(cuda(ew16), ids_f32.to(DeviceType::CUDA), out);
  metric("cuda_embedding_lookup_device_ids_out f16", out, want, 0);
  expect_throw("embedding CPU weight", [&] { cuda_embedding_lookup(ew, ids); });
  expect_throw("embedding rank", [&] { cuda_embedding_lookup(Tensor(DType::F32, {vocab, hidden, 1}, DeviceType::CUDA), ids); });
  expect_throw("embedding negative token", [&] { cuda_embedding_lookup(ew_cuda, {-1}); });
  expect_throw("embedding token out of range", [&] { cuda_embedding_lookup(ew_cuda, {vocab}); });
  expect_throw("embedding empty ids", [&] { cuda_embedding_lookup(ew_cuda, {}); });
}

static void tensor_and_allocation_cases() {
  Tensor cpu = Tensor::from_f32({2, 5}, {0, -1.25f, 2.5f, 0, 9, -7, 3.125f, 0.5f, -2, 4});
  Tensor gpu = cpu.to(DeviceType::CUDA);
  if (gpu.device() != DeviceType::CUDA || gpu.shape() != cpu.shape() || gpu.strides() != cpu.strides() || gpu.nbytes() != cpu.nbytes())
    fail("F32 metadata");
  if (values(gpu) != values(cpu)) fail("F32 round trip");
  Tensor view = gpu.reshape({5, 2}), copy = view.to(DeviceType::CUDA);
  if (copy.storage_bytes() != gpu.storage_bytes()) fail("CUDA view/copy lifetime");
  expect_throw("BF16 CUDA rejection", [] { Tensor b(DType::BF16, {2}); b.to(DeviceType::CUDA); });
  expect_throw("CUDA host access rejection", [&] { gpu.get_f32(0); });

  reset_cuda_allocation_stats();
  const CudaAllocationStats at_reset = cuda_allocation_stats();
  if (at_reset.cuda_malloc_calls != 0 || at_reset.cuda_free_calls != 0) fail("reset did not clear the call counters");
  const uint64_t baseline = at_reset.cuda_live_bytes;
  {
    Tensor host(DType::F32, {16, 16});
    if (cuda_allocation_stats().cuda_malloc_calls != 0) fail("CPU tensor counted as a CUDA allocation");
    Tensor device(DType::F32, {1024, 4}, DeviceType::CUDA);
    const CudaAllocationStats s = cuda_allocation_stats();
    if (s.cuda_malloc_calls != 1 || s.cuda_live_bytes != baseline + device.nbytes() || s.cuda_allocated_bytes_total != device.nbytes() ||
        s.cuda_peak_live_bytes < s.cuda_live_bytes)
      fail("allocation counters after one CUDA tensor");
    // an *_out operator allocates nothing
    Tensor o(DType::F32, {1024, 4}, DeviceType::CUDA);
    const uint64_t before = cuda_allocation_stats().cuda_malloc_calls;
    cuda_add_out(device, device, o);
    if (cuda_allocation_stats().cuda_malloc_calls != before) fail("cuda_add_out allocated");
  }
  const CudaAllocationStats after = cuda_allocation_stats();
  if (after.cuda_free_calls != 2 || after.cuda_live_bytes != baseline) fail("live bytes did not return to the baseline");
}

int main() {
  try {
    cudaDeviceProp prop{};
    CUDA_CHECK(cudaGetDeviceProperties(&prop, 0));
    std::cout << "CUDA device=" << prop.name << " compute_capability=" << prop.major << "." << prop.minor << "\n";
    operators_against_oracle();
    argmax_cases();
    lm_head_argmax_cases();
    embedding_cases();
    tensor_and_allocation_cases();
    CUDA_CHECK(cudaDeviceSynchronize());
    std::cout << "test_ops_cuda_b200 passed\n";
    return 0;
  } catch (const std::exception& e) {
    std::cerr << e.what() << "\n";
    return 1;
  }
}
