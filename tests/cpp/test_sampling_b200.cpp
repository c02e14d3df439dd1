// GPU checks of llm::CudaSampler (the reference's interface, include/llm/ops_cuda.h:46-74) on this
// library's sampling kernels.  The cases are those of the reference's tests/test_sampling_cuda.cpp:18-70
// (same inputs, same expectations, same rejections); in addition every sampled token is compared with the
// CPU restatement of the reference's rule (oracle/oracle.c, orc_sample_row) unless that token hangs on the
// last bits of a running sum.
#include "llm/cuda_check.h"
#include "llm/ops_cuda.h"

#include <cmath>
#include <functional>
#include <iostream>
#include <stdexcept>
#include <string>
#include <vector>

using namespace llm;

extern "C" {   // the CPU oracle (test infrastructure)
int32_t orc_sample_row(const float*, int64_t, float, int32_t, float, uint64_t, uint64_t, double*);
uint16_t orc_f32_to_f16_rn(float);
}

static void fail(const std::string& s) { throw std::runtime_error("test_sampling_b200: " + s); }
static Tensor f16(const Tensor& x) {
  Tensor y(DType::F16, x.shape());
  for (size_t i = 0; i < x.numel(); ++i) y.data_f16()[i] = orc_f32_to_f16_rn(x.get_f32(i));
  return y;
}
static void reject(const std::string& n, const std::function<void()>& f) {
  try { f(); } catch (const std::exception& e) { std::cout << "rejected " << n << ": " << e.what() << "\n"; return; }
  fail(n + " was accepted");
}
static bool in(const std::vector<int32_t>& ids, int32_t x) { for (auto v : ids) if (v == x) return true; return false; }
// the sampled token must be the restatement's unless the decision is numerically ambiguous
static int32_t checked(CudaSampler& sampler, const Tensor& host_f32, const Tensor& device, const SamplingConfig& c, uint64_t offset) {
  const int32_t got = sampler.sample_last_row(device, c, offset);
  const size_t vocab = size_t(host_f32.shape().back()), last = (size_t(host_f32.shape()[0]) - 1) * vocab;
  std::vector<float> row(vocab);
  Tensor widened = device.to(DeviceType::CPU);
  for (size_t i = 0; i < vocab; ++i) row[i] = widened.get_f32(last + i);
  double margin = 0;
  const int32_t want = orc_sample_row(row.data(), int64_t(vocab), c.temperature, c.top_k, c.top_p, c.seed, offset, &margin);
  if (got != want && margin > 1e-5) fail("token " + std::to_string(got) + " differs from the restatement's " + std::to_string(want));
  return got;
}

int main() {
  try {
    cudaDeviceProp p{};
    CUDA_CHECK(cudaGetDeviceProperties(&p, 0));
    std::cout << "CUDA device=" << p.name << " compute_capability=" << p.major << "." << p.minor << "\n";
    CudaSampler sampler(151936);
    Tensor x = Tensor::from_f32({2, 6}, {-3, 1, 8, 2, 4, 0, 2, 9, 1, 7, 3, 5});
    auto xf = x.to(DeviceType::CUDA);
    auto x16 = f16(x).to(DeviceType::CUDA);
    SamplingConfig zero; zero.temperature = 0; zero.top_k = 0; zero.top_p = 0.0f;   // ignored at temperature zero
    if (sampler.sample_last_row(xf, zero, 0) != cuda_argmax_last_row(xf) || sampler.sample_last_row(x16, zero, 0) != cuda_argmax_last_row(x16))
      fail("temperature zero is not argmax");
    SamplingConfig one; one.temperature = 1; one.top_k = 1; one.top_p = 1;
    if (sampler.sample_last_row(xf, one, 0) != cuda_argmax_last_row(xf)) fail("top_k=1 is not greedy");
    SamplingConfig d; d.temperature = 1; d.top_k = 3; d.top_p = 1; d.seed = 42;
    if (checked(sampler, x, xf, d, 7) != checked(sampler, x, xf, d, 7)) fail("same seed/offset is not deterministic");
    Tensor small_cpu = Tensor::from_f32({1, 6}, {10, 9, 0, -1, -2, -3});
    Tensor small = small_cpu.to(DeviceType::CUDA);
    SamplingConfig k2; k2.temperature = 1; k2.top_k = 2; k2.top_p = 1; k2.seed = 1;
    for (uint64_t i = 0; i < 20; ++i) if (!in({0, 1}, checked(sampler, small_cpu, small, k2, i))) fail("top_k boundary escaped");
    SamplingConfig combo; combo.temperature = 1; combo.top_k = 3; combo.top_p = .5f; combo.seed = 2;
    for (uint64_t i = 0; i < 20; ++i) if (!in({0, 1}, checked(sampler, small_cpu, small, combo, i))) fail("top_k/top_p combination escaped");
    Tensor crossing_cpu = Tensor::from_f32({1, 6}, {std::log(0.505f), std::log(0.495f), -20.f, -20.f, -20.f, -20.f});
    SamplingConfig crossing_cfg; crossing_cfg.temperature = 1.f; crossing_cfg.top_k = 0; crossing_cfg.top_p = .51f; crossing_cfg.seed = 77;
    for (const Tensor& t : {crossing_cpu.to(DeviceType::CUDA), f16(crossing_cpu).to(DeviceType::CUDA)}) {
      bool saw = false;
      for (uint64_t offset = 0; offset < 64; ++offset) {
        const int32_t id = checked(sampler, crossing_cpu, t, crossing_cfg, offset);
        if (id != 0 && id != 1) fail("top-p crossing selected a truncated token");
        if (id == 1) saw = true;
      }
      if (!saw) fail("top-p crossing token was never sampled");
    }
    std::cout << "top-p crossing: retained tokens={0,1}, crossing token observed (F32 and F16)\n";
    Tensor ties_cpu = Tensor::from_f32({1, 6}, {0.f, 0.f, 0.f, -10.f, -10.f, -10.f});
    SamplingConfig tie_cfg; tie_cfg.temperature = 1.f; tie_cfg.top_k = 0; tie_cfg.top_p = .30f; tie_cfg.seed = 88;
    for (const Tensor& t : {ties_cpu.to(DeviceType::CUDA), f16(ties_cpu).to(DeviceType::CUDA)})
      for (uint64_t offset = 0; offset < 64; ++offset)
        if (checked(sampler, ties_cpu, t, tie_cfg, offset) != 0) fail("tie-order did not prefer lowest token ID");
    std::cout << "tie-order: F32/F16 equal maxima always selected token 0\n";
    std::vector<float> large(151936, -2);
    large[123456] = 8;
    Tensor large_cpu = Tensor::from_f32({1, 151936}, large);
    Tensor lv = large_cpu.to(DeviceType::CUDA);
    if (sampler.sample_last_row(lv, zero, 0) != 123456 || sampler.sample_last_row(f16(large_cpu).to(DeviceType::CUDA), zero, 0) != 123456)
      fail("large vocab argmax failed");
    SamplingConfig wide; wide.temperature = 1.5f; wide.top_k = 0; wide.top_p = .9f; wide.seed = 5;
    for (uint64_t offset = 0; offset < 4; ++offset) checked(sampler, large_cpu, lv, wide, offset);   // whole-vocabulary sort path
    wide.top_k = 40;
    for (uint64_t offset = 0; offset < 4; ++offset) checked(sampler, large_cpu, lv, wide, offset);   // top-k select path
    // rank-2 rows and rank-3 last tokens
    Tensor b3 = Tensor::from_f32({2, 2, 3}, {0, 1, 2, 9, 1, 0, 3, 2, 1, 0, 0, 7}).to(DeviceType::CUDA);
    if (sampler.sample_last_token_of_batch(b3, 0, zero, 0) != 0 || sampler.sample_last_token_of_batch(b3, 1, zero, 0) != 2) fail("last token of batch");
    if (sampler.sample_row(xf, 0, zero, 0) != 2 || sampler.sample_row(xf, 1, zero, 0) != 1) fail("sample_row");
    reject("CPU", [&] { sampler.sample_last_row(x, one, 0); });
    reject("rank", [&] { sampler.sample_last_row(Tensor(DType::F32, {1, 2, 1}, DeviceType::CUDA), one, 0); });
    reject("BF16", [&] { sampler.sample_last_row(Tensor(DType::BF16, {1, 2}, DeviceType::CUDA), one, 0); });
    reject("zero shape", [&] { sampler.sample_last_row(Tensor(DType::F32, {0, 2}, DeviceType::CUDA), one, 0); });
    SamplingConfig bad = one; bad.temperature = -1; reject("negative temperature", [&] { sampler.sample_last_row(xf, bad, 0); });
    bad = one; bad.top_k = 7; reject("top_k too large", [&] { sampler.sample_last_row(xf, bad, 0); });
    bad = one; bad.top_p = 0; reject("top_p zero", [&] { sampler.sample_last_row(xf, bad, 0); });
    reject("batch index", [&] { sampler.sample_row(xf, 2, one, 0); });
    CUDA_CHECK(cudaDeviceSynchronize());
    std::cout << "test_sampling_b200 passed\n";
    return 0;
  } catch (const std::exception& e) { std::cerr << e.what() << "\n"; return 1; }
}
