// GPU checks of llm::CudaSampler (the reference's interface, include/llm/ops_cuda.h:46-74) on this
// library's sampling kernels.  The scenarios are those the reference's tests/test_sampling_cuda.cpp:18-70
// pins (greedy at temperature zero, top_k = 1, determinism, the top-k and top-p boundaries, the top-p
// crossing token, the tie order, a full-size vocabulary, and the rejections), written here as a table of
// scenarios; on top of that every sampled token is compared with the CPU restatement of the reference's
// rule (oracle/oracle.c, orc_sample_row) unless the decision hangs on the last bits of a running sum.
#include "llm/cuda_check.h"
#include "llm/ops_cuda.h"

#include <cmath>
#include <functional>
#include <iostream>
#include <set>
#include <stdexcept>
#include <string>
#include <vector>

using namespace llm;

extern "C" {   // the CPU oracle (test infrastructure)
int32_t orc_sample_row(const float*, int64_t, float, int32_t, float, uint64_t, uint64_t, double*);
uint16_t orc_f32_to_f16_rn(float);
}

namespace {

[[noreturn]] void fail(const std::string& what) { throw std::runtime_error("test_sampling_b200: " + what); }

Tensor as_half(const Tensor& x) {
  Tensor y(DType::F16, x.shape());
  for (size_t i = 0; i < x.numel(); ++i) y.data_f16()[i] = orc_f32_to_f16_rn(x.get_f32(i));
  return y;
}

SamplingConfig config(float temperature, int32_t top_k, float top_p, uint64_t seed = 0) {
  SamplingConfig c;
  c.temperature = temperature;
  c.top_k = top_k;
  c.top_p = top_p;
  c.seed = seed;
  return c;
}

// One draw from the last row of `device`, cross-checked against the restatement run on the same values.
int32_t draw(CudaSampler& sampler, const Tensor& device, const SamplingConfig& c, uint64_t offset) {
  const int32_t got = sampler.sample_last_row(device, c, offset);
  if (c.temperature == 0.0f) return got;
  const Tensor host = device.to(DeviceType::CPU);
  const size_t vocab = size_t(host.shape().back()), start = host.numel() - vocab;
  std::vector<float> row(vocab);
  for (size_t i = 0; i < vocab; ++i) row[i] = host.get_f32(start + i);
  double margin = 0;
  const int32_t want = orc_sample_row(row.data(), int64_t(vocab), c.temperature, c.top_k, c.top_p, c.seed, offset, &margin);
  if (got != want && margin > 1e-5)
    fail("token " + std::to_string(got) + " differs from the restatement's " + std::to_string(want));
  return got;
}

// Draws `draws` tokens (offsets 0, 1, ...) from both the F32 and the F16 form of `logits`; every token must lie in
// `allowed`, and every token of `must_see` must turn up at least once per dtype.
struct Scenario {
  std::string name;
  std::vector<float> logits;
  SamplingConfig cfg;
  int draws;
  std::set<int32_t> allowed, must_see;
};

void run(CudaSampler& sampler, const Scenario& s) {
  const Tensor cpu = Tensor::from_f32({1, int64_t(s.logits.size())}, s.logits);
  for (const bool half : {false, true}) {
    const Tensor device = (half ? as_half(cpu) : cpu).to(DeviceType::CUDA);
    std::set<int32_t> seen;
    for (int offset = 0; offset < s.draws; ++offset) {
      const int32_t id = draw(sampler, device, s.cfg, uint64_t(offset));
      if (!s.allowed.count(id)) fail(s.name + (half ? " (F16)" : " (F32)") + ": token " + std::to_string(id) + " escaped");
      seen.insert(id);
    }
    for (int32_t id : s.must_see)
      if (!seen.count(id)) fail(s.name + (half ? " (F16)" : " (F32)") + ": token " + std::to_string(id) + " never sampled");
  }
  std::cout << s.name << ": ok (F32 and F16, " << s.draws << " draws each)\n";
}

void must_throw(const std::string& name, const std::function<void()>& call) {
  try { call(); } catch (const std::exception& e) { std::cout << "rejected " << name << ": " << e.what() << "\n"; return; }
  fail(name + " was accepted");
}

}  // namespace

int main() {
  try {
    cudaDeviceProp prop{};
    CUDA_CHECK(cudaGetDeviceProperties(&prop, 0));
    std::cout << "CUDA device=" << prop.name << " compute_capability=" << prop.major << "." << prop.minor << "\n";
    CudaSampler sampler(151936);

    // greedy routes
    const Tensor two_rows = Tensor::from_f32({2, 6}, {-3, 1, 8, 2, 4, 0, 2, 9, 1, 7, 3, 5});
    const Tensor two_f32 = two_rows.to(DeviceType::CUDA), two_f16 = as_half(two_rows).to(DeviceType::CUDA);
    const SamplingConfig greedy = config(0, 0, 0.0f);          // top_k / top_p are ignored at temperature zero
    const SamplingConfig top1 = config(1, 1, 1);
    for (const Tensor* t : {&two_f32, &two_f16})
      if (sampler.sample_last_row(*t, greedy, 0) != cuda_argmax_last_row(*t)) fail("temperature zero is not argmax");
    if (draw(sampler, two_f32, top1, 0) != cuda_argmax_last_row(two_f32)) fail("top_k = 1 is not greedy");
    if (sampler.sample_row(two_f32, 0, greedy, 0) != 2 || sampler.sample_row(two_f32, 1, greedy, 0) != 1) fail("sample_row");
    const Tensor batch = Tensor::from_f32({2, 2, 3}, {0, 1, 2, 9, 1, 0, 3, 2, 1, 0, 0, 7}).to(DeviceType::CUDA);
    if (sampler.sample_last_token_of_batch(batch, 0, greedy, 0) != 0 || sampler.sample_last_token_of_batch(batch, 1, greedy, 0) != 2)
      fail("sample_last_token_of_batch");
    const SamplingConfig seeded = config(1, 3, 1, 42);
    if (draw(sampler, two_f32, seeded, 7) != draw(sampler, two_f32, seeded, 7)) fail("same seed and offset, different tokens");

    // boundaries
    const float lo = std::log(0.495f), hi = std::log(0.505f);
    const std::vector<Scenario> scenarios = {
        {"top_k boundary", {10, 9, 0, -1, -2, -3}, config(1, 2, 1, 1), 20, {0, 1}, {}},
        {"top_k with top_p", {10, 9, 0, -1, -2, -3}, config(1, 3, 0.5f, 2), 20, {0, 1}, {}},
        {"top_p crossing token", {hi, lo, -20, -20, -20, -20}, config(1, 0, 0.51f, 77), 64, {0, 1}, {1}},
        {"equal maxima, lowest id first", {0, 0, 0, -10, -10, -10}, config(1, 0, 0.30f, 88), 64, {0}, {0}},
    };
    for (const Scenario& s : scenarios) run(sampler, s);

    // a vocabulary-sized row: greedy, the whole-row sort (top_k = 0) and the two-pass top-k path
    std::vector<float> spike(151936, -2.0f);
    spike[123456] = 8.0f;
    const Tensor spike_cpu = Tensor::from_f32({1, 151936}, spike);
    const Tensor spike_f32 = spike_cpu.to(DeviceType::CUDA), spike_f16 = as_half(spike_cpu).to(DeviceType::CUDA);
    if (sampler.sample_last_row(spike_f32, greedy, 0) != 123456 || sampler.sample_last_row(spike_f16, greedy, 0) != 123456)
      fail("large vocabulary argmax");
    for (const int32_t k : {0, 40})
      for (uint64_t offset = 0; offset < 4; ++offset) draw(sampler, spike_f32, config(1.5f, k, 0.9f, 5), offset);

    // rejections
    must_throw("CPU logits", [&] { sampler.sample_last_row(two_rows, top1, 0); });
    must_throw("rank 3 for sample_last_row", [&] { sampler.sample_last_row(Tensor(DType::F32, {1, 2, 1}, DeviceType::CUDA), top1, 0); });
    must_throw("BF16 logits", [&] { sampler.sample_last_row(Tensor(DType::BF16, {1, 2}, DeviceType::CUDA), top1, 0); });
    must_throw("no rows", [&] { sampler.sample_last_row(Tensor(DType::F32, {0, 2}, DeviceType::CUDA), top1, 0); });
    must_throw("negative temperature", [&] { sampler.sample_last_row(two_f32, config(-1, 1, 1), 0); });
    must_throw("top_k above the vocabulary", [&] { sampler.sample_last_row(two_f32, config(1, 7, 1), 0); });
    must_throw("top_p zero", [&] { sampler.sample_last_row(two_f32, config(1, 1, 0), 0); });
    must_throw("row index past the batch", [&] { sampler.sample_row(two_f32, 2, top1, 0); });
    must_throw("vocabulary above the sampler's capacity", [&] { CudaSampler small(4); small.sample_last_row(two_f32, top1, 0); });
    CUDA_CHECK(cudaDeviceSynchronize());
    std::cout << "test_sampling_b200 passed\n";
    return 0;
  } catch (const std::exception& e) {
    std::cerr << e.what() << "\n";
    return 1;
  }
}
