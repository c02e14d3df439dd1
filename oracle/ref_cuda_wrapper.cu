// extern "C" doors into the reference's own, unmodified CUDA operators (reference
// include/llm/ops_cuda.h, src/ops_cuda.cu, src/tensor_cuda.cu), recompiled for sm_100a by
// oracle/Makefile from the reference tree where it lies.  TEST INFRASTRUCTURE ONLY: the tests use
// it as a second oracle (the deterministic mode must reproduce these kernels bit for bit) and the
// per-operator bench reports its timings beside ours.  Callers pass DEVICE pointers; each door
// copies them into reference Tensors, runs the reference operator and copies the result back.
#include "llm/cuda_check.h"
#include "llm/ops_cuda.h"

#include <cstring>
#include <exception>
#include <vector>

#define REFCU_API extern "C" __attribute__((visibility("default")))

namespace {
using llm::DeviceType;
using llm::DType;
using llm::Tensor;

DType dtype_of(int code) { return code == 0 ? DType::F32 : DType::F16; }

Tensor from_device(const void* p, DType d, std::vector<int64_t> shape) {
  Tensor t(d, std::move(shape), DeviceType::CUDA);
  CUDA_CHECK(cudaMemcpy(t.data(), p, t.nbytes(), cudaMemcpyDeviceToDevice));
  return t;
}
void to_device(const Tensor& t, void* p) {
  CUDA_CHECK(cudaMemcpy(p, t.data(), t.nbytes(), cudaMemcpyDeviceToDevice));
  CUDA_CHECK(cudaDeviceSynchronize());
}
// Every door first waits for the device: the reference runs on the per-thread default stream, which does not
// order itself after a caller's non-blocking stream, and its kernels trust what they read (the embedding kernel
// dereferences any id), so inputs still being written by the caller must have landed before they are copied.
template <class F> int guarded(F&& f) {
  try {
    CUDA_CHECK(cudaDeviceSynchronize());
    f();
    return 0;
  } catch (const std::invalid_argument&) { return -1; } catch (const std::exception&) { return -2; }
}
// milliseconds per call of `f`, CUDA events on the per-thread default stream (where the reference launches)
template <class F> float timed(F&& f, int reps) {
  cudaEvent_t a, b;
  CUDA_CHECK(cudaEventCreate(&a));
  CUDA_CHECK(cudaEventCreate(&b));
  f();
  CUDA_CHECK(cudaDeviceSynchronize());
  CUDA_CHECK(cudaEventRecord(a, cudaStreamPerThread));
  for (int i = 0; i < reps; ++i) f();
  CUDA_CHECK(cudaEventRecord(b, cudaStreamPerThread));
  CUDA_CHECK(cudaEventSynchronize(b));
  float ms = 0;
  CUDA_CHECK(cudaEventElapsedTime(&ms, a, b));
  cudaEventDestroy(a);
  cudaEventDestroy(b);
  return ms / float(reps);
}
}  // namespace

REFCU_API int refcu_rms_norm(const void* x, const void* w, void* out, int64_t rows, int64_t hidden, float eps, int dtype) {
  return guarded([&] {
    const DType d = dtype_of(dtype);
    to_device(llm::cuda_rms_norm(from_device(x, d, {rows, hidden}), from_device(w, d, {hidden}), eps), out);
  });
}

REFCU_API int refcu_add_rms_norm(const void* lhs, const void* rhs, const void* w, void* residual, void* normalized,
                                 int64_t rows, int64_t hidden, float eps, int dtype) {
  return guarded([&] {
    const DType d = dtype_of(dtype);
    Tensor res(d, {rows, hidden}, DeviceType::CUDA), nrm(d, {rows, hidden}, DeviceType::CUDA);
    llm::cuda_add_rms_norm_out(from_device(lhs, d, {rows, hidden}), from_device(rhs, d, {rows, hidden}),
                               from_device(w, d, {hidden}), eps, res, nrm);
    to_device(res, residual);
    to_device(nrm, normalized);
  });
}

REFCU_API int refcu_add(const void* a, const void* b, void* out, int64_t n, int dtype) {
  return guarded([&] { const DType d = dtype_of(dtype); to_device(llm::cuda_add(from_device(a, d, {n}), from_device(b, d, {n})), out); });
}

REFCU_API int refcu_swiglu(const void* g, const void* u, void* out, int64_t n, int dtype) {
  return guarded([&] { const DType d = dtype_of(dtype); to_device(llm::cuda_swiglu(from_device(g, d, {n}), from_device(u, d, {n})), out); });
}

// positions: HOST int32[tokens] (the reference's cuda_rope copies them to the device itself)
REFCU_API int refcu_rope(const void* x, const int32_t* positions, void* out, int64_t tokens, int64_t heads, int64_t head_dim,
                         float theta, int dtype) {
  return guarded([&] {
    std::vector<int32_t> p(positions, positions + tokens);
    to_device(llm::cuda_rope(from_device(x, dtype_of(dtype), {tokens, heads, head_dim}), p, theta), out);
  });
}

// positions: DEVICE int32[tokens]; fp16, heads in {16, 8}, head_dim 128 only (the reference's own restriction)
REFCU_API int refcu_rope_token_positions(const void* x, const int32_t* positions_device, void* out, int64_t tokens,
                                         int64_t heads, float theta) {
  return guarded([&] {
    Tensor pos(DType::I32, {tokens}, DeviceType::CUDA);
    CUDA_CHECK(cudaMemcpy(pos.data(), positions_device, size_t(tokens) * 4, cudaMemcpyDeviceToDevice));
    Tensor o(DType::F16, {tokens, heads, 128}, DeviceType::CUDA);
    llm::cuda_rope_token_positions_out(from_device(x, DType::F16, {tokens, heads, 128}), pos, theta, o);
    to_device(o, out);
  });
}

REFCU_API int refcu_softmax(const void* x, void* out, int64_t rows, int64_t width, int dtype) {
  return guarded([&] { to_device(llm::cuda_softmax_last_dim(from_device(x, dtype_of(dtype), {rows, width})), out); });
}

// ids: HOST int32[count], bounds-checked by the reference on the host
REFCU_API int refcu_embedding_lookup(const void* table, const int32_t* ids, void* out, int64_t count, int64_t hidden,
                                     int64_t vocab, int dtype) {
  return guarded([&] {
    std::vector<int32_t> v(ids, ids + count);
    to_device(llm::cuda_embedding_lookup(from_device(table, dtype_of(dtype), {vocab, hidden}), v), out);
  });
}

REFCU_API int refcu_argmax_last_row(const void* logits, int64_t rows, int64_t width, int dtype, int32_t* result_host) {
  return guarded([&] { *result_host = llm::cuda_argmax_last_row(from_device(logits, dtype_of(dtype), {rows, width})); });
}

// The decode tail of the reference: cuda_lm_head (a library GEMM into a fresh logits tensor) followed by
// cuda_argmax_last_row (reference src/ops_cuda.cu:885,871; src/qwen3_cuda_model.cpp:1070-1071,1339).
REFCU_API int refcu_lm_head_argmax(const void* hidden, const void* table, int64_t rows, int64_t hidden_size, int64_t vocab,
                                   int dtype, void* logits_out, int32_t* last_row_id_host) {
  return guarded([&] {
    const DType d = dtype_of(dtype);
    Tensor logits = llm::cuda_lm_head(from_device(hidden, d, {rows, hidden_size}), from_device(table, d, {vocab, hidden_size}));
    if (logits_out != nullptr) to_device(logits, logits_out);
    *last_row_id_host = llm::cuda_argmax_last_row(logits);
  });
}

// ---- timings of the reference kernels on tensors already on the device (copies excluded); ms per call, < 0 on error
REFCU_API float refcu_time_add_rms_norm(const void* lhs, const void* rhs, const void* w, int64_t rows, int64_t hidden, float eps,
                                        int dtype, int reps) {
  float ms = -1;
  guarded([&] {
    const DType d = dtype_of(dtype);
    Tensor a = from_device(lhs, d, {rows, hidden}), b = from_device(rhs, d, {rows, hidden}), g = from_device(w, d, {hidden});
    Tensor res(d, {rows, hidden}, DeviceType::CUDA), nrm(d, {rows, hidden}, DeviceType::CUDA);
    ms = timed([&] { llm::cuda_add_rms_norm_out(a, b, g, eps, res, nrm); }, reps);
  });
  return ms;
}
REFCU_API float refcu_time_rms_norm(const void* x, const void* w, int64_t rows, int64_t hidden, float eps, int dtype, int reps) {
  float ms = -1;
  guarded([&] {
    const DType d = dtype_of(dtype);
    Tensor a = from_device(x, d, {rows, hidden}), g = from_device(w, d, {hidden}), o(d, {rows, hidden}, DeviceType::CUDA);
    ms = timed([&] { llm::cuda_rms_norm_out(a, g, eps, o); }, reps);
  });
  return ms;
}
REFCU_API float refcu_time_binary(const void* a_, const void* b_, int64_t n, int dtype, int swiglu, int reps) {
  float ms = -1;
  guarded([&] {
    const DType d = dtype_of(dtype);
    Tensor a = from_device(a_, d, {n}), b = from_device(b_, d, {n}), o(d, {n}, DeviceType::CUDA);
    ms = timed([&] { if (swiglu) llm::cuda_swiglu_out(a, b, o); else llm::cuda_add_out(a, b, o); }, reps);
  });
  return ms;
}
REFCU_API float refcu_time_rope_token_positions(const void* x, const int32_t* positions_device, int64_t tokens, int64_t heads,
                                                float theta, int reps) {
  float ms = -1;
  guarded([&] {
    Tensor pos(DType::I32, {tokens}, DeviceType::CUDA);
    CUDA_CHECK(cudaMemcpy(pos.data(), positions_device, size_t(tokens) * 4, cudaMemcpyDeviceToDevice));
    Tensor a = from_device(x, DType::F16, {tokens, heads, 128}), o(DType::F16, {tokens, heads, 128}, DeviceType::CUDA);
    ms = timed([&] { llm::cuda_rope_token_positions_out(a, pos, theta, o); }, reps);
  });
  return ms;
}
// The in-scope operators of one decoder layer of a decode step, in the order the reference's layer launches them
// (src/qwen3_layer_cuda.cu:285-292,319-325): add + norm, the two per-head norms, the two rotary embeddings, add + norm,
// SwiGLU, add; Qwen3-0.6B shapes (hidden 1024, 16 + 8 heads of 128, intermediate 3072), fp16, `tokens` rows.  The
// projections and the attention between them are left out (not on this path), so the operators run back to back.
// graph != 0: the chain is captured once into a CUDA graph and the replays are timed.  Milliseconds per chain.
REFCU_API float refcu_time_decode_chain(int64_t tokens, float eps, float theta, int graph, int reps) {
  float ms = -1;
  guarded([&] {
    const DType d = DType::F16;
    auto zeros = [&](std::vector<int64_t> shape) {
      Tensor t(d, std::move(shape), DeviceType::CUDA);
      CUDA_CHECK(cudaMemset(t.data(), 0, t.nbytes()));
      return t;
    };
    Tensor x = zeros({tokens, 1024}), r = zeros({tokens, 1024}), g = zeros({1024}), res = zeros({tokens, 1024}), nrm = zeros({tokens, 1024});
    Tensor q = zeros({tokens, 16, 128}), k = zeros({tokens, 8, 128}), g128 = zeros({128}), qn = zeros({tokens, 16, 128}),
           kn = zeros({tokens, 8, 128}), qo = zeros({tokens, 16, 128}), ko = zeros({tokens, 8, 128});
    Tensor gate = zeros({tokens, 3072}), up = zeros({tokens, 3072}), act = zeros({tokens, 3072}), out = zeros({tokens, 1024});
    Tensor pos(DType::I32, {tokens}, DeviceType::CUDA);
    CUDA_CHECK(cudaMemset(pos.data(), 0, size_t(tokens) * 4));
    cudaStream_t s = cudaStreamPerThread;
    auto chain = [&] {
      llm::cuda_add_rms_norm_out(x, r, g, eps, res, nrm, s);
      llm::cuda_rms_norm_out(q, g128, eps, qn, s);
      llm::cuda_rms_norm_out(k, g128, eps, kn, s);
      llm::cuda_rope_token_positions_out(qn, pos, theta, qo, s);
      llm::cuda_rope_token_positions_out(kn, pos, theta, ko, s);
      llm::cuda_add_rms_norm_out(res, nrm, g, eps, x, r, s);
      llm::cuda_swiglu_out(gate, up, act, s);
      llm::cuda_add_out(x, r, out, s);
    };
    if (!graph) {
      ms = timed(chain, reps);
    } else {
      chain();
      CUDA_CHECK(cudaDeviceSynchronize());
      cudaGraph_t captured;
      cudaGraphExec_t exec;
      CUDA_CHECK(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
      chain();
      CUDA_CHECK(cudaStreamEndCapture(s, &captured));
      CUDA_CHECK(cudaGraphInstantiate(&exec, captured, 0));
      ms = timed([&] { CUDA_CHECK(cudaGraphLaunch(exec, s)); }, reps);
      cudaGraphExecDestroy(exec);
      cudaGraphDestroy(captured);
    }
  });
  return ms;
}
REFCU_API float refcu_time_embedding(const void* table, const int32_t* ids_device, int64_t count, int64_t hidden, int64_t vocab,
                                     int dtype, int reps) {
  float ms = -1;
  guarded([&] {
    const DType d = dtype_of(dtype);
    Tensor w = from_device(table, d, {vocab, hidden}), o(d, {count, hidden}, DeviceType::CUDA);
    Tensor ids(DType::F32, {count}, DeviceType::CUDA);   // the reference types its id buffer F32 (src/ops_cuda.cu:875)
    CUDA_CHECK(cudaMemcpy(ids.data(), ids_device, size_t(count) * 4, cudaMemcpyDeviceToDevice));
    ms = timed([&] { llm::cuda_embedding_lookup_device_ids_out(w, ids, o); }, reps);
  });
  return ms;
}
REFCU_API float refcu_time_softmax(const void* x, int64_t rows, int64_t width, int dtype, int reps) {
  float ms = -1;
  guarded([&] {
    Tensor a = from_device(x, dtype_of(dtype), {rows, width});
    ms = timed([&] { Tensor o = llm::cuda_softmax_last_dim(a); }, reps);
  });
  return ms;
}
// one call of the reference = one row (its only public argmax reaches the last row; the sampler loops rows on the host)
REFCU_API float refcu_time_argmax_last_row(const void* logits, int64_t rows, int64_t width, int dtype, int reps) {
  float ms = -1;
  guarded([&] {
    Tensor a = from_device(logits, dtype_of(dtype), {rows, width});
    ms = timed([&] { (void)llm::cuda_argmax_last_row(a); }, reps);
  });
  return ms;
}

REFCU_API float refcu_time_lm_head_argmax(const void* hidden, const void* table, int64_t rows, int64_t hidden_size, int64_t vocab,
                                          int dtype, int reps) {
  float ms = -1;
  guarded([&] {
    const DType d = dtype_of(dtype);
    Tensor h = from_device(hidden, d, {rows, hidden_size}), t = from_device(table, d, {vocab, hidden_size});
    ms = timed([&] { (void)llm::cuda_argmax_last_row(llm::cuda_lm_head(h, t)); }, reps);
  });
  return ms;
}

// ---- the reference's CudaSampler (include/llm/ops_cuda.h:53-74): one token per call, blocking
REFCU_API int refcu_sample_row(const void* logits, int64_t rows, int64_t vocab, int dtype, int64_t row, float temperature,
                               int32_t top_k, float top_p, uint64_t seed, uint64_t draw_offset, int32_t* result) {
  return guarded([&] {
    static llm::CudaSampler* sampler = nullptr;     // one workspace for the process, sized for the largest vocabulary seen
    static size_t capacity = 0;
    if (sampler == nullptr || size_t(vocab) > capacity) {
      delete sampler;
      capacity = size_t(vocab) < 151936 ? 151936 : size_t(vocab);
      sampler = new llm::CudaSampler(capacity);
    }
    llm::SamplingConfig config;
    config.temperature = temperature;
    config.top_k = top_k;
    config.top_p = top_p;
    config.seed = seed;
    *result = sampler->sample_row(from_device(logits, dtype_of(dtype), {rows, vocab}), size_t(row), config, draw_offset);
  });
}

// milliseconds per sampled row (the reference samples one row per blocking call)
REFCU_API float refcu_time_sample_row(const void* logits, int64_t rows, int64_t vocab, int dtype, float temperature, int32_t top_k,
                                      float top_p, int reps) {
  try {
    CUDA_CHECK(cudaDeviceSynchronize());
    llm::CudaSampler sampler{static_cast<size_t>(vocab)};
    llm::SamplingConfig config;
    config.temperature = temperature;
    config.top_k = top_k;
    config.top_p = top_p;
    config.seed = 1;
    Tensor t = from_device(logits, dtype_of(dtype), {rows, vocab});
    uint64_t draw = 0;
    return timed([&] { sampler.sample_row(t, size_t(draw % uint64_t(rows)), config, draw); ++draw; }, reps);
  } catch (const std::exception&) { return -1.0f; }
}
