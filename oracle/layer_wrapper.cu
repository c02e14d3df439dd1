// TEST INFRASTRUCTURE, not part of the product.
// An extern "C" door in front of the reference's own decoder-layer code
// (src/qwen3_layer_cuda.cu: qwen3_decoder_layer_cuda_trace and _trace_fp16), so that a test can run
// that code twice on the same inputs: once linked against the reference's operators and once with
// the in-scope operators (RMSNorm, RoPE, add, SwiGLU) replaced by this repository's, and compare
// the 17 trace nodes.  The reference's layer source is compiled unmodified from the reference tree.
#include "llm/qwen3_layer_cuda.h"
#ifdef LAYER_WITH_B200_OPS
#include "llm/ops_cuda.h"
#include "llm/ops_cuda_b200.h"
#include <memory>
#endif

#include <cstdio>
#include <cstring>
#include <exception>
#include <vector>

using namespace llm;

namespace {

Tensor upload(const float* host, std::vector<int64_t> shape, bool half) {
  size_t count = 1;
  for (int64_t d : shape) count *= static_cast<size_t>(d);
  Tensor t(half ? DType::F16 : DType::F32, shape);
  for (size_t i = 0; i < count; ++i) t.set_f32(i, host[i]);
  return t.to(DeviceType::CUDA);
}

void download(const Tensor& device, float* host) {
  Tensor t = device.to(DeviceType::CPU);
  for (size_t i = 0; i < t.numel(); ++i) host[i] = t.get_f32(i);
}

}  // namespace

// weights: input_norm[1024], q_proj[2048,1024], k_proj[1024,1024], v_proj[1024,1024], q_norm[128], k_norm[128],
//          o_proj[1024,2048], post_attention_norm[1024], gate_proj[3072,1024], up_proj[3072,1024], down_proj[1024,3072]
// nodes (outputs, fp32 on the host): input_norm, q_linear, k_linear, v_linear, q_norm_output, k_norm_output, q_rope,
//          k_rope, attention_output, o_proj_output, attention_residual, post_attention_norm, gate_proj_output,
//          up_proj_output, swiglu_output, down_proj_output, layer_output
extern "C" __attribute__((visibility("default"))) int layer_trace(int half, const float* hidden, int seq,
                                                                    const int32_t* positions, const float* const* weights,
                                                                    float eps, float theta, float* const* nodes, char* error,
                                                                    int error_len) {
  try {
    const int64_t H = 1024, Q = 2048, KV = 1024, I = 3072, D = 128;
    const bool h = half != 0;
    Qwen3CudaLayerWeights w{upload(weights[0], {H}, h),      upload(weights[1], {Q, H}, h), upload(weights[2], {KV, H}, h),
                            upload(weights[3], {KV, H}, h),  upload(weights[4], {D}, h),    upload(weights[5], {D}, h),
                            upload(weights[6], {H, Q}, h),   upload(weights[7], {H}, h),    upload(weights[8], {I, H}, h),
                            upload(weights[9], {I, H}, h),   upload(weights[10], {H, I}, h)};
    Tensor x = upload(hidden, {seq, H}, h);
    std::vector<int32_t> pos(positions, positions + seq);
    Qwen3LayerTrace t = h ? qwen3_decoder_layer_cuda_trace_fp16(x, pos, w, eps, theta)
                          : qwen3_decoder_layer_cuda_trace(x, pos, w, eps, theta);
    const Tensor* order[17] = {&t.input_norm,      &t.q_linear,      &t.k_linear,         &t.v_linear,
                               &t.q_norm_output,   &t.k_norm_output, &t.q_rope,           &t.k_rope,
                               &t.attention_output, &t.o_proj_output, &t.attention_residual, &t.post_attention_norm,
                               &t.gate_proj_output, &t.up_proj_output, &t.swiglu_output,   &t.down_proj_output,
                               &t.layer_output};
    for (int i = 0; i < 17; ++i) download(*order[i], nodes[i]);
    return 0;
  } catch (const std::exception& e) {
    if (error && error_len > 0) { std::strncpy(error, e.what(), size_t(error_len) - 1); error[error_len - 1] = 0; }
    return 1;
  }
}

// Which operators this library was linked with, and (drop-in build only) the switch between the fast
// and the deterministic reductions for the calling thread.  Returns 1 in the drop-in build, 0 in the
// all-reference build (where `deterministic` is ignored).
extern "C" __attribute__((visibility("default"))) int layer_select_reductions(int deterministic) {
#ifdef LAYER_WITH_B200_OPS
  thread_local std::unique_ptr<CudaReductionModeGuard> guard;
  guard.reset();
  if (deterministic) guard = std::make_unique<CudaReductionModeGuard>(CudaReductionMode::kDeterministic);
  return 1;
#else
  (void)deterministic;
  return 0;
#endif
}
