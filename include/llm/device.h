// Where a tensor's storage lives.  API-compatible with the reference's include/llm/device.h:3.
#pragma once

namespace llm {

// CPU: ordinary host memory, readable through Tensor's host accessors.
// CUDA: memory of the current CUDA device; only kernels and cudaMemcpy may touch it.
enum class DeviceType { CPU, CUDA };

// "CPU" or "CUDA", for messages.
inline const char* device_name(DeviceType d) { return d == DeviceType::CUDA ? "CUDA" : "CPU"; }
}  // namespace llm
