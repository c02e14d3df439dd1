// Where a tensor's storage lives.  API-compatible with the reference's include/llm/device.h:3.
#pragma once

namespace llm {
enum class DeviceType { CPU, CUDA };
inline const char* device_name(DeviceType d) { return d == DeviceType::CUDA ? "CUDA" : "CPU"; }
}  // namespace llm
