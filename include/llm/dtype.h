// Element types of llm::Tensor and the host-side 16-bit float codecs.
// API-compatible with the reference's include/llm/dtype.h:6-12.
#pragma once
#include <cstddef>
#include <cstdint>

namespace llm {

enum class DType { F32, F16, BF16, I32 };

inline size_t dtype_size(DType d) {
  switch (d) {
    case DType::F32: case DType::I32: return 4;
    default: return 2;
  }
}
inline const char* dtype_name(DType d) {
  switch (d) {
    case DType::F32: return "F32";
    case DType::F16: return "F16";
    case DType::BF16: return "BF16";
    default: return "I32";
  }
}

// Host codecs.  decode_* are exact.  encode_f16 keeps the reference's behaviour
// (src/tensor.cpp:12): normal numbers are TRUNCATED to 10 mantissa bits, not rounded;
// weights the reference converts on the host therefore keep their exact bit patterns.
// encode_bf16 truncates as well (src/tensor.cpp:11).
float decode_f16(uint16_t bits);
uint16_t encode_f16(float value);
float decode_bf16(uint16_t bits);
uint16_t encode_bf16(float value);

}  // namespace llm
