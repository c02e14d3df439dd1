// Host side of llm::Tensor: 16-bit float codecs, shape arithmetic, views and host accessors.
// Behaviour follows the reference's src/tensor.cpp (cited per function); the text is this
// library's own.
#include "llm/tensor.h"

#include <cmath>
#include <cstring>
#include <limits>
#include <stdexcept>
#include <string>
#include <utility>

namespace llm {

namespace detail {
void* cuda_allocate(size_t bytes);   // tensor_cuda.cu
void cuda_release(void* ptr);
}  // namespace detail

namespace {

uint32_t float_bits(float v) { uint32_t u; std::memcpy(&u, &v, sizeof u); return u; }
float bits_float(uint32_t u) { float v; std::memcpy(&v, &u, sizeof v); return v; }

using Shape = std::vector<int64_t>;

size_t element_count(const Shape& shape) {
  size_t n = 1;
  for (int64_t d : shape) {
    if (d < 0) throw std::invalid_argument("Tensor: negative shape dimension");
    if (d != 0 && n > std::numeric_limits<size_t>::max() / size_t(d))
      throw std::invalid_argument("Tensor: shape product overflow");
    n *= size_t(d);
  }
  return n;
}

Shape row_major_strides(const Shape& shape) {
  Shape strides(shape.size());
  int64_t run = 1;
  for (size_t k = shape.size(); k-- > 0;) {
    strides[k] = run;
    if (shape[k] != 0 && run > std::numeric_limits<int64_t>::max() / shape[k])
      throw std::invalid_argument("Tensor: stride overflow");
    run *= shape[k];
  }
  return strides;
}

void require_host(DeviceType device, const char* accessor) {
  if (device == DeviceType::CUDA)
    throw std::runtime_error(std::string("Tensor::") + accessor +
                             ": host access to CUDA storage is forbidden; use to(CPU)");
}

using HostBuffer = std::vector<uint8_t>;

}  // namespace

// ---- codecs (reference src/tensor.cpp:11-13)
// Host-side conversions only: the kernels use the hardware's round-to-nearest-even conversions.  The host F16
// encoder TRUNCATES the mantissa of normal numbers (and rounds only subnormals), which is what the reference's
// host code does; tests that need round-to-nearest-even bit patterns build them with the oracle's encoder.

uint16_t encode_bf16(float value) { return uint16_t(float_bits(value) >> 16); }
float decode_bf16(uint16_t bits) { return bits_float(uint32_t(bits) << 16); }

uint16_t encode_f16(float value) {
  const uint32_t u = float_bits(value);
  const uint32_t sign = (u >> 16) & 0x8000u, exponent = (u >> 23) & 0xffu;
  uint32_t mantissa = u & 0x7fffffu;
  if (exponent == 0xffu) return uint16_t(sign | 0x7c00u | (mantissa ? 0x200u : 0u));
  const int half_exponent = int(exponent) - 127 + 15;
  if (half_exponent >= 31) return uint16_t(sign | 0x7c00u);
  if (half_exponent <= 0) {
    if (half_exponent < -10) return uint16_t(sign);
    mantissa |= 0x800000u;   // subnormal halves: shift with a rounding bit, as the reference does
    return uint16_t(sign | ((mantissa >> (14 - half_exponent)) + ((mantissa >> (13 - half_exponent)) & 1u)));
  }
  return uint16_t(sign | (uint32_t(half_exponent) << 10) | (mantissa >> 13));   // truncation, not rounding
}

float decode_f16(uint16_t bits) {
  const uint32_t sign = uint32_t(bits & 0x8000u) << 16;
  const uint32_t exponent = (bits >> 10) & 31u, mantissa = bits & 1023u;
  if (exponent == 31u) return bits_float(sign | 0x7f800000u | (mantissa << 13));
  if (exponent == 0u) {
    const float magnitude = std::ldexp(float(mantissa), -24);   // zero or subnormal: exact
    return sign ? -magnitude : magnitude;
  }
  return bits_float(sign | ((exponent + 112u) << 23) | (mantissa << 13));
}

// ---- construction (reference src/tensor.cpp:16-19)
// CPU storage is a zero-filled byte vector owned through the shared_ptr's deleter; CUDA storage comes from the
// counted allocator of tensor_cuda.cu and is NOT initialised.  The private constructor makes views: it checks
// that the window [offset, offset + nbytes) lies inside the storage it is given.

Tensor::Tensor(DType dtype, std::vector<int64_t> shape, DeviceType device)
    : dtype_(dtype), device_(device), shape_(std::move(shape)), strides_(row_major_strides(shape_)),
      numel_(element_count(shape_)) {
  storage_size_ = nbytes();
  if (device == DeviceType::CUDA) {
    if (dtype == DType::BF16) throw std::runtime_error("Tensor CUDA: BF16 is unsupported on this path");
    storage_ = std::shared_ptr<void>(detail::cuda_allocate(storage_size_), detail::cuda_release);
  } else {
    auto* buffer = new HostBuffer(storage_size_);
    storage_ = std::shared_ptr<void>(buffer, [](void* p) { delete static_cast<HostBuffer*>(p); });
  }
}

Tensor::Tensor(DType dtype, DeviceType device, std::vector<int64_t> shape, std::vector<int64_t> strides,
               std::shared_ptr<void> storage, size_t storage_size, size_t offset, size_t numel)
    : dtype_(dtype), device_(device), shape_(std::move(shape)), strides_(std::move(strides)),
      storage_(std::move(storage)), storage_size_(storage_size), offset_(offset), numel_(numel) {
  if (device == DeviceType::CUDA && dtype == DType::BF16) throw std::runtime_error("Tensor view CUDA: BF16 unsupported");
  if (offset_ > storage_size_ || nbytes() > storage_size_ - offset_) throw std::runtime_error("Tensor view exceeds storage");
}

Tensor Tensor::from_f32(const std::vector<int64_t>& shape, const std::vector<float>& values) {
  Tensor t(DType::F32, shape);
  if (values.size() != t.numel()) throw std::invalid_argument("Tensor::from_f32 value count mismatch");
  if (!values.empty()) std::memcpy(t.data(), values.data(), values.size() * sizeof(float));
  return t;
}

// ---- views (reference src/tensor.cpp:20-45)
// All views need a contiguous source.  slice_first_dim moves the byte offset by whole rows of the first
// dimension; the result is only element-aligned, which is why every kernel has a path for unaligned pointers.

bool Tensor::is_contiguous() const { return strides_ == row_major_strides(shape_); }

Tensor Tensor::reshape(const std::vector<int64_t>& shape) const {
  if (!is_contiguous()) throw std::runtime_error("Tensor::reshape requires contiguous tensor");
  const size_t n = element_count(shape);
  if (n != numel_) throw std::invalid_argument("Tensor::reshape changes element count");
  return Tensor(dtype_, device_, shape, row_major_strides(shape), storage_, storage_size_, offset_, n);
}

Tensor Tensor::prefix_first_dim(size_t size) const {
  if (shape_.empty() || shape_[0] <= 0 || size == 0 || size > size_t(shape_[0]))
    throw std::invalid_argument("Tensor::prefix_first_dim: invalid prefix size");
  return slice_first_dim(0, size);
}

Tensor Tensor::slice_first_dim(size_t offset, size_t size) const {
  if (shape_.empty() || shape_[0] <= 0 || size == 0 || offset > size_t(shape_[0]) || size > size_t(shape_[0]) - offset)
    throw std::invalid_argument("Tensor::slice_first_dim: invalid slice");
  if (!is_contiguous()) throw std::runtime_error("Tensor::slice_first_dim requires contiguous tensor");
  Shape shape = shape_;
  shape[0] = int64_t(size);
  const size_t row_elements = numel_ / size_t(shape_[0]);
  return Tensor(dtype_, device_, shape, row_major_strides(shape), storage_, storage_size_,
                offset_ + offset * row_elements * dtype_size(dtype_), size * row_elements);
}

Tensor Tensor::contiguous() const {
  if (is_contiguous()) return *this;
  if (device_ == DeviceType::CUDA)
    throw std::runtime_error("Tensor::contiguous for non-contiguous CUDA storage is unsupported");
  Tensor copy(dtype_, shape_);
  for (size_t i = 0; i < numel_; ++i) copy.set_f32(i, get_f32(i));
  return copy;
}

// ---- data access (reference src/tensor.cpp:46-51)
// data() works for both devices (it is only an address); every typed or element accessor refuses CUDA storage
// with std::runtime_error and checks the dtype it is asked for.

void* Tensor::data() {
  if (!storage_) return nullptr;
  char* base = device_ == DeviceType::CPU ? reinterpret_cast<char*>(static_cast<HostBuffer*>(storage_.get())->data())
                                          : static_cast<char*>(storage_.get());
  return base + offset_;
}
const void* Tensor::data() const { return const_cast<Tensor*>(this)->data(); }

float Tensor::get_f32(size_t index) const {
  require_host(device_, "get_f32");
  if (dtype_ == DType::I32) throw std::runtime_error("Tensor::get_f32 is unavailable for I32");
  if (index >= numel_) throw std::out_of_range("Tensor element index");
  const void* p = data();
  if (dtype_ == DType::F32) return static_cast<const float*>(p)[index];
  const uint16_t raw = static_cast<const uint16_t*>(p)[index];
  return dtype_ == DType::F16 ? decode_f16(raw) : decode_bf16(raw);
}

void Tensor::set_f32(size_t index, float value) {
  require_host(device_, "set_f32");
  if (dtype_ == DType::I32) throw std::runtime_error("Tensor::set_f32 is unavailable for I32");
  if (index >= numel_) throw std::out_of_range("Tensor element index");
  void* p = data();
  if (dtype_ == DType::F32) static_cast<float*>(p)[index] = value;
  else static_cast<uint16_t*>(p)[index] = dtype_ == DType::F16 ? encode_f16(value) : encode_bf16(value);
}

namespace {
void require_dtype(DType have, DType want, const char* name) {
  if (have != want) throw std::runtime_error(std::string("Tensor dtype is not ") + name);
}
}  // namespace

float* Tensor::data_f32() { require_host(device_, "data_f32"); require_dtype(dtype_, DType::F32, "F32"); return static_cast<float*>(data()); }
const float* Tensor::data_f32() const { return const_cast<Tensor*>(this)->data_f32(); }
uint16_t* Tensor::data_f16() { require_host(device_, "data_f16"); require_dtype(dtype_, DType::F16, "F16"); return static_cast<uint16_t*>(data()); }
uint16_t* Tensor::data_bf16() { require_host(device_, "data_bf16"); require_dtype(dtype_, DType::BF16, "BF16"); return static_cast<uint16_t*>(data()); }
int32_t* Tensor::data_i32() { require_host(device_, "data_i32"); require_dtype(dtype_, DType::I32, "I32"); return static_cast<int32_t*>(data()); }
const int32_t* Tensor::data_i32() const { return const_cast<Tensor*>(this)->data_i32(); }

}  // namespace llm
