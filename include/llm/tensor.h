// llm::Tensor — the value type every operator argument travels in.
// API-compatible with the reference's include/llm/tensor.h:9-38: a handle (dtype, shape,
// strides, device) onto shared, reference-counted storage plus a byte offset; views share
// storage.  CUDA storage is allocated through the library's counted allocator, so
// cuda_allocation_stats() behaves as in the reference (src/tensor_cuda.cu:12-54).
#pragma once
#include "device.h"
#include "dtype.h"

#include <cstddef>
#include <cstdint>
#include <memory>
#include <vector>

namespace llm {

// Counters of the device allocations made on behalf of Tensor storage since the last reset (or process
// start): how many cudaMalloc / cudaFree calls, how many bytes each way, what is live now and the
// high-water mark.  A reset keeps the allocations that are live as the new baseline of the peak.
struct CudaAllocationStats {
  uint64_t cuda_malloc_calls = 0;
  uint64_t cuda_free_calls = 0;
  uint64_t cuda_allocated_bytes_total = 0;
  uint64_t cuda_freed_bytes_total = 0;
  uint64_t cuda_live_bytes = 0;
  uint64_t cuda_peak_live_bytes = 0;
};
CudaAllocationStats cuda_allocation_stats();
void reset_cuda_allocation_stats();

// Copying a Tensor copies the handle, not the bytes: both copies see the same storage, which is released
// when the last handle goes.  Element (i0, i1, ...) lives at storage_offset() + sum(i_k * strides()[k])
// elements from the start of the storage; strides are in elements, row-major for fresh tensors.
class Tensor {
 public:
  // An empty handle: no storage, no shape.  Only assignment makes it useful.
  Tensor() = default;
  // Fresh, zero-initialised (CPU) or uninitialised (CUDA) row-major storage.  BF16 is host-only.
  Tensor(DType dtype, std::vector<int64_t> shape, DeviceType device = DeviceType::CPU);
  // A CPU/F32 tensor holding `values` (as many as the shape has elements, else std::invalid_argument).
  static Tensor from_f32(const std::vector<int64_t>& shape, const std::vector<float>& values);

  // ---- what it is

  DType dtype() const { return dtype_; }
  DeviceType device() const { return device_; }
  const std::vector<int64_t>& shape() const { return shape_; }
  const std::vector<int64_t>& strides() const { return strides_; }
  size_t numel() const { return numel_; }
  size_t nbytes() const { return numel_ * dtype_size(dtype_); }
  size_t storage_bytes() const { return storage_size_; }
  size_t storage_offset() const { return offset_; }

  // ---- views and copies.  The view forms share storage with *this and need a contiguous source; reshape
  // keeps the element count, the two first-dimension forms keep every other dimension.
  bool is_contiguous() const;
  Tensor reshape(const std::vector<int64_t>& shape) const;       // view; same element count
  Tensor prefix_first_dim(size_t size) const;                    // view of rows [0, size)
  Tensor slice_first_dim(size_t offset, size_t size) const;      // view of rows [offset, offset + size)
  Tensor contiguous() const;
  Tensor to(DeviceType target) const;                            // blocking copy when the device changes

  // ---- the bytes.  data() is the address of element 0 of this view: a host pointer for CPU storage, a
  // device pointer for CUDA storage (never dereference that one on the host).
  void* data();
  const void* data() const;
  // Host accessors: throw std::runtime_error on CUDA storage or on a dtype mismatch.
  // get_f32 / set_f32 address the index-th element of a CONTIGUOUS tensor and widen / narrow F16 and BF16.
  float get_f32(size_t index) const;
  void set_f32(size_t index, float value);
  float* data_f32();
  const float* data_f32() const;
  uint16_t* data_f16();
  uint16_t* data_bf16();
  int32_t* data_i32();
  const int32_t* data_i32() const;

 private:
  // the constructor behind the view forms: a new handle onto existing storage
  Tensor(DType dtype, DeviceType device, std::vector<int64_t> shape, std::vector<int64_t> strides,
         std::shared_ptr<void> storage, size_t storage_size, size_t offset, size_t numel);

  DType dtype_ = DType::F32;
  DeviceType device_ = DeviceType::CPU;
  std::vector<int64_t> shape_, strides_;
  std::shared_ptr<void> storage_;   // CPU: a byte buffer; CUDA: a device pointer with a counted deleter
  size_t storage_size_ = 0, offset_ = 0, numel_ = 0;
};

}  // namespace llm
