// CUDA side of llm::Tensor: counted device allocation and the blocking host<->device copy.
// Replaces the reference's src/tensor_cuda.cu:12-56.  The counters live in the C ABI
// (b2_alloc / b2_free / b2_get_alloc_stats), so Tensor allocations and direct C callers are
// counted together, with the reference's semantics: reset zeroes the call and byte totals and
// restarts the peak from the bytes live at that moment.
#include "llm/cuda_check.h"
#include "llm/tensor.h"
#include "b2ops.h"

#include <exception>
#include <stdexcept>
#include <string>

namespace llm {

CudaAllocationStats cuda_allocation_stats() {
  b2_alloc_stats raw;
  b2_get_alloc_stats(&raw);
  CudaAllocationStats s;
  s.cuda_malloc_calls = raw.malloc_calls;
  s.cuda_free_calls = raw.free_calls;
  s.cuda_allocated_bytes_total = raw.allocated_bytes_total;
  s.cuda_freed_bytes_total = raw.freed_bytes_total;
  s.cuda_live_bytes = raw.live_bytes;
  s.cuda_peak_live_bytes = raw.peak_live_bytes;
  return s;
}

void reset_cuda_allocation_stats() { b2_reset_alloc_stats(); }

namespace detail {

void* cuda_allocate(size_t bytes) {
  void* p = b2_alloc(bytes);
  if (p == nullptr && bytes != 0)
    throw std::runtime_error(std::string("CUDA error: cudaMalloc(&p, n) at tensor_cuda.cu: ") + b2_last_error());
  return p;
}

// A failing cudaFree leaves the process in an unknown state: terminate, as the reference does (:43-44).
void cuda_release(void* ptr) {
  if (ptr != nullptr && b2_free(ptr) != B2_OK) std::terminate();
}

}  // namespace detail

Tensor Tensor::to(DeviceType target) const {
  if (target == device_) return *this;
  if (target == DeviceType::CUDA && dtype_ == DType::BF16) throw std::runtime_error("Tensor::to CUDA: BF16 is unsupported");
  Tensor out(dtype_, shape_, target);
  if (nbytes() != 0)
    CUDA_CHECK(cudaMemcpy(out.data(), data(), nbytes(),
                          target == DeviceType::CUDA ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost));
  return out;
}

}  // namespace llm
