// Host-only stand-ins for the five symbols the reference defines in its CUDA
// translation unit (reference src/tensor_cuda.cu:12-56), so that the reference's
// CPU sources link without a CUDA runtime.  TEST INFRASTRUCTURE ONLY.
#include "llm/tensor.h"
#include <stdexcept>

namespace llm {
CudaAllocationStats cuda_allocation_stats() { return {}; }
void reset_cuda_allocation_stats() {}
namespace detail {
void* cuda_allocate(size_t) { throw std::runtime_error("oracle build: no CUDA storage"); }
void cuda_release(void*) {}
}  // namespace detail
Tensor Tensor::to(DeviceType target) const {
  if (target == device_) return *this;
  throw std::runtime_error("oracle build: no CUDA storage");
}
}  // namespace llm
