// CUDA error -> std::runtime_error, with the message layout of the reference's
// include/llm/cuda_check.h:7 ("CUDA error: <expr> at <file>:<line>: <message>").
#pragma once
#include <cuda_runtime.h>
#include <stdexcept>
#include <string>

namespace llm {
inline void cuda_check(cudaError_t status, const char* expr, const char* file, int line) {
  if (status == cudaSuccess) return;
  throw std::runtime_error(std::string("CUDA error: ") + expr + " at " + file + ":" + std::to_string(line) + ": " +
                           cudaGetErrorString(status));
}
}  // namespace llm

#define CUDA_CHECK(expr) ::llm::cuda_check((expr), #expr, __FILE__, __LINE__)
#define CUDA_KERNEL_CHECK() CUDA_CHECK(cudaGetLastError())
