// CUDA error -> std::runtime_error, with the message layout of the reference's
// include/llm/cuda_check.h:7 ("CUDA error: <expr> at <file>:<line>: <message>").
#pragma once
#include <cuda_runtime.h>
#include <stdexcept>
#include <string>

namespace llm {

// Throws when a CUDA runtime call did not return cudaSuccess.  `expr` is the source text of the call;
// the failing call's own sticky error state is left to the caller (the kernel launchers clear it).
inline void cuda_check(cudaError_t status, const char* expr, const char* file, int line) {
  if (status == cudaSuccess) return;
  std::string message = "CUDA error: ";
  message += expr;
  message += " at ";
  message += file;
  message += ':';
  message += std::to_string(line);
  message += ": ";
  message += cudaGetErrorString(status);
  throw std::runtime_error(message);
}

}  // namespace llm

// CUDA_CHECK(call): evaluate `call` once and throw on failure.  CUDA_KERNEL_CHECK(): the same for the
// error a kernel launch leaves behind (asynchronous faults surface at the caller's next synchronisation).
#define CUDA_CHECK(expr) ::llm::cuda_check((expr), #expr, __FILE__, __LINE__)
#define CUDA_KERNEL_CHECK() CUDA_CHECK(cudaGetLastError())
