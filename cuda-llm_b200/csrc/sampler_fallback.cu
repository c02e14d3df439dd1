// The sampler's whole-row route for the rows the top-p route could not settle, launched FROM THE DEVICE: one tiny
// kernel lists those rows and, only when there are any, launches the two dozen kernels of the route over exactly
// those rows (tail launches: they run after the listing kernel, in order, and before whatever follows it in the
// stream).  A call whose rows were all settled -- the usual case -- pays for that one kernel; launched from the
// host, the idle route cost 66-74 us per call.  Relocatable device code (and the device runtime) is confined to
// this file.
#define B2_DEVICE_CHAIN
#define B2_NO_DEPENDENT_LAUNCH
#include "sampler_rows.cuh"
#include "kernels.h"

namespace b2 {
namespace {

__global__ void stream_order_kernel() {}

// The rows whose flag is up, as a list; when there are any, the whole-row route over exactly those rows, launched
// from here (the launches run after this kernel, in order, and before anything that follows it in the stream).
__global__ void __launch_bounds__(256) list_rows_kernel(const int* row_flags, int rows, int* list, int* count, const ChainArgs chain) {
  dependent_launch_prologue();
  __shared__ int n;
  if (threadIdx.x == 0) n = 0;
  __syncthreads();
  for (int r = threadIdx.x; r < rows; r += 256)
    if (row_flags[r] != 0) list[atomicAdd(&n, 1)] = r;
  __syncthreads();
  if (threadIdx.x != 0) return;
  *count = n;
  if (n > 0) whole_row_chain(chain, RowSet{list, count}, unsigned(n < kListedRowBlocks ? n : kListedRowBlocks), nullptr);
}
}  // namespace

int launch_sampler_rows_fallback(const int* row_flags, int64_t rows, int* list, int* count, const void* logits, int dtype,
                                 int64_t width, int64_t row_stride, int64_t padded, float temperature, int top_k, float top_p,
                                 unsigned long long seed, const unsigned long long* draw_offsets, unsigned long long* keys,
                                 float* running, int32_t* out_ids, cudaStream_t s) {
  const ChainArgs chain{logits, dtype, width, row_stride, padded, temperature, top_k, top_p, seed, draw_offsets, keys, running, out_ids};
  // Plain launches, no programmatic serialisation on either side of the listing kernel: a kernel that the stream
  // let start early would hold its thread blocks' resources while it waits for the listing kernel's grid to
  // complete, and that grid is complete only when its child grids -- which need those resources -- have run.
  // The empty kernel behind it is an ordinary stream dependency, so whatever the caller launches next (with or
  // without the attribute) starts after the children.
  list_rows_kernel<<<1, 256, 0, s>>>(row_flags, int(rows), list, count, chain);
  stream_order_kernel<<<1, 1, 0, s>>>();
  return launch_status("sample_rows (rows handed back)");
}

}  // namespace b2
