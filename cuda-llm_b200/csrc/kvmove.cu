// Row moves around the paged KV cache and the padded-prefill logits for sm_100a: no arithmetic, one
// indirection per row, 16-byte vectors.  One warp moves one row (or one key/value row pair), with up
// to four vectors in flight per lane; the row's destination comes from a block table.
//
// Replaces reference kernels paged_kv_write_decode_kernel / paged_kv_write_decode_batch_kernel
// (src/paged_attention_cuda.cu:219-262: one element per thread, the block-table lookup and two
// divisions repeated for every element), packed_kv_prefill_copy_kernel (src/ops_cuda.cu:1104-1121,
// likewise) and the loop of blocking device-to-device copies in select_last_valid_logits
// (src/qwen3_padded_prefill.cpp:137-143).
//
// Pool layout, as the reference's PagedKvCachePool keeps it (storage shape
// [layers, total_blocks, 2, block_size, kv_heads, head_dim]): the row of token slot `s` of block `b`,
// plane p (0 = key, 1 = value), layer l starts at element
//   (((l * total_blocks + b) * 2 + p) * block_size + s) * (kv_heads * head_dim).
#include "common.cuh"
#include "kernels.h"
#include "b2ops.h"

namespace b2 {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / kWarpSize;

// copies `bytes` (any count) from src to dst with one warp; 16-byte vectors when both are aligned
__device__ __forceinline__ void warp_copy_row(const unsigned char* src, unsigned char* dst, int64_t bytes, int lane) {
  if (((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst) | uintptr_t(bytes)) & 15u) == 0) {
    const uint4* s = reinterpret_cast<const uint4*>(src);
    uint4* d = reinterpret_cast<uint4*>(dst);
    const int64_t n = bytes >> 4;
    for (int64_t v0 = lane; v0 < n; v0 += kWarpSize * 4) {
      uint4 r[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) if (v0 + k * kWarpSize < n) r[k] = ld_stream(s + v0 + k * kWarpSize);
#pragma unroll
      for (int k = 0; k < 4; ++k) if (v0 + k * kWarpSize < n) st_stream(d + v0 + k * kWarpSize, r[k]);
    }
  } else if (((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst) | uintptr_t(bytes)) & 1u) == 0) {
    const uint16_t* s = reinterpret_cast<const uint16_t*>(src);
    uint16_t* d = reinterpret_cast<uint16_t*>(dst);
    for (int64_t i = lane; i < (bytes >> 1); i += kWarpSize) d[i] = s[i];
  } else {
    for (int64_t i = lane; i < bytes; i += kWarpSize) dst[i] = src[i];
  }
}

struct PoolShape { int64_t total_blocks, block_size, row_bytes; };   // row_bytes = kv_heads * head_dim * element size

__device__ __forceinline__ unsigned char* pool_row(unsigned char* storage, const PoolShape& p, int64_t layer, int64_t block,
                                                   int plane, int64_t slot) {
  return storage + ((((layer * p.total_blocks + block) * 2 + plane) * p.block_size + slot) * p.row_bytes);
}

// rows: one per (token, plane).  mode 0: decode batch, token b sits at positions[b] of ITS block table
// block_tables[b, :max_blocks]; mode 1: packed prefill, token t sits at slot t of the single block table;
// mode 2: single decode, the one token sits at *positions - 1 (a cache length; nothing is written when 0).
// A block id outside [0, total_blocks) or a negative position never reaches memory: bit 0 of *status is raised.
template <int kMode>
__global__ void __launch_bounds__(kThreads)
paged_kv_write_kernel(const unsigned char* key, const unsigned char* value, unsigned char* storage,
                      const int32_t* block_tables, const int32_t* positions, int64_t tokens, int64_t max_blocks,
                      int64_t layer, PoolShape pool, int32_t* status) {
  dependent_launch_prologue();
  const int lane = threadIdx.x & 31;
  const int64_t warps = int64_t(gridDim.x) * kWarps;
  for (int64_t w = int64_t(blockIdx.x) * kWarps + (threadIdx.x >> 5); w < tokens * 2; w += warps) {
    const int64_t token = w >> 1;
    const int plane = int(w & 1);
    int64_t position;
    const int32_t* table;
    if (kMode == 0) { position = positions[token]; table = block_tables + token * max_blocks; }
    else if (kMode == 1) { position = token; table = block_tables; }
    else { position = int64_t(positions[0]) - 1; table = block_tables; if (position < 0) return; }
    bool ok = position >= 0 && position / pool.block_size < max_blocks;
    int64_t block = 0;
    if (ok) { block = table[position / pool.block_size]; ok = block >= 0 && block < pool.total_blocks; }
    if (!ok) {
      if (lane == 0 && status != nullptr) atomicOr(status, 1);
      continue;
    }
    const unsigned char* src = (plane == 0 ? key : value) + token * pool.row_bytes;
    warp_copy_row(src, pool_row(storage, pool, layer, block, plane, position % pool.block_size), pool.row_bytes, lane);
  }
}

// out[b, :] = padded[b, valid_lengths[b] - 1, :]; a length outside [1, seq] raises bit 0 of *status and zero-fills the row
__global__ void __launch_bounds__(kThreads)
select_last_valid_kernel(const unsigned char* padded, const int32_t* valid_lengths, unsigned char* out, int64_t batch,
                         int64_t seq, int64_t row_bytes, int slices, int32_t* status) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = int64_t(gridDim.x) * kWarps;
  // a row of logits is long (hundreds of KB): `slices` warps share one row
  for (int64_t w = int64_t(blockIdx.x) * kWarps + (threadIdx.x >> 5); w < batch * slices; w += warps) {
    const int64_t b = w / slices;
    const int part = int(w - b * slices);
    int64_t per = ((row_bytes + slices - 1) / slices + 15) / 16 * 16;
    const int64_t lo = part * per, n = row_bytes - lo < per ? row_bytes - lo : per;
    if (n <= 0) continue;
    const int64_t length = valid_lengths[b];
    unsigned char* dst = out + b * row_bytes + lo;
    if (length < 1 || length > seq) {
      if (lane == 0 && status != nullptr) atomicOr(status, 1);
      for (int64_t i = lane; i < n; i += kWarpSize) dst[i] = 0;
      continue;
    }
    warp_copy_row(padded + (b * seq + (length - 1)) * row_bytes + lo, dst, n, lane);
  }
}

// one warp per row (or row part) and as many blocks as that takes: blocks dispatched in order walk memory in order
unsigned grid_for(int64_t warps_wanted) {
  const int64_t ctas = (warps_wanted + kWarps - 1) / kWarps, cap = 0x7fffffffll;
  return unsigned(ctas < 1 ? 1 : (ctas < cap ? ctas : cap));
}

}  // namespace

int launch_paged_kv_write(int mode, const void* key, const void* value, void* storage, const int32_t* block_tables,
                          const int32_t* positions, int64_t tokens, int64_t max_blocks, int64_t layer, int64_t total_blocks,
                          int64_t block_size, int64_t row_bytes, int32_t* status, cudaStream_t s) {
  if (tokens == 0) return B2_OK;
  const PoolShape pool{total_blocks, block_size, row_bytes};
  const unsigned grid = grid_for(tokens * 2);
  auto k = static_cast<const unsigned char*>(key);
  auto v = static_cast<const unsigned char*>(value);
  auto st = static_cast<unsigned char*>(storage);
  if (mode == 0)
    launch_kernel(paged_kv_write_kernel<0>, dim3(grid), dim3(kThreads), 0, s, k, v, st, block_tables, positions, tokens, max_blocks, layer, pool, status);
  else if (mode == 1)
    launch_kernel(paged_kv_write_kernel<1>, dim3(grid), dim3(kThreads), 0, s, k, v, st, block_tables, positions, tokens, max_blocks, layer, pool, status);
  else
    launch_kernel(paged_kv_write_kernel<2>, dim3(grid), dim3(kThreads), 0, s, k, v, st, block_tables, positions, tokens, max_blocks, layer, pool, status);
  return launch_status("paged_kv_write");
}

int launch_select_last_valid(const void* padded, const int32_t* valid_lengths, void* out, int64_t batch, int64_t seq,
                             int64_t row_bytes, int32_t* status, cudaStream_t s) {
  if (batch == 0 || row_bytes == 0) return B2_OK;
  // enough warps to fill the GPU even for a handful of rows, at least 4 KB per warp
  int64_t slices = (int64_t(sm_count()) * 8 * kWarps) / batch;
  const int64_t most = (row_bytes + 4095) / 4096;
  if (slices > most) slices = most;
  if (slices < 1) slices = 1;
  select_last_valid_kernel<<<grid_for(batch * slices), kThreads, 0, s>>>(static_cast<const unsigned char*>(padded), valid_lengths,
                                                                        static_cast<unsigned char*>(out), batch, seq, row_bytes,
                                                                        int(slices), status);
  return launch_status("select_last_valid_rows");
}

}  // namespace b2
