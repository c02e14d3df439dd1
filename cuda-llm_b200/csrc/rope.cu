// Rotary embedding (NeoX rotate-half) for sm_100a, alone or fused behind the
// per-head QK RMSNorm.  A warp takes a token: it first builds the token's cos/sin
// table in shared memory, once per (token, frequency) instead of once per
// (token, head, frequency) as the reference does, then streams every head of that
// token through 16-byte loads and stores.
//
// Replaces reference kernels ropek<T>, rope_batched_kernel<T> and
// rope_decode_batched_kernel<T> (src/ops_cuda.cu:133-135) and, in the fused form,
// the rmsk<T> launches in front of them (src/qwen3_layer_cuda.cu:289-292).
#include "common.cuh"
#include "bulk_copy.cuh"
#include "kernels.h"
#include "b2ops.h"

#include <cmath>

namespace b2 {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxTableHalf = 128;   // inverse-frequency table passed by value: head_dim <= 256

struct InvFreq { double v[kMaxTableHalf]; };

// cos/sin of positions[t] * theta^(-2j/D).
// Fast mode: the angle is formed in fp64 from a host-built table of
// pow(double(theta), -2j/D) (the same expression as the CPU operator,
// src/ops_cpu.cpp:11), reduced to [-pi, pi] in fp64 with a two-term 2*pi, and only
// then handed to the fp32 hardware sine/cosine: 4e-7 absolute at any position.
// Deterministic mode: the reference kernel's all-fp32 expression.
template <bool kOrdered>
__device__ __forceinline__ float2 rope_cos_sin(int32_t position, int j, int head_dim, float theta,
                                               const InvFreq& freq, int half) {
  if (kOrdered) {
    const float ang = float(position) * powf(theta, -2.f * float(j) / float(head_dim));
    return make_float2(cosf(ang), sinf(ang));
  }
  const double inv = half <= kMaxTableHalf ? freq.v[j]
                                           : pow(double(theta), -2.0 * double(j) / double(head_dim));
  const double angle = double(position) * inv;
  const double two_pi_hi = 6.283185307179586232e+00, two_pi_lo = 2.449293598294706414e-16;
  const double turns = rint(angle * 1.591549430918953456e-01);
  double r = fma(-turns, two_pi_hi, angle);
  r = fma(-turns, two_pi_lo, r);
  // |r| <= pi: the hardware sine/cosine are within 2^-21.4 (absolute) there, 25x inside the
  // 1e-5 parity bound and 1000x inside an fp16 ulp
  const float rf = float(r);
  return make_float2(__cosf(rf), __sinf(rf));
}

// rotate one (low, high) pair
template <bool kOrdered>
__device__ __forceinline__ void rotate(float a, float b, float2 cs, float& lo, float& hi) {
  if (kOrdered) {
    // written as in the reference kernel, contraction left to the compiler as it is there
    lo = a * cs.x - b * cs.y;
    hi = b * cs.x + a * cs.y;
  } else {
    lo = fmaf(a, cs.x, -(b * cs.y));
    hi = fmaf(a, cs.y, b * cs.x);
  }
}

struct HeadSet {           // one [tokens, heads, head_dim] tensor with its optional norm weight
  const void* x; const void* w; void* out; int heads;
};

// ---------------------------------------------------------------------------
// Vector kernel: one warp per token, no CTA-wide barrier anywhere.
// The warp first writes the token's cos/sin (head_dim/2 pairs, 2 per lane at
// head_dim 128) into its own slice of shared memory, then streams every head of
// the token.  Work item = one 16-byte vector of the low half of a head plus its
// partner in the high half; hv = (head_dim/2)/kPerVec items make one head and sit
// in consecutive lanes (hv is a power of two <= 32), so the fused norm reduces
// over them with xor-shuffles.  A lane always works on the same vector position
// `v` of a head, so its cos/sin values and norm weights are loaded once per token
// and the per-item work is: two 16-byte loads, the arithmetic, two stores.  The
// loads of kItemUnroll items are issued before any of them is used.
// The kernel is issue-bound before it is HBM-bound, hence the care about
// instruction count: shifts instead of divisions, hoisted weights, fused
// multiply-adds and the hardware reciprocal square root in fast mode.
// ---------------------------------------------------------------------------
constexpr int kItemUnroll = 4;
constexpr int kWarpsPerCta = kThreads / kWarpSize;

// cos and sin of the lane's frequencies, two consecutive frequencies per float2 (the layout of the
// packed fp32x2 instructions of sm_100: one instruction, two results)
template <int P> struct LaneAngles { float2 c[P], s[P], neg_s[P]; };

template <typename T, bool kNorm, bool kOrdered>
__device__ __forceinline__ void rope_token_heads(const uint4* x, const uint4* w, uint4* out, int items, int hv,
                                                 int hv_shift, int lane, const LaneAngles<Elem<T>::kPerVec / 2>& ang,
                                                 float inv_dim, float eps) {
  constexpr int P = Elem<T>::kPerVec / 2;   // element pairs per 16-byte vector
  const int v = lane & (hv - 1);
  float2 wl[P], wh[P];
  if (kNorm) {
    Elem<T>::unpack2(ld_reuse(w + v), wl);
    Elem<T>::unpack2(ld_reuse(w + hv + v), wh);
  }
  const int last = items - 1;
  // every lane runs the same number of steps, so the shuffles below are converged
  for (int base = 0; base < items; base += kWarpSize * kItemUnroll) {
    uint4 raw_lo[kItemUnroll], raw_hi[kItemUnroll];
    int where[kItemUnroll];
    bool ok[kItemUnroll];
#pragma unroll
    for (int u = 0; u < kItemUnroll; ++u) {
      const int item = base + u * kWarpSize + lane;
      ok[u] = item < items;
      // a lane past the end re-reads the last head (same vector position): valid memory, a consistent
      // group for the shuffles, and nothing is stored for it
      const int head = (ok[u] ? item : last) >> hv_shift;
      where[u] = (head << (hv_shift + 1)) + v;   // head * (2*hv) + v
      if (base + u * kWarpSize < items) {
        raw_lo[u] = ld_stream(x + where[u]);
        raw_hi[u] = ld_stream(x + where[u] + hv);
      }
    }
#pragma unroll
    for (int u = 0; u < kItemUnroll; ++u) {
      if (base + u * kWarpSize >= items) break;   // uniform across the warp
      float2 lo[P], hi[P];
      Elem<T>::unpack2(raw_lo[u], lo);
      Elem<T>::unpack2(raw_hi[u], hi);
      if (kNorm) {
        float2 acc = make_float2(0.0f, 0.0f);
#pragma unroll
        for (int e = 0; e < P; ++e) acc = __ffma2_rn(lo[e], lo[e], acc);
#pragma unroll
        for (int e = 0; e < P; ++e) acc = __ffma2_rn(hi[e], hi[e], acc);
        const float ss = group_sum(acc.x + acc.y, hv);
        const float inv = rsqrtf(fmaf(ss, inv_dim, eps));
        const float2 inv2 = make_float2(inv, inv);
#pragma unroll
        for (int e = 0; e < P; ++e) {
          lo[e] = __fmul2_rn(__fmul2_rn(lo[e], inv2), wl[e]);
          hi[e] = __fmul2_rn(__fmul2_rn(hi[e], inv2), wh[e]);
        }
      }
      float2 out_lo[P], out_hi[P];
#pragma unroll
      for (int e = 0; e < P; ++e) {
        if (kOrdered) {
          // written as in the reference kernel, contraction left to the compiler as it is there
          out_lo[e].x = lo[e].x * ang.c[e].x - hi[e].x * ang.s[e].x;
          out_hi[e].x = hi[e].x * ang.c[e].x + lo[e].x * ang.s[e].x;
          out_lo[e].y = lo[e].y * ang.c[e].y - hi[e].y * ang.s[e].y;
          out_hi[e].y = hi[e].y * ang.c[e].y + lo[e].y * ang.s[e].y;
        } else {
          out_lo[e] = __ffma2_rn(hi[e], ang.neg_s[e], __fmul2_rn(lo[e], ang.c[e]));   // a*c - b*s
          out_hi[e] = __ffma2_rn(lo[e], ang.s[e], __fmul2_rn(hi[e], ang.c[e]));       // a*s + b*c
        }
      }
      if (ok[u]) {
        st_stream(out + where[u], Elem<T>::pack2(out_lo));
        st_stream(out + where[u] + hv, Elem<T>::pack2(out_hi));
      }
    }
  }
}

template <typename T, bool kNorm, bool kOrdered>
__global__ void __launch_bounds__(kThreads, 2)
rope_tokens_kernel(HeadSet q, HeadSet k, const int32_t* __restrict__ positions, int64_t tokens, int head_dim, int hv,
                   int hv_shift, int64_t pos_period, float eps, float theta, const __grid_constant__ InvFreq freq) {
  constexpr int N = Elem<T>::kPerVec;
  extern __shared__ float table[];    // per warp: cos[half] then sin[half]
  dependent_launch_prologue();
  const int half = head_dim >> 1, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* cos_row = table + warp * head_dim;
  float* sin_row = cos_row + half;
  const int vecs_per_head = 2 * hv;
  const float inv_dim = 1.0f / float(head_dim);

  for (int64_t t = int64_t(blockIdx.x) * kWarpsPerCta + warp; t < tokens; t += int64_t(gridDim.x) * kWarpsPerCta) {
    const int32_t p = positions[pos_period ? t % pos_period : t];
    for (int j = lane; j < half; j += kWarpSize) {
      const float2 cs = rope_cos_sin<kOrdered>(p, j, head_dim, theta, freq, half);
      cos_row[j] = cs.x;
      sin_row[j] = cs.y;
    }
    __syncwarp();
    LaneAngles<N / 2> ang;              // this lane's frequencies: the same for every head
    const int first = (lane & (hv - 1)) * N;
#pragma unroll
    for (int e = 0; e < N / 2; ++e) {
      ang.c[e] = *reinterpret_cast<const float2*>(cos_row + first + 2 * e);
      ang.s[e] = *reinterpret_cast<const float2*>(sin_row + first + 2 * e);
      ang.neg_s[e] = make_float2(-ang.s[e].x, -ang.s[e].y);
    }

    rope_token_heads<T, kNorm, kOrdered>(
        reinterpret_cast<const uint4*>(q.x) + size_t(t) * q.heads * vecs_per_head, reinterpret_cast<const uint4*>(q.w),
        reinterpret_cast<uint4*>(q.out) + size_t(t) * q.heads * vecs_per_head, q.heads * hv, hv, hv_shift, lane, ang,
        inv_dim, eps);
    if (k.heads > 0)
      rope_token_heads<T, kNorm, kOrdered>(
          reinterpret_cast<const uint4*>(k.x) + size_t(t) * k.heads * vecs_per_head, reinterpret_cast<const uint4*>(k.w),
          reinterpret_cast<uint4*>(k.out) + size_t(t) * k.heads * vecs_per_head, k.heads * hv, hv, hv_shift, lane, ang,
          inv_dim, eps);
    __syncwarp();  // the warp's table slice is rewritten for its next token
  }
}

// ---------------------------------------------------------------------------
// Bulk-copy (TMA) form of the vector kernel, fast mode.  The register kernel above is
// bound by latency, not bandwidth: a warp's chain per token is position -> angles ->
// loads -> arithmetic -> stores, and few warps fit beside its registers.  Here lane 0 of
// each warp asks the copy engine for the NEXT token's q and k rows (one bulk copy each,
// into the warp's second shared-memory stage, tracked by an mbarrier) before the warp
// starts on the current token, so HBM reads are always one token ahead and cost no
// registers.  Persistent grid: a warp walks tokens warp_id, warp_id + all_warps, ...
// Shared memory per warp: two stages of (q row + k row) and the cos/sin table.
// ---------------------------------------------------------------------------
static __device__ unsigned int g_rope_bulk_timeouts = 0;   // bounded waits that ran out (0 in a healthy run)

// One step: the item at vector index `where` of the staged row (low half; partner at where + hv).
template <typename T, bool kNorm, int P>
__device__ __forceinline__ void rope_item_from_shared(const uint4* xs, uint4* out, int where, int hv, bool store,
                                                      const float2* wl, const float2* wh, const LaneAngles<P>& ang,
                                                      float inv_dim, float eps) {
  float2 lo[P], hi[P];
  Elem<T>::unpack2(xs[where], lo);
  Elem<T>::unpack2(xs[where + hv], hi);
  if (kNorm) {
    float2 acc = make_float2(0.0f, 0.0f);
#pragma unroll
    for (int e = 0; e < P; ++e) acc = __ffma2_rn(lo[e], lo[e], acc);
#pragma unroll
    for (int e = 0; e < P; ++e) acc = __ffma2_rn(hi[e], hi[e], acc);
    const float ss = group_sum(acc.x + acc.y, hv);
    const float inv = rsqrtf(fmaf(ss, inv_dim, eps));
    const float2 inv2 = make_float2(inv, inv);
#pragma unroll
    for (int e = 0; e < P; ++e) {
      lo[e] = __fmul2_rn(__fmul2_rn(lo[e], inv2), wl[e]);
      hi[e] = __fmul2_rn(__fmul2_rn(hi[e], inv2), wh[e]);
    }
  }
  float2 out_lo[P], out_hi[P];
#pragma unroll
  for (int e = 0; e < P; ++e) {
    out_lo[e] = __ffma2_rn(hi[e], ang.neg_s[e], __fmul2_rn(lo[e], ang.c[e]));   // a*c - b*s
    out_hi[e] = __ffma2_rn(lo[e], ang.s[e], __fmul2_rn(hi[e], ang.c[e]));       // a*s + b*c
  }
  if (store) {
    st_stream(out + where, Elem<T>::pack2(out_lo));
    st_stream(out + where + hv, Elem<T>::pack2(out_hi));
  }
}

// All heads of one tensor for one token, from the staged row.  kHv > 0 fixes hv (vectors per half head) at
// compile time.  The 32 lanes cover 32/hv heads per step, i.e. always 64 vectors: the lane's vector index simply
// advances by 64 per step, so full steps carry no index arithmetic and no predicates.
template <typename T, bool kNorm, int kHv>
__device__ __forceinline__ void rope_heads_from_shared(const uint4* xs, const uint4* w, uint4* out, int heads, int hv_rt,
                                                       int hv_shift_rt, int lane,
                                                       const LaneAngles<Elem<T>::kPerVec / 2>& ang, float inv_dim,
                                                       float eps) {
  constexpr int P = Elem<T>::kPerVec / 2;
  const int hv = kHv > 0 ? kHv : hv_rt;
  const int shift = kHv > 0 ? (kHv == 1 ? 0 : kHv == 2 ? 1 : kHv == 4 ? 2 : kHv == 8 ? 3 : kHv == 16 ? 4 : 5) : hv_shift_rt;
  const int v = lane & (hv - 1);
  float2 wl[P], wh[P];
  if (kNorm) {
    Elem<T>::unpack2(ld_reuse(w + v), wl);
    Elem<T>::unpack2(ld_reuse(w + hv + v), wh);
  }
  const int items = heads << shift;
  int where = ((lane >> shift) << (shift + 1)) + v;
  const int full = items >> 5;
  for (int i = 0; i < full; ++i, where += 2 * kWarpSize)
    rope_item_from_shared<T, kNorm, P>(xs, out, where, hv, true, wl, wh, ang, inv_dim, eps);
  if (items & 31) {
    // ragged last step: lanes past the end redo the last head (valid memory, converged shuffles) and store nothing
    const bool ok = (full << 5) + lane < items;
    const int last_where = (((items - 1) >> shift) << (shift + 1)) + v;
    rope_item_from_shared<T, kNorm, P>(xs, out, ok ? where : last_where, hv, ok, wl, wh, ang, inv_dim, eps);
  }
}

// Where the key and value rows of a token go when the kernel writes them straight into the paged KV cache
// (storage [layers, total_blocks, 2, block_size, kv_heads, head_dim], plane 0 = keys, 1 = values): token t uses
// row t / tokens_per_table of block_tables and cache position slot_positions[t] (or t % tokens_per_table).
struct PagedTarget {
  unsigned char* storage;
  const int32_t* block_tables;
  const int32_t* slot_positions;
  const unsigned char* value;      // [tokens, kv_heads, head_dim], copied unchanged into plane 1
  int64_t tokens_per_table, max_blocks, layer, total_blocks, block_size;
  int32_t* status;                 // bit 0: a block id or position out of range (that token's K/V were not written)
};

// Shared memory per warp: two stages of (q row + k row), then two cos/sin tables (one per stage).
// The table of the NEXT token is computed right after its rows have been requested and before the
// warp waits for the current rows, so the fp64 angle arithmetic runs under the copy's latency.
constexpr int kBulkWarps = 4, kBulkCtasPerSm = 4;
constexpr int kBulkFreqPerLane = kMaxTableHalf / kWarpSize;   // head_dim <= 256
constexpr int kBulkMaxStages = 4;

template <typename T, bool kNorm, int kHv, bool kPaged>
__global__ void __launch_bounds__(kBulkWarps * kWarpSize, kBulkCtasPerSm)
rope_tokens_bulk_kernel(HeadSet q, HeadSet k, const int32_t* __restrict__ positions, int64_t tokens, int head_dim, int hv,
                        int hv_shift, int64_t pos_period, float eps, float theta, int stages,
                        const __grid_constant__ InvFreq freq, const __grid_constant__ PagedTarget paged, int32_t* status) {
  constexpr int N = Elem<T>::kPerVec;
  extern __shared__ __align__(128) unsigned char bulk_smem[];
  dependent_launch_prologue();
  const int half = head_dim >> 1, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int vecs_per_head = 2 * hv;
  const int q_heads = q.heads, k_heads = k.heads;
  const uint32_t q_bytes = uint32_t(q_heads) * vecs_per_head * 16u, k_bytes = uint32_t(k_heads) * vecs_per_head * 16u;
  const uint32_t stage_bytes = q_bytes + k_bytes, table_bytes = uint32_t(head_dim) * 4u;
  const uint32_t per_warp = uint32_t(stages) * stage_bytes + 2u * table_bytes;
  unsigned char* mine = bulk_smem + size_t(warp) * per_warp;
  float* tables = reinterpret_cast<float*>(mine + uint32_t(stages) * stage_bytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(bulk_smem + size_t(warps) * per_warp) + kBulkMaxStages * warp;
  const float inv_dim = 1.0f / float(head_dim);
  const int q_vecs = q_heads * vecs_per_head, k_vecs = k_heads * vecs_per_head;
  const uint4* q_w = reinterpret_cast<const uint4*>(q.w);
  const uint4* k_w = reinterpret_cast<const uint4*>(k.w);
  uint4* q_out = reinterpret_cast<uint4*>(q.out);
  uint4* k_out = reinterpret_cast<uint4*>(k.out);

  if (lane == 0)
    for (int i = 0; i < stages; ++i) mbarrier_init(&bars[i], 1);
  __syncwarp();

  const int64_t stride = int64_t(gridDim.x) * warps;
  int64_t t = int64_t(blockIdx.x) * warps + warp;
  // lane 0 only: ask for one token's rows into a stage
  auto request = [&](int64_t token, int stage) {
    unsigned char* dst = mine + uint32_t(stage) * stage_bytes;
    mbarrier_expect_bytes(&bars[stage], stage_bytes);
    bulk_load(dst, static_cast<const unsigned char*>(q.x) + size_t(token) * q_bytes, q_bytes, &bars[stage]);
    if (k_bytes != 0u)
      bulk_load(dst + q_bytes, static_cast<const unsigned char*>(k.x) + size_t(token) * k_bytes, k_bytes, &bars[stage]);
  };
  // A lane always computes the same frequencies (lane, lane + 32, ...): their inverse wavelengths are read
  // from the parameter table once and kept in registers (a per-lane index into kernel parameters is a
  // divergent constant load, far too slow to repeat for every token).
  double lane_freq[kBulkFreqPerLane];
#pragma unroll
  for (int i = 0; i < kBulkFreqPerLane; ++i) lane_freq[i] = lane + i * kWarpSize < half ? freq.v[lane + i * kWarpSize] : 0.0;
  // every lane: cos/sin of one token's frequencies into one of the two tables
  auto fill_table = [&](int32_t p, int which) {
    float* cos_row = tables + which * head_dim;
    const double two_pi_hi = 6.283185307179586232e+00, two_pi_lo = 2.449293598294706414e-16;
#pragma unroll
    for (int i = 0; i < kBulkFreqPerLane; ++i) {
      const int j = lane + i * kWarpSize;
      if (j < half) {
        // as rope_cos_sin<false>: fp64 angle, fp64 reduction to [-pi, pi], hardware sine/cosine
        const double angle = double(p) * lane_freq[i];
        const double turns = rint(angle * 1.591549430918953456e-01);
        const float rf = float(fma(-turns, two_pi_lo, fma(-turns, two_pi_hi, angle)));
        cos_row[j] = __cosf(rf);
        cos_row[half + j] = __sinf(rf);
      }
    }
  };
  auto position_of = [&](int64_t token) { return token < tokens ? positions[pos_period ? token % pos_period : token] : 0; };
  // positions are fetched two tokens ahead of their use, so that no step waits for that load
  int32_t p_next = position_of(t + stride);
  if (t < tokens) {
    if (lane == 0)
      for (int i = 0; i < stages - 1 && t + i * stride < tokens; ++i) request(t + i * stride, i);
    fill_table(position_of(t), 0);
  }

  int stage = 0;        // it % stages
  uint32_t round = 0;   // it / stages
  for (int it = 0; t < tokens; ++it, t += stride) {
    const int64_t t_next = t + stride, t_ahead = t + (stages - 1) * stride;
    const int32_t p_after = position_of(t_next + stride);
    // the stage that the previous step read is free: every lane passed the __syncwarp that ends that step
    // after consuming what it read
    if (lane == 0 && t_ahead < tokens) {
      fence_before_bulk_copy();
      request(t_ahead, stage == 0 ? stages - 1 : stage - 1);
    }
    if (t_next < tokens) fill_table(p_next, (it + 1) & 1);
    p_next = p_after;
    __syncwarp();   // this step's table (written one step ago, or before the loop) is visible to every lane
    LaneAngles<N / 2> ang;
    const float* cos_row = tables + (it & 1) * head_dim;
    const int first = (lane & (hv - 1)) * N;
#pragma unroll
    for (int e = 0; e < N / 2; ++e) {
      ang.c[e] = *reinterpret_cast<const float2*>(cos_row + first + 2 * e);
      ang.s[e] = *reinterpret_cast<const float2*>(cos_row + half + first + 2 * e);
      ang.neg_s[e] = make_float2(-ang.s[e].x, -ang.s[e].y);
    }

    // the whole warp takes one decision (a lane whose wait succeeded at the last moment must not part from the rest)
    if (!__all_sync(0xffffffffu, mbarrier_wait_bounded(&bars[stage], round & 1u))) {
      // never expected: record it, give every stage's copy one more bounded chance to land, and stop
      if (lane == 0) {
        atomicAdd(&g_rope_bulk_timeouts, 1u);
        if (status != nullptr) atomicOr(status, kPaged ? 2 : 1);   // this call's outputs are incomplete
      }
      for (int i = 0; i < stages && t + i * stride < tokens; ++i) {   // copies in flight: tokens t .. t_ahead
        const bool wrapped = stage + i >= stages;
        mbarrier_wait_bounded(&bars[wrapped ? stage + i - stages : stage + i], (wrapped ? round + 1u : round) & 1u);
      }
      break;
    }
    const uint4* xs = reinterpret_cast<const uint4*>(mine + uint32_t(stage) * stage_bytes);
    rope_heads_from_shared<T, kNorm, kHv>(xs, q_w, q_out + size_t(t) * q_vecs, q_heads, hv, hv_shift, lane, ang, inv_dim, eps);
    if (kPaged) {
      // the key row goes to its slot of the paged cache, and the value row is copied beside it
      const int64_t table_row = t / paged.tokens_per_table;
      const int64_t position = paged.slot_positions != nullptr ? int64_t(paged.slot_positions[t]) : t - table_row * paged.tokens_per_table;
      bool ok = position >= 0 && position / paged.block_size < paged.max_blocks;
      int64_t block = 0;
      if (ok) {
        block = paged.block_tables[table_row * paged.max_blocks + position / paged.block_size];
        ok = block >= 0 && block < paged.total_blocks;
      }
      if (ok) {
        const int64_t row_bytes = int64_t(k_vecs) * 16;
        unsigned char* key_row = paged.storage +
            ((((paged.layer * paged.total_blocks + block) * 2) * paged.block_size + position % paged.block_size) * row_bytes);
        uint4* value_row = reinterpret_cast<uint4*>(key_row + paged.block_size * row_bytes);
        const uint4* value_src = reinterpret_cast<const uint4*>(paged.value) + size_t(t) * k_vecs;
        uint4 held[4];                       // the value row's loads fly under the key heads' arithmetic
#pragma unroll
        for (int i = 0; i < 4; ++i) if (lane + i * kWarpSize < k_vecs) held[i] = ld_stream(value_src + lane + i * kWarpSize);
        rope_heads_from_shared<T, kNorm, kHv>(xs + q_vecs, k_w, reinterpret_cast<uint4*>(key_row), k_heads, hv, hv_shift, lane,
                                              ang, inv_dim, eps);
#pragma unroll
        for (int i = 0; i < 4; ++i) if (lane + i * kWarpSize < k_vecs) st_stream(value_row + lane + i * kWarpSize, held[i]);
        for (int i = lane + 4 * kWarpSize; i < k_vecs; i += kWarpSize) st_stream(value_row + i, ld_stream(value_src + i));
      } else if (lane == 0 && paged.status != nullptr) {
        atomicOr(paged.status, 1);
      }
    } else if (k_heads > 0) {
      rope_heads_from_shared<T, kNorm, kHv>(xs + q_vecs, k_w, k_out + size_t(t) * k_vecs, k_heads, hv, hv_shift, lane, ang,
                                            inv_dim, eps);
    }
    __syncwarp();   // stage and table are free again
    if (++stage == stages) { stage = 0; ++round; }
  }
}

// ---------------------------------------------------------------------------
// Scalar kernel for shapes the vector kernel cannot take (tiny or odd head_dim,
// unaligned views): one (low, high) pair per thread per step.  With kNorm one warp
// owns a head and reduces it with shuffles.
// ---------------------------------------------------------------------------
template <typename T, bool kOrdered>
__global__ void __launch_bounds__(kThreads)
rope_scalar_kernel(const T* x, const int32_t* __restrict__ positions, T* out, int64_t tokens, int64_t heads,
                   int head_dim, int64_t pos_period, float theta, const __grid_constant__ InvFreq freq) {
  const int half = head_dim >> 1;
  const int64_t total = tokens * heads * half;
  for (int64_t i = int64_t(blockIdx.x) * kThreads + threadIdx.x; i < total; i += int64_t(gridDim.x) * kThreads) {
    const int j = int(i % half);
    const int64_t th = i / half, t = th / heads;
    const int32_t p = positions[pos_period ? t % pos_period : t];
    const float2 cs = rope_cos_sin<kOrdered>(p, j, head_dim, theta, freq, half);
    const int64_t base = th * head_dim;
    const float a = Elem<T>::load(x + base + j), b = Elem<T>::load(x + base + half + j);
    float lo, hi;
    rotate<kOrdered>(a, b, cs, lo, hi);
    Elem<T>::store(out + base + j, lo);
    Elem<T>::store(out + base + half + j, hi);
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
norm_rope_scalar_kernel(const T* x, const T* __restrict__ w, const int32_t* __restrict__ positions, T* out,
                        int64_t tokens, int64_t heads, int head_dim, float eps, float theta,
                        const __grid_constant__ InvFreq freq) {
  const int half = head_dim >> 1, lane = threadIdx.x & 31;
  const int64_t warps = int64_t(gridDim.x) * (kThreads / kWarpSize);
  for (int64_t th = int64_t(blockIdx.x) * (kThreads / kWarpSize) + (threadIdx.x >> 5); th < tokens * heads;
       th += warps) {
    const int64_t base = th * head_dim;
    const int32_t p = positions[th / heads];
    float ss = 0.0f;
    for (int j = lane; j < head_dim; j += kWarpSize) { const float v = Elem<T>::load(x + base + j); ss = fmaf(v, v, ss); }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / float(head_dim) + eps);
    for (int j = lane; j < half; j += kWarpSize) {
      const float a = __fmul_rn(__fmul_rn(Elem<T>::load(x + base + j), inv), Elem<T>::load(w + j));
      const float b = __fmul_rn(__fmul_rn(Elem<T>::load(x + base + half + j), inv), Elem<T>::load(w + half + j));
      const float2 cs = rope_cos_sin<false>(p, j, head_dim, theta, freq, half);
      float lo, hi;
      rotate<false>(a, b, cs, lo, hi);
      // a lane reads both of its elements before it writes either: in-place use is safe
      Elem<T>::store(out + base + j, lo);
      Elem<T>::store(out + base + half + j, hi);
    }
  }
}

InvFreq make_table(int64_t head_dim, float theta) {
  InvFreq f;
  const int64_t half = head_dim / 2;
  for (int64_t j = 0; j < kMaxTableHalf; ++j)
    f.v[j] = j < half ? std::pow(double(theta), -2.0 * double(j) / double(head_dim)) : 0.0;
  return f;
}

template <typename T> bool vector_shape_ok(int64_t head_dim, int* hv_out) {
  constexpr int N = Elem<T>::kPerVec;
  const int64_t half = head_dim / 2;
  if (half % N != 0) return false;
  const int64_t hv = half / N;
  if (hv > 32 || (hv & (hv - 1)) != 0) return false;
  *hv_out = int(hv);
  return true;
}

template <typename T, bool kNorm>
bool launch_bulk(HeadSet q, HeadSet k, const int32_t* positions, int64_t tokens, int64_t head_dim, int hv, int hv_shift,
                 int64_t pos_period, float eps, float theta, int32_t* status, cudaStream_t s, const PagedTarget* paged = nullptr) {
  constexpr int stages = 2, max_warps = kBulkWarps;   // deeper prefetch and other warp counts measured no faster
  const size_t stage = size_t(q.heads + k.heads) * size_t(2 * hv) * 16, per_warp = stages * stage + 2 * size_t(head_dim) * 4;
  const size_t bar_bytes = size_t(kBulkMaxStages) * 8;
  const size_t budget = (227 * 1024) / kBulkCtasPerSm - 1024;   // kBulkCtasPerSm CTAs share one SM's shared memory
  int warps = int(budget / (per_warp + bar_bytes));
  if (warps < 1 || head_dim / 2 > kMaxTableHalf) return false;   // rows too long for the stages: the register kernel takes over
  if (warps > max_warps) warps = max_warps;
  if (int64_t(warps) > tokens) warps = int(tokens);
  const size_t smem = size_t(warps) * (per_warp + bar_bytes);
  // the head size of the model family gets hv fixed at compile time (head_dim 128: 8 vectors of fp16, 16 of fp32
  // per half head); fixing the head counts as well measured no faster
  auto kernel = hv == 8 ? rope_tokens_bulk_kernel<T, kNorm, 8, false> : hv == 16 ? rope_tokens_bulk_kernel<T, kNorm, 16, false>
                                                                                 : rope_tokens_bulk_kernel<T, kNorm, 0, false>;
  if (paged != nullptr)
    kernel = hv == 8 ? rope_tokens_bulk_kernel<T, kNorm, 8, true> : hv == 16 ? rope_tokens_bulk_kernel<T, kNorm, 16, true>
                                                                             : rope_tokens_bulk_kernel<T, kNorm, 0, true>;
  if (smem > 48 * 1024 && cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  const int64_t ctas = (tokens + warps - 1) / warps, cap = int64_t(sm_count()) * kBulkCtasPerSm;
  launch_kernel(kernel, dim3(unsigned(ctas < cap ? ctas : cap)), dim3(warps * kWarpSize), smem, s, q, k, positions, tokens,
                int(head_dim), hv, hv_shift, pos_period, eps, theta, stages, make_table(head_dim, theta),
                paged != nullptr ? *paged : PagedTarget{}, paged != nullptr ? paged->status : status);
  return true;
}

template <typename T, bool kNorm, bool kOrdered>
int launch_vector(HeadSet q, HeadSet k, const int32_t* positions, int64_t tokens, int64_t head_dim, int hv,
                  int64_t pos_period, float eps, float theta, int32_t* status, cudaStream_t s, const char* what) {
  if (!kOrdered) {
    int shift = 0;
    while ((1 << shift) < hv) ++shift;
    if (launch_bulk<T, kNorm>(q, k, positions, tokens, head_dim, hv, shift, pos_period, eps, theta, status, s)) return launch_status(what);
  }
  const int64_t ctas = (tokens + kWarpsPerCta - 1) / kWarpsPerCta, cap = int64_t(sm_count()) * 64;
  const unsigned grid = unsigned(ctas < cap ? ctas : cap);
  const size_t smem = size_t(kWarpsPerCta) * size_t(head_dim) * sizeof(float);
  int hv_shift = 0;
  while ((1 << hv_shift) < hv) ++hv_shift;
  launch_kernel(rope_tokens_kernel<T, kNorm, kOrdered>, dim3(grid), dim3(kThreads), smem, s, q, k, positions, tokens,
                int(head_dim), hv, hv_shift, pos_period, eps, theta, make_table(head_dim, theta));
  return launch_status(what);
}

template <typename T>
int launch_rope_typed(const void* x, const int32_t* positions, void* out, int64_t tokens, int64_t heads,
                      int64_t head_dim, int64_t pos_period, float theta, int mode, int32_t* status, cudaStream_t s) {
  if (tokens == 0 || heads == 0 || head_dim == 0) return B2_OK;
  int hv = 0;
  const bool vec = vector_shape_ok<T>(head_dim, &hv) && aligned16(x) && aligned16(out) && heads <= (1 << 20);
  if (vec) {
    HeadSet q{x, nullptr, out, int(heads)}, none{nullptr, nullptr, nullptr, 0};
    return mode == B2_DETERMINISTIC
               ? launch_vector<T, false, true>(q, none, positions, tokens, head_dim, hv, pos_period, 0.f, theta, status, s,
                                               "rope (deterministic)")
               : launch_vector<T, false, false>(q, none, positions, tokens, head_dim, hv, pos_period, 0.f, theta, status, s,
                                                "rope");
  }
  const int64_t total = tokens * heads * (head_dim / 2);
  const int64_t blocks = (total + kThreads - 1) / kThreads, cap = int64_t(sm_count()) * 8;
  const unsigned grid = unsigned(blocks < cap ? blocks : cap);
  const InvFreq table = make_table(head_dim, theta);
  if (mode == B2_DETERMINISTIC)
    rope_scalar_kernel<T, true><<<grid, kThreads, 0, s>>>(static_cast<const T*>(x), positions, static_cast<T*>(out),
                                                          tokens, heads, int(head_dim), pos_period, theta, table);
  else
    rope_scalar_kernel<T, false><<<grid, kThreads, 0, s>>>(static_cast<const T*>(x), positions, static_cast<T*>(out),
                                                           tokens, heads, int(head_dim), pos_period, theta, table);
  return launch_status("rope (scalar)");
}

template <typename T>
int launch_qk_typed(const void* q, const void* k, const void* qw, const void* kw, const int32_t* positions,
                    void* q_out, void* k_out, int64_t tokens, int64_t q_heads, int64_t k_heads, int64_t head_dim,
                    float eps, float theta, int32_t* status, cudaStream_t s) {
  if (tokens == 0 || head_dim == 0 || q_heads + k_heads == 0) return B2_OK;
  int hv = 0;
  const bool vec = vector_shape_ok<T>(head_dim, &hv) && aligned16(q) && aligned16(q_out) && aligned16(qw) &&
                   (k_heads == 0 || (aligned16(k) && aligned16(k_out) && aligned16(kw))) &&
                   q_heads + k_heads <= (1 << 20);
  if (vec) {
    HeadSet qs{q, qw, q_out, int(q_heads)}, ks{k, kw, k_out, int(k_heads)};
    return launch_vector<T, true, false>(qs, ks, positions, tokens, head_dim, hv, 0, eps, theta, status, s, "qk_norm_rope");
  }
  const InvFreq table = make_table(head_dim, theta);
  const int warps_per_cta = kThreads / kWarpSize;
  const int64_t cap = int64_t(sm_count()) * 8;
  for (int pass = 0; pass < 2; ++pass) {
    const int64_t heads = pass == 0 ? q_heads : k_heads;
    if (heads == 0) continue;
    const int64_t blocks = (tokens * heads + warps_per_cta - 1) / warps_per_cta;
    norm_rope_scalar_kernel<T><<<unsigned(blocks < cap ? blocks : cap), kThreads, 0, s>>>(
        static_cast<const T*>(pass == 0 ? q : k), static_cast<const T*>(pass == 0 ? qw : kw), positions,
        static_cast<T*>(pass == 0 ? q_out : k_out), tokens, heads, int(head_dim), eps, theta, table);
  }
  return launch_status("qk_norm_rope (scalar)");
}

}  // namespace

int rope_bulk_timeouts(unsigned int* out) {
  return cudaMemcpyFromSymbol(out, g_rope_bulk_timeouts, sizeof(unsigned int)) == cudaSuccess ? B2_OK : launch_status("b2_bulk_copy_timeouts");
}

int launch_rope(const void* x, const int32_t* positions, void* out, int64_t tokens, int64_t heads, int64_t head_dim,
                int64_t pos_period, float theta, int dtype, int mode, int32_t* status, cudaStream_t s) {
  return dtype == B2_F32
             ? launch_rope_typed<float>(x, positions, out, tokens, heads, head_dim, pos_period, theta, mode, status, s)
             : launch_rope_typed<__half>(x, positions, out, tokens, heads, head_dim, pos_period, theta, mode, status, s);
}

int launch_qk_norm_rope(const void* q, const void* k, const void* qw, const void* kw, const int32_t* positions,
                        void* q_out, void* k_out, int64_t tokens, int64_t q_heads, int64_t k_heads, int64_t head_dim,
                        float eps, float theta, int dtype, int32_t* status, cudaStream_t s) {
  return dtype == B2_F32 ? launch_qk_typed<float>(q, k, qw, kw, positions, q_out, k_out, tokens, q_heads, k_heads,
                                                  head_dim, eps, theta, status, s)
                         : launch_qk_typed<__half>(q, k, qw, kw, positions, q_out, k_out, tokens, q_heads, k_heads,
                                                   head_dim, eps, theta, status, s);
}

// Fused form that leaves the keys and values in the paged KV cache.  Only the vector (bulk-copy) kernel has it:
// B2_ERR_UNSUPPORTED for shapes or alignments it cannot take, and the caller runs the separate operators instead.
int launch_qk_norm_rope_paged(const void* q, const void* k, const void* v, const void* qw, const void* kw,
                              const int32_t* positions, void* q_out, void* storage, const int32_t* block_tables,
                              const int32_t* slot_positions, int64_t tokens, int64_t q_heads, int64_t k_heads,
                              int64_t head_dim, float eps, float theta, int64_t tokens_per_table, int64_t max_blocks,
                              int64_t layer, int64_t total_blocks, int64_t block_size, int dtype, int32_t* status,
                              cudaStream_t s) {
  if (tokens == 0) return B2_OK;
  PagedTarget paged{static_cast<unsigned char*>(storage), block_tables, slot_positions, static_cast<const unsigned char*>(v),
                    tokens_per_table, max_blocks, layer, total_blocks, block_size, status};
  HeadSet qs{q, qw, q_out, int(q_heads)}, ks{k, kw, nullptr, int(k_heads)};
  const bool aligned = aligned16(q) && aligned16(q_out) && aligned16(qw) && aligned16(k) && aligned16(kw) && aligned16(v) &&
                       aligned16(storage);
  int hv = 0, shift = 0;
  bool launched = false;
  if (dtype == B2_F32) {
    if (aligned && vector_shape_ok<float>(head_dim, &hv)) {
      while ((1 << shift) < hv) ++shift;
      launched = launch_bulk<float, true>(qs, ks, positions, tokens, head_dim, hv, shift, 0, eps, theta, status, s, &paged);
    }
  } else if (aligned && vector_shape_ok<__half>(head_dim, &hv)) {
    while ((1 << shift) < hv) ++shift;
    launched = launch_bulk<__half, true>(qs, ks, positions, tokens, head_dim, hv, shift, 0, eps, theta, status, s, &paged);
  }
  if (!launched) {
    set_error("b2_qk_norm_rope_paged: this shape or alignment has no fused kernel; use b2_qk_norm_rope and b2_paged_kv_write_*");
    return B2_ERR_UNSUPPORTED;
  }
  return launch_status("qk_norm_rope_paged");
}

}  // namespace b2
