/*
 * CPU oracle for the tensor-op hot path.  TEST INFRASTRUCTURE ONLY: this file is
 * the checker that the CUDA kernels are compared against; nothing on the product
 * path may call it.
 *
 * Two families of functions live here:
 *
 *  orc_cpu_*   restate the reference's CPU operators (reference src/ops_cpu.cpp),
 *              fp32 in / fp32 out, same operation order, same libm calls.
 *  orc_dev_*   restate the arithmetic of the reference's CUDA kernels
 *              (reference src/ops_cuda.cu) for the ops whose device arithmetic is
 *              IEEE-exact (add, RMSNorm, fused add+RMSNorm, gather, argmax): the
 *              "deterministic mode" of the product must reproduce these bit for bit.
 *
 * Build with -O2 -ffp-contract=off and no -march flag: the reference's own build
 * targets baseline x86-64 (no FMA), so none of its products are fused.
 *
 * Parity status: pinned.  tests/test_oracle_golden.py checks every orc_cpu_*
 * function against the closed-form answers of the reference's tests/test_ops_cpu.cpp,
 * against the layer-0 activation fixtures exported by the reference
 * (artifacts/phase1/qwen3_layer0) and, when oracle/_ref is built, bit for bit
 * against the reference's own compiled ops_cpu.
 */
#include <math.h>
#include <stdlib.h>
#include <stdint.h>
#include <string.h>
#include <float.h>

#define ORC_API __attribute__((visibility("default")))

/* ---------------------------------------------------------------- fp16 codecs */

static uint32_t f32_bits(float x) { uint32_t u; memcpy(&u, &x, 4); return u; }
static float bits_f32(uint32_t u) { float x; memcpy(&x, &u, 4); return x; }

/* Exact half -> float widening (every half value is representable).
 * Same mapping as reference src/tensor.cpp:13 (decode_f16). */
ORC_API float orc_decode_f16(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  const int exp = (h >> 10) & 31;
  const uint32_t man = h & 1023u;
  if (exp == 31) return bits_f32(sign | 0x7f800000u | (man << 13));
  if (exp == 0) {
    /* zero or subnormal: man * 2^-24, exact in fp32 */
    float v = ldexpf((float)man, -24);
    return sign ? -v : v;
  }
  return bits_f32(sign | ((uint32_t)(exp + 112) << 23) | (man << 13));
}

/* float -> half, round-to-nearest-even: the rounding of the device's
 * __float2half used by every reference kernel store (src/ops_cuda.cu:75, wf<__half>). */
ORC_API uint16_t orc_f32_to_f16_rn(float x) {
  const uint32_t u = f32_bits(x);
  const uint16_t sign = (uint16_t)((u >> 16) & 0x8000u);
  const uint32_t a = u & 0x7fffffffu;
  if (a > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);           /* NaN */
  if (a >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);          /* >= 65520 -> inf */
  if (a < 0x33000001u) return sign;                                  /* <= 2^-25 -> 0 (tie to even) */
  int e = (int)(a >> 23) - 127;
  uint32_t m = (a & 0x7fffffu) | 0x800000u;                          /* 24-bit significand */
  int shift;                                                         /* bits dropped */
  uint32_t base;
  if (e >= -14) { shift = 13; base = (uint32_t)(e + 15) << 10; m &= 0x7fffffu; }
  else { shift = 13 + (-14 - e); base = 0; }
  uint32_t q = m >> shift;
  const uint32_t rem = m & ((1u << shift) - 1u);
  const uint32_t halfway = 1u << (shift - 1);
  if (rem > halfway || (rem == halfway && (q & 1u))) q += 1;         /* carries propagate into the exponent */
  return (uint16_t)(sign | (base + q));
}

/* The reference's HOST encoder (src/tensor.cpp:12, encode_f16): truncates normal
 * numbers instead of rounding them.  Kept only so tests can show that fixtures
 * must never be quantised with it. */
ORC_API uint16_t orc_encode_f16_host(float x) {
  const uint32_t u = f32_bits(x);
  const uint32_t sign = (u >> 16) & 0x8000u, e = (u >> 23) & 255u;
  uint32_t m = u & 0x7fffffu;
  if (e == 255) return (uint16_t)(sign | 0x7c00u | (m ? 0x200u : 0u));
  const int ne = (int)e - 127 + 15;
  if (ne >= 31) return (uint16_t)(sign | 0x7c00u);
  if (ne <= 0) {
    if (ne < -10) return (uint16_t)sign;
    m |= 0x800000u;
    return (uint16_t)(sign | ((m >> (14 - ne)) + ((m >> (13 - ne)) & 1u)));
  }
  return (uint16_t)(sign | ((uint32_t)ne << 10) | (m >> 13));
}

ORC_API void orc_decode_f16_array(const uint16_t* in, float* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = orc_decode_f16(in[i]);
}
ORC_API void orc_f32_to_f16_rn_array(const float* in, uint16_t* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = orc_f32_to_f16_rn(in[i]);
}

/* ------------------------------------------------- CPU operators (ops_cpu.cpp) */

/* reference src/ops_cpu.cpp:8 (embedding_lookup): row copy with host bounds check.
 * Returns 0, or -1 when an id is outside [0, vocab). */
ORC_API int orc_cpu_embedding_lookup(const float* table, int64_t vocab, int64_t hidden,
                                     const int32_t* ids, int64_t count, float* out) {
  for (int64_t t = 0; t < count; ++t) {
    if (ids[t] < 0 || (int64_t)ids[t] >= vocab) return -1;
    memcpy(out + t * hidden, table + (int64_t)ids[t] * hidden, (size_t)hidden * sizeof(float));
  }
  return 0;
}

/* reference src/ops_cpu.cpp:9 (linear) and :17 (lm_head = linear): out[i, j] = sum_k x[i, k] * w[j, k],
 * one fp32 accumulator per output, k ascending, product rounded before it is added (the reference
 * builds for baseline x86-64: no fused multiply-add). */
ORC_API void orc_cpu_linear(const float* x, const float* w, int64_t rows, int64_t in, int64_t out_features,
                            float* out) {
  for (int64_t i = 0; i < rows; ++i)
    for (int64_t j = 0; j < out_features; ++j) {
      float z = 0.0f;
      for (int64_t k = 0; k < in; ++k) z += x[i * in + k] * w[j * in + k];  /* built with -ffp-contract=off */
      out[i * out_features + j] = z;
    }
}

/* reference src/ops_cpu.cpp:10 (rms_norm): fp32 running sum of squares in index
 * order, r = 1/sqrt(sum/H + eps) in fp32, out = (x*r)*w. */
ORC_API void orc_cpu_rms_norm(const float* x, const float* w, float eps,
                              int64_t rows, int64_t hidden, float* out) {
  for (int64_t i = 0; i < rows; ++i) {
    const float* row = x + i * hidden;
    float acc = 0.0f;
    for (int64_t j = 0; j < hidden; ++j) { const float v = row[j]; acc += v * v; }
    const float r = 1.0f / sqrtf(acc / (float)hidden + eps);
    for (int64_t j = 0; j < hidden; ++j) out[i * hidden + j] = row[j] * r * w[j];
  }
}

/* reference src/ops_cpu.cpp:16 (add). */
ORC_API void orc_cpu_add(const float* a, const float* b, int64_t n, float* out) {
  for (int64_t i = 0; i < n; ++i) out[i] = a[i] + b[i];
}

/* reference src/ops_cpu.cpp:15 (swiglu): silu(gate)*up with the float exp. */
ORC_API void orc_cpu_swiglu(const float* gate, const float* up, int64_t n, float* out) {
  for (int64_t i = 0; i < n; ++i) {
    const float g = gate[i];
    out[i] = (g / (1.0f + expf(-g))) * up[i];
  }
}

/* reference src/ops_cpu.cpp:11 (rope): NeoX rotate-half on [T,H,D]; the angle and
 * its power are double, sin/cos are double then narrowed, the rotation is fp32.
 * Returns 0, or -1 for an odd head_dim / non-positive theta. */
ORC_API int orc_cpu_rope(const float* x, const int32_t* positions, float theta,
                         int64_t tokens, int64_t heads, int64_t head_dim, float* out) {
  if (head_dim % 2 != 0 || !(theta > 0.0f)) return -1;
  const int64_t half = head_dim / 2;
  for (int64_t t = 0; t < tokens; ++t)
    for (int64_t h = 0; h < heads; ++h) {
      const int64_t base = (t * heads + h) * head_dim;
      for (int64_t i = 0; i < half; ++i) {
        const double angle = (double)positions[t] *
                             pow((double)theta, -2.0 * (double)i / (double)head_dim);
        const float c = (float)cos(angle), s = (float)sin(angle);
        const float a = x[base + i], b = x[base + i + half];
        out[base + i] = a * c - b * s;
        out[base + i + half] = a * s + b * c;
      }
    }
  return 0;
}

/* reference src/ops_cpu.cpp:13 (softmax_last_dim): max from -inf, exp stored,
 * fp32 running sum in index order, then divide. */
ORC_API void orc_cpu_softmax(const float* x, int64_t rows, int64_t width, float* out) {
  for (int64_t r = 0; r < rows; ++r) {
    const float* row = x + r * width;
    float* o = out + r * width;
    float m = -INFINITY;
    for (int64_t j = 0; j < width; ++j) m = row[j] > m ? row[j] : m; /* std::max(m, v) */
    float z = 0.0f;
    for (int64_t j = 0; j < width; ++j) { const float e = expf(row[j] - m); o[j] = e; z += e; }
    for (int64_t j = 0; j < width; ++j) o[j] = o[j] / z;
  }
}

/* Softmax with a double accumulator: not a reference function.  It exists so the
 * tests can report how far the reference's own fp32 running sum is from the
 * exact answer at vocabulary width. */
ORC_API void orc_f64_softmax(const float* x, int64_t rows, int64_t width, double* out) {
  for (int64_t r = 0; r < rows; ++r) {
    const float* row = x + r * width;
    double* o = out + r * width;
    double m = -INFINITY;
    for (int64_t j = 0; j < width; ++j) m = row[j] > m ? (double)row[j] : m;
    double z = 0.0;
    for (int64_t j = 0; j < width; ++j) { o[j] = exp((double)row[j] - m); z += o[j]; }
    for (int64_t j = 0; j < width; ++j) o[j] /= z;
  }
}

/* Row argmax.  The reference has no CPU argmax; this follows its device rule
 * (src/ops_cuda.cu:562-563): start from (best = -FLT_MAX, id = 0), replace on
 * value > best or (value == best and index < id).  Scanning in ascending index
 * order makes the second clause unreachable, so: first element strictly greater
 * than everything before it; NaN, -inf and -FLT_MAX never win; nothing wins -> 0.
 * The source writes the start value as -CUDART_INF_F.  None of the headers that file includes defines that macro
 * (checked by preprocessing its include list with CUDA 12.9), so the file's own fallback applies: 3.402823466e+38F
 * (src/ops_cuda.cu:21-23), i.e. FLT_MAX, not infinity.  tests/test_gpu_reference_cuda.py asks the reference's
 * compiled kernel about rows that tell the two readings apart. */
ORC_API int32_t orc_argmax_row_f32(const float* x, int64_t width) {
  float best = -FLT_MAX;
  int32_t best_id = 0;
  for (int64_t i = 0; i < width; ++i)
    if (x[i] > best) { best = x[i]; best_id = (int32_t)i; }
  return best_id;
}
ORC_API int32_t orc_argmax_row_f16(const uint16_t* x, int64_t width) {
  float best = -FLT_MAX;
  int32_t best_id = 0;
  for (int64_t i = 0; i < width; ++i) {
    const float v = orc_decode_f16(x[i]);
    if (v > best) { best = v; best_id = (int32_t)i; }
  }
  return best_id;
}
ORC_API void orc_argmax_rows_f32(const float* x, int64_t rows, int64_t width, int32_t* out) {
  for (int64_t r = 0; r < rows; ++r) out[r] = orc_argmax_row_f32(x + r * width, width);
}

/* ------------------------------ device-order arithmetic (ops_cuda.cu kernels) */

/* dtype codes shared with the product's C ABI: 0 = fp32, 1 = fp16 */
static float load_elem(const void* p, int64_t i, int dtype) {
  return dtype == 0 ? ((const float*)p)[i] : orc_decode_f16(((const uint16_t*)p)[i]);
}
static void store_elem(void* p, int64_t i, int dtype, float v) {
  if (dtype == 0) ((float*)p)[i] = v; else ((uint16_t*)p)[i] = orc_f32_to_f16_rn(v);
}

/* reference src/ops_cuda.cu:76 (addk): round_T(float(a)+float(b)). */
ORC_API void orc_dev_add(const void* a, const void* b, int64_t n, void* out, int dtype) {
  for (int64_t i = 0; i < n; ++i) store_elem(out, i, dtype, load_elem(a, i, dtype) + load_elem(b, i, dtype));
}

static float dev_inverse_rms(double sum, int64_t hidden, float eps) {
  return (float)(1.0 / sqrt(sum / (double)hidden + (double)eps));
}

/* reference src/ops_cuda.cu:112-131 (rmsk): double running sum of exact squares in
 * index order; inv narrowed to fp32; out = round_T(rn(rn(x*inv)*w)). */
ORC_API void orc_dev_rms_norm(const void* x, const void* w, float eps,
                              int64_t rows, int64_t hidden, void* out, int dtype) {
  for (int64_t r = 0; r < rows; ++r) {
    double sum = 0.0;
    for (int64_t j = 0; j < hidden; ++j) {
      const float v = load_elem(x, r * hidden + j, dtype);
      sum += (double)v * (double)v;
    }
    const float inv = dev_inverse_rms(sum, hidden, eps);
    for (int64_t j = 0; j < hidden; ++j) {
      const float scaled = load_elem(x, r * hidden + j, dtype) * inv;
      store_elem(out, r * hidden + j, dtype, scaled * load_elem(w, j, dtype));
    }
  }
}

/* reference src/ops_cuda.cu:77-99 (add_rms_normk): v = lhs+rhs in fp32; residual =
 * round_T(v); the sum uses the UNROUNDED v; the normalised output re-reads the
 * ROUNDED residual. */
ORC_API void orc_dev_add_rms_norm(const void* lhs, const void* rhs, const void* w, float eps,
                                  int64_t rows, int64_t hidden,
                                  void* residual, void* normalized, int dtype) {
  for (int64_t r = 0; r < rows; ++r) {
    double sum = 0.0;
    for (int64_t j = 0; j < hidden; ++j) {
      const int64_t k = r * hidden + j;
      const float v = load_elem(lhs, k, dtype) + load_elem(rhs, k, dtype);
      store_elem(residual, k, dtype, v);
      sum += (double)v * (double)v;
    }
    const float inv = dev_inverse_rms(sum, hidden, eps);
    for (int64_t j = 0; j < hidden; ++j) {
      const int64_t k = r * hidden + j;
      const float scaled = load_elem(residual, k, dtype) * inv;
      store_elem(normalized, k, dtype, scaled * load_elem(w, j, dtype));
    }
  }
}

/* Packed (value, index) key used when a row's vocabulary is split over several
 * GPUs: signed 64-bit max over the shards' keys == (largest value, lowest global
 * index), the reference's tie rule.  Non-candidates (NaN, -inf, -FLT_MAX) give the
 * minimum key, which decodes to index 0 like the reference's initial state. */
ORC_API int64_t orc_argmax_key(float value, int64_t global_index) {
  if (!(value > -FLT_MAX)) return INT64_MIN;
  int32_t s = (int32_t)f32_bits(value);
  if (s < 0) s ^= 0x7fffffff;                       /* order negative floats */
  return (int64_t)(((uint64_t)(uint32_t)s << 32) | (uint64_t)(0xffffffffu - (uint32_t)global_index));
}
ORC_API int32_t orc_argmax_key_index(int64_t key) {
  if (key == INT64_MIN) return 0;
  return (int32_t)(0xffffffffu - (uint32_t)((uint64_t)key & 0xffffffffu));
}

/* ------------------------------------------------------------ timing helpers */

/* The reference's fused op has no CPU twin; on the CPU it is add followed by
 * rms_norm (src/qwen3_layer.cpp:48-49).  Used as the "port" CPU baseline. */
ORC_API void orc_cpu_add_rms_norm(const float* lhs, const float* rhs, const float* w, float eps,
                                  int64_t rows, int64_t hidden, float* residual, float* normalized) {
  orc_cpu_add(lhs, rhs, rows * hidden, residual);
  orc_cpu_rms_norm(residual, w, eps, rows, hidden, normalized);
}

/* Temperature / top-k / top-p sampling of one row, following the reference's CudaSampler
 * (src/ops_cuda.cu:575-617: sampler_fill, a stable descending sort of the scores, sampler_select;
 * hash and uniform draw :581-586,606-608).  The reference has no CPU sampler; this restates its
 * device algorithm with libm's expf, so a decision that hangs on the last bits of a running sum can
 * differ from the device.  `margin` (may be NULL) receives the smallest relative gap of any
 * comparison that decided the result: when it is well above 1e-6 the token is unambiguous. */
typedef struct { uint32_t ordered; int32_t id; float score; } orc_sample_item;
static int orc_sample_cmp(const void* a, const void* b) {
  const orc_sample_item* x = (const orc_sample_item*)a;
  const orc_sample_item* y = (const orc_sample_item*)b;
  if (x->ordered != y->ordered) return x->ordered > y->ordered ? -1 : 1;   /* higher score first */
  return x->id < y->id ? -1 : (x->id > y->id ? 1 : 0);                      /* stable: lower id first */
}
static uint64_t orc_sample_mix(uint64_t x) {
  x += 0x9e3779b97f4a7c15ULL;
  x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ULL;
  x = (x ^ (x >> 27)) * 0x94d049bb133111ebULL;
  return x ^ (x >> 31);
}
ORC_API int32_t orc_sample_row(const float* logits, int64_t n, float temperature, int32_t top_k, float top_p, uint64_t seed,
                               uint64_t offset, double* margin) {
  orc_sample_item* items = (orc_sample_item*)malloc((size_t)n * sizeof(orc_sample_item));
  double gap = 1.0;
  for (int64_t i = 0; i < n; ++i) {
    const float s = logits[i] / temperature;
    uint32_t b;
    memcpy(&b, &s, 4);
    items[i].ordered = (b & 0x80000000u) ? ~b : (b | 0x80000000u);   /* the order of a radix sort on floats */
    items[i].id = (int32_t)i;
    items[i].score = s;
  }
  qsort(items, (size_t)n, sizeof(orc_sample_item), orc_sample_cmp);
  const int64_t limit = top_k == 0 ? n : (top_k < n ? top_k : n);
  const float maximum = items[0].score;
  float total = 0.0f;
  for (int64_t i = 0; i < limit; ++i) total += expf(items[i].score - maximum);
  int64_t prefix = limit;
  if (top_p < 1.0f) {
    float cumulative = 0.0f;
    for (int64_t i = 0; i < limit; ++i) {
      cumulative += expf(items[i].score - maximum) / total;
      const double g = fabs((double)cumulative - (double)top_p);
      if (g < gap) gap = g;
      if (cumulative >= top_p) { prefix = i + 1; break; }
    }
  }
  float prefix_total = 0.0f;
  for (int64_t i = 0; i < prefix; ++i) prefix_total += expf(items[i].score - maximum);
  const uint64_t bits = orc_sample_mix(seed ^ (offset * 0xd1342543de82ef95ULL));
  const float u = ((float)((bits >> 11) & 0x1fffffffffffffULL) + 0.5f) / 9007199254740992.0f;
  const float target = u * prefix_total;
  float cumulative = 0.0f;
  int32_t selected = items[prefix - 1].id;
  for (int64_t i = 0; i < prefix; ++i) {
    cumulative += expf(items[i].score - maximum);
    const double g = fabs((double)target - (double)cumulative) / (double)prefix_total;
    if (g < gap) gap = g;
    if (target < cumulative) { selected = items[i].id; break; }
  }
  if (margin) *margin = gap;
  free(items);
  return selected;
}

/* Row moves around the paged KV cache: the index arithmetic of paged_kv_write_decode_batch_kernel
 * (src/paged_attention_cuda.cu:241-262), paged_kv_write_decode_kernel (:219-239) and
 * packed_kv_prefill_copy_kernel (src/ops_cuda.cu:1104-1121), element by element as the reference
 * writes it, on byte-sized elements of `esize` bytes.  mode 0: batch decode, 1: packed prefill,
 * 2: single decode with *positions = cache length. */
ORC_API void orc_paged_kv_write(int mode, const unsigned char* key, const unsigned char* value, unsigned char* storage,
                                const int32_t* block_tables, const int32_t* positions, int64_t tokens, int64_t max_blocks,
                                int64_t layer, int64_t total_blocks, int64_t block_size, int64_t kv_heads, int64_t head_dim,
                                int64_t esize) {
  const int64_t per_row = kv_heads * head_dim, plane_elements = block_size * per_row;
  for (int64_t t = 0; t < tokens; ++t) {
    int64_t token;
    const int32_t* table;
    if (mode == 0) { token = (int64_t)positions[t] + 1 - 1; table = block_tables + t * max_blocks; }
    else if (mode == 1) { token = t; table = block_tables; }
    else { if (positions[0] == 0) return; token = (int64_t)positions[0] - 1; table = block_tables; }
    const int64_t block = table[token / block_size], offset = token % block_size;
    const int64_t layer_block = (layer * total_blocks + block) * 2;
    for (int64_t e = 0; e < per_row; ++e) {
      memcpy(storage + (layer_block * plane_elements + offset * per_row + e) * esize, key + (t * per_row + e) * esize, (size_t)esize);
      memcpy(storage + ((layer_block + 1) * plane_elements + offset * per_row + e) * esize, value + (t * per_row + e) * esize,
             (size_t)esize);
    }
  }
}

/* select_last_valid_logits (src/qwen3_padded_prefill.cpp:118-148): row valid_lengths[b] - 1 of every prompt. */
ORC_API void orc_select_last_valid(const unsigned char* padded, const int32_t* valid_lengths, unsigned char* out, int64_t batch,
                                   int64_t seq, int64_t row_bytes) {
  for (int64_t b = 0; b < batch; ++b)
    memcpy(out + b * row_bytes, padded + (b * seq + (int64_t)valid_lengths[b] - 1) * row_bytes, (size_t)row_bytes);
}
