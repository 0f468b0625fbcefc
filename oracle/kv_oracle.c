/*
 * CPU oracle for the paged KV-cache write path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, what the reference plugin's two cache-write
 * ops compute, so that the CUDA kernels can be checked byte for byte.  It is
 * never linked into, imported by or called from the shipped library; only the
 * test-suite, the smoke check and the benchmark's CPU-baseline leg use it.
 *
 * What each function follows (paths are relative to the reference project):
 *   orc_reshape_and_cache_flash  csrc/cache.cpp:140-169 (device body) and
 *                                csrc/cache.cpp:461-489 (host sizes/strides),
 *                                tests/test_cache.py:284-292 (torch loop)
 *   orc_reshape_and_cache        csrc/cache.cpp:44-85 (index formulas :57-67),
 *                                tests/test_cache.py:155-164 (torch loop)
 *   orc_concat_and_cache_mla     csrc/cache.cpp:222-253 (device body), :513-550 (host),
 *                                tests/test_cache.py:370-375 (torch loop)
 *   orc_gather_cache             csrc/cache.cpp:305-366 (device body), :576-638 (host),
 *                                tests/test_cache.py:460-477 (torch loop)
 *   orc_static_scaled_fp8_quant, orc_absmax_scale, orc_per_token_fp8_quant
 *                                csrc/quantization/fp8/fp8_quant.cpp:15-45, :47-131,
 *                                fp8_quant.h:56-102; element rule quant_utils.h:80-91
 *                                (multiply by 1.0f/scale, clamp, cast)
 *   orc_rotary_embedding         csrc/pos_encoding_kernels.cpp:9-37 (pair update), :40-88 (loops over
 *                                heads), :174-232 (host sizes and strides); torch form
 *                                tests/ops/rotary_embedding_op.py:11-30, :85-118
 *   orc_paged_attention,         tests/flash_attn/test_flash_attn_varlen_func.py:27-110 (ref_paged_attn: paged,
 *   orc_paged_decode_attention   optional causal mask and sink column, no window) and mha_varlen_fwd,
 *                                csrc/flash_attn/flash_api.cpp:10-176 (decode branch :124-165)
 *   element conversion           csrc/quantization/fp8/quant_utils.h:62-78
 *                                (auto: bit copy; fp8: float(src) / scale,
 *                                then cast)
 *
 * The float -> fp8 cast itself is not reference code: the reference calls
 * PyTorch's c10::Float8_e4m3fn / c10::Float8_e5m2 constructors (pinned
 * torch==2.10.0+xpu in its pyproject.toml).  Their published algorithm is
 * round-to-nearest-even onto the 8-bit grid; it is restated here from the
 * format definition (e4m3fn: bias 7, 3 mantissa bits, no inf, max 448;
 * e5m2: bias 15, 2 mantissa bits, max finite 57344) with one deliberate
 * difference that this build's contract asks for: magnitudes above the largest
 * finite value SATURATE to it instead of becoming NaN/inf.  The two agree for
 * |x/scale| <= 464 (e4m3) and tests/golden pins exactly that against torch.
 * NaN maps to the canonical 0x7F (sign dropped), which is what the hardware
 * conversion produces.
 *
 * Pinning.  Slot placement and the unquantised ("auto") results are pinned by fixtures
 * generated with the reference's own test utilities and expected-result loops
 * (tests/golden/make_golden.py); the fp8 results are pinned against PyTorch's cast, the
 * conversion the reference calls, because the reference's own cache tests switch fp8 off
 * (tests/test_cache.py:37 there) -- there is no reference test vector for fp8 cache bytes.
 * The fp8 quantisation ops are pinned by the torch recipes of the reference's
 * tests/test_fp8_quant.py:20-75.  The rotary embedding is pinned by fixtures computed with the
 * reference's RotaryEmbedding.forward_native (tests/ops/rotary_embedding_op.py); its own test
 * (tests/test_rotary_embedding.py) checks the op's schema only, no values.
 *
 * The paged op divides by the scale like the flash op; the reference's paged
 * kernel multiplies (csrc/cache.cpp:70-79) in a branch its own tests disable.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

enum { ORC_F32 = 0, ORC_F16 = 1, ORC_BF16 = 2 };
enum { ORC_KV_AUTO = 0, ORC_KV_E4M3 = 1, ORC_KV_E5M2 = 2 };

static inline uint32_t f2u(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
}
static inline float u2f(uint32_t u) {
  float f;
  memcpy(&f, &u, 4);
  return f;
}

float orc_bf16_to_f32(uint16_t h) { return u2f((uint32_t)h << 16); }

float orc_f16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1Fu;
  uint32_t man = h & 0x3FFu;
  if (exp == 0x1F) return u2f(sign | 0x7F800000u | (man << 13));
  if (exp == 0) {
    if (man == 0) return u2f(sign);
    /* subnormal half: man * 2^-24, exact in float */
    float v = (float)man * 5.9604644775390625e-08f;
    return sign ? -v : v;
  }
  return u2f(sign | ((exp + 112u) << 23) | (man << 13));
}

/* Round-to-nearest-even of |f| onto a small float grid with `mbits` mantissa
 * bits, exponent bias `bias`, saturating at the bit pattern `max_code`
 * (whose float value has bits `max_f32`). */
static inline uint8_t f32_to_fp8_sat(float f, int mbits, int bias, uint32_t max_f32, uint8_t max_code) {
  const uint32_t u = f2u(f);
  const uint8_t sign = (uint8_t)((u >> 24) & 0x80u);
  const uint32_t a = u & 0x7FFFFFFFu;
  if (a > 0x7F800000u) return 0x7F; /* NaN */
  if (a >= max_f32) return (uint8_t)(sign | max_code);
  const int e = (int)(a >> 23);                 /* biased fp32 exponent */
  const int min_norm = 127 - bias + 1;          /* fp32 biased exp of the smallest normal */
  if (e >= min_norm) {
    const int sh = 23 - mbits;
    uint32_t r = a >> sh;
    const uint32_t rem = a & ((1u << sh) - 1u);
    const uint32_t half = 1u << (sh - 1);
    if (rem > half || (rem == half && (r & 1u))) r += 1u;
    r -= (uint32_t)(min_norm - 1) << mbits;
    if (r > max_code) r = max_code; /* rounding carried past the top: saturate */
    return (uint8_t)(sign | r);
  }
  /* subnormal target: units of 2^(1 - bias - mbits) */
  if (e == 0) return sign; /* fp32 zero / subnormal: far below half a unit */
  const uint32_t mant = (a & 0x7FFFFFu) | 0x800000u; /* value = mant * 2^(e-150) */
  const int sh = 150 - e + (1 - bias - mbits);       /* mant >> sh = value / unit */
  if (sh > 25) return sign;
  const uint32_t q0 = mant >> sh;
  const uint32_t rem = mant & ((1u << sh) - 1u);
  const uint32_t half = 1u << (sh - 1);
  uint32_t q = q0;
  if (rem > half || (rem == half && (q & 1u))) q += 1u;
  return (uint8_t)(sign | q);
}

uint8_t orc_f32_to_e4m3(float f) { return f32_to_fp8_sat(f, 3, 7, 0x43E00000u /*448*/, 0x7E); }
uint8_t orc_f32_to_e5m2(float f) { return f32_to_fp8_sat(f, 2, 15, 0x47600000u /*57344*/, 0x7B); }

static inline float load_as_f32(const void* p, int64_t i, int dt) {
  switch (dt) {
    case ORC_F32: return ((const float*)p)[i];
    case ORC_F16: return orc_f16_to_f32(((const uint16_t*)p)[i]);
    default: return orc_bf16_to_f32(((const uint16_t*)p)[i]);
  }
}
static inline int in_size(int dt) { return dt == ORC_F32 ? 4 : 2; }

/* One element: quant_utils.h:62-78.  `scale` is only read in fp8 modes. */
static inline void store_elem(void* dst, int64_t di, const void* src, int64_t si, int in_dt, int kv, float scale) {
  if (kv == ORC_KV_AUTO) {
    const int es = in_size(in_dt);
    memcpy((char*)dst + di * es, (const char*)src + si * es, (size_t)es);
  } else {
    const float x = load_as_f32(src, si, in_dt) / scale;
    ((uint8_t*)dst)[di] = (kv == ORC_KV_E4M3) ? orc_f32_to_e4m3(x) : orc_f32_to_e5m2(x);
  }
}

/* Conversion table over all 65536 16-bit input patterns (in_dt F16 or BF16). */
void orc_convert_table(int in_dt, int kv, float scale, uint8_t* out) {
  for (uint32_t b = 0; b < 65536u; ++b) {
    const float v = (in_dt == ORC_F16) ? orc_f16_to_f32((uint16_t)b) : orc_bf16_to_f32((uint16_t)b);
    const float x = v / scale;
    out[b] = (kv == ORC_KV_E5M2) ? orc_f32_to_e5m2(x) : orc_f32_to_e4m3(x);
  }
}

/* Array conversion for float inputs: out[i] = fp8(x[i] / scale). */
void orc_convert_f32(const float* x, int64_t n, int kv, float scale, uint8_t* out) {
  for (int64_t i = 0; i < n; ++i) store_elem(out, i, x, i, ORC_F32, kv, scale);
}

/*
 * Flash (NHD) layout: cache[block][offset][head][d], with arbitrary element
 * strides for dims 0..2 (block_stride, page_stride, head_stride) and for the
 * key/value token and head dims.  Strides are in ELEMENTS.  The reference
 * kernel assumes head_stride == D and key head stride == D; the general form
 * reduces to it.  Tokens with slot < 0 are skipped (cache.cpp:144-145).
 * Returns 0, or -1 when a slot is >= num_slots (num_slots < 0 disables the check).
 */
int orc_reshape_and_cache_flash(const void* key, const void* value, void* key_cache, void* value_cache,
                                const int64_t* slot_mapping, int64_t num_tokens, int64_t num_heads,
                                int64_t head_size, int64_t block_size, int64_t key_stride_t,
                                int64_t key_stride_h, int64_t value_stride_t, int64_t value_stride_h,
                                int64_t block_stride, int64_t page_stride, int64_t head_stride, int in_dt,
                                int kv, float k_scale, float v_scale, int64_t num_slots, int nthreads) {
  int bad = 0;
#ifdef _OPENMP
  if (nthreads < 1) nthreads = 1;
#pragma omp parallel for schedule(static) num_threads(nthreads) reduction(| : bad)
#endif
  for (int64_t t = 0; t < num_tokens; ++t) {
    const int64_t slot = slot_mapping[t];
    if (slot < 0) continue;
    if (num_slots >= 0 && slot >= num_slots) {
      bad |= 1;
      continue;
    }
    const int64_t blk = slot / block_size, off = slot % block_size;
    const int64_t dst0 = blk * block_stride + off * page_stride;
    for (int64_t h = 0; h < num_heads; ++h) {
      const int64_t ks = t * key_stride_t + h * key_stride_h;
      const int64_t vs = t * value_stride_t + h * value_stride_h;
      const int64_t d0 = dst0 + h * head_stride;
      if (kv == ORC_KV_AUTO) {
        const size_t es = (size_t)in_size(in_dt);
        memcpy((char*)key_cache + d0 * es, (const char*)key + ks * es, (size_t)head_size * es);
        memcpy((char*)value_cache + d0 * es, (const char*)value + vs * es, (size_t)head_size * es);
      } else {
        for (int64_t d = 0; d < head_size; ++d) {
          store_elem(key_cache, d0 + d, key, ks + d, in_dt, kv, k_scale);
          store_elem(value_cache, d0 + d, value, vs + d, in_dt, kv, v_scale);
        }
      }
    }
  }
  (void)nthreads;
  return bad ? -1 : 0;
}

/*
 * Paged layout: key_cache [num_blocks, H, D/x, block_size, x] and
 * value_cache [num_blocks, H, D, block_size], both contiguous
 * (cache.cpp:57-67 index formulas, widened to 64 bits).
 */
int orc_reshape_and_cache(const void* key, const void* value, void* key_cache, void* value_cache,
                          const int64_t* slot_mapping, int64_t num_tokens, int64_t num_heads,
                          int64_t head_size, int64_t block_size, int64_t x, int64_t key_stride_t,
                          int64_t key_stride_h, int64_t value_stride_t, int64_t value_stride_h, int in_dt,
                          int kv, float k_scale, float v_scale, int64_t num_slots, int nthreads) {
  int bad = 0;
#ifdef _OPENMP
  if (nthreads < 1) nthreads = 1;
#pragma omp parallel for schedule(static) num_threads(nthreads) reduction(| : bad)
#endif
  for (int64_t t = 0; t < num_tokens; ++t) {
    const int64_t slot = slot_mapping[t];
    if (slot < 0) continue;
    if (num_slots >= 0 && slot >= num_slots) {
      bad |= 1;
      continue;
    }
    const int64_t blk = slot / block_size, off = slot % block_size;
    for (int64_t h = 0; h < num_heads; ++h) {
      for (int64_t d = 0; d < head_size; ++d) {
        const int64_t kdst = blk * num_heads * (head_size / x) * block_size * x +
                             h * (head_size / x) * block_size * x + (d / x) * block_size * x + off * x +
                             d % x;
        const int64_t vdst =
            blk * num_heads * head_size * block_size + h * head_size * block_size + d * block_size + off;
        store_elem(key_cache, kdst, key, t * key_stride_t + h * key_stride_h + d, in_dt, kv, k_scale);
        store_elem(value_cache, vdst, value, t * value_stride_t + h * value_stride_h + d, in_dt, kv,
                   v_scale);
      }
    }
  }
  (void)nthreads;
  return bad ? -1 : 0;
}

/*
 * MLA: kv_cache[block][offset][0:R] = kv_c[t], [R:R+P] = k_pe[t]; strides in elements.
 * fp8 modes divide by the scale like the K/V ops (the reference kernel multiplies,
 * cache.cpp:240-244, in a branch its test cannot reach).
 */
int orc_concat_and_cache_mla(const void* kv_c, const void* k_pe, void* kv_cache, const int64_t* slot_mapping,
                             int64_t num_tokens, int64_t kv_lora_rank, int64_t pe_dim, int64_t block_size,
                             int64_t kv_c_stride, int64_t k_pe_stride, int64_t block_stride,
                             int64_t entry_stride, int in_dt, int kv, float scale, int64_t num_slots) {
  int bad = 0;
  for (int64_t t = 0; t < num_tokens; ++t) {
    const int64_t slot = slot_mapping[t];
    if (slot < 0) continue;
    if (num_slots >= 0 && slot >= num_slots) {
      bad = 1;
      continue;
    }
    const int64_t dst0 = (slot / block_size) * block_stride + (slot % block_size) * entry_stride;
    for (int64_t i = 0; i < kv_lora_rank; ++i) store_elem(kv_cache, dst0 + i, kv_c, t * kv_c_stride + i, in_dt, kv, scale);
    for (int64_t i = 0; i < pe_dim; ++i)
      store_elem(kv_cache, dst0 + kv_lora_rank + i, k_pe, t * k_pe_stride + i, in_dt, kv, scale);
  }
  return bad ? -1 : 0;
}

/*
 * gather: for each sequence b and each j < cu[b+1]-cu[b]:
 *   dst[cu[b]+j] = src[block_table[b][seq_starts[b]/bs + j/bs]][j%bs]   (cache.cpp:305-366).
 * Byte copy of entry_bytes per row; strides in BYTES.  Rows at or beyond num_dst_rows are not written.
 */
void orc_gather_cache(const void* src_cache, void* dst, const int32_t* block_table, const int32_t* cu_seq_lens,
                      const int32_t* seq_starts, int64_t batch_size, int64_t num_dst_rows, int64_t block_size,
                      int64_t entry_bytes, int64_t block_table_stride, int64_t cache_block_stride,
                      int64_t cache_entry_stride, int64_t dst_entry_stride) {
  for (int64_t b = 0; b < batch_size; ++b) {
    const int64_t start = cu_seq_lens[b], len = (int64_t)cu_seq_lens[b + 1] - start;
    const int64_t first = seq_starts ? seq_starts[b] / block_size : 0;
    for (int64_t j = 0; j < len; ++j) {
      if (start + j >= num_dst_rows) break;
      const int64_t blk = block_table[b * block_table_stride + first + j / block_size];
      memcpy((char*)dst + (start + j) * dst_entry_stride,
             (const char*)src_cache + blk * cache_block_stride + (j % block_size) * cache_entry_stride,
             (size_t)entry_bytes);
    }
  }
}

/*
 * fp8 activation quantisation.  quant_utils.h:80-91 with an inverted scale:
 * r = fmax(-M, fmin(x * inv, M)), then the fp8 cast; inv = 1.0f / scale in fp32
 * (fp8_quant.cpp:34).  fminf/fmaxf return the non-NaN operand like sycl::fmin/fmax.
 */
static inline float fp8_max_of(int kv) { return kv == ORC_KV_E5M2 ? 57344.0f : 448.0f; }

static inline uint8_t quant_elem(float x, float inv, int kv) {
  const float m = fp8_max_of(kv);
  const float r = fmaxf(-m, fminf(x * inv, m));
  return kv == ORC_KV_E5M2 ? orc_f32_to_e5m2(r) : orc_f32_to_e4m3(r);
}

void orc_static_scaled_fp8_quant(uint8_t* out, const void* in, int64_t n, int in_dt, int kv, float scale) {
  const float inv = 1.0f / scale;
  for (int64_t i = 0; i < n; ++i) out[i] = quant_elem(load_as_f32(in, i, in_dt), inv, kv);
}

/* fp8_quant.h:56-102: max over |x| (NaN never wins a max), divided by M */
float orc_absmax_scale(const void* in, int64_t n, int in_dt, int kv) {
  float m = 0.0f;
  for (int64_t i = 0; i < n; ++i) m = fmaxf(m, fabsf(load_as_f32(in, i, in_dt)));
  return m / fp8_max_of(kv);
}

/* fp8_quant.cpp:70-129: scale_t = max(min(absmax_t, ub) / M, 1 / (M * 512)) */
void orc_per_token_fp8_quant(uint8_t* out, float* scales, const void* in, int64_t tokens, int64_t hidden,
                             int in_dt, int kv, const float* scale_ub) {
  const float m = fp8_max_of(kv);
  for (int64_t t = 0; t < tokens; ++t) {
    float a = 0.0f;
    for (int64_t i = 0; i < hidden; ++i) a = fmaxf(a, fabsf(load_as_f32(in, t * hidden + i, in_dt)));
    if (scale_ub) a = fminf(a, *scale_ub);
    const float s = fmaxf(a / m, 1.0f / (m * 512.0f));
    scales[t] = s;
    const float inv = 1.0f / s;
    for (int64_t i = 0; i < hidden; ++i) out[t * hidden + i] = quant_elem(load_as_f32(in, t * hidden + i, in_dt), inv, kv);
  }
}

/* ------------------------------------------------------------------------------------------
 * rotary position embedding, in place on query and (optionally) key
 * ------------------------------------------------------------------------------------------ */
static inline uint16_t f32_to_bf16_rne(float f) {
  uint32_t u = f2u(f);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x0040u); /* quiet NaN */
  u += 0x7FFFu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

static inline uint16_t f32_to_f16_rne(float f) {
  const uint32_t u = f2u(f);
  const uint16_t sign = (uint16_t)((u >> 16) & 0x8000u);
  const uint32_t a = u & 0x7FFFFFFFu;
  if (a > 0x7F800000u) return (uint16_t)(sign | 0x7E00u);
  if (a >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u); /* >= 65520 rounds to inf */
  const int e = (int)(a >> 23);
  if (e >= 113) { /* normal half */
    uint32_t r = a >> 13;
    const uint32_t rem = a & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (r & 1u))) r += 1u;
    r -= (uint32_t)112 << 10;
    return (uint16_t)(sign | r);
  }
  if (e < 102) return sign; /* below half of the smallest subnormal (2^-25) rounds to zero */
  const uint32_t mant = (a & 0x7FFFFFu) | 0x800000u; /* value = mant * 2^(e-150); unit 2^-24 */
  const int sh = 126 - e;                            /* mant >> sh = value / 2^-24 */
  uint32_t q = mant >> sh;
  const uint32_t rem = mant & ((1u << sh) - 1u);
  const uint32_t half = 1u << (sh - 1);
  if (rem > half || (rem == half && (q & 1u))) q += 1u;
  return (uint16_t)(sign | q);
}

uint16_t orc_f32_to_bf16(float f) { return f32_to_bf16_rne(f); }
uint16_t orc_f32_to_f16(float f) { return f32_to_f16_rne(f); }

/* One arithmetic result rounded to the tensor's type, as a torch elementwise op on that dtype
 * does (compute in fp32, round once to the 16-bit type). */
static inline float round_to(float f, int dt) {
  if (dt == ORC_F16) return orc_f16_to_f32(f32_to_f16_rne(f));
  if (dt == ORC_BF16) return orc_bf16_to_f32(f32_to_bf16_rne(f));
  return f;
}
static inline void store_from_f32(void* p, int64_t i, float f, int dt) {
  if (dt == ORC_F32) ((float*)p)[i] = f;
  else if (dt == ORC_F16) ((uint16_t*)p)[i] = f32_to_f16_rne(f);
  else ((uint16_t*)p)[i] = f32_to_bf16_rne(f);
}

/* pos_encoding_kernels.cpp:9-37: x' = x*cos - y*sin, y' = y*cos + x*sin, every product and the
 * sum each rounded to the tensor's type (three roundings per output, no fused multiply-add). */
static void rope_heads(void* arr, int64_t heads, int64_t token_off, int64_t head_stride, const void* cs,
                       int64_t cs_off, int64_t embed_dim, int is_neox, int dt) {
  for (int64_t h = 0; h < heads; ++h) {
    const int64_t base = token_off + h * head_stride;
    for (int64_t r = 0; r < embed_dim; ++r) {
      const int64_t xi = is_neox ? r : 2 * r;
      const int64_t yi = is_neox ? embed_dim + r : 2 * r + 1;
      const float c = load_as_f32(cs, cs_off + r, dt);
      const float s = load_as_f32(cs, cs_off + embed_dim + r, dt);
      const float x = load_as_f32(arr, base + xi, dt);
      const float y = load_as_f32(arr, base + yi, dt);
      const float xc = round_to(x * c, dt), ys = round_to(y * s, dt);
      const float yc = round_to(y * c, dt), xs = round_to(x * s, dt);
      store_from_f32(arr, base + xi, xc - ys, dt);
      store_from_f32(arr, base + yi, yc + xs, dt);
    }
  }
}

/* Strides in elements.  `key` may be NULL.  Returns 1 if a position is outside [0, max_position). */
int orc_rotary_embedding(const int64_t* positions, void* query, void* key, const void* cos_sin_cache,
                         int64_t num_tokens, int64_t num_heads, int64_t num_kv_heads, int64_t rot_dim,
                         int64_t max_position, int64_t query_stride, int64_t key_stride,
                         int64_t query_head_stride, int64_t key_head_stride, int is_neox, int dt) {
  const int64_t embed_dim = rot_dim / 2;
  int bad = 0;
#pragma omp parallel for schedule(static) reduction(| : bad)
  for (int64_t t = 0; t < num_tokens; ++t) {
    const int64_t pos = positions[t];
    if (pos < 0 || pos >= max_position) {
      bad |= 1;
      continue;
    }
    rope_heads(query, num_heads, t * query_stride, query_head_stride, cos_sin_cache, pos * rot_dim, embed_dim,
               is_neox, dt);
    if (key)
      rope_heads(key, num_kv_heads, t * key_stride, key_head_stride, cos_sin_cache, pos * rot_dim, embed_dim,
                 is_neox, dt);
  }
  return bad;
}

/* ------------------------------------------------------------------------------------------
 * paged decode attention: one query token per sequence against that sequence's cached keys/values
 * ------------------------------------------------------------------------------------------ */
float orc_e4m3_to_f32(uint8_t b) {
  const int e = (b >> 3) & 0xF, m = b & 7;
  float v;
  if (e == 0xF && m == 7) return u2f(0x7FC00000u); /* the only NaN code; e4m3fn has no infinity */
  if (e == 0) v = (float)m * 0.001953125f;          /* m * 2^-9 */
  else v = ldexpf(1.0f + (float)m / 8.0f, e - 7);
  return (b & 0x80) ? -v : v;
}
float orc_e5m2_to_f32(uint8_t b) { return orc_f16_to_f32((uint16_t)b << 8); }

static inline float cache_elem(const void* p, int64_t i, int q_dt, int kv) {
  if (kv == ORC_KV_E4M3) return orc_e4m3_to_f32(((const uint8_t*)p)[i]);
  if (kv == ORC_KV_E5M2) return orc_e5m2_to_f32(((const uint8_t*)p)[i]);
  return load_as_f32(p, i, q_dt);
}

/* Query token t of sequence s (tokens cu_seqlens_q[s] .. cu_seqlens_q[s+1]; cu_seqlens_q == NULL means one
 * token per sequence, token s) and head h:
 *   out[t][h][:] = softmax_j(scale * q[t][h] . K[s][j][h/g]) @ V[s][:][h/g],  j < limit, g = Hq / Hkv,
 *   limit = seq_lens[s], or with `causal` seq_lens[s] - q_len_s + i + 1 for the i-th query token of the sequence
 *   (the query tokens are the LAST q_len_s positions of the sequence, tests/flash_attn/
 *   test_flash_attn_varlen_func.py:79-80 of the reference),
 *   K[s][j] = key_cache[block_table[s][j / bs]][j % bs] (times k_descale for an fp8 cache), V likewise.
 * A sink adds one more logit sink[h] to the softmax denominator only.  Everything is accumulated in
 * double and written as fp32: this is the ideal result, the kernels are held to a tolerance around it.
 * Strides in elements.  Rows with nothing to attend to give zeros. */
void orc_paged_attention_window(float* out, const void* query, const void* key_cache, const void* value_cache,
                                const int32_t* block_table, const int32_t* seq_lens, const int32_t* cu_seqlens_q,
                                const void* sink, float k_descale, float v_descale, int64_t num_seqs,
                                int64_t num_heads, int64_t num_kv_heads, int64_t head_size, int64_t block_size,
                                int64_t block_table_stride, int64_t query_stride_t, int64_t query_stride_h,
                                int64_t block_stride, int64_t page_stride, int64_t head_stride, float scale,
                                int causal, int64_t window_left, int64_t window_right, int q_dt, int kv) {
  const int64_t group = num_heads / num_kv_heads;
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int64_t s = 0; s < num_seqs; ++s) {
    for (int64_t h = 0; h < num_heads; ++h) {
      const int64_t t0 = cu_seqlens_q ? cu_seqlens_q[s] : s;
      const int64_t q_len = cu_seqlens_q ? cu_seqlens_q[s + 1] - cu_seqlens_q[s] : 1;
      const int64_t kvh = h / group;
      for (int64_t i = 0; i < q_len; ++i) {
        const int64_t t = t0 + i;
        /* the query token sits at position pos of its sequence and sees cached tokens lo <= j < n:
         * all of them; under the causal mask those up to pos; with a sliding window (a negative side is
         * open) those within [pos - left, pos + right] (tests/flash_attn/test_flash_attn_varlen_func.py:81-95) */
        const int64_t len = seq_lens[s];
        const int64_t pos = len - q_len + i;
        int64_t n = len, lo = 0;
        if (causal && pos + 1 < n) n = pos + 1;
        if (window_right >= 0 && pos + window_right + 1 < n) n = pos + window_right + 1;
        if (window_left >= 0 && pos - window_left > lo) lo = pos - window_left;
        float* o = out + (t * num_heads + h) * head_size;
        for (int64_t d = 0; d < head_size; ++d) o[d] = 0.0f;
        if (n <= lo) continue;
        double* logit = (double*)malloc((size_t)n * sizeof(double));
        double* acc = (double*)calloc((size_t)head_size, sizeof(double));
        double mx = sink ? (double)load_as_f32(sink, h, q_dt) : -INFINITY;
        for (int64_t j = lo; j < n; ++j) {
          const int64_t blk = block_table[s * block_table_stride + j / block_size];
          const int64_t base = blk * block_stride + (j % block_size) * page_stride + kvh * head_stride;
          double dot = 0.0;
          for (int64_t d = 0; d < head_size; ++d)
            dot += (double)load_as_f32(query, t * query_stride_t + h * query_stride_h + d, q_dt) *
                   (double)cache_elem(key_cache, base + d, q_dt, kv);
          logit[j] = dot * (double)scale * (double)k_descale;
          if (logit[j] > mx) mx = logit[j];
        }
        double denom = sink ? exp((double)load_as_f32(sink, h, q_dt) - mx) : 0.0;
        for (int64_t j = lo; j < n; ++j) {
          const double p = exp(logit[j] - mx);
          denom += p;
          const int64_t blk = block_table[s * block_table_stride + j / block_size];
          const int64_t base = blk * block_stride + (j % block_size) * page_stride + kvh * head_stride;
          for (int64_t d = 0; d < head_size; ++d) acc[d] += p * (double)cache_elem(value_cache, base + d, q_dt, kv);
        }
        for (int64_t d = 0; d < head_size; ++d) o[d] = (float)(acc[d] / denom * (double)v_descale);
        free(logit);
        free(acc);
      }
    }
  }
}

/* No sliding window. */
void orc_paged_attention(float* out, const void* query, const void* key_cache, const void* value_cache,
                         const int32_t* block_table, const int32_t* seq_lens, const int32_t* cu_seqlens_q,
                         const void* sink, float k_descale, float v_descale, int64_t num_seqs, int64_t num_heads,
                         int64_t num_kv_heads, int64_t head_size, int64_t block_size, int64_t block_table_stride,
                         int64_t query_stride_t, int64_t query_stride_h, int64_t block_stride, int64_t page_stride,
                         int64_t head_stride, float scale, int causal, int q_dt, int kv) {
  orc_paged_attention_window(out, query, key_cache, value_cache, block_table, seq_lens, cu_seqlens_q, sink, k_descale,
                             v_descale, num_seqs, num_heads, num_kv_heads, head_size, block_size, block_table_stride,
                             query_stride_t, query_stride_h, block_stride, page_stride, head_stride, scale, causal, -1,
                             -1, q_dt, kv);
}

/* One query token per sequence: the decode case. */
void orc_paged_decode_attention(float* out, const void* query, const void* key_cache, const void* value_cache,
                                const int32_t* block_table, const int32_t* seq_lens, const void* sink,
                                float k_descale, float v_descale, int64_t num_seqs, int64_t num_heads,
                                int64_t num_kv_heads, int64_t head_size, int64_t block_size,
                                int64_t block_table_stride, int64_t query_stride_t, int64_t query_stride_h,
                                int64_t block_stride, int64_t page_stride, int64_t head_stride, float scale,
                                int q_dt, int kv) {
  orc_paged_attention(out, query, key_cache, value_cache, block_table, seq_lens, NULL, sink, k_descale, v_descale,
                      num_seqs, num_heads, num_kv_heads, head_size, block_size, block_table_stride, query_stride_t,
                      query_stride_h, block_stride, page_stride, head_stride, scale, 0, q_dt, kv);
}

int orc_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
