// Rotary position embedding for NVIDIA B200 (sm_100a), alone and fused with the paged
// KV-cache write, and their C ABI.
//
//   kvc_rotary_embedding                  in place on query [T, Hq, D] and key [T, Hkv, D]
//   kvc_rotary_embedding_and_cache_flash  the same, and in the same pass the rotated key and the
//                                         value go to their cache slots (flash layout), so the
//                                         key is read from HBM once instead of twice
//
// Both are pure HBM traffic.  For token t at position p, and each rotated pair (x, y) of a head,
//   x' = x*cos[p][i] - y*sin[p][i]      y' = y*cos[p][i] + x*sin[p][i]
// with every product and the final sum rounded to the tensors' type (three roundings per output,
// nothing fused), which is what an elementwise tensor expression in that type computes.  Pairs are
// (i, i + rot_dim/2) in the GPT-NeoX style and (2i, 2i+1) in the GPT-J style; elements at and above
// rot_dim pass through.
//
// The reference plugin's counterpart of the first op is csrc/pos_encoding_kernels.cpp:9-162
// (device code) and :165-286 (host launcher); it has no fused op.
#include "kvc_common.cuh"
#include "kvc_convert.cuh"

namespace kvc {

// ---------------------------------------------------------------------------------------------
// arithmetic
// ---------------------------------------------------------------------------------------------
// Packed 16-bit operations, each correctly rounded and never contracted into an fma.
template <typename Tin>
__device__ __forceinline__ uint32_t mul2(uint32_t a, uint32_t b) {
  if constexpr (std::is_same_v<Tin, __half>) {
    const __half2 r = __hmul2_rn(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
  } else {
    const __nv_bfloat162 r =
        __hmul2_rn(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
  }
}
template <typename Tin>
__device__ __forceinline__ uint32_t add2(uint32_t a, uint32_t b) {
  if constexpr (std::is_same_v<Tin, __half>) {
    const __half2 r = __hadd2_rn(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
  } else {
    const __nv_bfloat162 r =
        __hadd2_rn(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
  }
}
// a - b == a + (-b) exactly; negating is a sign flip of both halves.
template <typename Tin>
__device__ __forceinline__ uint32_t sub2(uint32_t a, uint32_t b) {
  return add2<Tin>(a, b ^ 0x80008000u);
}

// NeoX pairing: x[i] pairs with y[i]; c and s hold the VEC cosines / sines of the same i.
template <typename Tin, int VEC>
__device__ __forceinline__ void rotate_neox(Chunk<VEC * (int)sizeof(Tin)>& x, Chunk<VEC * (int)sizeof(Tin)>& y,
                                            const Chunk<VEC * (int)sizeof(Tin)>& c,
                                            const Chunk<VEC * (int)sizeof(Tin)>& s) {
  if constexpr (sizeof(Tin) == 4) {
    float* xf = reinterpret_cast<float*>(x.b);
    float* yf = reinterpret_cast<float*>(y.b);
    const float* cf = reinterpret_cast<const float*>(c.b);
    const float* sf = reinterpret_cast<const float*>(s.b);
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const float xv = xf[i], yv = yf[i];
      xf[i] = __fsub_rn(__fmul_rn(xv, cf[i]), __fmul_rn(yv, sf[i]));
      yf[i] = __fadd_rn(__fmul_rn(yv, cf[i]), __fmul_rn(xv, sf[i]));
    }
  } else {
    static_assert(VEC % 2 == 0, "16-bit chunks are whole 32-bit words");
    uint32_t* xw = reinterpret_cast<uint32_t*>(x.b);
    uint32_t* yw = reinterpret_cast<uint32_t*>(y.b);
    const uint32_t* cw = reinterpret_cast<const uint32_t*>(c.b);
    const uint32_t* sw = reinterpret_cast<const uint32_t*>(s.b);
#pragma unroll
    for (int i = 0; i < VEC / 2; ++i) {
      const uint32_t xv = xw[i], yv = yw[i];
      xw[i] = sub2<Tin>(mul2<Tin>(xv, cw[i]), mul2<Tin>(yv, sw[i]));
      yw[i] = add2<Tin>(mul2<Tin>(yv, cw[i]), mul2<Tin>(xv, sw[i]));
    }
  }
}

// GPT-J pairing: xy holds VEC/2 interleaved pairs (x at even, y at odd positions); c and s hold
// the VEC/2 cosines / sines of those pairs.
template <typename Tin, int VEC>
__device__ __forceinline__ void rotate_gptj(Chunk<VEC * (int)sizeof(Tin)>& xy,
                                            const Chunk<(VEC / 2) * (int)sizeof(Tin)>& c,
                                            const Chunk<(VEC / 2) * (int)sizeof(Tin)>& s) {
  static_assert(VEC % 2 == 0, "whole pairs");
  if constexpr (sizeof(Tin) == 4) {
    float* f = reinterpret_cast<float*>(xy.b);
    const float* cf = reinterpret_cast<const float*>(c.b);
    const float* sf = reinterpret_cast<const float*>(s.b);
#pragma unroll
    for (int j = 0; j < VEC / 2; ++j) {
      const float xv = f[2 * j], yv = f[2 * j + 1];
      f[2 * j] = __fsub_rn(__fmul_rn(xv, cf[j]), __fmul_rn(yv, sf[j]));
      f[2 * j + 1] = __fadd_rn(__fmul_rn(yv, cf[j]), __fmul_rn(xv, sf[j]));
    }
  } else {
    uint32_t* w = reinterpret_cast<uint32_t*>(xy.b);
    const uint16_t* ch = reinterpret_cast<const uint16_t*>(c.b);
    const uint16_t* sh = reinterpret_cast<const uint16_t*>(s.b);
#pragma unroll
    for (int j = 0; j < VEC / 2; ++j) {
      const uint32_t v = w[j];                               // (x, y)
      const uint32_t swapped = __byte_perm(v, 0, 0x1032);    // (y, x)
      const uint32_t c2 = static_cast<uint32_t>(ch[j]) * 0x00010001u;
      const uint32_t s2 = static_cast<uint32_t>(sh[j]) * 0x00010001u;
      const uint32_t a = mul2<Tin>(v, c2);                   // (x*c, y*c)
      const uint32_t b = mul2<Tin>(swapped, s2) ^ 0x00008000u;  // (-(y*s), x*s)
      w[j] = add2<Tin>(a, b);                                // (x*c - y*s, y*c + x*s)
    }
  }
}

// ---------------------------------------------------------------------------------------------
// rotary embedding alone
// ---------------------------------------------------------------------------------------------
struct RopeParams {
  const int64_t* positions;
  void* query;
  void* key;  // only touched when there are key heads
  const void* cos_sin_cache;
  int64_t query_stride_t, query_stride_h, key_stride_t, key_stride_h;  // elements
  int64_t max_position;
  int32_t rot_dim, embed_dim;
  uint32_t num_q_heads;      // head indices below this are query heads, the others key heads
  uint32_t n_items;          // tokens_in_launch * items_per_token
  uint32_t items_per_token;  // (Hq + Hkv) * chunks_per_head
  uint32_t chunks_per_head;
  FastDiv div_items_per_token, div_chunks_per_head;
  uint32_t prefetch_ctas;
};

constexpr int kRopeThreads = 256;

// Start of head `head` (query heads first, then key heads) of token `tok`.
template <typename Tin>
__device__ __forceinline__ Tin* rope_head_base(const RopeParams& p, uint32_t tok, uint32_t head) {
  if (head < p.num_q_heads) return static_cast<Tin*>(p.query) + tok * p.query_stride_t + head * p.query_stride_h;
  return static_cast<Tin*>(p.key) + tok * p.key_stride_t + (head - p.num_q_heads) * p.key_stride_h;
}

// One thread rotates VEC pairs (NeoX: VEC x-elements and their VEC partners, two vectors;
// GPT-J: VEC/2 interleaved pairs, one vector).  VEC * sizeof(Tin) is the width of every data
// access and all of them are aligned to it (the host picks VEC accordingly).
template <typename Tin, bool NEOX, int VEC>
__global__ void __launch_bounds__(kRopeThreads) rope_kernel(const RopeParams p) {
  constexpr int ES = (int)sizeof(Tin);
  constexpr int VB = VEC * ES;
  constexpr int CS_VEC = NEOX ? VEC : VEC / 2;
  constexpr int CSB = CS_VEC * ES;

  const uint32_t item = blockIdx.x * kRopeThreads + threadIdx.x;
  if (item >= p.n_items) return;
  const uint32_t tok = p.div_items_per_token.div(item);
  const uint32_t rem = item - tok * p.items_per_token;
  const uint32_t head = p.div_chunks_per_head.div(rem);
  const uint32_t chunk = rem - head * p.chunks_per_head;
  Tin* xp = rope_head_base<Tin>(p, tok, head) + chunk * VEC;
  Tin* yp = xp + p.embed_dim;
  if (blockIdx.x < p.prefetch_ctas) {
    prefetch_l2(xp);
    if constexpr (NEOX) prefetch_l2(yp);
  }
  pdl_prologue();

  const int64_t pos = __ldg(p.positions + tok);
  if (pos < 0 || pos >= p.max_position) return;
  const Tin* cp = static_cast<const Tin*>(p.cos_sin_cache) + pos * p.rot_dim + chunk * CS_VEC;

  Chunk<VB> x;
  Chunk<CSB> c, s;
  load_chunk_inplace(x, xp);
  if constexpr (NEOX) {
    Chunk<VB> y;
    load_chunk_inplace(y, yp);
    load_chunk_shared_ro(c, cp);
    load_chunk_shared_ro(s, cp + p.embed_dim);
    rotate_neox<Tin, VEC>(x, y, c, s);
    store_chunk(xp, x, true);
    store_chunk(yp, y, true);
  } else {
    load_chunk_shared_ro(c, cp);
    load_chunk_shared_ro(s, cp + p.embed_dim);
    rotate_gptj<Tin, VEC>(x, c, s);
    store_chunk(xp, x, true);
  }
}

// One pair per thread with element-sized accesses: for layouts whose rows are not aligned to
// any vector width (odd strides, odd rot_dim / 2).
template <typename Tin, bool NEOX>
__global__ void __launch_bounds__(kRopeThreads) rope_pair_kernel(const RopeParams p) {
  const uint32_t item = blockIdx.x * kRopeThreads + threadIdx.x;
  if (item >= p.n_items) return;
  const uint32_t tok = p.div_items_per_token.div(item);
  const uint32_t rem = item - tok * p.items_per_token;
  const uint32_t head = p.div_chunks_per_head.div(rem);
  const uint32_t r = rem - head * p.chunks_per_head;
  Tin* base = rope_head_base<Tin>(p, tok, head);
  Tin* xp = base + (NEOX ? r : 2 * r);
  Tin* yp = base + (NEOX ? p.embed_dim + r : 2 * r + 1);
  pdl_prologue();

  const int64_t pos = __ldg(p.positions + tok);
  if (pos < 0 || pos >= p.max_position) return;
  const Tin* cp = static_cast<const Tin*>(p.cos_sin_cache) + pos * p.rot_dim + r;
  if constexpr (sizeof(Tin) == 4) {
    const float xv = *xp, yv = *yp, cv = __ldg(cp), sv = __ldg(cp + p.embed_dim);
    *xp = __fsub_rn(__fmul_rn(xv, cv), __fmul_rn(yv, sv));
    *yp = __fadd_rn(__fmul_rn(yv, cv), __fmul_rn(xv, sv));
  } else {
    const uint16_t* cu = reinterpret_cast<const uint16_t*>(cp);
    const uint32_t xv = *reinterpret_cast<const uint16_t*>(xp), yv = *reinterpret_cast<const uint16_t*>(yp);
    const uint32_t cv = __ldg(cu), sv = __ldg(cu + p.embed_dim);
    *reinterpret_cast<uint16_t*>(xp) = static_cast<uint16_t>(sub2<Tin>(mul2<Tin>(xv, cv), mul2<Tin>(yv, sv)));
    *reinterpret_cast<uint16_t*>(yp) = static_cast<uint16_t>(add2<Tin>(mul2<Tin>(yv, cv), mul2<Tin>(xv, sv)));
  }
}

// ---------------------------------------------------------------------------------------------
// rotary embedding fused with the flash-layout cache write
// ---------------------------------------------------------------------------------------------
struct RopeCacheParams {
  RopeParams r;  // items_per_token / n_items cover all four segments here
  const void* value;
  void* key_cache;
  void* value_cache;
  const int64_t* slot_mapping;
  const float* k_scale;
  const float* v_scale;
  int64_t value_stride_t, value_stride_h;           // elements
  int64_t block_stride, page_stride, head_stride;   // elements
  int64_t block_size;
  int64_t num_slot_tokens;  // tokens at and beyond this index have no cache slot
  int bs_shift;
  bool linear_slots;
  bool write_back_key;
  // A token's items, in order: query rotation | key rotation + store | key pass-through | value.
  uint32_t seg_key, seg_tail, seg_value;  // first item of the 2nd, 3rd and 4th segment
  uint32_t tail_chunks, value_chunks;     // chunks per head in the 3rd and 4th segment
  FastDiv div_tail_chunks, div_value_chunks;
};

template <typename Tin, int KV, bool NEOX, int VEC>
__global__ void __launch_bounds__(kRopeThreads) rope_cache_flash_kernel(const RopeCacheParams q) {
  constexpr int ES = (int)sizeof(Tin);
  constexpr int VB = VEC * ES;
  constexpr int CS_VEC = NEOX ? VEC : VEC / 2;
  constexpr int CSB = CS_VEC * ES;
  constexpr int OUT_ES = (KV == KVC_KV_AUTO) ? ES : 1;
  constexpr int OUT_B = VEC * OUT_ES;
  constexpr bool kWideOut = (OUT_B % 32) == 0;
  const RopeParams& p = q.r;

  const uint32_t item = blockIdx.x * kRopeThreads + threadIdx.x;
  if (item >= p.n_items) return;
  const uint32_t tok = p.div_items_per_token.div(item);
  const uint32_t rem = item - tok * p.items_per_token;

  // 0: query rotation, 1: key rotation + store, 2: key pass-through, 3: value
  int seg;
  uint32_t head, chunk;
  const Tin* src;  // first element this thread reads (x-chunk for a rotation)
  int32_t d0;      // its offset inside the head
  if (rem < q.seg_tail) {
    head = p.div_chunks_per_head.div(rem);  // query heads, then key heads: same chunking
    chunk = rem - head * p.chunks_per_head;
    seg = head < p.num_q_heads ? 0 : 1;
    d0 = static_cast<int32_t>(chunk) * VEC;
    src = rope_head_base<Tin>(p, tok, head) + d0;
    if (seg == 1) head -= p.num_q_heads;
  } else if (rem < q.seg_value) {
    const uint32_t j = rem - q.seg_tail;
    head = q.div_tail_chunks.div(j);
    chunk = j - head * q.tail_chunks;
    seg = 2;
    d0 = p.rot_dim + static_cast<int32_t>(chunk) * VEC;
    src = static_cast<const Tin*>(p.key) + tok * p.key_stride_t + head * p.key_stride_h + d0;
  } else {
    const uint32_t j = rem - q.seg_value;
    head = q.div_value_chunks.div(j);
    chunk = j - head * q.value_chunks;
    seg = 3;
    d0 = static_cast<int32_t>(chunk) * VEC;
    src = static_cast<const Tin*>(q.value) + tok * q.value_stride_t + head * q.value_stride_h + d0;
  }
  if (blockIdx.x < p.prefetch_ctas) {
    prefetch_l2(src);
    if (NEOX && seg < 2) prefetch_l2(src + p.embed_dim);
  }
  pdl_prologue();

  int64_t slot = -1;
  if (seg != 0 && tok < q.num_slot_tokens) slot = __ldg(q.slot_mapping + tok);
  if (seg >= 2 && slot < 0) return;

  Chunk<VB> x, y;
  if (seg < 2) {
    const int64_t pos = __ldg(p.positions + tok);
    const bool rotate = pos >= 0 && pos < p.max_position;
    if (!rotate && slot < 0) return;
    Tin* xp = const_cast<Tin*>(src);
    Tin* yp = xp + p.embed_dim;
    load_chunk_inplace(x, xp);
    if constexpr (NEOX) load_chunk_inplace(y, yp);
    if (rotate) {
      const Tin* cp = static_cast<const Tin*>(p.cos_sin_cache) + pos * p.rot_dim + chunk * CS_VEC;
      Chunk<CSB> c, s;
      load_chunk_shared_ro(c, cp);
      load_chunk_shared_ro(s, cp + p.embed_dim);
      if constexpr (NEOX) {
        rotate_neox<Tin, VEC>(x, y, c, s);
      } else {
        rotate_gptj<Tin, VEC>(x, c, s);
      }
      if (seg == 0 || q.write_back_key) {
        store_chunk(xp, x, true);
        if constexpr (NEOX) store_chunk(yp, y, true);
      }
    }
    if (slot < 0) return;
  } else if (seg == 2) {
    load_chunk_inplace(x, src);  // key memory: other threads of this launch write its rotated part
  } else {
    load_chunk(x, src, VB % 32 == 0);
  }

  int64_t dst;
  if (q.linear_slots) {
    dst = slot * q.page_stride;
  } else {
    int64_t blk, off;
    split_slot(slot, q.block_size, q.bs_shift, blk, off);
    dst = blk * q.block_stride + off * q.page_stride;
  }
  dst += head * q.head_stride + d0;

  ScaleCtx sc{};
  if constexpr (KV != KVC_KV_AUTO) sc = make_scale_ctx<Tin, KV>(seg == 3 ? q.v_scale : q.k_scale);
  char* cache = static_cast<char*>(seg == 3 ? q.value_cache : q.key_cache);
  Chunk<OUT_B> out;
  convert_chunk<Tin, KV, VEC>(x, out, sc);
  store_chunk(cache + dst * OUT_ES, out, kWideOut);
  if constexpr (NEOX) {
    if (seg == 1) {
      convert_chunk<Tin, KV, VEC>(y, out, sc);
      store_chunk(cache + (dst + p.embed_dim) * OUT_ES, out, kWideOut);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
namespace {

struct RopeGeometry {
  int64_t num_tokens, num_heads, num_kv_heads, head_size, rot_dim, max_position;
  int64_t query_stride_t, query_stride_h, key_stride_t, key_stride_h;
  bool is_neox;
  int in_dtype;
};

int check_rope(const int64_t* positions, const void* query, const void* key, const void* cos_sin_cache,
               const RopeGeometry& g) {
  if (g.in_dtype != KVC_IN_F32 && g.in_dtype != KVC_IN_F16 && g.in_dtype != KVC_IN_BF16)
    return fail(KVC_ERR_UNSUPPORTED, "rotary_embedding: unsupported tensor type code " + std::to_string(g.in_dtype));
  if (g.num_tokens < 0 || g.num_heads < 0 || g.num_kv_heads < 0 || g.head_size <= 0)
    return fail(KVC_ERR_INVALID_ARG, "rotary_embedding: negative size");
  if (g.rot_dim <= 0 || g.rot_dim % 2 || g.rot_dim > g.head_size)
    return fail(KVC_ERR_INVALID_ARG, "rotary_embedding: rot_dim must be even and in (0, head_size]");
  if (g.max_position <= 0) return fail(KVC_ERR_INVALID_ARG, "rotary_embedding: max_position must be positive");
  if (g.head_size > 0x3FFFFFFFll || g.num_heads > 0x3FFFFFFFll || g.num_kv_heads > 0x3FFFFFFFll)
    return fail(KVC_ERR_INVALID_ARG, "rotary_embedding: sizes out of range");
  if (g.num_tokens == 0 || g.num_heads + g.num_kv_heads == 0) return KVC_OK;
  if (!positions || !cos_sin_cache || (g.num_heads > 0 && !query) || (g.num_kv_heads > 0 && !key))
    return fail(KVC_ERR_INVALID_ARG, "rotary_embedding: positions, query, key (when it has heads) and "
                                     "cos_sin_cache must be non-NULL");
  const int es = in_elem_size(g.in_dtype);
  if (!aligned(positions, 8)) return fail(KVC_ERR_INVALID_ARG, "rotary_embedding: positions must be 8-byte aligned");
  if (!aligned(query, es) || !aligned(key, es) || !aligned(cos_sin_cache, es))
    return fail(KVC_ERR_INVALID_ARG, "rotary_embedding: tensors are not aligned to their element size");
  return KVC_OK;
}

// Largest access width in bytes out of `candidates` (descending) that every data address of the
// rotation honours; 0 if none does.
int pick_rope_bytes(const int* candidates, int n, const void* query, const void* key, const void* cos_sin_cache,
                    const RopeGeometry& g) {
  const int es = in_elem_size(g.in_dtype);
  const int64_t embed = g.rot_dim / 2;
  for (int i = 0; i < n; ++i) {
    const int vb = candidates[i];
    const int vec = vb / es;
    if (vec < 2) continue;  // single elements: the pair kernel
    if ((g.is_neox ? embed : g.rot_dim) % vec) continue;
    const int csb = g.is_neox ? vb : vb / 2;
    bool ok = aligned(cos_sin_cache, csb) && (g.rot_dim * es) % csb == 0 && (embed * es) % csb == 0;
    if (g.num_heads > 0)
      ok = ok && aligned(query, vb) && (g.query_stride_t * es) % vb == 0 && (g.query_stride_h * es) % vb == 0;
    if (g.num_kv_heads > 0)
      ok = ok && aligned(key, vb) && (g.key_stride_t * es) % vb == 0 && (g.key_stride_h * es) % vb == 0;
    if (g.is_neox) ok = ok && (embed * es) % vb == 0;
    if (ok) return vb;
  }
  return 0;
}

void fill_rope_params(RopeParams& p, const void* cos_sin_cache, const RopeGeometry& g) {
  p.cos_sin_cache = cos_sin_cache;
  p.query_stride_t = g.query_stride_t;
  p.query_stride_h = g.query_stride_h;
  p.key_stride_t = g.key_stride_t;
  p.key_stride_h = g.key_stride_h;
  p.max_position = g.max_position;
  p.rot_dim = static_cast<int32_t>(g.rot_dim);
  p.embed_dim = static_cast<int32_t>(g.rot_dim / 2);
  p.num_q_heads = static_cast<uint32_t>(g.num_heads);
}

int64_t launch_item_limit() {
  static const int64_t limit = [] {
    const char* e = getenv("KVC_TEST_MAX_ITEMS_PER_LAUNCH");
    const int64_t v = e ? strtoll(e, nullptr, 10) : 0;
    return (v > 0 && v < (1ll << 31) - kRopeThreads) ? v : (1ll << 31) - kRopeThreads;
  }();
  return limit;
}

template <typename Tin, bool NEOX>
cudaError_t launch_rope(int vb, const RopeParams& p, dim3 grid, cudaStream_t st) {
  constexpr int ES = (int)sizeof(Tin);
  switch (vb) {
    case 32: return launch_pdl(rope_kernel<Tin, NEOX, 32 / ES>, grid, kRopeThreads, p, st);
    case 16: return launch_pdl(rope_kernel<Tin, NEOX, 16 / ES>, grid, kRopeThreads, p, st);
    case 8: return launch_pdl(rope_kernel<Tin, NEOX, 8 / ES>, grid, kRopeThreads, p, st);
    case 4:
      if constexpr (ES == 2) return launch_pdl(rope_kernel<Tin, NEOX, 2>, grid, kRopeThreads, p, st);
      [[fallthrough]];
    default: return launch_pdl(rope_pair_kernel<Tin, NEOX>, grid, kRopeThreads, p, st);
  }
}

template <typename Tin>
cudaError_t launch_rope_style(bool neox, int vb, const RopeParams& p, dim3 grid, cudaStream_t st) {
  return neox ? launch_rope<Tin, true>(vb, p, grid, st) : launch_rope<Tin, false>(vb, p, grid, st);
}

template <typename Tin, int KV, bool NEOX>
cudaError_t launch_rope_cache(int vb, const RopeCacheParams& q, dim3 grid, cudaStream_t st) {
  constexpr int ES = (int)sizeof(Tin);
  if (vb == 32) return launch_pdl(rope_cache_flash_kernel<Tin, KV, NEOX, 32 / ES>, grid, kRopeThreads, q, st);
  return launch_pdl(rope_cache_flash_kernel<Tin, KV, NEOX, 16 / ES>, grid, kRopeThreads, q, st);
}

template <typename Tin, int KV>
cudaError_t launch_rope_cache_style(bool neox, int vb, const RopeCacheParams& q, dim3 grid, cudaStream_t st) {
  return neox ? launch_rope_cache<Tin, KV, true>(vb, q, grid, st) : launch_rope_cache<Tin, KV, false>(vb, q, grid, st);
}

template <typename Tin>
cudaError_t launch_rope_cache_kv(int kv, bool neox, int vb, const RopeCacheParams& q, dim3 grid, cudaStream_t st) {
  switch (kv) {
    case KVC_KV_AUTO: return launch_rope_cache_style<Tin, KVC_KV_AUTO>(neox, vb, q, grid, st);
    case KVC_KV_FP8_E4M3: return launch_rope_cache_style<Tin, KVC_KV_FP8_E4M3>(neox, vb, q, grid, st);
    default: return launch_rope_cache_style<Tin, KVC_KV_FP8_E5M2>(neox, vb, q, grid, st);
  }
}

}  // namespace

static int rope_impl(const int64_t* positions, void* query, void* key, const void* cos_sin_cache,
                     const RopeGeometry& g, cudaStream_t st) {
  if (int rc = check_rope(positions, query, key, cos_sin_cache, g)) return rc;
  const int64_t heads = g.num_heads + g.num_kv_heads;
  if (g.num_tokens == 0 || heads == 0) return KVC_OK;
  const int es = in_elem_size(g.in_dtype);
  static const int kWidths[4] = {32, 16, 8, 4};
  const int vb = pick_rope_bytes(kWidths, 4, query, key, cos_sin_cache, g);
  const int64_t embed = g.rot_dim / 2;
  const int64_t chunks = vb ? (g.is_neox ? embed : g.rot_dim) / (vb / es) : embed;
  const int64_t items_per_token = heads * chunks;
  if (items_per_token >= (1ll << 30)) return fail(KVC_ERR_INVALID_ARG, "rotary_embedding: heads * rot_dim too large");

  RopeParams p{};
  fill_rope_params(p, cos_sin_cache, g);
  p.items_per_token = static_cast<uint32_t>(items_per_token);
  p.chunks_per_head = static_cast<uint32_t>(chunks);
  p.div_items_per_token = FastDiv(p.items_per_token);
  p.div_chunks_per_head = FastDiv(p.chunks_per_head);

  int64_t step = launch_item_limit() / items_per_token;
  if (step < 1) step = 1;
  for (int64_t t0 = 0; t0 < g.num_tokens; t0 += step) {
    const int64_t nt = (g.num_tokens - t0 < step) ? g.num_tokens - t0 : step;
    p.positions = positions + t0;
    p.query = query ? static_cast<char*>(query) + t0 * g.query_stride_t * es : nullptr;
    p.key = key ? static_cast<char*>(key) + t0 * g.key_stride_t * es : nullptr;
    p.n_items = static_cast<uint32_t>(nt * items_per_token);
    const dim3 grid((p.n_items + kRopeThreads - 1) / kRopeThreads);
    p.prefetch_ctas = prefetch_cta_count(grid.x);
    cudaError_t e;
    if (g.in_dtype == KVC_IN_F32) e = launch_rope_style<float>(g.is_neox, vb, p, grid, st);
    else if (g.in_dtype == KVC_IN_F16) e = launch_rope_style<__half>(g.is_neox, vb, p, grid, st);
    else e = launch_rope_style<__nv_bfloat16>(g.is_neox, vb, p, grid, st);
    if (e != cudaSuccess)
      return fail(KVC_ERR_CUDA, std::string("rotary_embedding launch failed: ") + cudaGetErrorString(e));
  }
  return KVC_OK;
}

static int rope_cache_impl(const int64_t* positions, void* query, void* key, const void* value,
                           const void* cos_sin_cache, void* key_cache, void* value_cache,
                           const int64_t* slot_mapping, const RopeGeometry& g, int64_t num_slot_tokens,
                           int64_t block_size, int64_t value_stride_t, int64_t value_stride_h,
                           int64_t block_stride, int64_t page_stride, int64_t head_stride, bool write_back_key,
                           int kv_dtype, const float* k_scale, const float* v_scale, cudaStream_t st) {
  if (int rc = check_rope(positions, query, key, cos_sin_cache, g)) return rc;
  if (kv_dtype != KVC_KV_AUTO && kv_dtype != KVC_KV_FP8_E4M3 && kv_dtype != KVC_KV_FP8_E5M2)
    return fail(KVC_ERR_UNSUPPORTED, "Unsupported data type of kv cache: code " + std::to_string(kv_dtype));
  if (block_size <= 0) return fail(KVC_ERR_INVALID_ARG, "block_size must be positive");
  if (num_slot_tokens < 0 || num_slot_tokens > g.num_tokens)
    return fail(KVC_ERR_INVALID_ARG, "num_slot_tokens must be in [0, num_tokens]");
  if (g.num_tokens == 0) return KVC_OK;
  if (g.num_kv_heads == 0) return fail(KVC_ERR_INVALID_ARG, "the fused op needs key heads; use kvc_rotary_embedding");
  if (!value || !key_cache || !value_cache || (num_slot_tokens > 0 && !slot_mapping))
    return fail(KVC_ERR_INVALID_ARG, "value, key_cache, value_cache and slot_mapping must be non-NULL");
  if (kv_dtype != KVC_KV_AUTO && (!k_scale || !v_scale))
    return fail(KVC_ERR_INVALID_ARG, "k_scale and v_scale must be non-NULL for an fp8 cache");
  if (slot_mapping && !aligned(slot_mapping, 8))
    return fail(KVC_ERR_INVALID_ARG, "slot_mapping must be 8-byte aligned");

  const int es = in_elem_size(g.in_dtype);
  const int out_es = (kv_dtype == KVC_KV_AUTO) ? es : 1;
  static const int kWidths[2] = {32, 16};
  int vb = 0;
  for (int i = 0; i < 2 && !vb; ++i) {
    const int cand = pick_rope_bytes(kWidths + i, 1, query, key, cos_sin_cache, g);
    if (!cand) continue;
    const int vec = cand / es;
    const int64_t ob = static_cast<int64_t>(vec) * out_es;
    bool ok = g.head_size % vec == 0 && (g.head_size - g.rot_dim) % vec == 0;
    ok = ok && aligned(value, cand) && (value_stride_t * es) % cand == 0 && (value_stride_h * es) % cand == 0;
    ok = ok && aligned(key_cache, ob) && aligned(value_cache, ob) && (block_stride * out_es) % ob == 0 &&
         (page_stride * out_es) % ob == 0 && (head_stride * out_es) % ob == 0;
    if (ok) vb = cand;
  }
  if (!vb)
    return fail(KVC_ERR_UNSUPPORTED,
                "rotary_embedding_and_cache_flash needs rows, strides and rot_dim / head_size that allow 16-byte "
                "accesses; call kvc_rotary_embedding and kvc_reshape_and_cache_flash instead");
  const int vec = vb / es;
  const int64_t embed = g.rot_dim / 2;
  const int64_t rope_chunks = (g.is_neox ? embed : g.rot_dim) / vec;
  const int64_t tail_chunks = (g.head_size - g.rot_dim) / vec;
  const int64_t value_chunks = g.head_size / vec;
  const int64_t seg_key = g.num_heads * rope_chunks;
  const int64_t seg_tail = seg_key + g.num_kv_heads * rope_chunks;
  const int64_t seg_value = seg_tail + g.num_kv_heads * tail_chunks;
  const int64_t items_per_token = seg_value + g.num_kv_heads * value_chunks;
  if (items_per_token >= (1ll << 30)) return fail(KVC_ERR_INVALID_ARG, "heads * head_size too large");

  RopeCacheParams q{};
  fill_rope_params(q.r, cos_sin_cache, g);
  q.r.items_per_token = static_cast<uint32_t>(items_per_token);
  q.r.chunks_per_head = static_cast<uint32_t>(rope_chunks);
  q.r.div_items_per_token = FastDiv(q.r.items_per_token);
  q.r.div_chunks_per_head = FastDiv(q.r.chunks_per_head);
  q.key_cache = key_cache;
  q.value_cache = value_cache;
  q.k_scale = k_scale;
  q.v_scale = v_scale;
  q.value_stride_t = value_stride_t;
  q.value_stride_h = value_stride_h;
  q.block_stride = block_stride;
  q.page_stride = page_stride;
  q.head_stride = head_stride;
  q.block_size = block_size;
  q.bs_shift = pow2_shift(block_size);
  q.linear_slots = (block_stride == block_size * page_stride);
  q.write_back_key = write_back_key;
  q.seg_key = static_cast<uint32_t>(seg_key);
  q.seg_tail = static_cast<uint32_t>(seg_tail);
  q.seg_value = static_cast<uint32_t>(seg_value);
  q.tail_chunks = static_cast<uint32_t>(tail_chunks);
  q.value_chunks = static_cast<uint32_t>(value_chunks);
  q.div_tail_chunks = FastDiv(q.tail_chunks ? q.tail_chunks : 1);
  q.div_value_chunks = FastDiv(q.value_chunks);

  int64_t step = launch_item_limit() / items_per_token;
  if (step < 1) step = 1;
  for (int64_t t0 = 0; t0 < g.num_tokens; t0 += step) {
    const int64_t nt = (g.num_tokens - t0 < step) ? g.num_tokens - t0 : step;
    q.r.positions = positions + t0;
    q.r.query = query ? static_cast<char*>(query) + t0 * g.query_stride_t * es : nullptr;
    q.r.key = static_cast<char*>(key) + t0 * g.key_stride_t * es;
    q.value = static_cast<const char*>(value) + t0 * value_stride_t * es;
    q.slot_mapping = slot_mapping ? slot_mapping + t0 : nullptr;
    q.num_slot_tokens = num_slot_tokens - t0;  // may be <= 0: no slots in this launch
    q.r.n_items = static_cast<uint32_t>(nt * items_per_token);
    const dim3 grid((q.r.n_items + kRopeThreads - 1) / kRopeThreads);
    q.r.prefetch_ctas = prefetch_cta_count(grid.x);
    cudaError_t e;
    if (g.in_dtype == KVC_IN_F32) e = launch_rope_cache_kv<float>(kv_dtype, g.is_neox, vb, q, grid, st);
    else if (g.in_dtype == KVC_IN_F16) e = launch_rope_cache_kv<__half>(kv_dtype, g.is_neox, vb, q, grid, st);
    else e = launch_rope_cache_kv<__nv_bfloat16>(kv_dtype, g.is_neox, vb, q, grid, st);
    if (e != cudaSuccess)
      return fail(KVC_ERR_CUDA,
                  std::string("rotary_embedding_and_cache_flash launch failed: ") + cudaGetErrorString(e));
  }
  return KVC_OK;
}

}  // namespace kvc

// ---------------------------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------------------------
extern "C" {

KVC_API int kvc_rotary_embedding(const int64_t* positions, void* query, void* key, const void* cos_sin_cache,
                                 int64_t num_tokens, int64_t num_heads, int64_t num_kv_heads, int64_t head_size,
                                 int64_t rot_dim, int64_t max_position, int64_t query_stride_t,
                                 int64_t query_stride_h, int64_t key_stride_t, int64_t key_stride_h, int is_neox,
                                 int in_dtype, void* stream) {
  const kvc::RopeGeometry g{num_tokens, num_heads, key ? num_kv_heads : 0, head_size, rot_dim, max_position,
                            query_stride_t, query_stride_h, key_stride_t, key_stride_h, is_neox != 0, in_dtype};
  return kvc::rope_impl(positions, query, key, cos_sin_cache, g, static_cast<cudaStream_t>(stream));
}

KVC_API int kvc_rotary_embedding_and_cache_flash(
    const int64_t* positions, void* query, void* key, const void* value, const void* cos_sin_cache, void* key_cache,
    void* value_cache, const int64_t* slot_mapping, int64_t num_tokens, int64_t num_slot_tokens, int64_t num_heads,
    int64_t num_kv_heads, int64_t head_size, int64_t rot_dim, int64_t max_position, int64_t block_size,
    int64_t query_stride_t, int64_t query_stride_h, int64_t key_stride_t, int64_t key_stride_h,
    int64_t value_stride_t, int64_t value_stride_h, int64_t block_stride, int64_t page_stride, int64_t head_stride,
    int is_neox, int write_back_key, int in_dtype, int kv_dtype, const float* k_scale, const float* v_scale,
    void* stream) {
  const kvc::RopeGeometry g{num_tokens, num_heads, num_kv_heads, head_size, rot_dim, max_position,
                            query_stride_t, query_stride_h, key_stride_t, key_stride_h, is_neox != 0, in_dtype};
  return kvc::rope_cache_impl(positions, query, key, value, cos_sin_cache, key_cache, value_cache, slot_mapping, g,
                              num_slot_tokens, block_size, value_stride_t, value_stride_h, block_stride,
                              page_stride, head_stride, write_back_key != 0, kv_dtype, k_scale, v_scale,
                              static_cast<cudaStream_t>(stream));
}

}  // extern "C"
