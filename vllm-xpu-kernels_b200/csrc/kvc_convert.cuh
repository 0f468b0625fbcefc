// The element conversion of the cache-write kernels (copy, or divide by a per-tensor scale and
// round to fp8) and the slot -> (block, offset) split, shared by the translation units that
// write into the paged cache.
#pragma once
#include "kvc_common.cuh"

namespace kvc {

// RN(x / s) in three instructions, given s > 0 and r = RN(1/s): one Newton correction of the
// product x*r with an exact residual.  For 16-bit float x this equals the IEEE quotient
// for every significand pair (checked exhaustively on the CPU) as long as nothing under-
// or overflows; make_scale_ctx() bounds s, and the caller clamps |x| so x*r stays finite.
// The residual is formed negated (ne = q0*s - x) and subtracted: when it is exactly zero
// it is +0, (-ne)*r is -0, and adding -0 leaves q0 unchanged even when q0 is itself -0.
// (With e = x - q0*s the sum (+0) + (-0) would turn a -0 quotient into +0.)
__device__ __forceinline__ float quot_fast(float x, float s, float r) {
  const float q0 = __fmul_rn(x, r);
  const float ne = __fmaf_rn(q0, s, -x);
  return __fmaf_rn(-ne, r, q0);
}

struct ScaleCtx {
  float s;         // the scale
  float r;         // RN(1/s)
  uint32_t clamp2; // two copies of the 16-bit clamp bound c (see below)
  bool fast;       // s is inside the window where quot_fast is exact
};

// Fast-path window of the scale, per input type (fp8_e4m3 / fp8_e5m2 store):
//   bf16  2^-60 <= s <= 2^60            r is normal; for every x whose quotient can round to a
//                                       non-zero fp8 value the residual fma is exact (no underflow)
//   fp16  2^-20 <= s <= 64 / 0.25       same, and the clamp bound is a normal, finite fp16
// Inside it |x| is first clamped to c = trunc16(m*s), m = 512 for e4m3 (largest finite 448,
// everything above 464 saturates) and 131072 for e5m2 (57344, 61440): a clamped element has
// |x/s| >= c/s > 0.99*m before and exactly c/s after, both beyond the saturation point, and
// |x*r| <= 1.01*m can no longer overflow (inf inputs included).  NaN stays NaN.
// Outside the window (and for negative scales, legal but never seen) the IEEE divide is used.
template <typename Tin, int KV>
__device__ __forceinline__ ScaleCtx make_scale_ctx(const float* scale_ptr) {
  ScaleCtx c;
  c.s = __ldg(scale_ptr);
  c.r = __frcp_rn(c.s);
  constexpr float kM = (KV == KVC_KV_FP8_E5M2) ? 131072.0f : 512.0f;
  if constexpr (std::is_same_v<Tin, __nv_bfloat16>) {
    c.fast = (c.s >= 8.673617379884035e-19f) && (c.s <= 1.152921504606847e18f);
    const uint32_t h = __float_as_uint(c.s * kM) >> 16;
    c.clamp2 = h | (h << 16);
  } else if constexpr (std::is_same_v<Tin, __half>) {
    constexpr float kHi = (KV == KVC_KV_FP8_E5M2) ? 0.25f : 64.0f;
    c.fast = (c.s >= 9.5367431640625e-07f) && (c.s <= kHi);
    const uint32_t h = __half_as_ushort(__float2half_rz(c.s * kM));
    c.clamp2 = h | (h << 16);
  } else {
    c.fast = false;
    c.clamp2 = 0;
  }
  return c;
}

// Converts VEC input elements to VEC output elements (AUTO: bit copy).
template <typename Tin, int KV, int VEC>
__device__ __forceinline__ void convert_chunk(const Chunk<VEC * (int)sizeof(Tin)>& in,
                                              Chunk<(KV == KVC_KV_AUTO ? VEC * (int)sizeof(Tin) : VEC)>& out,
                                              const ScaleCtx& sc) {
  if constexpr (KV == KVC_KV_AUTO) {
    out = in;
  } else {
    constexpr int ES = (int)sizeof(Tin);
    if constexpr (VEC >= 4 && ES == 2) {
      if (sc.fast) {
#pragma unroll
        for (int i = 0; i < VEC; i += 4) {
          const uint32_t a = clamp_magnitude2<Tin>(*reinterpret_cast<const uint32_t*>(in.b + ES * i), sc.clamp2);
          const uint32_t b = clamp_magnitude2<Tin>(*reinterpret_cast<const uint32_t*>(in.b + ES * (i + 2)), sc.clamp2);
          float x0, x1, x2, x3;
          unpack2<Tin>(a, x0, x1);
          unpack2<Tin>(b, x2, x3);
          *reinterpret_cast<uint32_t*>(out.b + i) =
              cvt_fp8x2<KV>(quot_fast(x0, sc.s, sc.r), quot_fast(x1, sc.s, sc.r)) |
              (cvt_fp8x2<KV>(quot_fast(x2, sc.s, sc.r), quot_fast(x3, sc.s, sc.r)) << 16);
        }
        return;
      }
    }
    if constexpr (VEC >= 2) {
#pragma unroll
      for (int i = 0; i < VEC; i += 2) {
        const float x0 = to_f32<Tin>(in.b + ES * i);
        const float x1 = to_f32<Tin>(in.b + ES * (i + 1));
        *reinterpret_cast<uint16_t*>(out.b + i) =
            static_cast<uint16_t>(cvt_fp8x2<KV>(__fdiv_rn(x0, sc.s), __fdiv_rn(x1, sc.s)));
      }
    } else {
      out.b[0] = static_cast<unsigned char>(cvt_fp8x2<KV>(__fdiv_rn(to_f32<Tin>(in.b), sc.s), 0.f) & 0xFFu);
    }
  }
}

// slot -> (block, offset).  Power-of-two block sizes (the common case) take a shift.
__device__ __forceinline__ void split_slot(int64_t slot, int64_t block_size, int bs_shift, int64_t& blk,
                                           int64_t& off) {
  if (bs_shift >= 0) {
    blk = slot >> bs_shift;
    off = slot & (block_size - 1);
  } else if (slot < 0x7FFFFFFFll && block_size < 0x7FFFFFFFll) {
    const uint32_t s32 = static_cast<uint32_t>(slot), b32 = static_cast<uint32_t>(block_size);
    blk = s32 / b32;
    off = s32 - static_cast<uint32_t>(blk) * b32;
  } else {
    blk = slot / block_size;
    off = slot - blk * block_size;
  }
}

}  // namespace kvc
