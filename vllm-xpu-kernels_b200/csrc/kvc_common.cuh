// Device and host helpers shared by the translation units of libkvcache_b200.so:
// error plumbing, index division, programmatic-dependent-launch prologue, vector global
// memory access, and the scalar pieces of the float -> fp8 conversion.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdlib>
#include <string>
#include <type_traits>

#include "kvcache_b200.h"

namespace kvc {

// ---------------------------------------------------------------------------------------------
// error plumbing
// ---------------------------------------------------------------------------------------------
// Records `msg` as the calling thread's last error and returns `code` (defined in kvcache_kernels.cu).
int fail(int code, const std::string& msg);

#define KVC_CUDA_TRY(expr)                                                                      \
  do {                                                                                          \
    cudaError_t _e = (expr);                                                                    \
    if (_e != cudaSuccess)                                                                      \
      return fail(KVC_ERR_CUDA, std::string(#expr " failed: ") + cudaGetErrorString(_e));       \
  } while (0)

// ---------------------------------------------------------------------------------------------
// division of a 31-bit index by a launch constant: q = umulhi(n, mul) >> shr
// ---------------------------------------------------------------------------------------------
struct FastDiv {
  uint32_t d, mul, shr;
  __host__ FastDiv(uint32_t div = 1) : d(div), mul(0), shr(0) {
    if (div > 1) {
      uint32_t lg = 0;
      while ((1ull << lg) < div) ++lg;  // ceil(log2 div)
      const uint32_t p = 31 + lg;
      mul = static_cast<uint32_t>(((1ull << p) + div - 1) / div);
      shr = p - 32;
    }
  }
  // exact for 0 <= n < 2^31
  __device__ __forceinline__ uint32_t div(uint32_t n) const { return d == 1 ? n : (__umulhi(n, mul) >> shr); }
};

// ---------------------------------------------------------------------------------------------
// programmatic dependent launch.  Every kernel here is launched with the
// programmatic-stream-serialization attribute and starts with pdl_prologue(): it may be
// scheduled while the previous kernel of the stream drains, then waits until that kernel
// has completed and its writes are visible before it touches memory, and at once allows its
// own successor to be scheduled the same way.  Without a programmatic predecessor the wait
// returns immediately.  Launch latency and CTA scheduling thus overlap the predecessor's tail.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void pdl_prologue() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Work that is legal BEFORE the wait: asking L2 to fetch lines this thread will read.  A prefetch
// has no architectural effect, so it cannot observe or disturb the predecessor; CTAs that are
// resident while the predecessor drains thereby start the memory system early and find their
// inputs in L2 once the wait returns.  Only the first CTAs of a grid can be in that position
// (`blockIdx.x < prefetch_ctas`); later ones would pay two requests for one line.
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// A slot read before the wait is only a HINT for what to prefetch (the predecessor may still be
// writing slot_mapping); the value is read again, for real, after the wait.
__device__ __forceinline__ int64_t slot_hint(const int64_t* p) { return *reinterpret_cast<const volatile int64_t*>(p); }

// ---------------------------------------------------------------------------------------------
// vector global memory access.  Loads are read-once streams: bypass L1 allocation.
// ---------------------------------------------------------------------------------------------
template <int BYTES>
struct alignas(BYTES >= 16 ? 16 : BYTES) Chunk {
  unsigned char b[BYTES];
};

// `wide`: the address is 32-byte aligned, so 32-byte pieces go out as single 256-bit loads
// (one full sector per lane per instruction; two 16-byte loads 32 bytes apart would make
// both instructions of a warp touch every sector).
template <int BYTES>
__device__ __forceinline__ void load_chunk(Chunk<BYTES>& c, const void* gptr, bool wide) {
  if constexpr (BYTES >= 16) {
    static_assert(BYTES % 16 == 0, "wide chunks are whole 16-byte vectors");
    uint4* dst = reinterpret_cast<uint4*>(c.b);
    if constexpr (BYTES % 32 == 0) {
      if (wide) {
#pragma unroll
        for (int i = 0; i < BYTES / 32; ++i) {
          uint4 lo, hi;
          asm volatile("ld.global.nc.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                       : "=r"(lo.x), "=r"(lo.y), "=r"(lo.z), "=r"(lo.w), "=r"(hi.x), "=r"(hi.y), "=r"(hi.z),
                         "=r"(hi.w)
                       : "l"(static_cast<const char*>(gptr) + 32 * i));
          dst[2 * i] = lo;
          dst[2 * i + 1] = hi;
        }
        return;
      }
    }
#pragma unroll
    for (int i = 0; i < BYTES / 16; ++i) {
      uint4 v;
      asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                   : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                   : "l"(static_cast<const char*>(gptr) + 16 * i));
      dst[i] = v;
    }
  } else if constexpr (BYTES == 8) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(gptr));
    *reinterpret_cast<uint2*>(c.b) = v;
  } else if constexpr (BYTES == 4) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(gptr));
    *reinterpret_cast<uint32_t*>(c.b) = v;
  } else if constexpr (BYTES == 2) {
    uint16_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(gptr));
    *reinterpret_cast<uint16_t*>(c.b) = v;
  } else {
    static_assert(BYTES == 1, "unsupported chunk size");
    c.b[0] = *static_cast<const unsigned char*>(gptr);
  }
}

// The same for memory that the running kernel also WRITES (an in-place op): a plain weak load,
// because the non-coherent path is only defined for data that stays read-only during the kernel.
// BYTES == 32 is one 256-bit access and needs a 32-byte aligned address; smaller sizes need
// their own size as alignment.
template <int BYTES>
__device__ __forceinline__ void load_chunk_inplace(Chunk<BYTES>& c, const void* gptr) {
  if constexpr (BYTES == 32) {
    uint4 lo, hi;
    asm volatile("ld.global.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(lo.x), "=r"(lo.y), "=r"(lo.z), "=r"(lo.w), "=r"(hi.x), "=r"(hi.y), "=r"(hi.z), "=r"(hi.w)
                 : "l"(gptr)
                 : "memory");
    reinterpret_cast<uint4*>(c.b)[0] = lo;
    reinterpret_cast<uint4*>(c.b)[1] = hi;
  } else if constexpr (BYTES == 16) {
    uint4 v;
    asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(gptr)
                 : "memory");
    *reinterpret_cast<uint4*>(c.b) = v;
  } else if constexpr (BYTES == 8) {
    uint2 v;
    asm volatile("ld.global.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(gptr) : "memory");
    *reinterpret_cast<uint2*>(c.b) = v;
  } else if constexpr (BYTES == 4) {
    uint32_t v;
    asm volatile("ld.global.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(gptr) : "memory");
    *reinterpret_cast<uint32_t*>(c.b) = v;
  } else {
    static_assert(BYTES == 2, "unsupported chunk size");
    uint16_t v;
    asm volatile("ld.global.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(gptr) : "memory");
    *reinterpret_cast<uint16_t*>(c.b) = v;
  }
}

// Read-only data that several threads of a CTA share (table rows): non-coherent path, L1 kept.
template <int BYTES>
__device__ __forceinline__ void load_chunk_shared_ro(Chunk<BYTES>& c, const void* gptr) {
  if constexpr (BYTES == 32) {
    uint4 lo, hi;
    asm volatile("ld.global.nc.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(lo.x), "=r"(lo.y), "=r"(lo.z), "=r"(lo.w), "=r"(hi.x), "=r"(hi.y), "=r"(hi.z), "=r"(hi.w)
                 : "l"(gptr));
    reinterpret_cast<uint4*>(c.b)[0] = lo;
    reinterpret_cast<uint4*>(c.b)[1] = hi;
  } else if constexpr (BYTES == 16) {
    *reinterpret_cast<uint4*>(c.b) = __ldg(static_cast<const uint4*>(gptr));
  } else if constexpr (BYTES == 8) {
    *reinterpret_cast<uint2*>(c.b) = __ldg(static_cast<const uint2*>(gptr));
  } else if constexpr (BYTES == 4) {
    *reinterpret_cast<uint32_t*>(c.b) = __ldg(static_cast<const uint32_t*>(gptr));
  } else if constexpr (BYTES == 2) {
    *reinterpret_cast<uint16_t*>(c.b) = __ldg(static_cast<const uint16_t*>(gptr));
  } else {
    static_assert(BYTES == 1, "unsupported chunk size");
    c.b[0] = __ldg(static_cast<const unsigned char*>(gptr));
  }
}

// Stores PIECE bytes taken at byte offset `at` of the chunk; PIECE in {16,8,4,2,1}.
template <int PIECE, int BYTES>
__device__ __forceinline__ void store_piece(void* gptr, const Chunk<BYTES>& c, int at) {
  if constexpr (PIECE == 16) {
    *reinterpret_cast<uint4*>(gptr) = *reinterpret_cast<const uint4*>(c.b + at);
  } else if constexpr (PIECE == 8) {
    *reinterpret_cast<uint2*>(gptr) = *reinterpret_cast<const uint2*>(c.b + at);
  } else if constexpr (PIECE == 4) {
    *reinterpret_cast<uint32_t*>(gptr) = *reinterpret_cast<const uint32_t*>(c.b + at);
  } else if constexpr (PIECE == 2) {
    *reinterpret_cast<uint16_t*>(gptr) = *reinterpret_cast<const uint16_t*>(c.b + at);
  } else {
    *reinterpret_cast<unsigned char*>(gptr) = c.b[at];
  }
}

// `wide`: the address is 32-byte aligned, so 32-byte pieces go out as single 256-bit stores
// (a lane then fills a whole sector with one instruction instead of two half-sector writes).
template <int BYTES>
__device__ __forceinline__ void store_chunk(void* gptr, const Chunk<BYTES>& c, bool wide) {
  if constexpr (BYTES % 32 == 0) {
    if (wide) {
      const uint4* src = reinterpret_cast<const uint4*>(c.b);
#pragma unroll
      for (int i = 0; i < BYTES / 32; ++i) {
        const uint4 lo = src[2 * i], hi = src[2 * i + 1];
        asm volatile("st.global.v8.u32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(static_cast<char*>(gptr) + 32 * i),
                     "r"(lo.x), "r"(lo.y), "r"(lo.z), "r"(lo.w), "r"(hi.x), "r"(hi.y), "r"(hi.z), "r"(hi.w)
                     : "memory");
      }
      return;
    }
  }
  constexpr int P = BYTES >= 16 ? 16 : BYTES;
#pragma unroll
  for (int i = 0; i < BYTES / P; ++i) store_piece<P>(static_cast<char*>(gptr) + P * i, c, P * i);
}

// ---------------------------------------------------------------------------------------------
// element conversion
// ---------------------------------------------------------------------------------------------
template <typename Tin>
__device__ __forceinline__ float to_f32(const unsigned char* p);
template <>
__device__ __forceinline__ float to_f32<float>(const unsigned char* p) {
  return *reinterpret_cast<const float*>(p);
}
template <>
__device__ __forceinline__ float to_f32<__half>(const unsigned char* p) {
  return __half2float(*reinterpret_cast<const __half*>(p));
}
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(const unsigned char* p) {
  return __uint_as_float(static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(p)) << 16);
}

// The two 16-bit floats packed in `w` as fp32 (lo = bits 0..15).
template <typename Tin>
__device__ __forceinline__ void unpack2(uint32_t w, float& lo, float& hi) {
  if constexpr (std::is_same_v<Tin, __nv_bfloat16>) {
    lo = __uint_as_float(w << 16);
    hi = __uint_as_float(w & 0xFFFF0000u);
  } else {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
    lo = f.x;
    hi = f.y;
  }
}

// sign(x) * min(|x|, c) on both 16-bit halves in one instruction; NaN stays NaN.
template <typename Tin>
__device__ __forceinline__ uint32_t clamp_magnitude2(uint32_t w, uint32_t c2) {
  uint32_t d;
  if constexpr (std::is_same_v<Tin, __nv_bfloat16>) {
    asm("min.NaN.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(w), "r"(c2));
  } else {
    asm("min.NaN.xorsign.abs.f16x2 %0, %1, %2;" : "=r"(d) : "r"(w), "r"(c2));
  }
  return d;
}

// Two floats -> two fp8 bytes (lo in bits 0..7), round-to-nearest-even, saturating.
template <int KV>
__device__ __forceinline__ uint32_t cvt_fp8x2(float lo, float hi) {
  uint16_t r;
  if constexpr (KV == KVC_KV_FP8_E4M3) {
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  } else {
    asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  }
  return r;
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
static inline int in_elem_size(int in_dtype) { return in_dtype == KVC_IN_F32 ? 4 : 2; }

static inline int pow2_shift(int64_t v) {
  if (v <= 0 || (v & (v - 1))) return -1;
  int s = 0;
  while ((1ll << s) < v) ++s;
  return s;
}

static inline bool aligned(const void* p, int64_t bytes) { return (reinterpret_cast<uintptr_t>(p) % bytes) == 0; }

// All kernels go out with the programmatic-stream-serialization attribute (see pdl_prologue).
// How many CTAs of a grid prefetch before the dependency wait.  While a same-shaped predecessor
// runs its last, partly filled wave, about half of what the device holds at once for a
// 256-thread, <= 32-register kernel (8 CTAs per SM, i.e. sms * 4) of this grid's CTAs are already
// resident and waiting; on B200 the measured optimum for back-to-back launches of grids of several
// waves is flat between 0.4 and 0.55 of a wave.  A grid that fits the device together with its
// predecessor is resident as a whole, and there half of its CTAs is the best count (1024-CTA
// grids: 4.61 us per launch with 512 prefetching CTAs against 4.70 with 592 and 5.19 with all;
// 512-CTA grids: 3.03 with 256 against 3.09 with all).  KVC_PREFETCH_CTAS overrides the count
// (0 switches the prefetch off).
static inline uint32_t prefetch_cta_count(uint32_t grid_ctas) {
  static const long override_count = [] {
    const char* e = getenv("KVC_PREFETCH_CTAS");
    return e ? strtol(e, nullptr, 10) : -1L;
  }();
  if (override_count >= 0) return static_cast<uint32_t>(override_count);
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (cached[dev] == 0) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) return 0;
    cached[dev] = sms * 4;
  }
  const uint32_t half_wave = static_cast<uint32_t>(cached[dev]);
  const uint32_t half_grid = (grid_ctas + 1) / 2;
  return half_grid < half_wave ? half_grid : half_wave;
}

template <typename Params>
static inline cudaError_t launch_pdl(void (*kernel)(const Params), dim3 grid, int threads, const Params& p,
                              cudaStream_t st) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(static_cast<unsigned>(threads));
  cfg.dynamicSmemBytes = 0;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, p);
}

}  // namespace kvc
