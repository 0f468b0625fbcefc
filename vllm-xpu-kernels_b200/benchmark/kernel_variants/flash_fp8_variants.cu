// Stand-alone comparison of kernel structures for the bf16 -> fp8_e4m3 flash-layout scatter on the
// measured shape (rows of 8 x 128 elements, runs of 64 slots, 8 rotating batches, CUDA graphs of 64
// launches).  Not part of the library: it documents why the shipped kernel looks the way it does.
// Every variant's output is compared with variant A's; "Z" variants drop the arithmetic and are the
// copy-shaped bound of the access pattern (their output is meaningless and reported as DIFF).
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -lineinfo -o flash_fp8_variants flash_fp8_variants.cu
//   ./flash_fp8_variants [num_tokens=16384]
//
// Holds two 4 GiB caches plus a 4 GiB reference pair and 8 input batches on the device.
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <vector>
#include <algorithm>
#include <random>
#include <cstring>

#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("CUDA error %s at %s:%d\n", cudaGetErrorString(e), __FILE__, __LINE__); exit(1);} } while (0)

constexpr int ROW = 1024;      // H*D elements per token
constexpr int BS = 64;
constexpr int BS_SHIFT = 6;

struct P {
  const uint16_t* key; const uint16_t* value; uint8_t* kc; uint8_t* vc; const int64_t* slots;
  const float* ks; const float* vs; int T;
};

__device__ __forceinline__ uint32_t cvt2(float lo, float hi) {
  uint16_t r; asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo)); return r;
}
__device__ __forceinline__ float quot_fast(float x, float s, float r) {
  const float q0 = __fmul_rn(x, r); const float ne = __fmaf_rn(q0, s, -x); return __fmaf_rn(-ne, r, q0);
}
__device__ __forceinline__ bool has_nan_byte(uint32_t w) { return (((w & 0x7F7F7F7Fu) + 0x01010101u) & 0x80808080u) != 0u; }

// 2 input words (4 bf16) -> 1 output word
__device__ __forceinline__ uint32_t conv4(uint32_t a, uint32_t b, float s, float r) {
  const float x0 = __uint_as_float(a << 16), x1 = __uint_as_float(a & 0xFFFF0000u);
  const float x2 = __uint_as_float(b << 16), x3 = __uint_as_float(b & 0xFFFF0000u);
  uint32_t w = cvt2(quot_fast(x0, s, r), quot_fast(x1, s, r)) | (cvt2(quot_fast(x2, s, r), quot_fast(x3, s, r)) << 16);
  if (has_nan_byte(w)) w = cvt2(__fdiv_rn(x0, s), __fdiv_rn(x1, s)) | (cvt2(__fdiv_rn(x2, s), __fdiv_rn(x3, s)) << 16);
  return w;
}
__device__ __forceinline__ uint4 ld16(const void* p) { uint4 v; asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p)); return v; }
__device__ __forceinline__ void ld32(const void* p, uint4& a, uint4& b) {
  asm volatile("ld.global.nc.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];" : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w), "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w) : "l"(p)); }
__device__ __forceinline__ uint2 conv8(uint4 a, float s, float r) { return make_uint2(conv4(a.x, a.y, s, r), conv4(a.z, a.w, s, r)); }
__device__ __forceinline__ uint4 conv16(uint4 a, uint4 b, float s, float r) { return make_uint4(conv4(a.x, a.y, s, r), conv4(a.z, a.w, s, r), conv4(b.x, b.y, s, r), conv4(b.z, b.w, s, r)); }

// ---- A: baseline: thread = 16 elements (2 x 16B loads 32B apart), grid over items
__global__ void __launch_bounds__(256) kA(const P p) {
  const uint32_t item = blockIdx.x * 256 + threadIdx.x;
  const uint32_t tok = item >> 6, c = item & 63;
  if (tok >= p.T) return;
  const int64_t slot = __ldg(p.slots + tok); if (slot < 0) return;
  const uint16_t* ks = p.key + (size_t)tok * ROW + c * 16; const uint16_t* vs = p.value + (size_t)tok * ROW + c * 16;
  uint4 k0 = ld16(ks), k1 = ld16(ks + 8), v0 = ld16(vs), v1 = ld16(vs + 8);
  const float sk = __ldg(p.ks), sv = __ldg(p.vs); const float rk = __frcp_rn(sk), rv = __frcp_rn(sv);
  const size_t dst = (size_t)slot * ROW + c * 16;
  *reinterpret_cast<uint4*>(p.kc + dst) = conv16(k0, k1, sk, rk);
  *reinterpret_cast<uint4*>(p.vc + dst) = conv16(v0, v1, sv, rv);
}
// ---- B: 32-byte loads
__global__ void __launch_bounds__(256) kB(const P p) {
  const uint32_t item = blockIdx.x * 256 + threadIdx.x;
  const uint32_t tok = item >> 6, c = item & 63;
  if (tok >= p.T) return;
  const int64_t slot = __ldg(p.slots + tok); if (slot < 0) return;
  uint4 k0, k1, v0, v1;
  ld32(p.key + (size_t)tok * ROW + c * 16, k0, k1); ld32(p.value + (size_t)tok * ROW + c * 16, v0, v1);
  const float sk = __ldg(p.ks), sv = __ldg(p.vs); const float rk = __frcp_rn(sk), rv = __frcp_rn(sv);
  const size_t dst = (size_t)slot * ROW + c * 16;
  *reinterpret_cast<uint4*>(p.kc + dst) = conv16(k0, k1, sk, rk);
  *reinterpret_cast<uint4*>(p.vc + dst) = conv16(v0, v1, sv, rv);
}
// ---- C: warp per token, lane-contiguous 16B loads, 4 chunks of K and of V per thread (8 loads in flight)
template <int THREADS>
__global__ void __launch_bounds__(THREADS) kC(const P p) {
  const uint32_t tok = blockIdx.x * (THREADS / 32) + (threadIdx.x >> 5); const uint32_t lane = threadIdx.x & 31;
  if (tok >= p.T) return;
  const int64_t slot = __ldg(p.slots + tok); if (slot < 0) return;
  const uint16_t* ks = p.key + (size_t)tok * ROW + lane * 8; const uint16_t* vs = p.value + (size_t)tok * ROW + lane * 8;
  uint4 k[4], v[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) k[i] = ld16(ks + i * 256);
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = ld16(vs + i * 256);
  const float sk = __ldg(p.ks), sv = __ldg(p.vs); const float rk = __frcp_rn(sk), rv = __frcp_rn(sv);
  const size_t dst = (size_t)slot * ROW + lane * 8;
#pragma unroll
  for (int i = 0; i < 4; ++i) *reinterpret_cast<uint2*>(p.kc + dst + i * 256) = conv8(k[i], sk, rk);
#pragma unroll
  for (int i = 0; i < 4; ++i) *reinterpret_cast<uint2*>(p.vc + dst + i * 256) = conv8(v[i], sv, rv);
}
// ---- D: persistent, 32B loads, one-deep software prefetch
__global__ void __launch_bounds__(256) kD(const P p) {
  const uint32_t nitems = (uint32_t)p.T * 64u; const uint32_t stride = gridDim.x * 256;
  uint32_t item = blockIdx.x * 256 + threadIdx.x;
  const float sk = __ldg(p.ks), sv = __ldg(p.vs); const float rk = __frcp_rn(sk), rv = __frcp_rn(sv);
  uint4 k0, k1, v0, v1; int64_t slot = -1;
  if (item < nitems) { slot = __ldg(p.slots + (item >> 6)); if (slot >= 0) { ld32(p.key + (size_t)item * 16, k0, k1); ld32(p.value + (size_t)item * 16, v0, v1);} }
  while (item < nitems) {
    const uint32_t nxt = item + stride; uint4 nk0, nk1, nv0, nv1; int64_t nslot = -1;
    if (nxt < nitems) { nslot = __ldg(p.slots + (nxt >> 6)); if (nslot >= 0) { ld32(p.key + (size_t)nxt * 16, nk0, nk1); ld32(p.value + (size_t)nxt * 16, nv0, nv1);} }
    if (slot >= 0) {
      const size_t dst = (size_t)slot * ROW + (item & 63) * 16;
      *reinterpret_cast<uint4*>(p.kc + dst) = conv16(k0, k1, sk, rk);
      *reinterpret_cast<uint4*>(p.vc + dst) = conv16(v0, v1, sv, rv);
    }
    item = nxt; slot = nslot; k0 = nk0; k1 = nk1; v0 = nv0; v1 = nv1;
  }
}
// ---- E: B but two items per thread (item and item + half), all loads first
__global__ void __launch_bounds__(256) kE(const P p) {
  const uint32_t half = (uint32_t)p.T * 32u;  // items / 2
  const uint32_t i0 = blockIdx.x * 256 + threadIdx.x; if (i0 >= half) return; const uint32_t i1 = i0 + half;
  const int64_t s0 = __ldg(p.slots + (i0 >> 6)), s1 = __ldg(p.slots + (i1 >> 6));
  uint4 a0, a1, b0, b1, c0, c1, d0, d1;
  if (s0 >= 0) { ld32(p.key + (size_t)i0 * 16, a0, a1); ld32(p.value + (size_t)i0 * 16, b0, b1); }
  if (s1 >= 0) { ld32(p.key + (size_t)i1 * 16, c0, c1); ld32(p.value + (size_t)i1 * 16, d0, d1); }
  const float sk = __ldg(p.ks), sv = __ldg(p.vs); const float rk = __frcp_rn(sk), rv = __frcp_rn(sv);
  if (s0 >= 0) { const size_t dst = (size_t)s0 * ROW + (i0 & 63) * 16; *reinterpret_cast<uint4*>(p.kc + dst) = conv16(a0, a1, sk, rk); *reinterpret_cast<uint4*>(p.vc + dst) = conv16(b0, b1, sv, rv); }
  if (s1 >= 0) { const size_t dst = (size_t)s1 * ROW + (i1 & 63) * 16; *reinterpret_cast<uint4*>(p.kc + dst) = conv16(c0, c1, sk, rk); *reinterpret_cast<uint4*>(p.vc + dst) = conv16(d0, d1, sv, rv); }
}
// ---- Z: pure copy-shaped lower bound: same loads, same stores, no conversion math (writes garbage)
__global__ void __launch_bounds__(256) kZ(const P p) {
  const uint32_t item = blockIdx.x * 256 + threadIdx.x;
  const uint32_t tok = item >> 6, c = item & 63;
  if (tok >= p.T) return;
  const int64_t slot = __ldg(p.slots + tok); if (slot < 0) return;
  uint4 k0, k1, v0, v1;
  ld32(p.key + (size_t)tok * ROW + c * 16, k0, k1); ld32(p.value + (size_t)tok * ROW + c * 16, v0, v1);
  const size_t dst = (size_t)slot * ROW + c * 16;
  *reinterpret_cast<uint4*>(p.kc + dst) = make_uint4(k0.x ^ k1.x, k0.y ^ k1.y, k0.z ^ k1.z, k0.w ^ k1.w);
  *reinterpret_cast<uint4*>(p.vc + dst) = make_uint4(v0.x ^ v1.x, v0.y ^ v1.y, v0.z ^ v1.z, v0.w ^ v1.w);
}


// ---- F: 32B loads, magnitude clamp on the packed bf16 words instead of the NaN-byte check
__device__ __forceinline__ uint32_t clamp2(uint32_t w, uint32_t c2) {
  uint32_t d; asm("min.NaN.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(w), "r"(c2)); return d;
}
__device__ __forceinline__ uint32_t conv4c(uint32_t a, uint32_t b, float s, float r, uint32_t c2) {
  a = clamp2(a, c2); b = clamp2(b, c2);
  const float x0 = __uint_as_float(a << 16), x1 = __uint_as_float(a & 0xFFFF0000u);
  const float x2 = __uint_as_float(b << 16), x3 = __uint_as_float(b & 0xFFFF0000u);
  return cvt2(quot_fast(x0, s, r), quot_fast(x1, s, r)) | (cvt2(quot_fast(x2, s, r), quot_fast(x3, s, r)) << 16);
}
__device__ __forceinline__ uint4 conv16c(uint4 a, uint4 b, float s, float r, uint32_t c2) { return make_uint4(conv4c(a.x, a.y, s, r, c2), conv4c(a.z, a.w, s, r, c2), conv4c(b.x, b.y, s, r, c2), conv4c(b.z, b.w, s, r, c2)); }
__device__ __forceinline__ uint32_t clamp_const(float s) {  // bf16x2 of trunc_bf16(512*s)
  const uint32_t u = __float_as_uint(s * 512.0f) >> 16; return u | (u << 16);
}
template <bool PDL, bool SPEC>
__global__ void __launch_bounds__(256) kF(const P p) {
  const uint32_t item = blockIdx.x * 256 + threadIdx.x;
  const uint32_t tok = item >> 6, c = item & 63;
  if (tok >= p.T) return;
  if (PDL) {
    asm volatile("prefetch.global.L2 [%0];" :: "l"(p.slots + tok));
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
  }
  uint4 k0, k1, v0, v1;
  int64_t slot;
  if (SPEC && blockIdx.x < 888) {
    slot = __ldg(p.slots + tok);
    ld32(p.key + (size_t)tok * ROW + c * 16, k0, k1); ld32(p.value + (size_t)tok * ROW + c * 16, v0, v1);
    if (slot < 0) return;
  } else {
    slot = __ldg(p.slots + tok); if (slot < 0) return;
    ld32(p.key + (size_t)tok * ROW + c * 16, k0, k1); ld32(p.value + (size_t)tok * ROW + c * 16, v0, v1);
  }
  const float sk = __ldg(p.ks), sv = __ldg(p.vs); const float rk = __frcp_rn(sk), rv = __frcp_rn(sv);
  const uint32_t ck = clamp_const(sk), cv = clamp_const(sv);
  const size_t dst = (size_t)slot * ROW + c * 16;
  *reinterpret_cast<uint4*>(p.kc + dst) = conv16c(k0, k1, sk, rk, ck);
  *reinterpret_cast<uint4*>(p.vc + dst) = conv16c(v0, v1, sv, rv, cv);
}
template <typename K>
static void launch_pdl(K kern, int grid, const P& p, cudaStream_t s) {
  cudaLaunchConfig_t cfg = {}; cfg.gridDim = dim3(grid); cfg.blockDim = dim3(256); cfg.stream = s;
  cudaLaunchAttribute at[1]; at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  CK(cudaLaunchKernelEx(&cfg, kern, p));
}

// ---- G: F + PDL variants
template <int THREADS, int MODE>  // MODE 0: plain; 1: CTA-shared scale ctx in smem; 2: st.cs; 3: both
__global__ void __launch_bounds__(THREADS) kG(const P p) {
  __shared__ float sh[6];
  const uint32_t item = blockIdx.x * THREADS + threadIdx.x;
  const uint32_t tok = item >> 6, c = item & 63;
  const bool inr = tok < p.T;
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;");
  int64_t slot = -1;
  if (inr) slot = __ldg(p.slots + tok);
  uint4 k0, k1, v0, v1;
  if (slot >= 0) { ld32(p.key + (size_t)tok * ROW + c * 16, k0, k1); ld32(p.value + (size_t)tok * ROW + c * 16, v0, v1); }
  float sk, sv, rk, rv; uint32_t ck, cv;
  if (MODE & 1) {
    if (threadIdx.x < 2) {
      const float s = __ldg(threadIdx.x ? p.vs : p.ks);
      sh[threadIdx.x * 3 + 0] = s; sh[threadIdx.x * 3 + 1] = __frcp_rn(s); sh[threadIdx.x * 3 + 2] = __uint_as_float(clamp_const(s));
    }
    __syncthreads();
    sk = sh[0]; rk = sh[1]; ck = __float_as_uint(sh[2]); sv = sh[3]; rv = sh[4]; cv = __float_as_uint(sh[5]);
  } else {
    sk = __ldg(p.ks); sv = __ldg(p.vs); rk = __frcp_rn(sk); rv = __frcp_rn(sv); ck = clamp_const(sk); cv = clamp_const(sv);
  }
  if (slot < 0) return;
  const size_t dst = (size_t)slot * ROW + c * 16;
  const uint4 ok = conv16c(k0, k1, sk, rk, ck), ov = conv16c(v0, v1, sv, rv, cv);
  if (MODE & 2) {
    asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" :: "l"(p.kc + dst), "r"(ok.x), "r"(ok.y), "r"(ok.z), "r"(ok.w) : "memory");
    asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" :: "l"(p.vc + dst), "r"(ov.x), "r"(ov.y), "r"(ov.z), "r"(ov.w) : "memory");
  } else {
    *reinterpret_cast<uint4*>(p.kc + dst) = ok; *reinterpret_cast<uint4*>(p.vc + dst) = ov;
  }
}
template <typename K>
static void launch_pdl_t(K kern, int grid, int threads, const P& p, cudaStream_t s) {
  cudaLaunchConfig_t cfg = {}; cfg.gridDim = dim3(grid); cfg.blockDim = dim3(threads); cfg.stream = s;
  cudaLaunchAttribute at[1]; at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  CK(cudaLaunchKernelEx(&cfg, kern, p));
}
// Z with PDL
__global__ void __launch_bounds__(256) kZp(const P p) {
  const uint32_t item = blockIdx.x * 256 + threadIdx.x;
  const uint32_t tok = item >> 6, c = item & 63;
  if (tok >= p.T) return;
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;");
  const int64_t slot = __ldg(p.slots + tok); if (slot < 0) return;
  uint4 k0, k1, v0, v1;
  ld32(p.key + (size_t)tok * ROW + c * 16, k0, k1); ld32(p.value + (size_t)tok * ROW + c * 16, v0, v1);
  const size_t dst = (size_t)slot * ROW + c * 16;
  *reinterpret_cast<uint4*>(p.kc + dst) = make_uint4(k0.x ^ k1.x, k0.y ^ k1.y, k0.z ^ k1.z, k0.w ^ k1.w);
  *reinterpret_cast<uint4*>(p.vc + dst) = make_uint4(v0.x ^ v1.x, v0.y ^ v1.y, v0.z ^ v1.z, v0.w ^ v1.w);
}

// ---- H: F + PDL + pre-wait L2 prefetch of this thread's inputs, steered by a speculative slot read
template <int MODE>  // 0: hint-steered prefetch of K,V; 1: unconditional prefetch; 2: prefetch slots only
__global__ void __launch_bounds__(256) kH(const P p) {
  const uint32_t item = blockIdx.x * 256 + threadIdx.x;
  const uint32_t tok = item >> 6, c = item & 63;
  if (tok >= p.T) return;
  const uint16_t* ksrc = p.key + (size_t)tok * ROW + c * 16; const uint16_t* vsrc = p.value + (size_t)tok * ROW + c * 16;
  if (MODE == 0) {
    const int64_t hint = *reinterpret_cast<const volatile int64_t*>(p.slots + tok);
    if (hint >= 0) { asm volatile("prefetch.global.L2 [%0];" :: "l"(ksrc)); asm volatile("prefetch.global.L2 [%0];" :: "l"(vsrc)); }
  } else if (MODE == 1) {
    asm volatile("prefetch.global.L2 [%0];" :: "l"(ksrc)); asm volatile("prefetch.global.L2 [%0];" :: "l"(vsrc));
    asm volatile("prefetch.global.L2 [%0];" :: "l"(p.slots + tok));
  } else {
    asm volatile("prefetch.global.L2 [%0];" :: "l"(p.slots + tok));
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;");
  const int64_t slot = __ldg(p.slots + tok); if (slot < 0) return;
  uint4 k0, k1, v0, v1;
  ld32(ksrc, k0, k1); ld32(vsrc, v0, v1);
  const float sk = __ldg(p.ks), sv = __ldg(p.vs); const float rk = __frcp_rn(sk), rv = __frcp_rn(sv);
  const uint32_t ck = clamp_const(sk), cv = clamp_const(sv);
  const size_t dst = (size_t)slot * ROW + c * 16;
  *reinterpret_cast<uint4*>(p.kc + dst) = conv16c(k0, k1, sk, rk, ck);
  *reinterpret_cast<uint4*>(p.vc + dst) = conv16c(v0, v1, sv, rv, cv);
}

static uint16_t f2bf(float f) { uint32_t u; memcpy(&u, &f, 4); u += 0x7FFF + ((u >> 16) & 1); return (uint16_t)(u >> 16); }

int main(int argc, char** argv) {
  const int T = argc > 1 ? atoi(argv[1]) : 16384;
  const int NB = 65536, NBUF = 8, GS = 64, REPS = 16;
  const size_t cache_bytes = (size_t)NB * BS * ROW;
  uint8_t *kc, *vc, *kc_ref, *vc_ref; CK(cudaMalloc(&kc, cache_bytes)); CK(cudaMalloc(&vc, cache_bytes));
  CK(cudaMalloc(&kc_ref, cache_bytes)); CK(cudaMalloc(&vc_ref, cache_bytes));
  CK(cudaMemset(kc, 0, cache_bytes)); CK(cudaMemset(vc, 0, cache_bytes)); CK(cudaMemset(kc_ref, 0, cache_bytes)); CK(cudaMemset(vc_ref, 0, cache_bytes));
  std::mt19937_64 rng(3); std::normal_distribution<float> nd(0.f, 2.f);
  std::vector<P> ps(NBUF);
  float *ks, *vs; CK(cudaMalloc(&ks, 4)); CK(cudaMalloc(&vs, 4));
  float amax = 0;
  std::vector<uint16_t> h((size_t)T * ROW);
  for (int b = 0; b < NBUF; ++b) {
    uint16_t *dk, *dv; int64_t* ds; CK(cudaMalloc(&dk, h.size() * 2)); CK(cudaMalloc(&dv, h.size() * 2)); CK(cudaMalloc(&ds, (size_t)T * 8));
    for (auto& x : h) { float f = nd(rng); amax = std::max(amax, fabsf(f)); x = f2bf(f); }
    CK(cudaMemcpy(dk, h.data(), h.size() * 2, cudaMemcpyHostToDevice));
    for (auto& x : h) { float f = nd(rng); amax = std::max(amax, fabsf(f)); x = f2bf(f); }
    CK(cudaMemcpy(dv, h.data(), h.size() * 2, cudaMemcpyHostToDevice));
    std::vector<int64_t> blocks(NB); for (int i = 0; i < NB; ++i) blocks[i] = i; std::shuffle(blocks.begin(), blocks.end(), rng);
    std::vector<int64_t> slots(T); for (int t = 0; t < T; ++t) slots[t] = blocks[t / BS] * BS + t % BS;
    CK(cudaMemcpy(ds, slots.data(), (size_t)T * 8, cudaMemcpyHostToDevice));
    ps[b] = P{dk, dv, kc, vc, ds, ks, vs, T};
  }
  float sc = amax / 448.f; CK(cudaMemcpy(ks, &sc, 4, cudaMemcpyHostToDevice)); CK(cudaMemcpy(vs, &sc, 4, cudaMemcpyHostToDevice));
  int nsm = 148; cudaDeviceGetAttribute(&nsm, cudaDevAttrMultiProcessorCount, 0);
  cudaStream_t st; CK(cudaStreamCreate(&st));
  const double bytes = 8.0 * T + (double)T * ROW * 2 * 3;

  struct V { const char* name; void (*launch)(const P&, cudaStream_t, int nsm); };
  std::vector<V> vars = {
    {"A baseline 2x16B", [](const P& p, cudaStream_t s, int) { kA<<<(p.T * 64 + 255) / 256, 256, 0, s>>>(p); }},
    {"B 32B loads", [](const P& p, cudaStream_t s, int) { kB<<<(p.T * 64 + 255) / 256, 256, 0, s>>>(p); }},
    {"C warp/token 256thr", [](const P& p, cudaStream_t s, int) { kC<256><<<(p.T + 7) / 8, 256, 0, s>>>(p); }},
    {"C warp/token 128thr", [](const P& p, cudaStream_t s, int) { kC<128><<<(p.T + 3) / 4, 128, 0, s>>>(p); }},
    {"D persistent x4", [](const P& p, cudaStream_t s, int n) { kD<<<n * 4, 256, 0, s>>>(p); }},
    {"D persistent x6", [](const P& p, cudaStream_t s, int n) { kD<<<n * 6, 256, 0, s>>>(p); }},
    {"D persistent x8", [](const P& p, cudaStream_t s, int n) { kD<<<n * 8, 256, 0, s>>>(p); }},
    {"E two items/thread", [](const P& p, cudaStream_t s, int) { kE<<<(p.T * 32 + 255) / 256, 256, 0, s>>>(p); }},
    {"F clamp", [](const P& p, cudaStream_t s, int) { kF<false, false><<<(p.T * 64 + 255) / 256, 256, 0, s>>>(p); }},
    {"F clamp + spec 1st wave", [](const P& p, cudaStream_t s, int) { kF<false, true><<<(p.T * 64 + 255) / 256, 256, 0, s>>>(p); }},
    {"F clamp + PDL", [](const P& p, cudaStream_t s, int) { launch_pdl(kF<true, false>, (p.T * 64 + 255) / 256, p, s); }},
    {"F clamp + PDL + spec", [](const P& p, cudaStream_t s, int) { launch_pdl(kF<true, true>, (p.T * 64 + 255) / 256, p, s); }},
    {"G256 plain", [](const P& p, cudaStream_t s, int) { launch_pdl_t(kG<256, 0>, (p.T * 64 + 255) / 256, 256, p, s); }},
    {"G256 smem ctx", [](const P& p, cudaStream_t s, int) { launch_pdl_t(kG<256, 1>, (p.T * 64 + 255) / 256, 256, p, s); }},
    {"G256 st.cs", [](const P& p, cudaStream_t s, int) { launch_pdl_t(kG<256, 2>, (p.T * 64 + 255) / 256, 256, p, s); }},
    {"G256 smem+cs", [](const P& p, cudaStream_t s, int) { launch_pdl_t(kG<256, 3>, (p.T * 64 + 255) / 256, 256, p, s); }},
    {"G128 smem ctx", [](const P& p, cudaStream_t s, int) { launch_pdl_t(kG<128, 1>, (p.T * 64 + 127) / 128, 128, p, s); }},
    {"G512 smem ctx", [](const P& p, cudaStream_t s, int) { launch_pdl_t(kG<512, 1>, (p.T * 64 + 511) / 512, 512, p, s); }},
    {"G1024 smem ctx", [](const P& p, cudaStream_t s, int) { launch_pdl_t(kG<1024, 1>, (p.T * 64 + 1023) / 1024, 1024, p, s); }},
    {"H hint prefetch", [](const P& p, cudaStream_t s, int) { launch_pdl(kH<0>, (p.T * 64 + 255) / 256, p, s); }},
    {"H uncond prefetch", [](const P& p, cudaStream_t s, int) { launch_pdl(kH<1>, (p.T * 64 + 255) / 256, p, s); }},
    {"H slot prefetch", [](const P& p, cudaStream_t s, int) { launch_pdl(kH<2>, (p.T * 64 + 255) / 256, p, s); }},
    {"Zp copy bound + PDL", [](const P& p, cudaStream_t s, int) { launch_pdl(kZp, (p.T * 64 + 255) / 256, p, s); }},
    {"Z copy-shaped bound", [](const P& p, cudaStream_t s, int) { kZ<<<(p.T * 64 + 255) / 256, 256, 0, s>>>(p); }},
  };
  // reference output from A into kc_ref/vc_ref (buffer 0 only)
  { P r = ps[0]; r.kc = kc_ref; r.vc = vc_ref; vars[0].launch(r, st, nsm); CK(cudaStreamSynchronize(st)); }
  std::vector<uint8_t> ref((size_t)1 << 22), got((size_t)1 << 22);
  for (auto& v : vars) {
    // correctness on buffer 0 : compare the first written block region
    CK(cudaMemsetAsync(kc, 0, cache_bytes, st));
    v.launch(ps[0], st, nsm); CK(cudaStreamSynchronize(st)); CK(cudaGetLastError());
    // compare the block of token 0
    int64_t slot0; CK(cudaMemcpy(&slot0, ps[0].slots, 8, cudaMemcpyDeviceToHost));
    size_t off = (size_t)(slot0 / BS) * BS * ROW; size_t len = (size_t)BS * ROW;
    CK(cudaMemcpy(ref.data(), kc_ref + off, len, cudaMemcpyDeviceToHost)); CK(cudaMemcpy(got.data(), kc + off, len, cudaMemcpyDeviceToHost));
    bool same = memcmp(ref.data(), got.data(), len) == 0;
    cudaGraph_t g; cudaGraphExec_t ge;
    CK(cudaStreamBeginCapture(st, cudaStreamCaptureModeGlobal));
    for (int i = 0; i < GS; ++i) v.launch(ps[i % NBUF], st, nsm);
    CK(cudaStreamEndCapture(st, &g)); CK(cudaGraphInstantiate(&ge, g, 0));
    for (int i = 0; i < 3; ++i) CK(cudaGraphLaunch(ge, st));
    cudaEvent_t e0, e1; CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1));
    float best = 1e9, sum = 0;
    for (int rep = 0; rep < 5; ++rep) {
      CK(cudaEventRecord(e0, st));
      for (int i = 0; i < REPS; ++i) CK(cudaGraphLaunch(ge, st));
      CK(cudaEventRecord(e1, st)); CK(cudaStreamSynchronize(st));
      float ms; CK(cudaEventElapsedTime(&ms, e0, e1)); best = std::min(best, ms); sum += ms;
    }
    const double us = best * 1e3 / (GS * REPS), us_avg = sum / 5 * 1e3 / (GS * REPS);
    // isolated launches: a dummy ordinary kernel before each one, so no programmatic predecessor exists
    float iso = 0; {
      const int N = 64; std::vector<cudaEvent_t> a(N), b(N);
      for (int i = 0; i < N; ++i) { CK(cudaEventCreate(&a[i])); CK(cudaEventCreate(&b[i])); }
      for (int i = 0; i < N; ++i) { CK(cudaMemsetAsync(ks == nullptr ? nullptr : (void*)kc_ref, 0, 256, st)); CK(cudaEventRecord(a[i], st)); v.launch(ps[i % NBUF], st, nsm); CK(cudaEventRecord(b[i], st)); }
      CK(cudaStreamSynchronize(st));
      std::vector<float> ts(N); for (int i = 0; i < N; ++i) CK(cudaEventElapsedTime(&ts[i], a[i], b[i]));
      std::sort(ts.begin(), ts.end()); iso = ts[N / 2] * 1e3f;
    }
    printf("%-24s %s  best %.2f us/launch (%.0f GB/s)  avg %.2f us   isolated median %.2f us\n", v.name, same ? "ok  " : "DIFF", us, bytes / us / 1e3, us_avg, iso);
    CK(cudaGraphExecDestroy(ge)); CK(cudaGraphDestroy(g));
  }
  return 0;
}
