// fp8 activation quantisation for NVIDIA B200 (sm_100a): static per-tensor, dynamic per-tensor and
// dynamic per-token, sharing the conversion pieces of the KV-cache write kernels.
//
// Reference counterparts: csrc/quantization/fp8/fp8_quant.cpp:15-45 (static kernel), :47-131
// (per-token kernel), :135-250 (host launchers), csrc/quantization/fp8/fp8_quant.h:56-102 (absmax
// reduction with an atomic max), csrc/quantization/fp8/quant_utils.h:80-91 (the element rule).
//
// Element rule (quant_utils.h:80-91, is_scale_inverted = true):
//     q = fmax(-M, fmin(float(x) * inv, M));  byte = round_to_nearest_even_fp8(q)
// with inv = 1.0f / scale computed ONCE in fp32 and M the largest finite value of the fp8 type
// (448 / 57344).  This is a multiplication by a rounded reciprocal, NOT the correctly rounded
// division the KV-cache ops use; the two differ in the last place and the reference's tests pin
// this one (tests/test_fp8_quant.py:20-38 there).  fmin/fmax return the non-NaN operand, so a NaN
// product becomes +M, exactly as the reference's sycl::fmin/fmax do.
#include <cstdio>

#include "kvc_common.cuh"

namespace kvc {

template <int F8>
__device__ __forceinline__ constexpr float fp8_max() {
  return F8 == KVC_KV_FP8_E5M2 ? 57344.0f : 448.0f;
}

__device__ __forceinline__ float clamp_scaled(float x, float inv, float m) { return fmaxf(-m, fminf(__fmul_rn(x, inv), m)); }

// VEC consecutive elements -> VEC fp8 bytes.
template <typename Tin, int F8, int VEC>
__device__ __forceinline__ void quantise_chunk(const Chunk<VEC * (int)sizeof(Tin)>& in, Chunk<VEC>& out, float inv) {
  constexpr int ES = (int)sizeof(Tin);
  constexpr float M = fp8_max<F8>();
  if constexpr (VEC >= 2) {
#pragma unroll
    for (int i = 0; i < VEC; i += 2) {
      float x0, x1;
      if constexpr (ES == 2) {
        unpack2<Tin>(*reinterpret_cast<const uint32_t*>(in.b + ES * i), x0, x1);
      } else {
        x0 = to_f32<Tin>(in.b + ES * i);
        x1 = to_f32<Tin>(in.b + ES * (i + 1));
      }
      *reinterpret_cast<uint16_t*>(out.b + i) =
          static_cast<uint16_t>(cvt_fp8x2<F8>(clamp_scaled(x0, inv, M), clamp_scaled(x1, inv, M)));
    }
  } else {
    out.b[0] = static_cast<unsigned char>(cvt_fp8x2<F8>(clamp_scaled(to_f32<Tin>(in.b), inv, M), 0.f) & 0xFFu);
  }
}

// |x| maximum over the VEC elements of a chunk (NaN is ignored by fmaxf, as in the reference's sycl::max).
template <typename Tin, int VEC>
__device__ __forceinline__ float chunk_absmax(const Chunk<VEC * (int)sizeof(Tin)>& in, float m) {
#pragma unroll
  for (int i = 0; i < VEC; ++i) m = fmaxf(m, fabsf(to_f32<Tin>(in.b + (int)sizeof(Tin) * i)));
  return m;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
  return v;
}

constexpr int kQuantThreads = 256;

struct QuantParams {
  const void* input;
  void* out;
  const float* scale;  // per-tensor scale (static / second pass of dynamic)
  int64_t num_elems;
  int64_t n_chunks;    // num_elems / VEC
  bool wide_loads;
};

// out[i] = fp8(clamp(x[i] * (1/scale))): one VEC-element chunk per thread plus a scalar tail.
template <typename Tin, int F8, int VEC>
__global__ void __launch_bounds__(kQuantThreads) scaled_fp8_quant_kernel(const QuantParams p) {
  const int64_t c = static_cast<int64_t>(blockIdx.x) * kQuantThreads + threadIdx.x;
  const int64_t tail0 = p.n_chunks * VEC;
  if (c >= p.n_chunks + (p.num_elems - tail0)) return;
  pdl_prologue();
  const float inv = 1.0f / __ldg(p.scale);  // IEEE division, as the reference computes it
  if (c < p.n_chunks) {
    Chunk<VEC * (int)sizeof(Tin)> in;
    load_chunk(in, static_cast<const Tin*>(p.input) + c * VEC, p.wide_loads);
    Chunk<VEC> out;
    quantise_chunk<Tin, F8, VEC>(in, out, inv);
    store_chunk(static_cast<unsigned char*>(p.out) + c * VEC, out, false);
  } else {  // fewer than VEC elements left over
    const int64_t i = tail0 + (c - p.n_chunks);
    Chunk<(int)sizeof(Tin)> in;
    load_chunk(in, static_cast<const Tin*>(p.input) + i, false);
    Chunk<1> out;
    quantise_chunk<Tin, F8, 1>(in, out, inv);
    static_cast<unsigned char*>(p.out)[i] = out.b[0];
  }
}

// scale = max(scale, absmax(x) / M) by a grid-stride pass and one atomic per CTA.  Non-negative
// floats order like their bit patterns, so the atomic max runs on the integer view.  The caller
// zero-initialises *scale (the reference's wrapper does: tests/ops/fp8_quant_op.py:66).
template <typename Tin, int F8, int VEC>
__global__ void __launch_bounds__(kQuantThreads) absmax_to_scale_kernel(const QuantParams p, float* scale_out) {
  __shared__ float warp_part[kQuantThreads / 32];
  pdl_prologue();
  float m = 0.0f;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kQuantThreads;
  // four chunks per pass: four independent loads in flight per thread
  for (int64_t c0 = static_cast<int64_t>(blockIdx.x) * kQuantThreads + threadIdx.x; c0 < p.n_chunks; c0 += 4 * stride) {
    Chunk<VEC * (int)sizeof(Tin)> in[4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (c0 + u * stride < p.n_chunks)
        load_chunk(in[u], static_cast<const Tin*>(p.input) + (c0 + u * stride) * VEC, p.wide_loads);
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (c0 + u * stride < p.n_chunks) m = chunk_absmax<Tin, VEC>(in[u], m);
  }
  for (int64_t i = p.n_chunks * VEC + static_cast<int64_t>(blockIdx.x) * kQuantThreads + threadIdx.x; i < p.num_elems;
       i += stride)
    m = fmaxf(m, fabsf(to_f32<Tin>(reinterpret_cast<const unsigned char*>(static_cast<const Tin*>(p.input) + i))));
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < kQuantThreads / 32 ? warp_part[threadIdx.x] : 0.0f;
    v = warp_max(v);
    if (threadIdx.x == 0) atomicMax(reinterpret_cast<int*>(scale_out), __float_as_int(__fdiv_rn(v, fp8_max<F8>())));
  }
}

struct TokenQuantParams {
  const void* input;
  void* out;
  float* scales;
  const float* scale_ub;  // may be null
  int64_t hidden_size;
  int64_t n_chunks;       // hidden_size / VEC
  bool wide_loads;
};

// One CTA per token: |x| maximum over the row (first sweep), scale = max(min(absmax, ub) / M,
// 1 / (512 M)), then the row is swept again (it is at most a few tens of KB and still in L1/L2)
// and quantised with the reciprocal of that scale.
template <typename Tin, int F8, int VEC>
__global__ void __launch_bounds__(kQuantThreads) per_token_fp8_quant_kernel(const TokenQuantParams p) {
  __shared__ float warp_part[kQuantThreads / 32];
  __shared__ float token_scale;
  pdl_prologue();
  const int64_t tok = blockIdx.x;
  const Tin* row = static_cast<const Tin*>(p.input) + tok * p.hidden_size;
  unsigned char* orow = static_cast<unsigned char*>(p.out) + tok * p.hidden_size;
  const int64_t tail0 = p.n_chunks * VEC;

  float m = 0.0f;
  for (int64_t c = threadIdx.x; c < p.n_chunks; c += kQuantThreads) {
    Chunk<VEC * (int)sizeof(Tin)> in;
    // the row is read again below: let it allocate in L1 (plain load path) -- chunks of a row are small
    in = *reinterpret_cast<const Chunk<VEC * (int)sizeof(Tin)>*>(row + c * VEC);
    m = chunk_absmax<Tin, VEC>(in, m);
  }
  for (int64_t i = tail0 + threadIdx.x; i < p.hidden_size; i += kQuantThreads)
    m = fmaxf(m, fabsf(to_f32<Tin>(reinterpret_cast<const unsigned char*>(row + i))));
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < kQuantThreads / 32 ? warp_part[threadIdx.x] : 0.0f;
    v = warp_max(v);
    if (threadIdx.x == 0) {
      if (p.scale_ub != nullptr) v = fminf(v, __ldg(p.scale_ub));
      constexpr float M = fp8_max<F8>();
      const float s = fmaxf(__fdiv_rn(v, M), __fdiv_rn(1.0f, M * 512.0f));
      token_scale = s;
      p.scales[tok] = s;
    }
  }
  __syncthreads();
  const float inv = 1.0f / token_scale;

  for (int64_t c = threadIdx.x; c < p.n_chunks; c += kQuantThreads) {
    Chunk<VEC * (int)sizeof(Tin)> in = *reinterpret_cast<const Chunk<VEC * (int)sizeof(Tin)>*>(row + c * VEC);
    Chunk<VEC> out;
    quantise_chunk<Tin, F8, VEC>(in, out, inv);
    store_chunk(orow + c * VEC, out, false);
  }
  for (int64_t i = tail0 + threadIdx.x; i < p.hidden_size; i += kQuantThreads) {
    Chunk<(int)sizeof(Tin)> in = *reinterpret_cast<const Chunk<(int)sizeof(Tin)>*>(row + i);
    Chunk<1> out;
    quantise_chunk<Tin, F8, 1>(in, out, inv);
    orow[i] = out.b[0];
  }
}

// Register-resident form of the per-token op: the row is read from HBM ONCE, kept in registers
// (up to kRowChunks chunks per thread) across the reduction, and quantised from there.
//   WARP = true   a warp per token (rows of at most 32 * kRowChunks chunks): shuffles only, no barrier,
//                 eight tokens per CTA
//   WARP = false  a CTA of 64, 128 or 256 threads per token (the smallest that holds the row with
//                 kRowChunks chunks per thread, so every thread has several loads in flight):
//                 shuffles, one shared-memory step, one barrier
// VEC divides hidden_size (the host sees to it), so rows have no scalar tail here.
constexpr int kRowChunks = 4;

template <typename Tin, int F8, int VEC, bool WARP>
__global__ void __launch_bounds__(kQuantThreads) per_token_fp8_quant_regs_kernel(const TokenQuantParams p,
                                                                                  int64_t num_tokens) {
  const int G = WARP ? 32 : static_cast<int>(blockDim.x);
  __shared__ float warp_part[kQuantThreads / 32];
  const int g = WARP ? (threadIdx.x & 31) : threadIdx.x;
  const int64_t tok = WARP ? static_cast<int64_t>(blockIdx.x) * (kQuantThreads / 32) + (threadIdx.x >> 5)
                           : static_cast<int64_t>(blockIdx.x);
  if (WARP && tok >= num_tokens) return;  // whole warps leave together; no barrier is used in this mode
  pdl_prologue();
  const Tin* row = static_cast<const Tin*>(p.input) + tok * p.hidden_size;
  unsigned char* orow = static_cast<unsigned char*>(p.out) + tok * p.hidden_size;

  Chunk<VEC * (int)sizeof(Tin)> in[kRowChunks];
#pragma unroll
  for (int u = 0; u < kRowChunks; ++u) {
    const int64_t c = g + u * G;
    if (c < p.n_chunks) load_chunk(in[u], row + c * VEC, p.wide_loads);
  }
  float m = 0.0f;
#pragma unroll
  for (int u = 0; u < kRowChunks; ++u)
    if (g + u * G < p.n_chunks) m = chunk_absmax<Tin, VEC>(in[u], m);
  m = warp_max(m);
  if constexpr (!WARP) {
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = m;
    __syncthreads();
    float v = (threadIdx.x & 31) < (blockDim.x >> 5) ? warp_part[threadIdx.x & 31] : 0.0f;
    m = warp_max(v);  // every warp reduces the partials itself: no second barrier, no broadcast
  }
  if (p.scale_ub != nullptr) m = fminf(m, __ldg(p.scale_ub));
  constexpr float M = fp8_max<F8>();
  const float s = fmaxf(__fdiv_rn(m, M), __fdiv_rn(1.0f, M * 512.0f));
  if (g == 0) p.scales[tok] = s;
  const float inv = 1.0f / s;
#pragma unroll
  for (int u = 0; u < kRowChunks; ++u) {
    const int64_t c = g + u * G;
    if (c < p.n_chunks) {
      Chunk<VEC> out;
      quantise_chunk<Tin, F8, VEC>(in[u], out, inv);
      store_chunk(orow + c * VEC, out, false);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
static int check_quant_args(const void* out, const void* input, int in_dtype, int fp8_dtype) {
  if (in_dtype != KVC_IN_F32 && in_dtype != KVC_IN_F16 && in_dtype != KVC_IN_BF16)
    return fail(KVC_ERR_UNSUPPORTED, "fp8 quant: unsupported input dtype code " + std::to_string(in_dtype));
  if (fp8_dtype != KVC_KV_FP8_E4M3 && fp8_dtype != KVC_KV_FP8_E5M2)
    return fail(KVC_ERR_UNSUPPORTED, "fp8 quant: output must be fp8_e4m3 or fp8_e5m2");
  if (!out || !input) return fail(KVC_ERR_INVALID_ARG, "fp8 quant: out and input must be non-NULL");
  if (!aligned(input, in_elem_size(in_dtype))) return fail(KVC_ERR_INVALID_ARG, "fp8 quant: input is misaligned");
  return KVC_OK;
}

// vector width for a flat array: 16 when both sides allow 16-byte stores / whole-vector loads
static int flat_vec(const void* input, const void* out, int es_in) {
  int v = 16;
  while (v > 1 && (!aligned(out, v) || !aligned(input, (static_cast<int64_t>(v) * es_in >= 16) ? 16 : v * es_in))) v >>= 1;
  return v;
}

template <typename T>
struct TypeTag {
  using type = T;
};

#define KVC_QUANT_DISPATCH(IN_DTYPE, F8, VEC, FN, ...)                                               \
  [&]() -> cudaError_t {                                                                             \
    auto by_vec = [&](auto tin_tag, auto f8_tag) -> cudaError_t {                                    \
      using T = typename decltype(tin_tag)::type;                                                    \
      constexpr int kF8 = decltype(f8_tag)::value;                                                   \
      switch (VEC) {                                                                                 \
        case 16: return FN<T, kF8, 16>(__VA_ARGS__);                                                 \
        case 8: return FN<T, kF8, 8>(__VA_ARGS__);                                                   \
        case 4: return FN<T, kF8, 4>(__VA_ARGS__);                                                   \
        case 2: return FN<T, kF8, 2>(__VA_ARGS__);                                                   \
        default: return FN<T, kF8, 1>(__VA_ARGS__);                                                  \
      }                                                                                              \
    };                                                                                               \
    auto by_f8 = [&](auto tin_tag) -> cudaError_t {                                                  \
      return (F8) == KVC_KV_FP8_E5M2 ? by_vec(tin_tag, std::integral_constant<int, KVC_KV_FP8_E5M2>{}) \
                                     : by_vec(tin_tag, std::integral_constant<int, KVC_KV_FP8_E4M3>{}); \
    };                                                                                               \
    switch (IN_DTYPE) {                                                                              \
      case KVC_IN_F32: return by_f8(TypeTag<float>{});                                    \
      case KVC_IN_F16: return by_f8(TypeTag<__half>{});                                   \
      default: return by_f8(TypeTag<__nv_bfloat16>{});                                    \
    }                                                                                                \
  }()

template <typename Tin, int F8, int VEC>
static cudaError_t launch_static(const QuantParams& p, cudaStream_t st) {
  const int64_t threads = p.n_chunks + (p.num_elems - p.n_chunks * VEC);
  const dim3 grid(static_cast<unsigned>((threads + kQuantThreads - 1) / kQuantThreads));
  return launch_pdl(scaled_fp8_quant_kernel<Tin, F8, VEC>, grid, kQuantThreads, p, st);
}

template <typename Tin, int F8, int VEC>
static cudaError_t launch_absmax(const QuantParams& p, float* scale_out, cudaStream_t st) {
  int64_t blocks = (p.n_chunks + kQuantThreads - 1) / kQuantThreads;
  if (blocks < 1) blocks = 1;
  if (blocks > 148 * 8) blocks = 148 * 8;  // one resident wave on 148 SMs; the loop strides over the rest
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(blocks));
  cfg.blockDim = dim3(kQuantThreads);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, absmax_to_scale_kernel<Tin, F8, VEC>, p, scale_out);
}

template <typename K>
static cudaError_t launch_pdl2(K kernel, dim3 grid, int threads, const TokenQuantParams& p, int64_t num_tokens,
                               cudaStream_t st) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(static_cast<unsigned>(threads));
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, p, num_tokens);
}

template <typename Tin, int F8, int VEC>
static cudaError_t launch_per_token(const TokenQuantParams& p, int64_t num_tokens, cudaStream_t st) {
  if constexpr (VEC >= 8) {  // wide chunks: keep the row in registers when it fits
    if (p.n_chunks <= 32 * kRowChunks) {
      const int64_t ctas = (num_tokens + kQuantThreads / 32 - 1) / (kQuantThreads / 32);
      return launch_pdl2(per_token_fp8_quant_regs_kernel<Tin, F8, VEC, true>, dim3(static_cast<unsigned>(ctas)),
                         kQuantThreads, p, num_tokens, st);
    }
    if (p.n_chunks <= kQuantThreads * kRowChunks) {
      int threads = 64;
      while (static_cast<int64_t>(threads) * kRowChunks < p.n_chunks) threads *= 2;
      return launch_pdl2(per_token_fp8_quant_regs_kernel<Tin, F8, VEC, false>, dim3(static_cast<unsigned>(num_tokens)),
                         threads, p, num_tokens, st);
    }
  }
  return launch_pdl(per_token_fp8_quant_kernel<Tin, F8, VEC>, dim3(static_cast<unsigned>(num_tokens)), kQuantThreads,
                    p, st);
}

static int static_quant_impl(void* out, const void* input, const float* scale, int64_t num_elems, int in_dtype,
                             int fp8_dtype, cudaStream_t st) {
  if (num_elems < 0) return fail(KVC_ERR_INVALID_ARG, "fp8 quant: negative element count");
  if (num_elems == 0) return KVC_OK;
  if (int rc = check_quant_args(out, input, in_dtype, fp8_dtype)) return rc;
  if (!scale) return fail(KVC_ERR_INVALID_ARG, "fp8 quant: scale must be non-NULL");
  const int es = in_elem_size(in_dtype);
  const int vec = flat_vec(input, out, es);
  QuantParams p{};
  p.input = input;
  p.out = out;
  p.scale = scale;
  p.num_elems = num_elems;
  p.n_chunks = num_elems / vec;
  p.wide_loads = (static_cast<int64_t>(vec) * es) % 32 == 0 && aligned(input, 32);
  if (p.n_chunks + vec >= (1ll << 31) * kQuantThreads) return fail(KVC_ERR_INVALID_ARG, "fp8 quant: tensor too large");
  const cudaError_t e = KVC_QUANT_DISPATCH(in_dtype, fp8_dtype, vec, launch_static, p, st);
  if (e != cudaSuccess) return fail(KVC_ERR_CUDA, std::string("scaled_fp8_quant launch failed: ") + cudaGetErrorString(e));
  return KVC_OK;
}

}  // namespace kvc

using namespace kvc;

extern "C" {

int kvc_static_scaled_fp8_quant(void* out, const void* input, const float* scale, int64_t num_elems, int in_dtype,
                                int fp8_dtype, void* stream) {
  return static_quant_impl(out, input, scale, num_elems, in_dtype, fp8_dtype, static_cast<cudaStream_t>(stream));
}

int kvc_dynamic_scaled_fp8_quant(void* out, const void* input, float* scale, int64_t num_elems, int in_dtype,
                                 int fp8_dtype, void* stream) {
  if (num_elems < 0) return fail(KVC_ERR_INVALID_ARG, "fp8 quant: negative element count");
  if (num_elems == 0) return KVC_OK;
  if (int rc = check_quant_args(out, input, in_dtype, fp8_dtype)) return rc;
  if (!scale) return fail(KVC_ERR_INVALID_ARG, "fp8 quant: scale must be non-NULL");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int es = in_elem_size(in_dtype);
  const int vec = flat_vec(input, out, es);
  QuantParams p{};
  p.input = input;
  p.out = out;
  p.scale = scale;
  p.num_elems = num_elems;
  p.n_chunks = num_elems / vec;
  p.wide_loads = (static_cast<int64_t>(vec) * es) % 32 == 0 && aligned(input, 32);
  const cudaError_t e = KVC_QUANT_DISPATCH(in_dtype, fp8_dtype, vec, launch_absmax, p, scale, st);
  if (e != cudaSuccess) return fail(KVC_ERR_CUDA, std::string("absmax launch failed: ") + cudaGetErrorString(e));
  return static_quant_impl(out, input, scale, num_elems, in_dtype, fp8_dtype, st);
}

int kvc_dynamic_per_token_scaled_fp8_quant(void* out, const void* input, float* scales, const float* scale_ub,
                                           int64_t num_tokens, int64_t hidden_size, int in_dtype, int fp8_dtype,
                                           void* stream) {
  if (num_tokens < 0 || hidden_size < 0) return fail(KVC_ERR_INVALID_ARG, "fp8 quant: negative size");
  if (num_tokens == 0 || hidden_size == 0) return KVC_OK;
  if (int rc = check_quant_args(out, input, in_dtype, fp8_dtype)) return rc;
  if (!scales) return fail(KVC_ERR_INVALID_ARG, "fp8 quant: scales must be non-NULL");
  if (num_tokens > 0x7FFFFFFFll) return fail(KVC_ERR_INVALID_ARG, "fp8 quant: too many tokens for one call");
  const int es = in_elem_size(in_dtype);
  // every row start must keep the vector alignment: the width must divide hidden_size
  int vec = flat_vec(input, out, es);
  while (vec > 1 && hidden_size % vec) vec >>= 1;
  TokenQuantParams p{};
  p.input = input;
  p.out = out;
  p.scales = scales;
  p.scale_ub = scale_ub;
  p.hidden_size = hidden_size;
  p.n_chunks = hidden_size / vec;
  p.wide_loads = (static_cast<int64_t>(vec) * es) % 32 == 0 && aligned(input, 32) && (hidden_size * es) % 32 == 0;
  const cudaError_t e = KVC_QUANT_DISPATCH(in_dtype, fp8_dtype, vec, launch_per_token, p, num_tokens,
                                           static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess)
    return fail(KVC_ERR_CUDA, std::string("dynamic_per_token_scaled_fp8_quant launch failed: ") + cudaGetErrorString(e));
  return KVC_OK;
}

}  // extern "C"
