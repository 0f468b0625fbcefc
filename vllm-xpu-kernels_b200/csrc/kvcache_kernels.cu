// Paged KV-cache write kernels for NVIDIA B200 (sm_100a) and their C ABI.
//
// Two scatter operations, both pure HBM traffic (no contraction, no tensor cores):
//   flash layout   cache[block][offset][head][d]          (kvc_reshape_and_cache_flash)
//   paged layout   K cache[block][head][d/x][offset][x],
//                  V cache[block][head][d][offset]         (kvc_reshape_and_cache)
// Each token's key/value row goes to the cache slot named by slot_mapping; negative
// slots are skipped; in fp8 modes every element is divided by a per-tensor scale in
// IEEE fp32 and rounded to nearest even with saturation by the hardware cvt.
//
// The reference plugin's counterparts are csrc/cache.cpp:13-189 (device code) and
// :409-489 (host launchers); the per-element rule is
// csrc/quantization/fp8/quant_utils.h:62-78.
#include <cstdio>
#include <cstring>
#include <mutex>

#include "kvc_common.cuh"
#include "kvc_convert.cuh"

namespace kvc {

// ---------------------------------------------------------------------------------------------
// error plumbing (declared in kvc_common.cuh)
// ---------------------------------------------------------------------------------------------
static thread_local std::string g_last_error;

int fail(int code, const std::string& msg) {
  g_last_error = msg;
  return code;
}

// ---------------------------------------------------------------------------------------------
// flash layout
// ---------------------------------------------------------------------------------------------
struct FlashParams {
  const void* key;
  const void* value;
  void* key_cache;
  void* value_cache;
  const int64_t* slot_mapping;
  const float* k_scale;
  const float* v_scale;
  int64_t key_stride_t, key_stride_h, value_stride_t, value_stride_h;  // elements
  int64_t block_stride, page_stride, head_stride;                      // elements
  int64_t block_size;
  int bs_shift;
  bool linear_slots;         // block_stride == block_size * page_stride: address = slot * page_stride
  bool wide_loads;           // every source chunk address is 32-byte aligned
  bool wide_stores;          // every destination chunk address is 32-byte aligned
  uint32_t prefetch_ctas;  // CTAs that may prefetch before the dependency wait
  uint32_t n_items;          // tokens_in_launch * rows_per_token * chunks_per_row
  uint32_t items_per_token;  // rows_per_token * chunks_per_row
  uint32_t chunks_per_row;
  FastDiv div_items_per_token, div_chunks_per_row;
};

constexpr int kFlashThreads = 256;

// One thread moves VEC consecutive elements of one (token, row) of K and the same VEC
// elements of V: both loads are issued before the first store (64 bytes in flight per
// thread for bf16 -> fp8, VEC = 16; 32 registers, so 2048 threads per SM).  A "row" is one
// head, or the whole token when heads are contiguous on both sides (ONE_ROW; the host
// collapses that case).
template <typename Tin, int KV, int VEC, bool ONE_ROW>
__global__ void __launch_bounds__(kFlashThreads) flash_scatter_kernel(const FlashParams p) {
  constexpr int IN_B = VEC * (int)sizeof(Tin);
  constexpr int OUT_ES = (KV == KVC_KV_AUTO) ? (int)sizeof(Tin) : 1;
  constexpr int OUT_B = VEC * OUT_ES;

  const uint32_t item = blockIdx.x * kFlashThreads + threadIdx.x;
  if (item >= p.n_items) return;
  const uint32_t tok = p.div_items_per_token.div(item);
  const uint32_t rem = item - tok * p.items_per_token;
  uint32_t row = 0, chunk = rem;
  if constexpr (!ONE_ROW) {
    row = p.div_chunks_per_row.div(rem);
    chunk = rem - row * p.chunks_per_row;
  }
  const int64_t d0 = static_cast<int64_t>(chunk) * VEC;
  const Tin* ksrc = static_cast<const Tin*>(p.key) + tok * p.key_stride_t + d0;
  const Tin* vsrc = static_cast<const Tin*>(p.value) + tok * p.value_stride_t + d0;
  if constexpr (!ONE_ROW) {
    ksrc += row * p.key_stride_h;
    vsrc += row * p.value_stride_h;
  }
  if (blockIdx.x < p.prefetch_ctas && slot_hint(p.slot_mapping + tok) >= 0) {
    prefetch_l2(ksrc);
    prefetch_l2(vsrc);
  }
  pdl_prologue();

  const int64_t slot = __ldg(p.slot_mapping + tok);
  if (slot < 0) return;

  Chunk<IN_B> kin, vin;
  load_chunk(kin, ksrc, p.wide_loads);
  load_chunk(vin, vsrc, p.wide_loads);

  int64_t dst;
  if (p.linear_slots) {
    dst = slot * p.page_stride + d0;
  } else {
    int64_t blk, off;
    split_slot(slot, p.block_size, p.bs_shift, blk, off);
    dst = blk * p.block_stride + off * p.page_stride + d0;
  }
  if constexpr (!ONE_ROW) dst += row * p.head_stride;

  ScaleCtx ks{}, vs{};
  if constexpr (KV != KVC_KV_AUTO) {
    ks = make_scale_ctx<Tin, KV>(p.k_scale);
    vs = make_scale_ctx<Tin, KV>(p.v_scale);
  }
  Chunk<OUT_B> kout, vout;
  convert_chunk<Tin, KV, VEC>(kin, kout, ks);
  convert_chunk<Tin, KV, VEC>(vin, vout, vs);
  store_chunk(static_cast<char*>(p.key_cache) + dst * OUT_ES, kout, p.wide_stores);
  store_chunk(static_cast<char*>(p.value_cache) + dst * OUT_ES, vout, p.wide_stores);
}

// ---------------------------------------------------------------------------------------------
// paged layout
// ---------------------------------------------------------------------------------------------
struct PagedParams {
  const void* key;
  const void* value;
  void* key_cache;
  void* value_cache;
  const int64_t* slot_mapping;
  const float* k_scale;
  const float* v_scale;
  int64_t key_stride_t, key_stride_h, value_stride_t, value_stride_h;  // elements
  int64_t num_tokens;
  int64_t block_size;
  int bs_shift;
  bool wide_loads;
  uint32_t prefetch_ctas;  // CTAs that may prefetch before the dependency wait
  int32_t num_heads, head_size, x;
  int32_t piece_bytes;  // K-store width: bytes of min(VEC, x)-element groups, <= 16
  uint32_t n_warps;     // token_groups * num_heads * chunks_per_row
  uint32_t chunks_per_row;
  FastDiv div_chunks_per_row, div_heads;
};

constexpr int kPagedThreads = 256;

// Lane = token.  A warp owns 32 consecutive tokens x one head x VEC consecutive d, so that
// every store instruction walks the token axis: when consecutive tokens occupy consecutive
// offsets of one block (a sequence being prefilled) the 32 lanes write one contiguous run
// (32 x-chunks of K, 32 elements of one V row) and whole sectors leave the SM.
// The 8 warps of a CTA take adjacent d-chunks of the same rows, so the CTA reads whole rows.
//
// With scattered slots (decode batches, random placement) no two tokens share a sector and the
// lane = token order is the worst one for V: each of a lane's VEC stores goes to a line of its own,
// 32 lines per instruction.  A warp that finds fewer than half of its tokens adjacent to their
// successor therefore writes V in the transposed order: an instruction covers 32 / VEC tokens x VEC
// consecutive d, i.e. per token one run of VEC sectors (bs elements apart in the cache, VEC * 32
// bytes for 16-bit caches with 16-slot blocks), four sectors to a line.  The elements still arrive by
// one wide load per lane (lane = token) and change hands through a 1 KB tile of shared memory per warp.
// K is written by the owner lane either way: its x-element groups are separate lines in both orders.
template <typename Tin, int KV, int VEC>
__global__ void __launch_bounds__(kPagedThreads, 5) paged_scatter_kernel(const PagedParams p) {
  constexpr int ES = (int)sizeof(Tin);
  constexpr int IN_B = VEC * ES;
  constexpr int OUT_ES = (KV == KVC_KV_AUTO) ? ES : 1;
  constexpr int OUT_B = VEC * OUT_ES;

  const uint32_t warp = blockIdx.x * (kPagedThreads / 32) + (threadIdx.x >> 5);
  if (warp >= p.n_warps) return;
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t th = p.div_chunks_per_row.div(warp);  // token_group * H + head
  const uint32_t chunk = warp - th * p.chunks_per_row;
  const uint32_t tg = p.div_heads.div(th);
  const uint32_t head = th - tg * static_cast<uint32_t>(p.num_heads);
  const int64_t tok0 = static_cast<int64_t>(tg) * 32;
  const int64_t tok = tok0 + lane;
  const bool in_range = tok < p.num_tokens;
  const int d0 = static_cast<int>(chunk) * VEC;
  const Tin* ksrc = static_cast<const Tin*>(p.key) + tok * p.key_stride_t + head * p.key_stride_h + d0;
  const Tin* vsrc = static_cast<const Tin*>(p.value) + tok * p.value_stride_t + head * p.value_stride_h + d0;
  if (blockIdx.x < p.prefetch_ctas && in_range && slot_hint(p.slot_mapping + tok) >= 0) {
    prefetch_l2(ksrc);
    prefetch_l2(vsrc);
  }
  pdl_prologue();

  const int64_t slot = in_range ? __ldg(p.slot_mapping + tok) : -1;
  bool transposed = false;
  if constexpr (VEC > 1) {
    const int64_t next = __shfl_down_sync(0xffffffffu, slot, 1);
    const bool adjacent = slot >= 0 && lane < 31u && next == slot + 1;
    transposed = __popc(__ballot_sync(0xffffffffu, adjacent)) < 16;
  }
  const bool active = slot >= 0;

  int64_t blk = 0, off = 0;
  if (active) split_slot(slot, p.block_size, p.bs_shift, blk, off);
  const int64_t bh = blk * p.num_heads + head;
  const int64_t bs = p.block_size;
  const int x = p.x;
  char* kc = static_cast<char*>(p.key_cache);
  char* vc = static_cast<char*>(p.value_cache);
  // K: element d lives at ((bh * (D/x) + d/x) * bs + off) * x + d%x.
  const int64_t kbase = bh * (p.head_size / x);
  // V: element d lives at (bh * D + d) * bs + off.
  const int64_t vbase = active ? (bh * p.head_size + d0) * bs + off : -1;

  ScaleCtx ks{}, vs{};
  if constexpr (KV != KVC_KV_AUTO) {
    ks = make_scale_ctx<Tin, KV>(p.k_scale);
    vs = make_scale_ctx<Tin, KV>(p.v_scale);
  }

  auto k_write = [&](const Chunk<OUT_B>& kout) {
    auto k_store = [&](auto piece_tag) {
      constexpr int PIECE = decltype(piece_tag)::value;  // bytes per store
      constexpr int PE = PIECE / OUT_ES;                 // elements per store
      if constexpr (PE >= 1 && PIECE <= OUT_B) {
#pragma unroll
        for (int j = 0; j < VEC; j += PE) {
          const int d = d0 + j;
          const int64_t idx = ((kbase + d / x) * bs + off) * x + d % x;
          store_piece<PIECE>(kc + idx * OUT_ES, kout, j * OUT_ES);
        }
      }
    };
    switch (p.piece_bytes) {
      case 16: k_store(std::integral_constant<int, 16>{}); break;
      case 8: k_store(std::integral_constant<int, 8>{}); break;
      case 4: k_store(std::integral_constant<int, 4>{}); break;
      case 2: k_store(std::integral_constant<int, 2>{}); break;
      default: k_store(std::integral_constant<int, 1>{}); break;
    }
  };

  if constexpr (VEC > 1) {
    if (transposed) {
      // Each lane fetches its own token's VEC elements with one wide load (the memory-level parallelism of the
      // other order), the warp's 32 x VEC tile goes through shared memory, and every store instruction then
      // covers 32 / VEC tokens x VEC consecutive d.
      constexpr int TPI = 32 / VEC;  // tokens per instruction
      __shared__ __align__(16) unsigned char v_tile[kPagedThreads / 32][32 * IN_B];
      unsigned char* tile = v_tile[threadIdx.x >> 5];
      if (active) {
        Chunk<IN_B> vin;
        load_chunk(vin, vsrc, p.wide_loads);
        *reinterpret_cast<Chunk<IN_B>*>(tile + lane * IN_B) = vin;
      }
      __syncwarp();
      const uint32_t sub = lane / VEC, e = lane % VEC;
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        const uint32_t owner = i * TPI + sub;
        const int64_t dst = __shfl_sync(0xffffffffu, vbase, owner);
        if (dst >= 0) {
          const Chunk<ES> raw = *reinterpret_cast<const Chunk<ES>*>(tile + owner * IN_B + e * ES);
          Chunk<OUT_ES> o;
          convert_chunk<Tin, KV, 1>(raw, o, vs);
          store_piece<OUT_ES>(vc + (dst + static_cast<int64_t>(e) * bs) * OUT_ES, o, 0);
        }
      }
      if (!active) return;
      Chunk<IN_B> kin;
      load_chunk(kin, ksrc, p.wide_loads);
      Chunk<OUT_B> kout;
      convert_chunk<Tin, KV, VEC>(kin, kout, ks);
      k_write(kout);
      return;
    }
  }
  if (!active) return;

  Chunk<IN_B> kin, vin;
  load_chunk(kin, ksrc, p.wide_loads);
  load_chunk(vin, vsrc, p.wide_loads);
  Chunk<OUT_B> kout, vout;
  convert_chunk<Tin, KV, VEC>(kin, kout, ks);
  convert_chunk<Tin, KV, VEC>(vin, vout, vs);
  k_write(kout);
#pragma unroll
  for (int j = 0; j < VEC; ++j) store_piece<OUT_ES>(vc + (vbase + j * bs) * OUT_ES, vout, j * OUT_ES);
}

// ---------------------------------------------------------------------------------------------
// MLA: concatenate kv_c [T, R] and k_pe [T, P] into cache[block][offset][R + P]
// ---------------------------------------------------------------------------------------------
struct MlaParams {
  const void* kv_c;
  const void* k_pe;
  void* kv_cache;
  const int64_t* slot_mapping;
  const float* scale;
  int64_t kv_c_stride, k_pe_stride, block_stride, entry_stride;  // elements
  int64_t block_size;
  int64_t num_tokens;
  int bs_shift;
  bool wide_loads, wide_stores;
  bool linear_slots;       // block_stride == block_size * entry_stride: address = slot * entry_stride
  uint32_t prefetch_ctas;  // CTAs that may prefetch before the dependency wait
  uint32_t n_items;        // ceil(T / kMlaTokensPerThread) * chunks_per_token
  uint32_t chunks_per_token;
  uint32_t chunks_kv_c;    // chunks that come from kv_c; the rest come from k_pe
  FastDiv div_chunks_per_token;
};

constexpr int kMlaThreads = 256;
constexpr int kMlaTokensPerThread = 2;

// One thread moves the same VEC-element chunk of kMlaTokensPerThread consecutive tokens'
// concatenated rows, so that many independent loads are in flight per thread and the scale set-up
// and index arithmetic are shared.  Chunks below chunks_kv_c read kv_c, the others k_pe; VEC
// divides both widths (the host picks it), so a chunk never straddles.
template <typename Tin, int KV, int VEC>
__global__ void __launch_bounds__(kMlaThreads) mla_scatter_kernel(const MlaParams p) {
  constexpr int IN_B = VEC * (int)sizeof(Tin);
  constexpr int OUT_ES = (KV == KVC_KV_AUTO) ? (int)sizeof(Tin) : 1;
  constexpr int OUT_B = VEC * OUT_ES;
  constexpr int N = kMlaTokensPerThread;

  const uint32_t item = blockIdx.x * kMlaThreads + threadIdx.x;
  if (item >= p.n_items) return;
  const uint32_t group = p.div_chunks_per_token.div(item);
  const uint32_t chunk = item - group * p.chunks_per_token;
  const int64_t t0 = static_cast<int64_t>(group) * N;
  const bool from_pe = chunk >= p.chunks_kv_c;
  const Tin* base = static_cast<const Tin*>(from_pe ? p.k_pe : p.kv_c);
  const int64_t stride = from_pe ? p.k_pe_stride : p.kv_c_stride;
  const Tin* src = base + t0 * stride + static_cast<int64_t>(from_pe ? chunk - p.chunks_kv_c : chunk) * VEC;
  if (blockIdx.x < p.prefetch_ctas) {
#pragma unroll
    for (int i = 0; i < N; ++i)
      if (t0 + i < p.num_tokens && slot_hint(p.slot_mapping + t0 + i) >= 0) prefetch_l2(src + i * stride);
  }
  pdl_prologue();

  int64_t slot[N];
#pragma unroll
  for (int i = 0; i < N; ++i) slot[i] = (t0 + i < p.num_tokens) ? __ldg(p.slot_mapping + t0 + i) : -1;

  Chunk<IN_B> in[N];
#pragma unroll
  for (int i = 0; i < N; ++i)
    if (slot[i] >= 0) load_chunk(in[i], src + i * stride, p.wide_loads);

  ScaleCtx sc{};
  if constexpr (KV != KVC_KV_AUTO) sc = make_scale_ctx<Tin, KV>(p.scale);
#pragma unroll
  for (int i = 0; i < N; ++i) {
    if (slot[i] < 0) continue;
    int64_t dst;
    if (p.linear_slots) {
      dst = slot[i] * p.entry_stride;
    } else {
      int64_t blk, off;
      split_slot(slot[i], p.block_size, p.bs_shift, blk, off);
      dst = blk * p.block_stride + off * p.entry_stride;
    }
    dst += static_cast<int64_t>(chunk) * VEC;
    Chunk<OUT_B> out;
    convert_chunk<Tin, KV, VEC>(in[i], out, sc);
    store_chunk(static_cast<char*>(p.kv_cache) + dst * OUT_ES, out, p.wide_stores);
  }
}

// ---------------------------------------------------------------------------------------------
// gather: dst[cu_seq_lens[b] + j] = cache[block_table[b][seq_starts[b]/bs + j/bs]][j % bs]
// ---------------------------------------------------------------------------------------------
struct GatherParams {
  const void* src_cache;
  void* dst;
  const int32_t* block_table;
  const int32_t* cu_seq_lens;
  const int32_t* seq_starts;  // may be null
  int64_t block_table_stride;
  int64_t cache_block_stride, cache_entry_stride, dst_entry_stride;  // BYTES
  int64_t num_rows;  // rows of dst
  int32_t batch_size;
  int32_t block_size;
  int bs_shift;
  uint32_t n_warps;  // ceil(num_rows / kGatherRowsPerWarp)
  uint32_t chunks_per_row;
  FastDiv div_block_size;
};

constexpr int kGatherThreads = 256;
constexpr int kGatherRowsPerWarp = 4;

// A warp copies kGatherRowsPerWarp consecutive destination rows.  Lanes 0..7 each locate one
// row's source entry (bisection over cu_seq_lens: batch_size + 1 ints, cache resident), all
// at once, so the search costs one pass per eight rows; the addresses are handed round with
// shuffles and every lane then copies BYTES-wide pieces lane, lane + 32, ... of each row, two
// rows at a time.  Rows at or beyond cu_seq_lens[batch_size] have no source and are left
// alone, so the grid can be sized from dst's row count, which the host knows, instead of
// from the token total, which lives on the device.
template <int BYTES>
__global__ void __launch_bounds__(kGatherThreads) gather_cache_kernel(const GatherParams p) {
  const uint32_t warp = blockIdx.x * (kGatherThreads / 32) + (threadIdx.x >> 5);
  if (warp >= p.n_warps) return;
  const uint32_t lane = threadIdx.x & 31u;
  const int64_t row0 = static_cast<int64_t>(warp) * kGatherRowsPerWarp;
  pdl_prologue();

  unsigned long long src_addr = 0;  // 0 = this row has no source
  if (lane < kGatherRowsPerWarp && row0 + lane < p.num_rows) {
    const int32_t r = static_cast<int32_t>(row0 + lane);
    if (r < __ldg(p.cu_seq_lens + p.batch_size)) {
      int lo = 0, hi = p.batch_size;  // invariant: cu[lo] <= r < cu[hi]
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (__ldg(p.cu_seq_lens + mid) <= r) lo = mid; else hi = mid;
      }
      const int32_t j = r - __ldg(p.cu_seq_lens + lo);
      if (j >= 0) {  // negative only if cu_seq_lens does not start at <= r: nothing sensible to copy
        const uint32_t jb = p.bs_shift >= 0 ? (static_cast<uint32_t>(j) >> p.bs_shift) : p.div_block_size.div(j);
        const uint32_t off = static_cast<uint32_t>(j) - jb * static_cast<uint32_t>(p.block_size);
        int32_t first = 0;
        if (p.seq_starts != nullptr) first = __ldg(p.seq_starts + lo) / p.block_size;
        const int64_t block = __ldg(p.block_table + lo * p.block_table_stride + first + jb);
        src_addr = reinterpret_cast<unsigned long long>(static_cast<const char*>(p.src_cache) +
                                                        block * p.cache_block_stride +
                                                        static_cast<int64_t>(off) * p.cache_entry_stride);
      }
    }
  }

  char* drow = static_cast<char*>(p.dst) + row0 * p.dst_entry_stride;
#pragma unroll
  for (int k = 0; k < kGatherRowsPerWarp; k += 2) {
    const char* s0 = reinterpret_cast<const char*>(__shfl_sync(0xFFFFFFFFu, src_addr, k));
    const char* s1 = reinterpret_cast<const char*>(__shfl_sync(0xFFFFFFFFu, src_addr, k + 1));
    char* d0 = drow + k * p.dst_entry_stride;
    char* d1 = d0 + p.dst_entry_stride;
    // three pieces of each of the two rows per pass: up to six loads in flight per lane
    for (uint32_t c0 = lane; c0 < p.chunks_per_row; c0 += 96) {
      Chunk<BYTES> x0[3], x1[3];
#pragma unroll
      for (int u = 0; u < 3; ++u) {
        const uint32_t c = c0 + 32 * u;
        if (c < p.chunks_per_row) {
          const int64_t at = static_cast<int64_t>(c) * BYTES;
          if (s0) load_chunk(x0[u], s0 + at, false);
          if (s1) load_chunk(x1[u], s1 + at, false);
        }
      }
#pragma unroll
      for (int u = 0; u < 3; ++u) {
        const uint32_t c = c0 + 32 * u;
        if (c < p.chunks_per_row) {
          const int64_t at = static_cast<int64_t>(c) * BYTES;
          if (s0) store_chunk(d0 + at, x0[u], false);
          if (s1) store_chunk(d1 + at, x1[u], false);
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// debug: count out-of-range slots
// ---------------------------------------------------------------------------------------------
__global__ void count_bad_slots_kernel(const int64_t* __restrict__ slots, int64_t n, int64_t num_slots,
                                       unsigned long long* __restrict__ bad) {
  unsigned long long local = 0;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    local += (slots[i] >= num_slots) ? 1ull : 0ull;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xFFFFFFFFu, local, o);
  if ((threadIdx.x & 31) == 0 && local) atomicAdd(bad, local);
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
template <typename Tin, int KV, bool ONE_ROW>
static cudaError_t launch_flash_vec2(int vec, const FlashParams& p, dim3 grid, cudaStream_t st) {
  switch (vec) {
    case 16: return launch_pdl(flash_scatter_kernel<Tin, KV, 16, ONE_ROW>, grid, kFlashThreads, p, st);
    case 8: return launch_pdl(flash_scatter_kernel<Tin, KV, 8, ONE_ROW>, grid, kFlashThreads, p, st);
    case 4: return launch_pdl(flash_scatter_kernel<Tin, KV, 4, ONE_ROW>, grid, kFlashThreads, p, st);
    case 2: return launch_pdl(flash_scatter_kernel<Tin, KV, 2, ONE_ROW>, grid, kFlashThreads, p, st);
    default: return launch_pdl(flash_scatter_kernel<Tin, KV, 1, ONE_ROW>, grid, kFlashThreads, p, st);
  }
}

template <typename Tin, int KV>
static cudaError_t launch_flash_vec(int vec, bool one_row, const FlashParams& p, dim3 grid, cudaStream_t st) {
  return one_row ? launch_flash_vec2<Tin, KV, true>(vec, p, grid, st)
                 : launch_flash_vec2<Tin, KV, false>(vec, p, grid, st);
}

template <typename Tin, int KV>
static cudaError_t launch_paged_vec(int vec, const PagedParams& p, dim3 grid, cudaStream_t st) {
  switch (vec) {
    case 16: return launch_pdl(paged_scatter_kernel<Tin, KV, 16>, grid, kPagedThreads, p, st);
    case 8: return launch_pdl(paged_scatter_kernel<Tin, KV, 8>, grid, kPagedThreads, p, st);
    case 4: return launch_pdl(paged_scatter_kernel<Tin, KV, 4>, grid, kPagedThreads, p, st);
    case 2: return launch_pdl(paged_scatter_kernel<Tin, KV, 2>, grid, kPagedThreads, p, st);
    default: return launch_pdl(paged_scatter_kernel<Tin, KV, 1>, grid, kPagedThreads, p, st);
  }
}

// (input dtype) x (cache mode) -> template instance; the build's counterpart of the
// reference's DISPATCH_BY_KV_CACHE_DTYPE (csrc/quantization/fp8/quant_utils.h:136-173).
#define KVC_DISPATCH(IN_DTYPE, KV_DTYPE, FN, ...)                                     \
  [&]() -> cudaError_t {                                                              \
    switch ((IN_DTYPE) * 3 + (KV_DTYPE)) {                                            \
      case KVC_IN_F32 * 3 + KVC_KV_AUTO: return FN<float, KVC_KV_AUTO>(__VA_ARGS__);  \
      case KVC_IN_F32 * 3 + KVC_KV_FP8_E4M3: return FN<float, KVC_KV_FP8_E4M3>(__VA_ARGS__); \
      case KVC_IN_F32 * 3 + KVC_KV_FP8_E5M2: return FN<float, KVC_KV_FP8_E5M2>(__VA_ARGS__); \
      case KVC_IN_F16 * 3 + KVC_KV_AUTO: return FN<__half, KVC_KV_AUTO>(__VA_ARGS__); \
      case KVC_IN_F16 * 3 + KVC_KV_FP8_E4M3: return FN<__half, KVC_KV_FP8_E4M3>(__VA_ARGS__); \
      case KVC_IN_F16 * 3 + KVC_KV_FP8_E5M2: return FN<__half, KVC_KV_FP8_E5M2>(__VA_ARGS__); \
      case KVC_IN_BF16 * 3 + KVC_KV_AUTO: return FN<__nv_bfloat16, KVC_KV_AUTO>(__VA_ARGS__); \
      case KVC_IN_BF16 * 3 + KVC_KV_FP8_E4M3: return FN<__nv_bfloat16, KVC_KV_FP8_E4M3>(__VA_ARGS__); \
      default: return FN<__nv_bfloat16, KVC_KV_FP8_E5M2>(__VA_ARGS__);                \
    }                                                                                 \
  }()

static int check_common(const void* key, const void* value, void* key_cache, void* value_cache,
                        const int64_t* slot_mapping, int64_t num_tokens, int64_t num_heads,
                        int64_t head_size, int64_t block_size, int in_dtype, int kv_dtype,
                        const float* k_scale, const float* v_scale) {
  if (in_dtype != KVC_IN_F32 && in_dtype != KVC_IN_F16 && in_dtype != KVC_IN_BF16)
    return fail(KVC_ERR_UNSUPPORTED, "Unsupported input type of kv cache: code " + std::to_string(in_dtype));
  if (kv_dtype != KVC_KV_AUTO && kv_dtype != KVC_KV_FP8_E4M3 && kv_dtype != KVC_KV_FP8_E5M2)
    return fail(KVC_ERR_UNSUPPORTED, "Unsupported data type of kv cache: code " + std::to_string(kv_dtype));
  if (num_tokens < 0 || num_heads < 0 || head_size < 0)
    return fail(KVC_ERR_INVALID_ARG, "num_tokens, num_heads and head_size must be non-negative");
  if (block_size <= 0) return fail(KVC_ERR_INVALID_ARG, "block_size must be positive");
  if (num_tokens == 0 || num_heads == 0 || head_size == 0) return KVC_OK;
  if (!key || !value || !key_cache || !value_cache || !slot_mapping)
    return fail(KVC_ERR_INVALID_ARG, "key, value, key_cache, value_cache and slot_mapping must be non-NULL");
  if (kv_dtype != KVC_KV_AUTO && (!k_scale || !v_scale))
    return fail(KVC_ERR_INVALID_ARG, "k_scale and v_scale must be non-NULL for an fp8 cache");
  if (!aligned(slot_mapping, 8)) return fail(KVC_ERR_INVALID_ARG, "slot_mapping must be 8-byte aligned");
  const int es = in_elem_size(in_dtype);
  if (!aligned(key, es) || !aligned(value, es))
    return fail(KVC_ERR_INVALID_ARG, "key/value are not aligned to their element size");
  if (kv_dtype == KVC_KV_AUTO && (!aligned(key_cache, es) || !aligned(value_cache, es)))
    return fail(KVC_ERR_INVALID_ARG, "caches are not aligned to their element size");
  if (num_heads > 0x7FFFFFFFll || head_size > 0x7FFFFFFFll)
    return fail(KVC_ERR_INVALID_ARG, "num_heads / head_size out of range");
  return KVC_OK;
}

// Largest power-of-two element count (<= cap) such that chunks of that many elements of
// size `es` starting at `p` and displaced by any of `strides` stay aligned to
// min(16, count*es) bytes, and that divides `len`.
static int pick_vec(int cap, int64_t len, int es, const void* const* ptrs, int nptrs,
                    const int64_t* strides, int nstrides) {
  for (int v = cap; v > 1; v >>= 1) {
    if (len % v) continue;
    const int64_t a = (static_cast<int64_t>(v) * es >= 16) ? 16 : static_cast<int64_t>(v) * es;
    bool ok = true;
    for (int i = 0; i < nptrs && ok; ++i) ok = aligned(ptrs[i], a);
    for (int i = 0; i < nstrides && ok; ++i) ok = ((strides[i] * es) % a) == 0;
    if (ok) return v;
  }
  return 1;
}

static int flash_impl(const void* key, const void* value, void* key_cache, void* value_cache,
                      const int64_t* slot_mapping, int64_t num_tokens, int64_t num_heads, int64_t head_size,
                      int64_t block_size, int64_t key_stride_t, int64_t key_stride_h, int64_t value_stride_t,
                      int64_t value_stride_h, int64_t block_stride, int64_t page_stride, int64_t head_stride,
                      int in_dtype, int kv_dtype, const float* k_scale, const float* v_scale,
                      cudaStream_t st) {
  if (int rc = check_common(key, value, key_cache, value_cache, slot_mapping, num_tokens, num_heads,
                            head_size, block_size, in_dtype, kv_dtype, k_scale, v_scale))
    return rc;
  if (num_tokens == 0 || num_heads == 0 || head_size == 0) return KVC_OK;

  // Heads contiguous on both sides: one row per token.
  int64_t rows = num_heads, row_len = head_size;
  if (num_heads == 1 || (key_stride_h == head_size && value_stride_h == head_size && head_stride == head_size)) {
    rows = 1;
    row_len = num_heads * head_size;
  }
  const int es_in = in_elem_size(in_dtype);
  const int es_out = (kv_dtype == KVC_KV_AUTO) ? es_in : 1;

  // Vector width: bounded by source alignment and by destination alignment.
  const void* in_ptrs[2] = {key, value};
  const int64_t in_strides[4] = {key_stride_t, value_stride_t, rows > 1 ? key_stride_h : 0,
                                 rows > 1 ? value_stride_h : 0};
  const void* out_ptrs[2] = {key_cache, value_cache};
  const int64_t out_strides[3] = {block_stride, page_stride, rows > 1 ? head_stride : 0};
  int vec = pick_vec(16, row_len, es_in, in_ptrs, 2, in_strides, 4);
  vec = pick_vec(vec, row_len, es_out, out_ptrs, 2, out_strides, 3);

  // 256-bit loads need every chunk address on a 32-byte boundary
  bool wide = (static_cast<int64_t>(vec) * es_in) % 32 == 0 && aligned(key, 32) && aligned(value, 32);
  for (int i = 0; i < 4 && wide; ++i) wide = ((in_strides[i] * es_in) % 32) == 0;

  bool wide_st = (static_cast<int64_t>(vec) * es_out) % 32 == 0 && aligned(key_cache, 32) && aligned(value_cache, 32);
  for (int i = 0; i < 3 && wide_st; ++i) wide_st = ((out_strides[i] * es_out) % 32) == 0;

  const int64_t chunks_per_row = row_len / vec;
  const int64_t items_per_token = rows * chunks_per_row;
  if (items_per_token >= (1ll << 30)) return fail(KVC_ERR_INVALID_ARG, "num_heads * head_size too large");

  FlashParams p{};
  p.key_cache = key_cache;
  p.value_cache = value_cache;
  p.k_scale = k_scale;
  p.v_scale = v_scale;
  p.key_stride_t = key_stride_t;
  p.key_stride_h = key_stride_h;
  p.value_stride_t = value_stride_t;
  p.value_stride_h = value_stride_h;
  p.block_stride = block_stride;
  p.page_stride = page_stride;
  p.head_stride = head_stride;
  p.block_size = block_size;
  p.bs_shift = pow2_shift(block_size);
  p.linear_slots = (block_stride == block_size * page_stride);
  p.wide_loads = wide;
  p.wide_stores = wide_st;
  p.items_per_token = static_cast<uint32_t>(items_per_token);
  p.chunks_per_row = static_cast<uint32_t>(chunks_per_row);
  p.div_items_per_token = FastDiv(p.items_per_token);
  p.div_chunks_per_row = FastDiv(p.chunks_per_row);

  // Item indices are 31-bit: very large batches go out as several launches.  The limit can be
  // lowered through KVC_TEST_MAX_ITEMS_PER_LAUNCH so that tests reach the splitting code.
  static const int64_t item_limit = [] {
    const char* e = getenv("KVC_TEST_MAX_ITEMS_PER_LAUNCH");
    const int64_t v = e ? strtoll(e, nullptr, 10) : 0;
    return (v > 0 && v < (1ll << 31) - kFlashThreads) ? v : (1ll << 31) - kFlashThreads;
  }();
  int64_t max_tokens_per_launch = item_limit / items_per_token;
  if (max_tokens_per_launch < 1) max_tokens_per_launch = 1;
  for (int64_t t0 = 0; t0 < num_tokens; t0 += max_tokens_per_launch) {
    const int64_t nt = (num_tokens - t0 < max_tokens_per_launch) ? num_tokens - t0 : max_tokens_per_launch;
    p.key = static_cast<const char*>(key) + t0 * key_stride_t * es_in;
    p.value = static_cast<const char*>(value) + t0 * value_stride_t * es_in;
    p.slot_mapping = slot_mapping + t0;
    p.n_items = static_cast<uint32_t>(nt * items_per_token);
    const dim3 grid(static_cast<unsigned>((p.n_items + kFlashThreads - 1) / kFlashThreads));
    p.prefetch_ctas = prefetch_cta_count(grid.x);
    const cudaError_t e = KVC_DISPATCH(in_dtype, kv_dtype, launch_flash_vec, vec, rows == 1, p, grid, st);
    if (e != cudaSuccess)
      return fail(KVC_ERR_CUDA, std::string("reshape_and_cache_flash launch failed: ") + cudaGetErrorString(e));
  }
  return KVC_OK;
}

static int paged_impl(const void* key, const void* value, void* key_cache, void* value_cache,
                      const int64_t* slot_mapping, int64_t num_tokens, int64_t num_heads, int64_t head_size,
                      int64_t block_size, int64_t x, int64_t key_stride_t, int64_t key_stride_h,
                      int64_t value_stride_t, int64_t value_stride_h, int in_dtype, int kv_dtype,
                      const float* k_scale, const float* v_scale, cudaStream_t st) {
  if (int rc = check_common(key, value, key_cache, value_cache, slot_mapping, num_tokens, num_heads,
                            head_size, block_size, in_dtype, kv_dtype, k_scale, v_scale))
    return rc;
  if (x <= 0 || x > 0x7FFFFFFFll) return fail(KVC_ERR_INVALID_ARG, "x must be positive");
  if (head_size % x) return fail(KVC_ERR_INVALID_ARG, "head_size must be a multiple of x (key_cache.size(4))");
  if (num_tokens == 0 || num_heads == 0 || head_size == 0) return KVC_OK;

  const int es_in = in_elem_size(in_dtype);
  const int es_out = (kv_dtype == KVC_KV_AUTO) ? es_in : 1;
  const void* in_ptrs[2] = {key, value};
  const int64_t in_strides[4] = {key_stride_t, value_stride_t, key_stride_h, value_stride_h};
  // a lane reads at most 32 bytes (one sector) of K and of V
  const int vec = pick_vec(32 / es_in, head_size, es_in, in_ptrs, 2, in_strides, 4);

  bool wide = (static_cast<int64_t>(vec) * es_in) % 32 == 0 && aligned(key, 32) && aligned(value, 32);
  for (int i = 0; i < 4 && wide; ++i) wide = ((in_strides[i] * es_in) % 32) == 0;

  // K-store width: groups of min(vec, x) elements when x is a power of two and the cache
  // base is aligned for it; single elements otherwise.
  int64_t pe = 1;
  while (pe * 2 <= vec && x % (pe * 2) == 0 && pe * 2 * es_out <= 16) pe *= 2;
  while (pe > 1 && !aligned(key_cache, pe * es_out)) pe >>= 1;

  const int64_t chunks_per_row = head_size / vec;
  const int64_t token_groups = (num_tokens + 31) / 32;
  const int64_t n_warps = token_groups * num_heads * chunks_per_row;
  if (n_warps >= (1ll << 31)) return fail(KVC_ERR_INVALID_ARG, "num_tokens * num_heads * head_size too large for one call");

  PagedParams p{};
  p.key = key;
  p.value = value;
  p.key_cache = key_cache;
  p.value_cache = value_cache;
  p.slot_mapping = slot_mapping;
  p.k_scale = k_scale;
  p.v_scale = v_scale;
  p.key_stride_t = key_stride_t;
  p.key_stride_h = key_stride_h;
  p.value_stride_t = value_stride_t;
  p.value_stride_h = value_stride_h;
  p.num_tokens = num_tokens;
  p.block_size = block_size;
  p.bs_shift = pow2_shift(block_size);
  p.wide_loads = wide;
  p.num_heads = static_cast<int32_t>(num_heads);
  p.head_size = static_cast<int32_t>(head_size);
  p.x = static_cast<int32_t>(x);
  p.piece_bytes = static_cast<int32_t>(pe * es_out);
  p.n_warps = static_cast<uint32_t>(n_warps);
  p.chunks_per_row = static_cast<uint32_t>(chunks_per_row);
  p.div_chunks_per_row = FastDiv(p.chunks_per_row);
  p.div_heads = FastDiv(static_cast<uint32_t>(num_heads));
  constexpr int wpb = kPagedThreads / 32;
  const dim3 grid(static_cast<unsigned>((n_warps + wpb - 1) / wpb));
  p.prefetch_ctas = prefetch_cta_count(grid.x);
  const cudaError_t e = KVC_DISPATCH(in_dtype, kv_dtype, launch_paged_vec, vec, p, grid, st);
  if (e != cudaSuccess)
    return fail(KVC_ERR_CUDA, std::string("reshape_and_cache launch failed: ") + cudaGetErrorString(e));
  return KVC_OK;
}

template <typename Tin, int KV>
static cudaError_t launch_mla_vec(int vec, const MlaParams& p, dim3 grid, cudaStream_t st) {
  switch (vec) {
    case 16: return launch_pdl(mla_scatter_kernel<Tin, KV, 16>, grid, kMlaThreads, p, st);
    case 8: return launch_pdl(mla_scatter_kernel<Tin, KV, 8>, grid, kMlaThreads, p, st);
    case 4: return launch_pdl(mla_scatter_kernel<Tin, KV, 4>, grid, kMlaThreads, p, st);
    case 2: return launch_pdl(mla_scatter_kernel<Tin, KV, 2>, grid, kMlaThreads, p, st);
    default: return launch_pdl(mla_scatter_kernel<Tin, KV, 1>, grid, kMlaThreads, p, st);
  }
}

static int mla_impl(const void* kv_c, const void* k_pe, void* kv_cache, const int64_t* slot_mapping,
                    int64_t num_tokens, int64_t kv_lora_rank, int64_t pe_dim, int64_t block_size,
                    int64_t kv_c_stride, int64_t k_pe_stride, int64_t block_stride, int64_t entry_stride,
                    int in_dtype, int kv_dtype, const float* scale, cudaStream_t st) {
  // an empty half (width 0) may come with a NULL pointer: it is never dereferenced
  if (kv_lora_rank == 0 && kv_c == nullptr) kv_c = k_pe;
  if (pe_dim == 0 && k_pe == nullptr) k_pe = kv_c;
  // shares the argument rules of the K/V ops: kv_c plays key, k_pe plays value
  if (int rc = check_common(kv_c, k_pe, kv_cache, kv_cache, slot_mapping, num_tokens, 1, kv_lora_rank + pe_dim,
                            block_size, in_dtype, kv_dtype, scale, scale))
    return rc;
  if (kv_lora_rank < 0 || pe_dim < 0) return fail(KVC_ERR_INVALID_ARG, "kv_lora_rank and pe_dim must be non-negative");
  if (num_tokens == 0 || kv_lora_rank + pe_dim == 0) return KVC_OK;
  const int es_in = in_elem_size(in_dtype);
  const int es_out = (kv_dtype == KVC_KV_AUTO) ? es_in : 1;

  // one vector width for both sources: it must divide both widths and suit every base and stride
  const void* in_ptrs[2] = {kv_c, k_pe};
  const int64_t in_strides[2] = {kv_c_stride, k_pe_stride};
  const void* out_ptrs[1] = {kv_cache};
  const int64_t out_strides[3] = {block_stride, entry_stride, kv_lora_rank};
  int vec = 16;
  if (kv_lora_rank > 0) vec = pick_vec(vec, kv_lora_rank, es_in, in_ptrs, 1, in_strides, 1);
  if (pe_dim > 0) vec = pick_vec(vec, pe_dim, es_in, in_ptrs + 1, 1, in_strides + 1, 1);
  vec = pick_vec(vec, kv_lora_rank > 0 ? kv_lora_rank : pe_dim, es_out, out_ptrs, 1, out_strides, 3);
  if (pe_dim > 0 && pe_dim % vec) vec = pick_vec(vec, pe_dim, es_out, out_ptrs, 1, out_strides, 3);
  bool wide = (static_cast<int64_t>(vec) * es_in) % 32 == 0 && aligned(kv_c, 32) && aligned(k_pe, 32) &&
              (kv_c_stride * es_in) % 32 == 0 && (k_pe_stride * es_in) % 32 == 0;
  bool wide_st = (static_cast<int64_t>(vec) * es_out) % 32 == 0 && aligned(kv_cache, 32);
  for (int i = 0; i < 3 && wide_st; ++i) wide_st = ((out_strides[i] * es_out) % 32) == 0;

  const int64_t chunks = (kv_lora_rank + pe_dim) / vec;
  const int64_t pairs = (num_tokens + kMlaTokensPerThread - 1) / kMlaTokensPerThread;  // token groups
  if (chunks >= (1ll << 30) || pairs * chunks >= (1ll << 31) - kMlaThreads)
    return fail(KVC_ERR_INVALID_ARG, "num_tokens * (kv_lora_rank + pe_dim) too large for one call");

  MlaParams p{};
  p.kv_c = kv_c;
  p.k_pe = k_pe;
  p.kv_cache = kv_cache;
  p.slot_mapping = slot_mapping;
  p.scale = scale;
  p.kv_c_stride = kv_c_stride;
  p.k_pe_stride = k_pe_stride;
  p.block_stride = block_stride;
  p.entry_stride = entry_stride;
  p.block_size = block_size;
  p.num_tokens = num_tokens;
  p.bs_shift = pow2_shift(block_size);
  p.wide_loads = wide;
  p.wide_stores = wide_st;
  p.linear_slots = (block_stride == block_size * entry_stride);
  p.n_items = static_cast<uint32_t>(pairs * chunks);
  p.chunks_per_token = static_cast<uint32_t>(chunks);
  p.chunks_kv_c = static_cast<uint32_t>(kv_lora_rank / vec);
  p.div_chunks_per_token = FastDiv(p.chunks_per_token);
  const dim3 grid((p.n_items + kMlaThreads - 1) / kMlaThreads);
  p.prefetch_ctas = prefetch_cta_count(grid.x);
  const cudaError_t e = KVC_DISPATCH(in_dtype, kv_dtype, launch_mla_vec, vec, p, grid, st);
  if (e != cudaSuccess)
    return fail(KVC_ERR_CUDA, std::string("concat_and_cache_mla launch failed: ") + cudaGetErrorString(e));
  return KVC_OK;
}

static int gather_impl(const void* src_cache, void* dst, const int32_t* block_table, const int32_t* cu_seq_lens,
                       const int32_t* seq_starts, int64_t batch_size, int64_t num_dst_rows, int64_t block_size,
                       int64_t entry_size, int64_t elem_size, int64_t block_table_stride,
                       int64_t cache_block_stride, int64_t cache_entry_stride, int64_t dst_entry_stride,
                       cudaStream_t st) {
  if (elem_size != 1 && elem_size != 2 && elem_size != 4)
    return fail(KVC_ERR_UNSUPPORTED, "Unsupported data type width: " + std::to_string(elem_size * 8));
  if (batch_size < 0 || num_dst_rows < 0 || entry_size < 0 || batch_size > 0x7FFFFFFFll)
    return fail(KVC_ERR_INVALID_ARG, "gather_cache: negative or oversized batch_size / rows / entry_size");
  if (block_size <= 0 || block_size > 0x7FFFFFFFll) return fail(KVC_ERR_INVALID_ARG, "block_size must be positive");
  if (batch_size == 0 || num_dst_rows == 0 || entry_size == 0) return KVC_OK;
  if (!src_cache || !dst || !block_table || !cu_seq_lens)
    return fail(KVC_ERR_INVALID_ARG, "src_cache, dst, block_table and cu_seq_lens must be non-NULL");
  if (num_dst_rows > 0x7FFFFFFFll) return fail(KVC_ERR_INVALID_ARG, "dst has too many rows (cu_seq_lens is int32)");

  const int64_t row_bytes = entry_size * elem_size;
  const void* ptrs[2] = {src_cache, dst};
  const int64_t strides[3] = {cache_block_stride * elem_size, cache_entry_stride * elem_size,
                              dst_entry_stride * elem_size};
  const int piece = pick_vec(16, row_bytes, 1, ptrs, 2, strides, 3);  // bytes per thread, power of two <= 16
  const int64_t chunks = row_bytes / piece;
  const int64_t n_warps = (num_dst_rows + kGatherRowsPerWarp - 1) / kGatherRowsPerWarp;
  if (chunks >= (1ll << 31)) return fail(KVC_ERR_INVALID_ARG, "gather_cache: entries too large");

  GatherParams p{};
  p.src_cache = src_cache;
  p.dst = dst;
  p.block_table = block_table;
  p.cu_seq_lens = cu_seq_lens;
  p.seq_starts = seq_starts;
  p.block_table_stride = block_table_stride;
  p.cache_block_stride = cache_block_stride * elem_size;
  p.cache_entry_stride = cache_entry_stride * elem_size;
  p.dst_entry_stride = dst_entry_stride * elem_size;
  p.batch_size = static_cast<int32_t>(batch_size);
  p.block_size = static_cast<int32_t>(block_size);
  p.bs_shift = pow2_shift(block_size);
  p.num_rows = num_dst_rows;
  p.n_warps = static_cast<uint32_t>(n_warps);
  p.chunks_per_row = static_cast<uint32_t>(chunks);
  p.div_block_size = FastDiv(static_cast<uint32_t>(block_size));
  constexpr int wpb = kGatherThreads / 32;
  const dim3 grid(static_cast<unsigned>((n_warps + wpb - 1) / wpb));
  cudaError_t e;
  switch (piece) {
    case 16: e = launch_pdl(gather_cache_kernel<16>, grid, kGatherThreads, p, st); break;
    case 8: e = launch_pdl(gather_cache_kernel<8>, grid, kGatherThreads, p, st); break;
    case 4: e = launch_pdl(gather_cache_kernel<4>, grid, kGatherThreads, p, st); break;
    case 2: e = launch_pdl(gather_cache_kernel<2>, grid, kGatherThreads, p, st); break;
    default: e = launch_pdl(gather_cache_kernel<1>, grid, kGatherThreads, p, st); break;
  }
  if (e != cudaSuccess) return fail(KVC_ERR_CUDA, std::string("gather_cache launch failed: ") + cudaGetErrorString(e));
  return KVC_OK;
}

// ---------------------------------------------------------------------------------------------
// device staging for host-resident inputs (one set per device, grown on demand)
// ---------------------------------------------------------------------------------------------
struct Staging {
  void* buf = nullptr;
  size_t cap = 0;
};
constexpr int kMaxDevices = 64;
static Staging g_staging[kMaxDevices];
static std::mutex g_staging_mu;

static int staging_reserve(int dev, size_t bytes, void** out) {
  std::lock_guard<std::mutex> lk(g_staging_mu);
  Staging& s = g_staging[dev];
  if (s.cap < bytes) {
    if (s.buf) {
      KVC_CUDA_TRY(cudaDeviceSynchronize());  // earlier calls may still read the old buffer
      KVC_CUDA_TRY(cudaFree(s.buf));
      s.buf = nullptr;
      s.cap = 0;
    }
    KVC_CUDA_TRY(cudaMalloc(&s.buf, bytes));
    s.cap = bytes;
  }
  *out = s.buf;
  return KVC_OK;
}

static size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// ---------------------------------------------------------------------------------------------
// fixed staging for kvc_reshape_and_cache_flash_host_noalloc: lives in the module image, so
// every device that loads this library holds KVC_NOALLOC_STAGING_BYTES of it until exit.
// ---------------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_fixed_staging[KVC_NOALLOC_STAGING_BYTES];

// In host code `g_fixed_staging` is only a handle for the symbol, not an address a kernel or
// a copy may use; the per-device address comes from cudaGetSymbolAddress, asked once per
// device while that device is current.
static void* g_fixed_staging_addr[kMaxDevices];
static std::mutex g_fixed_staging_mu;

static int fixed_staging_address(int dev, void** out) {
  std::lock_guard<std::mutex> lk(g_fixed_staging_mu);
  if (g_fixed_staging_addr[dev] == nullptr) {
    void* ptr = nullptr;
    KVC_CUDA_TRY(cudaGetSymbolAddress((void**)&ptr, g_fixed_staging));
    if (ptr == nullptr) return fail(KVC_ERR_CUDA, "cudaGetSymbolAddress returned a null staging address");
    g_fixed_staging_addr[dev] = ptr;
  }
  *out = g_fixed_staging_addr[dev];
  return KVC_OK;
}

}  // namespace kvc

// ---------------------------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------------------------
using namespace kvc;

extern "C" {

int kvc_version(void) { return 100; }

const char* kvc_last_error(void) { return g_last_error.c_str(); }

int kvc_parse_kv_cache_dtype(const char* s, int* out) {
  if (!s || !out) return fail(KVC_ERR_INVALID_ARG, "kvc_parse_kv_cache_dtype: NULL argument");
  if (!std::strcmp(s, "auto")) {
    *out = KVC_KV_AUTO;
  } else if (!std::strcmp(s, "fp8") || !std::strcmp(s, "fp8_e4m3")) {
    *out = KVC_KV_FP8_E4M3;
  } else if (!std::strcmp(s, "fp8_e5m2")) {
    *out = KVC_KV_FP8_E5M2;
  } else {
    return fail(KVC_ERR_UNSUPPORTED, std::string("Unsupported data type of kv cache: ") + s);
  }
  return KVC_OK;
}

int kvc_reshape_and_cache_flash(const void* key, const void* value, void* key_cache, void* value_cache,
                                const int64_t* slot_mapping, int64_t num_tokens, int64_t num_heads,
                                int64_t head_size, int64_t block_size, int64_t key_stride_t,
                                int64_t key_stride_h, int64_t value_stride_t, int64_t value_stride_h,
                                int64_t block_stride, int64_t page_stride, int64_t head_stride, int in_dtype,
                                int kv_dtype, const float* k_scale, const float* v_scale, void* stream) {
  return flash_impl(key, value, key_cache, value_cache, slot_mapping, num_tokens, num_heads, head_size,
                    block_size, key_stride_t, key_stride_h, value_stride_t, value_stride_h, block_stride,
                    page_stride, head_stride, in_dtype, kv_dtype, k_scale, v_scale,
                    static_cast<cudaStream_t>(stream));
}

int kvc_reshape_and_cache(const void* key, const void* value, void* key_cache, void* value_cache,
                          const int64_t* slot_mapping, int64_t num_tokens, int64_t num_heads,
                          int64_t head_size, int64_t block_size, int64_t x, int64_t key_stride_t,
                          int64_t key_stride_h, int64_t value_stride_t, int64_t value_stride_h, int in_dtype,
                          int kv_dtype, const float* k_scale, const float* v_scale, void* stream) {
  return paged_impl(key, value, key_cache, value_cache, slot_mapping, num_tokens, num_heads, head_size,
                    block_size, x, key_stride_t, key_stride_h, value_stride_t, value_stride_h, in_dtype,
                    kv_dtype, k_scale, v_scale, static_cast<cudaStream_t>(stream));
}

int kvc_concat_and_cache_mla(const void* kv_c, const void* k_pe, void* kv_cache, const int64_t* slot_mapping,
                             int64_t num_tokens, int64_t kv_lora_rank, int64_t pe_dim, int64_t block_size,
                             int64_t kv_c_stride, int64_t k_pe_stride, int64_t block_stride, int64_t entry_stride,
                             int in_dtype, int kv_dtype, const float* scale, void* stream) {
  return mla_impl(kv_c, k_pe, kv_cache, slot_mapping, num_tokens, kv_lora_rank, pe_dim, block_size, kv_c_stride,
                  k_pe_stride, block_stride, entry_stride, in_dtype, kv_dtype, scale,
                  static_cast<cudaStream_t>(stream));
}

int kvc_gather_cache(const void* src_cache, void* dst, const int32_t* block_table, const int32_t* cu_seq_lens,
                     const int32_t* seq_starts, int64_t batch_size, int64_t num_dst_rows, int64_t block_size,
                     int64_t entry_size, int64_t elem_size, int64_t block_table_stride, int64_t cache_block_stride,
                     int64_t cache_entry_stride, int64_t dst_entry_stride, void* stream) {
  return gather_impl(src_cache, dst, block_table, cu_seq_lens, seq_starts, batch_size, num_dst_rows, block_size,
                     entry_size, elem_size, block_table_stride, cache_block_stride, cache_entry_stride,
                     dst_entry_stride, static_cast<cudaStream_t>(stream));
}

int kvc_reshape_and_cache_flash_host(const void* host_key, const void* host_value, void* key_cache,
                                     void* value_cache, const int64_t* host_slot_mapping, int64_t num_tokens,
                                     int64_t num_heads, int64_t head_size, int64_t block_size,
                                     int64_t key_stride_t, int64_t value_stride_t, int64_t block_stride,
                                     int64_t page_stride, int64_t head_stride, int in_dtype, int kv_dtype,
                                     const float* k_scale, const float* v_scale, void* stream) {
  if (int rc = check_common(host_key, host_value, key_cache, value_cache, host_slot_mapping, num_tokens,
                            num_heads, head_size, block_size, in_dtype, kv_dtype, k_scale, v_scale))
    return rc;
  if (num_tokens == 0 || num_heads == 0 || head_size == 0) return KVC_OK;
  const int64_t row = num_heads * head_size;
  if (key_stride_t < row || value_stride_t < row)
    return fail(KVC_ERR_INVALID_ARG, "host key/value token stride is smaller than num_heads*head_size");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int dev = 0;
  KVC_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(KVC_ERR_INVALID_ARG, "device ordinal out of range");
  const size_t es = static_cast<size_t>(in_elem_size(in_dtype));
  const size_t row_bytes = static_cast<size_t>(row) * es;
  const size_t kv_bytes = round_up(static_cast<size_t>(num_tokens) * row_bytes, 256);
  const size_t slot_bytes = round_up(static_cast<size_t>(num_tokens) * 8, 256);
  void* base = nullptr;
  if (int rc = staging_reserve(dev, 2 * kv_bytes + slot_bytes, &base)) return rc;
  char* dkey = static_cast<char*>(base);
  char* dval = dkey + kv_bytes;
  int64_t* dslots = reinterpret_cast<int64_t*>(dval + kv_bytes);
  // Rows are packed on the device whatever the host stride.
  const void* hsrc[2] = {host_key, host_value};
  char* ddst[2] = {dkey, dval};
  const int64_t hstride[2] = {key_stride_t, value_stride_t};
  for (int i = 0; i < 2; ++i) {
    if (hstride[i] == row) {
      KVC_CUDA_TRY(cudaMemcpyAsync(ddst[i], hsrc[i], static_cast<size_t>(num_tokens) * row_bytes,
                                   cudaMemcpyHostToDevice, st));
    } else {
      KVC_CUDA_TRY(cudaMemcpy2DAsync(ddst[i], row_bytes, hsrc[i], static_cast<size_t>(hstride[i]) * es, row_bytes,
                                     static_cast<size_t>(num_tokens), cudaMemcpyHostToDevice, st));
    }
  }
  KVC_CUDA_TRY(cudaMemcpyAsync(dslots, host_slot_mapping, static_cast<size_t>(num_tokens) * 8,
                               cudaMemcpyHostToDevice, st));
  return flash_impl(dkey, dval, key_cache, value_cache, dslots, num_tokens, num_heads, head_size, block_size,
                    row, head_size, row, head_size, block_stride, page_stride, head_stride, in_dtype, kv_dtype,
                    k_scale, v_scale, st);
}

int kvc_reshape_and_cache_flash_host_noalloc(const void* host_key, const void* host_value, void* key_cache,
                                             void* value_cache, const int64_t* host_slot_mapping,
                                             int64_t num_tokens, int64_t num_heads, int64_t head_size,
                                             int64_t block_size, int64_t key_stride_t, int64_t value_stride_t,
                                             int64_t block_stride, int64_t page_stride, int64_t head_stride,
                                             int in_dtype, int kv_dtype, const float* k_scale,
                                             const float* v_scale, void* stream) {
  if (int rc = check_common(host_key, host_value, key_cache, value_cache, host_slot_mapping, num_tokens,
                            num_heads, head_size, block_size, in_dtype, kv_dtype, k_scale, v_scale))
    return rc;
  if (num_tokens == 0 || num_heads == 0 || head_size == 0) return KVC_OK;
  const int64_t row = num_heads * head_size;
  if (key_stride_t < row || value_stride_t < row)
    return fail(KVC_ERR_INVALID_ARG, "host key/value token stride is smaller than num_heads*head_size");
  const size_t es = static_cast<size_t>(in_elem_size(in_dtype));
  const size_t row_bytes = static_cast<size_t>(row) * es;
  // capacity check first, in integers that cannot wrap
  const size_t cap = static_cast<size_t>(KVC_NOALLOC_STAGING_BYTES);
  if (row_bytes > cap || static_cast<size_t>(num_tokens) > cap / row_bytes)
    return fail(KVC_ERR_TOO_LARGE, "kvc_reshape_and_cache_flash_host_noalloc: batch does not fit the fixed staging area");
  const size_t kv_bytes = round_up(static_cast<size_t>(num_tokens) * row_bytes, 256);
  const size_t slot_bytes = round_up(static_cast<size_t>(num_tokens) * 8, 256);
  const size_t need = 2 * kv_bytes + slot_bytes;
  if (need > cap)
    return fail(KVC_ERR_TOO_LARGE,
                "kvc_reshape_and_cache_flash_host_noalloc: needs " + std::to_string(need) +
                    " bytes of staging (2 x tokens x heads x head_size x element size + 8 x tokens), the fixed "
                    "area holds " + std::to_string(cap) + "; split the batch or use kvc_reshape_and_cache_flash_host");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int dev = 0;
  KVC_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(KVC_ERR_INVALID_ARG, "device ordinal out of range");
  void* base = nullptr;
  if (int rc = fixed_staging_address(dev, &base)) return rc;
  char* dkey = static_cast<char*>(base);
  char* dval = dkey + kv_bytes;
  int64_t* dslots = reinterpret_cast<int64_t*>(dval + kv_bytes);
  // Every byte the kernel will read is overwritten here first; nothing relies on the area's old contents.
  const void* hsrc[2] = {host_key, host_value};
  char* ddst[2] = {dkey, dval};
  const int64_t hstride[2] = {key_stride_t, value_stride_t};
  for (int i = 0; i < 2; ++i) {
    if (hstride[i] == row) {
      KVC_CUDA_TRY(cudaMemcpyAsync(ddst[i], hsrc[i], static_cast<size_t>(num_tokens) * row_bytes,
                                   cudaMemcpyHostToDevice, st));
    } else {
      KVC_CUDA_TRY(cudaMemcpy2DAsync(ddst[i], row_bytes, hsrc[i], static_cast<size_t>(hstride[i]) * es, row_bytes,
                                     static_cast<size_t>(num_tokens), cudaMemcpyHostToDevice, st));
    }
  }
  KVC_CUDA_TRY(cudaMemcpyAsync(dslots, host_slot_mapping, static_cast<size_t>(num_tokens) * 8,
                               cudaMemcpyHostToDevice, st));
  return flash_impl(dkey, dval, key_cache, value_cache, dslots, num_tokens, num_heads, head_size, block_size,
                    row, head_size, row, head_size, block_stride, page_stride, head_stride, in_dtype, kv_dtype,
                    k_scale, v_scale, st);
}

int kvc_release_staging(void) {
  int dev = 0;
  KVC_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(KVC_ERR_INVALID_ARG, "device ordinal out of range");
  std::lock_guard<std::mutex> lk(g_staging_mu);
  Staging& s = g_staging[dev];
  if (s.buf) {
    KVC_CUDA_TRY(cudaDeviceSynchronize());
    KVC_CUDA_TRY(cudaFree(s.buf));
    s.buf = nullptr;
    s.cap = 0;
  }
  return KVC_OK;
}

int kvc_count_bad_slots(const int64_t* slot_mapping, int64_t num_tokens, int64_t num_slots, int64_t* bad_count,
                        void* stream) {
  if (!bad_count || num_tokens < 0 || (num_tokens > 0 && !slot_mapping))
    return fail(KVC_ERR_INVALID_ARG, "kvc_count_bad_slots: bad argument");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  KVC_CUDA_TRY(cudaMemsetAsync(bad_count, 0, sizeof(int64_t), st));
  if (num_tokens == 0) return KVC_OK;
  int64_t blocks = (num_tokens + 255) / 256;
  if (blocks > 1184) blocks = 1184;  // 8 CTAs per SM on 148 SMs; the loop strides over the rest
  count_bad_slots_kernel<<<static_cast<unsigned>(blocks), 256, 0, st>>>(
      slot_mapping, num_tokens, num_slots, reinterpret_cast<unsigned long long*>(bad_count));
  KVC_CUDA_TRY(cudaGetLastError());
  return KVC_OK;
}

}  // extern "C"
