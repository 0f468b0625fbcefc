// The many-rows attention kernel on the fifth-generation tensor cores (tcgen05, accumulators in tensor
// memory).  Included by paged_attention_kernels.cu after DecodeParams and the cp.async helpers.
//
// Division of labour: a CTA of 288 threads owns 128 query rows (token-major (token, head) pairs of one kv
// head) and walks the cached tokens in tiles of 64.  Eight warps do the softmax: row r belongs to thread r of
// each of two warpgroups (tensor-memory lane r is readable by warps r / 32 and r / 32 + 4); the first warpgroup
// works on columns [0, 32) of a tile's scores and columns [0, D / 2) of the accumulator, the second on the other
// halves.  The ninth warp issues the matrix products.  Per tile i
//   1. the softmax threads wait for S(i) = Q K(i)^T in tensor-memory columns [0, 64) or [64, 128) (it was issued
//      two tiles earlier and is there), and start the copy of K(i+2) into the slot S(i) has released (cp.async
//      with the 128-byte swizzle applied to the destination; fp8 caches: registers, widened to fp16),
//   2. the two threads of row r read their halves of row r of S, apply the mask, agree on the row's maximum
//      through two floats of shared memory and one named barrier, and compute their 32 probabilities (no
//      shuffle at all),
//   3. they wait for O += P(i-1) V(i-1) (long done), start the copy of V(i+1) into the slot it has released,
//      rescale O in tensor memory if the row's reference maximum moved (rare, the lazy rule of the other
//      kernels), store P(i) as 16-bit pairs over the scores they just read, and arrive on the `ready` mbarrier,
//   4. the issuing thread, on `ready`, issues O += P(i) V(i) (M = 128, N = D, K = 16, 4 instructions, A from
//      tensor memory, V as an MN-major B operand from shared memory; O in columns [128, 128 + D)) and
//      S(i+2) = Q K(i+2)^T (M = 128, N = 64, K = 16, D / 16 instructions, both operands from shared memory), each
//      followed by a commit to its mbarrier.  The tensor pipe runs one thread's instructions in order, which is
//      what lets P(i) and S(i+2) share columns.
// Head sizes 64 and 128: two CTAs share an SM (shared memory is sized for exactly two, and each allocates 256 of the 512
// tensor-memory columns, so an allocation never waits).  Head sizes 192 and 256: the accumulator
// alone takes 192 or 256 columns and the operand tiles 144 or 192 KB, so an SM holds one CTA, which allocates
// all 512 columns; each product O += P V then covers 192 or 256 columns, so the tensor pipe has two to three
// times the work per score and the softmax threads are no longer what the tile waits for.
//
// Every wait on an mbarrier is bounded; a wait that gives up sets the CTA's abort word, the CTA runs to its
// end, frees its tensor memory and raises g_umma_status.
#pragma once

#include "umma_sm100.cuh"

namespace kvc {
namespace {

constexpr int kUmmaRows = 128;
constexpr int kUmmaSoftmaxThreads = 256;  // two warpgroups: both own all 128 rows, each one half of a tile's 64 columns
constexpr int kUmmaThreads = kUmmaSoftmaxThreads + 32;  // and one warp that issues the matrix products
constexpr uint32_t kUmmaColS = 0;
constexpr uint32_t kUmmaColO = 128;

// 0 = fine; 1 = an mbarrier wait gave up; 2 = shared memory window not 1024-byte aligned
__device__ int g_umma_status = 0;

// a named barrier of the CTA (0 is __syncthreads) over `threads` threads
__device__ __forceinline__ void named_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

template <typename TQ, int KV, int D>
struct UmmaPrefillCfg {
  using T16 = std::conditional_t<KV == KVC_KV_AUTO, TQ, __half>;  // operand type of the matrix products
  static_assert(D == 64 || D == 128 || D == 192 || D == 256, "head sizes 64, 128, 192, 256");
  static constexpr int kCtasPerSm = D <= 128 ? 2 : 1;
  static constexpr uint32_t kTmemCols = D <= 128 ? 256 : 512;  // scores 128 + accumulator D, a power of two
  static constexpr int kTile = 64;
  static constexpr int kHalves = D / 64;                     // 128-byte-wide operand tiles per row
  static constexpr int kQHalfBytes = kUmmaRows * 128;        // 16 KB
  static constexpr int kQBytes = kQHalfBytes * kHalves;      // 32 KB at head size 128
  static constexpr int kKVHalfBytes = kTile * 128;           // 8 KB
  static constexpr int kKVBytes = kKVHalfBytes * kHalves;    // one K or V tile: 16 KB at head size 128
  static constexpr int kStages = 2;
  static constexpr int kOffQ = 0;
  static constexpr int kOffKV = kOffQ + kQBytes;             // [stage][K, V]
  static constexpr int kOffBar = kOffKV + kStages * 2 * kKVBytes;  // four mbarriers, tensor-memory slot, abort word
  static constexpr int kOffXch = kOffBar + 48;               // the warpgroups' exchange: [tile parity][warpgroup][row]
  // head size 64 would leave room for more than two CTAs (which together could ask for more tensor memory than
  // an SM has): its request is padded to the size that admits exactly two
  static constexpr int kSmemUsed = kOffXch + 4 * kUmmaRows * 4;
  static constexpr int kSmemBytes = (kCtasPerSm == 2 && 3 * (kSmemUsed + 1024) <= 233472) ? 233472 / 3 : kSmemUsed;
  // kCtasPerSm CTAs per SM: each takes its bytes + 1 KB the system keeps per CTA out of the SM's 228 KB
  static_assert(kCtasPerSm * (kSmemBytes + 1024) <= 233472, "the CTAs of an SM fit its shared memory");
  // and never one more, which could ask for more tensor memory than an SM has
  static_assert((kCtasPerSm + 1) * (kSmemBytes + 1024) > 233472, "no further CTA fits");
  static_assert(kCtasPerSm * kTmemCols <= 512 && kUmmaColO + D <= kTmemCols, "tensor-memory columns");
};

template <typename TQ, int KV, int D>
__global__ void __launch_bounds__(kUmmaThreads, (UmmaPrefillCfg<TQ, KV, D>::kCtasPerSm)) paged_prefill_umma_kernel(const DecodeParams p) {
  using Cfg = UmmaPrefillCfg<TQ, KV, D>;
  using T16 = typename Cfg::T16;
  constexpr bool kFp8 = KV != KVC_KV_AUTO;
  using namespace umma;
  constexpr int TN = Cfg::kTile;
  constexpr int KVB = Cfg::kKVBytes;

  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* s_q = smem + Cfg::kOffQ;
  unsigned char* s_kv = smem + Cfg::kOffKV;
  uint64_t* bar_s = reinterpret_cast<uint64_t*>(smem + Cfg::kOffBar);  // [2], one per score buffer: S(j) is complete
  uint64_t* bar_o = bar_s + 2;                                         // phase j: O += P(j) V(j) is complete
  uint64_t* bar_ready = bar_s + 3;  // phase j: all 256 softmax threads are done with tile j (P stored, copies landed)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_s + 4);
  volatile uint32_t* abort_word = tmem_slot + 1;
  volatile float* xch = reinterpret_cast<volatile float*>(smem + Cfg::kOffXch);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int wg = warp >> 2;               // warpgroup: which 32 of a tile's 64 columns (and which half of O)
  const int row = tid & (kUmmaRows - 1);  // tensor-memory lane = query row; warps w and w + 4 share their lanes
  const int seq = blockIdx.y;
  const int row_tile = p.row_tiles - 1 - static_cast<int>(blockIdx.x / p.num_kv_heads);  // heaviest first
  const int kvh = blockIdx.x % p.num_kv_heads;
  const int row0 = row_tile * kUmmaRows;

  pdl_prologue();

  const int q_start = p.cu_seqlens_q ? p.cu_seqlens_q[seq] : seq;
  const int q_len = p.cu_seqlens_q ? p.cu_seqlens_q[seq + 1] - q_start : 1;
  const int seq_rows = q_len * p.group;
  if (seq_rows <= kRows || row0 >= seq_rows) return;  // the decode kernel's sequence, or no rows here
  const int rows = min(kUmmaRows, seq_rows - row0);
  // rows are token-major: row R of the kv head is token R / group, head R % group of the group (a shift and a
  // mask for the usual power-of-two groups)
  const int g_shift = (p.group & (p.group - 1)) == 0 ? __ffs(p.group) - 1 : -1;
  auto row_token = [&](int r) { return g_shift >= 0 ? (row0 + r) >> g_shift : (row0 + r) / p.group; };
  auto row_head = [&](int r) {
    return kvh * p.group + (g_shift >= 0 ? (row0 + r) & (p.group - 1) : (row0 + r) % p.group);
  };
  const int n = p.seq_lens[seq];
  auto row_limit = [&](int r) {
    const int pos = n - q_len + row_token(r);
    int hi = n;
    if (p.causal) hi = min(hi, pos + 1);
    if (p.window_right >= 0) hi = min(hi, pos + p.window_right + 1);
    return max(0, hi);
  };
  auto row_lo = [&](int r) { return p.window_left >= 0 ? max(0, n - q_len + row_token(r) - p.window_left) : 0; };
  const int n_item = row_limit(rows - 1);
  const int lim_min = row_limit(0);
  const int lo_max = row_lo(rows - 1);
  const int tile_end = (n_item + TN - 1) / TN;
  const int tile_begin = row_lo(0) / TN;

  if (tile_end <= tile_begin) {  // no row sees any token
    for (int i = tid; i < rows * D; i += kUmmaThreads) {
      const int r = i / D;
      static_cast<TQ*>(p.out)[static_cast<int64_t>(q_start + row_token(r)) * p.out_stride_t +
                              row_head(r) * p.out_stride_h + i % D] = TQ(0.0f);
    }
    return;
  }
  if (smem_addr(smem) & 1023u) {  // the operand tiles' swizzle assumes 1024-byte alignment
    if (tid == 0) atomicMax(&g_umma_status, 2);
    return;
  }

  // ---- barriers and tensor memory ----------------------------------------------------------------------
  if (tid == 0) {
    mbar_init(bar_s, 1);
    mbar_init(bar_s + 1, 1);
    mbar_init(bar_o, 1);
    mbar_init(bar_ready, kUmmaSoftmaxThreads);
    *abort_word = 0;
    mbar_init_fence();
  }
  if (warp == 0) tmem_alloc(tmem_slot, Cfg::kTmemCols);

  // ---- producer: thread t copies chunk t % (D / 8) of rows t / (D / 8) + kRowsPerPass i of a K or a V tile -------
  const int32_t* table = p.block_table + seq * p.block_table_stride;
  const int64_t head_off = static_cast<int64_t>(kvh) * p.head_stride;
  // The thread's chunk of row r0 + 16 i sits 2048 i bytes after its chunk of row r0 (the swizzle repeats every
  // 8 rows).  With power-of-two blocks of at least 64 tokens a tile lies inside one block: one table lookup per
  // tile and a constant pointer step per row; other block sizes look every row up.
  constexpr int kChunks = D / 8;  // 16-byte chunks per row
  // rows per pass: a multiple of the swizzle period of 8 rows (16, 8, 8 for head sizes 128, 192, 256; at 192 the
  // last 64 softmax threads copy nothing)
  constexpr int kRowsPerPass = (kUmmaSoftmaxThreads / kChunks) / 8 * 8;
  const bool loader = tid < kRowsPerPass * kChunks;
  const int ld_r0 = tid / kChunks, ld_col = tid % kChunks;
  const uint32_t ld_dst = (ld_col >> 3) * Cfg::kKVHalfBytes + swizzled_offset(ld_r0, ld_col & 7);
  const bool tile_in_block = p.bs_shift >= 6;
  const int64_t row_step_bytes = p.page_stride * 2 * kRowsPerPass;
  // The table entry of a tile is fetched two iterations before the copy that needs it, so that its latency
  // stays out of the softmax threads' critical path.
  auto tile_blk = [&](int tile) -> int32_t {
    return (tile_in_block && tile < tile_end) ? __ldg(table + ((tile * TN) >> p.bs_shift)) : 0;
  };
  auto load_rows = [&](int tile, const void* cache, unsigned char* dst_tile, int32_t blk) {
    if (!loader) return;
    const int rows_left = n - tile * TN;
    const uint32_t dst0 = smem_addr(dst_tile) + ld_dst;
    if (tile_in_block) {
      const int token0 = tile * TN;
      const unsigned char* src =
          static_cast<const unsigned char*>(cache) +
          (static_cast<int64_t>(blk) * p.block_stride + static_cast<int64_t>((token0 & (p.block_size - 1)) + ld_r0) * p.page_stride + head_off) * 2 +
          ld_col * 16;
#pragma unroll
      for (int i = 0; i < TN / kRowsPerPass; ++i) {
        cp_async_16(dst0 + i * (kRowsPerPass * 128), src, ld_r0 + i * kRowsPerPass < rows_left ? 16 : 0);
        src += row_step_bytes;
      }
    } else {
#pragma unroll
      for (int i = 0; i < TN / kRowsPerPass; ++i) {
        const int r = ld_r0 + i * kRowsPerPass;
        const int token = tile * TN + r;
        const bool valid = r < rows_left;
        int64_t off = 0;
        if (valid) {
          const int blk_idx = p.bs_shift >= 0 ? (token >> p.bs_shift) : token / p.block_size;
          off = (static_cast<int64_t>(__ldg(table + blk_idx)) * p.block_stride +
                 static_cast<int64_t>(token - blk_idx * p.block_size) * p.page_stride + head_off) * 2;
        }
        cp_async_16(dst0 + i * (kRowsPerPass * 128), static_cast<const unsigned char*>(cache) + off + ld_col * 16, valid ? 16 : 0);
      }
    }
  };
  // fp8 caches: a row is D bytes.  Thread t copies a quarter of one (quarter t % 4 of row t / 4, D / 64 chunks of
  // 16 bytes) with cp.async into the tile's slot as raw bytes, later reads them back, widens them to fp16 (exact)
  // and stores them as chunks of the swizzled 16-bit layout.  Raw chunk k of row r lies in line r (128 bytes) of
  // operand half kHalves - 1 - k / 8, at byte 16 (k % 8): all of a row's raw bytes sit on bytes of the same row's
  // 16-bit lines, and the last half is overwritten by the widening of the last raw bytes.  The only bytes a store
  // can overwrite before they are read are therefore those of the same row, which the same warp reads: a
  // __syncwarp between the reads and the stores is all the ordering the conversion needs.
  constexpr int kRawChunks = D / 64;  // 16-byte chunks of raw bytes per thread
  struct Fp8Quarter {
    uint4 c[kRawChunks];
  };
  auto raw_offset = [](int r, int k) { return (Cfg::kHalves - 1 - (k >> 3)) * Cfg::kKVHalfBytes + r * 128 + (k & 7) * 16; };
  auto issue_raw_fp8 = [&](int tile, const void* cache, int32_t blk, unsigned char* dst_tile) {
    const int r = tid >> 2, token = tile * TN + r;
    const bool valid = token < n;
    int64_t off = 0;
    if (valid) {
      if (tile_in_block) {
        off = static_cast<int64_t>(blk) * p.block_stride + static_cast<int64_t>(token & (p.block_size - 1)) * p.page_stride;
      } else {
        const int blk_idx = p.bs_shift >= 0 ? (token >> p.bs_shift) : token / p.block_size;
        off = static_cast<int64_t>(__ldg(table + blk_idx)) * p.block_stride +
              static_cast<int64_t>(token - blk_idx * p.block_size) * p.page_stride;
      }
    }
    const unsigned char* src = static_cast<const unsigned char*>(cache) + off + head_off + (tid & 3) * (D / 4);
#pragma unroll
    for (int i = 0; i < kRawChunks; ++i)
      cp_async_16(smem_addr(dst_tile) + raw_offset(r, (tid & 3) * kRawChunks + i), src + 16 * i, valid ? 16 : 0);
  };
  auto read_raw_fp8 = [&](const unsigned char* dst_tile) {
    Fp8Quarter q;
#pragma unroll
    for (int i = 0; i < kRawChunks; ++i)
      q.c[i] = *reinterpret_cast<const uint4*>(dst_tile + raw_offset(tid >> 2, (tid & 3) * kRawChunks + i));
    return q;
  };
  auto store_fp8 = [&](const Fp8Quarter& q, unsigned char* dst_tile) {
    const int r = tid >> 2;
#pragma unroll
    for (int i = 0; i < kRawChunks; ++i) {
      const uint32_t src[4] = {q.c[i].x, q.c[i].y, q.c[i].z, q.c[i].w};
#pragma unroll
      for (int k = 0; k < 2; ++k) {  // raw chunk j holds the elements of 16-bit chunks 2 j and 2 j + 1
        uint4 o;
        o.x = fp8x2_to_f16x2<kFp8 ? KV : KVC_KV_FP8_E4M3>(src[2 * k]);
        o.y = fp8x2_to_f16x2<kFp8 ? KV : KVC_KV_FP8_E4M3>(src[2 * k] >> 16);
        o.z = fp8x2_to_f16x2<kFp8 ? KV : KVC_KV_FP8_E4M3>(src[2 * k + 1]);
        o.w = fp8x2_to_f16x2<kFp8 ? KV : KVC_KV_FP8_E4M3>(src[2 * k + 1] >> 16);
        const int chunk = 2 * ((tid & 3) * kRawChunks + i) + k;  // 16-bit chunk of the row: half chunk / 8
        *reinterpret_cast<uint4*>(dst_tile + (chunk >> 3) * Cfg::kKVHalfBytes + swizzled_offset(r, chunk & 7)) = o;
      }
    }
  };
  auto k_slot = [&](int i) { return s_kv + (i & 1) * 2 * KVB; };
  auto v_slot = [&](int i) { return s_kv + (i & 1) * 2 * KVB + KVB; };

  // ---- this thread's row ----------------------------------------------------------------------------------
  const float scale2 = p.softmax_scale * kLog2e * ((kFp8 && p.k_descale) ? __ldg(p.k_descale) : 1.0f);
  const float lazy_margin = 8.0f / scale2;
  const int lim = row < rows ? row_limit(row) : 0;
  const int lo = row < rows ? row_lo(row) : 0;
  float m_run = -INFINITY, l_run = 0.f;  // the reference maximum is kept by both warpgroups, the sum is partial

  // Tile i of this CTA (token tile tile_begin + i) lives in K slot i & 1 and V slot i & 1.  Copy groups in
  // commit order: {K(0), K(1)}, {V(0)}, then two groups per iteration i: {K(i+2)}, {V(i+1)}.  Waiting for all but
  // the newest group at the end of iteration i therefore covers K(i+2), which the next iteration's first act
  // consumes, and V(i); V(i+1) has another iteration to land.
  const int nt = tile_end - tile_begin;
  const bool softmax_thread = tid < kUmmaSoftmaxThreads;
  int32_t blk_v = 0, blk_k = 0;  // table entries of tiles it + 1 (next V copy) and it + 2 (next K copy)
  if (softmax_thread) {
    const int32_t b0 = tile_blk(tile_begin);
    blk_v = tile_blk(tile_begin + 1);
    blk_k = tile_blk(tile_begin + 2);
    if constexpr (kFp8) {
      issue_raw_fp8(tile_begin, p.key_cache, b0, k_slot(0));
      issue_raw_fp8(tile_begin + 1, p.key_cache, blk_v, k_slot(1));  // zeros past the sequence's end
      issue_raw_fp8(tile_begin, p.value_cache, b0, v_slot(0));
      cp_async_commit();
      cp_async_wait<0>();
      const Fp8Quarter k0 = read_raw_fp8(k_slot(0)), k1 = read_raw_fp8(k_slot(1)), v0 = read_raw_fp8(v_slot(0));
      __syncwarp();
      store_fp8(k0, k_slot(0));
      store_fp8(k1, k_slot(1));
      store_fp8(v0, v_slot(0));
    } else {
      load_rows(tile_begin, p.key_cache, k_slot(0), b0);
      if (nt > 1) load_rows(tile_begin + 1, p.key_cache, k_slot(1), blk_v);
      cp_async_commit();
      load_rows(tile_begin, p.value_cache, v_slot(0), b0);
      cp_async_commit();
    }
  }
  // ---- query rows -> shared memory (zero rows past the end), while the first copies are in flight -----------
  for (int c = tid; c < kUmmaRows * (D / 8); c += kUmmaThreads) {
    const int r = c / (D / 8), col = c % (D / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < rows) {
      const TQ* src = static_cast<const TQ*>(p.query) + static_cast<int64_t>(q_start + row_token(r)) * p.query_stride_t +
                      row_head(r) * p.query_stride_h + col * 8;
      v = *reinterpret_cast<const uint4*>(src);
      if constexpr (!std::is_same_v<TQ, T16>) {  // bf16 query over an fp8 cache: the products run in fp16
        uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float lo = __uint_as_float(w[i] << 16), hi = __uint_as_float(w[i] & 0xFFFF0000u);
          w[i] = pack2<__half>(lo, hi);
        }
      }
    }
    *reinterpret_cast<uint4*>(s_q + (col >> 3) * Cfg::kQHalfBytes + swizzled_offset(r, col & 7)) = v;
  }

  cp_async_wait<1>();           // K(0), K(1)
  fence_smem_to_async_proxy();  // and the query rows
  fence_before_thread_sync();
  __syncthreads();
  fence_after_thread_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
  constexpr uint32_t kIdescQK = instr_desc_f16<T16>(kUmmaRows, TN, false, false);
  constexpr uint32_t kIdescPV = instr_desc_f16<T16>(kUmmaRows, D, false, true);
  // Descriptors: the upper word is constant per operand role, the lower one is (address >> 4) plus the leading
  // byte offset; shared-memory addresses are below 2^18, so stepping an operand is an add on the lower word.
  constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);  // SBO 1024, version 1, 128-byte swizzle
  constexpr uint32_t kLboK = (16u >> 4) << 16;                          // K-major operands: unused, 16 by convention
  constexpr uint32_t kLboV = (static_cast<uint32_t>(Cfg::kKVHalfBytes) >> 4) << 16;  // V: distance of the D halves
  auto make_desc = [](uint32_t lo) { return (static_cast<uint64_t>(kDescHi) << 32) | lo; };
  const uint32_t q_lo = (smem_addr(s_q) >> 4) | kLboK;
  const uint32_t k_lo0 = (smem_addr(s_kv) >> 4) | kLboK;
  const uint32_t v_lo0 = (smem_addr(s_kv + KVB) >> 4) | kLboV;
  auto issue_qk = [&](int i) {  // S(i) = Q K(i)^T into the score buffer i & 1
    const uint32_t k_lo = k_lo0 + (i & 1) * ((2 * KVB) >> 4);
    const uint32_t s_col = tmem + kUmmaColS + (i & 1) * TN;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      const uint64_t da = make_desc(q_lo + (((kk >> 2) * Cfg::kQHalfBytes + (kk & 3) * 32) >> 4));
      const uint64_t db = make_desc(k_lo + (((kk >> 2) * Cfg::kKVHalfBytes + (kk & 3) * 32) >> 4));
      mma_f16_ss(s_col, da, db, kIdescQK, kk > 0 ? 1u : 0u);
    }
  };
  auto issue_pv = [&](int i) {  // O (+)= P(i) V(i), P from the first 32 columns of score buffer i & 1
    const uint32_t v_lo = v_lo0 + (i & 1) * ((2 * KVB) >> 4);
    const uint32_t p_col = tmem + kUmmaColS + (i & 1) * TN;
#pragma unroll
    for (int kk = 0; kk < TN / 16; ++kk) {
      const uint64_t db = make_desc(v_lo + ((kk * 16 * 128) >> 4));
      mma_f16_ts(tmem + kUmmaColO, p_col + kk * 8, db, kIdescPV, (i > 0 || kk > 0) ? 1u : 0u);
    }
  };
  // ---- the issuing warp -------------------------------------------------------------------------------------
  // The tensor pipe executes one thread's instructions in issue order: Q K(0)^T, Q K(1)^T, then per tile j, once
  // the softmax threads have reported it ready, P(j) V(j) and Q K(j+2)^T (into the score buffer whose P(j) the
  // product just before it reads).  S(j) is therefore complete about two softmaxes before it is needed, and the
  // softmax threads wait for the tensor pipe only where they depend on it.  A barrier of the scores serves every
  // second tile, so it cannot run two phases ahead of a thread that still waits on it.
  if (!softmax_thread) {
    if (tid == kUmmaSoftmaxThreads) {
      issue_qk(0);
      mma_commit(bar_s);
      if (nt > 1) {
        issue_qk(1);
        mma_commit(bar_s + 1);
      }
      for (int j = 0; j < nt; ++j) {
        mbar_wait_bounded(bar_ready, j & 1, abort_word);
        fence_after_thread_sync();
        issue_pv(j);
        mma_commit(bar_o);
        if (j + 2 < nt) {
          issue_qk(j + 2);
          mma_commit(bar_s + (j & 1));
        }
      }
    }
    __syncwarp();
  }

  for (int it = 0; softmax_thread && it < nt; ++it) {
    const int tile = tile_begin + it;
    mbar_wait_bounded(bar_s + (it & 1), (it >> 1) & 1, abort_word);  // S(it) is there, K slot it & 1 is free
    fence_after_thread_sync();
    const int32_t blk_next = tile_blk(tile + 3);
    if (it + 2 < nt) {
      if constexpr (kFp8) {
        issue_raw_fp8(tile + 2, p.key_cache, blk_k, k_slot(it));
      } else {
        load_rows(tile + 2, p.key_cache, k_slot(it), blk_k);
      }
    }
    cp_async_commit();

    // ---- softmax of this thread's half row: columns [32 wg, 32 wg + 32) of the tile ---------------------------
    uint32_t sa[32];
    tmem_ld_32x32(tmem + lane_base + kUmmaColS + (it & 1) * TN + wg * 32, sa);
    tmem_ld_wait();
    float2 s2[16];  // the scores as pairs, for the packed fp32 instructions
#pragma unroll
    for (int i = 0; i < 16; ++i) s2[i] = make_float2(__uint_as_float(sa[2 * i]), __uint_as_float(sa[2 * i + 1]));
    if ((tile + 1) * TN > lim_min || tile * TN < lo_max) {  // some row of the CTA has tokens to mask here
      const int tok0 = tile * TN + wg * 32;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        if (tok0 + 2 * i >= lim || tok0 + 2 * i < lo) s2[i].x = -INFINITY;
        if (tok0 + 2 * i + 1 >= lim || tok0 + 2 * i + 1 < lo) s2[i].y = -INFINITY;
      }
    }
    float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
    for (int i = 0; i < 16; ++i) mx4[i & 3] = max3(mx4[i & 3], s2[i].x, s2[i].y);
    float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
    // The row's maximum over both halves: each thread publishes its half's maximum and reads the other's after
    // one named barrier.  The slots alternate with the tile's parity: a thread that runs ahead writes the other
    // slot, and cannot reach this slot again before its partner has passed the next tile's barrier.
    {
      volatile float* slot = xch + (it & 1) * 2 * kUmmaRows;
      slot[wg * kUmmaRows + row] = mx;
      named_bar_sync(1, kUmmaSoftmaxThreads);
      mx = fmaxf(mx, slot[(wg ^ 1) * kUmmaRows + row]);
    }
    const bool move = mx > m_run + lazy_margin;
    const float alpha = move ? fast_exp2((m_run - mx) * scale2) : 1.0f;
    m_run = move ? mx : m_run;
    const float neg_ms = (m_run == -INFINITY) ? 0.f : -m_run * scale2;
    l_run *= alpha;
    const float2 sc2 = make_float2(scale2, scale2), nm2 = make_float2(neg_ms, neg_ms);
    float2 l_add[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
    uint32_t w[16];  // this thread's 32 probabilities, two 16-bit values per word
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float2 e = __ffma2_rn(s2[j], sc2, nm2);
      const float2 pr = make_float2(fast_exp2(e.x), fast_exp2(e.y));
      l_add[j & 1] = __fadd2_rn(l_add[j & 1], pr);
      w[j] = pack2<T16>(pr.x, pr.y);
    }
    l_run += (l_add[0].x + l_add[0].y) + (l_add[1].x + l_add[1].y);
    // The previous tile's second product has had this softmax to finish: O is up to date for a rescale and
    // V slot (it + 1) & 1 is free.
    if (it > 0) {
      mbar_wait_bounded(bar_o, (it - 1) & 1, abort_word);
      fence_after_thread_sync();
    }
    if (it + 1 < nt) {
      if constexpr (kFp8) {
        issue_raw_fp8(tile + 1, p.value_cache, blk_v, v_slot(it + 1));
      } else {
        load_rows(tile + 1, p.value_cache, v_slot(it + 1), blk_v);
      }
    }
    cp_async_commit();
    blk_v = blk_k;
    blk_k = blk_next;
    if (it > 0 && __any_sync(0xFFFFFFFFu, alpha != 1.0f)) {  // rare: a reference maximum of the warp moved
#pragma unroll 1
      for (int c = 0; c < D / 64; ++c) {  // this warpgroup's half of the accumulator's columns
        uint32_t o[32];
        const uint32_t col = kUmmaColO + wg * (D / 2) + c * 32;
        tmem_ld_32x32(tmem + lane_base + col, o);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
        tmem_st_32x32(tmem + lane_base + col, o);
      }
    }
    // P(it) takes the place of S(it): both warpgroups have read their halves (the exchange above orders that)
    tmem_st_32x16(tmem + lane_base + kUmmaColS + (it & 1) * TN + wg * 16, w);
    tmem_st_wait();
    cp_async_wait<1>();           // all but this iteration's V group: V(it) and K(it + 2) have landed
    if constexpr (kFp8) {         // as raw bytes: widen K(it + 2) and V(it) in place (V(0) was done up front)
      Fp8Quarter fk, fv;
      if (it + 2 < nt) fk = read_raw_fp8(k_slot(it));
      if (it > 0) fv = read_raw_fp8(v_slot(it));
      __syncwarp();
      if (it + 2 < nt) store_fp8(fk, k_slot(it));
      if (it > 0) store_fp8(fv, v_slot(it));
    }
    fence_smem_to_async_proxy();
    fence_before_thread_sync();
    mbar_arrive(bar_ready);
  }
  if (softmax_thread) {
    cp_async_wait<0>();
    const bool finished = mbar_wait_bounded(bar_o, (nt - 1) & 1, abort_word);
    fence_after_thread_sync();
    if (!finished && (tid & 31) == 0) atomicMax(&g_umma_status, 1);
  }

  // ---- the two threads of a row add up their sums, then each finishes its half of the row ---------------------
  {
    if (softmax_thread && wg == 1) xch[row] = l_run;
    __syncthreads();
    float l = l_run;
    if (softmax_thread && wg == 0) {
      l += xch[row];
      xch[row] = l;
    }
    __syncthreads();
    if (softmax_thread && wg == 1) l = xch[row];
    const bool live = softmax_thread && row < rows;
    const int head = live ? row_head(row) : 0;
    const float m = m_run * scale2;  // log2 domain; -inf if the row saw nothing
    float rescale = 1.0f;
    if (p.sink && live) {
      const float sk = static_cast<float>(static_cast<const TQ*>(p.sink)[head]) * kLog2e;
      const float mf = fmaxf(m, sk);
      rescale = (m == -INFINITY) ? 0.f : exp2f(m - mf);
      l = l * rescale + exp2f(sk - mf);
    }
    const float f = (l > 0.f) ? rescale / l * ((kFp8 && p.v_descale) ? __ldg(p.v_descale) : 1.0f) : 0.f;
    TQ* o = static_cast<TQ*>(p.out) + (live ? static_cast<int64_t>(q_start + row_token(row)) * p.out_stride_t +
                                                  static_cast<int64_t>(head) * p.out_stride_h + wg * (D / 2)
                                            : 0);
    const bool vec16 = ((reinterpret_cast<uintptr_t>(p.out) | static_cast<uintptr_t>(p.out_stride_t * 2) |
                         static_cast<uintptr_t>(p.out_stride_h * 2)) & 15u) == 0;
#pragma unroll 1
    for (int c = 0; softmax_thread && c < D / 64; ++c) {
      uint32_t acc[32];
      tmem_ld_32x32(tmem + lane_base + kUmmaColO + wg * (D / 2) + c * 32, acc);
      tmem_ld_wait();
      if (!live) continue;
      uint32_t w[16];
#pragma unroll
      for (int i = 0; i < 16; ++i)
        w[i] = pack2<TQ>(__uint_as_float(acc[2 * i]) * f, __uint_as_float(acc[2 * i + 1]) * f);
      if (vec16) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          *reinterpret_cast<uint4*>(o + c * 32 + i * 8) = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) *reinterpret_cast<uint32_t*>(o + c * 32 + 2 * i) = w[i];
      }
    }
  }
  fence_before_thread_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, Cfg::kTmemCols);
}

// The give-up path of the bounded waits, run on purpose: one CTA allocates tensor memory, waits on an mbarrier
// that receives no arrival with a limit of `tries` tries (about 20 us each), gives up, frees its tensor
// memory and raises the status word, exactly as a CTA of the kernel above does when a product or a copy never
// reports.  Nothing faults and nothing spins without a limit.
__global__ void __launch_bounds__(128) umma_wait_gives_up_kernel(uint32_t tries) {
  using namespace umma;
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t tmem_slot;
  __shared__ uint32_t abort_word;
  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid == 0) {
    mbar_init(&bar, 1);
    abort_word = 0;
    mbar_init_fence();
  }
  if (warp == 0) tmem_alloc(&tmem_slot, 32);
  fence_before_thread_sync();
  __syncthreads();
  fence_after_thread_sync();
  const uint32_t tmem = tmem_slot;
  const bool completed = mbar_wait_bounded(&bar, 0, &abort_word, tries);
  if (!completed && (tid & 31) == 0) atomicMax(&g_umma_status, 1);
  fence_before_thread_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 32);
}

}  // namespace
}  // namespace kvc
