// Paged decode attention for NVIDIA B200 (sm_100a): one query token per sequence against the keys
// and values that the cache-write kernels of this library stored, in their 16-bit type or as fp8
// bytes with per-tensor descales.  C ABI: kvc_paged_decode_attention.
//
//   out[s][h] = softmax_j( scale * q[s][h] . K[s][j][h / g] ) @ V[s][j][h / g],   j < seq_lens[s]
//   K[s][j] = key_cache[block_table[s][j / block_size]][j % block_size]   (flash layout [nb, bs, Hkv, D])
//
// The work is a stream over the sequence's cache blocks (HBM-bound: every cached byte is read once and
// meets 2 * g multiply-adds), so the kernel is organised around keeping loads in flight; the small
// matrix products run on mma.sync tiles (16 query rows x 16 tokens) fed by ldmatrix from shared memory.
// Long sequences are cut into splits that run as separate CTAs and are merged by a second kernel.
//
// The reference plugin's counterpart is the decode branch of mha_varlen_fwd,
// csrc/flash_attn/flash_api.cpp:124-165 (paged, max_seqlen_q == 1, no window), which launches a
// split-KV kernel plus a reduction; it reads 16-bit caches only (k_descale / v_descale raise
// NotImplementedError in vllm_xpu_kernels/flash_attn_interface.py:77-82).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdio>
#include <mutex>

#include "kvc_common.cuh"

namespace kvc {

namespace {

constexpr int kAttnThreads = 128;       // 4 warps
constexpr int kRows = 16;               // query rows per CTA (the heads of one kv group, padded)
constexpr float kLog2e = 1.4426950408889634f;

// ---------------------------------------------------------------------------------------------
// small PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

// 16-byte asynchronous copy global -> shared; src_bytes == 0 writes zeros instead.
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

// d += a (16x16, row) * b (16x8, col), fp32 accumulate.
template <typename T16>
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if constexpr (std::is_same_v<T16, __half>) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

// 2^x, one MUFU instruction (2 ulp; -inf gives 0).
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <typename T16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if constexpr (std::is_same_v<T16, __half>) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
  } else {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
}

// Two fp8 bytes (low 16 bits of `v`) -> two fp16 (exact: every e4m3 / e5m2 value is an fp16 value).
template <int KV>
__device__ __forceinline__ uint32_t fp8x2_to_f16x2(uint32_t v) {
  uint32_t r;
  const uint16_t h = static_cast<uint16_t>(v);
  if constexpr (KV == KVC_KV_FP8_E4M3) {
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(h));
  } else {
    asm("cvt.rn.f16x2.e5m2x2 %0, %1;" : "=r"(r) : "h"(h));
  }
  return r;
}

}  // namespace

// ---------------------------------------------------------------------------------------------
// parameters
// ---------------------------------------------------------------------------------------------
struct DecodeParams {
  void* out;               // [S, Hq, D] of the query's type
  const void* query;       // [S, Hq, D]
  const void* key_cache;   // [nb, bs, Hkv, D]: 16-bit type of the query, or fp8 bytes
  const void* value_cache;
  const int32_t* block_table;  // [S, block_table_stride]
  const int32_t* seq_lens;     // [S]
  const int32_t* cu_seqlens_q; // [S + 1] first query token of each sequence, or NULL: one token per sequence
  const void* sink;            // [Hq] of the query's type, or NULL
  const float* k_descale;      // device scalars, or NULL for 1
  const float* v_descale;
  float* part_lse;  // [S, Hq, splits]   log2-domain log-sum-exp of each split (-inf: empty)
  float* part_out;  // [S, Hq, splits, D] normalised partial results
  int64_t query_stride_t, query_stride_h, out_stride_t, out_stride_h;  // elements
  int64_t block_stride, page_stride, head_stride;                      // elements of the cache
  int64_t block_table_stride;
  // group = Hq / Hkv; a (sequence, kv head) has q_len * group query rows, token-major: row R is token R / group,
  // head R % group of the group; row_tiles = ceil(max_seqlen_q * group / 16)
  int32_t num_heads, num_kv_heads, group, row_tiles;
  int32_t block_size;
  int32_t bs_shift;  // log2(block_size), or -1
  int32_t num_splits, tiles_per_split;
  int32_t causal;  // query token i of q_len sees the first seq_len - q_len + i + 1 cached tokens
  int32_t many_rows_elsewhere;  // sequences with more than 16 rows per kv head are handled by paged_prefill_kernel
  // sliding window: the query token at position pos sees cached positions [pos - left, pos + right]; -1 = open
  int32_t window_left, window_right;
  float softmax_scale;
};

// ---------------------------------------------------------------------------------------------
// the decode kernel
// ---------------------------------------------------------------------------------------------
// TQ: type of query and output.  KV: KVC_KV_AUTO (cache holds TQ) or an fp8 code (cache holds bytes that
// are widened to fp16 on their way into shared memory; the products then run in fp16).  D: head size.
//
// A CTA owns (sequence, kv head, up to 16 query heads of its group, one split of the sequence) and walks
// the split in tiles of 64 (or 128) tokens through a two-stage shared-memory ring.  Warp w owns tokens
// [16w, 16w + 16) of every 64 tokens for BOTH products: it keeps its own running maximum, sum and a full
// 16 x D accumulator, the probabilities go from the first product's accumulators straight into the second
// product's A operand, and the four warps meet only at the pipeline barrier (one per tile) and in the
// final merge of their partial results.
template <typename TQ, int KV, int D, bool WIDE>
struct DecodeCfg {
  using T16 = std::conditional_t<KV == KVC_KV_AUTO, TQ, __half>;  // operand type of the matrix products
  static constexpr int kCacheES = (KV == KVC_KV_AUTO) ? 2 : 1;    // bytes per cached element
  static constexpr int kQRowBytes = D * 2 + 16;                   // shared-memory row of Q
  static constexpr int kRowBytes = D * kCacheES + 16;             // shared-memory row of K and V (16 B pad:
                                                                  // eight consecutive rows hit distinct banks)
  // Tokens per tile: 64, or (WIDE) 128 where a row is at most 128 bytes (fp8 with D <= 128, 16-bit with D = 64).
  // With 128 a warp owns two groups of 16 tokens per tile, whose first products are independent instruction
  // streams, and a CTA keeps twice the bytes in flight, at the price of fewer CTAs per SM; the host picks the
  // variant per launch.
  static_assert(!WIDE || D * kCacheES <= 128, "wide tiles only for rows of at most 128 bytes");
  static constexpr int kTile = WIDE ? 128 : 64;
  static constexpr int kGroups = kTile / 64;                      // 16-token groups per warp and tile
  static constexpr int kTileBytes = kTile * kRowBytes;            // one K or V tile
  // Two stages: one tile is consumed while the next one lands.  More stages were slower (fp8, D = 128: 110 us
  // with two stages and four CTAs per SM, 129 us with three stages and three CTAs, 185 us with four and two):
  // resident warps count for more than bytes in flight per CTA.
  static constexpr int kStages = 2;
  static constexpr bool kQInRegs = D <= 128;  // query fragments stay in registers (else re-read per tile)
  // The query rows pass through shared memory once on their way into registers; they borrow the second
  // stage of the ring, which is not written before every thread has fetched its fragments.
  static constexpr int kSmemQ = kQInRegs ? 0 : kRows * kQRowBytes;
  static_assert(kRows * kQRowBytes <= 2 * kTileBytes, "query rows fit in a stage");
  static constexpr int kSmemOff = kStages * kTile * (int)sizeof(int64_t);  // row offsets, one slot per stage
  static constexpr int kSmemBytes = kStages * 2 * kTileBytes + kSmemQ + kSmemOff;
  // the final merge reuses the ring: 4 warps x (16 x D fp32 + 32 floats of statistics)
  static_assert(4 * (kRows * D + 2 * kRows) * (int)sizeof(float) <= kStages * 2 * kTileBytes, "merge buffer fits");
  static_assert(D % 64 == 0 && D <= 256, "head sizes 64, 128, 192, 256");
  // CTAs per SM the register allocation has to leave room for: the 64-token fp8 instance of D = 128 lives on
  // four (43 KB of shared memory each); it measured 107 us with four and 123 us with three on the 64 x 4096 batch.
  // The other D = 128 instances hold three by shared memory (75-76 KB) and must not lose one to registers.
  static constexpr int kMinCtasPerSm = D != 128 ? 1 : (KV != KVC_KV_AUTO && !WIDE) ? 4 : 3;
};

// Within every group of 16 head dimensions the fp8 path works on a permuted order: an ldmatrix of fp8 rows
// hands lane t the four CONSECUTIVE elements 4t .. 4t+3, which become the operand pairs (k = 2t, 2t+1) and
// (k = 2t+8, 2t+9) of one mma step.  A dot product does not care about the order as long as Q uses the same
// one, so the query's 32-bit words are stored in that order: word W (elements 2W, 2W+1) of a group goes to
// position (W & 1) * 4 + (W >> 1).
__device__ __forceinline__ int fp8_q_word_position(int w) { return (w & 1) * 4 + (w >> 1); }

template <typename TQ, int KV, int D, bool WIDE>
__global__ void __launch_bounds__(kAttnThreads, DecodeCfg<TQ, KV, D, WIDE>::kMinCtasPerSm)
paged_decode_kernel(const DecodeParams p) {
  using Cfg = DecodeCfg<TQ, KV, D, WIDE>;
  using T16 = typename Cfg::T16;
  constexpr bool kFp8 = KV != KVC_KV_AUTO;
  constexpr int ES = Cfg::kCacheES;
  constexpr int QRB = Cfg::kQRowBytes;
  constexpr int RB = Cfg::kRowBytes;
  constexpr int NST = Cfg::kStages;
  constexpr int TN = Cfg::kTile;
  constexpr int NG = Cfg::kGroups;
  constexpr int NT = D / 8;  // 8-column tiles of the output accumulator

  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* s_kv = smem;                                       // NST stages x (K tile, V tile)
  unsigned char* s_q = Cfg::kQInRegs ? s_kv + 2 * Cfg::kTileBytes   // [16][QRB]: borrowed from stage 1, or own
                                     : s_kv + NST * 2 * Cfg::kTileBytes;
  int64_t* s_off = reinterpret_cast<int64_t*>(s_kv + NST * 2 * Cfg::kTileBytes + Cfg::kSmemQ);   // [NST][TN] byte offsets of the tokens' rows

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;  // accumulator row (and row + 8) and column pair of this lane
  const int seq = blockIdx.y;
  const int kvh = blockIdx.x / p.row_tiles, row_tile = blockIdx.x - kvh * p.row_tiles;
  const int split = blockIdx.z;
  const int row0 = row_tile * kRows;  // first query row of this CTA within its (sequence, kv head)

  pdl_prologue();

  const int q_start = p.cu_seqlens_q ? p.cu_seqlens_q[seq] : seq;
  const int q_len = p.cu_seqlens_q ? p.cu_seqlens_q[seq + 1] - q_start : 1;
  const int seq_rows = q_len * p.group;
  if (row0 >= seq_rows) return;                   // this sequence has fewer query rows than the longest one
  if (p.many_rows_elsewhere && seq_rows > kRows) return;  // the many-rows kernel's
  const int rows = min(kRows, seq_rows - row0);   // valid rows
  // row r of the CTA: query token (row0 + r) / group of the sequence, head kvh * group + (row0 + r) % group
  auto row_token = [&](int r) { return (row0 + r) / p.group; };
  auto row_head = [&](int r) { return kvh * p.group + (row0 + r) % p.group; };

  const int n = p.seq_lens[seq];
  // Cached tokens row r may see: [row_lo(r), row_limit(r)).  The query token of the row sits at position
  // pos = n - q_len + token; the causal mask ends its view at pos, a window at pos + right, and a window starts
  // it at pos - left.  Both ends grow with the token, so the CTA walks from its first row's start to its last
  // row's end.
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
  const int total_tiles = (n_item + TN - 1) / TN;
  const int tile_begin = row_lo(0) / TN + split * p.tiles_per_split;
  const int tile_end = min(tile_begin + p.tiles_per_split, total_tiles);

  if (tile_begin >= tile_end) {  // nothing to attend to in this split's range
    for (int i = tid; i < rows * (p.num_splits > 1 ? 1 : D); i += kAttnThreads) {
      const int r = p.num_splits > 1 ? i : i / D;
      const int64_t tok = q_start + row_token(r);
      if (p.num_splits > 1) {
        p.part_lse[(tok * p.num_heads + row_head(r)) * p.num_splits + split] = -INFINITY;
      } else {
        static_cast<TQ*>(p.out)[tok * p.out_stride_t + row_head(r) * p.out_stride_h + i % D] = TQ(0.0f);
      }
    }
    return;
  }

  // ---- query rows -> shared memory (as T16), rows beyond the group are zero -------------------
  {
    constexpr int kChunks = D / 8;  // 16-byte chunks (8 elements) per row
    for (int c = tid; c < kRows * kChunks; c += kAttnThreads) {
      const int r = c / kChunks, col = c - r * kChunks;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (r < rows) {
        const TQ* src = static_cast<const TQ*>(p.query) + static_cast<int64_t>(q_start + row_token(r)) * p.query_stride_t +
                        row_head(r) * p.query_stride_h + col * 8;
        v = *reinterpret_cast<const uint4*>(src);
        if constexpr (!std::is_same_v<TQ, T16>) {  // bf16 query, fp16 products
          uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float lo = __uint_as_float(w[i] << 16), hi = __uint_as_float(w[i] & 0xFFFF0000u);
            w[i] = pack2<__half>(lo, hi);
          }
        }
      }
      if constexpr (kFp8) {
        const uint32_t* w = reinterpret_cast<const uint32_t*>(&v);
        uint32_t* group = reinterpret_cast<uint32_t*>(s_q + r * QRB + (col >> 1) * 32);
#pragma unroll
        for (int i = 0; i < 4; ++i) group[fp8_q_word_position((col & 1) * 4 + i)] = w[i];
      } else {
        *reinterpret_cast<uint4*>(s_q + r * QRB + col * 16) = v;
      }
    }
  }

  // ---- producer ----------------------------------------------------------------------------------
  // Row offsets (block-table lookup, one per token) are computed by the first 64 threads one tile ahead of
  // the copy that needs them and handed over through shared memory; the copies themselves are fully
  // coalesced: consecutive threads take consecutive 16-byte chunks of a row.
  const int32_t* table = p.block_table + seq * p.block_table_stride;
  const int64_t head_off = static_cast<int64_t>(kvh) * p.head_stride;
  auto publish_offsets = [&](int tile) {  // by threads 0..63, into slot (tile - tile_begin) % NST
    if (tid < TN) {
      const int token = tile * TN + tid;
      int64_t off = 0;  // rows beyond the sequence are copied with size 0 from a valid address
      if (tile < tile_end && token < n) {
        const int blk_idx = p.bs_shift >= 0 ? (token >> p.bs_shift) : token / p.block_size;
        off = (static_cast<int64_t>(__ldg(table + blk_idx)) * p.block_stride +
               static_cast<int64_t>(token - blk_idx * p.block_size) * p.page_stride + head_off) * ES;
      }
      s_off[((tile - tile_begin) % NST) * TN + tid] = off;
    }
  };
  const int64_t v_minus_k =
      static_cast<const unsigned char*>(p.value_cache) - static_cast<const unsigned char*>(p.key_cache);
  auto load_tile = [&](int tile) {  // both tiles of `tile` into its stage; rows beyond the sequence become zeros
    constexpr int kChunks = D * ES / 16;  // 16-byte chunks per row
    const int slot = (tile - tile_begin) % NST;
    const int64_t* offs = s_off + slot * TN;
    unsigned char* ks = s_kv + slot * 2 * Cfg::kTileBytes;
    const int rows_left = n - tile * TN;  // rows of this tile that exist (may exceed the tile)
    auto copy_chunk = [&](int r, int col) {
      const unsigned char* src = static_cast<const unsigned char*>(p.key_cache) + col * 16 + offs[r];
      const uint32_t dst = smem_u32(ks + r * RB + col * 16);
      const int nbytes = r < rows_left ? 16 : 0;
      cp_async_16(dst, src, nbytes);
      cp_async_16(dst + Cfg::kTileBytes, src + v_minus_k, nbytes);
    };
    if constexpr (kAttnThreads % kChunks == 0) {
      constexpr int kRowsPerPass = kAttnThreads / kChunks;
      const int r0 = tid / kChunks, col = tid - r0 * kChunks;
#pragma unroll
      for (int i = 0; i < TN / kRowsPerPass; ++i) copy_chunk(r0 + i * kRowsPerPass, col);
    } else {  // D = 192: 24 or 12 chunks per row
      for (int c = tid; c < TN * kChunks; c += kAttnThreads) copy_chunk(c / kChunks, c % kChunks);
    }
  };

  // ---- running state of this warp ----------------------------------------------------------------
  const float scale2 = p.softmax_scale * kLog2e * ((kFp8 && p.k_descale) ? __ldg(p.k_descale) : 1.0f);
  const float lazy_margin = 8.0f / scale2;  // raw-logit distance that is worth a factor 2^8
  // cached tokens visible to this lane's rows g and g + 8 (padding rows: the CTA's limit; they are never stored)
  const int lim[2] = {g < rows ? row_limit(g) : n_item, g + 8 < rows ? row_limit(g + 8) : n_item};
  const int lo[2] = {g < rows ? row_lo(g) : 0, g + 8 < rows ? row_lo(g + 8) : 0};
  float m_run[2] = {-INFINITY, -INFINITY};  // reference point (a lagging maximum) of the raw logits of rows g, g + 8
  float l_run[2] = {0.f, 0.f};              // this lane's share of the running sums of rows g and g + 8
  // rows g (c0, c1) / g + 8 (c2, c3); columns of tile i: 16-bit cache  8i + 2t, + 1
  //                                                      fp8 cache     16 (i / 2) + 4t + (i % 2), + 2
  float o_acc[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;

  const uint32_t q_base = smem_u32(s_q);
  // ldmatrix lane addressing (fragment layouts of mma.m16n8k16; a "column step" is 16 bytes of a row):
  //   A operand (Q):  row = lane % 16, column step = lane / 16
  //   B operand from K rows (no transpose): token = lane % 8 + (lane / 16) * 8, column step = (lane / 8) % 2
  //   B operand from V rows (transposed):   token = lane % 8 + ((lane / 8) % 2) * 8, column step = lane / 16
  const uint32_t a_lane_off_q = (lane & 15) * QRB + (lane >> 4) * 16;
  const uint32_t k_lane_off = (warp * 16 + (lane & 7) + (lane >> 4) * 8) * RB + ((lane >> 3) & 1) * 16;
  const uint32_t v_lane_off = (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * RB + (lane >> 4) * 16;

  // ---- prologue of the pipeline -------------------------------------------------------------------
#pragma unroll
  for (int i = 0; i < NST; ++i) publish_offsets(tile_begin + i);
  __syncthreads();  // offsets and query rows are visible
#pragma unroll
  for (int i = 0; i < NST - 1; ++i) {
    if (tile_begin + i < tile_end) load_tile(tile_begin + i);
    cp_async_commit();
  }
  [[maybe_unused]] uint32_t qf[Cfg::kQInRegs ? D / 16 : 1][4];
  if constexpr (Cfg::kQInRegs) {
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) ldmatrix_x4(qf[kk], q_base + a_lane_off_q + kk * 32);
  }
  auto q_frag = [&](int kk, uint32_t (&a)[4]) {
    if constexpr (Cfg::kQInRegs) {
      a[0] = qf[kk][0]; a[1] = qf[kk][1]; a[2] = qf[kk][2]; a[3] = qf[kk][3];
    } else {
      ldmatrix_x4(a, q_base + a_lane_off_q + kk * 32);
    }
  };

  for (int tile = tile_begin; tile < tile_end; ++tile) {
    const int slot = (tile - tile_begin) % NST;
    cp_async_wait<NST - 2>();  // this tile has landed
    __syncthreads();           // ... for every thread; the stage and offset slot of the previous tile are free
    if (tile + NST - 1 < tile_end) load_tile(tile + NST - 1);
    cp_async_commit();
    publish_offsets(tile + NST);  // into the slot this tile's copies were issued from
    const uint32_t ks = smem_u32(s_kv + slot * 2 * Cfg::kTileBytes);
    const uint32_t vs = ks + Cfg::kTileBytes;

    // ---- S = Q K^T for this warp's groups of 16 tokens (group gi: rows 64 gi + 16 warp ..) -------
    float s_acc[NG][2][4];
#pragma unroll
    for (int gi = 0; gi < NG; ++gi)
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) s_acc[gi][nt][0] = s_acc[gi][nt][1] = s_acc[gi][nt][2] = s_acc[gi][nt][3] = 0.f;
    if constexpr (!kFp8) {
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        uint32_t a[4];
        q_frag(kk, a);
#pragma unroll
        for (int gi = 0; gi < NG; ++gi) {
          uint32_t b[4];
          ldmatrix_x4(b, ks + k_lane_off + gi * 64 * RB + kk * 32);
          mma_16816<T16>(s_acc[gi][0], a, b[0], b[1]);
          mma_16816<T16>(s_acc[gi][1], a, b[2], b[3]);
        }
      }
    } else {
#pragma unroll
      for (int jj = 0; jj < D / 32; ++jj) {  // 32 head dimensions = two mma steps per ldmatrix
        uint32_t a0[4], a1[4];
        q_frag(2 * jj, a0);
        q_frag(2 * jj + 1, a1);
#pragma unroll
        for (int gi = 0; gi < NG; ++gi) {
          uint32_t b[4];
          // tokens 0-7: d-groups (2jj, 2jj+1); tokens 8-15: the same
          ldmatrix_x4(b, ks + k_lane_off + gi * 64 * RB + jj * 32);
          mma_16816<T16>(s_acc[gi][0], a0, fp8x2_to_f16x2<KV>(b[0]), fp8x2_to_f16x2<KV>(b[0] >> 16));
          mma_16816<T16>(s_acc[gi][1], a0, fp8x2_to_f16x2<KV>(b[2]), fp8x2_to_f16x2<KV>(b[2] >> 16));
          mma_16816<T16>(s_acc[gi][0], a1, fp8x2_to_f16x2<KV>(b[1]), fp8x2_to_f16x2<KV>(b[1] >> 16));
          mma_16816<T16>(s_acc[gi][1], a1, fp8x2_to_f16x2<KV>(b[3]), fp8x2_to_f16x2<KV>(b[3] >> 16));
        }
      }
    }

    // ---- mask the tail, running maximum (of the raw logits: the scale is positive), P = 2^(scale (S - m)) --
    if ((tile + 1) * TN > lim_min || tile * TN < lo_max) {  // only tiles that cross some row's ends need masking
#pragma unroll
      for (int gi = 0; gi < NG; ++gi) {
        const int tok_base = tile * TN + gi * 64 + warp * 16 + 2 * t;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int token = tok_base + nt * 8 + (e & 1);
            if (token >= lim[e >> 1] || token < lo[e >> 1]) s_acc[gi][nt][e] = -INFINITY;
          }
        }
      }
    }
    // The reference point of the exponentials follows the maximum lazily: it moves only when a logit exceeds it
    // by more than 2^8 after scaling (probabilities then reach at most 256, harmless in fp16 / bf16 / fp32), so
    // that the accumulator is rescaled a few times per sequence instead of in most tiles.
    float alpha[2], neg_ms[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float mx = -INFINITY;
#pragma unroll
      for (int gi = 0; gi < NG; ++gi)
        mx = fmaxf(mx, fmaxf(fmaxf(s_acc[gi][0][2 * r], s_acc[gi][0][2 * r + 1]),
                             fmaxf(s_acc[gi][1][2 * r], s_acc[gi][1][2 * r + 1])));
      mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 2));
      const bool move = mx > m_run[r] + lazy_margin;  // also the first finite maximum (m_run = -inf)
      alpha[r] = move ? fast_exp2((m_run[r] - mx) * scale2) : 1.0f;
      m_run[r] = move ? mx : m_run[r];
      neg_ms[r] = (m_run[r] == -INFINITY) ? 0.f : -m_run[r] * scale2;  // all masked so far: 2^(-inf) = 0 below
      l_run[r] *= alpha[r];
    }
    // rounded to T16, the probabilities are the A operand of the second product; the running sums take them
    // unrounded, as the reference statement normalises before it rounds
    uint32_t pa[NG][4];
#pragma unroll
    for (int gi = 0; gi < NG; ++gi) {
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        float pv[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) pv[e] = fast_exp2(fmaf(s_acc[gi][nt][e], scale2, neg_ms[e >> 1]));
        l_run[0] += pv[0] + pv[1];
        l_run[1] += pv[2] + pv[3];
        pa[gi][2 * nt] = pack2<T16>(pv[0], pv[1]);      // row g,     tokens nt * 8 + 2t, + 1 of the group
        pa[gi][2 * nt + 1] = pack2<T16>(pv[2], pv[3]);  // row g + 8
      }
    }

    // ---- O = alpha * O + P V over this warp's tokens ----------------------------------------------
    if (__any_sync(0xFFFFFFFFu, alpha[0] != 1.0f || alpha[1] != 1.0f)) {  // rare, see above
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        o_acc[i][0] *= alpha[0];
        o_acc[i][1] *= alpha[0];
        o_acc[i][2] *= alpha[1];
        o_acc[i][3] *= alpha[1];
      }
    }
    if constexpr (!kFp8) {
#pragma unroll
      for (int np = 0; np < D / 16; ++np) {  // two 8-column tiles per ldmatrix
#pragma unroll
        for (int gi = 0; gi < NG; ++gi) {
          uint32_t b[4];
          ldmatrix_x4_trans(b, vs + v_lane_off + gi * 64 * RB + np * 32);
          mma_16816<T16>(o_acc[2 * np], pa[gi], b[0], b[1]);
          mma_16816<T16>(o_acc[2 * np + 1], pa[gi], b[2], b[3]);
        }
      }
    } else {
#pragma unroll
      for (int jj = 0; jj < D / 32; ++jj) {  // 32 head dimensions = four 8-column tiles per ldmatrix
#pragma unroll
        for (int gi = 0; gi < NG; ++gi) {
          uint32_t b[4];
          // transposed 16-bit units: b[i] = (V[2t][2g], V[2t][2g+1], V[2t+1][2g], V[2t+1][2g+1]) as bytes, for
          // tokens 0-7 / 8-15 (i = 0 / 1) of dimensions 32jj .. +15, and the same (i = 2 / 3) of 32jj+16 .. +31
          ldmatrix_x4_trans(b, vs + v_lane_off + gi * 64 * RB + jj * 32);
#pragma unroll
          for (int i = 0; i < 4; ++i) b[i] = __byte_perm(b[i], 0, 0x3120);  // (even d: tokens 2t, 2t+1 | odd d: same)
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            mma_16816<T16>(o_acc[4 * jj + 2 * h], pa[gi], fp8x2_to_f16x2<KV>(b[2 * h]),
                           fp8x2_to_f16x2<KV>(b[2 * h + 1]));
            mma_16816<T16>(o_acc[4 * jj + 2 * h + 1], pa[gi], fp8x2_to_f16x2<KV>(b[2 * h] >> 16),
                           fp8x2_to_f16x2<KV>(b[2 * h + 1] >> 16));
          }
        }
      }
    }
  }
  cp_async_wait<0>();

  // ---- merge the four warps' partial results through shared memory ---------------------------------
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xFFFFFFFFu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xFFFFFFFFu, l_run[r], 2);
  }
  __syncthreads();  // nobody reads the ring any more
  float* s_o = reinterpret_cast<float*>(smem);           // [4 warps][16 rows][D]
  float* s_m = s_o + 4 * kRows * D;                      // [4][16]
  float* s_l = s_m + 4 * kRows;                          // [4][16]
  if (t == 0) {  // maxima leave in the log2 domain (-inf stays -inf)
    s_m[warp * kRows + g] = m_run[0] * scale2;
    s_m[warp * kRows + g + 8] = m_run[1] * scale2;
    s_l[warp * kRows + g] = l_run[0];
    s_l[warp * kRows + g + 8] = l_run[1];
  }
#pragma unroll
  for (int i = 0; i < NT; ++i) {
    float* dst = s_o + (warp * kRows + g) * D;
    if constexpr (!kFp8) {
      dst += i * 8 + 2 * t;
      *reinterpret_cast<float2*>(dst) = make_float2(o_acc[i][0], o_acc[i][1]);
      *reinterpret_cast<float2*>(dst + 8 * D) = make_float2(o_acc[i][2], o_acc[i][3]);
    } else {
      dst += 16 * (i >> 1) + 4 * t + (i & 1);
      dst[0] = o_acc[i][0];
      dst[2] = o_acc[i][1];
      dst[8 * D] = o_acc[i][2];
      dst[8 * D + 2] = o_acc[i][3];
    }
  }
  __syncthreads();

  const float v_descale = (kFp8 && p.v_descale) ? __ldg(p.v_descale) : 1.0f;
  // thread -> (row, pair of columns): 16 rows x D / 2 pairs over 128 threads
  for (int idx = tid; idx < rows * (D / 2); idx += kAttnThreads) {
    const int row = idx / (D / 2), d = (idx - row * (D / 2)) * 2;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) m = fmaxf(m, s_m[w * kRows + row]);
    float l = 0.f, ox = 0.f, oy = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = s_m[w * kRows + row];
      const float f = (mw == -INFINITY) ? 0.f : fast_exp2(mw - m);
      l += f * s_l[w * kRows + row];
      const float2 o = *reinterpret_cast<const float2*>(s_o + (w * kRows + row) * D + d);
      ox += f * o.x;
      oy += f * o.y;
    }
    const int head = row_head(row);
    const int64_t tok = q_start + row_token(row);
    if (p.num_splits > 1) {
      const int64_t slot = (tok * p.num_heads + head) * p.num_splits + split;
      if (d == 0) p.part_lse[slot] = (l > 0.f) ? m + log2f(l) : -INFINITY;
      const float inv = (l > 0.f) ? 1.0f / l : 0.f;
      *reinterpret_cast<float2*>(p.part_out + slot * D + d) = make_float2(ox * inv, oy * inv);
    } else {
      float rescale = 1.0f;
      if (p.sink) {  // one more logit in the denominator
        const float sk = static_cast<float>(static_cast<const TQ*>(p.sink)[head]) * kLog2e;
        const float mf = fmaxf(m, sk);
        rescale = (m == -INFINITY) ? 0.f : exp2f(m - mf);
        l = l * rescale + exp2f(sk - mf);
      }
      const float f = (l > 0.f) ? rescale / l * v_descale : 0.f;  // a row that sees no token gives zeros
      TQ* o = static_cast<TQ*>(p.out) + tok * p.out_stride_t + head * p.out_stride_h + d;
      *reinterpret_cast<uint32_t*>(o) = pack2<TQ>(ox * f, oy * f);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// the many-rows kernel: sequences with more than 16 query rows per kv head (prefill chunks)
// ---------------------------------------------------------------------------------------------
// Same stream over the cached tokens, other division of labour: a CTA owns 64 query rows (token-major
// (token, head) pairs of one kv head) and every warp 16 of them against ALL tokens of a tile, so a tile of
// keys and values serves 64 rows instead of 16 and nothing is merged across warps.  Sequences with at most
// 16 rows per kv head are left to paged_decode_kernel (its launch skips the others).
constexpr int kPrefillRows = 64;

template <typename TQ, int KV, int D>
struct PrefillCfg {
  using T16 = std::conditional_t<KV == KVC_KV_AUTO, TQ, __half>;
  static constexpr int kCacheES = (KV == KVC_KV_AUTO) ? 2 : 1;
  static constexpr int kQRowBytes = D * 2 + 16;
  static constexpr int kRowBytes = D * kCacheES + 16;
  static constexpr int kTile = 64;
  static constexpr int kTileBytes = kTile * kRowBytes;
  static constexpr int kStages = 2;
  // the query rows pass through the second stage on their way into registers (D <= 128) or stay behind the ring
  static constexpr bool kQInRegs = D <= 128;
  static constexpr int kSmemQ = kQInRegs ? 0 : kPrefillRows * kQRowBytes;
  static_assert(kPrefillRows * kQRowBytes <= 2 * kTileBytes || !kQInRegs, "query rows fit in a stage");
  static constexpr int kSmemOff = kStages * kTile * (int)sizeof(int64_t);
  static constexpr int kSmemBytes = kStages * 2 * kTileBytes + kSmemQ + kSmemOff;
};

template <typename TQ, int KV, int D>
__global__ void __launch_bounds__(kAttnThreads, (D <= 128 ? 3 : 1)) paged_prefill_kernel(const DecodeParams p) {
  using Cfg = PrefillCfg<TQ, KV, D>;
  using T16 = typename Cfg::T16;
  constexpr bool kFp8 = KV != KVC_KV_AUTO;
  constexpr int ES = Cfg::kCacheES;
  constexpr int QRB = Cfg::kQRowBytes;
  constexpr int RB = Cfg::kRowBytes;
  constexpr int NST = Cfg::kStages;
  constexpr int TN = Cfg::kTile;
  constexpr int NG = TN / 16;  // 16-token groups of a tile, all of them this warp's
  constexpr int NT = D / 8;

  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* s_kv = smem;
  unsigned char* s_q = Cfg::kQInRegs ? s_kv + 2 * Cfg::kTileBytes : s_kv + NST * 2 * Cfg::kTileBytes;
  int64_t* s_off = reinterpret_cast<int64_t*>(s_kv + NST * 2 * Cfg::kTileBytes + Cfg::kSmemQ);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int seq = blockIdx.y;
  // the longest rows first: under the causal mask the last row tiles of a sequence see the most tokens, and
  // CTAs are handed out in index order
  const int row_tile = p.row_tiles - 1 - static_cast<int>(blockIdx.x / p.num_kv_heads);
  const int kvh = blockIdx.x % p.num_kv_heads;
  const int row0 = row_tile * kPrefillRows;

  pdl_prologue();

  const int q_start = p.cu_seqlens_q ? p.cu_seqlens_q[seq] : seq;  // NULL: one query token per sequence
  const int q_len = p.cu_seqlens_q ? p.cu_seqlens_q[seq + 1] - q_start : 1;
  const int seq_rows = q_len * p.group;
  if (seq_rows <= kRows || row0 >= seq_rows) return;  // few rows: the decode kernel's; or past this sequence's rows
  const int rows = min(kPrefillRows, seq_rows - row0);
  auto row_token = [&](int r) { return (row0 + r) / p.group; };
  auto row_head = [&](int r) { return kvh * p.group + (row0 + r) % p.group; };
  const int n = p.seq_lens[seq];
  auto row_limit = [&](int r) {  // cached tokens row r may see: [row_lo(r), row_limit(r)), as in the decode kernel
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

  // this lane's rows: 16 warp + g and + 8
  const int my_row[2] = {warp * 16 + g, warp * 16 + g + 8};
  const bool warp_has_rows = warp * 16 < rows;

  if (tile_end <= tile_begin) {  // no row sees any token
    for (int i = tid; i < rows * D; i += kAttnThreads) {
      const int r = i / D;
      static_cast<TQ*>(p.out)[static_cast<int64_t>(q_start + row_token(r)) * p.out_stride_t +
                              row_head(r) * p.out_stride_h + i % D] = TQ(0.0f);
    }
    return;
  }

  // ---- query rows -> shared memory (as T16; fp8 path: permuted inside groups of 16) ----------------
  {
    constexpr int kChunks = D / 8;
    for (int c = tid; c < kPrefillRows * kChunks; c += kAttnThreads) {
      const int r = c / kChunks, col = c - r * kChunks;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (r < rows) {
        const TQ* src = static_cast<const TQ*>(p.query) + static_cast<int64_t>(q_start + row_token(r)) * p.query_stride_t +
                        row_head(r) * p.query_stride_h + col * 8;
        v = *reinterpret_cast<const uint4*>(src);
        if constexpr (!std::is_same_v<TQ, T16>) {
          uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float lo = __uint_as_float(w[i] << 16), hi = __uint_as_float(w[i] & 0xFFFF0000u);
            w[i] = pack2<__half>(lo, hi);
          }
        }
      }
      if constexpr (kFp8) {
        const uint32_t* w = reinterpret_cast<const uint32_t*>(&v);
        uint32_t* group = reinterpret_cast<uint32_t*>(s_q + r * QRB + (col >> 1) * 32);
#pragma unroll
        for (int i = 0; i < 4; ++i) group[fp8_q_word_position((col & 1) * 4 + i)] = w[i];
      } else {
        *reinterpret_cast<uint4*>(s_q + r * QRB + col * 16) = v;
      }
    }
  }

  // ---- producer (as in the decode kernel) -----------------------------------------------------------
  const int32_t* table = p.block_table + seq * p.block_table_stride;
  const int64_t head_off = static_cast<int64_t>(kvh) * p.head_stride;
  auto publish_offsets = [&](int tile) {
    if (tid < TN) {
      const int token = tile * TN + tid;
      int64_t off = 0;
      if (tile < tile_end && token < n) {
        const int blk_idx = p.bs_shift >= 0 ? (token >> p.bs_shift) : token / p.block_size;
        off = (static_cast<int64_t>(__ldg(table + blk_idx)) * p.block_stride +
               static_cast<int64_t>(token - blk_idx * p.block_size) * p.page_stride + head_off) * ES;
      }
      s_off[((tile - tile_begin) % NST) * TN + tid] = off;
    }
  };
  const int64_t v_minus_k =
      static_cast<const unsigned char*>(p.value_cache) - static_cast<const unsigned char*>(p.key_cache);
  auto load_tile = [&](int tile) {
    constexpr int kChunks = D * ES / 16;
    const int slot = (tile - tile_begin) % NST;
    const int64_t* offs = s_off + slot * TN;
    unsigned char* ks = s_kv + slot * 2 * Cfg::kTileBytes;
    const int rows_left = n - tile * TN;
    auto copy_chunk = [&](int r, int col) {
      const unsigned char* src = static_cast<const unsigned char*>(p.key_cache) + col * 16 + offs[r];
      const uint32_t dst = smem_u32(ks + r * RB + col * 16);
      const int nbytes = r < rows_left ? 16 : 0;
      cp_async_16(dst, src, nbytes);
      cp_async_16(dst + Cfg::kTileBytes, src + v_minus_k, nbytes);
    };
    if constexpr (kAttnThreads % kChunks == 0) {
      constexpr int kRowsPerPass = kAttnThreads / kChunks;
      const int r0 = tid / kChunks, col = tid - r0 * kChunks;
#pragma unroll
      for (int i = 0; i < TN / kRowsPerPass; ++i) copy_chunk(r0 + i * kRowsPerPass, col);
    } else {
      for (int c = tid; c < TN * kChunks; c += kAttnThreads) copy_chunk(c / kChunks, c % kChunks);
    }
  };

  // ---- state of this warp's 16 rows ------------------------------------------------------------------
  const float scale2 = p.softmax_scale * kLog2e * ((kFp8 && p.k_descale) ? __ldg(p.k_descale) : 1.0f);
  const float lazy_margin = 8.0f / scale2;
  const int lim[2] = {my_row[0] < rows ? row_limit(my_row[0]) : 0, my_row[1] < rows ? row_limit(my_row[1]) : 0};
  const int lo[2] = {my_row[0] < rows ? row_lo(my_row[0]) : 0, my_row[1] < rows ? row_lo(my_row[1]) : 0};
  // the warp computes only between its first row's start and its last valid row's end (it keeps helping with
  // the copies outside that range)
  const int warp_limit = warp_has_rows ? row_limit(min(rows, warp * 16 + 16) - 1) : 0;
  const int warp_lo = warp_has_rows ? row_lo(warp * 16) : 0;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};
  float o_acc[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;

  const uint32_t q_base = smem_u32(s_q);
  const uint32_t a_lane_off_q = (warp * 16 + (lane & 15)) * QRB + (lane >> 4) * 16;
  const uint32_t k_lane_off = ((lane & 7) + (lane >> 4) * 8) * RB + ((lane >> 3) & 1) * 16;
  const uint32_t v_lane_off = ((lane & 7) + ((lane >> 3) & 1) * 8) * RB + (lane >> 4) * 16;

#pragma unroll
  for (int i = 0; i < NST; ++i) publish_offsets(tile_begin + i);
  __syncthreads();
#pragma unroll
  for (int i = 0; i < NST - 1; ++i) {
    if (tile_begin + i < tile_end) load_tile(tile_begin + i);
    cp_async_commit();
  }
  [[maybe_unused]] uint32_t qf[Cfg::kQInRegs ? D / 16 : 1][4];
  if constexpr (Cfg::kQInRegs) {
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) ldmatrix_x4(qf[kk], q_base + a_lane_off_q + kk * 32);
  }
  auto q_frag = [&](int kk, uint32_t (&a)[4]) {
    if constexpr (Cfg::kQInRegs) {
      a[0] = qf[kk][0]; a[1] = qf[kk][1]; a[2] = qf[kk][2]; a[3] = qf[kk][3];
    } else {
      ldmatrix_x4(a, q_base + a_lane_off_q + kk * 32);
    }
  };

  for (int tile = tile_begin; tile < tile_end; ++tile) {
    const int slot = (tile - tile_begin) % NST;
    cp_async_wait<NST - 2>();
    __syncthreads();
    if (tile + NST - 1 < tile_end) load_tile(tile + NST - 1);
    cp_async_commit();
    publish_offsets(tile + NST);
    if (tile * TN >= warp_limit || (tile + 1) * TN <= warp_lo) continue;  // nothing here for this warp's rows
    const uint32_t ks = smem_u32(s_kv + slot * 2 * Cfg::kTileBytes);
    const uint32_t vs = ks + Cfg::kTileBytes;

    float s_acc[NG][2][4];
#pragma unroll
    for (int gi = 0; gi < NG; ++gi)
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) s_acc[gi][nt][0] = s_acc[gi][nt][1] = s_acc[gi][nt][2] = s_acc[gi][nt][3] = 0.f;
    if constexpr (!kFp8) {
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        uint32_t a[4];
        q_frag(kk, a);
#pragma unroll
        for (int gi = 0; gi < NG; ++gi) {
          uint32_t b[4];
          ldmatrix_x4(b, ks + k_lane_off + gi * 16 * RB + kk * 32);
          mma_16816<T16>(s_acc[gi][0], a, b[0], b[1]);
          mma_16816<T16>(s_acc[gi][1], a, b[2], b[3]);
        }
      }
    } else {
#pragma unroll
      for (int jj = 0; jj < D / 32; ++jj) {
        uint32_t a0[4], a1[4];
        q_frag(2 * jj, a0);
        q_frag(2 * jj + 1, a1);
#pragma unroll
        for (int gi = 0; gi < NG; ++gi) {
          uint32_t b[4];
          ldmatrix_x4(b, ks + k_lane_off + gi * 16 * RB + jj * 32);
          mma_16816<T16>(s_acc[gi][0], a0, fp8x2_to_f16x2<KV>(b[0]), fp8x2_to_f16x2<KV>(b[0] >> 16));
          mma_16816<T16>(s_acc[gi][1], a0, fp8x2_to_f16x2<KV>(b[2]), fp8x2_to_f16x2<KV>(b[2] >> 16));
          mma_16816<T16>(s_acc[gi][0], a1, fp8x2_to_f16x2<KV>(b[1]), fp8x2_to_f16x2<KV>(b[1] >> 16));
          mma_16816<T16>(s_acc[gi][1], a1, fp8x2_to_f16x2<KV>(b[3]), fp8x2_to_f16x2<KV>(b[3] >> 16));
        }
      }
    }

    if ((tile + 1) * TN > lim_min || tile * TN < lo_max) {  // some row of the CTA has tokens to mask in this tile
#pragma unroll
      for (int gi = 0; gi < NG; ++gi) {
        const int tok_base = tile * TN + gi * 16 + 2 * t;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int token = tok_base + nt * 8 + (e & 1);
            if (token >= lim[e >> 1] || token < lo[e >> 1]) s_acc[gi][nt][e] = -INFINITY;
          }
        }
      }
    }
    float alpha[2], neg_ms[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float mx = -INFINITY;
#pragma unroll
      for (int gi = 0; gi < NG; ++gi)
        mx = fmaxf(mx, fmaxf(fmaxf(s_acc[gi][0][2 * r], s_acc[gi][0][2 * r + 1]),
                             fmaxf(s_acc[gi][1][2 * r], s_acc[gi][1][2 * r + 1])));
      mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 2));
      const bool move = mx > m_run[r] + lazy_margin;
      alpha[r] = move ? fast_exp2((m_run[r] - mx) * scale2) : 1.0f;
      m_run[r] = move ? mx : m_run[r];
      neg_ms[r] = (m_run[r] == -INFINITY) ? 0.f : -m_run[r] * scale2;
      l_run[r] *= alpha[r];
    }
    uint32_t pa[NG][4];
#pragma unroll
    for (int gi = 0; gi < NG; ++gi) {
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        float pv[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) pv[e] = fast_exp2(fmaf(s_acc[gi][nt][e], scale2, neg_ms[e >> 1]));
        l_run[0] += pv[0] + pv[1];
        l_run[1] += pv[2] + pv[3];
        pa[gi][2 * nt] = pack2<T16>(pv[0], pv[1]);
        pa[gi][2 * nt + 1] = pack2<T16>(pv[2], pv[3]);
      }
    }
    if (__any_sync(0xFFFFFFFFu, alpha[0] != 1.0f || alpha[1] != 1.0f)) {
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        o_acc[i][0] *= alpha[0];
        o_acc[i][1] *= alpha[0];
        o_acc[i][2] *= alpha[1];
        o_acc[i][3] *= alpha[1];
      }
    }
    if constexpr (!kFp8) {
#pragma unroll
      for (int np = 0; np < D / 16; ++np) {
#pragma unroll
        for (int gi = 0; gi < NG; ++gi) {
          uint32_t b[4];
          ldmatrix_x4_trans(b, vs + v_lane_off + gi * 16 * RB + np * 32);
          mma_16816<T16>(o_acc[2 * np], pa[gi], b[0], b[1]);
          mma_16816<T16>(o_acc[2 * np + 1], pa[gi], b[2], b[3]);
        }
      }
    } else {
#pragma unroll
      for (int jj = 0; jj < D / 32; ++jj) {
#pragma unroll
        for (int gi = 0; gi < NG; ++gi) {
          uint32_t b[4];
          ldmatrix_x4_trans(b, vs + v_lane_off + gi * 16 * RB + jj * 32);
#pragma unroll
          for (int i = 0; i < 4; ++i) b[i] = __byte_perm(b[i], 0, 0x3120);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            mma_16816<T16>(o_acc[4 * jj + 2 * h], pa[gi], fp8x2_to_f16x2<KV>(b[2 * h]),
                           fp8x2_to_f16x2<KV>(b[2 * h + 1]));
            mma_16816<T16>(o_acc[4 * jj + 2 * h + 1], pa[gi], fp8x2_to_f16x2<KV>(b[2 * h] >> 16),
                           fp8x2_to_f16x2<KV>(b[2 * h + 1] >> 16));
          }
        }
      }
    }
  }
  cp_async_wait<0>();

  // ---- every lane finishes its own two rows ---------------------------------------------------------
  const float v_descale = (kFp8 && p.v_descale) ? __ldg(p.v_descale) : 1.0f;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    float l = l_run[r];
    l += __shfl_xor_sync(0xFFFFFFFFu, l, 1);
    l += __shfl_xor_sync(0xFFFFFFFFu, l, 2);
    if (my_row[r] >= rows) continue;
    const int head = row_head(my_row[r]);
    const float m = m_run[r] * scale2;  // log2 domain; -inf if the row saw nothing
    float rescale = 1.0f;
    if (p.sink) {
      const float sk = static_cast<float>(static_cast<const TQ*>(p.sink)[head]) * kLog2e;
      const float mf = fmaxf(m, sk);
      rescale = (m == -INFINITY) ? 0.f : exp2f(m - mf);
      l = l * rescale + exp2f(sk - mf);
    }
    const float f = (l > 0.f) ? rescale / l * v_descale : 0.f;
    TQ* o = static_cast<TQ*>(p.out) + static_cast<int64_t>(q_start + row_token(my_row[r])) * p.out_stride_t +
            head * p.out_stride_h;
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      const float x = o_acc[i][2 * r] * f, y = o_acc[i][2 * r + 1] * f;
      if constexpr (!kFp8) {
        *reinterpret_cast<uint32_t*>(o + i * 8 + 2 * t) = pack2<TQ>(x, y);
      } else {  // columns 16 (i / 2) + 4t + (i % 2) and + 2
        TQ* dst = o + 16 * (i >> 1) + 4 * t + (i & 1);
        dst[0] = TQ(x);
        dst[2] = TQ(y);
      }
    }
  }
}

}  // namespace kvc

// the many-rows kernels on tcgen05
#include "paged_prefill_umma.cuh"
#include "paged_prefill_pair_umma.cuh"

namespace kvc {

// ---------------------------------------------------------------------------------------------
// merge of the splits: out = sum_p w_p o_p / (sum_p w_p [+ sink]),  w_p = exp2(lse_p - max lse)
// ---------------------------------------------------------------------------------------------
template <typename TQ>
__global__ void __launch_bounds__(128) paged_decode_merge_kernel(const DecodeParams p, int head_size) {
  const int seq = blockIdx.x / p.num_heads, head = blockIdx.x - seq * p.num_heads;  // "seq": a query token
  pdl_prologue();
  const int64_t base = (static_cast<int64_t>(seq) * p.num_heads + head) * p.num_splits;
  float m = -INFINITY;
  for (int s = 0; s < p.num_splits; ++s) m = fmaxf(m, p.part_lse[base + s]);
  float sk = -INFINITY;
  if (p.sink) sk = static_cast<float>(static_cast<const TQ*>(p.sink)[head]) * kLog2e;
  TQ* o = static_cast<TQ*>(p.out) + seq * p.out_stride_t + head * p.out_stride_h;
  if (m == -INFINITY) {  // no cached token at all
    for (int d = threadIdx.x; d < head_size; d += blockDim.x) o[d] = TQ(0.0f);
    return;
  }
  const float mf = fmaxf(m, sk);
  float denom = (sk == -INFINITY) ? 0.f : exp2f(sk - mf);
  for (int s = 0; s < p.num_splits; ++s) {
    const float lse = p.part_lse[base + s];
    if (lse != -INFINITY) denom += exp2f(lse - mf);
  }
  const float v_descale = p.v_descale ? __ldg(p.v_descale) : 1.0f;
  const float inv = v_descale / denom;
  for (int d = threadIdx.x; d < head_size; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < p.num_splits; ++s) {
      const float lse = p.part_lse[base + s];
      if (lse != -INFINITY) acc += exp2f(lse - mf) * p.part_out[(base + s) * head_size + d];
    }
    o[d] = TQ(acc * inv);
  }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
namespace {

constexpr int kMaxSplits = 128;

// How many CTAs of a kernel instance one SM holds (asked of the runtime once per instance and device).
template <typename TQ, int KV, int D, bool WIDE>
int decode_ctas_per_sm() {
  using Cfg = DecodeCfg<TQ, KV, D, WIDE>;
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 1;
  if (cached[dev] == 0) {
    int n = 0;
    cudaFuncSetAttribute(paged_decode_kernel<TQ, KV, D, WIDE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         Cfg::kSmemBytes);
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, paged_decode_kernel<TQ, KV, D, WIDE>, kAttnThreads,
                                                      Cfg::kSmemBytes) != cudaSuccess || n < 1)
      n = 1;
    cached[dev] = n;
  }
  return cached[dev];
}

// Wide tiles exist where a cached row is at most 128 bytes.
constexpr bool wide_exists(int kv, int d) { return d * (kv == KVC_KV_AUTO ? 2 : 1) <= 128; }

template <typename TQ, int KV>
int decode_ctas_per_sm_d(int head_size, bool wide) {
  switch (head_size) {
    case 64:
      if (wide) return decode_ctas_per_sm<TQ, KV, 64, true>();
      return decode_ctas_per_sm<TQ, KV, 64, false>();
    case 128:
      if constexpr (wide_exists(KV, 128)) {
        if (wide) return decode_ctas_per_sm<TQ, KV, 128, true>();
      }
      return decode_ctas_per_sm<TQ, KV, 128, false>();
    case 192: return decode_ctas_per_sm<TQ, KV, 192, false>();
    default: return decode_ctas_per_sm<TQ, KV, 256, false>();
  }
}

int decode_slots(int q_dtype, int kv, int head_size, bool wide) {  // CTAs the whole device holds at once
  // KVC_TEST_DECODE_SLOTS fixes the count, so that the planner can be exercised for a given device size
  // on a machine without one
  static const long forced = [] {
    const char* e = getenv("KVC_TEST_DECODE_SLOTS");
    return e ? strtol(e, nullptr, 10) : 0L;
  }();
  if (forced > 0) return static_cast<int>(forced);
  int per_sm;
  if (q_dtype == KVC_IN_F16) {
    per_sm = kv == KVC_KV_AUTO ? decode_ctas_per_sm_d<__half, KVC_KV_AUTO>(head_size, wide)
             : kv == KVC_KV_FP8_E4M3 ? decode_ctas_per_sm_d<__half, KVC_KV_FP8_E4M3>(head_size, wide)
                                     : decode_ctas_per_sm_d<__half, KVC_KV_FP8_E5M2>(head_size, wide);
  } else {
    per_sm = kv == KVC_KV_AUTO ? decode_ctas_per_sm_d<__nv_bfloat16, KVC_KV_AUTO>(head_size, wide)
             : kv == KVC_KV_FP8_E4M3 ? decode_ctas_per_sm_d<__nv_bfloat16, KVC_KV_FP8_E4M3>(head_size, wide)
                                     : decode_ctas_per_sm_d<__nv_bfloat16, KVC_KV_FP8_E5M2>(head_size, wide);
  }
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms * per_sm;
}

// Number of splits for sequences of `max_tiles` tiles when `base` CTAs exist without splitting and the device
// holds `slots` CTAs at once.  All CTAs of a launch are equally long (tiles_per_split tiles plus a fixed
// start-up cost of about two tiles), so the launch takes ceil(ctas / slots) rounds of that length; splitting
// adds the merge launch and its traffic, about three tiles' worth.  Pick the count that minimises the sum,
// the smaller one on ties.
int pick_splits(int64_t base, int64_t max_tiles, int64_t slots, int64_t max_splits, int64_t* cost_out) {
  int best = 1;
  int64_t best_cost = -1;
  const int64_t limit = max_tiles < max_splits ? max_tiles : max_splits;
  for (int64_t s = 1; s <= limit; ++s) {
    const int64_t tps = (max_tiles + s - 1) / s;
    const int64_t eff = (max_tiles + tps - 1) / tps;  // splits that are not empty
    if (eff != s) continue;
    const int64_t rounds = (base * s + slots - 1) / slots;
    const int64_t cost = rounds * (tps + 2) + (s > 1 ? 3 : 0);
    if (best_cost < 0 || cost < best_cost) {
      best_cost = cost;
      best = static_cast<int>(s);
    }
  }
  *cost_out = best_cost;
  return best;
}

template <typename TQ, int KV, int D, bool WIDE>
cudaError_t launch_decode(const DecodeParams& p, dim3 grid, cudaStream_t st) {
  using Cfg = DecodeCfg<TQ, KV, D, WIDE>;
  static std::once_flag once[64];
  static cudaError_t attr_err[64];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  std::call_once(once[dev], [&] {
    attr_err[dev] = cudaFuncSetAttribute(paged_decode_kernel<TQ, KV, D, WIDE>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
  });
  if (attr_err[dev] != cudaSuccess) return attr_err[dev];
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kAttnThreads);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, paged_decode_kernel<TQ, KV, D, WIDE>, p);
}

template <typename TQ, int KV>
cudaError_t launch_decode_d(int head_size, bool wide, const DecodeParams& p, dim3 grid, cudaStream_t st) {
  switch (head_size) {
    case 64:
      if (wide) return launch_decode<TQ, KV, 64, true>(p, grid, st);
      return launch_decode<TQ, KV, 64, false>(p, grid, st);
    case 128:
      if constexpr (wide_exists(KV, 128)) {
        if (wide) return launch_decode<TQ, KV, 128, true>(p, grid, st);
      }
      return launch_decode<TQ, KV, 128, false>(p, grid, st);
    case 192: return launch_decode<TQ, KV, 192, false>(p, grid, st);
    default: return launch_decode<TQ, KV, 256, false>(p, grid, st);
  }
}

template <typename TQ>
cudaError_t launch_decode_kv(int kv, int head_size, bool wide, const DecodeParams& p, dim3 grid, cudaStream_t st) {
  switch (kv) {
    case KVC_KV_AUTO: return launch_decode_d<TQ, KVC_KV_AUTO>(head_size, wide, p, grid, st);
    case KVC_KV_FP8_E4M3: return launch_decode_d<TQ, KVC_KV_FP8_E4M3>(head_size, wide, p, grid, st);
    default: return launch_decode_d<TQ, KVC_KV_FP8_E5M2>(head_size, wide, p, grid, st);
  }
}

template <typename TQ, int KV, int D>
cudaError_t launch_prefill(const DecodeParams& p, dim3 grid, cudaStream_t st) {
  using Cfg = PrefillCfg<TQ, KV, D>;
  static std::once_flag once[64];
  static cudaError_t attr_err[64];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  std::call_once(once[dev], [&] {
    attr_err[dev] = cudaFuncSetAttribute(paged_prefill_kernel<TQ, KV, D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::kSmemBytes);
  });
  if (attr_err[dev] != cudaSuccess) return attr_err[dev];
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kAttnThreads);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, paged_prefill_kernel<TQ, KV, D>, p);
}

template <typename TQ, int KV>
cudaError_t launch_prefill_d(int head_size, const DecodeParams& p, dim3 grid, cudaStream_t st) {
  switch (head_size) {
    case 64: return launch_prefill<TQ, KV, 64>(p, grid, st);
    case 128: return launch_prefill<TQ, KV, 128>(p, grid, st);
    case 192: return launch_prefill<TQ, KV, 192>(p, grid, st);
    default: return launch_prefill<TQ, KV, 256>(p, grid, st);
  }
}

template <typename TQ>
cudaError_t launch_prefill_kv(int kv, int head_size, const DecodeParams& p, dim3 grid, cudaStream_t st) {
  switch (kv) {
    case KVC_KV_AUTO: return launch_prefill_d<TQ, KVC_KV_AUTO>(head_size, p, grid, st);
    case KVC_KV_FP8_E4M3: return launch_prefill_d<TQ, KVC_KV_FP8_E4M3>(head_size, p, grid, st);
    default: return launch_prefill_d<TQ, KVC_KV_FP8_E5M2>(head_size, p, grid, st);
  }
}

// The one-tile tcgen05 kernel serves every head size (64, 128, 192, 256) over 16-bit and fp8 caches, once some
// sequence has more than 64 query rows per kv head (below that its 128-row tiles would be mostly padding).
// KVC_PREFILL_LEGACY=1 keeps every call on the mma.sync kernel (for comparisons).
inline bool prefill_umma_enabled() {
  static const bool off = [] {
    const char* e = getenv("KVC_PREFILL_LEGACY");
    return e && e[0] == '1';
  }();
  return !off;
}
inline bool prefill_uses_umma(int kv_dtype, int64_t head_size, int64_t max_rows_per_kv_head) {
  (void)kv_dtype;  // 16-bit and fp8 caches alike
  const bool shape_ok = head_size == 64 || head_size == 128 || head_size == 192 || head_size == 256;
  return prefill_umma_enabled() && shape_ok && max_rows_per_kv_head > kPrefillRows;
}

template <typename TQ, int KV, int D>
cudaError_t launch_prefill_umma(const DecodeParams& p, dim3 grid, cudaStream_t st) {
  using Cfg = UmmaPrefillCfg<TQ, KV, D>;
  static std::once_flag once[64];
  static cudaError_t attr_err[64];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  std::call_once(once[dev], [&] {
    attr_err[dev] = cudaFuncSetAttribute(paged_prefill_umma_kernel<TQ, KV, D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::kSmemBytes);
    // two CTAs per SM (or one with 190 KB) need the whole shared-memory carve-out
    if (attr_err[dev] == cudaSuccess)
      attr_err[dev] = cudaFuncSetAttribute(paged_prefill_umma_kernel<TQ, KV, D>,
                                           cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (getenv("KVC_DEBUG_OCCUPANCY")) {
      int ctas = -1;
      cudaOccupancyMaxActiveBlocksPerMultiprocessor(&ctas, paged_prefill_umma_kernel<TQ, KV, D>, kUmmaThreads, Cfg::kSmemBytes);
      fprintf(stderr, "kvc: paged_prefill_umma_kernel: %d CTAs per SM (%d bytes of shared memory each)\n", ctas,
              Cfg::kSmemBytes);
    }
  });
  if (attr_err[dev] != cudaSuccess) return attr_err[dev];
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kUmmaThreads);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, paged_prefill_umma_kernel<TQ, KV, D>, p);
}

template <typename TQ, int D>
cudaError_t launch_prefill_umma_d(int kv, const DecodeParams& p, dim3 grid, cudaStream_t st) {
  switch (kv) {
    case KVC_KV_AUTO: return launch_prefill_umma<TQ, KVC_KV_AUTO, D>(p, grid, st);
    case KVC_KV_FP8_E4M3: return launch_prefill_umma<TQ, KVC_KV_FP8_E4M3, D>(p, grid, st);
    default: return launch_prefill_umma<TQ, KVC_KV_FP8_E5M2, D>(p, grid, st);
  }
}

template <typename TQ>
cudaError_t launch_prefill_umma_kv(int kv, int head_size, const DecodeParams& p, dim3 grid, cudaStream_t st) {
  switch (head_size) {
    case 64: return launch_prefill_umma_d<TQ, 64>(kv, p, grid, st);
    case 128: return launch_prefill_umma_d<TQ, 128>(kv, p, grid, st);
    case 192: return launch_prefill_umma_d<TQ, 192>(kv, p, grid, st);
    default: return launch_prefill_umma_d<TQ, 256>(kv, p, grid, st);
  }
}

// ---- the paired-tile tcgen05 kernel (head size 128, or 64 over 16-bit caches; power-of-two blocks of at least 8 tokens) ----
// KVC_PREFILL_PAIR=0 keeps such calls on the one-tile tcgen05 kernel (for comparisons).
inline bool prefill_pair_enabled() {
  static const bool off = [] {
    const char* e = getenv("KVC_PREFILL_PAIR");
    return e && e[0] == '0';
  }();
  return !off;
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled of the driver, looked up through the runtime (the library links no driver stub)
inline EncodeTiledFn tensor_map_encoder() {
  static const EncodeTiledFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      f = nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

// Head size 128 over 16-bit and fp8 caches, head size 64 over 16-bit caches.
inline bool prefill_uses_pair(int kv_dtype, int64_t head_size, int64_t max_rows_per_kv_head, int64_t block_size) {
  const bool shape_ok = head_size == 128 || (head_size == 64 && kv_dtype == KVC_KV_AUTO);
  return prefill_pair_enabled() && prefill_umma_enabled() && shape_ok && max_rows_per_kv_head > kPrefillRows &&
         pow2_shift(block_size) >= 3 && tensor_map_encoder() != nullptr;
}

// A tensor map over a paged cache [block][token in block][kv head][d] of 16-bit elements (any strides that are
// multiples of 16 bytes): the box is min(block_size, 128) tokens x one head x 64 elements, stored with the
// 128-byte swizzle.  The block dimension is given its largest legal extent: block numbers come from the block
// table, and the map itself knows no allocation size.
// An fp8 cache is mapped as bytes: the box is the tokens' raw 128-byte rows, unswizzled (the kernel widens them).
inline bool make_cache_tensor_map(CUtensorMap* map, const void* cache, int q_dtype, int kv_dtype, int head_size,
                                  const DecodeParams& p) {
  const bool fp8 = kv_dtype != KVC_KV_AUTO;
  const cuuint64_t es = fp8 ? 1 : 2;
  const cuuint64_t dims[4] = {static_cast<cuuint64_t>(head_size), static_cast<cuuint64_t>(p.num_kv_heads),
                              static_cast<cuuint64_t>(p.block_size), 1ull << 31};
  const cuuint64_t strides[3] = {static_cast<cuuint64_t>(p.head_stride) * es, static_cast<cuuint64_t>(p.page_stride) * es,
                                 static_cast<cuuint64_t>(p.block_stride) * es};
  const cuuint32_t box[4] = {fp8 ? 128u : 64u, 1, static_cast<cuuint32_t>(p.block_size < kPairTile ? p.block_size : kPairTile), 1};
  const cuuint32_t elem_strides[4] = {1, 1, 1, 1};
  const CUtensorMapDataType dt = fp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                     : (q_dtype == KVC_IN_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16);
  const CUresult r = tensor_map_encoder()(
      map, dt, 4, const_cast<void*>(cache), dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
      fp8 ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// A tensor map over the query or the output [token][head][d]: the box is one row tile in its token-major row
// order, 128 / group tokens x group heads x 64 elements.  Tokens past the tensor's end read as zeros and are not
// written.
inline bool make_query_tensor_map(CUtensorMap* map, const void* base, int64_t stride_t, int64_t stride_h, int q_dtype,
                                  int head_size, const DecodeParams& p, int64_t total_q) {
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(head_size), static_cast<cuuint64_t>(p.num_heads),
                              static_cast<cuuint64_t>(total_q)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(stride_h) * 2, static_cast<cuuint64_t>(stride_t) * 2};
  const cuuint32_t box[3] = {64, static_cast<cuuint32_t>(p.group), static_cast<cuuint32_t>(kPairRows / p.group)};
  const cuuint32_t elem_strides[3] = {1, 1, 1};
  const CUresult r = tensor_map_encoder()(
      map, q_dtype == KVC_IN_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3,
      const_cast<void*>(base), dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

template <typename TQ, int KV, int D>
cudaError_t launch_prefill_pair(const DecodeParams& p, int q_dtype, int64_t total_q, int64_t num_seqs, cudaStream_t st) {
  static std::once_flag once[64];
  static cudaError_t attr_err[64];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  static int sm_count[64];
  std::call_once(once[dev], [&] {
    attr_err[dev] = cudaFuncSetAttribute(paged_prefill_pair_kernel<TQ, KV, D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         PairCfg<D>::kSmemBytes);
    if (attr_err[dev] == cudaSuccess)
      attr_err[dev] = cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
  });
  if (attr_err[dev] != cudaSuccess) return attr_err[dev];
  // One CTA per SM walks the work items (pairs of row tiles of a sequence and kv head, heaviest first) with a
  // stride of the grid: tensor memory is allocated once per CTA and the items' fixed costs are paid back to back
  // instead of once per CTA launch.
  const int64_t items = static_cast<int64_t>(p.row_tiles) * p.num_kv_heads * num_seqs;
  if (items <= 0 || items > 0x7FFFFFFFll) return cudaErrorInvalidValue;
  const dim3 grid(static_cast<unsigned>(items < sm_count[dev] ? items : sm_count[dev]));
  CUtensorMap map_k, map_v, map_q, map_o;
  if (!make_cache_tensor_map(&map_k, p.key_cache, q_dtype, KV, D, p) ||
      !make_cache_tensor_map(&map_v, p.value_cache, q_dtype, KV, D, p))
    return cudaErrorInvalidValue;
  // the query rows come by TMA where a row tile is a box: power-of-two groups of at most 128 heads (a bf16 query
  // over an fp8 cache is then converted to fp16 in shared memory by the widening warps); results likewise
  const bool box_rows_ok = (p.group & (p.group - 1)) == 0 && p.group <= kPairRows;
  int q_by_tma = box_rows_ok ? 1 : 0;
  int o_by_tma = box_rows_ok && aligned(p.out, 16) && (p.out_stride_t * 2) % 16 == 0 && (p.out_stride_h * 2) % 16 == 0;
  if (q_by_tma && !make_query_tensor_map(&map_q, p.query, p.query_stride_t, p.query_stride_h, q_dtype, D, p, total_q))
    q_by_tma = 0;
  if (o_by_tma && !make_query_tensor_map(&map_o, p.out, p.out_stride_t, p.out_stride_h, q_dtype, D, p, total_q))
    o_by_tma = 0;
  if (!q_by_tma) map_q = map_k;  // not read
  if (!o_by_tma) map_o = map_k;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kPairThreads);
  cfg.dynamicSmemBytes = PairCfg<D>::kSmemBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, paged_prefill_pair_kernel<TQ, KV, D>, p, map_k, map_v, map_q, map_o, q_by_tma, o_by_tma,
                            static_cast<int>(num_seqs), static_cast<int>(items));
}

template <typename TQ>
cudaError_t launch_prefill_pair_kv(int kv, int head_size, const DecodeParams& p, int q_dtype, int64_t total_q,
                                   int64_t num_seqs, cudaStream_t st) {
  if (head_size == 64) return launch_prefill_pair<TQ, KVC_KV_AUTO, 64>(p, q_dtype, total_q, num_seqs, st);
  switch (kv) {
    case KVC_KV_AUTO: return launch_prefill_pair<TQ, KVC_KV_AUTO, 128>(p, q_dtype, total_q, num_seqs, st);
    case KVC_KV_FP8_E4M3: return launch_prefill_pair<TQ, KVC_KV_FP8_E4M3, 128>(p, q_dtype, total_q, num_seqs, st);
    default: return launch_prefill_pair<TQ, KVC_KV_FP8_E5M2, 128>(p, q_dtype, total_q, num_seqs, st);
  }
}

struct DecodePlan {
  int splits;
  int tiles_per_split;
  bool wide;  // 128-token tiles
  int64_t row_tiles;  // 16-row tiles of the longest sequence's query rows
  int64_t workspace_bytes;
};

DecodePlan plan_decode(int64_t num_seqs, int64_t total_q, int64_t max_seqlen_q, int64_t num_heads,
                       int64_t num_kv_heads, int64_t head_size, int64_t max_seq_len, int q_dtype, int kv_dtype,
                       int64_t max_splits = kMaxSplits) {
  DecodePlan pl{1, 1, false, 1, 0};
  const int64_t group = num_kv_heads > 0 ? num_heads / num_kv_heads : 1;
  pl.row_tiles = (max_seqlen_q * group + kRows - 1) / kRows;
  if (max_seqlen_q * group > kRows) {
    // some sequence may have more than 16 query rows per kv head: those go to the many-rows kernel, the others
    // to the decode kernel with one row tile and no split (the merge would not know which tokens have partials)
    pl.row_tiles = 1;
    pl.tiles_per_split = static_cast<int>((max_seq_len + 63) / 64 > 0 ? (max_seq_len + 63) / 64 : 1);
    return pl;
  }
  // CTAs that do work without splitting: per kv head, ceil(q_len * group / 16) for every sequence (tiles do not
  // span sequences); exact for one token per sequence, else bounded through the total number of query rows
  const int64_t base = max_seqlen_q == 1 ? num_seqs * num_kv_heads * pl.row_tiles
                                         : num_kv_heads * (total_q * group / kRows + num_seqs);
  if (base <= 0) return pl;
  // both tile sizes where both exist: the cheaper plan wins.  A 128-token tile costs about 1.5 64-token tiles
  // of a CTA's time (measured on batches with many rounds: fewer barriers and more overlap per token).
  int64_t best_cost = -1;
  for (int wide = 0; wide <= (wide_exists(kv_dtype, static_cast<int>(head_size)) ? 1 : 0); ++wide) {
    const int tile_tokens = wide ? 128 : 64;
    int64_t max_tiles = (max_seq_len + tile_tokens - 1) / tile_tokens;
    if (max_tiles < 1) max_tiles = 1;
    int64_t cost = 0;
    const int s = pick_splits(base, max_tiles, decode_slots(q_dtype, kv_dtype, static_cast<int>(head_size), wide != 0),
                              max_splits, &cost);
    cost = wide ? (cost * 3 + 1) / 2 : cost;
    if (best_cost < 0 || cost <= best_cost) {  // ties go to the wide tile: fewer barriers per token
      best_cost = cost;
      pl.wide = wide != 0;
      pl.tiles_per_split = static_cast<int>((max_tiles + s - 1) / s);
      pl.splits = static_cast<int>((max_tiles + pl.tiles_per_split - 1) / pl.tiles_per_split);  // drop empty tails
    }
  }
  if (pl.splits > 1) pl.workspace_bytes = total_q * num_heads * pl.splits * (head_size + 1) * (int64_t)sizeof(float);
  return pl;
}

// The launch shape of kvc_paged_attention.  A closed window bounds what a query token can see whatever the
// sequence length, so the splits then cover the window, not the sequence.  A CTA of the decode kernel walks from
// its first row's start to its last row's end: window + 1 tokens plus one per further query token it holds (at
// most kRows), which touch at most floor((length - 2) / tile) + 2 tiles; the planner divides a token count by
// the tile size rounding up, so the count it gets carries 127 tokens of slack for the larger tile.
// The workspace is sized by kvc_paged_attention_workspace_bytes, which knows no window: the windowed plan never
// uses more splits than the plan for the whole sequence, and so never needs more workspace than that query
// reported (the cost model is not monotone in the tile count, the cap is what guarantees it).
DecodePlan plan_attention(int64_t num_seqs, int64_t total_q, int64_t max_seqlen_q, int64_t num_heads,
                          int64_t num_kv_heads, int64_t head_size, int64_t max_seq_len, int causal,
                          int64_t window_left, int64_t window_right, int q_dtype, int kv_dtype) {
  const DecodePlan whole = plan_decode(num_seqs, total_q, max_seqlen_q, num_heads, num_kv_heads, head_size,
                                       max_seq_len, q_dtype, kv_dtype);
  if (!(window_left >= 0 && (causal || window_right >= 0))) return whole;
  const int64_t spread = (max_seqlen_q < kRows ? max_seqlen_q : kRows) - 1;
  const int64_t w = window_left + 1 + (causal ? 0 : window_right) + spread + 127;
  if (w >= max_seq_len) return whole;
  DecodePlan pl = plan_decode(num_seqs, total_q, max_seqlen_q, num_heads, num_kv_heads, head_size, w, q_dtype, kv_dtype);
  if (pl.splits > whole.splits)
    pl = plan_decode(num_seqs, total_q, max_seqlen_q, num_heads, num_kv_heads, head_size, w, q_dtype, kv_dtype,
                     whole.splits);
  return pl;
}

}  // namespace
}  // namespace kvc

extern "C" {

KVC_API int kvc_paged_attention_plan(int64_t num_seqs, int64_t total_q, int64_t max_seqlen_q, int64_t num_heads,
                                     int64_t num_kv_heads, int64_t head_size, int64_t max_seq_len, int causal,
                                     int64_t window_left, int64_t window_right, int q_dtype, int kv_dtype,
                                     int32_t* splits, int32_t* tiles_per_split, int32_t* tile_tokens,
                                     int64_t* workspace_bytes) {
  using namespace kvc;
  if (num_seqs <= 0 || total_q <= 0 || max_seqlen_q <= 0 || num_heads <= 0 || num_kv_heads <= 0 || max_seq_len < 0 ||
      window_left < -1 || window_right < -1)
    return fail(KVC_ERR_INVALID_ARG, "paged_attention_plan: sizes must be positive, window sides -1 or >= 0");
  if (head_size != 64 && head_size != 128 && head_size != 192 && head_size != 256)
    return fail(KVC_ERR_UNSUPPORTED, "paged_attention_plan: head_size must be 64, 128, 192 or 256");
  if ((q_dtype != KVC_IN_F16 && q_dtype != KVC_IN_BF16) ||
      (kv_dtype != KVC_KV_AUTO && kv_dtype != KVC_KV_FP8_E4M3 && kv_dtype != KVC_KV_FP8_E5M2))
    return fail(KVC_ERR_UNSUPPORTED, "paged_attention_plan: unsupported query or cache type");
  const DecodePlan pl = plan_attention(num_seqs, total_q, max_seqlen_q, num_heads, num_kv_heads, head_size, max_seq_len,
                                       causal, window_left, window_right, q_dtype, kv_dtype);
  if (splits) *splits = pl.splits;
  if (tiles_per_split) *tiles_per_split = pl.tiles_per_split;
  if (tile_tokens) *tile_tokens = pl.wide ? 128 : 64;
  if (workspace_bytes) *workspace_bytes = pl.workspace_bytes;
  return KVC_OK;
}

KVC_API int64_t kvc_paged_attention_workspace_bytes(int64_t num_seqs, int64_t total_q, int64_t max_seqlen_q,
                                                    int64_t num_heads, int64_t num_kv_heads, int64_t head_size,
                                                    int64_t max_seq_len, int q_dtype, int kv_dtype) {
  if (num_seqs <= 0 || total_q <= 0 || max_seqlen_q <= 0 || num_heads <= 0 || num_kv_heads <= 0 || max_seq_len < 0)
    return 0;
  if (head_size != 64 && head_size != 128 && head_size != 192 && head_size != 256) return 0;
  if (q_dtype != KVC_IN_F16 && q_dtype != KVC_IN_BF16) return 0;
  if (kv_dtype != KVC_KV_AUTO && kv_dtype != KVC_KV_FP8_E4M3 && kv_dtype != KVC_KV_FP8_E5M2) return 0;
  return kvc::plan_decode(num_seqs, total_q, max_seqlen_q, num_heads, num_kv_heads, head_size, max_seq_len, q_dtype,
                          kv_dtype)
      .workspace_bytes;
}

KVC_API int64_t kvc_paged_decode_workspace_bytes(int64_t num_seqs, int64_t num_heads, int64_t num_kv_heads,
                                                 int64_t head_size, int64_t max_seq_len, int q_dtype, int kv_dtype) {
  return kvc_paged_attention_workspace_bytes(num_seqs, num_seqs, 1, num_heads, num_kv_heads, head_size, max_seq_len,
                                             q_dtype, kv_dtype);
}

KVC_API int kvc_paged_attention(void* out, const void* query, const void* key_cache, const void* value_cache,
                                const int32_t* block_table, const int32_t* seq_lens, const int32_t* cu_seqlens_q,
                                const void* sink, const float* k_descale, const float* v_descale, void* workspace,
                                int64_t workspace_bytes, int64_t num_seqs, int64_t total_q, int64_t max_seqlen_q,
                                int64_t num_heads, int64_t num_kv_heads, int64_t head_size, int64_t block_size,
                                int64_t block_table_stride, int64_t max_seq_len, int64_t query_stride_t,
                                int64_t query_stride_h, int64_t out_stride_t, int64_t out_stride_h,
                                int64_t block_stride, int64_t page_stride, int64_t head_stride, float softmax_scale,
                                int causal, int64_t window_left, int64_t window_right, int q_dtype, int kv_dtype,
                                void* stream) {
  using namespace kvc;
  if (window_left < -1 || window_right < -1 || window_left > 0x7FFFFFFFll || window_right > 0x7FFFFFFFll)
    return fail(KVC_ERR_INVALID_ARG, "paged_attention: a window side is -1 (open) or a non-negative number of tokens");
  if (q_dtype != KVC_IN_F16 && q_dtype != KVC_IN_BF16)
    return fail(KVC_ERR_UNSUPPORTED, "paged_attention: query must be fp16 or bf16");
  if (kv_dtype != KVC_KV_AUTO && kv_dtype != KVC_KV_FP8_E4M3 && kv_dtype != KVC_KV_FP8_E5M2)
    return fail(KVC_ERR_UNSUPPORTED, "Unsupported data type of kv cache: code " + std::to_string(kv_dtype));
  if (num_seqs < 0 || total_q < 0 || max_seqlen_q < 0 || num_heads <= 0 || num_kv_heads <= 0 || block_size <= 0 ||
      max_seq_len < 0)
    return fail(KVC_ERR_INVALID_ARG, "paged_attention: sizes must be positive");
  if (num_heads % num_kv_heads)
    return fail(KVC_ERR_INVALID_ARG, "paged_attention: num_heads must be a multiple of num_kv_heads");
  if (!(softmax_scale > 0.0f)) return fail(KVC_ERR_INVALID_ARG, "paged_attention: softmax_scale must be positive");
  if (head_size != 64 && head_size != 128 && head_size != 192 && head_size != 256)
    return fail(KVC_ERR_UNSUPPORTED, "paged_attention: head_size must be 64, 128, 192 or 256");
  if (num_seqs == 0 || total_q == 0 || max_seqlen_q == 0) return KVC_OK;
  if (!cu_seqlens_q && (total_q != num_seqs || max_seqlen_q != 1))
    return fail(KVC_ERR_INVALID_ARG, "paged_attention: without cu_seqlens_q every sequence has one query token");
  if (num_seqs > 65535)
    return fail(KVC_ERR_INVALID_ARG, "paged_attention: at most 65535 sequences per call");
  if (total_q > 0x7FFFFFFFll || max_seqlen_q > total_q || num_heads > 65535 * 16 || block_size > 0x7FFFFFFFll ||
      max_seq_len > 0x7FFFFFFFll)
    return fail(KVC_ERR_INVALID_ARG, "paged_attention: sizes out of range");
  if (!out || !query || !key_cache || !value_cache || !block_table || !seq_lens)
    return fail(KVC_ERR_INVALID_ARG, "paged_attention: out, query, caches, block_table and seq_lens must be non-NULL");
  const int ces = kv_dtype == KVC_KV_AUTO ? 2 : 1;
  const bool ok_align = aligned(query, 16) && aligned(out, 4) && aligned(key_cache, 16) && aligned(value_cache, 16) &&
                        (query_stride_t * 2) % 16 == 0 && (query_stride_h * 2) % 16 == 0 && (out_stride_t * 2) % 4 == 0 &&
                        (out_stride_h * 2) % 4 == 0 && (block_stride * ces) % 16 == 0 && (page_stride * ces) % 16 == 0 &&
                        (head_stride * ces) % 16 == 0 && aligned(block_table, 4) && aligned(seq_lens, 4) &&
                        aligned(cu_seqlens_q, 4);
  if (!ok_align) return fail(KVC_ERR_INVALID_ARG, "paged_attention: query and cache rows must be 16-byte aligned");

  const DecodePlan pl = plan_attention(num_seqs, total_q, max_seqlen_q, num_heads, num_kv_heads, head_size, max_seq_len,
                                       causal, window_left, window_right, q_dtype, kv_dtype);
  if (pl.splits > 1 && (!workspace || workspace_bytes < pl.workspace_bytes || !aligned(workspace, 16)))
    return fail(KVC_ERR_INVALID_ARG, "paged_attention: workspace missing, misaligned (16 bytes) or too small; ask "
                                     "kvc_paged_attention_workspace_bytes (" + std::to_string(pl.workspace_bytes) +
                                     " bytes)");

  DecodeParams p{};
  p.out = out;
  p.query = query;
  p.key_cache = key_cache;
  p.value_cache = value_cache;
  p.block_table = block_table;
  p.seq_lens = seq_lens;
  p.cu_seqlens_q = cu_seqlens_q;
  p.sink = sink;
  p.k_descale = k_descale;
  p.v_descale = v_descale;
  p.query_stride_t = query_stride_t;
  p.query_stride_h = query_stride_h;
  p.out_stride_t = out_stride_t;
  p.out_stride_h = out_stride_h;
  p.block_stride = block_stride;
  p.page_stride = page_stride;
  p.head_stride = head_stride;
  p.block_table_stride = block_table_stride;
  p.num_heads = static_cast<int32_t>(num_heads);
  p.num_kv_heads = static_cast<int32_t>(num_kv_heads);
  p.group = static_cast<int32_t>(num_heads / num_kv_heads);
  p.row_tiles = static_cast<int32_t>(pl.row_tiles);
  p.block_size = static_cast<int32_t>(block_size);
  p.bs_shift = pow2_shift(block_size);
  p.num_splits = pl.splits;
  p.tiles_per_split = pl.tiles_per_split;
  p.causal = causal ? 1 : 0;
  p.many_rows_elsewhere = (max_seqlen_q * p.group > kRows) ? 1 : 0;
  p.window_left = static_cast<int32_t>(window_left);
  p.window_right = static_cast<int32_t>(window_right);
  p.softmax_scale = softmax_scale;
  if (pl.splits > 1) {
    p.part_out = static_cast<float*>(workspace);  // first: its float2 stores need 8-byte alignment
    p.part_lse = p.part_out + total_q * num_heads * pl.splits * head_size;
  }
  const int64_t grid_x = static_cast<int64_t>(p.num_kv_heads) * p.row_tiles;
  if (grid_x > 0x7FFFFFFFll) return fail(KVC_ERR_INVALID_ARG, "paged_attention: too many query rows per sequence");
  const dim3 grid(static_cast<unsigned>(grid_x), static_cast<unsigned>(num_seqs), static_cast<unsigned>(pl.splits));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = (q_dtype == KVC_IN_F16)
                      ? launch_decode_kv<__half>(kv_dtype, static_cast<int>(head_size), pl.wide, p, grid, st)
                      : launch_decode_kv<__nv_bfloat16>(kv_dtype, static_cast<int>(head_size), pl.wide, p, grid, st);
  if (e != cudaSuccess)
    return fail(KVC_ERR_CUDA, std::string("paged_attention launch failed: ") + cudaGetErrorString(e));
  if (max_seqlen_q * p.group > kRows) {  // sequences with more than 16 query rows per kv head
    DecodeParams pp = p;
    const bool use_umma = prefill_uses_umma(kv_dtype, head_size, max_seqlen_q * p.group);
    const bool use_pair = prefill_uses_pair(kv_dtype, head_size, max_seqlen_q * p.group, block_size);
    const int64_t tile_rows = use_pair ? 2 * kPairRows : use_umma ? kUmmaRows : kPrefillRows;
    pp.row_tiles = static_cast<int32_t>((max_seqlen_q * p.group + tile_rows - 1) / tile_rows);
    const int64_t px = static_cast<int64_t>(pp.num_kv_heads) * pp.row_tiles;
    if (px > 0x7FFFFFFFll) return fail(KVC_ERR_INVALID_ARG, "paged_attention: too many query rows per sequence");
    const dim3 pgrid(static_cast<unsigned>(px), static_cast<unsigned>(num_seqs), 1);
    static const bool debug_dispatch = getenv("KVC_DEBUG_DISPATCH") != nullptr;
    if (debug_dispatch)
      fprintf(stderr, "kvc: many-rows attention on the %s kernel, grid %u x %u\n",
              use_pair ? "paired-tile tcgen05" : use_umma ? "one-tile tcgen05" : "mma.sync", pgrid.x, pgrid.y);
    if (use_pair)
      e = (q_dtype == KVC_IN_F16)
              ? launch_prefill_pair_kv<__half>(kv_dtype, static_cast<int>(head_size), pp, q_dtype, total_q, num_seqs, st)
              : launch_prefill_pair_kv<__nv_bfloat16>(kv_dtype, static_cast<int>(head_size), pp, q_dtype, total_q, num_seqs, st);
    else if (use_umma)
      e = (q_dtype == KVC_IN_F16)
              ? launch_prefill_umma_kv<__half>(kv_dtype, static_cast<int>(head_size), pp, pgrid, st)
              : launch_prefill_umma_kv<__nv_bfloat16>(kv_dtype, static_cast<int>(head_size), pp, pgrid, st);
    else
      e = (q_dtype == KVC_IN_F16) ? launch_prefill_kv<__half>(kv_dtype, static_cast<int>(head_size), pp, pgrid, st)
                                  : launch_prefill_kv<__nv_bfloat16>(kv_dtype, static_cast<int>(head_size), pp, pgrid, st);
    if (e != cudaSuccess)
      return fail(KVC_ERR_CUDA, std::string("paged_attention many-rows launch failed: ") + cudaGetErrorString(e));
  }
  if (pl.splits > 1) {
    const dim3 mgrid(static_cast<unsigned>(total_q * num_heads));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = mgrid;
    cfg.blockDim = dim3(128);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = (q_dtype == KVC_IN_F16)
            ? cudaLaunchKernelEx(&cfg, paged_decode_merge_kernel<__half>, p, static_cast<int>(head_size))
            : cudaLaunchKernelEx(&cfg, paged_decode_merge_kernel<__nv_bfloat16>, p, static_cast<int>(head_size));
    if (e != cudaSuccess)
      return fail(KVC_ERR_CUDA, std::string("paged_attention merge launch failed: ") + cudaGetErrorString(e));
  }
  return KVC_OK;
}

KVC_API int kvc_paged_attention_device_status(int* status) {
  using namespace kvc;
  if (!status) return fail(KVC_ERR_INVALID_ARG, "paged_attention_device_status: status must be non-NULL");
  int v = 0;
  const cudaError_t e = cudaMemcpyFromSymbol(&v, g_umma_status, sizeof(int));  // waits for the device's earlier work
  if (e != cudaSuccess)
    return fail(KVC_ERR_CUDA, std::string("paged_attention_device_status: ") + cudaGetErrorString(e));
  *status = v;
  return KVC_OK;
}

KVC_API int kvc_paged_attention_clear_device_status(void) {
  using namespace kvc;
  const int zero = 0;
  const cudaError_t e = cudaMemcpyToSymbol(g_umma_status, &zero, sizeof(int));  // waits for the device's earlier work
  if (e != cudaSuccess)
    return fail(KVC_ERR_CUDA, std::string("paged_attention_clear_device_status: ") + cudaGetErrorString(e));
  return KVC_OK;
}

KVC_API int kvc_selftest_bounded_wait_gives_up(int64_t tries, void* stream) {
  using namespace kvc;
  if (tries < 1 || tries > 5000)
    return fail(KVC_ERR_INVALID_ARG, "selftest_bounded_wait_gives_up: tries must be within 1..5000 (about 20 us each)");
  umma_wait_gives_up_kernel<<<1, 128, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint32_t>(tries));
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess)
    return fail(KVC_ERR_CUDA, std::string("selftest_bounded_wait_gives_up launch failed: ") + cudaGetErrorString(e));
  return KVC_OK;
}

KVC_API int kvc_paged_decode_attention(void* out, const void* query, const void* key_cache, const void* value_cache,
                                       const int32_t* block_table, const int32_t* seq_lens, const void* sink,
                                       const float* k_descale, const float* v_descale, void* workspace,
                                       int64_t workspace_bytes, int64_t num_seqs, int64_t num_heads,
                                       int64_t num_kv_heads, int64_t head_size, int64_t block_size,
                                       int64_t block_table_stride, int64_t max_seq_len, int64_t query_stride_t,
                                       int64_t query_stride_h, int64_t out_stride_t, int64_t out_stride_h,
                                       int64_t block_stride, int64_t page_stride, int64_t head_stride,
                                       float softmax_scale, int q_dtype, int kv_dtype, void* stream) {
  return kvc_paged_attention(out, query, key_cache, value_cache, block_table, seq_lens, nullptr, sink, k_descale,
                             v_descale, workspace, workspace_bytes, num_seqs, num_seqs, num_seqs > 0 ? 1 : 0, num_heads,
                             num_kv_heads, head_size, block_size, block_table_stride, max_seq_len, query_stride_t,
                             query_stride_h, out_stride_t, out_stride_h, block_stride, page_stride, head_stride,
                             softmax_scale, 0, -1, -1, q_dtype, kv_dtype, stream);
}

}  // extern "C"
