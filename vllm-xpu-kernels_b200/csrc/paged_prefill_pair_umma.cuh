// The many-rows attention kernel for head size 128 (16-bit and fp8 caches) and head size 64 (16-bit caches) on the
// fifth-generation tensor cores.
// One CTA per SM walks work items -- a pair of row tiles of 128 query rows each (token-major (token, head) pairs
// of one kv head of one sequence) that share every key/value tile -- in tiles of 128 cached tokens, and is
// specialised by warp:
//
//   warps 0-3   softmax of row tile A: thread r owns row r -- all 128 scores of a tile, the row's running
//   warps 4-7   maximum and sum, its accumulator row (same for row tile B).  No value ever crosses threads.
//   warp 8      issues O += P V (tcgen05.mma, M = 128, N = 128, K = 16, fp32 accumulation in tensor memory; P
//               read from tensor memory, V as an MN-major operand) and an item's first S = Q K^T (both operands
//               in shared memory); every later S batch has another issuer, see below.
//   warp 9      brings query, key and value tiles in with TMA tile copies (cp.async.bulk.tensor, 128-byte
//               swizzle, no multicast, this GPU's memory only).  Keys and values come straight from the paged
//               cache: a tensor map over [block][token in block][kv head][d] makes a cache block's rows one box,
//               the block table gives the block coordinate, one lane issues one box.
//   warps 10-11 fp8 caches only: widen a tile's raw rows (which the copy warp drops into the upper half of the
//               tile's slot) to fp16 in the operand layout; the products then run in fp16.  16-bit caches:
//               they issue the later S batches, warp 10 those that follow a read by row tile A, warp 11 those
//               that follow a read by row tile B.  (They complete the third warpgroup, whose registers go to
//               the softmax threads.)
//
// Tensor memory (512 columns, all of the SM's): O_A | O_B | X | P_A | P_B with 128, 128, 128, 64, 64 columns.
// X holds the scores of whichever row tile's turn it is: a softmax thread moves its row of X into registers
// at once (128 of the 224 registers it owns), and when the 128 threads of the row tile have done so the next use
// of X is issued -- the other row tile's scores of the same key tile, or this row tile's NEXT scores -- while
// this softmax is still running.  A row tile's chain of dependent steps is thus its softmax alone; what a step
// waits for is the chain X is handed along,
//
//   S_A(j) -> A reads -> S_B(j) -> B reads -> S_A(j+1) -> A reads -> ...
//
// and how long a link of it takes.  Three designs, in the order they were measured (a step is two row tiles x 128
// tokens; the tensor pipe needs 2 800 cycles of it, a softmax 2 250):
//   1. warp 8 issues everything, in a fixed order, and learns of each read and each "P stored" through an
//      mbarrier: 4 100 cycles.  While its thread is held by one batch (the pipe takes eight instructions in 800 to
//      1 100 cycles) it cannot answer the next event, and every link has two sleeping waiters.
//   2. a thread of the row tile that has just read X issues the next use itself (a named barrier among the 128,
//      then the batch): 3 800.  The link is short, but that thread's warp stands still for those 1 100 cycles
//      and the row tile is as late as its latest warp.  fp8 caches, whose warps 10 and 11 are busy, run this way.
//   3. 16-bit caches: warps 10 and 11 do nothing else than issue those uses.  They sleep on a named barrier at
//      which the softmax warps only arrive (one instruction, no wait), so the issuer is released with the last
//      arrival; warp 8 keeps O_g += P_g(j) V(j), released by a second such barrier when P is stored: 3 400.
// The probabilities have columns of their own, which PV(j) has finished reading before the softmax of tile j + 1
// stores into them (the wait for "O += P(j) V(j) complete" that a rescaling of O needs anyway).  tcgen05.commit
// tracks the instructions of the thread that executes it, so whoever issues a batch also commits it to the
// scores barrier, and after a tile's last batch to "key slot free", after the item's last to "query rows free".
//
// A softmax thread costs about 3.5 instructions per score (one tcgen05.ld of 32 columns per 32 scores, packed
// fp32 arithmetic, 3-input max, one ex2 per score, 16-bit packing); every fixed per-tile cost is spread over 128
// scores per thread.
//
// Work items are numbered heaviest first and dealt to the CTAs in a serpentine; a CTA allocates tensor memory
// once and re-arms its barriers per item.  Where the group size is a power of two a row tile is one box of the
// query tensor and of the output tensor [token][head][d]: queries arrive by TMA, and a full row tile of results
// leaves by TMA from the (then idle) query buffer; other group sizes and cut-off tiles take ordinary loads and
// stores.
//
// Rows past a sequence's end inside the last tile: their keys may be anything (the scores are masked before
// use), their values are zeroed in shared memory by the issuing warp before the product that reads them, so
// that a probability of exactly zero cannot meet a NaN.
//
// Every wait on an mbarrier is bounded; a wait that gives up sets the CTA's abort word, the CTA runs to its
// end, waits (bounded) for its copies in flight, frees its tensor memory and raises g_umma_status.
#pragma once

#include <cuda.h>

#include "paged_prefill_umma.cuh"

namespace kvc {
namespace {

constexpr int kPairRows = 128;     // rows of one row tile
constexpr int kPairTile = 128;     // cached tokens per tile
constexpr int kPairThreads = 384;  // three warpgroups: softmax A, softmax B, and {issuing warp, copy warp, two idle warps}
// Registers: 384 threads leave 168 per thread; the third warpgroup gives most of its share to the softmax
// threads, which hold a row's 128 scores at once (setmaxnreg, per warpgroup: 2 x 128 x 224 + 128 x 56 = 64512).
constexpr int kPairSoftmaxRegs = 224;
constexpr int kPairOtherRegs = 56;
constexpr uint32_t kPairTmemCols = 512;
constexpr uint32_t kColO = 0;    // O_A, O_B: 128 columns each
constexpr uint32_t kColX = 256;  // the scores of the row tile whose turn it is: 128 columns
constexpr uint32_t kColP = 384;  // P_A, P_B: 64 columns each (two 16-bit probabilities per column)

template <int HEAD>
struct PairCfg {
  static_assert(HEAD == 64 || HEAD == 128, "head size 64 or 128");
  static constexpr int D = HEAD;
  static constexpr int kHalves = D / 64;             // 64-element (128-byte) operand tiles per row
  static constexpr int kHalfBytes = 128 * 128;       // 128 rows x 64 sixteen-bit elements: 16 KB
  static constexpr int kTileBytes = kHalves * kHalfBytes;  // a Q row tile, a K tile or a V tile
  static constexpr int kOffQ = 0;                    // [row tile]
  static constexpr int kOffK = 2 * kTileBytes;       // [stage]
  static constexpr int kOffV = 4 * kTileBytes;       // [stage]
  static constexpr int kOffStage = 6 * kTileBytes;   // one row tile of results on its way out
  static constexpr int kOffBar = 7 * kTileBytes;     // mbarriers, tensor-memory slot, abort word
  static constexpr int kBarriers = 24;
  static constexpr int kUsedBytes = kOffBar + kBarriers * 8 + 16;  // + tensor-memory slot and abort word
  // One CTA per SM, whatever the head size: a CTA allocates all of the SM's tensor memory, and a second CTA on
  // the same SM would wait for the first to end while another SM stays empty.  Asking for more than half of an
  // SM's shared memory makes that impossible.
  static constexpr int kSmemBytes = kUsedBytes > 120 * 1024 ? kUsedBytes : 120 * 1024;
  static_assert(kSmemBytes + 1024 <= 232448, "fits one SM");
  static_assert(2 * (kSmemBytes + 1024) > 233472, "one CTA per SM");
};

// one box of a tiled 4-d tensor map -> shared memory of this CTA; completion is counted in bytes on `bar`
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2,
                                            int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(umma::smem_addr(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(umma::smem_addr(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
// one box of shared memory -> a tiled 3-d tensor map (rows outside the tensor are not written); asynchronous,
// tracked by the issuing thread's bulk group
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(src), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit_and_wait_read() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(umma::smem_addr(bar)), "r"(bytes) : "memory");
}
template <int N>
__device__ __forceinline__ void warpgroup_take_registers() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void warpgroup_give_registers() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

// explicit shared-space accesses (a generic pointer would go through the slower generic path)
__device__ __forceinline__ void st_shared_v4(uint32_t addr, const uint4& v) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}

// A wait that ignores the abort word (used only to let copies in flight land before the CTA ends): at most
// `tries` tries of about 20 us.
__device__ __forceinline__ bool mbar_wait_limited(uint64_t* bar, uint32_t parity, uint32_t tries) {
  for (uint32_t i = 0; i < tries; ++i)
    if (umma::mbar_try_wait(bar, parity, umma::kTryNs)) return true;
  return false;
}

// The item a CTA takes in round `round`: items are numbered heaviest first and the CTAs walk them in a
// serpentine -- forwards in even rounds, backwards in odd ones -- so that the CTA that got the heaviest item of
// one round gets the lightest of the next and all CTAs end up with nearly the same amount of work.
__device__ __forceinline__ int pair_item_of(int round, int num_items) {
  const int g = static_cast<int>(gridDim.x), c = static_cast<int>(blockIdx.x);
  (void)num_items;
  return round * g + ((round & 1) ? g - 1 - c : c);
}

// What one work item is: the pair of row tiles `pair` of (sequence, kv head), its rows and the range of
// key/value tiles it walks.
struct PairItem {
  int seq, kvh, row0;     // row0: first row of row tile A within the (sequence, kv head)
  int q_start, q_len, n;  // first query token, query tokens and cached tokens of the sequence
  int rows_all;           // rows of both tiles: A is full before B has any
  int tile_begin, nt;     // first tile and number of tiles
  bool has_b;
};

// S = Q_g K^T into the score columns: D / 16 instructions (M 128, N 128, K 16), both operands K-major in shared
// memory with the 128-byte swizzle.  Built where it is used (the issuing warp and the softmax threads), so that
// the roles that never issue it keep no registers for it.
template <typename T16, int D, typename Cfg>
struct PairScoresIssuer {
  static constexpr uint32_t kIdesc = umma::instr_desc_f16<T16>(kPairRows, 128, false, false);
  static constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);  // SBO 1024, version 1, 128-byte swizzle
  static constexpr uint32_t kLbo = (16u >> 4) << 16;                            // K-major operands: unused
  uint32_t q_lo, k_lo0, x_col;
  __device__ __forceinline__ PairScoresIssuer(const unsigned char* s_q, const unsigned char* s_k, uint32_t x)
      : q_lo((umma::smem_addr(s_q) >> 4) | kLbo), k_lo0((umma::smem_addr(s_k) >> 4) | kLbo), x_col(x) {}
  __device__ __forceinline__ void operator()(int g, int k_slot) const {
    const uint32_t qa = q_lo + g * (Cfg::kTileBytes >> 4);
    const uint32_t kb = k_lo0 + k_slot * (Cfg::kTileBytes >> 4);
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      const uint32_t step = ((kk >> 2) * Cfg::kHalfBytes + (kk & 3) * 32) >> 4;
      umma::mma_f16_ss(x_col, (static_cast<uint64_t>(kDescHi) << 32) | (qa + step),
                       (static_cast<uint64_t>(kDescHi) << 32) | (kb + step), kIdesc, kk > 0 ? 1u : 0u);
    }
  }
};

template <typename TQ, int KV, int HEAD>
__global__ void __launch_bounds__(kPairThreads, 1)
    paged_prefill_pair_kernel(const DecodeParams p, const __grid_constant__ CUtensorMap tmap_k,
                              const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_q,
                              const __grid_constant__ CUtensorMap tmap_o, const int q_by_tma, const int o_by_tma,
                              const int num_seqs, const int num_items) {
  using Cfg = PairCfg<HEAD>;
  static_assert(KV == KVC_KV_AUTO || HEAD == 128, "fp8 caches: head size 128 (a raw row is one 128-byte line)");
  using namespace umma;
  constexpr int D = Cfg::D, TN = kPairTile;
  // fp8 caches: the copy warp brings a tile's raw rows (128 bytes each) into the upper half of the tile's slot,
  // warps 10 and 11 widen them to fp16 (exact) in the swizzled operand layout, and the products run in fp16
  // (a bf16 query is converted on its way into shared memory); k_descale folds into the softmax scale,
  // v_descale into the output.
  constexpr bool kFp8 = KV != KVC_KV_AUTO;
  using T16 = std::conditional_t<kFp8, __half, TQ>;  // operand type of the matrix products
  constexpr bool kConvQ = !std::is_same_v<TQ, T16>;  // a bf16 query that arrived by TMA is converted in place

  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* s_q = smem + Cfg::kOffQ;
  unsigned char* s_k = smem + Cfg::kOffK;
  unsigned char* s_v = smem + Cfg::kOffV;
  unsigned char* s_stage = smem + Cfg::kOffStage;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kOffBar);
  uint64_t* bar_s = bars;          // [row tile]  S(j) of the row tile is complete
  uint64_t* bar_ready = bars + 2;  // [row tile]  its 128 softmax threads have stored P(j)
  uint64_t* bar_o = bars + 4;      // [row tile]  O += P(j) V(j) is complete
  uint64_t* bar_kfull = bars + 6;  // [stage]     the K tile has landed
  uint64_t* bar_vfull = bars + 8;
  uint64_t* bar_kfree = bars + 10;  // [stage]    every product that reads the K tile is complete
  uint64_t* bar_vfree = bars + 12;
  uint64_t* bar_xfree = bars + 14;  // the row tile A has read its scores out of X into registers (128 arrivals)
  uint64_t* bar_xfree_b = bars + 23;  // ... the row tile B
  uint64_t* bar_qfull = bars + 15;  // the query rows have landed (when they come by TMA)
  uint64_t* bar_qfree = bars + 16;  // every product that reads the item's query rows is complete
  uint64_t* bar_stage = bars + 17;  // the staging tile has been read by the TMA unit (or written out by its warps)
  uint64_t* bar_kconv = bars + 18;  // [stage]  fp8 caches: the K tile has been widened to fp16 (64 arrivals)
  uint64_t* bar_vconv = bars + 20;
  uint64_t* bar_qconv = bars + 22;  // fp8 caches, bf16 queries: the query rows have been converted to fp16 (64 arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + Cfg::kBarriers);
  volatile uint32_t* abort_word = tmem_slot + 1;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 9 * 32) {  // the tensor maps are kernel parameters: fetching them does not depend on the predecessor
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_k)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_v)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_q)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_o)) : "memory");
  }
  pdl_prologue();

  if (smem_addr(smem) & 1023u) {  // the operand tiles' swizzle assumes 1024-byte alignment
    if (tid == 0) atomicMax(&g_umma_status, 2);
    return;
  }
  if (tid == 0) {
    *abort_word = 0;
    mbar_init(bar_s, 1);
    mbar_init(bar_s + 1, 1);
    mbar_init(bar_ready, kPairRows);
    mbar_init(bar_ready + 1, kPairRows);
    mbar_init(bar_o, 1);
    mbar_init(bar_o + 1, 1);
    for (int i = 0; i < 8; ++i) mbar_init(bar_kfull + i, 1);  // kfull, vfull, kfree, vfree
    mbar_init(bar_xfree, kPairRows);
    mbar_init(bar_xfree_b, kPairRows);
    mbar_init(bar_qfull, 1);
    mbar_init(bar_qfree, 1);
    mbar_init(bar_stage, 1);
    for (int i = 0; i < 4; ++i) mbar_init(bar_kconv + i, 64);  // kconv, vconv
    mbar_init(bar_qconv, 64);
    mbar_init_fence();
  }
  if (warp == 0) tmem_alloc(tmem_slot, kPairTmemCols);
  fence_before_thread_sync();
  __syncthreads();
  fence_after_thread_sync();
  const uint32_t tmem = *tmem_slot;

  // rows are token-major: row R of the kv head is token R / group, head R % group of the group
  const int g_shift = (p.group & (p.group - 1)) == 0 ? __ffs(p.group) - 1 : -1;
  auto row_token = [&](int R) {
    if (g_shift >= 0) return R >> g_shift;
    return R / p.group;
  };
  auto row_head = [&](const PairItem& w, int R) {
    if (g_shift >= 0) return w.kvh * p.group + (R & (p.group - 1));
    return w.kvh * p.group + R % p.group;
  };
  auto row_limit = [&](const PairItem& w, int R) {
    const int pos = w.n - w.q_len + row_token(R);
    int hi = w.n;
    if (p.causal) hi = min(hi, pos + 1);
    if (p.window_right >= 0) hi = min(hi, pos + p.window_right + 1);
    return max(0, hi);
  };
  auto row_lo = [&](const PairItem& w, int R) {
    return p.window_left >= 0 ? max(0, w.n - w.q_len + row_token(R) - p.window_left) : 0;
  };

  // ---- what a work item covers; false when it has no work for the matrix products (each role decides this by
  // itself, from the same numbers).  Items are numbered heaviest first: the last pair of row tiles of every
  // sequence and kv head, then the pair before it, and so on.
  // The three numbers of an item's sequence are fetched one item ahead (`fetch` at the top of the item before),
  // so that their latency is not paid between two items.
  struct SeqNumbers {
    int q_start, q_end, n;
  };
  const int per_pair = num_seqs * p.num_kv_heads;
  auto fetch = [&](int item) -> SeqNumbers {
    SeqNumbers f{0, 0, 0};
    if (item < num_items) {
      const int seq = (item % per_pair) / p.num_kv_heads;
      f.q_start = p.cu_seqlens_q ? __ldg(p.cu_seqlens_q + seq) : seq;
      f.q_end = p.cu_seqlens_q ? __ldg(p.cu_seqlens_q + seq + 1) : seq + 1;
      f.n = __ldg(p.seq_lens + seq);
    }
    return f;
  };
  auto setup = [&](int item, const SeqNumbers& f, PairItem& w) -> bool {
    const int pair = p.row_tiles - 1 - item / per_pair;
    const int rem = item - (item / per_pair) * per_pair;
    w.seq = rem / p.num_kv_heads;
    w.kvh = rem - w.seq * p.num_kv_heads;
    w.row0 = pair * 2 * kPairRows;
    w.q_start = f.q_start;
    w.q_len = f.q_end - f.q_start;
    w.nt = 0;
    w.rows_all = 0;
    const int seq_rows = w.q_len * p.group;
    if (seq_rows <= kRows || w.row0 >= seq_rows) return false;  // the decode kernel's sequence, or no rows here
    w.rows_all = min(2 * kPairRows, seq_rows - w.row0);
    w.has_b = w.rows_all > kPairRows;
    w.n = f.n;
    // both ends grow with the row: the CTA walks from its first row's start to its last row's end
    const int tile_end = (row_limit(w, w.row0 + w.rows_all - 1) + TN - 1) / TN;
    w.tile_begin = row_lo(w, w.row0) / TN;
    w.nt = tile_end - w.tile_begin;
    return w.nt > 0;
  };
  // The barriers run on across items: tile `it` of an item is phase (tiles of the role's earlier items + it) of
  // the per-tile barriers, and so on.  The roles never meet between items, so the copy warp and the issuing warp
  // start on the next item while the softmax threads still write the last one's results.
  int tiles_done = 0;    // tiles of earlier items (row tile A takes part in every item)
  int tiles_done_b = 0;  // ... of earlier items that had a row tile B
  int items_done = 0;    // earlier items with work
  int stages_done = 0;   // uses of the staging tile by earlier items (one per row tile)
  bool prev_had_b = false;  // the item before had a row tile B
  auto account = [&](const PairItem& w) {
    stages_done += w.has_b ? 2 : 1;
    tiles_done += w.nt;
    if (w.has_b) tiles_done_b += w.nt;
    ++items_done;
    prev_had_b = w.has_b;
  };

  auto kfull_of = [&](int j) { return (kFp8 ? bar_kconv : bar_kfull) + ((tiles_done + j) & 1); };
  auto kfree_of = [&](int j) { return bar_kfree + ((tiles_done + j) & 1); };
  auto stage_parity = [&](int j) { return static_cast<uint32_t>((tiles_done + j) >> 1) & 1u; };
  // Use u of an item's score columns is S_A(u / groups) or, with two row tiles, S_B for odd u.  After the batch:
  // the row tile's scores barrier; after a tile's last batch its K slot is free; after the item's last the query.
  auto issue_use = [&](const PairScoresIssuer<T16, D, Cfg>& issue_qk, const PairItem& w, int g, int j) {
    issue_qk(g, (tiles_done + j) & 1);
    mma_commit(bar_s + g);
    if (g == (w.has_b ? 1 : 0)) {
      mma_commit(kfree_of(j));
      if (j == w.nt - 1) mma_commit(bar_qfree);
    }
  };

  if (warp >= 8) {
    warpgroup_give_registers<kPairOtherRegs>();
    PairItem w;
    SeqNumbers next = fetch(pair_item_of(0, num_items));
    for (int round = 0; round * static_cast<int>(gridDim.x) < num_items; ++round) {
      const int item = pair_item_of(round, num_items);
      const SeqNumbers cur = next;
      next = fetch(pair_item_of(round + 1, num_items));
      if (item >= num_items || !setup(item, cur, w)) continue;
      if (!q_by_tma && warp == 8) named_bar_sync(1, 9 * 32);  // the softmax warps have gathered the query rows
      if (warp == 9) {
        // ====================================================================================== copy warp
        if (q_by_tma) {
          // A row tile is a box of the query tensor [token][head][d] -- 128 / group tokens x group heads x 64
          // elements, rows in exactly the token-major order of the tile (rows past the tensor's end arrive as
          // zeros, rows of a following sequence are computed and never stored).
          const int tokens_per_tile = kPairRows >> g_shift;  // 128 / group
          if (items_done > 0) mbar_wait_bounded(bar_qfree, static_cast<uint32_t>(items_done - 1) & 1u, abort_word);
          if (lane == 0) mbar_arrive_expect_tx(bar_qfull, 2u * Cfg::kTileBytes);
          __syncwarp();
          if (lane < 2 * Cfg::kHalves)  // row tile lane / halves, half lane % halves
            tma_load_3d(smem_addr(s_q) + (lane / Cfg::kHalves) * Cfg::kTileBytes + (lane % Cfg::kHalves) * Cfg::kHalfBytes,
                        &tmap_q, bar_qfull, (lane % Cfg::kHalves) * 64, w.kvh * p.group,
                        w.q_start + (w.row0 >> g_shift) + (lane / Cfg::kHalves) * tokens_per_tile);
        }
        // A tile is 128 tokens: one box of 128 rows when a cache block holds at least 128 tokens, else 128 / bs
        // boxes of bs rows; every box exists twice, once per 64-element half of the head dimension.  Lane l
        // issues box l / 2, half l % 2.  Blocks that start at or beyond the sequence's end are not fetched.
        // fp8 caches: a box is box_rows raw rows of 128 bytes, one per tile and block, in the slot's upper half.
        const int32_t* table = p.block_table + w.seq * p.block_table_stride;
        const int box_rows = min(p.block_size, TN);
        const int ops = (TN / box_rows) * (kFp8 ? 1 : Cfg::kHalves);
        const uint32_t box_bytes = static_cast<uint32_t>(box_rows) * 128u;
        const int b = kFp8 ? lane : lane / Cfg::kHalves, half = kFp8 ? 1 : lane % Cfg::kHalves;
        auto load_tile = [&](int tile, const CUtensorMap* map, unsigned char* slot, uint64_t* full) {
          const int token0 = tile * TN + b * box_rows;
          const bool valid = lane < ops && token0 < w.n;
          const unsigned mask = __ballot_sync(0xFFFFFFFFu, valid);
          if (lane == 0) mbar_arrive_expect_tx(full, static_cast<uint32_t>(__popc(mask)) * box_bytes);
          __syncwarp();
          if (valid) {
            const int32_t blk = __ldg(table + (token0 >> p.bs_shift));
            tma_load_4d(smem_addr(slot) + half * Cfg::kHalfBytes + b * box_bytes, map, full, kFp8 ? 0 : half * 64, w.kvh,
                        token0 & (p.block_size - 1), blk);
          }
        };
        for (int j = 0; j < w.nt; ++j) {
          const int kt = tiles_done + j;  // the CTA's kt-th tile: stage kt & 1, that stage's use kt >> 1
          const int s = kt & 1;
          const uint32_t prev_use = static_cast<uint32_t>((kt >> 1) - 1) & 1u;
          if (kt >= 2) mbar_wait_bounded(bar_kfree + s, prev_use, abort_word);
          load_tile(w.tile_begin + j, &tmap_k, s_k + s * Cfg::kTileBytes, bar_kfull + s);
          if (kt >= 2) mbar_wait_bounded(bar_vfree + s, prev_use, abort_word);
          load_tile(w.tile_begin + j, &tmap_v, s_v + s * Cfg::kTileBytes, bar_vfull + s);
        }
        if (*abort_word) {  // something gave up: let the copies that are still in flight land before going on
          if (q_by_tma) mbar_wait_limited(bar_qfull, static_cast<uint32_t>(items_done) & 1u, 1000);
          for (int j = max(0, w.nt - 2); j < w.nt; ++j) {
            const int kt = tiles_done + j;
            mbar_wait_limited(bar_kfull + (kt & 1), (kt >> 1) & 1, 1000);
            mbar_wait_limited(bar_vfull + (kt & 1), (kt >> 1) & 1, 1000);
          }
        }
      } else if (warp == 8) {
        // ====================================================================================== issuing warp
        const PairScoresIssuer<T16, D, Cfg> issue_qk(s_q, s_k, tmem + kColX);
        constexpr uint32_t kIdescPV = instr_desc_f16<T16>(kPairRows, D, false, true);
        constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);  // SBO 1024, version 1, 128-byte swizzle
        auto make_desc = [](uint32_t lo) { return (static_cast<uint64_t>(kDescHi) << 32) | lo; };
        constexpr uint32_t kLboV = (static_cast<uint32_t>(Cfg::kHalfBytes) >> 4) << 16;  // V: distance of the D halves
        const uint32_t v_lo0 = (smem_addr(s_v) >> 4) | kLboV;
        auto issue_pv = [&](int g, int j) {  // O_g (+)= P_g(j) V(j): P_g is 64 columns of two 16-bit values
          const uint32_t vb = v_lo0 + ((tiles_done + j) & 1) * (Cfg::kTileBytes >> 4);
#pragma unroll
          for (int kk = 0; kk < TN / 16; ++kk)
            mma_f16_ts(tmem + kColO + g * 128, tmem + kColP + g * 64 + kk * 8, make_desc(vb + ((kk * 16 * 128) >> 4)),
                       kIdescPV, (j > 0 || kk > 0) ? 1u : 0u);
        };
        // Uses of the score columns X are numbered in issue order: with both row tiles use 2j is S_A(j) and use
        // 2j + 1 is S_B(j).  This warp issues an item's first use, once the threads of the use before it (the last
        // of the item before) have read their scores (bar_xfree); every later use is issued by a thread of the row
        // tile that has just taken its scores out of X, so that the chain X is handed along -- read, next batch,
        // read -- has one sleeping waiter per link instead of two.  S_g(j + 1) is thereby computed while the
        // softmax of S_g(j) is still running, and this warp's own waits are those of the second product alone.
        const int groups = w.has_b ? 2 : 1;
        if (q_by_tma) mbar_wait_bounded(kConvQ ? bar_qconv : bar_qfull, static_cast<uint32_t>(items_done) & 1u, abort_word);
        mbar_wait_bounded(kfull_of(0), stage_parity(0), abort_word);
        // the last use of X before this item: the last tile of the item before, by its row tile B if it had one
        if (items_done > 0)
          mbar_wait_bounded(prev_had_b ? bar_xfree_b : bar_xfree,
                            static_cast<uint32_t>((prev_had_b ? tiles_done_b : tiles_done) - 1) & 1u, abort_word);
        fence_after_thread_sync();
        if (lane == 0) issue_use(issue_qk, w, 0, 0);
        __syncwarp();
        for (int j = 0; j < w.nt; ++j) {
          const int s = (tiles_done + j) & 1;
          for (int g = 0; g < groups; ++g) {
            // O_g += P_g(j) V(j)
            if (g == 0) {
              mbar_wait_bounded((kFp8 ? bar_vconv : bar_vfull) + s, stage_parity(j), abort_word);
              const int valid_rows = w.n - (w.tile_begin + j) * TN;  // rows of the tile that hold tokens of the sequence
              if (valid_rows < TN) {
                unsigned char* v = s_v + s * Cfg::kTileBytes;
                const int first = max(valid_rows, 0);
                for (int i = lane; i < (TN - first) * (D / 8); i += 32) {  // 8 chunks per row and half
                  const int r = first + i / (D / 8), c = i % (D / 8);
                  *reinterpret_cast<uint4*>(v + (c >> 3) * Cfg::kHalfBytes + r * 128 + (c & 7) * 16) = make_uint4(0, 0, 0, 0);
                }
                fence_smem_to_async_proxy();
                __syncwarp();
              }
            }
            // the row tile's 128 threads have stored P(j).  16-bit caches: a named barrier they only arrive at (this
            // warp is released about 250 cycles sooner than an mbarrier wakes it); fp8 caches measured 4 % slower
            // that way (the thread that issues the scores makes its warp a late arriver) and keep the mbarrier.
            if constexpr (!kFp8)
              named_bar_sync(7 + g, kPairRows + 32);
            else
              mbar_wait_bounded(bar_ready + g, static_cast<uint32_t>((g == 0 ? tiles_done : tiles_done_b) + j) & 1u,
                                abort_word);
            fence_after_thread_sync();
            if (lane == 0) {
              issue_pv(g, j);
              mma_commit(bar_o + g);
              if (g == groups - 1) mma_commit(bar_vfree + s);
            }
            __syncwarp();
          }
        }
      } else if (!kFp8 && warp >= 10) {
        // ====================================================================================== scores issuers
        // 16-bit caches.  Warp 10 follows the reads of row tile A, warp 11 those of row tile B: when the row
        // tile's 128 threads have their scores in registers, it issues the item's next use of X -- S_B(it) after
        // S_A(it), S_A(it + 1) after S_B(it) (alone: S_A(it + 1) after S_A(it)).  A named barrier hands over: the
        // softmax warps arrive and go on, this warp is released with the last of them.
        const int g = warp - 10;
        if (g == 0 || w.has_b) {
          const PairScoresIssuer<T16, D, Cfg> issue_qk(s_q, s_k, tmem + kColX);
          for (int it = 0; it < w.nt; ++it) {
            const int ng = w.has_b ? g ^ 1 : 0;
            const int nj = (w.has_b && g == 0) ? it : it + 1;
            if (nj >= w.nt) break;
            if (nj != it) mbar_wait_bounded(kfull_of(nj), stage_parity(nj), abort_word);  // a new key tile: long there
            named_bar_sync(5 + g, kPairRows + 32);
            fence_after_thread_sync();
            if (lane == 0) issue_use(issue_qk, w, ng, nj);
            __syncwarp();
          }
        }
      } else if (kFp8 && D == 128 && warp >= 10) {
        // ====================================================================================== widening warps
        // Warps 10 and 11, 64 threads.  A tile's 128 raw rows are widened in two phases of 64 rows: a warp reads
        // 4 rows x 8 sixteen-byte chunks per instruction (512 contiguous bytes), every thread holds 8 chunks,
        // the 64 threads meet (everything a store of this phase can overwrite has been read: raw row r lies on
        // the bytes of row r of the second D half), then each chunk becomes two swizzled fp16 chunks.
        const int cw = warp - 10;
        auto widen = [&](unsigned char* slot) {
          const unsigned char* raw = slot + Cfg::kHalfBytes;
#pragma unroll 1
          for (int ph = 0; ph < 2; ++ph) {
            uint4 c[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int row = ph * 64 + cw * 32 + 4 * i + (lane >> 3);
              c[i] = *reinterpret_cast<const uint4*>(raw + row * 128 + (lane & 7) * 16);
            }
            named_bar_sync(4, 64);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int row = ph * 64 + cw * 32 + 4 * i + (lane >> 3), ch = lane & 7;  // raw chunk: d = 16 ch ..
              const uint32_t src[4] = {c[i].x, c[i].y, c[i].z, c[i].w};
              uint4 lo, hi;
              lo.x = fp8x2_to_f16x2<kFp8 ? KV : KVC_KV_FP8_E4M3>(src[0]);
              lo.y = fp8x2_to_f16x2<kFp8 ? KV : KVC_KV_FP8_E4M3>(src[0] >> 16);
              lo.z = fp8x2_to_f16x2<kFp8 ? KV : KVC_KV_FP8_E4M3>(src[1]);
              lo.w = fp8x2_to_f16x2<kFp8 ? KV : KVC_KV_FP8_E4M3>(src[1] >> 16);
              hi.x = fp8x2_to_f16x2<kFp8 ? KV : KVC_KV_FP8_E4M3>(src[2]);
              hi.y = fp8x2_to_f16x2<kFp8 ? KV : KVC_KV_FP8_E4M3>(src[2] >> 16);
              hi.z = fp8x2_to_f16x2<kFp8 ? KV : KVC_KV_FP8_E4M3>(src[3]);
              hi.w = fp8x2_to_f16x2<kFp8 ? KV : KVC_KV_FP8_E4M3>(src[3] >> 16);
              unsigned char* dst = slot + (ch >> 2) * Cfg::kHalfBytes;  // fp16 chunks 2 ch, 2 ch + 1 of the row
              *reinterpret_cast<uint4*>(dst + swizzled_offset(row, (2 * ch) & 7)) = lo;
              *reinterpret_cast<uint4*>(dst + swizzled_offset(row, (2 * ch + 1) & 7)) = hi;
            }
          }
        };
        if (kConvQ && q_by_tma) {  // the item's query rows, bf16 as they came: to fp16, element for element in place
          mbar_wait_bounded(bar_qfull, static_cast<uint32_t>(items_done) & 1u, abort_word);
          const int t64 = cw * 32 + lane;
#pragma unroll 4
          for (int i = 0; i < 2 * Cfg::kTileBytes / 16 / 64; ++i) {
            uint4* cell = reinterpret_cast<uint4*>(s_q) + i * 64 + t64;
            uint4 v = *cell;
            uint32_t* wq = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const float lo = __uint_as_float(wq[k] << 16), hi = __uint_as_float(wq[k] & 0xFFFF0000u);
              wq[k] = pack2<__half>(lo, hi);
            }
            *cell = v;
          }
          fence_smem_to_async_proxy();
          mbar_arrive(bar_qconv);
        }
        for (int j = 0; j < w.nt; ++j) {
          const int kt = tiles_done + j, s = kt & 1;
          const uint32_t par = static_cast<uint32_t>(kt >> 1) & 1u;
          mbar_wait_bounded(bar_kfull + s, par, abort_word);
          widen(s_k + s * Cfg::kTileBytes);
          fence_smem_to_async_proxy();
          mbar_arrive(bar_kconv + s);
          mbar_wait_bounded(bar_vfull + s, par, abort_word);
          widen(s_v + s * Cfg::kTileBytes);
          fence_smem_to_async_proxy();
          mbar_arrive(bar_vconv + s);
        }
      }
      account(w);
    }
  } else {
    warpgroup_take_registers<kPairSoftmaxRegs>();
    PairItem w;
    SeqNumbers next = fetch(pair_item_of(0, num_items));
    for (int round = 0; round * static_cast<int>(gridDim.x) < num_items; ++round) {
      const int item = pair_item_of(round, num_items);
      const SeqNumbers cur = next;
      next = fetch(pair_item_of(round + 1, num_items));
      if (item >= num_items) continue;
      if (!setup(item, cur, w)) {
        // rows that see no token at all (a window that ends before the cache begins): zeros
        for (int i = tid; i < w.rows_all * D; i += 8 * 32) {
          const int R = w.row0 + i / D;
          static_cast<TQ*>(p.out)[static_cast<int64_t>(w.q_start + row_token(R)) * p.out_stride_t +
                                  row_head(w, R) * p.out_stride_h + i % D] = TQ(0.0f);
        }
        continue;
      }
      if (!q_by_tma) {
        // Odd group sizes: the softmax warps gather the query rows of both row tiles (zero rows past the end).
        // All of a thread's loads are issued before its first store, so that the rows are fetched at memory
        // latency once, not once per 16-byte piece.
        constexpr int kQThreads = 256, kPerThread = 2 * kPairRows * (D / 8) / kQThreads;  // 16 pieces of 16 bytes
        if (items_done > 0) mbar_wait_bounded(bar_qfree, static_cast<uint32_t>(items_done - 1) & 1u, abort_word);
        uint4 piece[kPerThread];
#pragma unroll
        for (int i = 0; i < kPerThread; ++i) {
          const int c = tid + i * kQThreads;
          const int r = c / (D / 8), col = c % (D / 8);  // r: row of the pair, 0..255
          piece[i] = make_uint4(0, 0, 0, 0);
          if (r < w.rows_all) {
            const int R = w.row0 + r;
            piece[i] = *reinterpret_cast<const uint4*>(static_cast<const TQ*>(p.query) +
                                                       static_cast<int64_t>(w.q_start + row_token(R)) * p.query_stride_t +
                                                       row_head(w, R) * p.query_stride_h + col * 8);
            if constexpr (!std::is_same_v<TQ, T16>) {  // bf16 query over an fp8 cache: the products run in fp16
              uint32_t* wq = reinterpret_cast<uint32_t*>(&piece[i]);
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const float lo = __uint_as_float(wq[k] << 16), hi = __uint_as_float(wq[k] & 0xFFFF0000u);
                wq[k] = pack2<__half>(lo, hi);
              }
            }
          }
        }
#pragma unroll
        for (int i = 0; i < kPerThread; ++i) {
          const int c = tid + i * kQThreads;
          const int r = c / (D / 8), col = c % (D / 8);
          *reinterpret_cast<uint4*>(s_q + (r >> 7) * Cfg::kTileBytes + (col >> 3) * Cfg::kHalfBytes +
                                    swizzled_offset(r & 127, col & 7)) = piece[i];
        }
        fence_smem_to_async_proxy();
        named_bar_sync(1, 9 * 32);  // with the issuing warp, which reads Q through the async proxy after this
      }
      if (warp < 4 || w.has_b) {
        // ====================================================================================== softmax warps
        const int g = warp >> 2;  // row tile
        const int r = tid & 127;  // row of the tile = tensor-memory lane
        const int rows_g = g == 0 ? min(w.rows_all, kPairRows) : w.rows_all - kPairRows;
        const int Rg0 = w.row0 + g * kPairRows;
        const bool live = r < rows_g;
        const int lim = live ? row_limit(w, Rg0 + r) : 0;
        const int lo = live ? row_lo(w, Rg0 + r) : 0;
        const int lim_min = row_limit(w, Rg0);
        const int lo_max = row_lo(w, Rg0 + rows_g - 1);
        const float scale2 = p.softmax_scale * kLog2e * ((kFp8 && p.k_descale) ? __ldg(p.k_descale) : 1.0f);
        const float lazy_margin = 8.0f / scale2;
        const uint32_t t_lanes = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);  // this warp's 32 lanes
        const uint32_t t_x = t_lanes + kColX, t_p = t_lanes + kColP + g * 64, t_o = t_lanes + kColO + g * 128;
        float m_run = -INFINITY, l_run = 0.f;
        const int phase0 = g == 0 ? tiles_done : tiles_done_b;  // this row tile's earlier tiles

        for (int it = 0; it < w.nt; ++it) {
          const int tile = w.tile_begin + it;
          mbar_wait_bounded(bar_s + g, static_cast<uint32_t>(phase0 + it) & 1u, abort_word);
          fence_after_thread_sync();
          uint32_t sa[4][32];
#pragma unroll
          for (int c = 0; c < 4; ++c) tmem_ld_32x32(t_x + c * 32, sa[c]);
          tmem_ld_wait();
          fence_before_thread_sync();
          mbar_arrive(g == 0 ? bar_xfree : bar_xfree_b);  // the scores are in registers: the next use of X may begin
          {
            // the item's next use of X, if it has one: S_B(it) after S_A(it), S_A(it + 1) after S_B(it) (alone: S_A(it + 1))
            const int ng = w.has_b ? g ^ 1 : 0;
            const int nj = (w.has_b && g == 0) ? it : it + 1;
            if (nj < w.nt) {
              if constexpr (!kFp8) {
                // 16-bit caches: warp 10 + g, idle otherwise, sleeps on this named barrier and issues the batch the
                // moment the row tile's four warps have reported (which costs them one instruction)
                asm volatile("bar.arrive %0, %1;" ::"r"(5 + g), "r"(kPairRows + 32) : "memory");
              } else {
                // fp8 caches (warps 10 and 11 widen): one of the row tile's threads issues it.  Its warp stands
                // still for the 1 100 cycles in which the tensor pipe takes the eight instructions.
                named_bar_sync(5 + g, kPairRows);  // all 128 threads of the row tile have their scores
                if (r == 0) {
                  if (nj != it) mbar_wait_bounded(kfull_of(nj), stage_parity(nj), abort_word);  // a new key tile
                  fence_after_thread_sync();
                  issue_use(PairScoresIssuer<T16, D, Cfg>(s_q, s_k, tmem + kColX), w, ng, nj);
                }
              }
            }
          }
          if ((tile + 1) * TN > lim_min || tile * TN < lo_max) {  // some row of the tile has tokens to mask here
            const int tok0 = tile * TN;
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (tok0 + c * 32 + i >= lim || tok0 + c * 32 + i < lo) sa[c][i] = 0xFF800000u;  // -inf
          }
          float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int i = 0; i < 32; i += 2)
              mx4[(i >> 1) & 3] = max3(mx4[(i >> 1) & 3], __uint_as_float(sa[c][i]), __uint_as_float(sa[c][i + 1]));
          const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
          // the reference point of the exponentials follows the maximum lazily: it moves only when a score exceeds
          // it by more than 2^8 after scaling, so probabilities stay below 256 and O is rescaled a few times per row
          const bool move = mx > m_run + lazy_margin;
          const float alpha = move ? fast_exp2((m_run - mx) * scale2) : 1.0f;
          m_run = move ? mx : m_run;
          const float neg_ms = (m_run == -INFINITY) ? 0.f : -m_run * scale2;
          l_run *= alpha;
          // O += P(it - 1) V(it - 1) must be complete before O is rescaled or P's columns are overwritten.  That
          // product was issued when this row tile reported P(it - 1).  16-bit caches: the 128 scores first become 64
          // words of two 16-bit probabilities in the registers the scores leave -- nothing in that touches tensor
          // memory -- and the wait comes last (asked for before the exponentials it cost the row tile 290 cycles
          // per tile, and the row tile's own time is what a step waits for there).  fp8 caches measured 3 % slower
          // that way and wait first, storing each half of P as it is complete.
          auto wait_for_previous_product = [&]() {
            if (it > 0) {
              mbar_wait_bounded(bar_o + g, static_cast<uint32_t>(phase0 + it - 1) & 1u, abort_word);
              fence_after_thread_sync();
            }
            if (it > 0 && __any_sync(0xFFFFFFFFu, alpha != 1.0f)) {  // rare: a reference maximum of the warp moved
#pragma unroll 1
              for (int c = 0; c < D / 32; ++c) {
                uint32_t o[32];
                tmem_ld_32x32(t_o + c * 32, o);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                tmem_st_32x32(t_o + c * 32, o);
              }
            }
          };
          if constexpr (kFp8) wait_for_previous_product();
          const float2 sc2 = make_float2(scale2, scale2), nm2 = make_float2(neg_ms, neg_ms);
          float2 l_add[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
          uint32_t wd[2][32];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int cc = 0; cc < 2; ++cc)
#pragma unroll
              for (int i = 0; i < 32; i += 2) {
                const int c = 2 * h + cc;
                const float2 e = __ffma2_rn(make_float2(__uint_as_float(sa[c][i]), __uint_as_float(sa[c][i + 1])), sc2, nm2);
                const float2 pr = make_float2(fast_exp2(e.x), fast_exp2(e.y));
                l_add[(i >> 1) & 3] = __fadd2_rn(l_add[(i >> 1) & 3], pr);
                wd[h][cc * 16 + (i >> 1)] = pack2<T16>(pr.x, pr.y);
              }
            if constexpr (kFp8) tmem_st_32x32(t_p + h * 32, wd[h]);
          }
          if constexpr (!kFp8) {
            wait_for_previous_product();
            tmem_st_32x32(t_p, wd[0]);
            tmem_st_32x32(t_p + 32, wd[1]);
          }
          l_run += ((l_add[0].x + l_add[0].y) + (l_add[1].x + l_add[1].y)) +
                   ((l_add[2].x + l_add[2].y) + (l_add[3].x + l_add[3].y));
          tmem_st_wait();
          fence_before_thread_sync();
          if constexpr (!kFp8)
            asm volatile("bar.arrive %0, %1;" ::"r"(7 + g), "r"(kPairRows + 32) : "memory");
          else
            mbar_arrive(bar_ready + g);
        }
        const bool finished = mbar_wait_bounded(bar_o + g, static_cast<uint32_t>(phase0 + w.nt - 1) & 1u, abort_word);
        fence_after_thread_sync();
        if (!finished && lane == 0) atomicMax(&g_umma_status, 1);

        // ---- the row's result -------------------------------------------------------------------------------
        const int R = Rg0 + r;
        const int head = live ? row_head(w, R) : 0;
        const float m = m_run * scale2;  // log2 domain; -inf if the row saw nothing
        float l = l_run, rescale = 1.0f;
        if (p.sink && live) {
          const float sk = static_cast<float>(static_cast<const TQ*>(p.sink)[head]) * kLog2e;
          const float mf = fmaxf(m, sk);
          rescale = (m == -INFINITY) ? 0.f : exp2f(m - mf);
          l = l * rescale + exp2f(sk - mf);
        }
        const float f = (l > 0.f) ? rescale / l * ((kFp8 && p.v_descale) ? __ldg(p.v_descale) : 1.0f) : 0.f;
        // The row goes to global memory through the staging tile, which the two row tiles use in turn (use
        // stages_done + g; a use may begin when the one before it has been read out).  A full row tile is one box
        // of the output tensor, as it was of the query tensor: every thread stages its row in that layout and one
        // thread hands the tile to the TMA unit (two stores, one per 64-element half), which writes it while the
        // threads go on to the next item.  A tile that the sequence's end cuts short (a box would reach into the
        // next sequence's rows), odd group sizes and unaligned outputs take the second path: each thread stages
        // its own 256-byte row, 16-byte pieces swizzled against bank conflicts, and the warp writes its 32 rows two
        // at a time, 512 contiguous bytes per instruction where consecutive heads of a token are adjacent.
        const int stage_use = stages_done + g;
        if (stage_use > 0) mbar_wait_bounded(bar_stage, static_cast<uint32_t>(stage_use - 1) & 1u, abort_word);
        if (o_by_tma && rows_g == kPairRows) {  // uniform over the row tile's 128 threads
          const uint32_t tile = smem_addr(s_stage);
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t acc[32];
            tmem_ld_32x32(t_o + c * 32, acc);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 v;
              v.x = pack2<TQ>(__uint_as_float(acc[8 * i]) * f, __uint_as_float(acc[8 * i + 1]) * f);
              v.y = pack2<TQ>(__uint_as_float(acc[8 * i + 2]) * f, __uint_as_float(acc[8 * i + 3]) * f);
              v.z = pack2<TQ>(__uint_as_float(acc[8 * i + 4]) * f, __uint_as_float(acc[8 * i + 5]) * f);
              v.w = pack2<TQ>(__uint_as_float(acc[8 * i + 6]) * f, __uint_as_float(acc[8 * i + 7]) * f);
              const int chunk = c * 4 + i;  // 16-byte chunk of the row: half chunk / 8
              st_shared_v4(tile + (chunk >> 3) * Cfg::kHalfBytes + swizzled_offset(r, chunk & 7), v);
            }
          }
          fence_smem_to_async_proxy();
          named_bar_sync(2 + g, kPairRows);
          if (r == 0) {
            const int tok0 = w.q_start + (Rg0 >> g_shift);
#pragma unroll
            for (int h = 0; h < Cfg::kHalves; ++h)
              tma_store_3d(&tmap_o, tile + h * Cfg::kHalfBytes, h * 64, w.kvh * p.group, tok0);
            tma_store_commit_and_wait_read();  // shared memory has been read; the writes complete on their own
            mbar_arrive(bar_stage);
          }
        } else {
          constexpr int kRowBytes = D * 2, kPieces = D / 8, kRowsPerStore = 32 / kPieces;
          const uint32_t stage = smem_addr(s_stage) + (warp & 3) * 32 * kRowBytes;  // this warp's 32 rows
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t acc[32];
            tmem_ld_32x32(t_o + c * 32, acc);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 v;
              v.x = pack2<TQ>(__uint_as_float(acc[8 * i]) * f, __uint_as_float(acc[8 * i + 1]) * f);
              v.y = pack2<TQ>(__uint_as_float(acc[8 * i + 2]) * f, __uint_as_float(acc[8 * i + 3]) * f);
              v.z = pack2<TQ>(__uint_as_float(acc[8 * i + 4]) * f, __uint_as_float(acc[8 * i + 5]) * f);
              v.w = pack2<TQ>(__uint_as_float(acc[8 * i + 6]) * f, __uint_as_float(acc[8 * i + 7]) * f);
              st_shared_v4(stage + lane * kRowBytes + (((c * 4 + i) ^ (lane & (kPieces - 1))) << 4), v);
            }
          }
          __syncwarp();
          const bool vec16 = ((reinterpret_cast<uintptr_t>(p.out) | static_cast<uintptr_t>(p.out_stride_t * 2) |
                               static_cast<uintptr_t>(p.out_stride_h * 2)) & 15u) == 0;
          // (token, head) of the lane's first row once, then kRowsPerStore rows further per step: no division in the loop
          const int piece = lane % kPieces;  // 16-byte piece of the row
          int rr = lane / kPieces;           // row of the warp
          int tok_r = row_token(Rg0 + (warp & 3) * 32 + rr);
          int head_r = Rg0 + (warp & 3) * 32 + rr - tok_r * p.group;  // head within the group
#pragma unroll 4
          for (int i = 0; i < 32 / kRowsPerStore; ++i, rr += kRowsPerStore) {
            if ((warp & 3) * 32 + rr < rows_g) {
              const uint4 v = ld_shared_v4(stage + rr * kRowBytes + ((piece ^ (rr & (kPieces - 1))) << 4));
              TQ* dst = static_cast<TQ*>(p.out) + static_cast<int64_t>(w.q_start + tok_r) * p.out_stride_t +
                        static_cast<int64_t>(w.kvh * p.group + head_r) * p.out_stride_h + piece * 8;
              if (vec16) {
                *reinterpret_cast<uint4*>(dst) = v;
              } else {
                uint32_t* d32 = reinterpret_cast<uint32_t*>(dst);
                d32[0] = v.x;
                d32[1] = v.y;
                d32[2] = v.z;
                d32[3] = v.w;
              }
            }
            head_r += kRowsPerStore;
            while (head_r >= p.group) {
              head_r -= p.group;
              ++tok_r;
            }
          }
          named_bar_sync(2 + g, kPairRows);  // all four warps have read their rows back
          if (r == 0) mbar_arrive(bar_stage);
        }
      }
      account(w);
    }
    // the output tiles this thread handed to the TMA unit have been written
    if ((tid & 127) == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }
  fence_before_thread_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kPairTmemCols);
}

}  // namespace
}  // namespace kvc
