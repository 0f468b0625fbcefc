// Fifth-generation tensor core (tcgen05) plumbing for sm_100a: tensor-memory allocation, shared-memory
// matrix descriptors, the instruction descriptor of kind::f16, MMA issue and commit, tensor-memory loads
// and stores, and mbarrier waits that give up after a bounded time.
//
// Shared-memory operand layout used throughout (the "128-byte swizzle" canonical layout): a tile is a
// stack of rows of 128 bytes (64 sixteen-bit elements); eight rows form a 1024-byte atom; inside an atom
// the 16-byte chunk c of row r is stored at chunk position c ^ (r & 7).  Tiles start on 1024-byte
// boundaries, so (r & 7) and the chunk position are address bits 7-9 and 4-6.  A matrix wider than 64
// elements is a sequence of such tiles ("halves" for 128 elements) at a fixed byte distance.
//
// The same bytes serve both operand roles:
//  * K-major (the contraction runs along the 128-byte rows: Q and K in Q K^T, P in P V): one MMA of
//    K = 16 consumes 32 bytes of every row; the descriptor is advanced by 32 bytes per step inside a
//    tile and by the tile distance between tiles.  SBO = 1024 (distance of 8-row groups); LBO unused.
//  * MN-major (the contraction runs down the rows: V in P V, N = head dimension): one MMA of K = 16
//    consumes 16 rows; the descriptor is advanced by 16 * 128 bytes per step.  SBO = 1024 (distance of
//    8-row groups along K), LBO = distance between the 64-element tiles along N.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <type_traits>

namespace kvc {
namespace umma {

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

// byte offset of 16-byte chunk `chunk` (0..7) of row `row` inside a tile of 128-byte rows
__device__ __forceinline__ uint32_t swizzled_offset(int row, int chunk) {
  return static_cast<uint32_t>(row) * 128u + (static_cast<uint32_t>(chunk ^ (row & 7)) << 4);
}

// ---- descriptors ---------------------------------------------------------------------------------
// Shared-memory matrix descriptor: start address >> 4 in bits [0,14), leading byte offset >> 4 in
// [16,30), stride byte offset >> 4 in [32,46), descriptor version 1 in [46,48), layout type in [61,64)
// (2 = 128-byte swizzle).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr >> 4) & 0x3FFFu);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;
  d |= 2ull << 61;
  return d;
}

// Instruction descriptor of tcgen05.mma kind::f16 with fp32 accumulation: accumulator format in [4,6)
// (1 = f32), A and B formats in [7,10) and [10,13) (0 = f16, 1 = bf16), A and B major-ness in bits 15 and
// 16 (0 = K-major, 1 = MN-major), N >> 3 in [17,23), M >> 4 in [24,29).
template <typename T16>
__host__ __device__ constexpr uint32_t instr_desc_f16(int m, int n, bool a_mn_major, bool b_mn_major) {
  const uint32_t fmt = std::is_same<T16, __nv_bfloat16>::value ? 1u : 0u;
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// the encodings the kernels here run with (checked on a B200 against a CPU product of the same operands)
static_assert(instr_desc_f16<__nv_bfloat16>(128, 64, false, false) == 0x08100490u, "S = Q K^T, bf16, M 128, N 64");
static_assert(instr_desc_f16<__nv_bfloat16>(128, 128, false, true) == 0x08210490u, "O += P V, bf16, V MN-major");
static_assert(instr_desc_f16<__half>(128, 128, false, true) == 0x08210010u, "O += P V, fp16, V MN-major");

// ---- tensor memory ---------------------------------------------------------------------------------
// Whole-warp calls.  `columns` is a power of two >= 32; the address of the allocation lands in *slot
// (shared memory).  The allocation blocks while the SM has fewer free columns than asked for, so a kernel
// must size its shared memory such that co-resident CTAs can never ask for more than 512 in total.
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(slot)), "r"(columns)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}

__device__ __forceinline__ void fence_before_thread_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_thread_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// makes this thread's earlier generic-proxy writes to shared memory visible to the async proxy (the MMA unit)
__device__ __forceinline__ void fence_smem_to_async_proxy() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem]; one thread issues
__device__ __forceinline__ void mma_f16_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]: A is M lanes x K 16-bit values, two per 32-bit column (K / 2 columns per
// instruction), lane = row
__device__ __forceinline__ void mma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n" ::"r"(tmem_d),
      "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// the mbarrier gets one arrival when every MMA this thread issued before has completed
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar))
               : "memory");
}

// 32 lanes x 32 columns of 32 bits: lane i of the warp gets columns [col, col + 32) of tensor-memory lane
// (warp's lane base + i).  `taddr` = (lane base << 16) | column.  Whole-warp calls.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---- mbarriers --------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(arrivals) : "memory");
}
__device__ __forceinline__ void mbar_inval(uint64_t* bar) {
  asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
// One bounded try: the hardware parks the thread until the phase with the given parity completes or a time
// limit of about `hint_ns` passes, whichever is first.
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t done;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(done)
      : "r"(smem_addr(bar)), "r"(parity), "r"(hint_ns)
      : "memory");
  return done != 0;
}
// Non-blocking test: has the phase with the given parity completed?  (A few cycles, where a try_wait costs about
// two hundred even when the phase is already complete.)
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(done)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return done != 0;
}
// Waits until the phase with the given parity has completed, for at most kMaxTries tries of about 20 us each:
// half a second in all, where a tile of work takes microseconds, so that a context that is switched out for a
// while on a shared GPU does not trip it.  Returns false when it gave up or when *abort is already set, and sets
// *abort (a shared-memory word of the CTA) so that every later wait of the CTA returns at once: the kernel then
// runs to its end on whatever it finds, frees its tensor memory and reports through its status word.
constexpr uint32_t kMaxTries = 25000;
constexpr uint32_t kTryNs = 20000;
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, volatile uint32_t* abort,
                                                  uint32_t max_tries = kMaxTries) {
  if (mbar_test_wait(bar, parity)) return true;  // the common case: what is waited for happened long ago
  for (uint32_t i = 0; i < max_tries; ++i) {
    if (mbar_try_wait(bar, parity, kTryNs)) return true;
    if (*abort) return false;
  }
  *abort = 1u;
  return false;
}

}  // namespace umma
}  // namespace kvc
