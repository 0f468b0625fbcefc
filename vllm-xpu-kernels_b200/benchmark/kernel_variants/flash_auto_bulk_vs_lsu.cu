// Stand-alone comparison for the UNQUANTISED flash-layout scatter (bf16 -> bf16, 2 KB rows):
// 256-bit LSU loads/stores (what the library does) against bulk asynchronous copies
// (cp.async.bulk global -> shared -> global) driven by one thread per CTA through a ring of stages.
// Not part of the library; it records the measurement behind the choice.  Plain CTA-local copies, no
// cluster launch; every mbarrier wait is bounded and reports through an error flag.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -lineinfo -o flash_auto_bulk_vs_lsu flash_auto_bulk_vs_lsu.cu
//   ./flash_auto_bulk_vs_lsu [num_tokens=16384]
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <vector>
#include <algorithm>
#include <random>
#include <cstring>

#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("CUDA error %s at %s:%d\n", cudaGetErrorString(e), __FILE__, __LINE__); exit(1);} } while (0)

constexpr int ROW = 1024;  // elements per token row (bf16)
constexpr int ROWB = ROW * 2;
constexpr int BS = 64;

struct P { const uint16_t* key; const uint16_t* value; uint16_t* kc; uint16_t* vc; const int64_t* slots; int T; int* err; };

__device__ __forceinline__ void ld32(const void* p, uint4& a, uint4& b) {
  asm volatile("ld.global.nc.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];" : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w), "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w) : "l"(p)); }
__device__ __forceinline__ void st32(void* p, uint4 a, uint4 b) {
  asm volatile("st.global.v8.u32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" :: "l"(p), "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w) : "memory"); }

// LSU: thread = 32 bytes of K and of V
__global__ void __launch_bounds__(256) kLsu(const P p) {
  const uint32_t item = blockIdx.x * 256 + threadIdx.x; const uint32_t tok = item >> 6, c = item & 63;
  if (tok >= p.T) return;
  asm volatile("griddepcontrol.wait;" ::: "memory"); asm volatile("griddepcontrol.launch_dependents;");
  const int64_t slot = __ldg(p.slots + tok); if (slot < 0) return;
  uint4 k0, k1, v0, v1;
  ld32(p.key + (size_t)tok * ROW + c * 16, k0, k1); ld32(p.value + (size_t)tok * ROW + c * 16, v0, v1);
  st32(p.kc + (size_t)slot * ROW + c * 16, k0, k1); st32(p.vc + (size_t)slot * ROW + c * 16, v0, v1);
}

// bulk: one thread per CTA drives a ring of STAGES stages (K row + V row each)
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
template <int STAGES>
__global__ void __launch_bounds__(32) kBulk(const P p) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t full[STAGES];
  if (threadIdx.x != 0) return;
  for (int s = 0; s < STAGES; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(smem_u32(&full[s])));
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory"); asm volatile("griddepcontrol.launch_dependents;");
  const int stride = gridDim.x;
  int n = 0; for (int t = blockIdx.x; t < p.T; t += stride) ++n;
  // prologue: fill the ring
  int issued = 0, done = 0;
  auto issue = [&](int i) {
    const int t = blockIdx.x + i * stride; const int s = i % STAGES;
    const int64_t slot = __ldg(p.slots + t);
    const uint32_t bar = smem_u32(&full[s]); const uint32_t dst = smem_u32(smem + (size_t)s * 2 * ROWB);
    if (slot < 0) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory"); return; }
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(2 * ROWB) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" :: "r"(dst), "l"(p.key + (size_t)t * ROW), "r"(ROWB), "r"(bar) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" :: "r"(dst + ROWB), "l"(p.value + (size_t)t * ROW), "r"(ROWB), "r"(bar) : "memory");
  };
  for (; issued < n && issued < STAGES; ++issued) issue(issued);
  for (done = 0; done < n; ++done) {
    const int s = done % STAGES; const uint32_t parity = (done / STAGES) & 1; const uint32_t bar = smem_u32(&full[s]);
    uint32_t ok = 0; int spins = 0;
    while (!ok) {
      asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
      if (!ok && ++spins > (1 << 22)) { atomicExch(p.err, 1); goto out; }  // bounded wait
    }
    {
      const int t = blockIdx.x + done * stride; const int64_t slot = __ldg(p.slots + t);
      if (slot >= 0) {
        const uint32_t src = smem_u32(smem + (size_t)s * 2 * ROWB);
        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" :: "l"(p.kc + (size_t)slot * ROW), "r"(src), "r"(ROWB) : "memory");
        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" :: "l"(p.vc + (size_t)slot * ROW), "r"(src + ROWB), "r"(ROWB) : "memory");
      }
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    }
    if (issued < n) {
      // the stage to refill is the one just stored: its smem must have been read by the store first
      asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
      issue(issued); ++issued;
    }
  }
out:
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

template <typename K>
static void launch_pdl(K kern, int grid, int threads, size_t smem, const P& p, cudaStream_t s) {
  cudaLaunchConfig_t cfg = {}; cfg.gridDim = dim3(grid); cfg.blockDim = dim3(threads); cfg.stream = s; cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute at[1]; at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = 1; CK(cudaLaunchKernelEx(&cfg, kern, p));
}

int main(int argc, char** argv) {
  const int T = argc > 1 ? atoi(argv[1]) : 16384;
  const int NB = 8192, NBUF = 8, GS = 64, REPS = 16;
  const size_t cache_elems = (size_t)NB * BS * ROW;
  uint16_t *kc, *vc, *kc_ref; CK(cudaMalloc(&kc, cache_elems * 2)); CK(cudaMalloc(&vc, cache_elems * 2)); CK(cudaMalloc(&kc_ref, cache_elems * 2));
  int* err; CK(cudaMalloc(&err, 4)); CK(cudaMemset(err, 0, 4));
  std::mt19937_64 rng(3); std::vector<P> ps(NBUF); std::vector<uint16_t> h((size_t)T * ROW);
  for (int b = 0; b < NBUF; ++b) {
    uint16_t *dk, *dv; int64_t* ds; CK(cudaMalloc(&dk, h.size() * 2)); CK(cudaMalloc(&dv, h.size() * 2)); CK(cudaMalloc(&ds, (size_t)T * 8));
    for (auto& x : h) x = (uint16_t)rng(); CK(cudaMemcpy(dk, h.data(), h.size() * 2, cudaMemcpyHostToDevice));
    for (auto& x : h) x = (uint16_t)rng(); CK(cudaMemcpy(dv, h.data(), h.size() * 2, cudaMemcpyHostToDevice));
    std::vector<int64_t> blocks(NB); for (int i = 0; i < NB; ++i) blocks[i] = i; std::shuffle(blocks.begin(), blocks.end(), rng);
    std::vector<int64_t> slots(T); for (int t = 0; t < T; ++t) slots[t] = blocks[t / BS] * BS + t % BS;
    CK(cudaMemcpy(ds, slots.data(), (size_t)T * 8, cudaMemcpyHostToDevice));
    ps[b] = P{dk, dv, kc, vc, ds, T, err};
  }
  int nsm = 148; cudaDeviceGetAttribute(&nsm, cudaDevAttrMultiProcessorCount, 0);
  cudaStream_t st; CK(cudaStreamCreate(&st));
  const double bytes = 8.0 * T + (double)T * ROW * 2 * 4;
  CK(cudaFuncSetAttribute(kBulk<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 2 * ROWB));
  CK(cudaFuncSetAttribute(kBulk<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * 2 * ROWB));
  CK(cudaFuncSetAttribute(kBulk<12>, cudaFuncAttributeMaxDynamicSharedMemorySize, 12 * 2 * ROWB));
  struct V { const char* name; void (*launch)(const P&, cudaStream_t, int); };
  std::vector<V> vars = {
    {"LSU 256-bit ld/st", [](const P& p, cudaStream_t s, int) { launch_pdl(kLsu, (p.T * 64 + 255) / 256, 256, 0, p, s); }},
    {"bulk 4 stages x6/SM", [](const P& p, cudaStream_t s, int n) { launch_pdl(kBulk<4>, n * 6, 32, 4 * 2 * ROWB, p, s); }},
    {"bulk 8 stages x4/SM", [](const P& p, cudaStream_t s, int n) { launch_pdl(kBulk<8>, n * 4, 32, 8 * 2 * ROWB, p, s); }},
    {"bulk 8 stages x6/SM", [](const P& p, cudaStream_t s, int n) { launch_pdl(kBulk<8>, n * 6, 32, 8 * 2 * ROWB, p, s); }},
    {"bulk 12 stages x4/SM", [](const P& p, cudaStream_t s, int n) { launch_pdl(kBulk<12>, n * 4, 32, 12 * 2 * ROWB, p, s); }},
    {"bulk 4 stages x12/SM", [](const P& p, cudaStream_t s, int n) { launch_pdl(kBulk<4>, n * 12, 32, 4 * 2 * ROWB, p, s); }},
  };
  { P r = ps[0]; r.kc = kc_ref; vars[0].launch(r, st, nsm); CK(cudaStreamSynchronize(st)); }
  std::vector<uint8_t> ref((size_t)BS * ROWB), got((size_t)BS * ROWB);
  for (auto& v : vars) {
    CK(cudaMemsetAsync(kc, 0, cache_elems * 2, st));
    v.launch(ps[0], st, nsm); CK(cudaStreamSynchronize(st)); CK(cudaGetLastError());
    int64_t slot0; CK(cudaMemcpy(&slot0, ps[0].slots, 8, cudaMemcpyDeviceToHost));
    size_t off = (size_t)(slot0 / BS) * BS * ROW;
    CK(cudaMemcpy(ref.data(), kc_ref + off, ref.size(), cudaMemcpyDeviceToHost)); CK(cudaMemcpy(got.data(), kc + off, got.size(), cudaMemcpyDeviceToHost));
    bool same = memcmp(ref.data(), got.data(), ref.size()) == 0;
    cudaGraph_t g; cudaGraphExec_t ge;
    CK(cudaStreamBeginCapture(st, cudaStreamCaptureModeGlobal));
    for (int i = 0; i < GS; ++i) v.launch(ps[i % NBUF], st, nsm);
    CK(cudaStreamEndCapture(st, &g)); CK(cudaGraphInstantiate(&ge, g, 0));
    for (int i = 0; i < 3; ++i) CK(cudaGraphLaunch(ge, st));
    cudaEvent_t e0, e1; CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1)); float best = 1e9;
    for (int rep = 0; rep < 5; ++rep) {
      CK(cudaEventRecord(e0, st)); for (int i = 0; i < REPS; ++i) CK(cudaGraphLaunch(ge, st)); CK(cudaEventRecord(e1, st)); CK(cudaStreamSynchronize(st));
      float ms; CK(cudaEventElapsedTime(&ms, e0, e1)); best = std::min(best, ms);
    }
    int herr = 0; CK(cudaMemcpy(&herr, err, 4, cudaMemcpyDeviceToHost));
    const double us = best * 1e3 / (GS * REPS);
    printf("%-24s %s err=%d  %.2f us/launch (%.0f GB/s)\n", v.name, same ? "ok  " : "DIFF", herr, us, bytes / us / 1e3);
    CK(cudaGraphExecDestroy(ge)); CK(cudaGraphDestroy(g));
  }
  return 0;
}
