#!/usr/bin/env python
"""Benchmark of the KV-cache write path: reshape_and_cache_flash, bf16 -> fp8_e4m3.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]
                    [--workload C4|C2|C3|C5-fp8|C5-bf16|C1|<op>] [--scaling weak|strong]

One step = one call of the op over one batch (the "C4" batch by default: 16384 tokens,
8 KV heads x 128, cache of 65536 blocks x 64 slots, fp8_e4m3 store, slots in runs of 64).
Prints ONE JSON line (rank 0).  Fields beyond the usual ones:

  value / ms_per_step   K steps replayed from CUDA graphs with inputs resident in HBM, timed
                        with CUDA events on the launching stream, max over ranks
  roofline              algorithmic bytes per launch / average launch duration, against the
                        measured HBM copy bandwidth in MEASURED_PEAKS.json
  e2e                   same metric through the C ABI's host-buffer entry point: every step
                        copies key, value and slot_mapping from pinned host memory, runs the
                        kernel and reads two written cache rows back
  cpu_baseline          the CPU oracle (a C port of the reference's algorithm, all host
                        threads) on a bounded sample of the same batch -- reported, never a target
  clocks                SM clock / throttle reasons sampled through NVML during the timed region

Under torchrun every rank runs the same per-rank batch on its own GPU and cache slice
("weak": the model has 8 KV heads per GPU, no rank needs another rank's data), or, with
--scaling strong, the batch's 8 heads are divided over the ranks.  There is no collective
on the data path; NCCL only carries the barrier and the max-over-ranks of the times.

--impl reference times the CPU oracle alone (rank 0 only), in the same units.

The ops around the cache write have workloads of their own, measured and reported the same way
(--workload mla-fp8 | gather | quant-static | quant-token | rope | rope-cache-fp8 | decode-bf16 |
decode-fp8 | prefill-bf16 | prefill-fp8 | ...; sizes in benchmark/op_workloads.py).  The default single-GPU C4 line
carries a short figure of each of them under "ops" (and of the metric's other configurations under "also").  Their e2e figure moves the step's inputs from pinned
host memory through torch copies, calls the C ABI and reads the step's result back.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import statistics
import sys
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
PKG_ROOT = os.path.join(REPO, "vllm-xpu-kernels_b200")
for _p in (REPO, PKG_ROOT, os.path.join(PKG_ROOT, "benchmark")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

import op_workloads  # noqa: E402
import workloads  # noqa: E402

NBUF = 8            # distinct input sets rotated through, so inputs come from HBM, not L2
GRAPH_STEPS = 64    # steps captured per CUDA graph


# --------------------------------------------------------------------------------------------
# helpers
# --------------------------------------------------------------------------------------------
def measured_tensor_peak() -> tuple[float, str]:
    """Dense bf16 TFLOP/s of a library GEMM run alone on this pool (burst figure), else the stated fallback."""
    try:
        with open(os.path.join(REPO, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["bf16_tflops"]), "measured"
    except Exception:
        return 1590.0, "fallback"


def measured_peaks() -> tuple[float, str]:
    path = os.path.join(REPO, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only) in a thread."""

    REASONS = {
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
        0x80: "hw_power_brake", 0x2: "applications_clocks_setting", 0x100: "display_clock_setting",
    }

    def __init__(self, index: int, period_s: float = 0.004):
        self.samples: list[tuple[int, int, float]] = []
        self.sm_max = None
        self._stop = threading.Event()
        self._thr = None
        self._h = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            # NVML enumerates physical GPUs; honour CUDA_VISIBLE_DEVICES when it lists indices
            vis = os.environ.get("CUDA_VISIBLE_DEVICES", "")
            phys = index
            if vis:
                ids = [v.strip() for v in vis.split(",") if v.strip()]
                if index < len(ids) and ids[index].isdigit():
                    phys = int(ids[index])
            self._h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.sm_max = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._h = None
        self._period = period_s

    def _loop(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                clk = int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                rs = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)) if hasattr(
                    nv, "nvmlDeviceGetCurrentClocksEventReasons") else int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h))
                pw = nv.nvmlDeviceGetPowerUsage(self._h) / 1000.0
                self.samples.append((clk, rs, pw))
            except Exception:
                pass
            self._stop.wait(self._period)

    def start(self):
        if self._h is not None:
            self._thr = threading.Thread(target=self._loop, daemon=True)
            self._thr.start()

    def stop(self) -> dict:
        if self._thr is not None:
            self._stop.set()
            self._thr.join()
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": [], "samples": 0}
        clks = [s[0] for s in self.samples]
        bits = 0
        for s in self.samples:
            bits |= s[1]
        reasons = sorted(name for bit, name in self.REASONS.items() if bits & bit)
        return {"sm_mhz": statistics.median(clks), "sm_max_mhz": self.sm_max, "reasons": reasons,
                "samples": len(clks), "power_w_max": round(max(s[2] for s in self.samples), 1)}


class LibraryChatterToStderr:
    """Points file descriptor 1 at stderr while libraries initialise (NCCL prints a version banner
    on stdout), so that stdout carries the JSON line and nothing else; C stdio is flushed before
    the descriptor is restored."""

    def __enter__(self):
        sys.stdout.flush()
        self._saved = os.dup(1)
        os.dup2(2, 1)
        return self

    def __exit__(self, *exc):
        import ctypes
        sys.stdout.flush()
        try:
            ctypes.CDLL(None).fflush(None)
        except Exception:
            pass
        os.dup2(self._saved, 1)
        os.close(self._saved)
        return False


def dist_setup(n_gpus: int):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        return dist, rank, world, local
    if n_gpus > 1:
        raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    return None, 0, 1, 0


def barrier(dist):
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(dist, v: float, device="cuda") -> float:
    if dist is None:
        return v
    t = torch.tensor([v], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(dist, v: float, device="cuda") -> float:
    if dist is None:
        return v
    t = torch.tensor([v], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def host_threads() -> int:
    """Threads for the CPU legs: every core this process may run on (torchrun presets
    OMP_NUM_THREADS=1, which the explicit thread count overrides)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def make_batch_sets(name: str, rank: int, world: int, scaling: str, nbuf: int | None, tokens: int | None = None):
    """Independent batches of the named workload for this rank (CPU tensors).  ``tokens`` resizes the C4
    batch (size studies only; the named configuration is the default).

    Replicated job: ``nbuf`` batches.  Head-sharded job: ``nbuf * world`` sets, so that a rank's rotating
    inputs stay as large as the whole batch's (several times L2) although each set is ``world`` times
    smaller: set j is the slice of batch ``j % nbuf`` that holds heads of rank ``(rank + j // nbuf) %
    world`` -- the rank's own heads for the first ``nbuf`` sets, other ranks' rows of the same batch (same
    shape, same slots, same scales) as further distinct inputs after that."""
    def make(variant: int):
        if tokens is not None and name == "C4":
            return workloads.c4(variant=variant, num_tokens=tokens)
        return workloads.BY_NAME[name](variant=variant)

    if nbuf is None:  # enough sets for about 512 MB of inputs, between NBUF and 64
        first = make(0)
        per_set = first.key.numel() * first.key.element_size() * 2
        nbuf = max(NBUF, min(64, -(-(512 << 20) // per_set)))
    if scaling != "strong":
        return [make(b + 100 * rank) for b in range(nbuf)]
    batches = [make(b) for b in range(nbuf)]
    sets = []
    for j in range(nbuf * world):
        w = workloads.shard_heads(batches[j % nbuf], (rank + j // nbuf) % world, world)
        if world > 1:  # a rank holds its heads only, packed
            w = dataclasses.replace(w, key=w.key.contiguous(), value=w.value.contiguous())
        sets.append(w)
    return sets


# --------------------------------------------------------------------------------------------
# CPU oracle timing (cpu_baseline leg and --impl reference)
# --------------------------------------------------------------------------------------------
def cpu_oracle_pass(w, tokens: int | None = None, host_blocks: int = 4096):
    """(run, T, blocks, threads): ``run()`` is one pass of the CPU oracle over (a prefix of) batch ``w``.
    The host cache keeps the batch's layout, block size and row shape but only ``host_blocks`` blocks, so
    that it fits in ordinary host memory; the tokens' blocks are renumbered into it, runs of slots intact."""
    import oracle
    from oracle import torch_views as H  # numpy views of torch tensors

    T = w.num_tokens if tokens is None else min(tokens, w.num_tokens)
    key, value = w.key[:T].contiguous(), w.value[:T].contiguous()
    slots = w.slot_mapping[:T].clone()
    bs = w.block_size
    act = slots >= 0
    uniq, inv = torch.unique(torch.div(slots[act], bs, rounding_mode="floor"), return_inverse=True)
    host_blocks = max(host_blocks, int(uniq.numel()))
    slots[act] = inv * bs + slots[act] % bs
    cdt = torch.uint8 if w.kv_cache_dtype != "auto" else key.dtype
    if w.layout == "flash":
        kc = torch.zeros(host_blocks, bs, w.num_heads, w.head_size, dtype=cdt)
        vc = torch.zeros_like(kc)
        fn = oracle.reshape_and_cache_flash
    else:
        x = 16 // torch.empty((), dtype=cdt).element_size()
        kc = torch.zeros(host_blocks, w.num_heads, w.head_size // x, bs, x, dtype=cdt)
        vc = torch.zeros(host_blocks, w.num_heads, w.head_size, bs, dtype=cdt)
        fn = oracle.reshape_and_cache
    threads = host_threads()
    args = (H.as_np(key), H.as_np(value), H.as_np(kc), H.as_np(vc), slots.numpy(), w.kv_cache_dtype,
            float(w.k_scale), float(w.v_scale), H.ORC_IN[key.dtype])

    def run() -> None:
        fn(*args, threads=threads)

    return run, T, host_blocks, threads


def cpu_oracle_rate(w, budget_s: float, tokens: int | None = None):
    """tokens/s of the CPU oracle on (a prefix of) batch ``w``, measured for about ``budget_s`` seconds."""
    run, T, _, threads = cpu_oracle_pass(w, tokens)
    run()  # warm-up: page in, spin up the thread pool
    n, t0 = 0, time.perf_counter()
    while True:
        run()
        n += 1
        dt = time.perf_counter() - t0
        if dt >= budget_s and n >= 3:
            break
    return T * n / dt, threads, T, n, dt


def cpu_torch_loop_rate(w, budget_s: float, host_blocks: int = 4096):
    """tokens/s of the reference's own CPU statement of the op: the per-token torch loop of its tests
    (oracle/torch_reference.py), same bounded sample as ``cpu_oracle_pass``."""
    from oracle import torch_reference

    T = w.num_tokens
    key, value = w.key.contiguous(), w.value.contiguous()
    slots = w.slot_mapping.clone()
    bs = w.block_size
    act = slots >= 0
    uniq, inv = torch.unique(torch.div(slots[act], bs, rounding_mode="floor"), return_inverse=True)
    host_blocks = max(host_blocks, int(uniq.numel()))
    slots[act] = inv * bs + slots[act] % bs
    cdt = w.cache_dtype
    raw = torch.uint8 if cdt != key.dtype else cdt
    if w.layout == "flash":
        kc = torch.zeros(host_blocks, bs, w.num_heads, w.head_size, dtype=raw)
        vc = torch.zeros_like(kc)
        fn = torch_reference.reshape_and_cache_flash
    else:
        x = 16 // torch.empty((), dtype=cdt).element_size()
        kc = torch.zeros(host_blocks, w.num_heads, w.head_size // x, bs, x, dtype=raw)
        vc = torch.zeros(host_blocks, w.num_heads, w.head_size, bs, dtype=raw)
        fn = torch_reference.reshape_and_cache
    if cdt != key.dtype:
        kc, vc = kc.view(cdt), vc.view(cdt)
    torch.set_num_threads(host_threads())
    args = (key, value, kc, vc, slots, w.kv_cache_dtype, float(w.k_scale), float(w.v_scale))
    fn(*args)
    n, t0 = 0, time.perf_counter()
    while True:
        fn(*args)
        n += 1
        dt = time.perf_counter() - t0
        if dt >= budget_s:
            break
    return T * n / dt, torch.get_num_threads(), n, dt


def run_reference_arm(ns) -> None:
    """--impl reference: the CPU implementation of the path alone, same metric and config."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    w = workloads.BY_NAME[ns.workload](variant=0)
    # size the per-step sample so that warmup + steps end within about two minutes
    rate0, threads, _, _, _ = cpu_oracle_rate(w, 2.0)
    per_step = int(max(64, min(w.num_tokens, rate0 * 100.0 / max(1, ns.steps + ns.warmup))))
    per_step -= per_step % w.block_size
    per_step = max(w.block_size, per_step)
    run, T, blocks, threads = cpu_oracle_pass(w, per_step)
    for _ in range(ns.warmup):
        run()
    t0 = time.perf_counter()
    for _ in range(ns.steps):
        run()
    dt = time.perf_counter() - t0
    value_tps = T * ns.steps / dt
    sample = (f"{T} of the batch's {w.num_tokens} tokens per step into a {blocks}-block host cache, "
              f"{ns.steps} steps, {threads} OpenMP threads")
    line = {
        "impl": "reference", "metric": metric_name(w), "value": value_tps, "unit": "tokens/s", "n_gpus": ns.gpus,
        "steps": ns.steps, "warmup": ns.warmup, "ms_per_step": dt / ns.steps * 1e3, "higher_is_better": True,
        "scaling": ns.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": describe_workload(w, ns.workload), "tokens_per_step": T},
        "cpu_baseline": {"value": value_tps, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value_tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def metric_name(w) -> str:
    """The headline metric for the fp8 flash workloads; the other layouts/modes name themselves."""
    op = "reshape_and_cache_flash" if w.layout == "flash" else "reshape_and_cache"
    return f"{op}_fp8_tokens_per_s" if w.kv_cache_dtype != "auto" else f"{op}_tokens_per_s"


def describe_workload(w, name: str) -> str:
    op = "reshape_and_cache_flash" if w.layout == "flash" else "reshape_and_cache"
    return (f"{name}: {op} {str(w.key.dtype).replace('torch.', '')}->{w.kv_cache_dtype}, "
            f"T={w.num_tokens} (active {w.num_active}), H={w.num_heads}, D={w.head_size}, "
            f"block_size={w.block_size}, num_blocks={w.num_blocks}")


# --------------------------------------------------------------------------------------------
# the B200 arm
# --------------------------------------------------------------------------------------------
def to_device_same_layout(t: torch.Tensor, dev, moved: dict) -> torch.Tensor:
    """``t`` on the device with the strides it has on the host.  A view (C5's key and value are slices
    of one fused qkv tensor) moves with the tensor it is a view of, once, so that the kernel meets the
    same row stride and the same neighbours in memory as the configuration describes; ``Tensor.to``
    alone would hand back a packed copy."""
    base = t._base
    if base is None or t.is_contiguous():
        return t.to(dev)
    if id(base) not in moved:
        moved[id(base)] = base.to(dev)
    return moved[id(base)].as_strided(t.shape, t.stride(), t.storage_offset())


class DeviceCase:
    """One cache-write workload resident on one GPU: its rotating input sets, the two caches, ``step(i)``."""

    def __init__(self, cabi, name: str, rank: int, world: int, scaling: str, dev, tokens: int | None = None,
                 nbuf: int | None = NBUF):
        self.cabi, self.name, self.dev = cabi, name, dev
        self.sets = make_batch_sets(name, rank, world, scaling, nbuf, tokens)
        w0 = self.w0 = self.sets[0]
        self.paged = w0.layout == "paged"
        ksh, vsh = w0.cache_shapes()
        cdt = w0.cache_dtype
        # torch.zeros: the allocation is touched once so first-use effects stay out of the timed region
        self.key_cache = torch.zeros(ksh, dtype=torch.uint8 if cdt != w0.key.dtype else cdt, device=dev)
        self.value_cache = torch.zeros(vsh, dtype=self.key_cache.dtype, device=dev)
        if cdt != w0.key.dtype:
            self.key_cache, self.value_cache = self.key_cache.view(cdt), self.value_cache.view(cdt)
        self.dsets = []
        for w in self.sets:
            moved: dict = {}
            self.dsets.append((to_device_same_layout(w.key, dev, moved), to_device_same_layout(w.value, dev, moved),
                               w.slot_mapping.to(dev), w.k_scale.to(dev), w.v_scale.to(dev)))
        self.in_bytes = sum(w.key.numel() * w.key.element_size() * 2 for w in self.sets)
        self.kv = w0.kv_cache_dtype

    def step(self, i: int) -> None:
        k, v, s, ks, vs = self.dsets[i % len(self.dsets)]
        if self.paged:
            self.cabi.reshape_and_cache(k, v, self.key_cache, self.value_cache, s, self.kv, ks, vs)
        else:
            self.cabi.reshape_and_cache_flash(k, v, self.key_cache, self.value_cache, s, self.kv, ks, vs)

    def rows_written(self, blk: torch.Tensor, off: torch.Tensor, key_cache, value_cache):
        """The cache rows at (block, offset) as [n, H*D] byte tensors, for either layout."""
        if self.paged:
            k = key_cache[blk, :, :, off]          # [n, H, D/x, x]
            v = value_cache[blk, :, :, off]        # [n, H, D]
        else:
            k, v = key_cache[blk, off], value_cache[blk, off]
        n = blk.numel()
        return k.contiguous().view(torch.uint8).reshape(n, -1), v.contiguous().view(torch.uint8).reshape(n, -1)

    def parity_rows(self, nrows: int = 64, which: int = 0) -> tuple[int, int]:
        """(rows compared, rows that differ): runs input set ``which`` once more, reads ``nrows`` of the
        cache rows it wrote and compares them byte for byte with what the CPU oracle writes for the same
        tokens (into a small host cache: token i of the sample goes to slot i)."""
        import oracle
        from oracle import torch_views as H

        w = self.sets[which]
        self.step(which)
        torch.cuda.synchronize()
        act = torch.nonzero(w.slot_mapping >= 0).flatten()
        if act.numel() == 0:
            return 0, 0
        g = torch.Generator().manual_seed(1234 + which)
        idx = act[torch.randperm(act.numel(), generator=g)[:nrows]].sort().values
        n, bs = int(idx.numel()), w.block_size
        key, value = w.key[idx].contiguous(), w.value[idx].contiguous()
        raw = torch.uint8 if w.cache_dtype != key.dtype else key.dtype
        hb = (n + bs - 1) // bs
        if self.paged:
            x = 16 // torch.empty((), dtype=w.cache_dtype).element_size()
            hk = torch.zeros(hb, w.num_heads, w.head_size // x, bs, x, dtype=raw)
            hv = torch.zeros(hb, w.num_heads, w.head_size, bs, dtype=raw)
            fn = oracle.reshape_and_cache
        else:
            hk = torch.zeros(hb, bs, w.num_heads, w.head_size, dtype=raw)
            hv = torch.zeros_like(hk)
            fn = oracle.reshape_and_cache_flash
        hs = torch.arange(n, dtype=torch.long)
        fn(H.as_np(key), H.as_np(value), H.as_np(hk), H.as_np(hv), hs.numpy(), w.kv_cache_dtype,
           float(w.k_scale), float(w.v_scale), H.ORC_IN[key.dtype], threads=1)
        ek, ev = self.rows_written(hs // bs, hs % bs, hk, hv)
        slots = w.slot_mapping[idx].to(self.dev)
        dk, dv = self.rows_written(slots // bs, slots % bs, self.key_cache, self.value_cache)
        bad = (dk.cpu() != ek).any(dim=1) | (dv.cpu() != ev).any(dim=1)
        return n, int(bad.sum())


def time_passes(step, steps: int, warmup: int, dist, local: int, min_region_s: float, nsets: int = NBUF) -> dict:
    """Times ``repeats`` passes of exactly ``steps`` steps each, back to back between one pair of CUDA
    events on the launching stream.  A pass is replayed from CUDA graphs (one graph when ``steps`` is at
    most GRAPH_STEPS); ``repeats`` is the smallest count that makes the timed region at least
    ``min_region_s`` long, found from two untimed passes and agreed over the ranks.  An event after
    every pass gives the spread between passes.  Successive graph replays continue the rotation over the
    ``nsets`` input sets where the previous one stopped (a graph is captured per starting set)."""
    def capture(n: int, start: int = 0):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(n):
                step(start + i)
        return g

    for i in range(nsets):  # eager warm-up before capture (module load, first touch)
        step(i)
    torch.cuda.synchronize()
    g_full = capture(GRAPH_STEPS) if steps >= GRAPH_STEPS or warmup >= GRAPH_STEPS else None
    rem = steps % GRAPH_STEPS
    # a short pass does not reach every input set: successive passes start where the last one stopped
    n_rem = 0 if not rem else (1 if steps >= GRAPH_STEPS else max(1, min(8, -(-nsets // rem))))
    g_rem = [capture(rem, k * rem) for k in range(n_rem)]
    g_wrem = capture(warmup % GRAPH_STEPS) if warmup % GRAPH_STEPS else None
    passes_done = [0]

    def one_pass() -> None:
        for _ in range(steps // GRAPH_STEPS):
            g_full.replay()
        if g_rem:
            g_rem[passes_done[0] % len(g_rem)].replay()
        passes_done[0] += 1

    for _ in range(warmup // GRAPH_STEPS):
        g_full.replay()
    if g_wrem is not None:
        g_wrem.replay()
    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    one_pass()
    c0.record()
    one_pass()
    one_pass()
    c1.record()
    torch.cuda.synchronize()
    est_pass_ms = max(max_over_ranks(dist, c0.elapsed_time(c1) / 2), 1e-4)
    repeats = max(1, min(100_000, int(min_region_s * 1e3 / est_pass_ms + 0.999)))

    sampler = ClockSampler(local)
    events = [torch.cuda.Event(enable_timing=True) for _ in range(repeats + 1)]
    barrier(dist)
    sampler.start()
    events[0].record()
    for r in range(repeats):
        one_pass()
        events[r + 1].record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    barrier(dist)
    own_ms = events[0].elapsed_time(events[repeats])
    per_pass = sorted(events[r].elapsed_time(events[r + 1]) / steps * 1e3 for r in range(repeats))
    return {
        "own_ms_per_step": own_ms / (repeats * steps),
        "ms_per_step": max_over_ranks(dist, own_ms) / (repeats * steps),
        "repeats": repeats, "launches": repeats * steps, "region_ms": own_ms, "clocks": clocks,
        "pass_us_per_step": {"min": per_pass[0], "median": per_pass[len(per_pass) // 2], "max": per_pass[-1]},
        "graphs": (f"a pass is one CUDA graph of {steps} launches ({len(g_rem)} such graph(s), each starting at the next input sets, "
                   f"taken in turn)" if steps < GRAPH_STEPS else f"CUDA graphs of {GRAPH_STEPS} launches"),
    }


def timing_note(t: dict, steps: int) -> str:
    return (f"{t['graphs']}, a pass of {steps} steps replayed {t['repeats']} times back to back between one pair "
            f"of CUDA events on the launching stream ({t['region_ms']:.0f} ms), after the warm-up steps and three "
            f"untimed passes; ms_per_step = region / (repeats * steps)")


def run_b200_arm(ns):
    from vllm_xpu_kernels import cabi  # raises if the CUDA library is not built

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path); use --impl reference for the CPU oracle")
    dist, rank, world, local = dist_setup(ns.gpus)
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    cabi.lib()
    peak, peak_src = measured_peaks()
    # --shard-of G on one GPU: this GPU runs the part rank 0 of G ranks would run
    shard_rank, shard_world = (rank, world) if ns.shard_of is None else (0, ns.shard_of)

    case = DeviceCase(cabi, ns.workload, shard_rank, shard_world, ns.scaling, dev, ns.tokens)
    sets, w0, paged, in_bytes = case.sets, case.w0, case.paged, case.in_bytes
    t = time_passes(case.step, ns.steps, ns.warmup, dist, local, ns.min_region_ms * 1e-3, len(case.dsets))
    ms_per_step = t["ms_per_step"]
    tokens_all = sum_over_ranks(dist, float(w0.num_tokens)) if ns.scaling == "weak" else float(w0.num_tokens)
    value = tokens_all / (ms_per_step * 1e-3)
    bytes_launch = w0.algorithmic_bytes()
    achieved = bytes_launch / (t["own_ms_per_step"] * 1e-3) / 1e9  # this rank's own kernel
    hbm_all = sum_over_ranks(dist, float(bytes_launch)) / (ms_per_step * 1e-3) / 1e9

    # single launches bracketed by their own events (eager), for the launch-latency picture
    singles = []
    for i in range(min(200, max(8, ns.steps))):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        case.step(i)
        b.record()
        singles.append((a, b))
    torch.cuda.synchronize()
    single_us = statistics.median(a.elapsed_time(b) for a, b in singles) * 1e3

    # ---------------------------------------------------------------- every rank checks bytes it wrote
    rows, bad = case.parity_rows(64, which=rank % NBUF)  # one of the rank's own-head sets
    parity = {"rows": int(sum_over_ranks(dist, float(rows))), "mismatches": int(sum_over_ranks(dist, float(bad))),
              "how": "64 cache rows per rank written by one more call, byte for byte against the CPU oracle"}

    # ---------------------------------------------------------------- end to end, host buffers
    key_cache, value_cache, dsets, kv = case.key_cache, case.value_cache, case.dsets, case.kv
    e2e_steps = max(1, min(ns.steps, 40))
    hsets = [(w.key.contiguous().pin_memory(), w.value.contiguous().pin_memory(), w.slot_mapping.pin_memory())
             for w in sets[:4]]
    last_slots = [int(w.slot_mapping[w.slot_mapping >= 0][-1]) for w in sets[:4]]
    if paged:
        # the paged op has no host-buffer entry point: copies go through torch, the call through the C ABI;
        # the step's result read back is the cache block (K and V) the last token was written into
        kflat = key_cache.view(torch.uint8).view(w0.num_blocks, -1)
        vflat = value_cache.view(torch.uint8).view(w0.num_blocks, -1)
        last_rows = [s // w0.block_size for s in last_slots]
        e2e_api = "pinned host tensors -> .to(device) -> kvc_reshape_and_cache"
    else:
        kflat = key_cache.view(torch.uint8).view(w0.num_blocks * w0.block_size, -1)
        vflat = value_cache.view(torch.uint8).view(w0.num_blocks * w0.block_size, -1)
        last_rows = last_slots
        e2e_api = "kvc_reshape_and_cache_flash_host (pinned host key/value/slot_mapping)"
    probes = [(torch.empty(kflat.shape[1], dtype=torch.uint8).pin_memory(),
               torch.empty(vflat.shape[1], dtype=torch.uint8).pin_memory()) for _ in range(4)]

    def e2e_step(i: int) -> None:
        j = i % 4
        hk, hv, hs = hsets[j]
        if paged:
            cabi.reshape_and_cache(hk.to(dev, non_blocking=True), hv.to(dev, non_blocking=True), key_cache, value_cache,
                                   hs.to(dev, non_blocking=True), kv, dsets[j][3], dsets[j][4])
        else:
            cabi.reshape_and_cache_flash_host(hk, hv, key_cache, value_cache, hs, kv, dsets[j][3], dsets[j][4])
        probes[j][0].copy_(kflat[last_rows[j]], non_blocking=True)  # the step's result, read back
        probes[j][1].copy_(vflat[last_rows[j]], non_blocking=True)

    for i in range(4):
        e2e_step(i)
    barrier(dist)
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        e2e_step(i)
    torch.cuda.synchronize()
    e2e_s = max_over_ranks(dist, time.perf_counter() - t0)
    barrier(dist)
    e2e_value = tokens_all * e2e_steps / e2e_s
    h2d = sets[0].key.numel() * sets[0].key.element_size() * 2 + sets[0].num_tokens * 8
    d2h = probes[0][0].numel() + probes[0][1].numel()
    if not paged:
        cabi.release_staging()
    launches = t["launches"]

    # ---------------------------------------------------------------- N > 1: the replicated job as well
    weak = None
    if world > 1 and ns.scaling == "strong" and not ns.no_also:
        del case, key_cache, value_cache, dsets, kflat, vflat
        torch.cuda.empty_cache()
        wcase = DeviceCase(cabi, ns.workload, rank, world, "weak", dev, ns.tokens)
        wt = time_passes(wcase.step, ns.steps, ns.warmup, dist, local, ns.min_region_ms * 1e-3 / 2)
        wtokens = sum_over_ranks(dist, float(wcase.w0.num_tokens))
        weak = {"value": wtokens / (wt["ms_per_step"] * 1e-3), "unit": "tokens/s", "ms_per_step": wt["ms_per_step"],
                "repeats": wt["repeats"],
                "what": f"every rank writes the whole batch ({wcase.w0.num_heads} KV heads) into a cache of its own"}
        launches += wt["launches"]
        del wcase

    # ---------------------------------------------------------------- N = 1: the metric's other configurations
    also = None
    if world == 1 and ns.workload == "C4" and ns.shard_of is None and ns.tokens is None and not ns.no_also:
        del case, key_cache, value_cache, dsets, kflat, vflat
        torch.cuda.empty_cache()
        also = {}
        for name in ("C2", "C5-fp8", "C5-bf16", "C3", "C1"):
            try:  # a secondary figure must not cost the headline its line
                c = DeviceCase(cabi, name, 0, 1, "weak", dev, nbuf=None)
                ct = time_passes(c.step, ns.steps, ns.warmup, None, local, 0.05, len(c.dsets))
                nbytes = c.w0.algorithmic_bytes()
                gbs = nbytes / (ct["ms_per_step"] * 1e-3) / 1e9
                rws, bd = c.parity_rows(64)
                also[name] = {"us_per_step": ct["ms_per_step"] * 1e3, "gbs": gbs, "frac": gbs / peak,
                              "tokens_per_s": c.w0.num_tokens / (ct["ms_per_step"] * 1e-3),
                              "algorithmic_bytes_per_launch": nbytes, "repeats": ct["repeats"],
                              "parity_check": {"rows": rws, "mismatches": bd},
                              "input_sets": len(c.dsets), "input_mb": round(c.in_bytes / 1e6),
                              "workload": describe_workload(c.w0, name)}
                launches += ct["launches"]
                del c
            except Exception as exc:  # noqa: BLE001
                also[name] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
            torch.cuda.empty_cache()

    # ---------------------------------------------------------------- N = 1: the ops around the cache write
    ops = None
    if also is not None:
        ops = {}
        tpeak, _ = measured_tensor_peak()
        for name, make in op_workloads.BY_NAME.items():
            try:  # a secondary figure must not cost the headline its line
                ow = make()
                ostep, oe2e, _, _ = ow.make_steps(dev, 2)
                ot = time_passes(ostep, ns.steps, ns.warmup, None, local, 0.05)
                sec = ot["ms_per_step"] * 1e-3
                if ow.flops > 0:
                    ach, unit, bound, pk = ow.flops / sec / 1e12, "TFLOP/s", "tensor", tpeak
                else:
                    ach, unit, bound, pk = ow.algorithmic_bytes / sec / 1e9, "GB/s", "hbm", peak
                ops[name] = {"us_per_step": sec * 1e6, "tokens_per_s": ow.units_per_step / sec, "bound": bound,
                             "achieved": ach, "unit": unit, "frac": ach / pk, "repeats": ot["repeats"],
                             "workload": ow.describe}
                launches += ot["launches"] * ow.launches_per_step
                del ostep, oe2e, ow
            except Exception as exc:  # noqa: BLE001
                ops[name] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
            torch.cuda.empty_cache()

    # ---------------------------------------------------------------- CPU baseline (rank 0, N = 1)
    cpu = None
    if rank == 0 and world == 1 and not ns.no_cpu_baseline:
        rate, threads, T, n, dt = cpu_oracle_rate(workloads.BY_NAME[ns.workload](variant=0), ns.cpu_seconds)
        cpu = {"value": rate, "unit": "tokens/s", "cores": threads, "kind": "port",
               "sample": f"{n} passes over {T} tokens of the batch into a 4096-block host cache, {dt:.1f} s"}
        # also what the reference itself runs on a CPU: the per-token torch loop of its tests
        trate, tthreads, tn, tdt = cpu_torch_loop_rate(workloads.BY_NAME[ns.workload](variant=0), 3.0)
        cpu["torch_loop"] = {"value": trate, "unit": "tokens/s", "cores": tthreads,
                             "sample": f"{tn} passes of the reference tests' per-token torch loop, {tdt:.1f} s"}

    line = None
    if rank == 0:
        total_heads = w0.num_heads * (shard_world if ns.scaling == "strong" else 1)
        head = (f"all {w0.num_heads} KV heads per rank" if ns.scaling == "weak"
                else f"{w0.num_heads} of {total_heads} KV heads per rank")
        line = {
            "metric": metric_name(w0), "value": value, "unit": "tokens/s", "n_gpus": world, "steps": ns.steps,
            "warmup": ns.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": ns.scaling,
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {
                "workload": describe_workload(sets[0], ns.workload),
                "sharding": f"by KV head, no collective; {head}",
                "l2": f"inputs rotate over {len(sets)} input sets ({in_bytes / 1e6:.0f} MB per rank, L2 is 126 MB); "
                      f"each set writes its own cache blocks",
                "timing": timing_note(t, ns.steps),
            },
            "repeats": t["repeats"],
            "pass_us_per_step": t["pass_us_per_step"],
            "hbm_gbs": hbm_all,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": TRAFFIC_BYTES_PER_LAUNCH.get(ns.workload) if shard_world == 1 and ns.tokens is None else None,
                         "peak_source": peak_src,
                         "algorithmic_bytes_per_launch": bytes_launch, "frac_of_nominal_8000": achieved / 8000.0,
                         "single_launch_us_eager": single_us},
            "parity_check": parity,
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps, "api": e2e_api},
            "clocks": t["clocks"],
            "gpu_launches": launches,
        }
        if weak is not None:
            line["weak"] = weak
        if also is not None:
            line["also"] = also
        if ops is not None:
            line["ops"] = ops
        if ns.shard_of is not None:
            line["config"]["sharding"] += f" (one GPU running the share of rank 0 of {ns.shard_of})"
    if dist is not None:
        dist.destroy_process_group()
    return line


# --------------------------------------------------------------------------------------------
# the ops around the cache write (MLA, gather, fp8 quantisation, rotary embedding, decode attention)
# --------------------------------------------------------------------------------------------
def run_op_reference_arm(ns) -> None:
    """--impl reference for an op workload: the CPU oracle alone, a bounded sample per step."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    w = op_workloads.BY_NAME[ns.workload]()
    rate0, _, _, _, _ = op_workloads.cpu_rate(w, 1.0)
    per_step = int(max(64, min(w.units_per_step, rate0 * 100.0 / max(1, ns.steps + ns.warmup))))
    run, n, threads = w.cpu_run(per_step)
    for _ in range(ns.warmup):
        run()
    t0 = time.perf_counter()
    for _ in range(ns.steps):
        run()
    dt = time.perf_counter() - t0
    value = n * ns.steps / dt
    sample = f"{n} of the step's {w.units_per_step} tokens per step, {ns.steps} steps, {threads} thread(s)"
    print(json.dumps({
        "impl": "reference", "metric": w.metric, "value": value, "unit": "tokens/s", "n_gpus": ns.gpus,
        "steps": ns.steps, "warmup": ns.warmup, "ms_per_step": dt / ns.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": w.arithmetic, "data": "synthetic",
        "config": {"workload": f"{w.name}: {w.describe}", "tokens_per_step": n},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }), flush=True)


def run_op_arm(ns):
    """One of the ops around the cache write, measured like the cache write itself: CUDA graphs of
    GRAPH_STEPS steps over rotating inputs, device events, max over ranks; every rank runs the same work."""
    from vllm_xpu_kernels import cabi  # raises if the CUDA library is not built

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path); use --impl reference for the CPU oracle")
    dist, rank, world, local = dist_setup(ns.gpus)
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    cabi.lib()
    w = op_workloads.BY_NAME[ns.workload]()
    nbuf = 2
    step, e2e_step, h2d, d2h = w.make_steps(dev, nbuf)

    steps, warmup = ns.steps, ns.warmup
    t = time_passes(step, steps, warmup, dist, local, ns.min_region_ms * 1e-3)
    clocks = t["clocks"]
    ms_per_step = t["ms_per_step"]
    own_s = t["own_ms_per_step"] * 1e-3
    value = w.units_per_step * world / (ms_per_step * 1e-3)
    achieved = w.algorithmic_bytes / own_s / 1e9
    peak, peak_src = measured_peaks()
    if w.flops > 0:  # compute-bound step: useful flops against the measured dense bf16 GEMM rate
        tf = w.flops / own_s / 1e12
        tpeak, tsrc = measured_tensor_peak()
        roofline = {"bound": "tensor", "achieved": tf, "peak": tpeak, "unit": "TFLOP/s", "frac": tf / tpeak,
                    "traffic": None, "peak_source": tsrc, "useful_flops_per_launch": w.flops,
                    "note": "tcgen05.mma, accumulators and probabilities in tensor memory" +
                            ("; fp8 rows widened to fp16 on their way into shared memory" if "fp8" in w.name else "")}
    else:
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                    "traffic": None, "peak_source": peak_src, "algorithmic_bytes_per_launch": w.algorithmic_bytes,
                    "frac_of_nominal_8000": achieved / 8000.0}

    e2e_steps = max(1, min(steps, 20))
    for i in range(2):
        e2e_step(i)
    torch.cuda.synchronize()
    barrier(dist)
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        e2e_step(i)
    torch.cuda.synchronize()
    e2e_s = max_over_ranks(dist, time.perf_counter() - t0)
    barrier(dist)

    cpu = None
    if rank == 0 and world == 1 and not ns.no_cpu_baseline:
        rate, threads, n, passes, dt = op_workloads.cpu_rate(w, min(ns.cpu_seconds, 10.0))
        cpu = {"value": rate, "unit": "tokens/s", "cores": threads, "kind": "port",
               "sample": f"{passes} passes of the CPU oracle over {n} of the step's {w.units_per_step} tokens, {dt:.1f} s"}
    line = None
    if rank == 0:
        line = {
            "metric": w.metric, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": w.arithmetic, "data": "synthetic",
            "config": {"workload": f"{w.name}: {w.describe}", "sharding": "every rank runs the whole step on its own data",
                       "l2": f"inputs rotate over {nbuf} sets; one step moves {w.algorithmic_bytes / 1e6:.0f} MB "
                             f"(L2 is 126 MB)",
                       "timing": timing_note(t, steps)},
            "repeats": t["repeats"],
            "pass_us_per_step": t["pass_us_per_step"],
            "hbm_gbs": achieved * world,
            "roofline": roofline,
            "cpu_baseline": cpu,
            "e2e": {"value": w.units_per_step * world * e2e_steps / e2e_s, "unit": "tokens/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                    "api": "pinned host tensors -> .to(device) -> C ABI call -> result read back"},
            "clocks": clocks,
            "gpu_launches": t["launches"] * w.launches_per_step,
        }
    if dist is not None:
        dist.destroy_process_group()
    return line


# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the C4 kernel, from an ncu
# capture of the same kernel on 32768 tokens: the full-size workload holds too much memory for a
# multi-pass capture, and traffic grows in proportion to the tokens, so a 16384-token launch is half
# of it: 134 504 704 / 2 bytes read, plus the 33 554 432 bytes written, all of which reach DRAM once
# (the capture window itself saw 47 % of them leave L2 before the kernel ended, the rest are written
# back later).
TRAFFIC_BYTES_PER_LAUNCH: dict[str, int | None] = {"C4": 67_252_352 + 33_554_432}


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8192)
    ap.add_argument("--warmup", type=int, default=128)
    ap.add_argument("--impl", choices=["b200", "reference"], default="b200")
    ap.add_argument("--workload", choices=list(workloads.BY_NAME) + list(op_workloads.BY_NAME), default="C4",
                    help="C1..C5: the cache-write configurations (C4 is the headline); the others are the ops "
                         "around the write, measured the same way")
    ap.add_argument("--scaling", choices=["weak", "strong"], default="strong",
                    help="strong (default): the batch's KV heads are divided over the ranks, each rank owning its "
                         "heads' cache slice; weak: every rank writes the whole batch into a cache of its own")
    ap.add_argument("--shard-of", type=int, default=None, metavar="G",
                    help="one GPU only: run the share that rank 0 of G ranks would run (sizing studies)")
    ap.add_argument("--min-region-ms", type=float, default=120.0,
                    help="the pass of --steps steps is repeated until the timed region is at least this long")
    ap.add_argument("--no-also", action="store_true",
                    help="skip the secondary measurements (other configurations at N = 1, replicated job at N > 1)")
    ap.add_argument("--tokens", type=int, default=None, help="resize the C4 batch (size studies; default 16384)")
    ap.add_argument("--cpu-seconds", type=float, default=10.0, help="time budget of the cpu_baseline leg")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ns = ap.parse_args()
    if ns.steps < 1 or ns.warmup < 0:
        raise SystemExit("--steps must be >= 1 and --warmup >= 0")
    is_op = ns.workload in op_workloads.BY_NAME
    if ns.impl == "reference":
        (run_op_reference_arm if is_op else run_reference_arm)(ns)
    else:
        with LibraryChatterToStderr():
            line = (run_op_arm if is_op else run_b200_arm)(ns)
        if line is not None:
            print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
