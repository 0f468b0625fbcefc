"""Shared pieces of the two latency sweeps (CUDA-event timing, cache factories, CLI)."""
from __future__ import annotations

import argparse
import os
import random
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from vllm_xpu_kernels import ops  # noqa: E402,F401  (registers torch.ops._C_cache_ops.*)

DTYPES = {"half": torch.half, "bfloat16": torch.bfloat16, "float": torch.float}


def cache_dtype(dtype: torch.dtype, kv_cache_dtype: str) -> torch.dtype:
    if kv_cache_dtype == "auto":
        return dtype
    return torch.float8_e5m2 if kv_cache_dtype == "fp8_e5m2" else torch.float8_e4m3fn


def make_inputs(num_tokens: int, num_heads: int, head_size: int, block_size: int, num_blocks: int,
                dtype: torch.dtype, kv_cache_dtype: str, device: str, seed: int = 42):
    """Random key/value rows, distinct random slots and amax/64 scales -- the recipe of the
    reference's sweeps (benchmark_reshape_and_cache_flash.py:34-73 there)."""
    if kv_cache_dtype != "auto" and head_size % 16:
        raise ValueError("fp8 kv-cache requires head_size to be a multiple of 16.")
    if num_tokens > num_blocks * block_size:
        raise ValueError("num_tokens cannot exceed the total number of cache slots")
    random.seed(seed)
    torch.manual_seed(seed)
    key = torch.randn(num_tokens, num_heads, head_size, device=device).to(dtype)
    value = torch.randn(num_tokens, num_heads, head_size, device=device).to(dtype)
    slots = torch.tensor(random.sample(range(num_blocks * block_size), num_tokens), dtype=torch.long, device=device)
    k_scale = (key.amax() / 64.0).to(torch.float32)
    v_scale = (value.amax() / 64.0).to(torch.float32)
    return key, value, slots, k_scale, v_scale


def time_op(fn, iters: int, warmup: int = 5, flush_l2: bool = True) -> tuple[float, float]:
    """(median, min) seconds per call from per-call CUDA events on the current stream.
    With ``flush_l2`` a 256 MB buffer is rewritten before every timed call, so the call
    starts from a cold L2 (126 MB on B200)."""
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush_l2 else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        times.append(a.elapsed_time(b) * 1e-3)
    times.sort()
    return times[len(times) // 2], times[0]


def common_parser(description: str) -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description=description)
    ap.add_argument("--head-size", type=int, choices=[64, 80, 96, 112, 120, 128, 192, 256], default=128)
    ap.add_argument("--block-size", type=int, choices=[16, 32, 64], default=64)
    ap.add_argument("--dtype", type=str, choices=["half", "bfloat16"], default="half")
    ap.add_argument("--kv-cache-dtype", type=str, choices=["auto", "fp8", "fp8_e4m3", "fp8_e5m2"], default="auto")
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--warm-l2", action="store_true", help="do not flush L2 between timed calls")
    return ap
