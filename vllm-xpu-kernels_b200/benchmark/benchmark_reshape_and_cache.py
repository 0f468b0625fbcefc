#!/usr/bin/env python
"""Latency sweep of ``reshape_and_cache`` (split paged layout) on CUDA.

Same grid as the reference's benchmark/benchmark_reshape_and_cache.py: num_tokens = 2 .. 2048 x
head counts 12 32 40 48 64 96 128, 1024 blocks (tests/utils.py:411-427 there).  The reference
compares its kernel with an IPEX provider through triton's do_bench; here there is one provider and
the timing is per-call CUDA events (median, 20th and 80th percentile are what do_bench reported).
``--slots runs`` places consecutive tokens in consecutive offsets of a block, the pattern a
prefill produces and the one this layout can be written efficiently for.
"""
from __future__ import annotations

import itertools

import torch
from tabulate import tabulate

from _common import DTYPES, cache_dtype, common_parser, make_inputs, ops, time_op


def make_case(num_tokens: int, num_heads: int, head_size: int, block_size: int, num_blocks: int,
              dtype: torch.dtype, kv_cache_dtype: str, slots_mode: str = "random", device: str = "cuda"):
    """(call, tensors): the inputs of one sweep point and the op call the sweep times."""
    key, value, slots, k_scale, v_scale = make_inputs(num_tokens, num_heads, head_size, block_size, num_blocks,
                                                      dtype, kv_cache_dtype, device)
    if slots_mode == "runs":
        nblk = (num_tokens + block_size - 1) // block_size
        perm = torch.randperm(num_blocks, device=device)[:nblk]
        slots = (perm[:, None] * block_size + torch.arange(block_size, device=device)[None, :]).flatten()[:num_tokens]
        slots = slots.contiguous()
    cdt = cache_dtype(dtype, kv_cache_dtype)
    x = 16 // torch.empty((), dtype=cdt).element_size()
    raw = torch.uint8 if cdt != dtype else dtype
    key_cache = torch.zeros(num_blocks, num_heads, head_size // x, block_size, x, dtype=raw, device=device)
    value_cache = torch.zeros(num_blocks, num_heads, head_size, block_size, dtype=raw, device=device)
    if cdt != dtype:
        key_cache, value_cache = key_cache.view(cdt), value_cache.view(cdt)

    def call():
        ops.reshape_and_cache(key, value, key_cache, value_cache, slots, kv_cache_dtype, k_scale, v_scale)

    return call, (key, value, key_cache, value_cache, slots, k_scale, v_scale)


@torch.inference_mode()
def run_benchmark(num_tokens: int, num_heads: int, head_size: int, block_size: int, num_blocks: int,
                  dtype: torch.dtype, kv_cache_dtype: str, num_iters: int, slots_mode: str, flush_l2: bool,
                  device: str = "cuda") -> tuple[float, float]:
    """(median, min) latency in seconds for one sweep point."""
    call, _ = make_case(num_tokens, num_heads, head_size, block_size, num_blocks, dtype, kv_cache_dtype,
                        slots_mode, device)
    return time_op(call, num_iters, flush_l2=flush_l2)


def main(args) -> None:
    dtype = DTYPES[args.dtype]
    rows = []
    for n_tok, heads in itertools.product([2 ** i for i in range(1, 12)], args.head_num_range):
        med, best = run_benchmark(n_tok, heads, args.head_size, args.block_size, args.num_blocks, dtype,
                                  args.kv_cache_dtype, args.iters, args.slots, flush_l2=not args.warm_l2)
        rows.append([n_tok, heads, args.head_size, args.block_size, args.num_blocks, args.dtype, args.kv_cache_dtype,
                     args.slots, f"{med * 1e6:.3f}", f"{best * 1e6:.3f}"])
    print(tabulate(rows, headers=["num_tokens", "num_heads", "head_size", "block_size", "num_blocks", "dtype",
                                  "kv_cache_dtype", "slots", "latency (us)", "min (us)"]))


if __name__ == "__main__":
    parser = common_parser(__doc__)
    parser.add_argument("--num-blocks", type=int, default=1024)
    parser.add_argument("--head-num-range", type=int, nargs="+", default=[12, 32, 40, 48, 64, 96, 128])
    parser.add_argument("--slots", choices=["random", "runs"], default="random")
    parser.set_defaults(iters=30)
    main(parser.parse_args())
