#!/usr/bin/env python
"""Latency sweep of ``reshape_and_cache_flash`` on CUDA: num_tokens = 2, 4, ..., 2048.

Same sweep, defaults and flags as the reference's benchmark/benchmark_reshape_and_cache_flash.py
(8 heads x 128, block_size 64, 512 blocks, fp16, kv_cache_dtype auto, 100 iterations, scales
amax/64, seed 42), timed with CUDA events instead of a host clock and extended with the
bandwidth each latency corresponds to.
"""
from __future__ import annotations

import torch
from tabulate import tabulate

from _common import DTYPES, cache_dtype, common_parser, make_inputs, ops, time_op


def make_case(num_tokens: int, num_heads: int, head_size: int, block_size: int, num_blocks: int,
              dtype: torch.dtype, kv_cache_dtype: str, device: str = "cuda"):
    """(call, tensors): the inputs of one sweep point and the op call the sweep times."""
    key, value, slots, k_scale, v_scale = make_inputs(num_tokens, num_heads, head_size, block_size, num_blocks,
                                                      dtype, kv_cache_dtype, device)
    cdt = cache_dtype(dtype, kv_cache_dtype)
    # one allocation, key cache = [:, 0], value cache = [:, 1], as vLLM lays the flash cache out
    both = torch.zeros(num_blocks, 2, block_size, num_heads, head_size,
                       dtype=torch.uint8 if cdt != dtype else dtype, device=device)
    both = both.view(cdt) if cdt != dtype else both
    key_cache, value_cache = both[:, 0], both[:, 1]

    def call():
        ops.reshape_and_cache_flash(key, value, key_cache, value_cache, slots, kv_cache_dtype, k_scale, v_scale)

    return call, (key, value, key_cache, value_cache, slots, k_scale, v_scale)


@torch.inference_mode()
def run_benchmark(num_tokens: int, num_heads: int, head_size: int, block_size: int, num_blocks: int,
                  dtype: torch.dtype, kv_cache_dtype: str, num_iters: int, flush_l2: bool = True,
                  device: str = "cuda") -> tuple[float, float]:
    """(median, min) latency in seconds for one num_tokens."""
    call, _ = make_case(num_tokens, num_heads, head_size, block_size, num_blocks, dtype, kv_cache_dtype, device)
    return time_op(call, num_iters, flush_l2=flush_l2)


def main(args) -> None:
    dtype = DTYPES[args.dtype]
    s_in = torch.empty((), dtype=dtype).element_size()
    s_out = s_in if args.kv_cache_dtype == "auto" else 1
    rows = []
    for exp in range(1, 12):
        n_tok = 2 ** exp
        med, best = run_benchmark(n_tok, args.num_heads, args.head_size, args.block_size, args.num_blocks, dtype,
                                  args.kv_cache_dtype, args.iters, flush_l2=not args.warm_l2)
        nbytes = 8 * n_tok + n_tok * args.num_heads * args.head_size * 2 * (s_in + s_out)
        rows.append([n_tok, args.num_heads, args.head_size, args.block_size, args.num_blocks, args.dtype,
                     args.kv_cache_dtype, f"{med * 1e6:.3f}", f"{best * 1e6:.3f}", f"{nbytes / med / 1e9:.1f}"])
    print(tabulate(rows, headers=["num_tokens", "num_heads", "head_size", "block_size", "num_blocks", "dtype",
                                  "kv_cache_dtype", "latency (us)", "min (us)", "GB/s"]))


if __name__ == "__main__":
    parser = common_parser(__doc__)
    parser.add_argument("--num-heads", type=int, default=8)
    parser.add_argument("--num-blocks", type=int, default=512)
    main(parser.parse_args())
