"""Seeded synthetic workloads for the KV-cache write ops.

The five named configurations are the ones the project is measured on; each is
generated on the CPU from a fixed seed so that the CUDA kernels and any CPU
checker see identical bytes.  The reference plugin's own benchmarks use the same
kind of data (``randn`` rows, ``random.sample`` slots:
benchmark/benchmark_reshape_and_cache_flash.py:34-56 there); no dataset is involved.

A workload holds CPU tensors only.  ``shard_heads`` cuts it along the KV-head
axis the way tensor parallelism does: every rank keeps all tokens and all slots
but only its heads, and owns a cache with that many heads, so no rank ever needs
another rank's data.
"""
from __future__ import annotations

import dataclasses
import random

import torch

FP8_MAX = {"fp8": 448.0, "fp8_e4m3": 448.0, "fp8_e5m2": 57344.0}


@dataclasses.dataclass
class Workload:
    name: str
    layout: str            # "flash" | "paged"
    kv_cache_dtype: str    # "auto" | "fp8" | "fp8_e4m3" | "fp8_e5m2"
    key: torch.Tensor      # [T, H, D], maybe a strided view
    value: torch.Tensor
    slot_mapping: torch.Tensor  # int64 [T]
    num_blocks: int
    block_size: int
    k_scale: torch.Tensor  # float32 0-dim
    v_scale: torch.Tensor

    @property
    def num_tokens(self) -> int:
        return self.slot_mapping.shape[0]

    @property
    def num_active(self) -> int:
        return int((self.slot_mapping >= 0).sum())

    @property
    def num_heads(self) -> int:
        return self.key.shape[1]

    @property
    def head_size(self) -> int:
        return self.key.shape[2]

    @property
    def cache_dtype(self) -> torch.dtype:
        if self.kv_cache_dtype == "auto":
            return self.key.dtype
        return torch.float8_e5m2 if self.kv_cache_dtype == "fp8_e5m2" else torch.float8_e4m3fn

    def cache_shapes(self) -> tuple[tuple[int, ...], tuple[int, ...]]:
        H, D, nb, bs = self.num_heads, self.head_size, self.num_blocks, self.block_size
        if self.layout == "flash":
            return (nb, bs, H, D), (nb, bs, H, D)
        x = 16 // torch.empty((), dtype=self.cache_dtype).element_size()
        return (nb, H, D // x, bs, x), (nb, H, D, bs)

    def algorithmic_bytes(self) -> int:
        """Bytes the op must move: every slot entry once, and for each token that is not
        skipped its K and V rows read once and written once."""
        s_in = self.key.element_size()
        s_out = s_in if self.kv_cache_dtype == "auto" else 1
        return 8 * self.num_tokens + self.num_active * self.num_heads * self.head_size * 2 * (s_in + s_out)


def _scales(key: torch.Tensor, value: torch.Tensor, kv_cache_dtype: str) -> tuple[torch.Tensor, torch.Tensor]:
    if kv_cache_dtype == "auto":
        return torch.tensor(1.0), torch.tensor(1.0)
    m = FP8_MAX[kv_cache_dtype]
    return ((key.float().abs().amax() / m).to(torch.float32), (value.float().abs().amax() / m).to(torch.float32))


def _distinct_slots(num_slots: int, n: int) -> torch.Tensor:
    return torch.tensor(random.sample(range(num_slots), n), dtype=torch.long)


def _seed(seed: int) -> None:
    random.seed(seed)
    torch.manual_seed(seed)


def c1(variant: int = 0) -> Workload:
    """flash, bf16 -> bf16, 83 tokens, 8 heads x 128, 1024 blocks of 16 (seed 0)."""
    _seed(0 + 1000 * variant)
    key = torch.randn(83, 8, 128).to(torch.bfloat16)
    value = torch.randn(83, 8, 128).to(torch.bfloat16)
    slots = _distinct_slots(1024 * 16, 83)
    return Workload("C1", "flash", "auto", key, value, slots, 1024, 16, *_scales(key, value, "auto"))


def c2(variant: int = 0) -> Workload:
    """flash, bf16 -> fp8_e4m3, 4096 tokens, 8 x 128, 8192 blocks of 64, scale = amax/448 (seed 1)."""
    _seed(1 + 1000 * variant)
    key = torch.randn(4096, 8, 128).to(torch.bfloat16)
    value = torch.randn(4096, 8, 128).to(torch.bfloat16)
    slots = _distinct_slots(8192 * 64, 4096)
    return Workload("C2", "flash", "fp8_e4m3", key, value, slots, 8192, 64, *_scales(key, value, "fp8_e4m3"))


def c3(variant: int = 0) -> Workload:
    """paged layout, fp16 -> fp16, 2048 tokens, 32 x 128, 4096 blocks of 16 (seed 2)."""
    _seed(2 + 1000 * variant)
    key = torch.randn(2048, 32, 128).to(torch.float16)
    value = torch.randn(2048, 32, 128).to(torch.float16)
    slots = _distinct_slots(4096 * 16, 2048)
    return Workload("C3", "paged", "auto", key, value, slots, 4096, 16, *_scales(key, value, "auto"))


def c4(variant: int = 0, num_tokens: int = 16384, num_blocks: int = 65536) -> Workload:
    """Llama-3-70B-shaped prefill chunk: flash, bf16 -> fp8_e4m3, 16384 tokens, 8 x 128,
    65536 blocks of 64; values ~ N(0, std 2); slots are whole runs of 64 inside randomly
    chosen blocks, as a sequence being prefilled gets them (seed 3)."""
    _seed(3 + 1000 * variant)
    key = (2.0 * torch.randn(num_tokens, 8, 128)).to(torch.bfloat16)
    value = (2.0 * torch.randn(num_tokens, 8, 128)).to(torch.bfloat16)
    bs = 64
    nblk = (num_tokens + bs - 1) // bs
    perm = torch.randperm(num_blocks)[:nblk]
    slots = (perm[:, None] * bs + torch.arange(bs)[None, :]).flatten()[:num_tokens].contiguous()
    return Workload("C4", "flash", "fp8_e4m3", key, value, slots, num_blocks, bs, *_scales(key, value, "fp8_e4m3"))


def c5(kv_cache_dtype: str = "auto", variant: int = 0) -> Workload:
    """Padding-heavy strided decode batch: key/value are views into one fused qkv
    [8192, (32+2*32)*64] bf16 tensor, half of the slots are -1 (seed 4)."""
    _seed(4 + 1000 * variant)
    T, H, D = 8192, 32, 64
    qkv = torch.randn(T, (H + 2 * H) * D).to(torch.bfloat16)
    key = qkv[:, H * D:2 * H * D].view(T, H, D)
    value = qkv[:, 2 * H * D:3 * H * D].view(T, H, D)
    skipped = torch.randperm(T)[:T // 2]
    slots = _distinct_slots(32768 * 16, T)
    slots[skipped] = -1
    name = "C5-bf16" if kv_cache_dtype == "auto" else "C5-fp8"
    return Workload(name, "flash", kv_cache_dtype, key, value, slots, 32768, 16, *_scales(key, value, kv_cache_dtype))


BY_NAME = {
    "C1": c1,
    "C2": c2,
    "C3": c3,
    "C4": c4,
    "C5-bf16": lambda variant=0: c5("auto", variant),
    "C5-fp8": lambda variant=0: c5("fp8_e4m3", variant),
}


def shard_heads(w: Workload, rank: int, world: int) -> Workload:
    """The part of ``w`` that rank ``rank`` of ``world`` owns: heads
    [rank*H/world, (rank+1)*H/world), all tokens, all slots, both scales."""
    H = w.num_heads
    if H % world:
        raise ValueError(f"{H} KV heads do not split over {world} ranks")
    h0, h1 = rank * H // world, (rank + 1) * H // world
    return dataclasses.replace(w, name=f"{w.name}[heads {h0}:{h1}]", key=w.key[:, h0:h1], value=w.value[:, h0:h1])
