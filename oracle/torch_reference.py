"""The reference's own CPU statement of the cache-write ops, in PyTorch -- TEST INFRASTRUCTURE ONLY.

The reference project checks its kernels against per-token torch loops written inline in its tests
(tests/test_cache.py:155-164 for the paged layout, :284-292 for the flash layout there); they are
restated here so that (a) the C oracle can be cross-checked against them on arbitrary inputs and
(b) the benchmark can time them on the host as "what the reference itself runs on a CPU".
fp8: ``(x.float() / scale).clamp(-max, max).to(float8)`` -- torch's cast is the conversion the reference
kernels call; the clamp is this build's saturation rule (identical while |x/scale| <= 464).
Tokens with a negative slot are skipped (csrc/cache.cpp:49, :145 of the reference).
"""
from __future__ import annotations

import torch

_FP8 = {"fp8": (torch.float8_e4m3fn, 448.0), "fp8_e4m3": (torch.float8_e4m3fn, 448.0),
        "fp8_e5m2": (torch.float8_e5m2, 57344.0)}


def _rows(x: torch.Tensor, kv_cache_dtype: str, scale: float) -> torch.Tensor:
    if kv_cache_dtype == "auto":
        return x
    dt, m = _FP8[kv_cache_dtype]
    return (x.float() / torch.tensor(scale, dtype=torch.float32)).clamp(-m, m).to(dt)


def reshape_and_cache_flash(key, value, key_cache, value_cache, slot_mapping, kv_cache_dtype: str,
                            k_scale: float, v_scale: float) -> None:
    """caches [num_blocks, block_size, H, D] (fp8 caches as float8 tensors), in place."""
    bs = key_cache.shape[1]
    slots = slot_mapping.tolist()
    k, v = _rows(key[:len(slots)], kv_cache_dtype, k_scale), _rows(value[:len(slots)], kv_cache_dtype, v_scale)
    for i, s in enumerate(slots):
        if s < 0:
            continue
        key_cache[s // bs, s % bs, :, :] = k[i]
        value_cache[s // bs, s % bs, :, :] = v[i]


def reshape_and_cache(key, value, key_cache, value_cache, slot_mapping, kv_cache_dtype: str,
                      k_scale: float, v_scale: float) -> None:
    """key_cache [num_blocks, H, D/x, block_size, x], value_cache [num_blocks, H, D, block_size], in place."""
    bs, x = key_cache.shape[3], key_cache.shape[4]
    H, D = key.shape[1], key.shape[2]
    slots = slot_mapping.tolist()
    k, v = _rows(key[:len(slots)], kv_cache_dtype, k_scale), _rows(value[:len(slots)], kv_cache_dtype, v_scale)
    k = k.reshape(len(slots), H, D // x, x)
    for i, s in enumerate(slots):
        if s < 0:
            continue
        key_cache[s // bs, :, :, s % bs, :] = k[i]
        value_cache[s // bs, :, :, s % bs] = v[i]
