"""Shared helpers of the test-suite: golden fixtures, torch <-> numpy views, oracle calls."""
from __future__ import annotations

import glob
import os

import numpy as np
import torch

import oracle
from oracle.torch_views import ORC_IN, as_np  # noqa: F401
from oracle import torch_views

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

TORCH_DT = {"half": torch.float16, "bfloat16": torch.bfloat16, "float": torch.float32}


def golden_files(kind: str = "kv") -> list[str]:
    """Fixture files of one kind: "kv" (flash_* and paged_*), "mla" or "gather"."""
    with open(os.path.join(GOLDEN_DIR, "MANIFEST.txt")) as f:
        names = [ln.strip() for ln in f if ln.strip() and not ln.startswith("#")]
    prefixes = {"kv": ("flash_", "paged_"), "mla": ("mla_",), "gather": ("gather_",), "quant": ("quant_",),
                "rope": ("rope_",), "decode_attn": ("decode_attn_",),
                "varlen_attn": ("varlen_attn_",), "window_attn": ("window_attn_",)}[kind]
    return [n for n in names if n.startswith(prefixes)]


class MlaCase:
    def __init__(self, fname: str):
        z = np.load(os.path.join(GOLDEN_DIR, fname))
        self.dtype = TORCH_DT[str(z["dtype"])]
        self.kv_cache_dtype = str(z["kv_cache_dtype"])
        self.kv_c = from_bits(z["kv_c"], self.dtype)
        self.k_pe = from_bits(z["k_pe"], self.dtype)
        self.slot_mapping = torch.from_numpy(z["slot_mapping"].astype(np.int64))
        self.scale = float(z["scale"])
        cdt = cache_torch_dtype(self.dtype, self.kv_cache_dtype)
        self.cache_before = from_bits(z["cache_before"], cdt)
        self.cache_after = from_bits(z["cache_after"], cdt)


class QuantCase:
    def __init__(self, fname: str):
        z = np.load(os.path.join(GOLDEN_DIR, fname))
        self.dtype = TORCH_DT[str(z["dtype"])]
        self.fp8 = str(z["fp8"])
        self.fp8_dtype = torch.float8_e5m2 if self.fp8 == "fp8_e5m2" else torch.float8_e4m3fn
        self.x = from_bits(z["x"], self.dtype)
        self.scale = float(z["scale"])
        self.out_tensor = torch.from_numpy(z["out_tensor"])
        self.scales = torch.from_numpy(z["scales"])
        self.out_token = torch.from_numpy(z["out_token"])
        self.scale_ub = float(z["scale_ub"]) if "scale_ub" in z.files else None


class RopeCase:
    """A rotary-embedding fixture with the memory layout it was made with: query/key are
    [..., :head_size] cuts of wider allocations when the heads are padded, or flattened to
    [T, heads * head_size]."""

    def __init__(self, fname: str):
        z = np.load(os.path.join(GOLDEN_DIR, fname))
        self.dtype = TORCH_DT[str(z["dtype"])]
        self.is_neox = bool(z["is_neox"])
        self.head_size = int(z["head_size"])
        self.rot_dim = int(z["rot_dim"])
        self.flat = bool(z["flat"])
        self.positions = torch.from_numpy(z["positions"].astype(np.int64))
        self.cos_sin_cache = from_bits(z["cos_sin_cache"], self.dtype)
        self.query_store = from_bits(z["query_store"], self.dtype)
        self.key_store = from_bits(z["key_store"], self.dtype) if "key_store" in z.files else None
        self.query_after = from_bits(z["query_after"], self.dtype)
        self.key_after = from_bits(z["key_after"], self.dtype) if "key_after" in z.files else None

    def views(self, q_store: torch.Tensor, k_store):
        """(query, key) views of the given allocations, as the op is handed them."""
        q = q_store[..., :self.head_size]
        k = None if k_store is None else k_store[..., :self.head_size]
        if self.flat:
            q = q.flatten(start_dim=-2)
            k = None if k is None else k.flatten(start_dim=-2)
        return q, k


class DecodeAttnCase:
    """A paged attention fixture: query tokens (one per sequence in the decode fixtures, query_lens otherwise),
    caches [nb, bs, Hkv, D]."""

    def __init__(self, fname: str):
        z = np.load(os.path.join(GOLDEN_DIR, fname))
        self.dtype = TORCH_DT[str(z["dtype"])]
        self.kv_cache_dtype = str(z["kv_cache_dtype"])
        cdt = cache_torch_dtype(self.dtype, self.kv_cache_dtype)
        self.query = from_bits(z["query"], self.dtype)
        self.key_cache = from_bits(z["key_cache"], cdt)
        self.value_cache = from_bits(z["value_cache"], cdt)
        self.block_tables = torch.from_numpy(z["block_tables"].astype(np.int32))
        self.kv_lens = torch.from_numpy(z["kv_lens"].astype(np.int32))
        self.scale = float(z["scale"])
        self.descale = float(z["descale"])
        self.sink = from_bits(z["sink"], self.dtype) if "sink" in z.files else None
        self.expected = from_bits(z["expected"], self.dtype)
        self.query_lens = torch.from_numpy(z["query_lens"].astype(np.int32))
        self.causal = bool(z["causal"])
        self.cu_seqlens_q = torch.cat([torch.zeros(1, dtype=torch.int32),
                                       torch.cumsum(self.query_lens, 0).to(torch.int32)])
        self.window = tuple(int(x) for x in z["window"]) if "window" in z.files else (-1, -1)
        self.paged = bool(z["paged"]) if "paged" in z.files else True
        if not self.paged:
            # keys/values of all sequences back to back [total_k, H, D]: the same thing as a cache of one-token
            # blocks with the identity table block_tables[s][j] = cu_seqlens_k[s] + j
            self.cu_seqlens_k = torch.cat([torch.zeros(1, dtype=torch.int32),
                                           torch.cumsum(self.kv_lens, 0).to(torch.int32)])
            self.dense_key, self.dense_value = self.key_cache, self.value_cache
            self.key_cache, self.value_cache = self.key_cache[:, None], self.value_cache[:, None]
            j = torch.arange(int(self.kv_lens.max()), dtype=torch.int32)[None, :]
            self.block_tables = torch.minimum(self.cu_seqlens_k[:-1, None] + j,
                                              torch.tensor(self.key_cache.shape[0] - 1, dtype=torch.int32))


# The reference's own tolerance for this op (tests/flash_attn/test_flash_attn_varlen_func.py:265, :386).
ATTN_ATOL = ATTN_RTOL = 1e-2


class GatherCase:
    def __init__(self, fname: str):
        z = np.load(os.path.join(GOLDEN_DIR, fname))
        self.dtype = TORCH_DT[str(z["dtype"])]
        self.src_cache = from_bits(z["src_cache"], self.dtype)
        self.block_table = torch.from_numpy(z["block_table"].astype(np.int32))
        self.cu_seq_lens = torch.from_numpy(z["cu_seq_lens"].astype(np.int32))
        self.batch_size = int(z["batch_size"])
        self.seq_starts = torch.from_numpy(z["seq_starts"].astype(np.int32)) if "seq_starts" in z.files else None
        self.expected = from_bits(z["expected"], self.dtype)


def from_bits(a: np.ndarray, dtype: torch.dtype) -> torch.Tensor:
    """Inverse of the fixtures' storage: uint16 bit patterns -> half/bf16 tensor."""
    a = np.ascontiguousarray(a)
    if dtype in (torch.float16, torch.bfloat16):
        return torch.from_numpy(a.view(np.int16)).view(dtype)
    if dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
        return torch.from_numpy(a).view(dtype)
    return torch.from_numpy(a)


def cache_torch_dtype(in_dtype: torch.dtype, kv_cache_dtype: str) -> torch.dtype:
    if kv_cache_dtype == "auto":
        return in_dtype
    return torch.float8_e5m2 if kv_cache_dtype == "fp8_e5m2" else torch.float8_e4m3fn


class GoldenCase:
    """One fixture, rebuilt with the reference's memory layout: key/value are slices of
    a [T, 3, H, D] tensor, flash caches are the [:, 0] and [:, 1] views of one allocation."""

    def __init__(self, fname: str):
        z = np.load(os.path.join(GOLDEN_DIR, fname))
        self.name = fname
        self.layout = str(z["layout"])
        self.kv_cache_dtype = str(z["kv_cache_dtype"])
        self.dtype = TORCH_DT[str(z["dtype"])]
        self.block_size = int(z["block_size"])
        self.k_scale = float(z["k_scale"])
        self.v_scale = float(z["v_scale"])
        self.max_abs_scaled = float(z["max_abs_scaled"])
        self.qkv = from_bits(z["qkv"], self.dtype)
        self.key, self.value = self.qkv[:, 1], self.qkv[:, 2]
        self.slot_mapping = torch.from_numpy(z["slot_mapping"].astype(np.int64))
        cdt = cache_torch_dtype(self.dtype, self.kv_cache_dtype)
        kb, vb = from_bits(z["key_cache_before"], cdt), from_bits(z["value_cache_before"], cdt)
        if self.layout == "flash":
            both = torch.stack([kb.view(torch.uint8), vb.view(torch.uint8)], dim=1).contiguous()
            both = both.view(cdt) if cdt != torch.uint8 else both
            self.alloc = both
            self.key_cache, self.value_cache = both[:, 0], both[:, 1]
        else:
            self.alloc = None
            self.key_cache, self.value_cache = kb.clone(), vb.clone()
        self.key_cache_after = from_bits(z["key_cache_after"], cdt)
        self.value_cache_after = from_bits(z["value_cache_after"], cdt)


def oracle_call(layout: str, key, value, key_cache, value_cache, slot_mapping, kv_cache_dtype: str,
                k_scale: float, v_scale: float, threads: int = 1) -> None:
    """Runs the CPU oracle in place on CPU torch tensors (views keep their strides)."""
    torch_views.run(layout, key, value, key_cache, value_cache, slot_mapping, kv_cache_dtype, k_scale, v_scale,
                    threads=threads)


def same_bytes(a: torch.Tensor, b: torch.Tensor) -> bool:
    """Bit-for-bit equality (NaN-safe, sign-of-zero-safe)."""
    a, b = a.contiguous(), b.contiguous()
    if a.shape != b.shape or a.dtype != b.dtype:
        return False
    return bool(torch.equal(a.view(torch.uint8), b.view(torch.uint8)))


def fill_pattern_(t: torch.Tensor, seed: int) -> torch.Tensor:
    """Deterministic, recognisable non-constant fill of a cache (any dtype, any device)."""
    g = torch.Generator(device=t.device)
    g.manual_seed(seed)
    raw = t.view(torch.uint8) if t.is_contiguous() else None
    assert raw is not None, "fill contiguous allocations, then take views"
    n = raw.numel()
    src = torch.randint(0, 120, (min(n, 1 << 20),), dtype=torch.uint8, device=t.device, generator=g)
    flat = raw.view(-1)
    reps = (n + src.numel() - 1) // src.numel()
    flat.copy_(src.repeat(reps)[:n])
    return t


OPCHECK_UTILS = ("test_schema", "test_autograd_registration", "test_faketensor", "test_aot_dispatch_dynamic")


def opcheck(op, args, kwargs=None, test_utils=OPCHECK_UTILS):
    """``torch.library.opcheck`` with ``torch.allclose`` replaced by a comparison in float64, so that
    fp8 tensors can be compared (what the reference's tests/utils.py:21-67 does for the same reason)."""
    import unittest.mock

    def allclose64(a, b, rtol=1e-05, atol=1e-08, equal_nan=False):
        return bool(torch.all(torch.isclose(a.double(), b.double(), rtol=rtol, atol=atol, equal_nan=equal_nan)).item())

    with unittest.mock.patch("torch.allclose", new=allclose64):
        return torch.library.opcheck(op, args, kwargs, test_utils=test_utils)
