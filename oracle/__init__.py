"""CPU oracle for the paged KV-cache write path -- TEST INFRASTRUCTURE ONLY.

Thin ctypes/numpy front end over ``kv_oracle.c`` (built by ``make -C oracle``).
Only the test-suite, ``__graft_entry__.smoke()`` and the CPU-baseline leg of
``bench.py`` may import this package; the shipped library never does.

Arrays are numpy views; 16-bit float inputs travel as ``uint16`` bit patterns
(``in_dtype`` says whether they are "f16" or "bf16"), fp8 caches as ``uint8``.
Strides are taken from the numpy views, so strided key/value slices and
``[:, 0]``-style cache views behave as in the reference's tests
(tests/test_cache.py:92-93, tests/utils.py:200-223 of the reference).
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liborc.so")

IN_DTYPES = {"f32": 0, "f16": 1, "bf16": 2}
KV_DTYPES = {"auto": 0, "fp8": 1, "fp8_e4m3": 1, "fp8_e5m2": 2}

_lib = None


def build(force: bool = False) -> str:
    """Compile ``liborc.so`` with gcc if it is missing (or ``force``)."""
    if force or not os.path.exists(_LIB_PATH):
        subprocess.run(["make", "-C", _HERE, "liborc.so"] + (["-B"] if force else []),
                       check=True, capture_output=True)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_LIB_PATH)
        i64, f32, vp, ci = ctypes.c_int64, ctypes.c_float, ctypes.c_void_p, ctypes.c_int
        L.orc_reshape_and_cache_flash.restype = ci
        L.orc_reshape_and_cache_flash.argtypes = [vp, vp, vp, vp, vp] + [i64] * 11 + [ci, ci, f32, f32, i64, ci]
        L.orc_reshape_and_cache.restype = ci
        L.orc_reshape_and_cache.argtypes = [vp, vp, vp, vp, vp] + [i64] * 9 + [ci, ci, f32, f32, i64, ci]
        L.orc_concat_and_cache_mla.restype = ci
        L.orc_concat_and_cache_mla.argtypes = [vp, vp, vp, vp] + [i64] * 8 + [ci, ci, f32, i64]
        L.orc_gather_cache.restype = None
        L.orc_gather_cache.argtypes = [vp] * 5 + [i64] * 8
        L.orc_static_scaled_fp8_quant.restype = None
        L.orc_static_scaled_fp8_quant.argtypes = [vp, vp, i64, ci, ci, f32]
        L.orc_absmax_scale.restype = f32
        L.orc_absmax_scale.argtypes = [vp, i64, ci, ci]
        L.orc_per_token_fp8_quant.restype = None
        L.orc_per_token_fp8_quant.argtypes = [vp, vp, vp, i64, i64, ci, ci, vp]
        L.orc_convert_table.restype = None
        L.orc_convert_table.argtypes = [ci, ci, f32, vp]
        L.orc_convert_f32.restype = None
        L.orc_convert_f32.argtypes = [vp, i64, ci, f32, vp]
        L.orc_f32_to_e4m3.restype = ctypes.c_uint8
        L.orc_f32_to_e4m3.argtypes = [f32]
        L.orc_f32_to_e5m2.restype = ctypes.c_uint8
        L.orc_f32_to_e5m2.argtypes = [f32]
        L.orc_rotary_embedding.restype = ci
        L.orc_rotary_embedding.argtypes = [vp, vp, vp, vp] + [i64] * 9 + [ci, ci]
        L.orc_f32_to_bf16.restype = ctypes.c_uint16
        L.orc_f32_to_bf16.argtypes = [f32]
        L.orc_f32_to_f16.restype = ctypes.c_uint16
        L.orc_f32_to_f16.argtypes = [f32]
        L.orc_paged_decode_attention.restype = None
        L.orc_paged_decode_attention.argtypes = [vp] * 7 + [f32, f32] + [i64] * 11 + [f32, ci, ci]
        L.orc_paged_attention.restype = None
        L.orc_paged_attention.argtypes = [vp] * 8 + [f32, f32] + [i64] * 11 + [f32, ci, ci, ci]
        L.orc_paged_attention_window.restype = None
        L.orc_paged_attention_window.argtypes = [vp] * 8 + [f32, f32] + [i64] * 11 + [f32, ci, i64, i64, ci, ci]
        L.orc_e4m3_to_f32.restype = f32
        L.orc_e4m3_to_f32.argtypes = [ctypes.c_uint8]
        L.orc_e5m2_to_f32.restype = f32
        L.orc_e5m2_to_f32.argtypes = [ctypes.c_uint8]
        L.orc_max_threads.restype = ci
        _lib = L
    return _lib


def max_threads() -> int:
    return int(lib().orc_max_threads())


def _estrides(a: np.ndarray) -> list[int]:
    for s in a.strides:
        if s % a.itemsize:
            raise ValueError("stride is not a whole number of elements")
    return [s // a.itemsize for s in a.strides]


def _check_in(a: np.ndarray, in_dtype: str) -> None:
    want = np.float32 if in_dtype == "f32" else np.uint16
    if a.dtype != want:
        raise TypeError(f"{in_dtype} input must be a {np.dtype(want)} array, got {a.dtype}")
    if a.ndim != 3 or (a.shape[2] > 1 and _estrides(a)[2] != 1):
        raise ValueError("key/value must be [T, H, D] with a contiguous last dim")


def reshape_and_cache_flash(key, value, key_cache, value_cache, slot_mapping, kv_cache_dtype: str,
                            k_scale: float, v_scale: float, in_dtype: str, threads: int = 1,
                            check_slots: bool = True) -> None:
    """In-place oracle for ``_C_cache_ops.reshape_and_cache_flash``.

    key/value: [>=T, H, D]; caches: [num_blocks, block_size, H, D] views;
    slot_mapping: int64 [T] (T, not key.shape[0], is the token count:
    csrc/cache.cpp:470 of the reference).
    """
    _check_in(key, in_dtype)
    _check_in(value, in_dtype)
    kv = KV_DTYPES[kv_cache_dtype]
    want = key.dtype if kv == 0 else np.uint8
    if key_cache.dtype != want or value_cache.dtype != want:
        raise TypeError(f"cache arrays must be {np.dtype(want)}")
    slot_mapping = np.ascontiguousarray(slot_mapping, dtype=np.int64)
    T = slot_mapping.shape[0]
    H, D = key.shape[1], key.shape[2]
    nb, bs = key_cache.shape[0], key_cache.shape[1]
    ks, vs, cs, cvs = _estrides(key), _estrides(value), _estrides(key_cache), _estrides(value_cache)
    if cs[:3] != cvs[:3]:
        raise ValueError("key_cache and value_cache must share strides")
    if T > key.shape[0] or T > value.shape[0]:
        raise ValueError("slot_mapping is longer than key/value")
    rc = lib().orc_reshape_and_cache_flash(
        key.ctypes.data, value.ctypes.data, key_cache.ctypes.data, value_cache.ctypes.data,
        slot_mapping.ctypes.data, T, H, D, bs, ks[0], ks[1], vs[0], vs[1], cs[0], cs[1], cs[2],
        IN_DTYPES[in_dtype], kv, float(k_scale), float(v_scale), nb * bs if check_slots else -1, threads)
    if rc != 0:
        raise IndexError("slot_mapping holds a slot >= num_blocks * block_size")


def reshape_and_cache(key, value, key_cache, value_cache, slot_mapping, kv_cache_dtype: str,
                      k_scale: float, v_scale: float, in_dtype: str, threads: int = 1,
                      check_slots: bool = True) -> None:
    """In-place oracle for ``_C_cache_ops.reshape_and_cache`` (split paged layout).

    key_cache: contiguous [num_blocks, H, D/x, block_size, x];
    value_cache: contiguous [num_blocks, H, D, block_size].
    """
    _check_in(key, in_dtype)
    _check_in(value, in_dtype)
    kv = KV_DTYPES[kv_cache_dtype]
    want = key.dtype if kv == 0 else np.uint8
    if key_cache.dtype != want or value_cache.dtype != want:
        raise TypeError(f"cache arrays must be {np.dtype(want)}")
    if not (key_cache.flags.c_contiguous and value_cache.flags.c_contiguous):
        raise ValueError("paged caches must be contiguous")
    slot_mapping = np.ascontiguousarray(slot_mapping, dtype=np.int64)
    T = slot_mapping.shape[0]
    H, D = key.shape[1], key.shape[2]
    nb, bs, x = key_cache.shape[0], key_cache.shape[3], key_cache.shape[4]
    if key_cache.shape != (nb, H, D // x, bs, x) or value_cache.shape != (nb, H, D, bs):
        raise ValueError("cache shapes do not match key/value")
    ks, vs = _estrides(key), _estrides(value)
    rc = lib().orc_reshape_and_cache(
        key.ctypes.data, value.ctypes.data, key_cache.ctypes.data, value_cache.ctypes.data,
        slot_mapping.ctypes.data, T, H, D, bs, x, ks[0], ks[1], vs[0], vs[1], IN_DTYPES[in_dtype], kv,
        float(k_scale), float(v_scale), nb * bs if check_slots else -1, threads)
    if rc != 0:
        raise IndexError("slot_mapping holds a slot >= num_blocks * block_size")


def concat_and_cache_mla(kv_c, k_pe, kv_cache, slot_mapping, kv_cache_dtype: str, scale: float, in_dtype: str,
                         check_slots: bool = True) -> None:
    """In-place oracle for ``_C_cache_ops.concat_and_cache_mla``.

    kv_c [>=T, R], k_pe [>=T, P] (last dim contiguous), kv_cache [num_blocks, block_size, R + P] view."""
    want_in = np.float32 if in_dtype == "f32" else np.uint16
    if kv_c.dtype != want_in or k_pe.dtype != want_in:
        raise TypeError(f"{in_dtype} inputs must be {np.dtype(want_in)} arrays")
    kv = KV_DTYPES[kv_cache_dtype]
    if kv_cache.dtype != (want_in if kv == 0 else np.uint8):
        raise TypeError("kv_cache array has the wrong dtype")
    slot_mapping = np.ascontiguousarray(slot_mapping, dtype=np.int64)
    T = slot_mapping.shape[0]
    R, P = kv_c.shape[1], k_pe.shape[1]
    nb, bs = kv_cache.shape[0], kv_cache.shape[1]
    if kv_cache.shape[2] != R + P:
        raise ValueError("kv_cache.shape[2] must be kv_lora_rank + pe_dim")
    cs = _estrides(kv_cache)
    for a in (kv_c, k_pe, kv_cache):
        if a.shape[-1] > 1 and _estrides(a)[-1] != 1:
            raise ValueError("last dim must be contiguous")
    rc = lib().orc_concat_and_cache_mla(
        kv_c.ctypes.data, k_pe.ctypes.data, kv_cache.ctypes.data, slot_mapping.ctypes.data, T, R, P, bs,
        _estrides(kv_c)[0], _estrides(k_pe)[0], cs[0], cs[1], IN_DTYPES[in_dtype], kv, float(scale),
        nb * bs if check_slots else -1)
    if rc != 0:
        raise IndexError("slot_mapping holds a slot >= num_blocks * block_size")


def gather_cache(src_cache, dst, block_table, cu_seq_lens, batch_size: int, seq_starts=None) -> None:
    """In-place oracle for ``_C_cache_ops.gather_cache``: src_cache [num_blocks, block_size, entry...] view
    with contiguous entries, dst [rows, entry...] with contiguous rows, int32 tables."""
    if src_cache.dtype != dst.dtype:
        raise TypeError("src_cache and dst must have the same dtype")
    block_table = np.ascontiguousarray(block_table, dtype=np.int32)
    cu_seq_lens = np.ascontiguousarray(cu_seq_lens, dtype=np.int32)
    ss = None if seq_starts is None else np.ascontiguousarray(seq_starts, dtype=np.int32)
    entry_bytes = int(np.prod(src_cache.shape[2:])) * src_cache.itemsize
    lib().orc_gather_cache(
        src_cache.ctypes.data, dst.ctypes.data, block_table.ctypes.data, cu_seq_lens.ctypes.data,
        None if ss is None else ss.ctypes.data, batch_size, dst.shape[0], src_cache.shape[1], entry_bytes,
        block_table.shape[1], src_cache.strides[0], src_cache.strides[1], dst.strides[0])


def static_scaled_fp8_quant(x: np.ndarray, scale: float, in_dtype: str, fp8: str) -> np.ndarray:
    """fp8 bytes of ``clamp(x * (1/scale))`` for a contiguous array (the reference's static quant)."""
    x = np.ascontiguousarray(x)
    out = np.empty(x.shape, dtype=np.uint8)
    lib().orc_static_scaled_fp8_quant(out.ctypes.data, x.ctypes.data, x.size, IN_DTYPES[in_dtype], KV_DTYPES[fp8],
                                      float(scale))
    return out


def absmax_scale(x: np.ndarray, in_dtype: str, fp8: str) -> np.float32:
    x = np.ascontiguousarray(x)
    return np.float32(lib().orc_absmax_scale(x.ctypes.data, x.size, IN_DTYPES[in_dtype], KV_DTYPES[fp8]))


def per_token_fp8_quant(x: np.ndarray, in_dtype: str, fp8: str, scale_ub=None):
    """(bytes, scales[T, 1]) of the reference's dynamic per-token quant for x [T, hidden]."""
    x = np.ascontiguousarray(x)
    T, hidden = x.shape
    out = np.empty((T, hidden), dtype=np.uint8)
    scales = np.empty((T, 1), dtype=np.float32)
    ub = None if scale_ub is None else ctypes.byref(ctypes.c_float(float(scale_ub)))
    lib().orc_per_token_fp8_quant(out.ctypes.data, scales.ctypes.data, x.ctypes.data, T, hidden, IN_DTYPES[in_dtype],
                                  KV_DTYPES[fp8], ctypes.cast(ub, ctypes.c_void_p) if ub is not None else None)
    return out, scales


def rotary_embedding(positions, query, key, head_size: int, cos_sin_cache, is_neox: bool, in_dtype: str) -> None:
    """In-place oracle for ``_C.rotary_embedding``.  ``query`` / ``key`` (or None) are numpy views shaped
    ``[T, heads, head_size]`` (any token and head stride, contiguous last dim) or ``[T, heads * head_size]``;
    ``positions`` int64 ``[T]``; ``cos_sin_cache`` contiguous ``[max_position, rot_dim]`` of the same type."""
    positions = np.ascontiguousarray(positions, dtype=np.int64).reshape(-1)
    T = positions.shape[0]

    def geometry(a):
        if a.ndim == 2:
            if a.shape[1] % head_size or (a.shape[1] > 1 and _estrides(a)[1] != 1):
                raise ValueError("flat query/key must be [T, heads * head_size] with a contiguous last dim")
            return a.shape[1] // head_size, _estrides(a)[0], head_size
        if a.ndim != 3 or a.shape[2] != head_size or _estrides(a)[2] != 1:
            raise ValueError("query/key must be [T, heads, head_size] with a contiguous last dim")
        return a.shape[1], _estrides(a)[0], _estrides(a)[1]

    want = np.float32 if in_dtype == "f32" else np.uint16
    for a in (query, key, cos_sin_cache):
        if a is not None and a.dtype != want:
            raise TypeError(f"{in_dtype} tensors must be {np.dtype(want)} arrays")
    if query.shape[0] != T or (key is not None and key.shape[0] != T):
        raise ValueError("query, key and positions must have the same number of tokens")
    if not cos_sin_cache.flags.c_contiguous:
        raise ValueError("cos_sin_cache must be contiguous")
    hq, qs, qhs = geometry(query)
    hk, ks, khs = geometry(key) if key is not None else (hq, 0, 0)
    max_pos, rot_dim = cos_sin_cache.shape
    if rot_dim % 2 or rot_dim > head_size:
        raise ValueError("rot_dim must be even and at most head_size")
    rc = lib().orc_rotary_embedding(
        positions.ctypes.data, query.ctypes.data, None if key is None else key.ctypes.data,
        cos_sin_cache.ctypes.data, T, hq, hk, rot_dim, max_pos, qs, ks, qhs, khs, int(bool(is_neox)),
        IN_DTYPES[in_dtype])
    if rc != 0:
        raise IndexError("positions holds an entry outside [0, max_position)")


def paged_decode_attention(query, key_cache, value_cache, block_table, seq_lens, scale: float, in_dtype: str,
                           kv_cache_dtype: str = "auto", k_descale: float = 1.0, v_descale: float = 1.0,
                           sink=None, cu_seqlens_q=None, causal: bool = False, window=(-1, -1)) -> np.ndarray:
    """fp32 ``[tokens, num_heads, head_size]`` result of attention over a paged cache.  ``query`` [tokens, Hq, D]
    (contiguous last dim): one token per sequence, or with ``cu_seqlens_q`` (int32 [S + 1]) the last q_len_s
    positions of each sequence, optionally under a causal mask; caches [num_blocks, block_size, Hkv, D] views
    with the same strides, of the query's type (uint16 bit patterns / float32) or uint8 fp8 bytes;
    ``block_table`` int32 [S, max_blocks]; ``seq_lens`` int32 [S]; ``sink`` [Hq] of the query's type or None;
    ``window`` = (left, right) limits attention to positions [pos - left, pos + right], a negative side is open."""
    want = np.float32 if in_dtype == "f32" else np.uint16
    kv = KV_DTYPES[kv_cache_dtype]
    if query.dtype != want or (sink is not None and sink.dtype != want):
        raise TypeError(f"{in_dtype} query/sink must be {np.dtype(want)} arrays")
    if key_cache.dtype != (want if kv == 0 else np.uint8) or value_cache.dtype != key_cache.dtype:
        raise TypeError("cache arrays do not fit kv_cache_dtype")
    if key_cache.shape != value_cache.shape or key_cache.strides != value_cache.strides:
        raise ValueError("key_cache and value_cache must have the same shape and strides")
    T, hq, D = query.shape
    cu = None
    if cu_seqlens_q is not None:
        cu = np.ascontiguousarray(cu_seqlens_q, dtype=np.int32)
        if cu.ndim != 1 or cu[0] != 0 or cu[-1] != T or np.any(np.diff(cu) < 0):
            raise ValueError("cu_seqlens_q must run from 0 to the number of query tokens")
    S = T if cu is None else cu.shape[0] - 1
    nb, bs, hk, Dc = key_cache.shape
    if Dc != D or hq % hk or _estrides(query)[2] != 1 or _estrides(key_cache)[3] != 1:
        raise ValueError("shapes of query and caches do not fit")
    block_table = np.ascontiguousarray(block_table, dtype=np.int32)
    seq_lens = np.ascontiguousarray(seq_lens, dtype=np.int32)
    if block_table.shape[0] != S or seq_lens.shape[0] != S:
        raise ValueError("block_table / seq_lens do not fit the number of sequences")
    if S and int(seq_lens.max(initial=0)) > block_table.shape[1] * bs:
        raise ValueError("a sequence is longer than its block table")
    if block_table.size and (block_table.min() < 0 or block_table.max() >= nb):
        raise IndexError("block_table names a block outside the cache")
    sink_c = None if sink is None else np.ascontiguousarray(sink)
    out = np.empty((T, hq, D), dtype=np.float32)
    qs, cs = _estrides(query), _estrides(key_cache)
    lib().orc_paged_attention_window(
        out.ctypes.data, query.ctypes.data, key_cache.ctypes.data, value_cache.ctypes.data, block_table.ctypes.data,
        seq_lens.ctypes.data, None if cu is None else cu.ctypes.data, None if sink_c is None else sink_c.ctypes.data,
        float(k_descale), float(v_descale), S, hq, hk, D, bs, block_table.shape[1], qs[0], qs[1], cs[0], cs[1], cs[2],
        float(scale), int(bool(causal)), int(window[0]), int(window[1]), IN_DTYPES[in_dtype], kv)
    return out


def convert_table(in_dtype: str, kv_cache_dtype: str, scale: float) -> np.ndarray:
    """fp8 byte for each of the 65536 f16/bf16 bit patterns at one scale."""
    out = np.empty(65536, dtype=np.uint8)
    lib().orc_convert_table(IN_DTYPES[in_dtype], KV_DTYPES[kv_cache_dtype], float(scale), out.ctypes.data)
    return out


def convert_f32(x: np.ndarray, kv_cache_dtype: str, scale: float) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint8)
    lib().orc_convert_f32(x.ctypes.data, x.size, KV_DTYPES[kv_cache_dtype], float(scale), out.ctypes.data)
    return out


def np_f32_to_e4m3(x: np.ndarray) -> np.ndarray:
    """Independent numpy restatement of RNE + saturate onto e4m3fn.

    Enumerates the 127 non-negative finite codes, decodes them, and picks the
    nearest (ties to the even code).  Used to cross-check the C converter.
    """
    codes = np.arange(0x7F, dtype=np.uint8)
    e = (codes >> 3).astype(np.int32)
    m = (codes & 7).astype(np.float64)
    grid = np.where(e == 0, m * 2.0**-9, (1 + m / 8) * 2.0 ** (e - 7))
    x = np.asarray(x, dtype=np.float32)
    a = np.abs(x.astype(np.float64))
    hi = np.clip(np.searchsorted(grid, a, side="left"), 0, 0x7E)
    lo = np.clip(hi - 1, 0, 0x7E)
    dlo, dhi = a - grid[lo], grid[hi] - a
    pick_hi = (dhi < dlo) | ((dhi == dlo) & (hi % 2 == 0))
    code = np.where(pick_hi, hi, lo).astype(np.uint8)
    code = np.where(a >= 448.0, np.uint8(0x7E), code)
    sign = (x.view(np.uint32) >> 24).astype(np.uint8) & np.uint8(0x80)
    out = code | sign
    return np.where(np.isnan(x), np.uint8(0x7F), out).astype(np.uint8)
