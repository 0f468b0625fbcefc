"""ctypes binding of ``libkvcache_b200.so`` (the C ABI declared in include/kvcache_b200.h).

The functions here take torch tensors only to read ``data_ptr()``, sizes and
strides; everything crosses the boundary as plain pointers and integers, the
way a binding in any other language would call it.  Argument meaning and error
behaviour mirror the reference's operators (csrc/cache.cpp:409-489 there): a
failing call raises ``RuntimeError`` with the library's message.
"""
from __future__ import annotations

import ctypes
import functools
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libkvcache_b200.so")

IN_DTYPE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}

# every symbol include/kvcache_b200.h declares
SYMBOLS = (
    "kvc_version",
    "kvc_last_error",
    "kvc_parse_kv_cache_dtype",
    "kvc_reshape_and_cache_flash",
    "kvc_reshape_and_cache",
    "kvc_concat_and_cache_mla",
    "kvc_gather_cache",
    "kvc_reshape_and_cache_flash_host",
    "kvc_reshape_and_cache_flash_host_noalloc",
    "kvc_release_staging",
    "kvc_count_bad_slots",
    "kvc_static_scaled_fp8_quant",
    "kvc_dynamic_scaled_fp8_quant",
    "kvc_dynamic_per_token_scaled_fp8_quant",
    "kvc_rotary_embedding",
    "kvc_rotary_embedding_and_cache_flash",
    "kvc_paged_decode_workspace_bytes",
    "kvc_paged_decode_attention",
    "kvc_paged_attention_workspace_bytes",
    "kvc_paged_attention",
    "kvc_paged_attention_device_status",
    "kvc_paged_attention_plan",
    "kvc_paged_attention_clear_device_status",
    "kvc_selftest_bounded_wait_gives_up",
)

_lib = None


def lib() -> ctypes.CDLL:
    """Loads the library (once).  A missing build is an error, never a fallback."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is not built; run `python build.py` in the package root")
        L = ctypes.CDLL(LIB_PATH)
        i64, vp, ci = ctypes.c_int64, ctypes.c_void_p, ctypes.c_int
        L.kvc_version.restype = ci
        L.kvc_version.argtypes = []
        L.kvc_last_error.restype = ctypes.c_char_p
        L.kvc_last_error.argtypes = []
        L.kvc_parse_kv_cache_dtype.restype = ci
        L.kvc_parse_kv_cache_dtype.argtypes = [ctypes.c_char_p, ctypes.POINTER(ci)]
        L.kvc_reshape_and_cache_flash.restype = ci
        L.kvc_reshape_and_cache_flash.argtypes = [vp] * 5 + [i64] * 11 + [ci, ci, vp, vp, vp]
        L.kvc_reshape_and_cache.restype = ci
        L.kvc_reshape_and_cache.argtypes = [vp] * 5 + [i64] * 9 + [ci, ci, vp, vp, vp]
        L.kvc_concat_and_cache_mla.restype = ci
        L.kvc_concat_and_cache_mla.argtypes = [vp] * 4 + [i64] * 8 + [ci, ci, vp, vp]
        L.kvc_gather_cache.restype = ci
        L.kvc_gather_cache.argtypes = [vp] * 5 + [i64] * 9 + [vp]
        L.kvc_reshape_and_cache_flash_host.restype = ci
        L.kvc_reshape_and_cache_flash_host.argtypes = [vp] * 5 + [i64] * 9 + [ci, ci, vp, vp, vp]
        L.kvc_reshape_and_cache_flash_host_noalloc.restype = ci
        L.kvc_reshape_and_cache_flash_host_noalloc.argtypes = [vp] * 5 + [i64] * 9 + [ci, ci, vp, vp, vp]
        L.kvc_release_staging.restype = ci
        L.kvc_release_staging.argtypes = []
        L.kvc_static_scaled_fp8_quant.restype = ci
        L.kvc_static_scaled_fp8_quant.argtypes = [vp, vp, vp, i64, ci, ci, vp]
        L.kvc_dynamic_scaled_fp8_quant.restype = ci
        L.kvc_dynamic_scaled_fp8_quant.argtypes = [vp, vp, vp, i64, ci, ci, vp]
        L.kvc_dynamic_per_token_scaled_fp8_quant.restype = ci
        L.kvc_dynamic_per_token_scaled_fp8_quant.argtypes = [vp, vp, vp, vp, i64, i64, ci, ci, vp]
        L.kvc_count_bad_slots.restype = ci
        L.kvc_count_bad_slots.argtypes = [vp, i64, i64, vp, vp]
        L.kvc_paged_decode_workspace_bytes.restype = i64
        L.kvc_paged_decode_workspace_bytes.argtypes = [i64] * 5 + [ci, ci]
        L.kvc_paged_decode_attention.restype = ci
        L.kvc_paged_decode_attention.argtypes = [vp] * 10 + [i64] * 15 + [ctypes.c_float, ci, ci, vp]
        L.kvc_paged_attention_workspace_bytes.restype = i64
        L.kvc_paged_attention_workspace_bytes.argtypes = [i64] * 7 + [ci, ci]
        L.kvc_paged_attention.restype = ci
        L.kvc_paged_attention.argtypes = [vp] * 11 + [i64] * 17 + [ctypes.c_float, ci, i64, i64, ci, ci, vp]
        L.kvc_paged_attention_device_status.restype = ci
        L.kvc_paged_attention_device_status.argtypes = [ctypes.POINTER(ci)]
        L.kvc_paged_attention_plan.restype = ci
        L.kvc_paged_attention_plan.argtypes = ([i64] * 7 + [ci, i64, i64, ci, ci] + [ctypes.POINTER(ctypes.c_int32)] * 3 +
                                               [ctypes.POINTER(i64)])
        L.kvc_paged_attention_clear_device_status.restype = ci
        L.kvc_paged_attention_clear_device_status.argtypes = []
        L.kvc_selftest_bounded_wait_gives_up.restype = ci
        L.kvc_selftest_bounded_wait_gives_up.argtypes = [i64, vp]
        L.kvc_rotary_embedding.restype = ci
        L.kvc_rotary_embedding.argtypes = [vp] * 4 + [i64] * 10 + [ci, ci, vp]
        L.kvc_rotary_embedding_and_cache_flash.restype = ci
        L.kvc_rotary_embedding_and_cache_flash.argtypes = [vp] * 8 + [i64] * 17 + [ci, ci, ci, ci, vp, vp, vp]
        _lib = L
    return _lib


def last_error() -> str:
    return lib().kvc_last_error().decode()


def _check(rc: int) -> None:
    if rc != 0:
        raise RuntimeError(last_error())


def parse_kv_cache_dtype(s: str) -> int:
    out = ctypes.c_int(-1)
    _check(lib().kvc_parse_kv_cache_dtype(s.encode(), ctypes.byref(out)))
    return out.value


def _in_dtype(t: torch.Tensor) -> int:
    try:
        return IN_DTYPE[t.dtype]
    except KeyError:
        raise RuntimeError(f"Unsupported input type of kv cache: {t.dtype}") from None


def _stream(stream) -> int:
    if stream is None:
        return torch.cuda.current_stream().cuda_stream
    return stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream)


def _on_tensors_device(fn):
    """Runs ``fn`` with the device of its first CUDA tensor argument current, as the torch ops do under their
    device guard: the default stream argument is then that device's current stream, and the entry points that
    keep per-device state (host staging) pick the right device.  Pointers of one device handed to a launch on
    another would fault or, with peer access on, silently cross the link."""
    @functools.wraps(fn)
    def wrapper(*args, **kwargs):
        for a in list(args) + list(kwargs.values()):
            if isinstance(a, torch.Tensor) and a.is_cuda:
                if a.device.index != torch.cuda.current_device():
                    with torch.cuda.device(a.device):
                        return fn(*args, **kwargs)
                break
        return fn(*args, **kwargs)
    return wrapper


def _scale_ptr(s, kv: int) -> int:
    if kv == 0 or s is None:
        return 0
    return s.data_ptr()


@_on_tensors_device
def reshape_and_cache_flash(key, value, key_cache, value_cache, slot_mapping, kv_cache_dtype: str,
                            k_scale=None, v_scale=None, stream=None) -> None:
    """``kvc_reshape_and_cache_flash`` on device tensors (caches [num_blocks, block_size, H, D])."""
    kv = parse_kv_cache_dtype(kv_cache_dtype)
    _check(lib().kvc_reshape_and_cache_flash(
        key.data_ptr(), value.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr(),
        slot_mapping.data_ptr(), slot_mapping.shape[0], key.shape[1], key.shape[2], key_cache.shape[1],
        key.stride(0), key.stride(1), value.stride(0), value.stride(1),
        key_cache.stride(0), key_cache.stride(1), key_cache.stride(2),
        _in_dtype(key), kv, _scale_ptr(k_scale, kv), _scale_ptr(v_scale, kv), _stream(stream)))


@_on_tensors_device
def reshape_and_cache(key, value, key_cache, value_cache, slot_mapping, kv_cache_dtype: str,
                      k_scale=None, v_scale=None, stream=None) -> None:
    """``kvc_reshape_and_cache`` on device tensors (K [nb,H,D/x,bs,x], V [nb,H,D,bs], contiguous)."""
    kv = parse_kv_cache_dtype(kv_cache_dtype)
    _check(lib().kvc_reshape_and_cache(
        key.data_ptr(), value.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr(),
        slot_mapping.data_ptr(), slot_mapping.shape[0], key.shape[1], key.shape[2],
        key_cache.shape[3], key_cache.shape[4],
        key.stride(0), key.stride(1), value.stride(0), value.stride(1),
        _in_dtype(key), kv, _scale_ptr(k_scale, kv), _scale_ptr(v_scale, kv), _stream(stream)))


@_on_tensors_device
def concat_and_cache_mla(kv_c, k_pe, kv_cache, slot_mapping, kv_cache_dtype: str, scale=None, stream=None) -> None:
    """``kvc_concat_and_cache_mla`` on device tensors (kv_cache [num_blocks, block_size, R + P])."""
    kv = parse_kv_cache_dtype(kv_cache_dtype)
    _check(lib().kvc_concat_and_cache_mla(
        kv_c.data_ptr(), k_pe.data_ptr(), kv_cache.data_ptr(), slot_mapping.data_ptr(), slot_mapping.shape[0],
        kv_c.shape[1], k_pe.shape[1], kv_cache.shape[1], kv_c.stride(0), k_pe.stride(0),
        kv_cache.stride(0), kv_cache.stride(1), _in_dtype(kv_c), kv, _scale_ptr(scale, kv), _stream(stream)))


@_on_tensors_device
def gather_cache(src_cache, dst, block_table, cu_seq_lens, batch_size: int, seq_starts=None, stream=None) -> None:
    """``kvc_gather_cache`` on device tensors (src_cache [num_blocks, block_size, entry], dst [rows, entry])."""
    entry = 1
    for d in src_cache.shape[2:]:
        entry *= d
    _check(lib().kvc_gather_cache(
        src_cache.data_ptr(), dst.data_ptr(), block_table.data_ptr(), cu_seq_lens.data_ptr(),
        0 if seq_starts is None else seq_starts.data_ptr(), batch_size, dst.shape[0], src_cache.shape[1], entry,
        src_cache.element_size(), block_table.stride(0), src_cache.stride(0), src_cache.stride(1), dst.stride(0),
        _stream(stream)))


def _host_entry_args(host_key, host_value, host_slot_mapping, kv_cache_dtype: str):
    """Checks shared by the two host-buffer entry points; returns (kv code, num_heads, head_size)."""
    kv = parse_kv_cache_dtype(kv_cache_dtype)
    for t in (host_key, host_value, host_slot_mapping):
        if t.is_cuda:
            raise RuntimeError("host entry point needs CPU tensors for key, value and slot_mapping")
    H, D = host_key.shape[1], host_key.shape[2]
    if H > 1 and (host_key.stride(1) != D or host_value.stride(1) != D):
        raise RuntimeError("host key/value must have contiguous heads")
    return kv, H, D


@_on_tensors_device
def reshape_and_cache_flash_host(host_key, host_value, key_cache, value_cache, host_slot_mapping,
                                 kv_cache_dtype: str, k_scale=None, v_scale=None, stream=None) -> None:
    """``kvc_reshape_and_cache_flash_host``: key/value/slot_mapping are HOST tensors
    ([T, H, D] with contiguous heads; pinned for asynchronous copies), caches and scales on the device."""
    kv, H, D = _host_entry_args(host_key, host_value, host_slot_mapping, kv_cache_dtype)
    _check(lib().kvc_reshape_and_cache_flash_host(
        host_key.data_ptr(), host_value.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr(),
        host_slot_mapping.data_ptr(), host_slot_mapping.shape[0], H, D, key_cache.shape[1],
        host_key.stride(0), host_value.stride(0),
        key_cache.stride(0), key_cache.stride(1), key_cache.stride(2),
        _in_dtype(host_key), kv, _scale_ptr(k_scale, kv), _scale_ptr(v_scale, kv), _stream(stream)))


NOALLOC_STAGING_BYTES = 16 * 1024 * 1024  # KVC_NOALLOC_STAGING_BYTES in include/kvcache_b200.h


@_on_tensors_device
def reshape_and_cache_flash_host_noalloc(host_key, host_value, key_cache, value_cache, host_slot_mapping,
                                         kv_cache_dtype: str, k_scale=None, v_scale=None, stream=None) -> None:
    """``kvc_reshape_and_cache_flash_host_noalloc``: like ``reshape_and_cache_flash_host`` but the
    device staging is the library's fixed 16 MiB area, for processes that can no longer call
    cudaMalloc (all free GPU memory already belongs to the serving framework's pool) or must not
    pay its synchronisation.  Batches that do not fit raise ``RuntimeError``; calls that overlap on
    the GPU race on the shared area; the first call per device should precede any stream capture."""
    kv, H, D = _host_entry_args(host_key, host_value, host_slot_mapping, kv_cache_dtype)
    _check(lib().kvc_reshape_and_cache_flash_host_noalloc(
        host_key.data_ptr(), host_value.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr(),
        host_slot_mapping.data_ptr(), host_slot_mapping.shape[0], H, D, key_cache.shape[1],
        host_key.stride(0), host_value.stride(0),
        key_cache.stride(0), key_cache.stride(1), key_cache.stride(2),
        _in_dtype(host_key), kv, _scale_ptr(k_scale, kv), _scale_ptr(v_scale, kv), _stream(stream)))


def release_staging() -> None:
    _check(lib().kvc_release_staging())


@_on_tensors_device
def count_bad_slots(slot_mapping, num_slots: int, stream=None) -> int:
    """Number of slots >= num_slots (debug aid; synchronises to read the answer)."""
    out = torch.zeros(1, dtype=torch.int64, device=slot_mapping.device)
    _check(lib().kvc_count_bad_slots(slot_mapping.data_ptr(), slot_mapping.shape[0], num_slots,
                                     out.data_ptr(), _stream(stream)))
    return int(out.item())


FP8_CODE = {torch.float8_e4m3fn: 1, torch.float8_e5m2: 2}


@_on_tensors_device
def static_scaled_fp8_quant(out, input, scale, stream=None) -> None:
    """``kvc_static_scaled_fp8_quant``: out (fp8) <- clamp(input * (1/scale)); all contiguous, on the device."""
    _check(lib().kvc_static_scaled_fp8_quant(out.data_ptr(), input.data_ptr(), scale.data_ptr(), input.numel(),
                                             _in_dtype(input), FP8_CODE[out.dtype], _stream(stream)))


@_on_tensors_device
def dynamic_scaled_fp8_quant(out, input, scale, stream=None) -> None:
    """``kvc_dynamic_scaled_fp8_quant``: scale (zero-initialised by the caller) <- absmax / fp8_max, then as static."""
    _check(lib().kvc_dynamic_scaled_fp8_quant(out.data_ptr(), input.data_ptr(), scale.data_ptr(), input.numel(),
                                              _in_dtype(input), FP8_CODE[out.dtype], _stream(stream)))


@_on_tensors_device
def dynamic_per_token_scaled_fp8_quant(out, input, scales, scale_ub=None, stream=None) -> None:
    """``kvc_dynamic_per_token_scaled_fp8_quant`` for input [..., hidden]: one scale per row."""
    hidden = input.shape[-1]
    tokens = input.numel() // hidden if hidden else 0
    _check(lib().kvc_dynamic_per_token_scaled_fp8_quant(
        out.data_ptr(), input.data_ptr(), scales.data_ptr(), 0 if scale_ub is None else scale_ub.data_ptr(), tokens,
        hidden, _in_dtype(input), FP8_CODE[out.dtype], _stream(stream)))


def _rope_geometry(t, head_size: int, lead: int):
    """(heads, token stride, head stride) of a query/key tensor whose first ``lead`` dims index
    tokens: [.., heads, head_size] or [.., heads * head_size] (csrc/pos_encoding_kernels.cpp:196-211
    of the reference).  With two leading dims the batch dim must be the seq dim's continuation."""
    if t.stride(-1) != 1 and t.shape[-1] > 1:
        raise RuntimeError("rotary_embedding: the last dim of query/key must be contiguous")
    if lead == 2 and t.shape[0] > 1 and t.stride(0) != t.shape[1] * t.stride(1):
        raise RuntimeError("rotary_embedding: [batch, seq, ...] tensors must be contiguous across batch and seq")
    if t.dim() == lead + 2:
        if t.shape[-1] != head_size:
            raise RuntimeError("rotary_embedding: last dim of query/key must be head_size")
        return t.shape[-2], t.stride(lead - 1), t.stride(-2)
    if t.dim() != lead + 1 or t.shape[-1] % head_size:
        raise RuntimeError("rotary_embedding: query/key must be [.., heads, head_size] or [.., heads * head_size]")
    return t.shape[-1] // head_size, t.stride(lead - 1), head_size


def _rope_args(positions, query, key, head_size: int, cos_sin_cache):
    lead = positions.dim()
    if lead not in (1, 2):
        raise RuntimeError("positions must have shape [num_tokens] or [batch_size, seq_len]")
    if not positions.is_contiguous() or positions.dtype != torch.int64:
        raise RuntimeError("rotary_embedding: positions must be a contiguous int64 tensor")
    for t in (query, key):
        if t is not None and tuple(t.shape[:lead]) != tuple(positions.shape):
            raise RuntimeError("query, key and positions must have the same number of tokens" if lead == 1 else
                               "query, key and positions must have the same batch_size and seq_len")
    if cos_sin_cache.dim() != 2 or not cos_sin_cache.is_contiguous() or cos_sin_cache.dtype != query.dtype:
        raise RuntimeError("rotary_embedding: cos_sin_cache must be a contiguous [max_position, rot_dim] tensor of "
                           "the query's dtype")
    hq, qst, qsh = _rope_geometry(query, head_size, lead)
    hk, kst, ksh = _rope_geometry(key, head_size, lead) if key is not None else (0, 0, 0)
    return positions.numel(), hq, hk, qst, qsh, kst, ksh


@_on_tensors_device
def rotary_embedding(positions, query, key, head_size: int, cos_sin_cache, is_neox: bool, stream=None) -> None:
    """``kvc_rotary_embedding``: in place on query and key (key may be None)."""
    T, hq, hk, qst, qsh, kst, ksh = _rope_args(positions, query, key, head_size, cos_sin_cache)
    _check(lib().kvc_rotary_embedding(
        positions.data_ptr(), query.data_ptr(), 0 if key is None else key.data_ptr(), cos_sin_cache.data_ptr(),
        T, hq, hk, head_size, cos_sin_cache.shape[1], cos_sin_cache.shape[0], qst, qsh, kst, ksh,
        int(bool(is_neox)), _in_dtype(query), _stream(stream)))


@_on_tensors_device
def rotary_embedding_and_cache_flash(positions, query, key, value, head_size: int, cos_sin_cache, is_neox: bool,
                                     key_cache, value_cache, slot_mapping, kv_cache_dtype: str, k_scale=None,
                                     v_scale=None, write_back_key: bool = True, stream=None) -> None:
    """``kvc_rotary_embedding_and_cache_flash``: rotary embedding of query and key in place, and the rotated key
    and ``value`` [T, Hkv, head_size] into their cache slots (caches [num_blocks, block_size, Hkv, head_size])."""
    T, hq, hk, qst, qsh, kst, ksh = _rope_args(positions, query, key, head_size, cos_sin_cache)
    kv = parse_kv_cache_dtype(kv_cache_dtype)
    if value.dim() != 3 or value.shape[0] != T or value.shape[1] != hk or value.shape[2] != head_size:
        raise RuntimeError("rotary_embedding_and_cache_flash: value must be [num_tokens, num_kv_heads, head_size]")
    if slot_mapping.shape[0] > T:
        raise RuntimeError("rotary_embedding_and_cache_flash: slot_mapping is longer than positions")
    _check(lib().kvc_rotary_embedding_and_cache_flash(
        positions.data_ptr(), query.data_ptr(), key.data_ptr(), value.data_ptr(), cos_sin_cache.data_ptr(),
        key_cache.data_ptr(), value_cache.data_ptr(), slot_mapping.data_ptr(), T, slot_mapping.shape[0], hq, hk,
        head_size, cos_sin_cache.shape[1], cos_sin_cache.shape[0], key_cache.shape[1], qst, qsh, kst, ksh,
        value.stride(0), value.stride(1), key_cache.stride(0), key_cache.stride(1), key_cache.stride(2),
        int(bool(is_neox)), int(bool(write_back_key)), _in_dtype(query), kv, _scale_ptr(k_scale, kv),
        _scale_ptr(v_scale, kv), _stream(stream)))


@_on_tensors_device
def paged_decode_attention(query, key_cache, value_cache, block_table, seq_lens, softmax_scale: float,
                           max_seq_len: int, kv_cache_dtype: str = "auto", k_descale=None, v_descale=None, sink=None,
                           out=None, stream=None):
    """``kvc_paged_decode_attention``: query [S, Hq, D] (fp16 / bf16), caches [num_blocks, block_size, Hkv, D]
    (the query's type, or fp8 / uint8 bytes with ``kv_cache_dtype`` "fp8*"), block_table int32 [S, max_blocks],
    seq_lens int32 [S]; ``k_descale`` / ``v_descale`` device fp32 scalars; ``sink`` [Hq].  Returns ``out``."""
    kv = parse_kv_cache_dtype(kv_cache_dtype)
    S, hq, D = query.shape
    hk = key_cache.shape[2]
    if out is None:
        out = torch.empty_like(query)
    nbytes = lib().kvc_paged_decode_workspace_bytes(S, hq, hk, D, max_seq_len, _in_dtype(query), kv)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=query.device)
    _check(lib().kvc_paged_decode_attention(
        out.data_ptr(), query.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr(), block_table.data_ptr(),
        seq_lens.data_ptr(), 0 if sink is None else sink.data_ptr(), _scale_ptr(k_descale, kv),
        _scale_ptr(v_descale, kv), ws.data_ptr(), ws.numel(), S, hq, hk, D, key_cache.shape[1], block_table.stride(0),
        max_seq_len, query.stride(0), query.stride(1), out.stride(0), out.stride(1), key_cache.stride(0),
        key_cache.stride(1), key_cache.stride(2), float(softmax_scale), _in_dtype(query), kv, _stream(stream)))
    return out


@_on_tensors_device
def paged_attention(query, key_cache, value_cache, block_table, seq_lens, cu_seqlens_q, max_seqlen_q: int,
                    softmax_scale: float, max_seq_len: int, causal: bool = True, kv_cache_dtype: str = "auto",
                    k_descale=None, v_descale=None, sink=None, out=None, stream=None, window=(-1, -1)):
    """``kvc_paged_attention``: like ``paged_decode_attention`` with several query tokens per sequence: query
    [total_q, Hq, D], ``cu_seqlens_q`` int32 [S + 1] on the device, the query tokens being the last positions of
    their sequences (``causal``: token i of q_len sees seq_len - q_len + i + 1 cached tokens); ``window`` =
    (left, right) keeps positions [pos - left, pos + right], -1 = open.  Returns ``out``."""
    kv = parse_kv_cache_dtype(kv_cache_dtype)
    T, hq, D = query.shape
    S = seq_lens.shape[0]
    hk = key_cache.shape[2]
    if out is None:
        out = torch.empty_like(query)
    nbytes = lib().kvc_paged_attention_workspace_bytes(S, T, max_seqlen_q, hq, hk, D, max_seq_len, _in_dtype(query), kv)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=query.device)
    _check(lib().kvc_paged_attention(
        out.data_ptr(), query.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr(), block_table.data_ptr(),
        seq_lens.data_ptr(), cu_seqlens_q.data_ptr(), 0 if sink is None else sink.data_ptr(), _scale_ptr(k_descale, kv),
        _scale_ptr(v_descale, kv), ws.data_ptr(), ws.numel(), S, T, max_seqlen_q, hq, hk, D, key_cache.shape[1],
        block_table.stride(0), max_seq_len, query.stride(0), query.stride(1), out.stride(0), out.stride(1),
        key_cache.stride(0), key_cache.stride(1), key_cache.stride(2), float(softmax_scale), int(bool(causal)),
        int(window[0]), int(window[1]), _in_dtype(query), kv, _stream(stream)))
    return out


def paged_attention_device_status() -> int:
    """``kvc_paged_attention_device_status``: waits for the device and returns the status word of the tcgen05
    many-rows kernel (0 = fine, 1 = a bounded wait inside a kernel gave up, 2 = shared memory misaligned)."""
    v = ctypes.c_int(0)
    _check(lib().kvc_paged_attention_device_status(ctypes.byref(v)))
    return int(v.value)


def paged_attention_clear_device_status() -> None:
    """``kvc_paged_attention_clear_device_status``: waits for the device and puts the status word back to 0."""
    _check(lib().kvc_paged_attention_clear_device_status())


def paged_attention_plan(num_seqs: int, total_q: int, max_seqlen_q: int, num_heads: int, num_kv_heads: int,
                         head_size: int, max_seq_len: int, causal: bool = True, window=(-1, -1),
                         q_dtype: torch.dtype = torch.bfloat16, kv_cache_dtype: str = "auto") -> dict:
    """``kvc_paged_attention_plan``: the launch shape ``paged_attention`` uses for these arguments."""
    i32 = ctypes.c_int32
    splits, tps, tile = i32(0), i32(0), i32(0)
    ws = ctypes.c_int64(0)
    _check(lib().kvc_paged_attention_plan(num_seqs, total_q, max_seqlen_q, num_heads, num_kv_heads, head_size,
                                          max_seq_len, int(bool(causal)), int(window[0]), int(window[1]),
                                          IN_DTYPE[q_dtype], parse_kv_cache_dtype(kv_cache_dtype), ctypes.byref(splits),
                                          ctypes.byref(tps), ctypes.byref(tile), ctypes.byref(ws)))
    return {"splits": splits.value, "tiles_per_split": tps.value, "tile_tokens": tile.value,
            "workspace_bytes": ws.value}


def selftest_bounded_wait_gives_up(tries: int = 50, stream=None) -> None:
    """``kvc_selftest_bounded_wait_gives_up``: launches the one-CTA kernel whose bounded wait runs out (about
    20 us per try); afterwards ``paged_attention_device_status()`` is 1 until it is cleared."""
    _check(lib().kvc_selftest_bounded_wait_gives_up(int(tries), _stream(stream)))
