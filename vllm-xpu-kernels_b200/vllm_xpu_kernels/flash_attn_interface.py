"""``flash_attn_varlen_func`` with the reference's signature (vllm_xpu_kernels/flash_attn_interface.py:24-125
there): paged keys/values (``block_table`` + ``seqused_k``) or the non-paged form (``cu_seqlens_k``), causal
mask, sliding windows, sink -- decode (one query token per sequence) at HBM speed; several query tokens per
sequence on the same kernel (runs of at most 16 rows per kv head), on a tcgen05 kernel with scores and
accumulators in tensor memory (runs of more than 64 rows per kv head; every head size, 16-bit and fp8 caches) or on an
mma.sync kernel (runs of 17 to 64 rows).
softcap, alibi, dropout and returning the softmax are not supported.  On top of the reference,
the cache may hold fp8 bytes: pass ``k_descale`` / ``v_descale`` (the inverse of the k_scale / v_scale the
cache was written with), which the reference's interface names but rejects."""
from typing import Optional

import torch

from . import _vllm_fa2_C  # noqa: F401

FA2_UNAVAILABLE_REASON = None
FA2_AVAILABLE = True
DEFAULT_FA_VERSION = 2

_FP8_NAMES = {torch.float8_e4m3fn: "fp8_e4m3", torch.float8_e5m2: "fp8_e5m2", torch.uint8: "fp8_e4m3"}


def maybe_contiguous(x):
    return x.contiguous() if x is not None and x.stride(-1) != 1 else x


def flash_attn_varlen_func(
    q,
    k,
    v,
    max_seqlen_q,
    cu_seqlens_q,
    max_seqlen_k,
    cu_seqlens_k=None,  # only used for non-paged prefill
    seqused_k=None,
    q_v=None,
    dropout_p=0.0,
    softmax_scale=None,
    causal=False,
    window_size: Optional[list[int]] = None,
    softcap=0.0,  # 0.0 means deactivated
    alibi_slopes=None,
    deterministic=False,
    return_attn_probs=False,
    block_table=None,
    return_softmax_lse=False,
    out=None,
    # FA3 Only
    scheduler_metadata=None,
    q_descale=None,
    k_descale=None,
    v_descale=None,
    num_splits: int = 0,
    # Version selector
    fa_version: int = DEFAULT_FA_VERSION,
    s_aux: Optional[torch.Tensor] = None,
    # fp8 caches handed over as uint8: "fp8_e4m3" (default) or "fp8_e5m2"
    kv_cache_dtype: Optional[str] = None,
):
    assert cu_seqlens_k is not None or seqused_k is not None, \
        "cu_seqlens_k or seqused_k must be provided"
    assert cu_seqlens_k is None or seqused_k is None, \
        "cu_seqlens_k and seqused_k cannot be provided at the same time"
    assert block_table is None or seqused_k is not None, \
        "when enable block_table, seqused_k is needed"
    assert block_table is not None or cu_seqlens_k is not None, \
        "when block_table is disabled, cu_seqlens_k is needed"
    if fa_version != 2:
        raise NotImplementedError("not support yet")
    if q_v is not None or q_descale is not None or scheduler_metadata is not None:
        raise NotImplementedError("q_v, q_descale and scheduler_metadata are not supported")
    if return_softmax_lse or return_attn_probs:
        raise NotImplementedError("softmax_lse / attention probabilities are not returned")

    if softmax_scale is None:
        softmax_scale = q.shape[-1]**(-0.5)
    real_window_size = (-1, -1) if window_size is None else (window_size[0], window_size[1])
    q, k, v = [maybe_contiguous(x) for x in (q, k, v)]

    fp8_cache = k.dtype in _FP8_NAMES
    if fp8_cache or k_descale is not None or v_descale is not None:
        if not fp8_cache:
            raise NotImplementedError("k_descale / v_descale need an fp8 (or uint8) cache")
        if block_table is None or softcap or dropout_p or alibi_slopes is not None:
            raise NotImplementedError("fp8 caches: only the paged form is built (no softcap, dropout, alibi)")
        if out is None:
            out = torch.empty_like(q)
        name = kv_cache_dtype or _FP8_NAMES[k.dtype]
        torch.ops._vllm_fa2_C.paged_decode_attention(q, k, v, out, seqused_k, block_table, max_seqlen_k,
                                                     float(softmax_scale), s_aux, name, k_descale, v_descale,
                                                     cu_seqlens_q, max_seqlen_q, causal, real_window_size[0],
                                                     real_window_size[1])
        return out

    dummy_cu_seqlens_k = torch.empty_like(cu_seqlens_q)
    out, softmax_lse = torch.ops._vllm_fa2_C.varlen_fwd(
        q, k, v, out, cu_seqlens_q,
        # cu_seqlens_k is not used with seqused_k, but the op's schema wants a tensor
        dummy_cu_seqlens_k if cu_seqlens_k is None else cu_seqlens_k,
        seqused_k, None, block_table, alibi_slopes, max_seqlen_q, max_seqlen_k, dropout_p, softmax_scale, s_aux,
        False, causal, real_window_size[0], real_window_size[1], softcap, False, None)
    return out
