"""numpy views of CPU torch tensors for the oracle -- TEST INFRASTRUCTURE ONLY.

The oracle itself is torch-free; callers that hold torch tensors (tests, the smoke check,
the benchmark's CPU-baseline leg) use these views so strides survive the hand-over."""
import numpy as np
import torch

ORC_IN = {torch.float16: "f16", torch.bfloat16: "bf16", torch.float32: "f32"}


def as_np(t: torch.Tensor) -> np.ndarray:
    """numpy view with the same strides; 16-bit floats as uint16 bit patterns, fp8 as uint8."""
    assert not t.is_cuda
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.view(torch.int16).numpy().view(np.uint16)
    if t.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
        return t.view(torch.uint8).numpy()
    return t.numpy()


def run(layout: str, key, value, key_cache, value_cache, slot_mapping, kv_cache_dtype: str,
        k_scale: float, v_scale: float, threads: int = 1) -> None:
    """Runs the oracle in place on CPU torch tensors."""
    import oracle
    fn = oracle.reshape_and_cache_flash if layout == "flash" else oracle.reshape_and_cache
    fn(as_np(key), as_np(value), as_np(key_cache), as_np(value_cache), slot_mapping.numpy(), kv_cache_dtype,
       float(k_scale), float(v_scale), ORC_IN[key.dtype], threads=threads)


def run_mla(kv_c, k_pe, kv_cache, slot_mapping, kv_cache_dtype: str, scale: float) -> None:
    import oracle
    oracle.concat_and_cache_mla(as_np(kv_c), as_np(k_pe), as_np(kv_cache), slot_mapping.numpy(), kv_cache_dtype,
                                float(scale), ORC_IN[kv_c.dtype])


def run_gather(src_cache, dst, block_table, cu_seq_lens, batch_size: int, seq_starts=None) -> None:
    import oracle
    oracle.gather_cache(as_np(src_cache), as_np(dst), block_table.numpy(), cu_seq_lens.numpy(), batch_size,
                        None if seq_starts is None else seq_starts.numpy())


def run_rope(positions, query, key, head_size: int, cos_sin_cache, is_neox: bool) -> None:
    """In-place rotary embedding on CPU torch tensors: positions [T] or [B, S]; query/key
    [.., heads, head_size] or [.., heads * head_size] (leading dims collapse to tokens)."""
    import oracle

    def tokens_first(t):
        if t is None:
            return None
        lead = positions.dim()
        return t.reshape(-1, *t.shape[lead:]) if lead > 1 else t

    q, k = tokens_first(query), tokens_first(key)
    assert q.data_ptr() == query.data_ptr() and (k is None or k.data_ptr() == key.data_ptr()), "reshape copied"
    oracle.rotary_embedding(positions.reshape(-1).numpy(), as_np(q), None if k is None else as_np(k), head_size,
                            as_np(cos_sin_cache), is_neox, ORC_IN[query.dtype])


def run_paged_decode_attention(query, key_cache, value_cache, block_table, seq_lens, scale: float,
                               kv_cache_dtype: str = "auto", k_descale: float = 1.0, v_descale: float = 1.0,
                               sink=None, cu_seqlens_q=None, causal: bool = False, window=(-1, -1)) -> torch.Tensor:
    """fp32 [tokens, Hq, D] result of the oracle's paged attention on CPU torch tensors (one query token per
    sequence unless ``cu_seqlens_q`` says otherwise)."""
    import oracle
    out = oracle.paged_decode_attention(
        as_np(query), as_np(key_cache), as_np(value_cache), block_table.numpy(), seq_lens.numpy(), scale,
        ORC_IN[query.dtype], kv_cache_dtype, k_descale, v_descale, None if sink is None else as_np(sink),
        None if cu_seqlens_q is None else cu_seqlens_q.numpy(), causal, window)
    return torch.from_numpy(out)
