"""What can be checked about the drop-in boundary without a GPU: the C ABI library loads
and exports every declared symbol, argument validation answers before any CUDA call,
and the torch extension registers the reference's schemas (CUDA only, no CPU path)."""
import ctypes
import os
import re

import pytest
import torch

from tests.conftest import REPO
from vllm_xpu_kernels import cabi


def declared_symbols() -> list[str]:
    names = []
    inc = os.path.join(REPO, "include")
    for fn in sorted(os.listdir(inc)):
        if fn.endswith(".h"):
            text = open(os.path.join(inc, fn)).read()
            names += re.findall(r"KVC_API\s+[\w\s\*]+?\b(kvc_\w+)\s*\(", text)
    return names


def test_header_symbols_are_exported():
    names = declared_symbols()
    assert set(names) == set(cabi.SYMBOLS) and len(names) >= 14
    L = cabi.lib()
    for n in names:
        assert getattr(L, n) is not None
    assert L.kvc_version() >= 100


def test_kv_cache_dtype_strings():
    assert cabi.parse_kv_cache_dtype("auto") == 0
    assert cabi.parse_kv_cache_dtype("fp8") == 1
    assert cabi.parse_kv_cache_dtype("fp8_e4m3") == 1
    assert cabi.parse_kv_cache_dtype("fp8_e5m2") == 2
    with pytest.raises(RuntimeError, match="Unsupported data type of kv cache: int8"):
        cabi.parse_kv_cache_dtype("int8")


def test_argument_validation_needs_no_device():
    L = cabi.lib()
    buf = (ctypes.c_char * 4096)()
    p = ctypes.addressof(buf)
    args = dict(num_tokens=4, H=2, D=16, bs=4)

    def flash(key=p, slots=p, num_tokens=4, in_dtype=2, kv=0, block_size=4, k_scale=0):
        return L.kvc_reshape_and_cache_flash(key, p, p, p, slots, num_tokens, args["H"], args["D"], block_size,
                                             32, 16, 32, 16, 128, 32, 16, in_dtype, kv, k_scale, 0, None)

    assert flash(num_tokens=0) == 0                     # nothing to do: no launch, no error
    assert flash(key=None) == 1 and "non-NULL" in cabi.last_error()
    assert flash(num_tokens=-1) == 1
    assert flash(block_size=0) == 1
    assert flash(in_dtype=7) == 2 and "Unsupported input type" in cabi.last_error()
    assert flash(kv=9) == 2 and "Unsupported data type" in cabi.last_error()
    assert flash(kv=1, k_scale=0) == 1 and "k_scale" in cabi.last_error()
    assert flash(key=p + 1) == 1                         # misaligned for bf16
    # paged: x must divide head_size
    rc = L.kvc_reshape_and_cache(p, p, p, p, p, 4, 2, 16, 4, 5, 32, 16, 32, 16, 2, 0, None, None, None)
    assert rc == 1 and "multiple of x" in cabi.last_error()
    assert L.kvc_count_bad_slots(p, 4, 16, None, None) == 1
    # gather: element width must be 1, 2 or 4 bytes (message of csrc/cache.cpp:636 in the reference)
    rc = L.kvc_gather_cache(p, p, p, p, None, 2, 8, 4, 16, 8, 4, 64, 16, 16, None)
    assert rc == 2 and "Unsupported data type width: 64" in cabi.last_error()
    assert L.kvc_gather_cache(p, p, p, p, None, 0, 8, 4, 16, 2, 4, 64, 16, 16, None) == 0  # empty batch
    assert L.kvc_concat_and_cache_mla(None, p, p, p, 4, 16, 8, 4, 16, 8, 96, 24, 2, 0, None, None) == 1


def test_torch_extension_registers_reference_schemas():
    import vllm_xpu_kernels._C  # noqa: F401
    ops = torch.ops._C_cache_ops
    # the reference's schema text (csrc/torch_bindings.cpp:107-112, :116-122), parsed by torch
    want = ("(Tensor key, Tensor value, Tensor! key_cache, Tensor! value_cache, Tensor slot_mapping, "
            "str kv_cache_dtype, Tensor k_scale, Tensor v_scale) -> ()")
    for name in ("reshape_and_cache", "reshape_and_cache_flash"):
        schema = getattr(ops, name).default._schema
        assert str(schema) == str(torch._C.parse_schema(f"_C_cache_ops::{name}{want}"))
        assert [a.name for a in schema.arguments] == ["key", "value", "key_cache", "value_cache", "slot_mapping",
                                                      "kv_cache_dtype", "k_scale", "v_scale"]
        muts = [a.name for a in schema.arguments if a.alias_info is not None and a.alias_info.is_write]
        assert muts == ["key_cache", "value_cache"]
    # the other two ops of the namespace (csrc/torch_bindings.cpp:127-133, :136-139 of the reference)
    others = {
        "concat_and_cache_mla": "(Tensor kv_c, Tensor k_pe, Tensor! kv_cache, Tensor slot_mapping, "
                                "str kv_cache_dtype, Tensor scale) -> ()",
        "gather_cache": "(Tensor src_cache, Tensor! dst, Tensor block_table, Tensor cu_seq_lens, int batch_size, "
                        "Tensor? seq_starts) -> ()",
    }
    for name, sig in others.items():
        assert str(getattr(ops, name).default._schema) == str(torch._C.parse_schema(f"_C_cache_ops::{name}{sig}"))
    quant = {
        "static_scaled_fp8_quant": "(Tensor! result, Tensor input, Tensor scale) -> ()",
        "dynamic_scaled_fp8_quant": "(Tensor! result, Tensor input, Tensor! scale) -> ()",
        "dynamic_per_token_scaled_fp8_quant": "(Tensor! result, Tensor input, Tensor! scale, Tensor? scale_ub) -> ()",
    }
    for name, sig in quant.items():  # csrc/torch_bindings.cpp:67-88 of the reference
        assert str(getattr(torch.ops._C, name).default._schema) == str(torch._C.parse_schema(f"_C::{name}{sig}"))
    # csrc/torch_bindings.cpp:61-64 of the reference
    rope = "(Tensor positions, Tensor! query, Tensor!? key, int head_size, Tensor cos_sin_cache, bool is_neox) -> ()"
    assert str(torch.ops._C.rotary_embedding.default._schema) == str(
        torch._C.parse_schema("_C::rotary_embedding" + rope))
    # csrc/flash_attn/flash_api.cpp:179-193 of the reference
    fa = ("(Tensor q, Tensor k, Tensor v, Tensor!? out, Tensor cu_seqlens_q, Tensor cu_seqlens_k, Tensor? seqused_k, "
          "Tensor? leftpad_k, Tensor? block_table, Tensor? alibi_slopes, int max_seqlen_q, int max_seqlen_k, "
          "float p_dropout, float softmax_scale, Tensor? softmax_sink, bool zero_tensors, bool is_causal, "
          "int window_size_left, int window_size_right, float softcap, bool return_softmax, Generator? gen) -> Tensor[]")
    assert str(torch.ops._vllm_fa2_C.varlen_fwd.default._schema) == str(
        torch._C.parse_schema("_vllm_fa2_C::varlen_fwd" + fa))
    from vllm_xpu_kernels import flash_attn_interface
    import inspect
    params = list(inspect.signature(flash_attn_interface.flash_attn_varlen_func).parameters)
    # vllm_xpu_kernels/flash_attn_interface.py:24-53 of the reference, in order
    assert params[:27] == ["q", "k", "v", "max_seqlen_q", "cu_seqlens_q", "max_seqlen_k", "cu_seqlens_k", "seqused_k",
                           "q_v", "dropout_p", "softmax_scale", "causal", "window_size", "softcap", "alibi_slopes",
                           "deterministic", "return_attn_probs", "block_table", "return_softmax_lse", "out",
                           "scheduler_metadata", "q_descale", "k_descale", "v_descale", "num_splits", "fa_version",
                           "s_aux"]
    from vllm_xpu_kernels import ops as wrappers
    for fn in ("reshape_and_cache", "reshape_and_cache_flash", "concat_and_cache_mla", "gather_cache",
               "rotary_embedding", "rotary_embedding_and_cache_flash"):
        assert callable(getattr(wrappers, fn))


def test_rotary_entry_points_validate_without_touching_the_device():
    L = cabi.lib()
    p = ctypes.c_void_p(0x1000)
    # empty batch / no heads: nothing to do
    assert L.kvc_rotary_embedding(p, p, p, p, 0, 8, 2, 64, 64, 100, 512, 64, 128, 64, 1, 2, None) == 0
    assert L.kvc_rotary_embedding(p, None, None, p, 4, 0, 0, 64, 64, 100, 0, 0, 0, 0, 1, 2, None) == 0
    # odd rot_dim, rot_dim > head_size, bad type code, missing table
    assert L.kvc_rotary_embedding(p, p, p, p, 4, 8, 2, 64, 63, 100, 512, 64, 128, 64, 1, 2, None) == 1
    assert "rot_dim" in cabi.last_error()
    assert L.kvc_rotary_embedding(p, p, p, p, 4, 8, 2, 64, 128, 100, 512, 64, 128, 64, 1, 2, None) == 1
    assert L.kvc_rotary_embedding(p, p, p, p, 4, 8, 2, 64, 64, 100, 512, 64, 128, 64, 1, 7, None) == 2
    assert L.kvc_rotary_embedding(p, p, p, None, 4, 8, 2, 64, 64, 100, 512, 64, 128, 64, 1, 2, None) == 1
    # fused: rows of 36 halves cannot be moved in 16-byte pieces -> unsupported, with advice
    args = [p] * 8 + [4, 4, 2, 2, 36, 12, 100, 16, 72, 36, 72, 36, 72, 36, 16 * 72, 72, 36, 1, 1, 1, 0, None, None, None]
    assert L.kvc_rotary_embedding_and_cache_flash(*args) == 2
    assert "kvc_reshape_and_cache_flash" in cabi.last_error()
    args[9] = 5  # more slot tokens than tokens
    assert L.kvc_rotary_embedding_and_cache_flash(*args) == 1


def test_decode_attention_entry_point_validates_without_touching_the_device():
    L = cabi.lib()
    p = ctypes.c_void_p(0x1000)
    f = ctypes.c_float
    # workspace_bytes, num_seqs (0: every call returns before it would launch), num_heads, num_kv_heads, head_size,
    # block_size, block_table_stride, max_seq_len, 4 query/out strides, 3 cache strides, scale, q_dtype, kv_dtype
    base = [p] * 10 + [0, 0, 8, 2, 128, 16, 8, 100, 1024, 128, 1024, 128, 4096, 256, 128, f(0.1), 1, 0, None]
    assert L.kvc_paged_decode_attention(*base) == 0  # no sequences
    bad = list(base); bad[14] = 96      # head size 96
    assert L.kvc_paged_decode_attention(*bad) == 2 and "head_size" in cabi.last_error()
    bad = list(base); bad[12] = 7       # 7 query heads over 2 kv heads
    assert L.kvc_paged_decode_attention(*bad) == 1
    bad = list(base); bad[25] = f(0.0)  # scale must be positive
    assert L.kvc_paged_decode_attention(*bad) == 1 and "softmax_scale" in cabi.last_error()
    bad = list(base); bad[26] = 0       # fp32 query
    assert L.kvc_paged_decode_attention(*bad) == 2
    assert L.kvc_paged_decode_workspace_bytes(0, 8, 2, 128, 100, 1, 0) == 0
    assert L.kvc_paged_decode_workspace_bytes(4, 8, 2, 96, 100, 1, 0) == 0


def test_no_cpu_fallback():
    import vllm_xpu_kernels._C  # noqa: F401
    k = torch.zeros(2, 2, 8)
    c = torch.zeros(2, 2, 2, 8)
    with pytest.raises(NotImplementedError):
        torch.ops._C_cache_ops.reshape_and_cache_flash(k, k, c, c.clone(), torch.zeros(2, dtype=torch.long), "auto",
                                                       torch.ones(1), torch.ones(1))
