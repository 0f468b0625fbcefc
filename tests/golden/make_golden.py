"""Generates the golden fixtures in this folder from the reference project.

Run where the reference checkout is available (it is NOT needed to run the tests):

    python tests/golden/make_golden.py --reference <path to a checkout of the reference project>

What comes from the reference, imported as Python and executed on the CPU:
  * the cache factories ``create_kv_caches_with_random`` (paged layout) and
    ``create_kv_caches_with_random_flash`` (flash layout, ``[:, 0]`` / ``[:, 1]``
    views of one allocation) and ``seed_everything`` from its tests/utils.py;
  * PyTorch's own ``float -> float8`` cast, which is the conversion the reference
    kernels call (csrc/quantization/fp8/quant_utils.h:70-74 there).
  * ``RotaryEmbedding`` from its tests/ops/rotary_embedding_op.py: the cos/sin table recipe and
    ``forward_native``, the torch statement of the rotary embedding op (imported with empty
    stand-ins for the compiled ``vllm_xpu_kernels._C*`` modules, which that file imports but
    ``forward_native`` never calls).
What is restated here because it only exists inline in GPU-only test functions:
  * the MLA and gather recipes and expectations (tests/test_cache.py:337-375, :423-477);
  * the input recipe (``qkv = randn(T, 3, H, D); _, key, value = qkv.unbind(1)``,
    ``random.sample`` slots: tests/test_cache.py:88-93, :211-222) and
  * the expected-result loops (tests/test_cache.py:155-164 paged, :284-292 flash).

Each ``*.npz`` holds the inputs, the caches before the call and the caches the
reference's loop produces.  16-bit floats are stored as uint16 bit patterns and
fp8 as uint8, so the files are readable without torch.
"""
from __future__ import annotations

import argparse
import importlib
import importlib.util
import os
import random
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

DT = {"half": torch.half, "bfloat16": torch.bfloat16, "float": torch.float}


def load_reference_utils(ref_root: str):
    spec = importlib.util.spec_from_file_location("reference_tests_utils", os.path.join(ref_root, "tests", "utils.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def load_reference_rotary(ref_root: str):
    """The reference's RotaryEmbedding class.  Its module imports the compiled extension modules at
    import time; forward_native is pure torch, so empty stand-ins are enough."""
    saved = {k: sys.modules.pop(k) for k in list(sys.modules) if k == "tests" or k.startswith("tests.")
             or k == "vllm_xpu_kernels" or k.startswith("vllm_xpu_kernels.")}
    try:
        pkg = types.ModuleType("vllm_xpu_kernels")
        pkg.__path__ = []
        sys.modules["vllm_xpu_kernels"] = pkg
        for sub in ("_C", "_moe_C", "_xpu_C"):
            sys.modules["vllm_xpu_kernels." + sub] = types.ModuleType("vllm_xpu_kernels." + sub)
        sys.path.insert(0, ref_root)
        try:
            mod = importlib.import_module("tests.ops.rotary_embedding_op")
        finally:
            sys.path.remove(ref_root)
        return mod.RotaryEmbedding
    finally:
        for k in [k for k in sys.modules if k == "tests" or k.startswith("tests.") or k == "vllm_xpu_kernels"
                  or k.startswith("vllm_xpu_kernels.")]:
            del sys.modules[k]
        sys.modules.update(saved)


def load_reference_paged_attn(ref_root: str):
    """``ref_paged_attn`` from the reference's tests/flash_attn/test_flash_attn_varlen_func.py.  That file
    imports the compiled attention interface at import time; the reference function is pure torch."""
    names = ("vllm_xpu_kernels", "vllm_xpu_kernels.flash_attn_interface")
    saved = {k: sys.modules.pop(k) for k in list(sys.modules) if k in names}
    try:
        pkg = types.ModuleType("vllm_xpu_kernels")
        pkg.__path__ = []
        iface = types.ModuleType("vllm_xpu_kernels.flash_attn_interface")
        iface.flash_attn_varlen_func = None
        sys.modules.update({names[0]: pkg, names[1]: iface})
        spec = importlib.util.spec_from_file_location(
            "reference_test_flash_attn", os.path.join(ref_root, "tests", "flash_attn", "test_flash_attn_varlen_func.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        return mod.ref_paged_attn
    finally:
        for k in names:
            sys.modules.pop(k, None)
        sys.modules.update(saved)


def bits(t: torch.Tensor) -> np.ndarray:
    """Raw storage of a (possibly strided) tensor as a contiguous numpy array."""
    t = t.contiguous()
    if t.dtype in (torch.half, torch.bfloat16):
        return t.view(torch.int16).numpy().view(np.uint16).copy()
    if t.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
        return t.view(torch.uint8).numpy().copy()
    return t.numpy().copy()


def quantise_like_reference(x: torch.Tensor, scale: torch.Tensor, kv_cache_dtype: str) -> torch.Tensor:
    """float(src) / scale, then torch's cast (quant_utils.h:70-74 of the reference)."""
    q = x.float() / scale
    return q.to(torch.float8_e5m2 if kv_cache_dtype == "fp8_e5m2" else torch.float8_e4m3fn)


def make_case(ru, layout: str, dtype: str, kv_cache_dtype: str, T: int, H: int, D: int, bs: int, nb: int,
              seed: int, scale_div: float, n_skip: int = 0) -> dict:
    tdt = DT[dtype]
    ru.seed_everything(seed)
    slots = random.sample(range(nb * bs), T)
    for i in random.sample(range(T), n_skip):
        slots[i] = -1
    slot_mapping = torch.tensor(slots, dtype=torch.long)
    qkv = torch.randn(T, 3, H, D, dtype=tdt)
    _, key, value = qkv.unbind(dim=1)
    factory = ru.create_kv_caches_with_random_flash if layout == "flash" else ru.create_kv_caches_with_random
    kcs, vcs = factory(nb, bs, 1, H, D, kv_cache_dtype, tdt, seed=seed, device="cpu")
    key_cache, value_cache = kcs[0], vcs[0]
    if scale_div == 64.0:  # the reference tests' recipe (tests/test_cache.py:110-111)
        k_scale = (key.amax() / scale_div).to(torch.float32)
        v_scale = (value.amax() / scale_div).to(torch.float32)
    else:  # deployment recipe: nothing saturates
        k_scale = (key.float().abs().amax() / scale_div).to(torch.float32)
        v_scale = (value.float().abs().amax() / scale_div).to(torch.float32)

    exp_k, exp_v = key_cache.contiguous().clone(), value_cache.contiguous().clone()
    if kv_cache_dtype == "auto":
        src_k, src_v = key, value
    else:
        src_k = quantise_like_reference(key, k_scale, kv_cache_dtype)
        src_v = quantise_like_reference(value, v_scale, kv_cache_dtype)
    for i in range(T):
        if slots[i] < 0:  # csrc/cache.cpp:49, :145
            continue
        blk, off = slots[i] // bs, slots[i] % bs
        if layout == "flash":
            exp_k[blk, off, :, :] = src_k[i]
            exp_v[blk, off, :, :] = src_v[i]
        else:
            x = exp_k.shape[4]
            exp_k[blk, :, :, off, :] = src_k[i].reshape(H, D // x, x)
            exp_v[blk, :, :, off] = src_v[i]
    return dict(
        layout=layout, dtype=dtype, kv_cache_dtype=kv_cache_dtype, T=T, H=H, D=D, block_size=bs, num_blocks=nb,
        qkv=bits(qkv), slot_mapping=slot_mapping.numpy(), key_cache_before=bits(key_cache),
        value_cache_before=bits(value_cache), key_cache_after=bits(exp_k), value_cache_after=bits(exp_v),
        k_scale=np.float32(k_scale.item()), v_scale=np.float32(v_scale.item()),
        max_abs_scaled=np.float32(max((key.float() / k_scale).abs().max().item(),
                                      (value.float() / v_scale).abs().max().item())),
        cache_is_view=np.bool_(layout == "flash"))


def make_mla_case(ru, dtype: str, kv_cache_dtype: str, T: int, R: int, P: int, bs: int, nb: int, seed: int,
                  n_skip: int = 0) -> dict:
    """Recipe of tests/test_cache.py:337-375 of the reference (inputs, zero cache, placement loop);
    fp8 expectation = torch's cast of float(x) / scale."""
    tdt = DT[dtype]
    ru.seed_everything(seed)
    slots = random.sample(range(nb * bs), T)
    for i in random.sample(range(T), n_skip):
        slots[i] = -1
    kv_c = torch.randn(T, R, dtype=tdt)
    k_pe = torch.randn(T, P, dtype=tdt)
    scale = torch.tensor(0.1, dtype=torch.float32)
    cdt = tdt if kv_cache_dtype == "auto" else torch.float8_e4m3fn
    before = torch.zeros(nb, bs, R + P, dtype=torch.uint8 if cdt != tdt else tdt)
    before = before.view(cdt) if cdt != tdt else before
    after = before.clone()
    src_c = kv_c if kv_cache_dtype == "auto" else quantise_like_reference(kv_c, scale, kv_cache_dtype)
    src_p = k_pe if kv_cache_dtype == "auto" else quantise_like_reference(k_pe, scale, kv_cache_dtype)
    for i in range(T):
        if slots[i] < 0:
            continue
        blk, off = slots[i] // bs, slots[i] % bs
        after[blk, off, :R] = src_c[i]
        after[blk, off, R:] = src_p[i]
    return dict(op="mla", dtype=dtype, kv_cache_dtype=kv_cache_dtype, kv_c=bits(kv_c), k_pe=bits(k_pe),
                slot_mapping=np.array(slots, dtype=np.int64), block_size=bs, scale=np.float32(0.1),
                cache_before=bits(before), cache_after=bits(after))


def make_gather_case(ru, dtype: str, entry: int, bs: int, nb: int, batch: int, max_seq_len: int, seed: int,
                     with_seq_starts: bool) -> dict:
    """Recipe of tests/test_cache.py:423-477 of the reference: random cache, per-sequence block
    permutations, expected = concatenation of the sequences' blocks (last one partial)."""
    tdt = DT[dtype]
    ru.seed_everything(seed)
    src = torch.randn(nb, bs, entry, dtype=tdt)
    seq_lens = torch.randint(0, max_seq_len + 1, (batch,))
    cu = torch.zeros(batch + 1, dtype=torch.int32)
    cu[1:] = seq_lens.cumsum(0).to(torch.int32)
    block_table = torch.stack([torch.randperm(nb) for _ in range(batch)]).to(torch.int32)
    seq_starts = None
    if with_seq_starts:
        seq_starts = (torch.randint(0, 3, (batch,)) * bs + torch.randint(0, bs, (batch,))).to(torch.int32)
    rows = []
    for b in range(batch):
        s_len = int(seq_lens[b])
        if s_len == 0:
            continue
        first = int(seq_starts[b]) // bs if with_seq_starts else 0
        tot = (s_len + bs - 1) // bs
        blocks = block_table[b, first:first + tot].tolist()
        parts = [src[blk] for blk in blocks[:-1]]
        parts.append(src[blocks[-1], :s_len - (tot - 1) * bs])
        rows.append(torch.cat(parts, dim=0))
    expected = torch.cat(rows, dim=0) if rows else torch.zeros(0, entry, dtype=tdt)
    out = dict(op="gather", dtype=dtype, src_cache=bits(src), block_table=block_table.numpy(), cu_seq_lens=cu.numpy(),
               batch_size=batch, expected=bits(expected))
    if with_seq_starts:
        out["seq_starts"] = seq_starts.numpy()
    return out


def make_quant_case(ru, dtype: str, fp8: str, T: int, hidden: int, seed: int, with_ub: bool) -> dict:
    """The torch recipes of tests/test_fp8_quant.py:20-75 of the reference, run on the CPU:
    dynamic per-tensor (out = cast(clamp(x * (1/scale))), scale = absmax / fp8_max) and dynamic per-token
    (scales = clamp(min(absmax_t, ub) / fp8_max, min = 1/(512 fp8_max)), out = cast(clamp(x / scales)))."""
    tdt = DT[dtype]
    fdt = torch.float8_e5m2 if fp8 == "fp8_e5m2" else torch.float8_e4m3fn
    fi = torch.finfo(fdt)
    ru.seed_everything(seed)
    x = torch.rand(T, hidden, dtype=tdt) + 1e-6
    fp8_max = torch.as_tensor(fi.max, dtype=torch.float32)
    one = torch.as_tensor(1.0, dtype=torch.float32)
    scale = x.abs().max().to(torch.float32) / fp8_max
    out_tensor = (x.to(torch.float32) * (one / scale)).clamp(fi.min, fi.max).to(fdt)
    tok_max = x.abs().max(dim=-1)[0].to(torch.float32)
    ub = torch.mean(x).to(torch.float32) if with_ub else None
    if ub is not None:
        tok_max = tok_max.clamp(max=ub)
    scales = (tok_max / fp8_max)[:, None].clamp(min=one / (fp8_max * 512.0))
    out_token = (x.to(torch.float32) / scales).clamp(fi.min, fi.max).to(fdt)
    d = dict(op="quant", dtype=dtype, fp8=fp8, x=bits(x), scale=np.float32(scale.item()), out_tensor=bits(out_tensor),
             scales=scales.numpy(), out_token=bits(out_token))
    if ub is not None:
        d["scale_ub"] = np.float32(ub.item())
    return d


def make_rope_case(RotaryEmbedding, dtype: str, is_neox: bool, head_size: int, rot_dim: int, max_position: int,
                   seq_len: int, num_heads: int, num_kv_heads: int, use_key: bool, head_pad: int, flat: bool,
                   seed: int) -> dict:
    """Inputs as in tests/test_rotary_embedding.py:52-87 of the reference (randint positions, randn
    query/key cut out of a wider last dim when ``head_pad``, optionally flattened to
    [.., heads * head_size]); expected = RotaryEmbedding.forward_native on the CPU with the table cast
    to the tensors' type, which is what the op is handed (tests/test_rotary_embedding.py:21)."""
    tdt = DT[dtype]
    torch.manual_seed(seed)
    rot = RotaryEmbedding(head_size, rot_dim, max_position, 10000, is_neox, torch.float32)
    table = rot.cos_sin_cache.to(tdt)
    rot.cos_sin_cache = table
    positions = torch.randint(0, max_position, (seq_len,))
    q_store = torch.randn(seq_len, num_heads, head_size + head_pad, dtype=tdt)
    k_store = torch.randn(seq_len, num_kv_heads, head_size + head_pad, dtype=tdt)
    query = q_store[..., :head_size]
    key = k_store[..., :head_size] if use_key else None
    if flat:
        assert head_pad == 0
        query = query.flatten(start_dim=-2)
        key = key.flatten(start_dim=-2) if use_key else None
    q_out, k_out = rot.forward_native(positions, query.clone(), key.clone() if use_key else None)
    d = dict(op="rope", dtype=dtype, is_neox=np.bool_(is_neox), head_size=head_size, rot_dim=rot_dim, flat=np.bool_(flat),
             head_pad=head_pad, positions=positions.numpy(), cos_sin_cache=bits(table), query_store=bits(q_store),
             query_after=bits(q_out.reshape(seq_len, num_heads, head_size)))
    if use_key:
        d["key_store"] = bits(k_store)
        d["key_after"] = bits(k_out.reshape(seq_len, num_kv_heads, head_size))
    return d


def make_decode_attn_case(ref_paged_attn, dtype: str, num_heads: int, num_kv_heads: int, head_size: int,
                          kv_lens: list, block_size: int, num_blocks: int, with_sink: bool, kv_cache_dtype: str,
                          descale: float, seed: int, query_lens: list | None = None, causal: bool = False,
                          window: tuple = (-1, -1), paged: bool = True) -> dict:
    """Inputs as in test_decode_with_paged_kv of the reference (tests/flash_attn/test_flash_attn_varlen_func.py:
    274-372: one query token per sequence, randn query and caches, randint block tables, optional randn sink);
    expected = its ref_paged_attn on the CPU.  For an fp8 cache the caches are first cast to fp8; the reference
    function then sees their exact 16-bit images times a power-of-two descale."""
    tdt = DT[dtype]
    torch.manual_seed(seed)
    num_seqs = len(kv_lens)
    query_lens = query_lens or [1] * num_seqs
    query = torch.randn(sum(query_lens), num_heads, head_size, dtype=tdt)
    if paged:
        key_cache = torch.randn(num_blocks, block_size, num_kv_heads, head_size, dtype=tdt)
    else:  # keys/values of all sequences back to back: [sum(kv_lens), heads, head_size]
        key_cache = torch.randn(sum(kv_lens), num_kv_heads, head_size, dtype=tdt)
    value_cache = torch.randn_like(key_cache)
    max_blocks = (max(kv_lens) + block_size - 1) // block_size
    block_tables = torch.randint(0, num_blocks, (num_seqs, max_blocks), dtype=torch.int32)
    sink = torch.randn(num_heads, dtype=tdt) if with_sink else None
    stored_k, stored_v = key_cache, value_cache
    if kv_cache_dtype != "auto":
        fdt = torch.float8_e5m2 if kv_cache_dtype == "fp8_e5m2" else torch.float8_e4m3fn
        stored_k, stored_v = (key_cache / descale).to(fdt), (value_cache / descale).to(fdt)
        key_cache, value_cache = (stored_k.to(tdt) * descale), (stored_v.to(tdt) * descale)
        assert torch.equal(key_cache.float(), stored_k.float() * descale)  # the 16-bit image is exact
    scale = head_size ** -0.5
    expected = ref_paged_attn(query=query.clone(), key_cache=key_cache, value_cache=value_cache,
                              query_lens=query_lens, kv_lens=kv_lens, block_tables=block_tables, scale=scale,
                              casual=causal, is_paged=paged, sink=sink, window_size_left=window[0],
                              window_size_right=window[1])
    d = dict(op="decode_attn", dtype=dtype, kv_cache_dtype=kv_cache_dtype, query=bits(query),
             key_cache=bits(stored_k), value_cache=bits(stored_v), block_tables=block_tables.numpy(),
             kv_lens=np.array(kv_lens, dtype=np.int32), query_lens=np.array(query_lens, dtype=np.int32),
             causal=np.bool_(causal), window=np.array(window, dtype=np.int64), paged=np.bool_(paged),
             scale=np.float32(scale), descale=np.float32(descale), expected=bits(expected))
    if with_sink:
        d["sink"] = bits(sink)
    return d


def make_tables() -> dict:
    """torch's e4m3 / e5m2 cast over every bf16 and fp16 bit pattern at a few scales."""
    out = {}
    pats = torch.arange(65536, dtype=torch.int32).to(torch.int16)
    scales = np.array([1.0, 0.0078125, 0.013671875, 3.7, 0.3333333432674408, 2.2321429569274187e-03], dtype=np.float32)
    out["scales"] = scales
    for name, tdt in (("bf16", torch.bfloat16), ("f16", torch.float16)):
        x = pats.view(tdt).float()
        for kv, fdt in (("e4m3", torch.float8_e4m3fn), ("e5m2", torch.float8_e5m2)):
            rows = [(x / torch.tensor(float(s), dtype=torch.float32)).to(fdt).view(torch.uint8).numpy() for s in scales]
            out[f"{name}_{kv}"] = np.stack(rows)
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path to a checkout of the reference project")
    ap.add_argument("--only", default=None, help="write only the fixtures whose name starts with this prefix")
    ns = ap.parse_args()
    ru = load_reference_utils(ns.reference)
    RotaryEmbedding = load_reference_rotary(ns.reference)
    ref_paged_attn = load_reference_paged_attn(ns.reference)

    def wanted(name: str) -> bool:
        return ns.only is None or name.startswith(ns.only)

    cases = []
    # auto: the reference's own matrix (dtypes x head sizes x block sizes, tests/test_cache.py:14-19),
    # shrunk in tokens/heads/blocks so the fixtures stay small
    hs_bs = [(64, 8), (80, 16), (120, 32), (256, 16), (128, 16)]
    for layout in ("flash", "paged"):
        for dtype in ("half", "bfloat16", "float"):
            for D, bs in hs_bs:
                if dtype == "float" and D in (80, 128):
                    continue
                cases.append(dict(layout=layout, dtype=dtype, kv_cache_dtype="auto", T=20, H=2, D=D, bs=bs,
                                  nb=max(2, 32 // bs + 1), seed=0, scale_div=64.0))
        # the reference's MINI profile (tests/test_cache.py:40-46): 1 token, head_size 8, 4 blocks of 8
        cases.append(dict(layout=layout, dtype="half", kv_cache_dtype="auto", T=1, H=8, D=8, bs=8, nb=4, seed=0,
                          scale_div=64.0))
        # padding: a third of the tokens carry slot -1
        cases.append(dict(layout=layout, dtype="bfloat16", kv_cache_dtype="auto", T=21, H=2, D=64, bs=16, nb=3,
                          seed=5, scale_div=64.0, n_skip=7))
        # fp8: scale = amax/64 as in the reference's (disabled) fp8 branch, and amax/448 as deployed
        for dtype in ("half", "bfloat16"):
            for div in (64.0, 448.0):
                cases.append(dict(layout=layout, dtype=dtype, kv_cache_dtype="fp8", T=20, H=2, D=64 if div == 64.0 else 128,
                                  bs=16, nb=3, seed=1, scale_div=div))
        cases.append(dict(layout=layout, dtype="float", kv_cache_dtype="fp8", T=20, H=2, D=64, bs=16, nb=3, seed=2,
                          scale_div=448.0))
        cases.append(dict(layout=layout, dtype="bfloat16", kv_cache_dtype="fp8_e5m2", T=20, H=2, D=64, bs=16, nb=3,
                          seed=3, scale_div=64.0))

    names = []
    for c in cases:
        name = "{layout}_{dtype}_{kv_cache_dtype}_T{T}_H{H}_D{D}_bs{bs}_nb{nb}_s{seed}_div{d}".format(
            d=int(c["scale_div"]), **c) + ("_skip" if c.get("n_skip") else "")
        names.append(name)
        if wanted(name):
            np.savez_compressed(os.path.join(HERE, name + ".npz"), **make_case(ru, **c))
    extra = []
    for dtype in ("half", "bfloat16", "float"):
        extra.append(("mla_%s_auto_T42_R512_P64_bs16_nb8" % dtype, make_mla_case(ru, dtype, "auto", 42, 512, 64, 16, 8, 0)))
    extra.append(("mla_bfloat16_fp8_T42_R512_P64_bs16_nb8", make_mla_case(ru, "bfloat16", "fp8", 42, 512, 64, 16, 8, 1)))
    extra.append(("mla_half_fp8_T21_R64_P16_bs8_nb4_skip", make_mla_case(ru, "half", "fp8", 21, 64, 16, 8, 4, 2, n_skip=6)))
    extra.append(("mla_half_auto_T1_R512_P64_bs8_nb4", make_mla_case(ru, "half", "auto", 1, 512, 64, 8, 4, 0)))
    extra.append(("gather_float_E576_bs16_nb16_B4", make_gather_case(ru, "float", 576, 16, 16, 4, 60, 0, False)))
    extra.append(("gather_bfloat16_E576_bs16_nb24_B6_starts", make_gather_case(ru, "bfloat16", 576, 16, 24, 6, 64, 1, True)))
    extra.append(("gather_half_E40_bs8_nb16_B5", make_gather_case(ru, "half", 40, 8, 16, 5, 30, 2, False)))
    qi = 0
    for dtype in ("half", "bfloat16", "float"):
        for fp8 in ("fp8_e4m3", "fp8_e5m2"):
            for T, hidden in ((7, 67), (5, 1024), (3, 1031)):
                extra.append(("quant_%s_%s_T%d_h%d" % (dtype, fp8, T, hidden),
                              make_quant_case(ru, dtype, fp8, T, hidden, qi, with_ub=bool(qi % 2))))
                qi += 1
    # rotary embedding: the reference test's matrix (tests/test_rotary_embedding.py:43-51: neox / gpt-j,
    # head sizes 32 and 108 with rotary_dim 32, with and without key, padded heads, flat layout), shrunk to
    # 11 tokens, in all three types, plus full rotation at head size 128 with grouped kv heads
    ri = 100
    for dtype in ("float", "half", "bfloat16"):
        for is_neox in (True, False):
            for head_size, rot_dim, hq, hk, use_key, pad, flat in (
                    (32, 32, 7, 7, True, 0, False), (108, 32, 7, 7, True, 64, False), (108, 32, 7, 7, False, 0, True),
                    (32, 32, 7, 7, True, 0, True), (128, 128, 8, 2, True, 0, False), (64, 48, 3, 1, True, 0, False)):
                ri += 1
                name = "rope_%s_%s_D%d_R%d_Hq%d_Hk%d%s%s%s" % (
                    dtype, "neox" if is_neox else "gptj", head_size, rot_dim, hq, hk, "" if use_key else "_nokey",
                    "_pad%d" % pad if pad else "", "_flat" if flat else "")
                extra.append((name, lambda a=(dtype, is_neox, head_size, rot_dim, 257 if ri % 2 else 11, 11, hq, hk,
                                               use_key, pad, flat, ri): make_rope_case(RotaryEmbedding, *a)))
    # paged decode attention: the head-count pairs, both types and the sink switch of the reference's decode
    # test (tests/flash_attn/test_flash_attn_varlen_func.py:14-24, :274-288), with smaller caches and shorter
    # sequences (one of them a single token, one crossing many blocks); fp8 caches on top
    ai = 200
    for dtype, hq, hk, D, lens, bs, nb, sink, kv, descale in (
            ("bfloat16", 8, 2, 128, [300, 37, 129], 16, 24, False, "auto", 1.0),
            ("half", 4, 4, 64, [1, 523, 64], 16, 16, True, "auto", 1.0),
            ("bfloat16", 10, 2, 64, [65, 17, 250], 16, 16, True, "auto", 1.0),
            ("half", 16, 1, 128, [200, 33], 32, 8, False, "auto", 1.0),
            ("bfloat16", 16, 1, 192, [100], 64, 3, False, "auto", 1.0),
            ("half", 8, 2, 256, [130, 5], 64, 4, True, "auto", 1.0),
            ("bfloat16", 8, 2, 128, [300, 37, 129], 16, 24, False, "fp8", 0.5),
            ("half", 4, 4, 64, [70, 523], 16, 16, True, "fp8", 2.0),
            ("bfloat16", 10, 2, 128, [90, 260], 32, 10, True, "fp8_e5m2", 1.0)):
        ai += 1
        name = "decode_attn_%s_%s_Hq%d_Hk%d_D%d_bs%d%s" % (dtype, kv, hq, hk, D, bs, "_sink" if sink else "")
        extra.append((name, lambda a=(dtype, hq, hk, D, lens, bs, nb, sink, kv, descale, ai):
                      make_decode_attn_case(ref_paged_attn, *a)))
    # variable query lengths: the sequence list of the reference's test_varlen_with_paged_kv
    # (tests/flash_attn/test_flash_attn_varlen_func.py:121: (1, 1328), (5, 18), (129, 463)), shortened, with and
    # without the causal mask and the sink, plus an fp8 cache
    for dtype, hq, hk, D, lens, bs, nb, sink, kv, descale, causal in (
            ("bfloat16", 8, 2, 128, [(1, 328), (5, 18), (129, 263)], 16, 24, False, "auto", 1.0, True),
            ("half", 4, 4, 64, [(1, 328), (5, 18), (129, 263)], 16, 24, True, "auto", 1.0, True),
            ("bfloat16", 10, 2, 64, [(7, 7), (33, 200), (1, 1)], 16, 16, True, "auto", 1.0, False),
            ("half", 16, 1, 128, [(40, 100), (3, 64)], 32, 8, False, "auto", 1.0, True),
            ("bfloat16", 8, 2, 128, [(1, 328), (5, 18), (129, 263)], 16, 24, True, "fp8", 0.5, True)):
        ai += 1
        name = "varlen_attn_%s_%s_Hq%d_Hk%d_D%d_bs%d%s%s" % (dtype, kv, hq, hk, D, bs, "_sink" if sink else "",
                                                         "_causal" if causal else "")
        extra.append((name, lambda a=(dtype, hq, hk, D, [k for _, k in lens], bs, nb, sink, kv, descale, ai,
                                       [q for q, _ in lens], causal): make_decode_attn_case(ref_paged_attn, *a)))
    # sliding windows (the reference's SLIDING_WINDOWS, tests/flash_attn/test_flash_attn_varlen_func.py:20) and the
    # non-paged form (keys/values of all sequences back to back, as many kv heads as query heads, :183-187)
    for dtype, hq, hk, D, lens, bs, nb, sink, causal, window, paged in (
            ("bfloat16", 8, 2, 128, [(1, 328), (5, 18), (129, 263)], 16, 24, False, False, (-1, 127), True),
            ("half", 8, 2, 64, [(1, 328), (5, 18), (129, 263)], 16, 24, True, True, (127, -1), True),
            ("bfloat16", 4, 4, 64, [(1, 328), (5, 18), (129, 263)], 16, 24, False, True, (127, 127), True),
            ("half", 10, 2, 128, [(1, 700), (40, 300)], 32, 24, True, False, (63, 0), True),
            ("bfloat16", 4, 4, 64, [(1, 328), (5, 18), (129, 263)], 16, 24, False, True, (-1, -1), False),
            ("half", 4, 4, 128, [(129, 263), (1, 40)], 16, 24, True, False, (-1, -1), False)):
        ai += 1
        name = "window_attn_%s_Hq%d_Hk%d_D%d%s%s_w%s_%s%s" % (
            dtype, hq, hk, D, "_sink" if sink else "", "_causal" if causal else "",
            str(window[0]).replace("-", "m"), str(window[1]).replace("-", "m"), "" if paged else "_dense")
        extra.append((name, lambda a=(dtype, hq, hk, D, [k for _, k in lens], bs, nb, sink, "auto", 1.0, ai,
                                       [q for q, _ in lens], causal, window, paged):
                      make_decode_attn_case(ref_paged_attn, *a)))
    for name, data in extra:
        names.append(name)
        if wanted(name):
            np.savez_compressed(os.path.join(HERE, name + ".npz"), **(data() if callable(data) else data))
    if wanted("fp8_tables"):
        np.savez_compressed(os.path.join(HERE, "fp8_tables.npz"), **make_tables())
    with open(os.path.join(HERE, "MANIFEST.txt"), "w") as f:
        f.write("# written by make_golden.py with torch %s\n" % torch.__version__)
        for n in names + ["fp8_tables"]:
            f.write(n + ".npz\n")
    total = sum(os.path.getsize(os.path.join(HERE, n + ".npz")) for n in names + ["fp8_tables"])
    print(f"{len(names)} cases + tables, {total / 1e6:.2f} MB")


if __name__ == "__main__":
    main()
