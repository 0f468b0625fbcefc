"""The CPU oracle against the fixtures generated from the reference (tests/golden/)."""
import os
import subprocess

import numpy as np
import pytest
import torch

import oracle
from oracle import torch_views
from tests import helpers as H


@pytest.mark.parametrize("fname", H.golden_files())
def test_oracle_reproduces_reference_fixture(fname):
    c = H.GoldenCase(fname)
    if c.kv_cache_dtype != "auto":
        # the reference's cast does not saturate; the two definitions agree while |x/scale| <= 464
        limit = 464.0 if c.kv_cache_dtype != "fp8_e5m2" else 57344.0
        assert c.max_abs_scaled <= limit
    H.oracle_call(c.layout, c.key, c.value, c.key_cache, c.value_cache, c.slot_mapping, c.kv_cache_dtype,
                  c.k_scale, c.v_scale)
    assert H.same_bytes(c.key_cache, c.key_cache_after)
    assert H.same_bytes(c.value_cache, c.value_cache_after)


@pytest.mark.parametrize("fname", H.golden_files("mla"))
def test_oracle_reproduces_reference_mla_fixture(fname):
    c = H.MlaCase(fname)
    cache = c.cache_before.clone()
    torch_views.run_mla(c.kv_c, c.k_pe, cache, c.slot_mapping, c.kv_cache_dtype, c.scale)
    assert H.same_bytes(cache, c.cache_after)


@pytest.mark.parametrize("fname", H.golden_files("gather"))
def test_oracle_reproduces_reference_gather_fixture(fname):
    c = H.GatherCase(fname)
    total = int(c.cu_seq_lens[-1])
    dst = torch.zeros(total + 3, c.expected.shape[1], dtype=c.dtype)  # three spare rows must stay zero
    torch_views.run_gather(c.src_cache, dst, c.block_table, c.cu_seq_lens, c.batch_size, c.seq_starts)
    assert H.same_bytes(dst[:total], c.expected)
    assert not bool(dst[total:].view(torch.uint8).any())


@pytest.mark.parametrize("fname", H.golden_files("quant"))
def test_oracle_reproduces_reference_quant_recipes(fname):
    c = H.QuantCase(fname)
    xn, name = torch_views.as_np(c.x), torch_views.ORC_IN[c.dtype]
    # dynamic per-tensor: same arithmetic as the reference's recipe -> bit-exact, scale included
    assert float(oracle.absmax_scale(xn, name, c.fp8)) == c.scale
    assert np.array_equal(oracle.static_scaled_fp8_quant(xn, c.scale, name, c.fp8), c.out_tensor.numpy())
    # dynamic per-token: the reference's recipe divides where its kernel multiplies by the reciprocal; its own
    # test allows 0.5 % of the bytes to differ (tests/test_fp8_quant.py:199-203) and exact scales
    got, scales = oracle.per_token_fp8_quant(xn, name, c.fp8, c.scale_ub)
    assert np.array_equal(scales, c.scales.numpy())
    assert (got != c.out_token.numpy()).mean() <= 0.005


@pytest.mark.parametrize("fname", H.golden_files("rope"))
def test_oracle_reproduces_reference_rotary_fixture(fname):
    """Expected values come from the reference's RotaryEmbedding.forward_native."""
    c = H.RopeCase(fname)
    q_store = c.query_store.clone()
    k_store = None if c.key_store is None else c.key_store.clone()
    q, k = c.views(q_store, k_store)
    torch_views.run_rope(c.positions, q, k, c.head_size, c.cos_sin_cache, c.is_neox)
    assert H.same_bytes(q_store[..., :c.head_size], c.query_after)
    assert H.same_bytes(q_store[..., c.head_size:], c.query_store[..., c.head_size:])  # padding untouched
    if k_store is not None:
        assert H.same_bytes(k_store[..., :c.head_size], c.key_after)


@pytest.mark.parametrize("fname", H.golden_files("decode_attn"))
def test_oracle_reproduces_reference_decode_attention_fixture(fname):
    """Expected values come from the reference's ref_paged_attn, which rounds the scaled query, the logits and
    the probabilities to the 16-bit type; the oracle keeps everything in double.  Tolerance: the reference
    test's own (atol = rtol = 1e-2)."""
    c = H.DecodeAttnCase(fname)
    got = torch_views.run_paged_decode_attention(c.query, c.key_cache, c.value_cache, c.block_tables, c.kv_lens,
                                                 c.scale, c.kv_cache_dtype, c.descale, c.descale, c.sink)
    torch.testing.assert_close(got, c.expected.float(), atol=H.ATTN_ATOL, rtol=H.ATTN_RTOL)


@pytest.mark.parametrize("fname", H.golden_files("varlen_attn"))
def test_oracle_reproduces_reference_varlen_attention_fixture(fname):
    """Several query tokens per sequence, causal or not: expected values from the reference's ref_paged_attn."""
    c = H.DecodeAttnCase(fname)
    got = torch_views.run_paged_decode_attention(c.query, c.key_cache, c.value_cache, c.block_tables, c.kv_lens,
                                                 c.scale, c.kv_cache_dtype, c.descale, c.descale, c.sink,
                                                 c.cu_seqlens_q, c.causal)
    torch.testing.assert_close(got, c.expected.float(), atol=H.ATTN_ATOL, rtol=H.ATTN_RTOL)


@pytest.mark.parametrize("fname", H.golden_files("window_attn"))
def test_oracle_reproduces_reference_window_and_dense_attention_fixture(fname):
    """Sliding windows (one side open, both closed, with and without the causal mask) and the non-paged form."""
    c = H.DecodeAttnCase(fname)
    got = torch_views.run_paged_decode_attention(c.query, c.key_cache, c.value_cache, c.block_tables, c.kv_lens,
                                                 c.scale, c.kv_cache_dtype, c.descale, c.descale, c.sink,
                                                 c.cu_seqlens_q, c.causal, c.window)
    torch.testing.assert_close(got, c.expected.float(), atol=H.ATTN_ATOL, rtol=H.ATTN_RTOL)


def test_decode_attention_shards_by_kv_head():
    """Tensor parallelism over kv heads: each rank holds its kv heads' cache slice and the query heads of those
    groups; concatenating the ranks' outputs along the head axis gives the unsharded result (nothing is exchanged)."""
    torch.manual_seed(4)
    S, hq, hk, D, bs, nb = 3, 16, 4, 64, 16, 12
    query = torch.randn(S, hq, D).to(torch.bfloat16)
    kc = torch.randn(nb, bs, hk, D).to(torch.bfloat16)
    vc = torch.randn(nb, bs, hk, D).to(torch.bfloat16)
    bt = torch.randint(0, nb, (S, 6), dtype=torch.int32)
    lens = torch.tensor([90, 1, 33], dtype=torch.int32)
    sink = torch.randn(hq).to(torch.bfloat16)
    whole = torch_views.run_paged_decode_attention(query, kc, vc, bt, lens, 0.125, sink=sink)
    for world in (2, 4):
        g = hq // hk
        parts = []
        for rank in range(world):
            k0, k1 = rank * hk // world, (rank + 1) * hk // world
            parts.append(torch_views.run_paged_decode_attention(
                query[:, k0 * g:k1 * g], kc[:, :, k0:k1], vc[:, :, k0:k1], bt, lens, 0.125,
                sink=sink[k0 * g:k1 * g].contiguous()))
        assert torch.equal(torch.cat(parts, dim=1), whole)


def test_fp8_decoders_invert_the_encoders():
    L = oracle.lib()
    for b in range(256):
        v4, v5 = L.orc_e4m3_to_f32(b), L.orc_e5m2_to_f32(b)
        want4 = torch.tensor([b], dtype=torch.uint8).view(torch.float8_e4m3fn).float().item()
        want5 = torch.tensor([b], dtype=torch.uint8).view(torch.float8_e5m2).float().item()
        assert (v4 != v4 and want4 != want4) or v4 == want4, b
        assert (v5 != v5 and want5 != want5) or v5 == want5, b
        if v4 == v4:
            assert L.orc_f32_to_e4m3(v4) == b


def test_rotary_oracle_rounding_helpers_match_torch():
    """The oracle's float -> f16 / bf16 roundings against torch's casts, over a dense sweep."""
    L = oracle.lib()
    g = torch.Generator().manual_seed(11)
    bits = torch.randint(-2**31, 2**31 - 1, (200000,), generator=g, dtype=torch.int64).to(torch.int32)
    x = bits.view(torch.float32)
    x = x[~torch.isnan(x)]
    edge = torch.tensor([65504.0, 65519.9, 65520.0, 6.1e-5, 5.96e-8, 2.98e-8, 2.9802322e-8, 8.9e-8, 0.0, -0.0,
                         float("inf"), -float("inf"), 3.3895314e38, 1e-40, 9.2e-41])
    x = torch.cat([x, edge, -edge])
    want_h = x.to(torch.float16).view(torch.int16).numpy().view(np.uint16)
    want_b = x.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    xs = x.numpy()
    step = max(1, len(xs) // 20000)
    for i in list(range(0, len(xs), step)) + list(range(len(xs) - 2 * len(edge), len(xs))):
        assert L.orc_f32_to_f16(float(xs[i])) == want_h[i], xs[i]
        assert L.orc_f32_to_bf16(float(xs[i])) == want_b[i], xs[i]


@pytest.mark.parametrize("in_dtype,tdt", [("bf16", torch.bfloat16), ("f16", torch.float16)])
def test_conversion_tables_match_torch_cast(in_dtype, tdt):
    z = np.load(os.path.join(H.GOLDEN_DIR, "fp8_tables.npz"))
    pats = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(tdt).float().numpy()
    for si, scale in enumerate(z["scales"]):
        q = pats / np.float32(scale)
        finite = ~np.isnan(q)
        for kv, name, lim in (("fp8_e4m3", "e4m3", 464.0), ("fp8_e5m2", "e5m2", 57344.0)):
            want = z[f"{in_dtype}_{name}"][si]
            got = oracle.convert_table(in_dtype, kv, float(scale))
            agree = finite & (np.abs(q) <= lim)
            assert np.array_equal(got[agree], want[agree]), (in_dtype, kv, scale)
            # beyond that the oracle saturates where torch produces NaN / inf
            over = finite & ~agree
            top = 0x7E if kv == "fp8_e4m3" else 0x7B
            assert np.all((got[over] & 0x7F) == top)
            assert np.all((got[over] >> 7) == (q[over] < 0))
            assert np.all(got[~finite] == 0x7F)


def test_e4m3_converter_against_independent_numpy_restatement():
    rng = np.random.default_rng(0)
    x = np.concatenate([
        rng.standard_normal(200000).astype(np.float32) * 100,
        rng.standard_normal(200000).astype(np.float32) * 0.01,
        (rng.integers(0, 2**32, 400000, dtype=np.uint64).astype(np.uint32)).view(np.float32),
        np.array([0.0, -0.0, 2.0**-10, -(2.0**-10), 1.5 * 2.0**-10, 2.0**-9, 3 * 2.0**-10, 2.0**-6, 0.0165,
                  447.9, 448.0, 463.9, 464.0, 465.0, 1e9, -1e9, np.inf, -np.inf, np.nan, 17.0, 18.0, 19.0, 0.9375 * 2**-6],
                 dtype=np.float32),
    ])
    got = oracle.convert_f32(x, "fp8_e4m3", 1.0)
    want = oracle.np_f32_to_e4m3(x)
    assert np.array_equal(got, want)
    # known answers
    ka = [(0.0, 0x00), (-0.0, 0x80), (2.0**-10, 0x00), (1.5 * 2.0**-10, 0x01), (2.0**-9, 0x01),
          (3 * 2.0**-10, 0x02), (2.0**-6, 0x08), (448.0, 0x7E), (464.0, 0x7E), (1e9, 0x7E), (-1e9, 0xFE),
          (1.0, 0x38), (17.0, 0x58), (19.0, 0x5A)]
    for v, code in ka:
        assert oracle.lib().orc_f32_to_e4m3(v) == code, v
    assert oracle.lib().orc_f32_to_e4m3(float("inf")) == 0x7E
    assert oracle.lib().orc_f32_to_e4m3(float("nan")) == 0x7F


def test_skip_short_slot_mapping_and_range_check():
    T, Hh, D, bs, nb = 6, 2, 16, 4, 3
    key = torch.randn(T + 3, Hh, D).to(torch.bfloat16)
    value = torch.randn(T + 3, Hh, D).to(torch.bfloat16)
    kc = torch.zeros(nb, bs, Hh, D, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    slots = torch.tensor([5, -1, 0, 11, -1, 7])
    H.oracle_call("flash", key, value, kc, vc, slots, "auto", 1.0, 1.0)
    flat = kc.view(nb * bs, Hh, D)
    for i, s in enumerate(slots.tolist()):
        if s >= 0:
            assert H.same_bytes(flat[s], key[i])
    untouched = [s for s in range(nb * bs) if s not in (5, 0, 11, 7)]
    assert bool((flat[untouched] == 0).all())
    with pytest.raises(IndexError):
        H.oracle_call("flash", key, value, kc, vc, torch.tensor([nb * bs]), "auto", 1.0, 1.0)


def test_threads_do_not_change_results():
    w_key = torch.randn(300, 4, 32).to(torch.float16)
    w_val = torch.randn(300, 4, 32).to(torch.float16)
    slots = torch.randperm(64 * 8)[:300]
    outs = []
    for th in (1, 4):
        kc = torch.zeros(64, 8, 4, 32, dtype=torch.uint8)
        vc = torch.zeros_like(kc)
        H.oracle_call("flash", w_key, w_val, kc, vc, slots, "fp8", 0.01, 0.02, threads=th)
        outs.append((kc, vc))
    assert H.same_bytes(outs[0][0], outs[1][0]) and H.same_bytes(outs[0][1], outs[1][1])


def test_three_instruction_division_is_exact_on_a_subsample():
    """Every 16th scale significand x every 16-bit-float significand; the full set is
    `oracle/prove_fast_div 1` (2^33 cases, a few seconds)."""
    exe = os.path.join(os.path.dirname(oracle.__file__), "prove_fast_div")
    if not os.path.exists(exe):
        subprocess.run(["make", "-C", os.path.dirname(exe), "prove_fast_div"], check=True, capture_output=True)
    r = subprocess.run([exe, "16"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "mismatches 0" in r.stdout


@pytest.mark.parametrize("layout", ["flash", "paged"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("kv", ["auto", "fp8", "fp8_e5m2"])
def test_c_oracle_equals_the_torch_loops_of_the_reference_tests(layout, dtype, kv):
    """Beyond the committed fixtures: the C oracle against the torch restatement of the reference's
    expected-result loops on fresh random inputs (strided key/value, padding, several scales)."""
    from oracle import torch_reference
    torch.manual_seed(hash((layout, str(dtype), kv)) % 1000)
    T, Hh, D, bs, nb = 97, 3, 32, 8, 20
    qkv = (torch.randn(T, 3, Hh, D) * 2).to(dtype)
    key, value = qkv[:, 1], qkv[:, 2]
    slots = torch.randperm(nb * bs)[:T]
    slots[::6] = -1
    cdt = H.cache_torch_dtype(dtype, kv)
    x = 16 // torch.empty((), dtype=cdt).element_size()
    shapes = ((nb, bs, Hh, D), (nb, bs, Hh, D)) if layout == "flash" else ((nb, Hh, D // x, bs, x), (nb, Hh, D, bs))
    for ks, vs in ((0.011, 0.013), (1.0, 0.5), (float(key.float().abs().max()) / 448, 3.0)):
        a = [H.fill_pattern_(torch.empty(s, dtype=cdt), i) for i, s in enumerate(shapes)]
        b = [t.clone() for t in a]
        H.oracle_call(layout, key, value, a[0], a[1], slots, kv, ks, vs)
        getattr(torch_reference, "reshape_and_cache_flash" if layout == "flash" else "reshape_and_cache")(
            key, value, b[0], b[1], slots, kv, ks, vs)
        assert H.same_bytes(a[0], b[0]) and H.same_bytes(a[1], b[1]), (ks, vs)
