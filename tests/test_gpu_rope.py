"""GPU parity of the rotary embedding (alone and fused with the flash-layout cache write) against the
fixtures computed with the reference's ``RotaryEmbedding.forward_native`` and against the CPU oracle.

Tolerance: none.  The op is floating point, but its contract fixes every rounding (each product and the
sum rounded to the tensors' type, nothing fused), so results are compared bit for bit.  NaN outputs are
not part of any case (their payload is unspecified)."""
import os
import random
import subprocess
import sys

import pytest
import torch

from oracle import torch_views
from tests import helpers as H
from vllm_xpu_kernels import cabi, ops

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.float16, torch.bfloat16]


def cos_sin_table(max_position: int, rot_dim: int, dtype: torch.dtype, base: float = 10000.0) -> torch.Tensor:
    """[max_position, rot_dim]: cosines then sines (tests/ops/rotary_embedding_op.py:59-79 of the reference)."""
    inv_freq = 1.0 / (base ** (torch.arange(0, rot_dim, 2, dtype=torch.float) / rot_dim))
    freqs = torch.einsum("i,j -> ij", torch.arange(max_position, dtype=torch.float), inv_freq)
    return torch.cat((freqs.cos(), freqs.sin()), dim=-1).to(dtype)


# ------------------------------------------------------------------------------------ fixtures
@pytest.mark.parametrize("fname", H.golden_files("rope"))
@pytest.mark.parametrize("face", ["cabi", "op"])
def test_rope_golden(fname, face, cuda_device):
    c = H.RopeCase(fname)
    q_store = c.query_store.to(cuda_device)
    k_store = None if c.key_store is None else c.key_store.to(cuda_device)
    q, k = c.views(q_store, k_store)
    fn = cabi.rotary_embedding if face == "cabi" else ops.rotary_embedding
    fn(c.positions.to(cuda_device), q, k, c.head_size, c.cos_sin_cache.to(cuda_device), c.is_neox)
    torch.cuda.synchronize()
    assert H.same_bytes(q_store.cpu()[..., :c.head_size], c.query_after)
    assert H.same_bytes(q_store.cpu()[..., c.head_size:], c.query_store[..., c.head_size:])
    if k_store is not None:
        assert H.same_bytes(k_store.cpu()[..., :c.head_size], c.key_after)
        assert H.same_bytes(k_store.cpu()[..., c.head_size:], c.key_store[..., c.head_size:])


@pytest.mark.parametrize("max_position", [11, 4096])
@pytest.mark.parametrize("is_neox_style", [True, False])
@pytest.mark.parametrize("head_size", [32, 108])
@pytest.mark.parametrize("seq_len", [11, 1024])
@pytest.mark.parametrize("use_key", [True, False])
@pytest.mark.parametrize("head_stride_is_contiguous", [True, False])
def test_rotary_embedding_opcheck(max_position, is_neox_style, head_size, seq_len, use_key,
                                  head_stride_is_contiguous, cuda_device):
    """The reference's own test of this op (tests/test_rotary_embedding.py:43-87 there): schema, fake-tensor
    and dispatch checks over its matrix of layouts, fp32, rotary_dim 32, 7 heads."""
    rotary_dim, num_heads, batch_size = 32, 7, 1
    table = cos_sin_table(max_position, rotary_dim, torch.float32).to(cuda_device)
    positions = torch.randint(0, max_position, (batch_size, seq_len), device=cuda_device)
    head_stride = head_size + (64 if head_stride_is_contiguous else 0)
    query = torch.randn(batch_size, seq_len, num_heads, head_stride, dtype=torch.float32, device=cuda_device)
    key = torch.randn_like(query) if use_key else None
    query = query[..., :head_size]
    key = key[..., :head_size] if use_key else None
    H.opcheck(torch.ops._C.rotary_embedding, (positions, query, key, head_size, table, is_neox_style))
    if head_stride_is_contiguous:
        H.opcheck(torch.ops._C.rotary_embedding,
                  (positions, query.flatten(start_dim=-2), key.flatten(start_dim=-2) if use_key else None, head_size,
                   table, is_neox_style))


# ------------------------------------------------------------------------------------ vs oracle
SHAPES = [
    # T, Hq, Hkv, head_size, rot_dim, head_pad, token_pad   (pads in elements; odd pads force narrow accesses)
    (67, 8, 2, 128, 128, 0, 0),      # full rotation, grouped kv heads, 32-byte accesses
    (33, 4, 4, 64, 64, 0, 64),       # token stride wider than the row
    (19, 7, 7, 108, 32, 0, 0),       # the reference test's odd head size
    (19, 7, 7, 108, 32, 64, 0),      # ... with padded heads
    (21, 3, 1, 80, 80, 0, 8),        # rot_dim / 2 = 40: 16-byte accesses at best
    (17, 2, 2, 36, 12, 0, 0),        # rot_dim / 2 = 6
    (23, 5, 5, 33, 22, 0, 0),        # odd head size: element accesses (pair kernel)
    (11, 3, 3, 16, 6, 1, 1),         # odd everything
    (5, 1, 1, 256, 256, 0, 0),
    (300, 16, 4, 128, 64, 0, 0),     # partial rotation at a model-like shape
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("is_neox", [True, False])
@pytest.mark.parametrize("shape", SHAPES)
def test_rope_vs_oracle(dtype, is_neox, shape, cuda_device):
    T, hq, hk, D, R, head_pad, token_pad = shape
    torch.manual_seed(T * 131 + D)
    max_pos = 777
    table = cos_sin_table(max_pos, R, dtype)
    positions = torch.randint(0, max_pos, (T,))
    q_alloc = torch.randn(T, hq * (D + head_pad) + token_pad).to(dtype)
    k_alloc = torch.randn(T, hk * (D + head_pad) + token_pad).to(dtype)

    def views(qa, ka):
        q = qa[:, :hq * (D + head_pad)].view(T, hq, D + head_pad)[..., :D]
        k = ka[:, :hk * (D + head_pad)].view(T, hk, D + head_pad)[..., :D]
        return q, k

    dq, dk = q_alloc.to(cuda_device), k_alloc.to(cuda_device)
    cabi.rotary_embedding(positions.to(cuda_device), *views(dq, dk), D, table.to(cuda_device), is_neox)
    torch.cuda.synchronize()
    torch_views.run_rope(positions, *views(q_alloc, k_alloc), D, table, is_neox)
    assert H.same_bytes(dq.cpu(), q_alloc)
    assert H.same_bytes(dk.cpu(), k_alloc)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("is_neox", [True, False])
def test_rope_layouts_flat_batched_and_without_key(dtype, is_neox, cuda_device):
    """positions [batch, seq] with [batch, seq, heads * head_size] tensors, and key = None
    (csrc/pos_encoding_kernels.cpp:174-211 of the reference)."""
    B, S, hq, hk, D, R = 3, 13, 6, 2, 64, 32
    torch.manual_seed(5)
    table = cos_sin_table(100, R, dtype)
    positions = torch.randint(0, 100, (B, S))
    q = torch.randn(B, S, hq * D).to(dtype)
    k = torch.randn(B, S, hk * D).to(dtype)
    dq, dk = q.to(cuda_device), k.to(cuda_device)
    cabi.rotary_embedding(positions.to(cuda_device), dq, dk, D, table.to(cuda_device), is_neox)
    torch_views.run_rope(positions, q, k, D, table, is_neox)
    assert H.same_bytes(dq.cpu(), q) and H.same_bytes(dk.cpu(), k)
    # 4-D form, no key
    q4 = torch.randn(B, S, hq, D).to(dtype)
    dq4 = q4.to(cuda_device)
    cabi.rotary_embedding(positions.to(cuda_device), dq4, None, D, table.to(cuda_device), is_neox)
    torch_views.run_rope(positions, q4, None, D, table, is_neox)
    assert H.same_bytes(dq4.cpu(), q4)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("is_neox", [True, False])
def test_rope_special_values(dtype, is_neox, cuda_device):
    """Every exponent of the 16-bit type (subnormals, the largest finite values, signed zeros, infinities that
    meet a finite factor) against table entries of either sign and of magnitude 0, tiny, 1: the packed 16-bit
    arithmetic must round exactly like fp32 arithmetic followed by one rounding."""
    pats = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(dtype)
    finite = pats[torch.isfinite(pats.float())]
    g = torch.Generator().manual_seed(3)
    D = R = 64
    T, heads = 128, 8
    n = T * heads * D
    vals = finite[torch.randint(0, finite.numel(), (n,), generator=g)]
    q = vals.view(T, heads, D).clone()
    k = finite[torch.randint(0, finite.numel(), (T * 2 * D,), generator=g)].view(T, 2, D).clone()
    table = cos_sin_table(T, R, dtype)
    # a few hand-made rows: exact zeros and ones, tiny factors, negative cosines
    table[1] = 0
    table[2, :R // 2] = 1
    table[2, R // 2:] = 0
    table[3] = torch.tensor(6e-8 if dtype == torch.float16 else 1e-38).to(dtype)
    table[4] = -1
    positions = torch.arange(T)
    dq, dk = q.to(cuda_device), k.to(cuda_device)
    cabi.rotary_embedding(positions.to(cuda_device), dq, dk, D, table.to(cuda_device), is_neox)
    torch_views.run_rope(positions, q, k, D, table, is_neox)
    got_q, got_k = dq.cpu(), dk.cpu()
    for got, want in ((got_q, q), (got_k, k)):
        nan = torch.isnan(want.float())
        assert torch.equal(torch.isnan(got.float()), nan)  # inf - inf and 0 * inf
        assert torch.equal(got.view(torch.int16)[~nan], want.view(torch.int16)[~nan])
    assert int(torch.isnan(q.float()).sum()) < q.numel() // 50  # the case is not mostly NaN


def test_rope_float_is_not_contracted(cuda_device):
    """fp32: x*c - y*s with separately rounded products; a fused multiply-add would differ in the last bit
    on a good share of random inputs."""
    torch.manual_seed(9)
    T, heads, D = 257, 4, 128
    table = cos_sin_table(4096, D, torch.float32)
    positions = torch.randint(0, 4096, (T,))
    q = torch.randn(T, heads, D)
    dq = q.to(cuda_device)
    cabi.rotary_embedding(positions.to(cuda_device), dq, None, D, table.to(cuda_device), True)
    cos, sin = table[positions][:, None, :D // 2], table[positions][:, None, D // 2:]
    x, y = q[..., :D // 2], q[..., D // 2:]
    want = torch.cat((x * cos - y * sin, y * cos + x * sin), dim=-1)
    assert H.same_bytes(dq.cpu(), want)


def test_rope_positions_outside_the_table_leave_the_token_unrotated(cuda_device):
    T, heads, D = 16, 2, 64
    torch.manual_seed(1)
    table = cos_sin_table(32, D, torch.bfloat16)
    positions = torch.randint(0, 32, (T,))
    positions[3], positions[7], positions[11] = -1, 32, 2**40
    q = torch.randn(T, heads, D).to(torch.bfloat16)
    dq = q.to(cuda_device)
    cabi.rotary_embedding(positions.to(cuda_device), dq, None, D, table.to(cuda_device), True)
    got = dq.cpu()
    bad = torch.tensor([3, 7, 11])
    assert H.same_bytes(got[bad], q[bad])
    ok = torch.tensor([i for i in range(T) if i not in (3, 7, 11)])
    q_ok = q[ok].clone()
    torch_views.run_rope(positions[ok], q_ok, None, D, table, True)
    assert H.same_bytes(got[ok], q_ok)


def test_rope_rejects_bad_arguments(cuda_device):
    dev = cuda_device
    table = cos_sin_table(8, 32, torch.float16).to(dev)
    pos = torch.zeros(4, dtype=torch.long, device=dev)
    q = torch.zeros(4, 2, 32, dtype=torch.float16, device=dev)
    with pytest.raises(RuntimeError, match="same number of tokens"):
        cabi.rotary_embedding(pos, q[:3], None, 32, table, True)
    with pytest.raises(RuntimeError, match="rot_dim"):
        cabi.rotary_embedding(pos, q[..., :16], None, 16, table, True)  # rot_dim 32 > head_size 16
    with pytest.raises(RuntimeError, match="dtype"):
        cabi.rotary_embedding(pos, q, None, 32, table.float(), True)
    with pytest.raises(RuntimeError, match="positions"):
        cabi.rotary_embedding(pos.int(), q, None, 32, table, True)
    cabi.rotary_embedding(pos[:0], q[:0], None, 32, table, True)  # empty batch: nothing to do


# ------------------------------------------------------------------------------------ fused op
def _fused_case(dtype, kv, is_neox, T, hq, hk, D, R, bs, nb, n_slot_tokens, seed, device, qkv_fused=True):
    random.seed(seed)
    torch.manual_seed(seed)
    max_pos = 500
    table = cos_sin_table(max_pos, R, dtype)
    positions = torch.randint(0, max_pos, (T,))
    if qkv_fused:  # query, key and value as column ranges of one projection output
        qkv = torch.randn(T, (hq + 2 * hk) * D).to(dtype)
        split = lambda t: (t[:, :hq * D].view(T, hq, D), t[:, hq * D:(hq + hk) * D].view(T, hk, D),
                           t[:, (hq + hk) * D:].view(T, hk, D))
    else:
        qkv = torch.randn(3, T, max(hq, hk), D).to(dtype)
        split = lambda t: (t[0, :, :hq], t[1, :, :hk], t[2, :, :hk])
    slots = random.sample(range(nb * bs), n_slot_tokens)
    for i in random.sample(range(n_slot_tokens), n_slot_tokens // 6):
        slots[i] = -1
    slots = torch.tensor(slots, dtype=torch.long)
    cdt = H.cache_torch_dtype(dtype, kv)
    both = H.fill_pattern_(torch.empty(nb, 2, bs, hk, D, dtype=cdt), seed)
    if kv == "auto":
        k_scale = v_scale = 1.0
    else:
        m = 448.0 if kv != "fp8_e5m2" else 57344.0
        k_scale = float(qkv.float().abs().max() * 1.5 / m)
        v_scale = float(qkv.float().abs().max() / m)
    return table, positions, qkv, split, slots, both, k_scale, v_scale


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kv", ["auto", "fp8", "fp8_e5m2"])
@pytest.mark.parametrize("is_neox", [True, False])
@pytest.mark.parametrize("geom", [
    # T, Hq, Hkv, D, rot_dim, block_size, num_blocks, tokens with a slot
    (77, 8, 2, 128, 128, 16, 8, 77),
    (50, 4, 4, 64, 32, 8, 10, 41),     # partial rotation, padded tail of the batch
    (9, 2, 1, 256, 64, 16, 2, 9),
])
def test_fused_rope_cache_equals_the_two_ops_in_sequence(dtype, kv, is_neox, geom, cuda_device):
    T, hq, hk, D, R, bs, nb, nslot = geom
    dev = cuda_device
    table, positions, qkv, split, slots, both, k_scale, v_scale = _fused_case(
        dtype, kv, is_neox, T, hq, hk, D, R, bs, nb, nslot, seed=T + D, device=dev)
    ks = torch.tensor(k_scale, dtype=torch.float32, device=dev)
    vs = torch.tensor(v_scale, dtype=torch.float32, device=dev)

    # fused
    d_qkv, d_both = qkv.to(dev), both.to(dev)
    q, k, v = split(d_qkv)
    cabi.rotary_embedding_and_cache_flash(positions.to(dev), q, k, v, D, table.to(dev), is_neox, d_both[:, 0],
                                          d_both[:, 1], slots.to(dev), kv, ks, vs)
    # the two ops in sequence
    d_qkv2, d_both2 = qkv.to(dev), both.to(dev)
    q2, k2, v2 = split(d_qkv2)
    cabi.rotary_embedding(positions.to(dev), q2, k2, D, table.to(dev), is_neox)
    cabi.reshape_and_cache_flash(k2, v2, d_both2[:, 0], d_both2[:, 1], slots.to(dev), kv, ks, vs)
    torch.cuda.synchronize()
    assert H.same_bytes(d_qkv.cpu(), d_qkv2.cpu())
    assert H.same_bytes(d_both.cpu(), d_both2.cpu())

    # and the oracle's two steps
    cq, ck, cv = split(qkv)
    torch_views.run_rope(positions, cq, ck, D, table, is_neox)
    H.oracle_call("flash", ck, cv, both[:, 0], both[:, 1], slots, kv, k_scale, v_scale)
    assert H.same_bytes(d_qkv.cpu(), qkv)
    assert H.same_bytes(d_both.cpu(), both)


@pytest.mark.parametrize("is_neox", [True, False])
def test_fused_rope_cache_without_key_write_back(is_neox, cuda_device):
    """write_back_key = False: key stays as it was, the cache gets the rotated rows."""
    dev = cuda_device
    T, hq, hk, D, R, bs, nb = 40, 4, 2, 128, 128, 16, 4
    table, positions, qkv, split, slots, both, k_scale, v_scale = _fused_case(
        torch.bfloat16, "fp8", is_neox, T, hq, hk, D, R, bs, nb, T, seed=8, device=dev, qkv_fused=False)
    ks = torch.tensor(k_scale, dtype=torch.float32, device=dev)
    vs = torch.tensor(v_scale, dtype=torch.float32, device=dev)
    d_qkv, d_both = qkv.to(dev), both.to(dev)
    q, k, v = split(d_qkv)
    cabi.rotary_embedding_and_cache_flash(positions.to(dev), q, k, v, D, table.to(dev), is_neox, d_both[:, 0],
                                          d_both[:, 1], slots.to(dev), "fp8", ks, vs, write_back_key=False)
    torch.cuda.synchronize()
    key_before = split(qkv)[1].clone()
    cq, ck, cv = split(qkv)
    torch_views.run_rope(positions, cq, ck, D, table, is_neox)
    H.oracle_call("flash", ck, cv, both[:, 0], both[:, 1], slots, "fp8", k_scale, v_scale)
    got_q, got_k, got_v = split(d_qkv.cpu())
    assert H.same_bytes(got_q, cq)
    assert H.same_bytes(got_k, key_before)
    assert H.same_bytes(d_both.cpu(), both)


def test_fused_rope_cache_torch_op(cuda_device):
    """The torch face of the fused op: same bytes as the C ABI call, opcheck-clean, usable on a side stream
    and from a device other than the current one's default tensors."""
    dev = cuda_device
    T, hq, hk, D, R, bs, nb = 64, 8, 2, 128, 128, 16, 8
    table, positions, qkv, split, slots, both, k_scale, v_scale = _fused_case(
        torch.float16, "fp8", True, T, hq, hk, D, R, bs, nb, 60, seed=4, device=dev)
    ks = torch.tensor(k_scale, dtype=torch.float32, device=dev)
    vs = torch.tensor(v_scale, dtype=torch.float32, device=dev)
    d1, c1 = qkv.to(dev), both.to(dev)
    d2, c2 = qkv.to(dev), both.to(dev)
    q, k, v = split(d1)
    cabi.rotary_embedding_and_cache_flash(positions.to(dev), q, k, v, D, table.to(dev), True, c1[:, 0], c1[:, 1],
                                          slots.to(dev), "fp8", ks, vs)
    q2, k2, v2 = split(d2)
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        ops.rotary_embedding_and_cache_flash(positions.to(dev), q2, k2, v2, D, table.to(dev), True, c2[:, 0], c2[:, 1],
                                             slots.to(dev), "fp8", ks, vs)
    side.synchronize()
    torch.cuda.synchronize()
    assert H.same_bytes(d1.cpu(), d2.cpu()) and H.same_bytes(c1.cpu(), c2.cpu())
    d3, c3 = qkv.to(dev), both.to(dev)
    q3, k3, v3 = split(d3)
    H.opcheck(torch.ops._C_cache_ops.rotary_embedding_and_cache_flash,
              (positions.to(dev), q3, k3, v3, D, table.to(dev), True, c3[:, 0], c3[:, 1], slots.to(dev), "fp8", ks, vs))
    with pytest.raises(RuntimeError, match="value must be"):
        ops.rotary_embedding_and_cache_flash(positions.to(dev), q3, k3, v3[:, :1], D, table.to(dev), True, c3[:, 0],
                                             c3[:, 1], slots.to(dev), "fp8", ks, vs)
    with pytest.raises(RuntimeError, match="Unsupported data type of kv cache"):
        ops.rotary_embedding_and_cache_flash(positions.to(dev), q3, k3, v3, D, table.to(dev), True, c3[:, 0],
                                             c3[:, 1], slots.to(dev), "int4", ks, vs)


def test_rope_in_a_cuda_graph(cuda_device):
    """Both ops only enqueue work and read their scalars on the device: capture and replay."""
    dev = cuda_device
    T, hq, hk, D, R, bs, nb = 48, 4, 2, 64, 64, 16, 6
    table, positions, qkv, split, slots, both, k_scale, v_scale = _fused_case(
        torch.bfloat16, "fp8", False, T, hq, hk, D, R, bs, nb, T, seed=6, device=dev)
    ks = torch.tensor(k_scale, dtype=torch.float32, device=dev)
    vs = torch.tensor(v_scale, dtype=torch.float32, device=dev)
    d_qkv, d_both = qkv.to(dev), both.to(dev)
    d_pos, d_tab, d_slots = positions.to(dev), table.to(dev), slots.to(dev)
    q, k, v = split(d_qkv)
    pristine = d_qkv.clone()
    ops.rotary_embedding_and_cache_flash(d_pos, q, k, v, D, d_tab, False, d_both[:, 0], d_both[:, 1], d_slots, "fp8",
                                         ks, vs)  # warm-up outside capture
    torch.cuda.synchronize()
    d_qkv.copy_(pristine)
    d_both.copy_(both.to(dev))
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        ops.rotary_embedding_and_cache_flash(d_pos, q, k, v, D, d_tab, False, d_both[:, 0], d_both[:, 1], d_slots,
                                             "fp8", ks, vs)
    d_qkv.copy_(pristine)
    g.replay()
    torch.cuda.synchronize()
    cq, ck, cv = split(qkv)
    torch_views.run_rope(positions, cq, ck, D, table, False)
    H.oracle_call("flash", ck, cv, both[:, 0], both[:, 1], slots, "fp8", k_scale, v_scale)
    assert H.same_bytes(d_qkv.cpu(), qkv) and H.same_bytes(d_both.cpu(), both)


def test_fused_rope_cache_refuses_layouts_without_16_byte_access(cuda_device):
    dev = cuda_device
    T, D = 4, 36  # rows of 72 bytes
    table = cos_sin_table(8, 12, torch.float16).to(dev)
    pos = torch.zeros(T, dtype=torch.long, device=dev)
    q = torch.zeros(T, 2, D, dtype=torch.float16, device=dev)
    k, v = torch.zeros_like(q), torch.zeros_like(q)
    cache = torch.zeros(2, 2, 8, 2, D, dtype=torch.float16, device=dev)
    slots = torch.arange(T, device=dev)
    with pytest.raises(RuntimeError, match="16-byte"):
        cabi.rotary_embedding_and_cache_flash(pos, q, k, v, D, table, True, cache[:, 0], cache[:, 1], slots, "auto")


def test_rope_batches_beyond_the_launch_limit_are_split(cuda_device):
    """A child process lowers the per-launch item limit so that a small batch takes several launches."""
    root = H.GOLDEN_DIR.rsplit("/tests/", 1)[0]
    code = r'''
import sys, torch
sys.path[:0] = [%r, %r]
from oracle import torch_views
from tests.test_gpu_rope import cos_sin_table, _fused_case
from tests import helpers as H
from vllm_xpu_kernels import cabi
dev = torch.device("cuda:0")
T, hq, hk, D, R, bs, nb = 500, 4, 2, 64, 64, 16, 40
table, positions, qkv, split, slots, both, ks, vs = _fused_case(torch.bfloat16, "fp8", True, T, hq, hk, D, R, bs, nb,
                                                                 430, seed=2, device=dev)
d_qkv, d_both = qkv.to(dev), both.to(dev)
q, k, v = split(d_qkv)
s = lambda x: torch.tensor(x, dtype=torch.float32, device=dev)
cabi.rotary_embedding_and_cache_flash(positions.to(dev), q, k, v, D, table.to(dev), True, d_both[:, 0], d_both[:, 1],
                                      slots.to(dev), "fp8", s(ks), s(vs))
d_plain = qkv.to(dev)
pq, pk, _ = split(d_plain)
cabi.rotary_embedding(positions.to(dev), pq, pk, D, table.to(dev), True)
torch.cuda.synchronize()
cq, ck, cv = split(qkv)
torch_views.run_rope(positions, cq, ck, D, table, True)
H.oracle_call("flash", ck, cv, both[:, 0], both[:, 1], slots, "fp8", ks, vs)
assert H.same_bytes(d_qkv.cpu(), qkv) and H.same_bytes(d_both.cpu(), both) and H.same_bytes(d_plain.cpu(), qkv)
print("split ok")
''' % (root, root + "/vllm-xpu-kernels_b200")
    env = dict(os.environ, KVC_TEST_MAX_ITEMS_PER_LAUNCH="700")
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "split ok" in r.stdout, r.stdout + r.stderr
