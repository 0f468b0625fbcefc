"""GPU parity of ``concat_and_cache_mla`` and ``gather_cache`` (C ABI and torch op) against the
fixtures generated from the reference's recipes and against the CPU oracle.  Bit-exact."""
import random

import pytest
import torch

from oracle import torch_views
from tests import helpers as H
from vllm_xpu_kernels import cabi, ops

pytestmark = pytest.mark.gpu


def dev_scale(v, device):
    return torch.tensor(v, dtype=torch.float32, device=device)


# ------------------------------------------------------------------------------------------ MLA
@pytest.mark.parametrize("fname", H.golden_files("mla"))
@pytest.mark.parametrize("face", ["cabi", "op"])
def test_mla_golden(fname, face, cuda_device):
    c = H.MlaCase(fname)
    cache = c.cache_before.to(cuda_device)
    args = (c.kv_c.to(cuda_device), c.k_pe.to(cuda_device), cache, c.slot_mapping.to(cuda_device), c.kv_cache_dtype,
            dev_scale(c.scale, cuda_device))
    (cabi.concat_and_cache_mla if face == "cabi" else ops.concat_and_cache_mla)(*args)
    torch.cuda.synchronize()
    assert H.same_bytes(cache.cpu(), c.cache_after)


@pytest.mark.parametrize("dtype", [torch.half, torch.bfloat16, torch.float])
@pytest.mark.parametrize("kv", ["auto", "fp8", "fp8_e5m2"])
@pytest.mark.parametrize("shape", [(42, 512, 64, 16, 8), (257, 512, 64, 64, 16), (33, 48, 24, 12, 5), (7, 9, 3, 8, 2)])
def test_mla_vs_oracle(dtype, kv, shape, cuda_device):
    """(T, kv_lora_rank, pe_dim, block_size, num_blocks): the reference's test shape
    (tests/test_cache.py:20-25 there), a larger odd-T batch, and widths that force narrow vectors."""
    T, R, P, bs, nb = shape
    random.seed(T)
    torch.manual_seed(T)
    # inputs as column slices of wider tensors: token strides differ from the widths
    big_c = torch.randn(T + 2, R + 8).to(dtype)
    big_p = torch.randn(T + 2, P + 16).to(dtype)
    kv_c, k_pe = big_c[:, :R], big_p[:, 8:8 + P]
    slots = random.sample(range(nb * bs), T)
    for i in random.sample(range(T), T // 5):
        slots[i] = -1
    slots = torch.tensor(slots, dtype=torch.long)
    cdt = H.cache_torch_dtype(dtype, kv)
    # cache as a view with padded entries: entry_stride > R + P
    alloc = H.fill_pattern_(torch.empty(nb, bs, R + P + 16, dtype=cdt), 3)
    cache = alloc[:, :, :R + P]
    dalloc = alloc.to(cuda_device)
    dcache = dalloc[:, :, :R + P]
    scale = 0.07 if kv != "fp8_e5m2" else 0.0003
    torch_views.run_mla(kv_c, k_pe, cache, slots, kv, scale)
    cabi.concat_and_cache_mla(big_c.to(cuda_device)[:, :R], big_p.to(cuda_device)[:, 8:8 + P], dcache,
                              slots.to(cuda_device), kv, dev_scale(scale, cuda_device))
    torch.cuda.synchronize()
    assert H.same_bytes(dalloc.cpu(), alloc)


def test_mla_short_and_empty_slot_mapping(cuda_device):
    dev = cuda_device
    kv_c = torch.randn(10, 512, device=dev).to(torch.bfloat16)
    k_pe = torch.randn(10, 64, device=dev).to(torch.bfloat16)
    cache = torch.zeros(4, 16, 576, dtype=torch.bfloat16, device=dev)
    cabi.concat_and_cache_mla(kv_c, k_pe, cache, torch.empty(0, dtype=torch.long, device=dev), "auto")
    assert not bool(cache.any())
    slots = torch.tensor([5, -1, 63], device=dev)
    ops.concat_and_cache_mla(kv_c, k_pe, cache, slots, "auto", dev_scale(1.0, dev))
    flat = cache.view(64, 576)
    assert H.same_bytes(flat[5, :512], kv_c[0]) and H.same_bytes(flat[5, 512:], k_pe[0])
    assert H.same_bytes(flat[63, :512], kv_c[2]) and H.same_bytes(flat[63, 512:], k_pe[2])
    assert int((flat != 0).any(dim=1).sum()) == 2


def test_mla_opcheck_and_errors(cuda_device):
    dev = cuda_device
    kv_c = torch.randn(8, 512, device=dev).to(torch.half)
    k_pe = torch.randn(8, 64, device=dev).to(torch.half)
    cache = torch.zeros(2, 16, 576, dtype=torch.half, device=dev)
    slots = torch.randperm(32, device=dev)[:8]
    torch.library.opcheck(torch.ops._C_cache_ops.concat_and_cache_mla,
                          (kv_c, k_pe, cache, slots, "auto", dev_scale(0.1, dev)),
                          test_utils=("test_schema", "test_autograd_registration", "test_faketensor",
                                      "test_aot_dispatch_dynamic"))
    with pytest.raises(RuntimeError, match="kv_lora_rank \\+ pe_dim"):
        ops.concat_and_cache_mla(kv_c, k_pe[:, :32], cache, slots, "auto", dev_scale(0.1, dev))
    with pytest.raises(RuntimeError, match="Unsupported data type of kv cache"):
        ops.concat_and_cache_mla(kv_c, k_pe, cache, slots, "int4", dev_scale(0.1, dev))
    with pytest.raises(RuntimeError, match="does not match kv_cache_dtype"):
        ops.concat_and_cache_mla(kv_c, k_pe, cache, slots, "fp8", dev_scale(0.1, dev))


# --------------------------------------------------------------------------------------- gather
@pytest.mark.parametrize("fname", H.golden_files("gather"))
@pytest.mark.parametrize("face", ["cabi", "op"])
def test_gather_golden(fname, face, cuda_device):
    c = H.GatherCase(fname)
    total = int(c.cu_seq_lens[-1])
    dst = torch.zeros(total + 5, c.expected.shape[1], dtype=c.dtype, device=cuda_device)
    ss = None if c.seq_starts is None else c.seq_starts.to(cuda_device)
    fn = cabi.gather_cache if face == "cabi" else ops.gather_cache
    fn(c.src_cache.to(cuda_device), dst, c.block_table.to(cuda_device), c.cu_seq_lens.to(cuda_device), c.batch_size, ss)
    torch.cuda.synchronize()
    assert H.same_bytes(dst[:total].cpu(), c.expected)
    assert not bool(dst[total:].view(torch.uint8).any())  # rows past the last sequence are left alone


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.uint8])
@pytest.mark.parametrize("entry,bs", [(576, 16), (576, 64), (40, 12), (7, 8)])
@pytest.mark.parametrize("with_starts", [False, True])
def test_gather_vs_oracle(dtype, entry, bs, with_starts, cuda_device):
    """The reference's test shape (entry 512+64, batch 8, tests/test_cache.py:423-431 there) and odd ones,
    with the cache taken as a strided view and ragged sequence lengths including empty sequences."""
    nb, batch, max_len = 96, 8, 5 * bs + 3
    g = torch.Generator().manual_seed(entry * 131 + bs)
    alloc = torch.randint(0, 255, (nb, bs, entry + 4), dtype=torch.uint8, generator=g)
    if dtype != torch.uint8:
        alloc = torch.randn(nb, bs, entry + 4, generator=g).to(dtype)
    src = alloc[:, :, :entry]
    seq_lens = torch.randint(0, max_len + 1, (batch,), generator=g)
    seq_lens[2] = 0
    cu = torch.zeros(batch + 1, dtype=torch.int32)
    cu[1:] = seq_lens.cumsum(0).to(torch.int32)
    table = torch.stack([torch.randperm(nb, generator=g) for _ in range(batch)]).to(torch.int32)
    starts = (torch.randint(0, 4 * bs, (batch,), generator=g)).to(torch.int32) if with_starts else None
    total = int(cu[-1])
    want = torch.zeros(total + 2, entry, dtype=dtype)
    torch_views.run_gather(src, want, table, cu, batch, starts)
    dst = torch.zeros(total + 2, entry, dtype=dtype, device=cuda_device)
    cabi.gather_cache(alloc.to(cuda_device)[:, :, :entry], dst, table.to(cuda_device), cu.to(cuda_device), batch,
                      None if starts is None else starts.to(cuda_device))
    torch.cuda.synchronize()
    assert H.same_bytes(dst.cpu(), want)


def test_write_then_gather_round_trip(cuda_device):
    """concat_and_cache_mla followed by gather_cache returns the rows that went in (auto mode)."""
    dev = cuda_device
    bs, nb, R, P = 16, 64, 512, 64
    seq_lens = [37, 0, 16, 5, 64]
    T = sum(seq_lens)
    torch.manual_seed(11)
    kv_c = torch.randn(T, R, device=dev).to(torch.bfloat16)
    k_pe = torch.randn(T, P, device=dev).to(torch.bfloat16)
    table = torch.stack([torch.randperm(nb)[:8] + 0 for _ in seq_lens]).to(torch.int32)
    # make the block sets of different sequences disjoint
    perm = torch.randperm(nb).to(torch.int32)
    table = perm[:len(seq_lens) * 8].view(len(seq_lens), 8).contiguous()
    slots = []
    for b, n in enumerate(seq_lens):
        slots += [int(table[b, j // bs]) * bs + j % bs for j in range(n)]
    cache = torch.zeros(nb, bs, R + P, dtype=torch.bfloat16, device=dev)
    ops.concat_and_cache_mla(kv_c, k_pe, cache, torch.tensor(slots, device=dev), "auto", dev_scale(1.0, dev))
    cu = torch.tensor([0] + list(torch.tensor(seq_lens).cumsum(0)), dtype=torch.int32, device=dev)
    dst = torch.zeros(T, R + P, dtype=torch.bfloat16, device=dev)
    ops.gather_cache(cache, dst, table.to(dev), cu, len(seq_lens))
    assert H.same_bytes(dst, torch.cat([kv_c, k_pe], dim=1))


def test_gather_opcheck_and_errors(cuda_device):
    dev = cuda_device
    src = torch.randn(8, 16, 576, device=dev)
    table = torch.arange(8, dtype=torch.int32, device=dev).repeat(2, 1)
    cu = torch.tensor([0, 20, 50], dtype=torch.int32, device=dev)
    dst = torch.zeros(50, 576, device=dev)
    torch.library.opcheck(torch.ops._C_cache_ops.gather_cache, (src, dst, table, cu, 2, None),
                          test_utils=("test_schema", "test_autograd_registration", "test_faketensor",
                                      "test_aot_dispatch_dynamic"))
    with pytest.raises(RuntimeError, match="block_table must be int32"):
        ops.gather_cache(src, dst, table.long(), cu, 2)
    with pytest.raises(RuntimeError, match="cu_seq_lens must be int32"):
        ops.gather_cache(src, dst, table, cu.long(), 2)
    with pytest.raises(RuntimeError, match="same dtype"):
        ops.gather_cache(src, dst.half(), table, cu, 2)
    with pytest.raises(RuntimeError, match="Unsupported data type width: 64"):
        ops.gather_cache(src.double(), dst.double(), table, cu, 2)
    with pytest.raises(RuntimeError, match="same device"):
        ops.gather_cache(src, dst, table.cpu(), cu, 2)
