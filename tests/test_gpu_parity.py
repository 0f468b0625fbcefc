"""GPU parity of the CUDA kernels, called through the C ABI, against the CPU oracle and the
fixtures generated from the reference.  Integer/byte work: every comparison is bit-exact."""
import random

import pytest
import torch

from tests import helpers as H
from vllm_xpu_kernels import cabi

import workloads

pytestmark = pytest.mark.gpu


def dev_scale(v: float, device) -> torch.Tensor:
    return torch.tensor(v, dtype=torch.float32, device=device)


def run_cabi(layout, key, value, key_cache, value_cache, slots, kv, k_scale, v_scale):
    fn = cabi.reshape_and_cache_flash if layout == "flash" else cabi.reshape_and_cache
    fn(key, value, key_cache, value_cache, slots, kv, k_scale, v_scale)
    torch.cuda.synchronize()


# ----------------------------------------------------------------------------------------------
# fixtures produced by the reference's factories / loops / torch cast
# ----------------------------------------------------------------------------------------------
@pytest.mark.parametrize("fname", H.golden_files())
def test_golden_fixture(fname, cuda_device):
    c = H.GoldenCase(fname)
    qkv = c.qkv.to(cuda_device)
    key, value = qkv[:, 1], qkv[:, 2]  # strided views, stride(0) = 3*H*D as in the reference's tests
    if c.layout == "flash":
        alloc = c.alloc.to(cuda_device)
        kc, vc = alloc[:, 0], alloc[:, 1]  # non-contiguous cache views (stride(0) = 2*bs*H*D)
    else:
        kc, vc = c.key_cache.to(cuda_device), c.value_cache.to(cuda_device)
    run_cabi(c.layout, key, value, kc, vc, c.slot_mapping.to(cuda_device), c.kv_cache_dtype,
             dev_scale(c.k_scale, cuda_device), dev_scale(c.v_scale, cuda_device))
    assert H.same_bytes(kc.cpu(), c.key_cache_after)
    assert H.same_bytes(vc.cpu(), c.value_cache_after)


# ----------------------------------------------------------------------------------------------
# the reference's test matrix (tests/test_cache.py:14-37 there) at its own sizes, vs the oracle
# ----------------------------------------------------------------------------------------------
def _matrix_case(layout, dtype, kv, D, bs, device, T=42, Hh=8, nb=128, seed=0, skip=0):
    random.seed(seed)
    torch.manual_seed(seed)
    slots = random.sample(range(nb * bs), T)
    for i in random.sample(range(T), skip):
        slots[i] = -1
    slots = torch.tensor(slots, dtype=torch.long)
    qkv = torch.randn(T, 3, Hh, D, dtype=torch.float32).to(dtype)
    key, value = qkv[:, 1], qkv[:, 2]
    cdt = H.cache_torch_dtype(dtype, kv)
    es = torch.empty((), dtype=cdt).element_size()
    if layout == "flash":
        alloc = H.fill_pattern_(torch.empty(nb, 2, bs, Hh, D * es, dtype=torch.uint8), seed).view(cdt)
        kc, vc = alloc[:, 0], alloc[:, 1]
    else:
        x = 16 // es
        kc = H.fill_pattern_(torch.empty(nb, Hh, D // x, bs, x, dtype=cdt), seed)
        vc = H.fill_pattern_(torch.empty(nb, Hh, D, bs, dtype=cdt), seed + 1)
        alloc = None
    fmax = {"auto": 1.0, "fp8": 448.0, "fp8_e4m3": 448.0, "fp8_e5m2": 57344.0}[kv]
    ks = float(key.float().abs().amax() / fmax)
    vs = float(value.float().abs().amax() / fmax)
    # device copies first (the oracle mutates the CPU caches in place)
    d = dict(qkv=qkv.to(device), slots=slots.to(device))
    if layout == "flash":
        dalloc = alloc.to(device)
        d["kc"], d["vc"] = dalloc[:, 0], dalloc[:, 1]
    else:
        d["kc"], d["vc"] = kc.to(device), vc.to(device)
    H.oracle_call(layout, key, value, kc, vc, slots, kv, ks, vs)
    run_cabi(layout, d["qkv"][:, 1], d["qkv"][:, 2], d["kc"], d["vc"], d["slots"], kv, dev_scale(ks, device),
             dev_scale(vs, device))
    assert H.same_bytes(d["kc"].cpu(), kc.contiguous()), "key cache differs"
    assert H.same_bytes(d["vc"].cpu(), vc.contiguous()), "value cache differs"


@pytest.mark.parametrize("layout", ["flash", "paged"])
@pytest.mark.parametrize("dtype", [torch.half, torch.bfloat16, torch.float])
@pytest.mark.parametrize("head_size", [64, 80, 120, 256])
@pytest.mark.parametrize("block_size", [8, 16, 32])
def test_reference_matrix_auto(layout, dtype, head_size, block_size, cuda_device):
    _matrix_case(layout, dtype, "auto", head_size, block_size, cuda_device)


@pytest.mark.parametrize("layout", ["flash", "paged"])
@pytest.mark.parametrize("dtype", [torch.half, torch.bfloat16, torch.float])
@pytest.mark.parametrize("kv", ["fp8", "fp8_e4m3", "fp8_e5m2"])
@pytest.mark.parametrize("head_size,block_size", [(64, 8), (80, 16), (128, 16), (256, 32), (16, 8)])
def test_reference_matrix_fp8(layout, dtype, kv, head_size, block_size, cuda_device):
    _matrix_case(layout, dtype, kv, head_size, block_size, cuda_device, skip=5)


@pytest.mark.parametrize("layout", ["flash", "paged"])
@pytest.mark.parametrize("kv", ["auto", "fp8"])
def test_mini_profile_and_odd_shapes(layout, kv, cuda_device):
    # the reference's MINI profile: 1 token, head_size 8, 4 blocks of 8 (tests/test_cache.py:40-46);
    # the paged fp8 layout has x = 16 > 8, so that combination does not exist
    if not (layout == "paged" and kv == "fp8"):
        _matrix_case(layout, torch.half, kv, 8, 8, cuda_device, T=1, nb=4)
    # block sizes that are not powers of two, an odd head count, an odd block count
    for bs in (12, 48):
        _matrix_case(layout, torch.bfloat16, kv, 32, bs, cuda_device, T=100, Hh=5, nb=37, skip=11)


def test_flash_head_size_not_multiple_of_vector(cuda_device):
    # head_size 20: rows of 40 bytes in bf16, 20 bytes in fp8 -> narrow vectors on both sides
    for kv in ("auto", "fp8"):
        _matrix_case("flash", torch.bfloat16, kv, 20, 16, cuda_device, T=33, Hh=3, nb=16)
        _matrix_case("flash", torch.half, kv, 7, 16, cuda_device, T=33, Hh=3, nb=16)


# ----------------------------------------------------------------------------------------------
# the five measured configurations
# ----------------------------------------------------------------------------------------------
def _run_workload_full(w, device):
    """Whole-cache equality against the oracle (small enough caches)."""
    ksh, vsh = w.cache_shapes()
    cdt = w.cache_dtype
    kc = H.fill_pattern_(torch.empty(ksh, dtype=cdt), 11)
    vc = H.fill_pattern_(torch.empty(vsh, dtype=cdt), 12)
    dkc, dvc = kc.to(device), vc.to(device)
    H.oracle_call(w.layout, w.key, w.value, kc, vc, w.slot_mapping, w.kv_cache_dtype, float(w.k_scale),
                  float(w.v_scale), threads=8)
    run_cabi(w.layout, w.key.to(device), w.value.to(device), dkc, dvc, w.slot_mapping.to(device), w.kv_cache_dtype,
             w.k_scale.to(device), w.v_scale.to(device))
    assert H.same_bytes(dkc.cpu(), kc) and H.same_bytes(dvc.cpu(), vc)


def test_config_c1(cuda_device):
    _run_workload_full(workloads.c1(), cuda_device)


def test_config_c2(cuda_device):
    w = workloads.c2()
    assert float((w.key.float() / w.k_scale).abs().max()) <= 464.0  # saturating and non-saturating casts agree
    _run_workload_full(w, cuda_device)


def test_config_c3(cuda_device):
    _run_workload_full(workloads.c3(), cuda_device)


def _run_workload_rows(w, device, qkv_on_device=None):
    """Full-size caches stay on the GPU.  The oracle writes the same tokens into a compact
    cache (slot i -> row i); the rows the kernel wrote are gathered from their real slots and
    compared byte for byte, and every other slot must still hold its pre-call fill."""
    T, Hh, D, bs, nb = w.num_tokens, w.num_heads, w.head_size, w.block_size, w.num_blocks
    cdt = w.cache_dtype
    active = (w.slot_mapping >= 0).nonzero().flatten()
    compact_slots = torch.full((T,), -1, dtype=torch.long)
    compact_slots[active] = torch.arange(active.numel())
    nbc = (active.numel() + bs - 1) // bs
    ekc = torch.zeros(nbc, bs, Hh, D, dtype=cdt)
    evc = torch.zeros(nbc, bs, Hh, D, dtype=cdt)
    H.oracle_call("flash", w.key, w.value, ekc, evc, compact_slots, w.kv_cache_dtype, float(w.k_scale),
                  float(w.v_scale), threads=8)
    exp_k = ekc.view(nbc * bs, Hh * D)[:active.numel()].view(torch.uint8)
    exp_v = evc.view(nbc * bs, Hh * D)[:active.numel()].view(torch.uint8)

    es = torch.empty((), dtype=cdt).element_size()
    row_bytes = Hh * D * es
    kc = torch.empty(nb * bs, row_bytes, dtype=torch.uint8, device=device)
    vc = torch.empty(nb * bs, row_bytes, dtype=torch.uint8, device=device)
    H.fill_pattern_(kc, 21)
    H.fill_pattern_(vc, 22)
    # remember the fill of each row as a cheap per-row checksum
    def row_sig(c):
        return c.view(nb * bs, -1, 8).view(torch.int64).sum(dim=1)
    sig_k, sig_v = row_sig(kc), row_sig(vc)

    if qkv_on_device is None:
        dkey, dval = w.key.to(device), w.value.to(device)
    else:
        dkey, dval = qkv_on_device
    kc4 = kc.view(cdt).view(nb, bs, Hh, D)
    vc4 = vc.view(cdt).view(nb, bs, Hh, D)
    run_cabi("flash", dkey, dval, kc4, vc4, w.slot_mapping.to(device), w.kv_cache_dtype, w.k_scale.to(device),
             w.v_scale.to(device))
    dslots = w.slot_mapping[active].to(device)
    assert torch.equal(kc[dslots].cpu(), exp_k), "written key rows differ from the oracle"
    assert torch.equal(vc[dslots].cpu(), exp_v), "written value rows differ from the oracle"
    touched = torch.zeros(nb * bs, dtype=torch.bool, device=device)
    touched[dslots] = True
    assert bool((row_sig(kc)[~touched] == sig_k[~touched]).all()), "an untouched key slot changed"
    assert bool((row_sig(vc)[~touched] == sig_v[~touched]).all()), "an untouched value slot changed"
    # a written row differs from its fill (the fill never repeats a whole row of data)
    assert bool((row_sig(kc)[touched] != sig_k[touched]).all())


def test_config_c4_full_size(cuda_device):
    w = workloads.c4()
    assert w.num_tokens == 16384 and w.num_blocks == 65536
    assert float((w.key.float() / w.k_scale).abs().max()) <= 464.0
    # element offsets inside one cache exceed 2^31: 65536 * 64 * 8 * 128 = 2^32
    assert int(w.slot_mapping.max()) * w.num_heads * w.head_size >= 2**31
    _run_workload_rows(w, cuda_device)


def test_config_c4_head_shards_concatenate(cuda_device):
    """Sharding by KV head: the shard caches, concatenated along the head axis, are the unsharded cache."""
    w = workloads.c4(num_tokens=2048, num_blocks=512)
    dev = cuda_device

    def run(wl):
        ksh, _ = wl.cache_shapes()
        kc = torch.zeros(ksh, dtype=torch.uint8, device=dev).view(wl.cache_dtype)
        vc = torch.zeros(ksh, dtype=torch.uint8, device=dev).view(wl.cache_dtype)
        run_cabi("flash", wl.key.to(dev), wl.value.to(dev), kc, vc, wl.slot_mapping.to(dev), wl.kv_cache_dtype,
                 wl.k_scale.to(dev), wl.v_scale.to(dev))
        return kc.view(torch.uint8), vc.view(torch.uint8)

    full_k, full_v = run(w)
    for world in (2, 4, 8):
        parts = [run(workloads.shard_heads(w, r, world)) for r in range(world)]
        assert torch.equal(torch.cat([p[0] for p in parts], dim=2), full_k)
        assert torch.equal(torch.cat([p[1] for p in parts], dim=2), full_v)


@pytest.mark.parametrize("kv", ["auto", "fp8_e4m3"])
def test_config_c5_full_size(kv, cuda_device):
    w = workloads.c5(kv)
    assert w.key.stride(0) == 6144 and not w.key.is_contiguous()
    assert w.num_active == 4096
    # keep key/value as views of ONE fused qkv tensor on the device as well
    qkv = torch.empty(8192, 6144, dtype=torch.bfloat16)
    qkv[:, 2048:4096] = w.key.reshape(8192, 2048)
    qkv[:, 4096:6144] = w.value.reshape(8192, 2048)
    dq = qkv.to(cuda_device)
    dkey = dq[:, 2048:4096].view(8192, 32, 64)
    dval = dq[:, 4096:6144].view(8192, 32, 64)
    _run_workload_rows(w, cuda_device, qkv_on_device=(dkey, dval))


# ----------------------------------------------------------------------------------------------
# properties and edge cases
# ----------------------------------------------------------------------------------------------
def _small_flash(device, kv="fp8", T=500, Hh=4, D=64, bs=16, nb=64, seed=7):
    torch.manual_seed(seed)
    key = torch.randn(T, Hh, D).to(torch.bfloat16).to(device)
    value = torch.randn(T, Hh, D).to(torch.bfloat16).to(device)
    slots = torch.randperm(nb * bs)[:T].to(device)
    cdt = H.cache_torch_dtype(torch.bfloat16, kv)
    kc = H.fill_pattern_(torch.empty(nb, bs, Hh, D, dtype=cdt, device=device), 1)
    vc = H.fill_pattern_(torch.empty(nb, bs, Hh, D, dtype=cdt, device=device), 2)
    return key, value, kc, vc, slots, dev_scale(0.011, device), dev_scale(0.013, device)


@pytest.mark.parametrize("kv", ["auto", "fp8"])
def test_idempotent_and_batch_split(kv, cuda_device):
    key, value, kc, vc, slots, ks, vs = _small_flash(cuda_device, kv)
    kc0, vc0 = kc.clone(), vc.clone()
    run_cabi("flash", key, value, kc, vc, slots, kv, ks, vs)
    once_k, once_v = kc.clone(), vc.clone()
    run_cabi("flash", key, value, kc, vc, slots, kv, ks, vs)  # same call again: nothing changes
    assert H.same_bytes(kc, once_k) and H.same_bytes(vc, once_v)
    # two calls over a split of the tokens = one call over all of them
    run_cabi("flash", key[:123], value[:123], kc0, vc0, slots[:123], kv, ks, vs)
    run_cabi("flash", key[123:], value[123:], kc0, vc0, slots[123:], kv, ks, vs)
    assert H.same_bytes(kc0, once_k) and H.same_bytes(vc0, once_v)


@pytest.mark.parametrize("layout", ["flash", "paged"])
def test_empty_all_skipped_and_short_slot_mapping(layout, cuda_device):
    dev = cuda_device
    T, Hh, D, bs, nb = 40, 2, 32, 8, 16
    key = torch.randn(T, Hh, D, dtype=torch.float16, device=dev)
    value = torch.randn(T, Hh, D, dtype=torch.float16, device=dev)
    if layout == "flash":
        kc = torch.zeros(nb, bs, Hh, D, dtype=torch.float16, device=dev)
        vc = torch.zeros_like(kc)
    else:
        kc = torch.zeros(nb, Hh, D // 8, bs, 8, dtype=torch.float16, device=dev)
        vc = torch.zeros(nb, Hh, D, bs, dtype=torch.float16, device=dev)
    # empty slot_mapping
    run_cabi(layout, key, value, kc, vc, torch.empty(0, dtype=torch.long, device=dev), "auto", None, None)
    assert not bool(kc.any()) and not bool(vc.any())
    # every token skipped
    run_cabi(layout, key, value, kc, vc, torch.full((T,), -1, dtype=torch.long, device=dev), "auto", None, None)
    assert not bool(kc.any()) and not bool(vc.any())
    # slot_mapping shorter than key: only its tokens are written (csrc/cache.cpp:470 of the reference)
    slots = torch.tensor([3, 9, -1, 100, 127], device=dev)
    run_cabi(layout, key, value, kc, vc, slots, "auto", None, None)
    ck, cv = torch.zeros_like(kc).cpu(), torch.zeros_like(vc).cpu()
    H.oracle_call(layout, key.cpu(), value.cpu(), ck, cv, slots.cpu(), "auto", 1.0, 1.0)
    assert H.same_bytes(kc.cpu(), ck) and H.same_bytes(vc.cpu(), cv)
    assert int((kc != 0).any(dim=-1).sum()) > 0


def test_flash_head_strided_cache_and_inputs(cuda_device):
    """Caches stored [num_blocks, H, block_size, D] and viewed as [nb, bs, H, D] (head_stride != D),
    inputs with a padded head stride: the general strides of the C ABI."""
    dev = cuda_device
    T, Hh, D, bs, nb = 77, 4, 64, 16, 8
    torch.manual_seed(3)
    kpad = torch.randn(T, Hh, D + 16).to(torch.bfloat16)
    vpad = torch.randn(T, Hh, D + 16).to(torch.bfloat16)
    key, value = kpad[:, :, :D], vpad[:, :, 8:8 + D]
    slots = torch.randperm(nb * bs)[:T]
    for kv in ("auto", "fp8"):
        cdt = H.cache_torch_dtype(torch.bfloat16, kv)
        kbase = H.fill_pattern_(torch.empty(nb, Hh, bs, D, dtype=cdt), 5)
        vbase = H.fill_pattern_(torch.empty(nb, Hh, bs, D, dtype=cdt), 6)
        dk, dv = kbase.to(dev), vbase.to(dev)
        H.oracle_call("flash", key, value, kbase.permute(0, 2, 1, 3), vbase.permute(0, 2, 1, 3), slots, kv, 0.02, 0.03)
        run_cabi("flash", kpad.to(dev)[:, :, :D], vpad.to(dev)[:, :, 8:8 + D], dk.permute(0, 2, 1, 3),
                 dv.permute(0, 2, 1, 3), slots.to(dev), kv, dev_scale(0.02, dev), dev_scale(0.03, dev))
        assert H.same_bytes(dk.cpu(), kbase) and H.same_bytes(dv.cpu(), vbase)


def test_guard_bands_stay_intact(cuda_device):
    """The caches sit inside a larger allocation; the bytes either side must not change."""
    dev = cuda_device
    T, Hh, D, bs, nb = 64, 8, 128, 16, 4
    key = torch.randn(T, Hh, D, device=dev).to(torch.bfloat16)
    value = torch.randn(T, Hh, D, device=dev).to(torch.bfloat16)
    slots = torch.randperm(nb * bs, device=dev)[:T]
    n = nb * bs * Hh * D
    guard = 4096
    for layout in ("flash", "paged"):
        for kv in ("auto", "fp8"):
            es = 2 if kv == "auto" else 1
            bufk = torch.full((n * es + 2 * guard,), 0xA5, dtype=torch.uint8, device=dev)
            bufv = torch.full((n * es + 2 * guard,), 0x5A, dtype=torch.uint8, device=dev)
            cdt = H.cache_torch_dtype(torch.bfloat16, kv)
            kflat, vflat = bufk[guard:guard + n * es].view(cdt), bufv[guard:guard + n * es].view(cdt)
            if layout == "flash":
                kc, vc = kflat.view(nb, bs, Hh, D), vflat.view(nb, bs, Hh, D)
            else:
                x = 16 // es
                kc, vc = kflat.view(nb, Hh, D // x, bs, x), vflat.view(nb, Hh, D, bs)
            run_cabi(layout, key, value, kc, vc, slots, kv, dev_scale(0.01, dev), dev_scale(0.01, dev))
            for buf, fill in ((bufk, 0xA5), (bufv, 0x5A)):
                assert bool((buf[:guard] == fill).all()) and bool((buf[-guard:] == fill).all())
            # full coverage: every slot was written, nothing of the fill is left inside
            assert int((kflat.view(torch.uint8) == 0xA5).sum()) < n * es // 50


def test_count_bad_slots(cuda_device):
    slots = torch.tensor([0, 5, -1, 63, 64, 1000, -7], device=cuda_device)
    assert cabi.count_bad_slots(slots, 64) == 2
    assert cabi.count_bad_slots(slots, 2000) == 0
    big = torch.arange(1_000_000, device=cuda_device)
    assert cabi.count_bad_slots(big, 999_990) == 10


def test_host_entry_matches_device_entry(cuda_device):
    dev = cuda_device
    T, Hh, D, bs, nb = 1000, 8, 128, 64, 32
    torch.manual_seed(9)
    key = torch.randn(T, Hh, D).to(torch.bfloat16).pin_memory()
    value = torch.randn(T, Hh, D).to(torch.bfloat16).pin_memory()
    slots = torch.randperm(nb * bs)[:T].pin_memory()
    ks, vs = dev_scale(0.01, dev), dev_scale(0.012, dev)
    for kv in ("auto", "fp8"):
        cdt = H.cache_torch_dtype(torch.bfloat16, kv)
        kc1 = torch.zeros(nb, bs, Hh, D, dtype=torch.bfloat16 if kv == "auto" else torch.uint8, device=dev).view(cdt)
        vc1, kc2, vc2 = kc1.clone(), kc1.clone(), kc1.clone()
        run_cabi("flash", key.to(dev), value.to(dev), kc1, vc1, slots.to(dev), kv, ks, vs)
        cabi.reshape_and_cache_flash_host(key, value, kc2, vc2, slots, kv, ks, vs)
        torch.cuda.synchronize()
        assert H.same_bytes(kc1, kc2) and H.same_bytes(vc1, vc2)
    cabi.release_staging()


def test_very_large_batches_are_split_into_several_launches(cuda_device):
    """Batches beyond 2^31 work items go out as several launches.  No test can hold such a batch, so a
    child process lowers the per-launch limit (KVC_TEST_MAX_ITEMS_PER_LAUNCH) and checks a small one."""
    import os
    import subprocess
    import sys
    code = r'''
import sys, torch
sys.path[:0] = [%r, %r]
from oracle import torch_views
from vllm_xpu_kernels import cabi
torch.manual_seed(0)
T, H, D, bs, nb = 1000, 4, 64, 16, 64
key = torch.randn(T, H, D).to(torch.bfloat16); value = torch.randn(T, H, D).to(torch.bfloat16)
slots = torch.randperm(nb * bs)[:T]; slots[::7] = -1
kc = torch.zeros(nb, bs, H, D, dtype=torch.uint8); vc = torch.zeros_like(kc)
dev = torch.device("cuda:0")
dk, dv = kc.to(dev), vc.to(dev)
s = torch.tensor(0.02, device=dev)
cabi.reshape_and_cache_flash(key.to(dev), value.to(dev), dk, dv, slots.to(dev), "fp8", s, s)
torch.cuda.synchronize()
torch_views.run("flash", key, value, kc, vc, slots, "fp8", 0.02, 0.02)
assert torch.equal(dk.cpu(), kc) and torch.equal(dv.cpu(), vc)
print("split ok")
''' % (H.GOLDEN_DIR.rsplit("/tests/", 1)[0], H.GOLDEN_DIR.rsplit("/tests/", 1)[0] + "/vllm-xpu-kernels_b200")
    env = dict(os.environ, KVC_TEST_MAX_ITEMS_PER_LAUNCH="1500")  # 16 items per token -> 93 tokens per launch
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "split ok" in r.stdout, r.stdout + r.stderr


@pytest.mark.parametrize("dtype,kv", [(torch.half, "auto"), (torch.bfloat16, "fp8"), (torch.bfloat16, "auto"),
                                      (torch.float, "auto"), (torch.half, "fp8_e5m2")])
@pytest.mark.parametrize("bs", [16, 32, 64, 8, 48])
def test_paged_sequence_like_slots(dtype, kv, bs, cuda_device):
    """Slot patterns a prefill produces -- whole aligned runs, runs that start mid-block, cross a block
    boundary, contain padding or run backwards -- exercise the vector V stores and their fallbacks."""
    dev = cuda_device
    Hh, D, nb = 3, 64, 40
    g = torch.Generator().manual_seed(bs)
    blocks = torch.randperm(nb, generator=g).tolist()
    slots = []
    b = iter(blocks)
    def run(block, start, n):
        return [block * bs + start + i for i in range(n)]
    slots += run(next(b), 0, bs)                       # a whole block
    slots += run(next(b), 0, bs) + run(next(b), 0, bs)  # two whole blocks back to back
    slots += run(next(b), bs // 2, bs - bs // 2)       # starts mid-block
    slots += run(next(b), 0, bs // 2)                  # ends mid-block
    hole = run(next(b), 0, bs)
    hole[bs // 3] = -1                                 # padding inside a run
    slots += hole
    slots += list(reversed(run(next(b), 0, bs)))       # descending offsets
    blk2 = next(b)
    slots += [blk2 * bs + (i * 7) % bs for i in range(bs)] if bs % 7 else run(blk2, 0, bs)  # permuted offsets
    slots += run(next(b), 0, 16 if bs >= 16 else bs)   # a run of 16 at offset 0
    slots += run(next(b), 16, 16) if bs >= 32 else []  # a run of 16 at offset 16
    slots += run(next(b), 8, 16) if bs >= 32 else []   # a run of 16 at offset 8 (not vector-aligned)
    slots += [-1] * 5 + run(next(b), 0, bs)            # padding shifts the run against the warp's halves
    T = len(slots)
    slots = torch.tensor(slots, dtype=torch.long)
    torch.manual_seed(bs + 1)
    key = torch.randn(T, Hh, D).to(dtype)
    value = torch.randn(T, Hh, D).to(dtype)
    cdt = H.cache_torch_dtype(dtype, kv)
    x = 16 // torch.empty((), dtype=cdt).element_size()
    kc = H.fill_pattern_(torch.empty(nb, Hh, D // x, bs, x, dtype=cdt), 5)
    vc = H.fill_pattern_(torch.empty(nb, Hh, D, bs, dtype=cdt), 6)
    dkc, dvc = kc.to(dev), vc.to(dev)
    fmax = 57344.0 if kv == "fp8_e5m2" else 448.0
    ks = float(key.float().abs().amax() / fmax)
    vs = float(value.float().abs().amax() / fmax)
    H.oracle_call("paged", key, value, kc, vc, slots, kv, ks, vs)
    run_cabi("paged", key.to(dev), value.to(dev), dkc, dvc, slots.to(dev), kv, dev_scale(ks, dev), dev_scale(vs, dev))
    assert H.same_bytes(dkc.cpu(), kc), "key cache differs"
    assert H.same_bytes(dvc.cpu(), vc), "value cache differs"
    # a misaligned value cache base must fall back to element stores and still be right
    buf = torch.zeros(vc.numel() * vc.element_size() + 64, dtype=torch.uint8, device=dev)
    es = vc.element_size()
    dvc2 = buf[16:16 + vc.numel() * es].view(cdt).view(vc.shape)
    dvc2.copy_(H.fill_pattern_(torch.empty(nb, Hh, D, bs, dtype=cdt), 6).to(dev))
    dkc2 = H.fill_pattern_(torch.empty(nb, Hh, D // x, bs, x, dtype=cdt), 5).to(dev)
    run_cabi("paged", key.to(dev), value.to(dev), dkc2, dvc2, slots.to(dev), kv, dev_scale(ks, dev), dev_scale(vs, dev))
    assert H.same_bytes(dvc2.cpu(), vc), "value cache (16-byte-offset base) differs"


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,kv", [(torch.half, "auto"), (torch.bfloat16, "fp8"), (torch.float, "auto"),
                                      (torch.float, "fp8"), (torch.half, "fp8_e5m2")])
@pytest.mark.parametrize("D", [128, 40, 20, 6])
def test_paged_runs_and_scattered_slots_in_one_batch(dtype, kv, D, cuda_device):
    """Groups of 32 tokens that hold runs, groups with scattered slots, groups that are half and half, padding
    and a ragged tail in one call: each warp picks the order of its V stores from its own 32 slots (lane =
    token for runs, lane = head dimension for scattered slots), and both orders must give the oracle's bytes
    for every vector width the head size allows."""
    if kv != "auto" and D % 2:
        pytest.skip("fp8 caches pack two elements")
    dev = cuda_device
    Hh, bs, nb = 3, 16, 96
    g = torch.Generator().manual_seed(D)
    free = torch.randperm(nb * bs, generator=g).tolist()
    blocks = torch.randperm(nb, generator=g).tolist()
    slots: list[int] = []
    used: set[int] = set()

    def run(n):
        b = blocks.pop()
        out = [b * bs + i for i in range(n)]
        used.update(out)
        return out

    def scattered(n):
        out = []
        while len(out) < n:
            s = free.pop()
            if s // bs in blocks:  # blocks still unassigned to a run
                blocks.remove(s // bs)
            if s not in used:
                used.add(s)
                out.append(s)
        return out

    slots += run(16) + run(16)            # a warp of runs
    slots += scattered(32)                # a warp of scattered slots
    slots += run(16) + scattered(16)      # 15 adjacent pairs: scattered order
    slots += run(16) + run(8) + scattered(8)   # 22 adjacent pairs: run order
    mixed = scattered(32)
    for i in (0, 5, 6, 31):
        mixed[i] = -1                     # padding among scattered slots
    slots += mixed
    slots += [-1] * 32                    # a warp with nothing to do
    slots += scattered(11)                # ragged tail
    T = len(slots)
    slots_t = torch.tensor(slots, dtype=torch.long)
    torch.manual_seed(D + 3)
    key = torch.randn(T, Hh, D).to(dtype)
    value = torch.randn(T, Hh, D).to(dtype)
    cdt = H.cache_torch_dtype(dtype, kv)
    x = 16 // torch.empty((), dtype=cdt).element_size()
    if D % x:
        x = 2 if D % 2 == 0 else 1
    kc = H.fill_pattern_(torch.empty(nb, Hh, D // x, bs, x, dtype=cdt), 5)
    vc = H.fill_pattern_(torch.empty(nb, Hh, D, bs, dtype=cdt), 6)
    dkc, dvc = kc.to(dev), vc.to(dev)
    fmax = 57344.0 if kv == "fp8_e5m2" else 448.0
    ks = float(key.float().abs().amax() / fmax)
    vs = float(value.float().abs().amax() / fmax)
    H.oracle_call("paged", key, value, kc, vc, slots_t, kv, ks, vs)
    run_cabi("paged", key.to(dev), value.to(dev), dkc, dvc, slots_t.to(dev), kv, dev_scale(ks, dev), dev_scale(vs, dev))
    assert H.same_bytes(dkc.cpu(), kc), "key cache differs"
    assert H.same_bytes(dvc.cpu(), vc), "value cache differs"
