"""The allocation-free host entry point against the allocating one.

Some callers reach the cache write when the serving framework already owns all free GPU
memory, or sit on a path where cudaMalloc's synchronisation is not acceptable; for them
``kvc_reshape_and_cache_flash_host_noalloc`` stages key/value/slot_mapping in a fixed 16 MiB
area inside the library instead of allocating.  This file is named to be collected last, so a
failure here cannot hide the result of any other test; it passes alone in a fresh process and
after the rest of the suite.  Results are compared bit for bit, the tolerance every test of
this integer/byte path uses, on two calls in a row that share the staging area, with the
library's other entry points and with the CPU oracle.
"""
import pytest
import torch

from tests import helpers as H_
from vllm_xpu_kernels import cabi

pytestmark = pytest.mark.gpu


def _same(a: torch.Tensor, b: torch.Tensor) -> bool:
    return bool(torch.equal(a.contiguous().view(torch.uint8), b.contiguous().view(torch.uint8)))


def _batch(T, H, D, nb, bs, seed, skip_every=0):
    torch.manual_seed(seed)
    key = torch.randn(T, H, D).to(torch.bfloat16).pin_memory()
    value = torch.randn(T, H, D).to(torch.bfloat16).pin_memory()
    slots = torch.randperm(nb * bs)[:T].clone()
    if skip_every:
        slots[::skip_every] = -1
    return key, value, slots.pin_memory()


@pytest.mark.parametrize("kv", ["fp8", "auto"])
def test_noalloc_entry_matches_allocating_entry_twice_in_a_row(kv, cuda_device):
    dev = cuda_device
    H, D, bs, nb = 8, 128, 64, 64
    cdt = torch.uint8 if kv == "fp8" else torch.bfloat16
    ks = torch.tensor(0.011, dtype=torch.float32, device=dev)
    vs = torch.tensor(0.013, dtype=torch.float32, device=dev)
    kc_new = torch.zeros(nb, bs, H, D, dtype=cdt, device=dev)
    vc_new = torch.zeros_like(kc_new)
    kc_old, vc_old = torch.zeros_like(kc_new), torch.zeros_like(kc_new)
    # first call fills most of the fixed area; the second is smaller, has padding, and must not see leftovers
    for T, seed, skip in ((4000, 1, 0), (777, 2, 5)):
        key, value, slots = _batch(T, H, D, nb, bs, seed, skip)
        cabi.reshape_and_cache_flash_host_noalloc(key, value, kc_new, vc_new, slots, kv, ks, vs)
        cabi.reshape_and_cache_flash_host(key, value, kc_old, vc_old, slots, kv, ks, vs)
        torch.cuda.synchronize()
        assert _same(kc_new, kc_old), f"key cache differs after the T={T} call"
        assert _same(vc_new, vc_old), f"value cache differs after the T={T} call"
        assert bool(kc_new.view(torch.uint8).any())
    # and against the device-pointer entry on the last batch
    kc_dev, vc_dev = torch.zeros_like(kc_new), torch.zeros_like(kc_new)
    for T, seed, skip in ((4000, 1, 0), (777, 2, 5)):
        key, value, slots = _batch(T, H, D, nb, bs, seed, skip)
        cabi.reshape_and_cache_flash(key.to(dev), value.to(dev), kc_dev, vc_dev, slots.to(dev), kv, ks, vs)
    torch.cuda.synchronize()
    assert _same(kc_new, kc_dev) and _same(vc_new, vc_dev)
    # and against the CPU oracle directly, both batches into one host cache
    cache_dt = torch.float8_e4m3fn if kv == "fp8" else torch.bfloat16
    kc_cpu = torch.zeros(nb, bs, H, D, dtype=cdt).view(cache_dt)
    vc_cpu = torch.zeros(nb, bs, H, D, dtype=cdt).view(cache_dt)
    for T, seed, skip in ((4000, 1, 0), (777, 2, 5)):
        key, value, slots = _batch(T, H, D, nb, bs, seed, skip)
        H_.oracle_call("flash", key, value, kc_cpu, vc_cpu, slots, kv, float(ks), float(vs))
    assert _same(kc_new.cpu(), kc_cpu), "key cache differs from the oracle's"
    assert _same(vc_new.cpu(), vc_cpu), "value cache differs from the oracle's"
    cabi.release_staging()


def test_noalloc_entry_strided_host_rows(cuda_device):
    """Host rows taken out of a fused qkv buffer (token stride 3*H*D) are packed on the way in."""
    dev = cuda_device
    T, H, D, bs, nb = 512, 4, 64, 16, 64
    torch.manual_seed(3)
    qkv = torch.randn(T, 3, H, D).to(torch.bfloat16).pin_memory()
    key, value = qkv[:, 1], qkv[:, 2]
    slots = torch.randperm(nb * bs)[:T].pin_memory()
    a = [torch.zeros(nb, bs, H, D, dtype=torch.bfloat16, device=dev) for _ in range(4)]
    cabi.reshape_and_cache_flash_host_noalloc(key, value, a[0], a[1], slots, "auto")
    cabi.reshape_and_cache_flash(key.to(dev), value.to(dev), a[2], a[3], slots.to(dev), "auto")
    torch.cuda.synchronize()
    assert _same(a[0], a[2]) and _same(a[1], a[3])


def test_noalloc_entry_rejects_what_does_not_fit(cuda_device):
    dev = cuda_device
    H, D, bs, nb = 8, 128, 64, 128
    T = 4100  # 2 * 4100 * 2048 B + slots > 16 MiB
    key, value, slots = _batch(T, H, D, nb, bs, 4)
    kc = torch.zeros(nb, bs, H, D, dtype=torch.bfloat16, device=dev)
    vc = torch.zeros_like(kc)
    with pytest.raises(RuntimeError, match="fixed"):
        cabi.reshape_and_cache_flash_host_noalloc(key, value, kc, vc, slots, "auto")
    torch.cuda.synchronize()
    assert not bool(kc.any()) and not bool(vc.any())  # nothing was enqueued
    assert cabi.NOALLOC_STAGING_BYTES == 16 * 1024 * 1024
