"""Seeded random sweep over shapes, strides, dtypes and store modes: every case is compared
byte for byte with the CPU oracle.  Catches index-arithmetic and vector-width selection errors
that the fixed matrices do not reach (odd head counts, padded rows, views with offsets)."""
import random

import pytest
import torch

from oracle import torch_views
from tests import helpers as H
from vllm_xpu_kernels import cabi

pytestmark = pytest.mark.gpu

DTYPES = [torch.float16, torch.bfloat16, torch.float32]


def _rand_case(rng: random.Random):
    layout = rng.choice(["flash", "flash", "paged", "mla"])
    dtype = rng.choice(DTYPES)
    kv = rng.choice(["auto", "fp8", "fp8_e5m2"])
    T = rng.choice([1, 2, 3, 17, 63, 64, 65, 200, 511])
    bs = rng.choice([1, 2, 8, 12, 16, 32, 64])
    nb = max(2, (T + bs - 1) // bs + rng.randint(0, 5))
    return layout, dtype, kv, T, bs, nb


@pytest.mark.parametrize("seed", range(120))
def test_random_case(seed, cuda_device):
    rng = random.Random(seed)
    torch.manual_seed(seed)
    layout, dtype, kv, T, bs, nb = _rand_case(rng)
    dev = cuda_device
    cdt = H.cache_torch_dtype(dtype, kv)
    es_out = torch.empty((), dtype=cdt).element_size()
    slots = rng.sample(range(nb * bs), T)
    for i in rng.sample(range(T), rng.randint(0, T // 3)):
        slots[i] = -1
    slots = torch.tensor(slots, dtype=torch.long)
    scale_k = rng.choice([0.013, 1.0, 0.5, 3.0e-4, 11.0])
    scale_v = rng.choice([0.021, 2.0, 7.0e-3])
    pad_t = rng.choice([0, 0, 8, 16, 3])      # extra elements per token row
    off = rng.choice([0, 0, 8, 16, 1])        # view offset inside the row

    if layout == "mla":
        R, P = rng.choice([(512, 64), (64, 16), (48, 24), (10, 6), (128, 0), (0, 64)])
        big_c = torch.randn(T + 1, R + pad_t + off).to(dtype)
        big_p = torch.randn(T + 1, P + pad_t + off).to(dtype)
        kv_c, k_pe = big_c[:, off:off + R], big_p[:, off:off + P]
        alloc = H.fill_pattern_(torch.empty(nb, bs, R + P + pad_t, dtype=cdt), seed)
        cache = alloc[:, :, :R + P]
        dalloc = alloc.to(dev)
        torch_views.run_mla(kv_c, k_pe, cache, slots, kv, scale_k)
        cabi.concat_and_cache_mla(big_c.to(dev)[:, off:off + R], big_p.to(dev)[:, off:off + P],
                                  dalloc[:, :, :R + P], slots.to(dev), kv,
                                  torch.tensor(scale_k, dtype=torch.float32, device=dev))
        torch.cuda.synchronize()
        assert H.same_bytes(dalloc.cpu(), alloc), (layout, dtype, kv, T, bs, nb, R, P, pad_t, off)
        return

    Hh = rng.choice([1, 2, 3, 8, 5])
    if layout == "paged":
        x = 16 // es_out
        D = x * rng.choice([1, 2, 4, 8, 5])
    else:
        D = rng.choice([8, 16, 20, 64, 80, 96, 128, 7, 256])
    # key/value as views of a fused tensor: token stride and head stride both larger than needed
    head_pad = rng.choice([0, 0, 8, 16])
    fused = torch.randn(T + 2, 2, Hh, D + head_pad + off).to(dtype)
    key, value = fused[:, 0, :, off:off + D], fused[:, 1, :, off:off + D]
    dfused = fused.to(dev)
    dkey, dvalue = dfused[:, 0, :, off:off + D], dfused[:, 1, :, off:off + D]
    if layout == "flash":
        # both caches inside one allocation with a padded head dim: strided in dims 0..2
        alloc = H.fill_pattern_(torch.empty(nb, 2, bs, Hh, D + pad_t, dtype=cdt), seed)
        kc, vc = alloc[:, 0, :, :, :D], alloc[:, 1, :, :, :D]
        dalloc = alloc.to(dev)
        dkc, dvc = dalloc[:, 0, :, :, :D], dalloc[:, 1, :, :, :D]
        torch_views.run("flash", key, value, kc, vc, slots, kv, scale_k, scale_v)
        cabi.reshape_and_cache_flash(dkey, dvalue, dkc, dvc, slots.to(dev), kv,
                                     torch.tensor(scale_k, dtype=torch.float32, device=dev),
                                     torch.tensor(scale_v, dtype=torch.float32, device=dev))
        torch.cuda.synchronize()
        assert H.same_bytes(dalloc.cpu(), alloc), (layout, dtype, kv, T, Hh, D, bs, nb, pad_t, off, head_pad)
    else:
        kc = H.fill_pattern_(torch.empty(nb, Hh, D // x, bs, x, dtype=cdt), seed)
        vc = H.fill_pattern_(torch.empty(nb, Hh, D, bs, dtype=cdt), seed + 1)
        dkc, dvc = kc.to(dev), vc.to(dev)
        torch_views.run("paged", key, value, kc, vc, slots, kv, scale_k, scale_v)
        cabi.reshape_and_cache(dkey, dvalue, dkc, dvc, slots.to(dev), kv,
                               torch.tensor(scale_k, dtype=torch.float32, device=dev),
                               torch.tensor(scale_v, dtype=torch.float32, device=dev))
        torch.cuda.synchronize()
        assert H.same_bytes(dkc.cpu(), kc) and H.same_bytes(dvc.cpu(), vc), (layout, dtype, kv, T, Hh, D, bs, nb, off)
