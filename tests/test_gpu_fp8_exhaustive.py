"""Every 16-bit input pattern x many scales through the fp8 store path, against the oracle.

The kernels divide with a three-instruction sequence inside a scale window and with the
IEEE divide outside it; both, and every vector width, must give the oracle's byte."""
import numpy as np
import pytest
import torch

import oracle
from vllm_xpu_kernels import cabi

pytestmark = pytest.mark.gpu

ORC = {torch.bfloat16: "bf16", torch.float16: "f16"}


def all_patterns(dtype, device):
    return torch.arange(65536, dtype=torch.int32).to(torch.int16).view(dtype).to(device)


def scale_set(n_random: int, seed: int) -> np.ndarray:
    rng = np.random.default_rng(seed)
    rnd = np.exp2(rng.uniform(-24, 24, n_random)).astype(np.float32)
    rnd[::7] *= -1  # negative scales are legal IEEE operands
    near_one = (1.0 + rng.uniform(-1e-3, 1e-3, 32)).astype(np.float32)
    special = np.array([
        1.0, 2.0, 0.5, 3.0, 1 / 3, 448.0, 1 / 448, 0.0078125, 2.0**-60, 2.0**60, np.nextafter(np.float32(2.0**-60), 0),
        np.nextafter(np.float32(2.0**60), np.float32(np.inf)), 2.0**-61, 2.0**61, 1e-30, 1e30, 1e-38, 1e-40, 1e-45,
        3.4028235e38, -1.0, -0.37, 0.0, -0.0, np.inf, -np.inf, np.nan, 2.0**-126, 2.0**-100, 2.0**100, 2.0**127,
        # edges of the fp16 fast window [2^-20, 64] and scales where 512*s leaves the fp16 range
        2.0**-20, np.nextafter(np.float32(2.0**-20), np.float32(0)), 64.0, np.nextafter(np.float32(64.0), np.float32(100)),
        100.0, 127.9, 128.0, 1000.0, 2.0**-21, 2.0**-23, 2.0**-24, 0.25, np.nextafter(np.float32(0.25), np.float32(1)), 0.49, 1.07,
    ], dtype=np.float32)
    return np.concatenate([special, near_one, rnd])


def run_flash(x_dev, shape, kv, scale, device, cache_stride_pad=0):
    T, Hh, D = shape
    key = x_dev.view(T, Hh, D)
    bs = 16
    nb = (T + bs - 1) // bs
    kc = torch.zeros(nb, bs, Hh, D + cache_stride_pad, dtype=torch.uint8, device=device)[..., :D]
    vc = torch.zeros(nb, bs, Hh, D + cache_stride_pad, dtype=torch.uint8, device=device)[..., :D]
    slots = torch.arange(T, device=device)
    s = torch.tensor(scale, dtype=torch.float32, device=device)
    cabi.reshape_and_cache_flash(key, key, kc, vc, slots, kv, s, s)
    return kc.reshape(-1)[:65536], vc.reshape(-1)[:65536]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("kv", ["fp8_e4m3", "fp8_e5m2"])
def test_all_inputs_many_scales(dtype, kv, cuda_device):
    x = all_patterns(dtype, cuda_device)
    scales = scale_set(1500 if kv == "fp8_e4m3" else 300, seed=1)
    bad = []
    for s in scales:
        want = torch.from_numpy(oracle.convert_table(ORC[dtype], kv, float(s))).to(cuda_device)
        gk, gv = run_flash(x, (64, 8, 128), kv, float(s), cuda_device)
        if not (torch.equal(gk, want) and torch.equal(gv, want)):
            idx = (gk != want).nonzero().flatten()[:4].tolist()
            bad.append((float(s), [(i, int(gk[i]), int(want[i])) for i in idx]))
    assert not bad, f"{len(bad)} scales differ, first: {bad[:3]}"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("head_size,pad", [(8, 0), (4, 0), (2, 0), (1, 0), (12, 4), (6, 2)])
def test_narrow_vector_paths(dtype, head_size, pad, cuda_device):
    """Head sizes that force 8-, 4-, 2- and 1-element chunks (the last two always use the IEEE divide)."""
    x = all_patterns(dtype, cuda_device)
    n = 65536 // head_size * head_size
    for s in scale_set(24, seed=2):
        want = torch.from_numpy(oracle.convert_table(ORC[dtype], "fp8", float(s))).to(cuda_device)[:n]
        T = n // head_size // 4
        gk, gv = run_flash(x[:T * 4 * head_size], (T, 4, head_size), "fp8", float(s), cuda_device, cache_stride_pad=pad)
        assert torch.equal(gk[:T * 4 * head_size], want[:T * 4 * head_size]), (float(s), head_size)
        assert torch.equal(gv[:T * 4 * head_size], want[:T * 4 * head_size]), (float(s), head_size)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_paged_layout_conversion(dtype, cuda_device):
    """Same conversion core in the paged kernel: K cache [nb, H, D/16, bs, 16], V cache [nb, H, D, bs]."""
    x = all_patterns(dtype, cuda_device)
    T, Hh, D, bs = 64, 8, 128, 16
    key = x.view(T, Hh, D)
    slots = torch.arange(T, device=cuda_device)
    for s in scale_set(48, seed=3):
        want = torch.from_numpy(oracle.convert_table(ORC[dtype], "fp8", float(s))).to(cuda_device).view(T, Hh, D)
        kc = torch.zeros(T // bs, Hh, D // 16, bs, 16, dtype=torch.uint8, device=cuda_device)
        vc = torch.zeros(T // bs, Hh, D, bs, dtype=torch.uint8, device=cuda_device)
        sc = torch.tensor(float(s), dtype=torch.float32, device=cuda_device)
        cabi.reshape_and_cache(key, key, kc, vc, slots, "fp8", sc, sc)
        # undo the layouts: token t = block t//bs, offset t%bs
        k_back = kc.permute(0, 3, 1, 2, 4).reshape(T, Hh, D)
        v_back = vc.permute(0, 3, 1, 2).reshape(T, Hh, D)
        assert torch.equal(k_back, want) and torch.equal(v_back, want), float(s)


def test_float32_inputs_use_ieee_division(cuda_device):
    rng = np.random.default_rng(5)
    raw = rng.integers(0, 2**32, 1 << 18, dtype=np.uint64).astype(np.uint32).view(np.float32)
    vals = np.concatenate([raw, rng.standard_normal(1 << 18).astype(np.float32) * 3]).astype(np.float32)
    x = torch.from_numpy(vals).to(cuda_device)
    T = vals.size // (8 * 128)
    for s in scale_set(16, seed=4):
        want = torch.from_numpy(oracle.convert_f32(vals, "fp8", float(s))).to(cuda_device)
        kc = torch.zeros(T // 16, 16, 8, 128, dtype=torch.uint8, device=cuda_device)
        vc = torch.zeros_like(kc)
        sc = torch.tensor(float(s), dtype=torch.float32, device=cuda_device)
        key = x.view(T, 8, 128)
        cabi.reshape_and_cache_flash(key, key, kc, vc, torch.arange(T, device=cuda_device), "fp8", sc, sc)
        assert torch.equal(kc.view(-1), want) and torch.equal(vc.view(-1), want), float(s)
