"""Concurrent use: independent calls on different streams and from different host threads must not
disturb each other (the device-pointer entry points keep no shared mutable state; the error text is
per thread)."""
import threading

import pytest
import torch

from tests import helpers as H
from vllm_xpu_kernels import cabi

pytestmark = pytest.mark.gpu


def _case(dev, seed, T=3000, Hh=8, D=128, bs=16, nb=256):
    g = torch.Generator().manual_seed(seed)
    key = torch.randn(T, Hh, D, generator=g).to(torch.bfloat16)
    value = torch.randn(T, Hh, D, generator=g).to(torch.bfloat16)
    slots = torch.randperm(nb * bs, generator=g)[:T]
    kc = torch.zeros(nb, bs, Hh, D, dtype=torch.uint8)
    vc = torch.zeros_like(kc)
    scale = 0.01 + 0.001 * seed
    H.oracle_call("flash", key, value, kc, vc, slots, "fp8", scale, scale, threads=4)
    d = dict(key=key.to(dev), value=value.to(dev), slots=slots.to(dev), kc=torch.zeros_like(kc, device=dev),
             vc=torch.zeros_like(vc, device=dev), s=torch.tensor(scale, dtype=torch.float32, device=dev))
    return d, kc, vc


def test_two_streams(cuda_device):
    cases = [_case(cuda_device, s) for s in (1, 2)]
    streams = [torch.cuda.Stream() for _ in cases]
    torch.cuda.synchronize()
    for _ in range(20):  # interleave launches of the two streams
        for (d, _, _), st in zip(cases, streams):
            cabi.reshape_and_cache_flash(d["key"], d["value"], d["kc"], d["vc"], d["slots"], "fp8", d["s"], d["s"],
                                         stream=st)
    torch.cuda.synchronize()
    for d, kc, vc in cases:
        assert torch.equal(d["kc"].cpu(), kc) and torch.equal(d["vc"].cpu(), vc)


def test_host_threads(cuda_device):
    n = 4
    cases = [_case(cuda_device, 10 + i, T=1000) for i in range(n)]
    streams = [torch.cuda.Stream() for _ in range(n)]
    errors = []

    def work(i):
        try:
            torch.cuda.set_device(cuda_device)
            d = cases[i][0]
            for _ in range(50):
                cabi.reshape_and_cache_flash(d["key"], d["value"], d["kc"], d["vc"], d["slots"], "fp8", d["s"], d["s"],
                                             stream=streams[i])
            # a failing call on this thread must report its own message
            try:
                cabi.parse_kv_cache_dtype(f"bogus{i}")
            except RuntimeError as e:
                assert f"bogus{i}" in str(e)
            else:
                raise AssertionError("expected an error")
        except Exception as e:  # noqa: BLE001
            errors.append((i, repr(e)))

    threads = [threading.Thread(target=work, args=(i,)) for i in range(n)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    torch.cuda.synchronize()
    assert not errors, errors
    for d, kc, vc in cases:
        assert torch.equal(d["kc"].cpu(), kc) and torch.equal(d["vc"].cpu(), vc)
