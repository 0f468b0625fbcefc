"""The two latency sweeps retargeted to CUDA (benchmark/benchmark_reshape_and_cache{,_flash}.py; the
reference's are benchmark/benchmark_reshape_and_cache_flash.py:16-144 and
benchmark/benchmark_reshape_and_cache.py:57-207 there): one point of each sweep runs, reports a finite
positive latency, and leaves in the caches exactly the bytes the CPU oracle writes for that input."""
import math

import pytest
import torch

import benchmark_reshape_and_cache as sweep_paged
import benchmark_reshape_and_cache_flash as sweep_flash
from tests import helpers as H

pytestmark = pytest.mark.gpu


def _oracle_caches(layout, tensors, kv):
    key, value, key_cache, value_cache, slots, k_scale, v_scale = tensors
    # the oracle starts from the caches as the sweep allocates them: zeros
    kc = torch.zeros(key_cache.shape, dtype=torch.uint8 if key_cache.element_size() == 1 else key_cache.dtype)
    vc = torch.zeros(value_cache.shape, dtype=kc.dtype)
    if key_cache.element_size() == 1:
        kc, vc = kc.view(key_cache.dtype), vc.view(value_cache.dtype)
    H.oracle_call(layout, key.cpu(), value.cpu(), kc, vc, slots.cpu(), kv, float(k_scale), float(v_scale))
    return kc, vc


@pytest.mark.parametrize("dtype,kv", [(torch.half, "auto"), (torch.bfloat16, "fp8_e4m3")])
def test_flash_sweep_point(dtype, kv, cuda_device):
    args = dict(num_tokens=256, num_heads=8, head_size=128, block_size=64, num_blocks=512, dtype=dtype,
                kv_cache_dtype=kv)
    med, best = sweep_flash.run_benchmark(num_iters=10, **args)
    assert math.isfinite(med) and math.isfinite(best) and 0 < best <= med < 1e-2
    call, tensors = sweep_flash.make_case(**args)
    call()
    torch.cuda.synchronize()
    kc, vc = _oracle_caches("flash", tensors, kv)
    assert H.same_bytes(tensors[2].cpu(), kc), "key cache differs from the oracle's"
    assert H.same_bytes(tensors[3].cpu(), vc), "value cache differs from the oracle's"


@pytest.mark.parametrize("slots_mode", ["random", "runs"])
def test_paged_sweep_point(slots_mode, cuda_device):
    args = dict(num_tokens=256, num_heads=12, head_size=128, block_size=64, num_blocks=1024, dtype=torch.half,
                kv_cache_dtype="auto")
    med, best = sweep_paged.run_benchmark(num_iters=10, slots_mode=slots_mode, flush_l2=True, **args)
    assert math.isfinite(med) and math.isfinite(best) and 0 < best <= med < 1e-2
    call, tensors = sweep_paged.make_case(slots_mode=slots_mode, **args)
    call()
    torch.cuda.synchronize()
    kc, vc = _oracle_caches("paged", tensors, "auto")
    assert H.same_bytes(tensors[2].cpu(), kc), "key cache differs from the oracle's"
    assert H.same_bytes(tensors[3].cpu(), vc), "value cache differs from the oracle's"
