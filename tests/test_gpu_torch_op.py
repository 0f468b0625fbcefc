"""The torch-dispatcher face of the library (``torch.ops._C_cache_ops.*``), as vLLM calls it."""
import pytest
import torch

from tests import helpers as H
from vllm_xpu_kernels import cabi
from vllm_xpu_kernels import ops  # imports vllm_xpu_kernels._C

pytestmark = pytest.mark.gpu

OPCHECK_UTILS = ("test_schema", "test_autograd_registration", "test_faketensor", "test_aot_dispatch_dynamic")


def _inputs(device, layout, kv, dtype=torch.bfloat16, T=42, Hh=8, D=64, bs=16, nb=32, seed=0):
    torch.manual_seed(seed)
    qkv = torch.randn(T, 3, Hh, D, device=device).to(dtype)
    _, key, value = qkv.unbind(dim=1)
    slots = torch.randperm(nb * bs, device=device)[:T]
    cdt = H.cache_torch_dtype(dtype, kv)
    if layout == "flash":
        both = H.fill_pattern_(torch.empty(nb, 2, bs, Hh, D, dtype=cdt, device=device), 3)
        kc, vc = both[:, 0], both[:, 1]
    else:
        x = 16 // torch.empty((), dtype=cdt).element_size()
        kc = H.fill_pattern_(torch.empty(nb, Hh, D // x, bs, x, dtype=cdt, device=device), 3)
        vc = H.fill_pattern_(torch.empty(nb, Hh, D, bs, dtype=cdt, device=device), 4)
    ks = (key.float().abs().amax() / 448).to(torch.float32)
    vs = (value.float().abs().amax() / 448).to(torch.float32)
    return key, value, kc, vc, slots, ks, vs


@pytest.mark.parametrize("layout", ["flash", "paged"])
@pytest.mark.parametrize("kv", ["auto", "fp8", "fp8_e4m3"])
def test_op_equals_c_abi(layout, kv, cuda_device):
    key, value, kc, vc, slots, ks, vs = _inputs(cuda_device, layout, kv)
    kc2, vc2 = kc.clone(), vc.clone()
    ock, ocv = kc.cpu(), vc.cpu()  # contiguous CPU copies of the caches before the call
    fn = ops.reshape_and_cache_flash if layout == "flash" else ops.reshape_and_cache
    fn(key, value, kc, vc, slots, kv, ks, vs)
    cfn = cabi.reshape_and_cache_flash if layout == "flash" else cabi.reshape_and_cache
    cfn(key, value, kc2, vc2, slots, kv, ks, vs)
    torch.cuda.synchronize()
    assert H.same_bytes(kc, kc2) and H.same_bytes(vc, vc2)
    H.oracle_call(layout, key.cpu(), value.cpu(), ock, ocv, slots.cpu(), kv, float(ks), float(vs))
    assert H.same_bytes(kc.cpu(), ock) and H.same_bytes(vc.cpu(), ocv)


def test_uint8_cache_is_accepted_for_fp8(cuda_device):
    key, value, kc, vc, slots, ks, vs = _inputs(cuda_device, "flash", "fp8")
    kc8, vc8 = kc.clone().view(torch.uint8), vc.clone().view(torch.uint8)
    ops.reshape_and_cache_flash(key, value, kc, vc, slots, "fp8", ks, vs)
    ops.reshape_and_cache_flash(key, value, kc8, vc8, slots, "fp8", ks, vs)
    assert H.same_bytes(kc.view(torch.uint8), kc8) and H.same_bytes(vc.view(torch.uint8), vc8)


@pytest.mark.parametrize("layout", ["flash", "paged"])
def test_opcheck(layout, cuda_device):
    key, value, kc, vc, slots, ks, vs = _inputs(cuda_device, layout, "auto", dtype=torch.float16)
    op = torch.ops._C_cache_ops.reshape_and_cache_flash if layout == "flash" else torch.ops._C_cache_ops.reshape_and_cache
    torch.library.opcheck(op, (key, value, kc, vc, slots, "auto", ks, vs), test_utils=OPCHECK_UTILS)


def test_errors(cuda_device):
    key, value, kc, vc, slots, ks, vs = _inputs(cuda_device, "flash", "auto")
    f = ops.reshape_and_cache_flash
    with pytest.raises(RuntimeError, match="Unsupported data type of kv cache: int8"):
        f(key, value, kc, vc, slots, "int8", ks, vs)
    with pytest.raises(RuntimeError, match="Unsupported input type of kv cache"):
        f(key.to(torch.float64), value.to(torch.float64), kc, vc, slots, "auto", ks, vs)
    with pytest.raises(RuntimeError, match="slot_mapping must be int64"):
        f(key, value, kc, vc, slots.to(torch.int32), "auto", ks, vs)
    with pytest.raises(RuntimeError, match="same strides"):
        f(key, value, kc, vc.contiguous(), slots, "auto", ks, vs)
    with pytest.raises(RuntimeError, match="does not match kv_cache_dtype"):
        f(key, value, kc, vc, slots, "fp8", ks, vs)
    with pytest.raises(RuntimeError, match="longer than key"):
        f(key[:10], value[:10], kc, vc, slots, "auto", ks, vs)
    with pytest.raises(RuntimeError, match="same device"):
        f(key, value, kc, vc, slots.cpu(), "auto", ks, vs)
    with pytest.raises(RuntimeError, match="key_cache shape"):
        f(key[:, :4], value[:, :4], kc, vc, slots, "auto", ks, vs)
    key8, value8, kc8, vc8, slots8, ks8, vs8 = _inputs(cuda_device, "flash", "fp8")
    with pytest.raises(RuntimeError, match="read by the kernel"):
        f(key8, value8, kc8, vc8, slots8, "fp8", ks8.cpu(), vs8.cpu())
    pk, pv, pkc, pvc, ps, pks, pvs = _inputs(cuda_device, "paged", "auto")
    with pytest.raises(RuntimeError, match="contiguous"):
        ops.reshape_and_cache(pk, pv, pkc.transpose(1, 2).contiguous().transpose(1, 2), pvc, ps, "auto", pks, pvs)


def test_cuda_graph_capture_and_replay(cuda_device):
    """No allocation, no host sync, scales read on the device: the op can be captured."""
    key, value, kc, vc, slots, ks, vs = _inputs(cuda_device, "flash", "fp8", T=128, nb=64)
    want_k, want_v = kc.clone(), vc.clone()
    ops.reshape_and_cache_flash(key, value, want_k, want_v, slots, "fp8", ks, vs)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(s):
        with torch.cuda.graph(g, stream=s):
            ops.reshape_and_cache_flash(key, value, kc, vc, slots, "fp8", ks, vs)
    torch.cuda.current_stream().wait_stream(s)
    g.replay()
    torch.cuda.synchronize()
    assert H.same_bytes(kc, want_k) and H.same_bytes(vc, want_v)
    # new data in the same buffers, replay again
    key.copy_(torch.randn_like(key.float()).to(key.dtype))
    ops.reshape_and_cache_flash(key, value, want_k, want_v, slots, "fp8", ks, vs)
    g.replay()
    torch.cuda.synchronize()
    assert H.same_bytes(kc, want_k)


def test_runs_on_the_current_stream(cuda_device):
    key, value, kc, vc, slots, ks, vs = _inputs(cuda_device, "flash", "auto", T=4096, Hh=8, D=128, bs=16, nb=512)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        big = torch.randn(64 << 20, device=cuda_device)  # keeps `side` busy before the op
        big.mul_(2.0)
        ops.reshape_and_cache_flash(key, value, kc, vc, slots, "auto", ks, vs)
        ev = torch.cuda.Event()
        ev.record(side)
    ev.synchronize()  # waiting for `side` alone must be enough
    flat = kc.reshape(-1, 8, 128)  # copy of the strided view
    assert H.same_bytes(flat[slots], key.contiguous())


def test_device_guard_on_second_gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("one GPU visible")
    dev = torch.device("cuda:1")
    key, value, kc, vc, slots, ks, vs = _inputs(dev, "flash", "auto")
    torch.cuda.set_device(0)  # ambient device differs from the tensors' device
    ops.reshape_and_cache_flash(key, value, kc, vc, slots, "auto", ks, vs)
    torch.cuda.synchronize(dev)
    assert H.same_bytes(kc.reshape(-1, 8, 64)[slots], key.contiguous())


def test_debug_slot_validation_is_opt_in(cuda_device):
    """KVC_DEBUG_SLOTS=1 makes the torch layer count out-of-range slots on the device and raise BEFORE
    the scatter is launched (nothing is ever written through a bad slot); off by default."""
    import os
    import subprocess
    import sys
    from tests.conftest import PKG_ROOT, REPO
    code = r'''
import sys, torch
sys.path[:0] = [%r, %r]
from vllm_xpu_kernels import ops
dev = torch.device("cuda:0")
key = torch.randn(8, 2, 64, device=dev).to(torch.bfloat16); value = torch.randn_like(key)
kc = torch.zeros(4, 16, 2, 64, dtype=torch.bfloat16, device=dev); vc = torch.zeros_like(kc)
one = torch.ones(1, device=dev)
good = torch.tensor([0, 5, -1, 63, 17, 2, 9, 33], device=dev)
ops.reshape_and_cache_flash(key, value, kc, vc, good, "auto", one, one)
bad = good.clone(); bad[3] = 64; bad[6] = 1000
try:
    ops.reshape_and_cache_flash(key, value, kc, vc, bad, "auto", one, one)
except RuntimeError as e:
    assert "2 entries of slot_mapping are >= num_blocks * block_size = 64" in str(e), str(e)
    print("rejected")
torch.cuda.synchronize()
''' % (REPO, PKG_ROOT)
    env = dict(os.environ, KVC_DEBUG_SLOTS="1")
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "rejected" in r.stdout, r.stdout + r.stderr
