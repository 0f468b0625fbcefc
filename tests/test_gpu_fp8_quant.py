"""GPU parity of the fp8 activation-quantisation ops against the CPU oracle (bit-exact: the oracle
restates the kernel arithmetic x * (1/scale)) and against the fixtures made with the reference's torch
recipes (per-tensor exact; per-token within the reference's own 0.5 % byte-mismatch allowance)."""
import numpy as np
import pytest
import torch

import oracle
from oracle.torch_views import ORC_IN, as_np
from tests import helpers as H
from vllm_xpu_kernels import cabi
from vllm_xpu_kernels.fp8_quant import scaled_fp8_quant

pytestmark = pytest.mark.gpu

FP8 = {"fp8_e4m3": torch.float8_e4m3fn, "fp8_e5m2": torch.float8_e5m2}
# the reference's grid (tests/test_fp8_quant.py:115-134 there)
HIDDEN_SIZES = [1, 2, 3, 4, 16, 67, 768, 2048, 5120, 5137, 8192, 8193] + list(range(1024, 1033))


@pytest.mark.parametrize("fname", H.golden_files("quant"))
def test_quant_golden(fname, cuda_device):
    c = H.QuantCase(fname)
    x = c.x.to(cuda_device)
    out, scale = scaled_fp8_quant(x, fp8_dtype=c.fp8_dtype)
    assert float(scale) == c.scale
    assert torch.equal(out.view(torch.uint8).cpu(), c.out_tensor)
    out_s, _ = scaled_fp8_quant(x, scale=torch.tensor([c.scale], device=cuda_device), fp8_dtype=c.fp8_dtype)
    assert torch.equal(out_s.view(torch.uint8).cpu(), c.out_tensor)
    ub = None if c.scale_ub is None else torch.tensor(c.scale_ub, dtype=torch.float32, device=cuda_device)
    out_t, scales = scaled_fp8_quant(x, scale_ub=ub, use_per_token_if_dynamic=True, fp8_dtype=c.fp8_dtype)
    assert torch.equal(scales.cpu(), c.scales)
    assert float((out_t.view(torch.uint8).cpu() != c.out_token).float().mean()) <= 0.005


@pytest.mark.parametrize("dtype", [torch.half, torch.bfloat16, torch.float])
@pytest.mark.parametrize("fp8", ["fp8_e4m3", "fp8_e5m2"])
@pytest.mark.parametrize("hidden_size", HIDDEN_SIZES)
def test_quant_matrix_vs_oracle(dtype, fp8, hidden_size, cuda_device):
    for num_tokens in (1, 7, 83):
        torch.manual_seed(hidden_size * 7 + num_tokens)
        x = (torch.randn(num_tokens, hidden_size) * 3).to(dtype)
        xn, name = as_np(x), ORC_IN[dtype]
        dx = x.to(cuda_device)
        # dynamic per tensor (through the torch op wrapper) and static with that scale (through the C ABI)
        out, scale = scaled_fp8_quant(dx, fp8_dtype=FP8[fp8])
        want_scale = oracle.absmax_scale(xn, name, fp8)
        assert float(scale) == float(want_scale)
        want = torch.from_numpy(oracle.static_scaled_fp8_quant(xn, float(want_scale), name, fp8))
        assert torch.equal(out.view(torch.uint8).cpu(), want), (num_tokens, "dynamic")
        out2 = torch.empty_like(out)
        cabi.static_scaled_fp8_quant(out2, dx, scale)
        assert torch.equal(out2.view(torch.uint8).cpu(), want), (num_tokens, "static")
        # per token, with and without an upper bound
        for ub in (None, float(x.float().abs().mean())):
            dub = None if ub is None else torch.tensor(ub, dtype=torch.float32, device=cuda_device)
            out_t, scales = scaled_fp8_quant(dx, scale_ub=dub, use_per_token_if_dynamic=True, fp8_dtype=FP8[fp8])
            want_t, want_s = oracle.per_token_fp8_quant(xn, name, fp8, ub)
            assert np.array_equal(scales.cpu().numpy(), want_s), (num_tokens, ub)
            assert torch.equal(out_t.view(torch.uint8).cpu(), torch.from_numpy(want_t)), (num_tokens, ub)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float])
def test_quant_many_tokens_and_special_values(dtype, cuda_device):
    torch.manual_seed(1)
    x = (torch.randn(4096, 1031) * 10).to(dtype)
    x[5, 7] = float("inf")
    x[9, 0] = float("-inf")
    x[11, 3] = float("nan")
    x[100] = 0.0  # an all-zero row: scale falls back to the minimum scaling factor
    dx = x.to(cuda_device)
    for fp8 in ("fp8_e4m3", "fp8_e5m2"):
        out_t, scales = scaled_fp8_quant(dx, use_per_token_if_dynamic=True, fp8_dtype=FP8[fp8])
        want_t, want_s = oracle.per_token_fp8_quant(as_np(x), ORC_IN[dtype], fp8)
        assert np.array_equal(scales.cpu().numpy(), want_s)
        assert torch.equal(out_t.view(torch.uint8).cpu(), torch.from_numpy(want_t))
        s = torch.tensor([0.37], device=cuda_device)
        out_s, _ = scaled_fp8_quant(dx, scale=s, fp8_dtype=FP8[fp8])
        want = torch.from_numpy(oracle.static_scaled_fp8_quant(as_np(x), 0.37, ORC_IN[dtype], fp8))
        assert torch.equal(out_s.view(torch.uint8).cpu(), want)


def test_quant_large_index(cuda_device):
    """More elements than an int32 can index (the reference's regression case, tests/test_fp8_quant.py:207-233
    there, is 1 024 000 x 1152); checked on a sample of rows and on the final rows."""
    T, hidden = 1_024_000, 2112  # 2.16e9 elements
    x = torch.rand(T, hidden, dtype=torch.bfloat16, device=cuda_device)
    scale = torch.tensor([1.0 / 448.0], device=cuda_device)
    out, _ = scaled_fp8_quant(x, scale=scale, fp8_dtype=torch.float8_e4m3fn)
    rows = [0, 1, 12345, T // 2, T - 2, T - 1]
    want = oracle.static_scaled_fp8_quant(as_np(x[rows].cpu()), 1.0 / 448.0, "bf16", "fp8_e4m3")
    assert torch.equal(out[rows].view(torch.uint8).cpu(), torch.from_numpy(want))


def test_quant_opcheck_and_errors(cuda_device):
    x = torch.rand(7, 67, dtype=torch.half, device=cuda_device)
    out = torch.empty(7, 67, dtype=torch.float8_e4m3fn, device=cuda_device)
    scale = torch.tensor([0.01], device=cuda_device)
    H.opcheck(torch.ops._C.static_scaled_fp8_quant, (out, x, scale))
    H.opcheck(torch.ops._C.dynamic_scaled_fp8_quant, (out, x, torch.zeros(1, device=cuda_device)))
    H.opcheck(torch.ops._C.dynamic_per_token_scaled_fp8_quant, (out, x, torch.zeros(7, 1, device=cuda_device), None))
    with pytest.raises(RuntimeError, match="float8"):
        torch.ops._C.static_scaled_fp8_quant(torch.empty(7, 67, dtype=torch.int8, device=cuda_device), x, scale)
    with pytest.raises(RuntimeError, match="contiguous"):
        torch.ops._C.static_scaled_fp8_quant(out, x.t().contiguous().t(), scale)
    with pytest.raises(RuntimeError, match="Unsupported input type"):
        torch.ops._C.static_scaled_fp8_quant(out, x.double(), scale)
    with pytest.raises(RuntimeError, match="scale must be"):
        torch.ops._C.dynamic_per_token_scaled_fp8_quant(out, x, torch.zeros(3, 1, device=cuda_device), None)
