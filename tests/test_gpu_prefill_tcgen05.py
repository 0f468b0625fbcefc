"""GPU parity of the many-rows attention kernel that runs on the tcgen05 tensor cores (head size 128, some
sequence with more than 64 query rows per kv head; 16-bit and fp8 caches) against the CPU oracle, and against the mma.sync
kernel it replaces for those calls.

Floating point.  Tolerance: atol = rtol = 1e-2, the reference test's own for this op
(tests/flash_attn/test_flash_attn_varlen_func.py:386 there).  After every case the kernel's status word must
be 0: no bounded wait gave up."""
import os
import subprocess
import sys

import pytest
import torch

from oracle import torch_views
from tests import helpers as H
from tests.test_gpu_decode_attention import cu_of, make_case
from vllm_xpu_kernels import cabi
from vllm_xpu_kernels.flash_attn_interface import flash_attn_varlen_func

pytestmark = pytest.mark.gpu

TOL = dict(atol=H.ATTN_ATOL, rtol=H.ATTN_RTOL)


def run_case(dev, dtype, hq, hk, q_lens, kv_lens, bs, causal, sink, seed, window=(-1, -1), scale=None, out=None,
             kv="auto", descale=1.0, D=128):
    nb = max(64, sum((n + bs - 1) // bs for n in kv_lens) + 8)
    torch.manual_seed(seed)
    query = torch.randn(sum(q_lens), hq, D).to(dtype)
    _, kc, vc, bt, lens, sk = make_case(dtype, hq, hk, D, kv_lens, bs, nb, sink, seed=seed + 1, kv=kv, descale=descale)
    cu = cu_of(q_lens)
    scale = D ** -0.5 if scale is None else scale
    kcd, vcd = (kc.view(torch.uint8), vc.view(torch.uint8)) if kv != "auto" else (kc, vc)
    ds = torch.tensor(descale, dtype=torch.float32, device=dev) if kv != "auto" else None
    got = cabi.paged_attention(query.to(dev), kcd.to(dev), vcd.to(dev), bt.to(dev), lens.to(dev), cu.to(dev),
                               max(q_lens), scale, max(kv_lens), causal, kv, ds, ds,
                               sink=None if sk is None else sk.to(dev), window=window, out=out)
    assert cabi.paged_attention_device_status() == 0
    want = torch_views.run_paged_decode_attention(query, kc, vc, bt, lens, scale, kv, descale, descale, sink=sk,
                                                  cu_seqlens_q=cu, causal=causal, window=window)
    torch.testing.assert_close(got.cpu().float(), want, **TOL)
    return got


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("kv,descale", [("fp8", 0.04), ("fp8_e5m2", 0.002)])
@pytest.mark.parametrize("bs", [16, 64, 48])
def test_prefill_fp8_caches(dtype, kv, descale, bs, cuda_device):
    """fp8 caches are widened to fp16 on their way into shared memory (exact) and the products run in fp16, for
    bf16 queries too; k_descale folds into the softmax scale, v_descale into the output."""
    run_case(cuda_device, dtype, 8, 2, q_lens=[300, 1, 70, 140], kv_lens=[777, 300, 70, 1100], bs=bs, causal=True,
             sink=(bs == 64), seed=900 + bs, kv=kv, descale=descale)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("heads", [(4, 4), (8, 2), (6, 2), (16, 1)])
@pytest.mark.parametrize("causal", [False, True])
def test_prefill_heads_and_types(dtype, heads, causal, cuda_device):
    """Group sizes 1, 4, 3 (rows of a token do not divide a tile) and 16; ragged query and cache lengths, a
    sequence that is pure decode, one whose rows fill less than a tile, one that spans several row tiles."""
    hq, hk = heads
    run_case(cuda_device, dtype, hq, hk, q_lens=[200, 1, 70, 513], kv_lens=[777, 300, 70, 1500], bs=64, causal=causal,
             sink=(hq == 8), seed=100 + hq)


@pytest.mark.parametrize("bs", [16, 48, 128])
def test_prefill_block_sizes(bs, cuda_device):
    """Blocks shorter and longer than a 64-token tile, and a block size that is no power of two."""
    run_case(cuda_device, torch.bfloat16, 8, 2, q_lens=[333, 129], kv_lens=[1000, 129], bs=bs, causal=True, sink=False,
             seed=200 + bs)


@pytest.mark.parametrize("window", [(-1, 127), (127, -1), (127, 127), (0, 0), (1000, 3)])
@pytest.mark.parametrize("causal", [False, True])
def test_prefill_windows(window, causal, cuda_device):
    """Sliding windows: rows of a tile start and end at different cached tokens, whole tiles are skipped."""
    run_case(cuda_device, torch.float16, 8, 2, q_lens=[400, 90], kv_lens=[2000, 500], bs=32, causal=causal, sink=True,
             seed=300, window=window, scale=0.09)


def test_prefill_query_run_longer_than_the_cache_and_large_scores(cuda_device):
    """More query tokens than cached ones (the first rows see nothing: zeros) and a softmax scale that makes
    the running maximum move often, so that the accumulator is rescaled in tensor memory."""
    got = run_case(cuda_device, torch.bfloat16, 4, 1, q_lens=[300], kv_lens=[200], bs=16, causal=True, sink=False,
                   seed=400, scale=1.5)
    assert torch.count_nonzero(got[:100]) == 0


def test_prefill_output_rows_that_are_not_16_byte_aligned(cuda_device):
    """The output may be a view whose rows start on 4-byte boundaries only (the narrow store path)."""
    dev = cuda_device
    hq, D, T = 8, 128, 150
    buf = torch.zeros(T, hq, D + 2, dtype=torch.bfloat16, device=dev)
    out = buf[:, :, 2:]
    got = run_case(dev, torch.bfloat16, hq, 2, q_lens=[T], kv_lens=[640], bs=64, causal=True, sink=False, seed=500,
                   out=out)
    assert got.data_ptr() == out.data_ptr()
    assert torch.count_nonzero(buf[:, :, :2]) == 0


def test_prefill_long_prompt_multi_tile(cuda_device):
    """A 2048-token prompt from an empty cache, 8 query heads per kv head: 128 row tiles x 32 token tiles."""
    run_case(cuda_device, torch.bfloat16, 8, 1, q_lens=[2048], kv_lens=[2048], bs=64, causal=True, sink=False, seed=600)


def test_prefill_non_paged_form(cuda_device):
    """The interface's dense form (cu_seqlens_k, no block table) reaches the same kernel as a cache of
    one-token blocks."""
    dev = cuda_device
    hq, hk, D = 8, 2, 128
    lens = [257, 130]
    torch.manual_seed(700)
    q = torch.randn(sum(lens), hq, D).to(torch.float16)
    k = torch.randn(sum(lens), hk, D).to(torch.float16)
    v = torch.randn(sum(lens), hk, D).to(torch.float16)
    cu = cu_of(lens)
    out = flash_attn_varlen_func(q.to(dev), k.to(dev), v.to(dev), max(lens), cu.to(dev), max(lens),
                                 cu_seqlens_k=cu.to(dev), softmax_scale=D ** -0.5, causal=True, block_table=None)
    assert cabi.paged_attention_device_status() == 0
    bt = torch.stack([torch.arange(int(cu[i]), int(cu[i]) + max(lens), dtype=torch.int32) for i in range(2)])
    bt = bt.clamp(max=sum(lens) - 1)
    want = torch_views.run_paged_decode_attention(q, k.unsqueeze(1), v.unsqueeze(1), bt,
                                                  torch.tensor(lens, dtype=torch.int32), D ** -0.5, cu_seqlens_q=cu,
                                                  causal=True)
    torch.testing.assert_close(out.cpu().float(), want, **TOL)


def test_prefill_agrees_with_the_mma_sync_kernel(cuda_device):
    """The same call in a child process with KVC_PREFILL_LEGACY=1 (the switch is read once per process)."""
    dev = cuda_device
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = (
        "import sys, torch\n"
        "sys.path[:0] = [%r, %r]\n"
        "from tests.test_gpu_decode_attention import cu_of, make_case\n"
        "from vllm_xpu_kernels import cabi\n"
        "torch.manual_seed(800)\n"
        "q = torch.randn(700, 8, 128).to(torch.bfloat16)\n"
        "_, kc, vc, bt, lens, sk = make_case(torch.bfloat16, 8, 2, 128, [900, 400], 64, 64, True, seed=801)\n"
        "cu = cu_of([500, 200]); dev = 'cuda:0'\n"
        "out = cabi.paged_attention(q.to(dev), kc.to(dev), vc.to(dev), bt.to(dev), lens.to(dev), cu.to(dev), 500, 0.09,"
        " 900, True, sink=sk.to(dev))\n"
        "torch.save(out.cpu(), sys.argv[1])\n") % (repo, os.path.join(repo, "vllm-xpu-kernels_b200"))
    import tempfile
    outs = []
    for legacy in ("0", "1"):
        with tempfile.NamedTemporaryFile(suffix=".pt") as f:
            env = dict(os.environ, KVC_PREFILL_LEGACY=legacy)
            subprocess.run([sys.executable, "-c", code, f.name], check=True, env=env, timeout=300, cwd=repo)
            outs.append(torch.load(f.name))
    assert dev is not None
    torch.testing.assert_close(outs[0].float(), outs[1].float(), **TOL)


def test_a_bounded_wait_that_runs_out(cuda_device):
    """The give-up path of the kernel's bounded mbarrier waits, run on purpose by the library's self-test kernel:
    one CTA allocates tensor memory, waits about a millisecond for an arrival that never comes, gives up, frees
    its tensor memory and raises the status word.  The context stays usable: the word reads 1, clears to 0, and a
    normal call right after is correct."""
    import time
    dev = cuda_device
    assert cabi.paged_attention_device_status() == 0
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    cabi.selftest_bounded_wait_gives_up(50)
    assert cabi.paged_attention_device_status() == 1   # waits for the kernel
    waited = time.perf_counter() - t0
    assert waited < 5.0, f"the bounded wait took {waited:.3f} s"
    cabi.paged_attention_clear_device_status()
    assert cabi.paged_attention_device_status() == 0
    # tensor memory was given back and nothing is stuck: a full-size call right behind it
    run_case(dev, torch.bfloat16, 8, 2, q_lens=[300, 140], kv_lens=[777, 1100], bs=64, causal=True, sink=False, seed=31)
    assert cabi.paged_attention_device_status() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("heads", [(4, 4), (8, 2), (6, 2), (16, 1)])
@pytest.mark.parametrize("bs", [16, 64])
def test_prefill_head_size_64(dtype, heads, bs, cuda_device):
    """Head size 64 over 16-bit caches runs on the paired-tile tcgen05 kernel too (one 64-element operand tile
    per row instead of two): ragged lengths, groups that are and are not powers of two, a window, a sink."""
    hq, hk = heads
    run_case(cuda_device, dtype, hq, hk, q_lens=[200, 1, 70, 513], kv_lens=[777, 300, 70, 1500], bs=bs, causal=True,
             sink=(hq == 8), seed=640 + hq + bs, D=64)
    run_case(cuda_device, dtype, hq, hk, q_lens=[300, 129], kv_lens=[1000, 700], bs=bs, causal=(hq != 4), sink=False,
             seed=650 + hq + bs, window=(127, -1) if hq == 16 else (-1, -1), D=64)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("D", [192, 256])
@pytest.mark.parametrize("heads", [(4, 4), (8, 2), (6, 2), (16, 1)])
@pytest.mark.parametrize("bs", [16, 64, 48])
def test_prefill_head_sizes_192_and_256(dtype, D, heads, bs, cuda_device):
    """Head sizes 192 and 256 over 16-bit caches run on the one-tile tcgen05 kernel (one CTA per SM, all 512
    tensor-memory columns): ragged lengths, groups that are and are not powers of two, block sizes of either
    copy path (48 looks every row up), a window, a sink."""
    hq, hk = heads
    run_case(cuda_device, dtype, hq, hk, q_lens=[200, 1, 70, 513], kv_lens=[777, 300, 70, 1500], bs=bs, causal=True,
             sink=(hq == 8), seed=1920 + D + hq + bs, D=D)
    run_case(cuda_device, dtype, hq, hk, q_lens=[300, 129], kv_lens=[1000, 700], bs=bs, causal=(hq != 4), sink=False,
             seed=2560 + D + hq + bs, window=(127, -1) if hq == 16 else (-1, -1), D=D)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("D", [64, 192, 256])
@pytest.mark.parametrize("kv,descale", [("fp8", 0.04), ("fp8_e5m2", 0.002)])
@pytest.mark.parametrize("bs", [16, 64, 48])
def test_prefill_fp8_caches_other_head_sizes(dtype, D, kv, descale, bs, cuda_device):
    """fp8 rows of 64, 192 and 256 bytes are widened in place like those of 128 (a thread owns a quarter of a row);
    groups of 4 and 3, a sink, a window."""
    run_case(cuda_device, dtype, 8, 2, q_lens=[300, 1, 70, 140], kv_lens=[777, 300, 70, 1100], bs=bs, causal=True,
             sink=(bs == 64), seed=3000 + D + bs, kv=kv, descale=descale, D=D)
    run_case(cuda_device, dtype, 6, 2, q_lens=[150, 260], kv_lens=[400, 900], bs=bs, causal=True, sink=False,
             seed=3100 + D + bs, kv=kv, descale=descale, window=(200, -1), D=D)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("heads", [(8, 2), (6, 2)])
def test_prefill_head_size_64_block_size_that_is_no_tma_box(dtype, heads, cuda_device):
    """Head size 64 with 48-token blocks: the one-tile kernel (two CTAs per SM, 64 accumulator columns)."""
    hq, hk = heads
    run_case(cuda_device, dtype, hq, hk, q_lens=[200, 1, 70, 513], kv_lens=[777, 300, 70, 1500], bs=48, causal=True,
             sink=(hq == 8), seed=6448 + hq, D=64)
    run_case(cuda_device, dtype, hq, hk, q_lens=[300, 129], kv_lens=[1000, 700], bs=48, causal=False, sink=False,
             seed=6449 + hq, D=64)
