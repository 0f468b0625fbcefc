"""GPU parity of the paged decode attention against the fixtures computed with the reference's
``ref_paged_attn`` and against the CPU oracle.

Floating point.  Tolerance: atol = rtol = 1e-2, the reference test's own for this op
(tests/flash_attn/test_flash_attn_varlen_func.py:386 there), against both the fixtures (which carry the
reference statement's 16-bit roundings) and the oracle (which keeps everything in double)."""
import pytest
import torch

from oracle import torch_views
from tests import helpers as H
from vllm_xpu_kernels import cabi
from vllm_xpu_kernels.flash_attn_interface import flash_attn_varlen_func

pytestmark = pytest.mark.gpu

TOL = dict(atol=H.ATTN_ATOL, rtol=H.ATTN_RTOL)


def dscalar(v, dev):
    return torch.tensor(v, dtype=torch.float32, device=dev)


def run_gpu(dev, query, key_cache, value_cache, block_tables, kv_lens, scale, kv="auto", k_descale=1.0, v_descale=1.0,
            sink=None, max_seq_len=None, caches_on_device=None):
    kc, vc = caches_on_device if caches_on_device is not None else (key_cache.to(dev), value_cache.to(dev))
    out = cabi.paged_decode_attention(
        query.to(dev), kc, vc, block_tables.to(dev), kv_lens.to(dev), scale,
        int(kv_lens.max()) if max_seq_len is None else max_seq_len, kv,
        dscalar(k_descale, dev) if kv != "auto" else None, dscalar(v_descale, dev) if kv != "auto" else None,
        None if sink is None else sink.to(dev))
    torch.cuda.synchronize()
    return out.cpu()


# ------------------------------------------------------------------------------------ fixtures
@pytest.mark.parametrize("fname", H.golden_files("decode_attn"))
def test_decode_attention_golden(fname, cuda_device):
    c = H.DecodeAttnCase(fname)
    got = run_gpu(cuda_device, c.query, c.key_cache, c.value_cache, c.block_tables, c.kv_lens, c.scale,
                  c.kv_cache_dtype, c.descale, c.descale, c.sink)
    assert got.dtype == c.dtype
    torch.testing.assert_close(got.float(), c.expected.float(), **TOL)
    want = torch_views.run_paged_decode_attention(c.query, c.key_cache, c.value_cache, c.block_tables, c.kv_lens,
                                                  c.scale, c.kv_cache_dtype, c.descale, c.descale, c.sink)
    torch.testing.assert_close(got.float(), want, **TOL)


# ------------------------------------------------------------------------------------ the reference's decode matrix
def make_case(dtype, hq, hk, D, kv_lens, bs, nb, sink, seed, kv="auto", descale=1.0):
    torch.manual_seed(seed)
    S = len(kv_lens)
    query = torch.randn(S, hq, D).to(dtype)
    key_cache = torch.randn(nb, bs, hk, D).to(dtype)
    value_cache = torch.randn(nb, bs, hk, D).to(dtype)
    max_blocks = (max(max(kv_lens), 1) + bs - 1) // bs
    block_tables = torch.randint(0, nb, (S, max_blocks), dtype=torch.int32)
    lens = torch.tensor(kv_lens, dtype=torch.int32)
    sk = torch.randn(hq).to(dtype) if sink else None
    if kv != "auto":
        fdt = torch.float8_e5m2 if kv == "fp8_e5m2" else torch.float8_e4m3fn
        key_cache = (key_cache.float() / descale).to(fdt)
        value_cache = (value_cache.float() / descale).to(fdt)
    return query, key_cache, value_cache, block_tables, lens, sk


@pytest.mark.parametrize("seq_lens", [[1025], [523, 37, 2011], [13000], [523, 37, 2011, 5000]])
@pytest.mark.parametrize("num_heads", [(4, 4), (8, 2), (10, 2), (16, 1)])
@pytest.mark.parametrize("head_size", [64, 128, 192, 256])
def test_decode_attention_reference_matrix(seq_lens, num_heads, head_size, cuda_device):
    """Shapes of test_decode_with_paged_kv of the reference (tests/flash_attn/test_flash_attn_varlen_func.py:
    274-288): block size 64, 2048 blocks; type and sink alternate over the matrix instead of multiplying it."""
    hq, hk = num_heads
    idx = len(seq_lens) + hq + head_size // 64
    dtype = torch.bfloat16 if idx % 2 else torch.float16
    sink = bool((idx // 2) % 2)
    query, kc, vc, bt, lens, sk = make_case(dtype, hq, hk, head_size, seq_lens, 64, 2048, sink, seed=42)
    scale = head_size ** -0.5
    got = run_gpu(cuda_device, query, kc, vc, bt, lens, scale, sink=sk)
    want = torch_views.run_paged_decode_attention(query, kc, vc, bt, lens, scale, sink=sk)
    torch.testing.assert_close(got.float(), want, **TOL)


def test_decode_attention_block_indices_beyond_32_bits(cuda_device):
    """32768 blocks of 64 x 4 heads x 128 (the reference's large NUM_BLOCKS): byte offsets pass 2^32."""
    dev = cuda_device
    torch.manual_seed(1)
    nb, bs, hk, hq, D = 32768, 64, 4, 8, 128
    kc = torch.randn(nb, bs, hk, D, device=dev, dtype=torch.float16)
    vc = torch.randn(nb, bs, hk, D, device=dev, dtype=torch.float16)
    lens = torch.tensor([700, 64, 1], dtype=torch.int32)
    bt = torch.randint(nb - 40, nb, (3, 11), dtype=torch.int32)
    query = torch.randn(3, hq, D).to(torch.float16)
    got = run_gpu(dev, query, None, None, bt, lens, D ** -0.5, caches_on_device=(kc, vc))
    # the oracle sees a compact copy: the blocks the tables name, renumbered
    used, inv = torch.unique(bt, return_inverse=True)
    small_k, small_v = kc[used.to(dev).long()].cpu(), vc[used.to(dev).long()].cpu()
    want = torch_views.run_paged_decode_attention(query, small_k, small_v, inv.to(torch.int32), lens, D ** -0.5)
    torch.testing.assert_close(got.float(), want, **TOL)


# ------------------------------------------------------------------------------------ fp8 caches
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("kv,descale", [("fp8", 0.03), ("fp8_e4m3", 1.0), ("fp8_e5m2", 0.002)])
@pytest.mark.parametrize("geom", [(8, 2, 128, [300, 37, 1290], 16), (4, 4, 64, [65, 1], 64), (16, 1, 256, [777], 32),
                                  (10, 2, 192, [130, 4000], 128)])
def test_decode_attention_fp8_cache(dtype, kv, descale, geom, cuda_device):
    hq, hk, D, lens, bs = geom
    nb = 96
    query, kc, vc, bt, lens_t, sk = make_case(dtype, hq, hk, D, lens, bs, nb, True, seed=7, kv=kv, descale=descale)
    scale = D ** -0.5
    got = run_gpu(cuda_device, query, kc.view(torch.uint8), vc.view(torch.uint8), bt, lens_t, scale, kv, descale,
                  descale * 0.5, sk)
    want = torch_views.run_paged_decode_attention(query, kc, vc, bt, lens_t, scale, kv, descale, descale * 0.5, sk)
    torch.testing.assert_close(got.float(), want, **TOL)


# ------------------------------------------------------------------------------------ edges
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_decode_attention_edge_lengths_and_layouts(dtype, cuda_device):
    """Lengths around the 64-token tile and the block size, an empty sequence, a block size that is not a power
    of two, 32 query heads per kv head (two row tiles), caches that are the [:, 0] / [:, 1] views of one
    allocation, and a query cut out of a wider projection output."""
    dev = cuda_device
    torch.manual_seed(3)
    hq, hk, D, bs, nb = 32, 1, 128, 48, 40
    lens = [0, 1, 47, 48, 49, 63, 64, 65, 127, 128, 129, 400]
    S = len(lens)
    both = torch.randn(nb, 2, bs, hk, D).to(dtype)
    wide = torch.randn(S, hq * D + 256).to(dtype)
    query = wide[:, 128:128 + hq * D].view(S, hq, D)
    bt = torch.randint(0, nb, (S, 9), dtype=torch.int32)
    lens_t = torch.tensor(lens, dtype=torch.int32)
    sk = torch.randn(hq).to(dtype)
    d_both = both.to(dev)
    d_query = wide.to(dev)[:, 128:128 + hq * D].view(S, hq, D)
    out = cabi.paged_decode_attention(d_query, d_both[:, 0], d_both[:, 1], bt.to(dev), lens_t.to(dev), 0.11, 400,
                                      sink=sk.to(dev))
    torch.cuda.synchronize()
    want = torch_views.run_paged_decode_attention(query, both[:, 0], both[:, 1], bt, lens_t, 0.11, sink=sk)
    torch.testing.assert_close(out.cpu().float(), want, **TOL)
    assert torch.count_nonzero(out[0]) == 0  # the empty sequence
    # no sink: an empty sequence still gives zeros, not NaN
    out2 = cabi.paged_decode_attention(d_query, d_both[:, 0], d_both[:, 1], bt.to(dev), lens_t.to(dev), 0.11, 400)
    want2 = torch_views.run_paged_decode_attention(query, both[:, 0], both[:, 1], bt, lens_t, 0.11)
    torch.testing.assert_close(out2.cpu().float(), want2, **TOL)


def test_decode_attention_split_count_does_not_change_the_result(cuda_device):
    """max_seq_len only sizes the split: a larger bound gives more, shorter splits of the same sums."""
    query, kc, vc, bt, lens, sk = make_case(torch.bfloat16, 8, 2, 128, [3000, 200], 64, 128, True, seed=11)
    a = run_gpu(cuda_device, query, kc, vc, bt, lens, 0.09, sink=sk, max_seq_len=3000)
    b = run_gpu(cuda_device, query, kc, vc, bt, lens, 0.09, sink=sk, max_seq_len=60000)
    want = torch_views.run_paged_decode_attention(query, kc, vc, bt, lens, 0.09, sink=sk)
    torch.testing.assert_close(a.float(), want, **TOL)
    torch.testing.assert_close(b.float(), want, **TOL)
    # many sequences: enough CTAs without splitting
    query, kc, vc, bt, lens, sk = make_case(torch.float16, 8, 8, 64, [100 + 7 * i for i in range(300)], 16, 512, False,
                                            seed=12)
    c = run_gpu(cuda_device, query, kc, vc, bt, lens, 0.125)
    want = torch_views.run_paged_decode_attention(query, kc, vc, bt, lens, 0.125)
    torch.testing.assert_close(c.float(), want, **TOL)


def test_decode_attention_head_shards_concatenate(cuda_device):
    """Tensor parallelism: a rank that holds kv heads [k0, k1) and their query heads computes exactly its slice of
    the output; no exchange.  (Tolerance, not bits: the split count depends on how many heads a launch has.)"""
    query, kc, vc, bt, lens, sk = make_case(torch.bfloat16, 16, 4, 128, [1500, 64, 700], 16, 128, True, seed=31)
    whole = run_gpu(cuda_device, query, kc, vc, bt, lens, 0.09, sink=sk)
    for world in (2, 4):
        parts = []
        for rank in range(world):
            k0, k1 = rank * 4 // world, (rank + 1) * 4 // world
            parts.append(run_gpu(cuda_device, query[:, k0 * 4:k1 * 4], kc[:, :, k0:k1], vc[:, :, k0:k1], bt, lens, 0.09,
                                 sink=sk[k0 * 4:k1 * 4].contiguous(), max_seq_len=1500))
        torch.testing.assert_close(torch.cat(parts, dim=1).float(), whole.float(), **TOL)


def test_write_fp8_cache_then_attend(cuda_device):
    """The two halves together: reshape_and_cache_flash stores fp8 keys and values with k_scale / v_scale, the
    decode attention reads them back with the same scales as descales.  Checked against the oracle's own
    write followed by its attention, and against attention over the unquantised rows within fp8's error."""
    dev = cuda_device
    torch.manual_seed(5)
    hq, hk, D, bs, nb = 8, 2, 128, 16, 64
    lens = [333, 90]
    S = len(lens)
    bt = torch.randperm(nb)[:S * 21].view(S, 21).to(torch.int32)  # no block belongs to two sequences
    keys = [torch.randn(n, hk, D).to(torch.bfloat16) for n in lens]
    values = [torch.randn(n, hk, D).to(torch.bfloat16) for n in lens]
    slots = torch.cat([bt[s, torch.arange(n) // bs].long() * bs + torch.arange(n) % bs for s, n in enumerate(lens)])
    key, value = torch.cat(keys), torch.cat(values)
    k_scale = float(key.float().abs().max() / 448)
    v_scale = float(value.float().abs().max() / 448)
    cache = torch.zeros(nb, 2, bs, hk, D, dtype=torch.uint8)
    d_cache = cache.to(dev)
    cabi.reshape_and_cache_flash(key.to(dev), value.to(dev), d_cache[:, 0], d_cache[:, 1], slots.to(dev), "fp8",
                                 dscalar(k_scale, dev), dscalar(v_scale, dev))
    query = torch.randn(S, hq, D).to(torch.bfloat16)
    lens_t = torch.tensor(lens, dtype=torch.int32)
    out = cabi.paged_decode_attention(query.to(dev), d_cache[:, 0], d_cache[:, 1], bt.to(dev), lens_t.to(dev),
                                      D ** -0.5, max(lens), "fp8", dscalar(k_scale, dev), dscalar(v_scale, dev))
    torch.cuda.synchronize()
    H.oracle_call("flash", key, value, cache[:, 0], cache[:, 1], slots, "fp8", k_scale, v_scale)
    assert H.same_bytes(d_cache.cpu(), cache)
    want = torch_views.run_paged_decode_attention(query, cache[:, 0], cache[:, 1], bt, lens_t, D ** -0.5, "fp8",
                                                  k_scale, v_scale)
    torch.testing.assert_close(out.cpu().float(), want, **TOL)
    # against the unquantised rows: fp8 storage costs a few percent
    dense = torch.zeros(nb, 2, bs, hk, D, dtype=torch.bfloat16)
    H.oracle_call("flash", key, value, dense[:, 0], dense[:, 1], slots, "auto", 1.0, 1.0)
    ideal = torch_views.run_paged_decode_attention(query, dense[:, 0], dense[:, 1], bt, lens_t, D ** -0.5)
    torch.testing.assert_close(out.cpu().float(), ideal, atol=0.15, rtol=0.15)


def test_decode_attention_rejects_bad_arguments(cuda_device):
    dev = cuda_device
    q = torch.zeros(2, 8, 128, dtype=torch.float16, device=dev)
    kc = torch.zeros(4, 16, 2, 128, dtype=torch.float16, device=dev)
    bt = torch.zeros(2, 4, dtype=torch.int32, device=dev)
    lens = torch.ones(2, dtype=torch.int32, device=dev)
    with pytest.raises(RuntimeError, match="head_size"):
        cabi.paged_decode_attention(q[..., :96].contiguous(), kc[..., :96].contiguous(), kc[..., :96].contiguous(), bt,
                                    lens, 1.0, 1)
    with pytest.raises(RuntimeError, match="multiple of num_kv_heads"):
        cabi.paged_decode_attention(q[:, :7].contiguous(), kc, kc, bt, lens, 1.0, 1)
    with pytest.raises(RuntimeError, match="fp16 or bf16"):
        cabi.paged_decode_attention(q.float(), kc, kc, bt, lens, 1.0, 1)
    with pytest.raises(RuntimeError, match="Unsupported data type of kv cache"):
        cabi.paged_decode_attention(q, kc, kc, bt, lens, 1.0, 1, "int8")
    out = cabi.paged_decode_attention(q[:0], kc, kc, bt[:0], lens[:0], 1.0, 0)  # no sequences: nothing to do
    assert out.shape[0] == 0


# ------------------------------------------------------------------------------------ the reference-facing call
@pytest.mark.parametrize("fname", H.golden_files("decode_attn"))
def test_flash_attn_varlen_func_on_the_fixtures(fname, cuda_device):
    """The call of the reference's test (tests/flash_attn/test_flash_attn_varlen_func.py:355-366 there), through
    this package's flash_attn_varlen_func; fp8 fixtures add the descales."""
    dev = cuda_device
    c = H.DecodeAttnCase(fname)
    S = c.query.shape[0]
    cu_q = torch.arange(S + 1, dtype=torch.int32, device=dev)
    kw = {}
    if c.kv_cache_dtype != "auto":
        kw = dict(k_descale=dscalar(c.descale, dev).expand(S, c.key_cache.shape[2]),
                  v_descale=dscalar(c.descale, dev).expand(S, c.key_cache.shape[2]))
    out = flash_attn_varlen_func(c.query.to(dev), c.key_cache.to(dev), c.value_cache.to(dev), 1, cu_q,
                                 int(c.kv_lens.max()), seqused_k=c.kv_lens.to(dev), softmax_scale=c.scale,
                                 causal=False, block_table=c.block_tables.to(dev), window_size=(-1, -1),
                                 s_aux=None if c.sink is None else c.sink.to(dev), **kw)
    torch.cuda.synchronize()
    torch.testing.assert_close(out.cpu().float(), c.expected.float(), **TOL)


def test_attention_ops_pass_opcheck_and_refuse_what_is_not_built(cuda_device):
    dev = cuda_device
    query, kc, vc, bt, lens, sk = make_case(torch.float16, 8, 2, 64, [70, 200, 5], 16, 32, True, seed=21)
    q, kc, vc, bt, lens, sk = (x.to(dev) for x in (query, kc, vc, bt, lens, sk))
    cu_q = torch.arange(4, dtype=torch.int32, device=dev)
    args = (q, kc, vc, None, cu_q, torch.empty_like(cu_q), lens, None, bt, None, 1, 200, 0.0, 0.125, sk, False, False,
            -1, -1, 0.0, False, None)
    # the reference's schema pairs a mutable optional `out` with a Tensor[] return, which torch's AOT
    # functionalisation refuses for any custom op; the other three checks apply
    H.opcheck(torch.ops._vllm_fa2_C.varlen_fwd, args,
              test_utils=("test_schema", "test_autograd_registration", "test_faketensor"))
    k8 = (kc.float() / 0.05).to(torch.float8_e4m3fn)
    v8 = (vc.float() / 0.05).to(torch.float8_e4m3fn)
    out = torch.empty_like(q)
    H.opcheck(torch.ops._vllm_fa2_C.paged_decode_attention,
              (q, k8, v8, out, lens, bt, 200, 0.125, sk, "fp8", dscalar(0.05, dev), dscalar(0.05, dev)))
    torch.ops._vllm_fa2_C.paged_decode_attention(q, k8, v8, out, lens, bt, 200, 0.125, sk, "fp8", dscalar(0.05, dev),
                                                 dscalar(0.05, dev))  # opcheck works on copies
    want = torch_views.run_paged_decode_attention(query, k8.cpu(), v8.cpu(), bt.cpu(), lens.cpu(), 0.125, "fp8", 0.05,
                                                  0.05, sk.cpu())
    torch.testing.assert_close(out.cpu().float(), want, **TOL)
    # uint8 view of the same cache, named explicitly
    out2 = flash_attn_varlen_func(q, k8.view(torch.uint8), v8.view(torch.uint8), 1, cu_q, 200, seqused_k=lens,
                                  softmax_scale=0.125, block_table=bt, s_aux=sk, k_descale=dscalar(0.05, dev),
                                  v_descale=dscalar(0.05, dev), kv_cache_dtype="fp8_e4m3")
    assert H.same_bytes(out2.cpu(), out.cpu())
    # a larger bound on the query length changes nothing for one-token sequences
    out3 = flash_attn_varlen_func(q, kc, vc, 2, cu_q, 200, seqused_k=lens, softmax_scale=0.125, block_table=bt,
                                  causal=True)
    out4 = flash_attn_varlen_func(q, kc, vc, 1, cu_q, 200, seqused_k=lens, softmax_scale=0.125, block_table=bt)
    torch.testing.assert_close(out3.float(), out4.float(), **TOL)
    # what is not built is refused, loudly
    with pytest.raises(RuntimeError, match="softcap"):
        flash_attn_varlen_func(q, kc, vc, 1, cu_q, 200, seqused_k=lens, softmax_scale=0.125, block_table=bt,
                               softcap=30.0)
    with pytest.raises(RuntimeError, match="page_table must have dtype torch.int32"):
        flash_attn_varlen_func(q, kc, vc, 1, cu_q, 200, seqused_k=lens, softmax_scale=0.125, block_table=bt.long())
    with pytest.raises(RuntimeError, match="only supports fp16 and bf16"):
        flash_attn_varlen_func(q.float(), kc.float(), vc.float(), 1, cu_q, 200, seqused_k=lens, softmax_scale=0.125,
                               block_table=bt)


def test_decode_attention_in_a_cuda_graph(cuda_device):
    dev = cuda_device
    query, kc, vc, bt, lens, sk = make_case(torch.bfloat16, 8, 2, 128, [900, 40], 16, 64, False, seed=23)
    q, kc, vc, bt, lens = (x.to(dev) for x in (query, kc, vc, bt, lens))
    cu_q = torch.arange(3, dtype=torch.int32, device=dev)
    call = lambda: flash_attn_varlen_func(q, kc, vc, 1, cu_q, 900, seqused_k=lens, softmax_scale=0.09, block_table=bt)
    eager = call()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        captured = call()
    captured.zero_()
    g.replay()
    torch.cuda.synchronize()
    assert H.same_bytes(captured.cpu(), eager.cpu())
    want = torch_views.run_paged_decode_attention(query, kc.cpu(), vc.cpu(), bt.cpu(), lens.cpu(), 0.09)
    torch.testing.assert_close(captured.cpu().float(), want, **TOL)


# ------------------------------------------------------------------------------------ several query tokens per sequence
def cu_of(lens):
    return torch.cat([torch.zeros(1, dtype=torch.int32), torch.cumsum(torch.tensor(lens), 0).to(torch.int32)])


@pytest.mark.parametrize("fname", H.golden_files("varlen_attn"))
@pytest.mark.parametrize("face", ["cabi", "interface"])
def test_varlen_attention_golden(fname, face, cuda_device):
    """Fixtures from the reference's ref_paged_attn with query lengths (1, 5, 129), (7, 33, 1), (40, 3)."""
    dev = cuda_device
    c = H.DecodeAttnCase(fname)
    S = c.kv_lens.shape[0]
    ds = dscalar(c.descale, dev)
    if face == "cabi":
        out = cabi.paged_attention(c.query.to(dev), c.key_cache.to(dev), c.value_cache.to(dev), c.block_tables.to(dev),
                                   c.kv_lens.to(dev), c.cu_seqlens_q.to(dev), int(c.query_lens.max()), c.scale,
                                   int(c.kv_lens.max()), c.causal, c.kv_cache_dtype, ds, ds,
                                   None if c.sink is None else c.sink.to(dev))
    else:
        kw = dict(k_descale=ds.expand(S, c.key_cache.shape[2]), v_descale=ds.expand(S, c.key_cache.shape[2])) \
            if c.kv_cache_dtype != "auto" else {}
        out = flash_attn_varlen_func(c.query.to(dev), c.key_cache.to(dev), c.value_cache.to(dev),
                                     int(c.query_lens.max()), c.cu_seqlens_q.to(dev), int(c.kv_lens.max()),
                                     seqused_k=c.kv_lens.to(dev), softmax_scale=c.scale, causal=c.causal,
                                     block_table=c.block_tables.to(dev), window_size=(-1, -1),
                                     s_aux=None if c.sink is None else c.sink.to(dev), **kw)
    torch.cuda.synchronize()
    torch.testing.assert_close(out.cpu().float(), c.expected.float(), **TOL)


@pytest.mark.parametrize("num_heads", [(4, 4), (8, 2), (10, 2), (16, 1)])
@pytest.mark.parametrize("head_size", [64, 128, 192, 256])
@pytest.mark.parametrize("causal", [False, True])
def test_varlen_attention_reference_matrix(num_heads, head_size, causal, cuda_device):
    """The sequence list of the reference's test_varlen_with_paged_kv: (1, 1328), (5, 18), (129, 463), block size
    64, over its head pairs and head sizes, with and without the causal mask; type and sink alternate."""
    dev = cuda_device
    hq, hk = num_heads
    q_lens, kv_lens = [1, 5, 129], [1328, 18, 463]
    idx = hq + head_size // 64 + int(causal)
    dtype = torch.bfloat16 if idx % 2 else torch.float16
    torch.manual_seed(42)
    query = torch.randn(sum(q_lens), hq, head_size).to(dtype)
    _, kc, vc, bt, lens, sk = make_case(dtype, hq, hk, head_size, kv_lens, 64, 2048, bool((idx // 2) % 2), seed=43)
    cu = cu_of(q_lens)
    scale = head_size ** -0.5
    out = cabi.paged_attention(query.to(dev), kc.to(dev), vc.to(dev), bt.to(dev), lens.to(dev), cu.to(dev), 129, scale,
                               1328, causal, sink=None if sk is None else sk.to(dev))
    torch.cuda.synchronize()
    want = torch_views.run_paged_decode_attention(query, kc, vc, bt, lens, scale, sink=sk, cu_seqlens_q=cu,
                                                  causal=causal)
    torch.testing.assert_close(out.cpu().float(), want, **TOL)


@pytest.mark.parametrize("kv,descale", [("auto", 1.0), ("fp8", 0.04), ("fp8_e5m2", 0.002)])
def test_varlen_attention_mixed_batch_and_edges(kv, descale, cuda_device):
    """A batch as a serving step sees it: decodes, a prefill chunk that starts mid-sequence, a whole short
    prompt, a query run longer than its cached sequence (its first tokens see nothing: zeros), an empty
    sequence; 5 query heads per kv head, so rows of different tokens share a 16-row tile."""
    dev = cuda_device
    hq, hk, D, bs, nb = 10, 2, 128, 16, 200
    q_lens = [1, 300, 40, 1, 9, 0, 1]
    kv_lens = [700, 1000, 40, 1, 5, 0, 64]
    dtype = torch.bfloat16
    torch.manual_seed(50)
    query = torch.randn(sum(q_lens), hq, D).to(dtype)
    _, kc, vc, bt, lens, sk = make_case(dtype, hq, hk, D, kv_lens, bs, nb, True, seed=51, kv=kv, descale=descale)
    cu = cu_of(q_lens)
    kcd, vcd = (kc.view(torch.uint8), vc.view(torch.uint8)) if kv != "auto" else (kc, vc)
    out = cabi.paged_attention(query.to(dev), kcd.to(dev), vcd.to(dev), bt.to(dev), lens.to(dev), cu.to(dev), 300, 0.09,
                               1000, True, kv, dscalar(descale, dev), dscalar(descale, dev), sk.to(dev))
    torch.cuda.synchronize()
    want = torch_views.run_paged_decode_attention(query, kc, vc, bt, lens, 0.09, kv, descale, descale, sk, cu, True)
    torch.testing.assert_close(out.cpu().float(), want, **TOL)
    first_of_run5 = int(cu[4])
    assert torch.count_nonzero(out[first_of_run5:first_of_run5 + 4]) == 0  # 9 queries over 5 tokens: 4 see nothing


def test_varlen_attention_long_chunk(cuda_device):
    """A 1024-token chunk over 3072 cached tokens: 64 row tiles x up to 48 token tiles on the many-rows kernel."""
    dev = cuda_device
    hq, hk, D = 8, 1, 128
    torch.manual_seed(60)
    query = torch.randn(1024, hq, D).to(torch.float16)
    _, kc, vc, bt, lens, _ = make_case(torch.float16, hq, hk, D, [3072], 64, 64, False, seed=61)
    cu = cu_of([1024])
    out = cabi.paged_attention(query.to(dev), kc.to(dev), vc.to(dev), bt.to(dev), lens.to(dev), cu.to(dev), 1024,
                               D ** -0.5, 3072, True)
    torch.cuda.synchronize()
    want = torch_views.run_paged_decode_attention(query, kc, vc, bt, lens, D ** -0.5, cu_seqlens_q=cu, causal=True)
    torch.testing.assert_close(out.cpu().float(), want, **TOL)


# ------------------------------------------------------------------------------------ sliding windows, non-paged form
@pytest.mark.parametrize("fname", H.golden_files("window_attn"))
@pytest.mark.parametrize("face", ["cabi", "interface"])
def test_window_and_dense_attention_golden(fname, face, cuda_device):
    """Fixtures from the reference's ref_paged_attn: windows (-1, 127), (127, -1), (127, 127), (63, 0) and the
    non-paged form, which the C ABI takes as a cache of one-token blocks and the interface as cu_seqlens_k."""
    dev = cuda_device
    c = H.DecodeAttnCase(fname)
    sink = None if c.sink is None else c.sink.to(dev)
    if face == "cabi":
        out = cabi.paged_attention(c.query.to(dev), c.key_cache.to(dev), c.value_cache.to(dev), c.block_tables.to(dev),
                                   c.kv_lens.to(dev), c.cu_seqlens_q.to(dev), int(c.query_lens.max()), c.scale,
                                   int(c.kv_lens.max()), c.causal, sink=sink, window=c.window)
    elif c.paged:
        out = flash_attn_varlen_func(c.query.to(dev), c.key_cache.to(dev), c.value_cache.to(dev),
                                     int(c.query_lens.max()), c.cu_seqlens_q.to(dev), int(c.kv_lens.max()),
                                     seqused_k=c.kv_lens.to(dev), softmax_scale=c.scale, causal=c.causal,
                                     block_table=c.block_tables.to(dev), window_size=list(c.window), s_aux=sink)
    else:
        out = flash_attn_varlen_func(c.query.to(dev), c.dense_key.to(dev), c.dense_value.to(dev),
                                     int(c.query_lens.max()), c.cu_seqlens_q.to(dev), int(c.kv_lens.max()),
                                     cu_seqlens_k=c.cu_seqlens_k.to(dev), softmax_scale=c.scale, causal=c.causal,
                                     block_table=None, window_size=list(c.window), s_aux=sink)
    torch.cuda.synchronize()
    torch.testing.assert_close(out.cpu().float(), c.expected.float(), **TOL)


@pytest.mark.parametrize("window", [(-1, 127), (127, -1), (127, 127), (0, 0), (1000, 3)])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("kv", ["auto", "fp8"])
def test_window_attention_vs_oracle(window, causal, kv, cuda_device):
    """The reference's SLIDING_WINDOWS over its sequence list plus long decodes (the window then starts far into
    the sequence: whole tiles and splits are skipped), 16-bit and fp8 caches."""
    dev = cuda_device
    hq, hk, D, bs, nb = 8, 2, 128, 64, 256
    q_lens, kv_lens = [1, 5, 129, 1, 1], [1328, 18, 463, 9000, 130]
    torch.manual_seed(70)
    query = torch.randn(sum(q_lens), hq, D).to(torch.bfloat16)
    ds = 0.04 if kv != "auto" else 1.0  # descales only exist for fp8 caches
    _, kc, vc, bt, lens, sk = make_case(torch.bfloat16, hq, hk, D, kv_lens, bs, nb, True, seed=71, kv=kv, descale=ds)
    cu = cu_of(q_lens)
    kcd, vcd = (kc.view(torch.uint8), vc.view(torch.uint8)) if kv != "auto" else (kc, vc)
    out = cabi.paged_attention(query.to(dev), kcd.to(dev), vcd.to(dev), bt.to(dev), lens.to(dev), cu.to(dev), 129, 0.09,
                               9000, causal, kv, dscalar(ds, dev), dscalar(ds, dev), sk.to(dev), window=window)
    torch.cuda.synchronize()
    want = torch_views.run_paged_decode_attention(query, kc, vc, bt, lens, 0.09, kv, ds, ds, sk, cu, causal, window)
    torch.testing.assert_close(out.cpu().float(), want, **TOL)


def test_window_decode_with_splits(cuda_device):
    """Pure decode (no cu_seqlens_q through the decode entry's kernel path) with a left window on long sequences:
    the split covers the window, not the sequence."""
    dev = cuda_device
    hq, hk, D, bs, nb = 16, 2, 128, 16, 1200
    kv_lens = [16000, 5000, 300, 40]
    torch.manual_seed(72)
    query = torch.randn(4, hq, D).to(torch.float16)
    _, kc, vc, bt, lens, _ = make_case(torch.float16, hq, hk, D, kv_lens, bs, nb, False, seed=73)
    cu = cu_of([1, 1, 1, 1])
    for window in [(2047, -1), (4095, 0), (511, 511)]:
        out = cabi.paged_attention(query.to(dev), kc.to(dev), vc.to(dev), bt.to(dev), lens.to(dev), cu.to(dev), 1, 0.09,
                                   16000, True, window=window)
        torch.cuda.synchronize()
        want = torch_views.run_paged_decode_attention(query, kc, vc, bt, lens, 0.09, cu_seqlens_q=cu, causal=True,
                                                      window=window)
        torch.testing.assert_close(out.cpu().float(), want, **TOL)


def test_windowed_multi_token_decode_over_a_tile_period(cuda_device):
    """Four query tokens per sequence behind a closed left window, one sequence for every length of more than a
    128-token period: a CTA's rows then span window + 4 tokens, which for some lengths touch one tile more than
    the window alone does.  Every row must still see its newest tokens (the plan has to provide that tile); the
    shape is one the planner runs on 128-token tiles."""
    dev = cuda_device
    hq, hk, D, bs, nb = 4, 1, 128, 64, 512
    # a batch size for which the planner takes 128-token tiles on this device (its cost model counts the CTAs
    # the device holds at once); every candidate covers more than a full 128-token period of lengths
    for count in (141, 180, 240, 320, 480):
        kv_lens = list(range(1150, 1150 + count))
        plan = cabi.paged_attention_plan(count, 4 * count, 4, hq, hk, D, max(kv_lens), True, (1023, -1),
                                         torch.bfloat16, "fp8")
        if plan["tile_tokens"] == 128:
            break
    q_lens = [4] * len(kv_lens)
    assert plan["tile_tokens"] == 128, plan
    need = (1024 + 3 + 254) // 128  # tiles that window + 4 tokens can touch
    assert plan["splits"] * plan["tiles_per_split"] >= need, plan
    torch.manual_seed(80)
    query = torch.randn(sum(q_lens), hq, D).to(torch.bfloat16)
    _, kc, vc, bt, lens, _ = make_case(torch.bfloat16, hq, hk, D, kv_lens, bs, nb, False, seed=81, kv="fp8", descale=0.05)
    cu = cu_of(q_lens)
    out = cabi.paged_attention(query.to(dev), kc.view(torch.uint8).to(dev), vc.view(torch.uint8).to(dev), bt.to(dev),
                               lens.to(dev), cu.to(dev), 4, 0.09, max(kv_lens), True, "fp8", dscalar(0.05, dev),
                               dscalar(0.05, dev), window=(1023, -1))
    torch.cuda.synchronize()
    want = torch_views.run_paged_decode_attention(query, kc, vc, bt, lens, 0.09, "fp8", 0.05, 0.05, None, cu, True,
                                                  (1023, -1))
    torch.testing.assert_close(out.cpu().float(), want, **TOL)


@pytest.mark.parametrize("slots_window", [(4096, -1), (1024, -1), (63, 0)])
def test_windowed_decode_needs_no_more_workspace_than_the_size_query(slots_window, cuda_device):
    """A windowed split decode with exactly the workspace kvc_paged_attention_workspace_bytes reports (which
    knows no window) must be accepted and right, whatever the window does to the planner's choice."""
    dev = cuda_device
    hq, hk, D, bs, nb = 64, 8, 128, 64, 256
    kv_lens = [8192]
    torch.manual_seed(82)
    query, kc, vc, bt, lens, _ = make_case(torch.bfloat16, hq, hk, D, kv_lens, bs, nb, False, seed=83)
    cu = cu_of([1])
    out = cabi.paged_attention(query.to(dev), kc.to(dev), vc.to(dev), bt.to(dev), lens.to(dev), cu.to(dev), 1, 0.09,
                               8192, True, window=slots_window)
    torch.cuda.synchronize()
    want = torch_views.run_paged_decode_attention(query, kc, vc, bt, lens, 0.09, cu_seqlens_q=cu, causal=True,
                                                  window=slots_window)
    torch.testing.assert_close(out.cpu().float(), want, **TOL)
    p = cabi.paged_attention_plan(1, 1, 1, hq, hk, D, 8192, True, slots_window)
    ws = cabi.lib().kvc_paged_attention_workspace_bytes(1, 1, 1, hq, hk, D, 8192, cabi.IN_DTYPE[torch.bfloat16], 0)
    assert p["workspace_bytes"] <= ws


@pytest.mark.parametrize("window", [(0, 0), (-1, 0), (0, -1), (5, 0)])
@pytest.mark.parametrize("causal", [False, True])
def test_torch_op_window_rule_is_the_reference_ops(window, causal, cuda_device):
    """Through flash_attn_varlen_func a window side is open only when it is -1 (csrc/flash_attn/flash_api.cpp:94
    of the reference): (0, 0) keeps the diagonal, (-1, 0) is a causal band without the causal flag."""
    dev = cuda_device
    hq, hk, D, bs, nb = 8, 2, 128, 16, 64
    q_lens, kv_lens = [5, 1, 33], [40, 7, 33]
    torch.manual_seed(84)
    query = torch.randn(sum(q_lens), hq, D).to(torch.float16)
    _, kc, vc, bt, lens, _ = make_case(torch.float16, hq, hk, D, kv_lens, bs, nb, False, seed=85)
    cu = cu_of(q_lens)
    out = flash_attn_varlen_func(query.to(dev), kc.to(dev), vc.to(dev), max(q_lens), cu.to(dev), max(kv_lens),
                                 seqused_k=lens.to(dev), softmax_scale=0.09, causal=causal, block_table=bt.to(dev),
                                 window_size=list(window))
    torch.cuda.synchronize()
    want = torch_views.run_paged_decode_attention(query, kc, vc, bt, lens, 0.09, cu_seqlens_q=cu, causal=causal,
                                                  window=window)
    torch.testing.assert_close(out.cpu().float(), want, **TOL)
