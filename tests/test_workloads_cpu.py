"""The five measured configurations are generated as specified: shapes, dtypes, strides, slot
patterns, scales, and the algorithmic byte counts used for every bandwidth figure."""
import torch

import workloads


def test_shapes_and_algorithmic_bytes():
    w = workloads.c1()
    assert (w.num_tokens, w.num_heads, w.head_size, w.block_size, w.num_blocks) == (83, 8, 128, 16, 1024)
    assert w.key.dtype == torch.bfloat16 and w.kv_cache_dtype == "auto" and w.layout == "flash"
    assert w.algorithmic_bytes() == 680_600
    w = workloads.c2()
    assert (w.num_tokens, w.num_heads, w.head_size, w.block_size, w.num_blocks) == (4096, 8, 128, 64, 8192)
    assert w.cache_dtype == torch.float8_e4m3fn and w.algorithmic_bytes() == 25_198_592
    w = workloads.c3()
    assert w.layout == "paged" and w.key.dtype == torch.float16
    assert w.cache_shapes() == ((4096, 32, 16, 16, 8), (4096, 32, 128, 16))
    assert w.algorithmic_bytes() == 67_125_248


def test_distinct_slots_and_scales():
    for w in (workloads.c1(), workloads.c2(), workloads.c3()):
        s = w.slot_mapping
        assert s.dtype == torch.int64 and s.unique().numel() == s.numel()
        assert 0 <= int(s.min()) and int(s.max()) < w.num_blocks * w.block_size
    w = workloads.c2()
    # scale = amax(|x|)/448: the largest scaled magnitude is 448, nothing saturates
    assert abs(float((w.key.float() / w.k_scale).abs().max()) - 448.0) < 1e-3
    assert abs(float((w.value.float() / w.v_scale).abs().max()) - 448.0) < 1e-3


def test_c4_is_runs_of_64_in_permuted_blocks():
    w = workloads.c4()
    assert (w.num_tokens, w.num_heads, w.head_size, w.block_size, w.num_blocks) == (16384, 8, 128, 64, 65536)
    assert w.algorithmic_bytes() == 100_794_368
    s = w.slot_mapping.view(-1, 64)
    assert bool((s % 64 == torch.arange(64)).all())               # whole runs, offsets 0..63
    blocks = s[:, 0] // 64
    assert blocks.unique().numel() == 256 and not bool((blocks[1:] > blocks[:-1]).all())  # distinct, not sorted
    assert 1.9 < float(w.key.float().std()) < 2.1                   # "N(0,2)" read as standard deviation 2
    # different variants use different blocks and data, same shape
    w2 = workloads.c4(variant=1)
    assert not torch.equal(w2.slot_mapping, w.slot_mapping) and not torch.equal(w2.key, w.key)


def test_c5_strided_views_and_padding():
    for kv, nbytes in (("auto", 67_174_400), ("fp8_e4m3", 50_397_184)):
        w = workloads.c5(kv)
        assert (w.num_tokens, w.num_heads, w.head_size, w.block_size, w.num_blocks) == (8192, 32, 64, 16, 32768)
        assert w.key.stride() == (6144, 64, 1) and w.value.stride() == (6144, 64, 1)
        assert w.key.data_ptr() + 2048 * 2 == w.value.data_ptr()   # slices of one fused qkv tensor
        assert w.num_active == 4096 and int((w.slot_mapping == -1).sum()) == 4096
        act = w.slot_mapping[w.slot_mapping >= 0]
        assert act.unique().numel() == 4096
        assert w.algorithmic_bytes() == nbytes


def test_head_shards_partition_the_batch():
    w = workloads.c4(num_tokens=128, num_blocks=8)
    for world in (1, 2, 4, 8):
        parts = [workloads.shard_heads(w, r, world) for r in range(world)]
        assert sum(p.num_heads for p in parts) == 8
        assert sum(p.algorithmic_bytes() - 8 * p.num_tokens for p in parts) == w.algorithmic_bytes() - 8 * w.num_tokens
