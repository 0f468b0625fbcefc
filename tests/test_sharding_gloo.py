"""The multi-rank plumbing on CPU (gloo, world_size 2): head sharding needs no exchange, the
shard caches concatenate to the unsharded cache, and the benchmark's max/sum-over-ranks
reductions behave.  The compute here is the CPU oracle (the checker), never the product path."""
import os
import socket
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests import helpers as H


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str) -> None:
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for p in (here, os.path.join(here, "vllm-xpu-kernels_b200", "benchmark")):
        if p not in sys.path:
            sys.path.insert(0, p)
    import bench
    import workloads
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        w = workloads.c4(num_tokens=256, num_blocks=16)
        mine = workloads.shard_heads(w, rank, world)
        assert mine.num_heads == w.num_heads // world and mine.num_tokens == w.num_tokens
        ksh, _ = mine.cache_shapes()
        kc = torch.zeros(ksh, dtype=torch.uint8)
        vc = torch.zeros(ksh, dtype=torch.uint8)
        H.oracle_call("flash", mine.key, mine.value, kc, vc, mine.slot_mapping, mine.kv_cache_dtype,
                      float(mine.k_scale), float(mine.v_scale))
        # no data-path collective: results only meet on rank 0 for the check
        gathered_k = [torch.empty_like(kc) for _ in range(world)] if rank == 0 else None
        gathered_v = [torch.empty_like(vc) for _ in range(world)] if rank == 0 else None
        dist.gather(kc, gathered_k, dst=0)
        dist.gather(vc, gathered_v, dst=0)
        # the benchmark's reductions
        t_max = bench.max_over_ranks(dist, 1.0 + rank, device="cpu")
        t_sum = bench.sum_over_ranks(dist, float(mine.num_tokens), device="cpu")
        assert t_max == float(world) and t_sum == float(world * w.num_tokens)
        if rank == 0:
            fk = torch.zeros(w.cache_shapes()[0], dtype=torch.uint8)
            fv = torch.zeros_like(fk)
            H.oracle_call("flash", w.key, w.value, fk, fv, w.slot_mapping, w.kv_cache_dtype, float(w.k_scale),
                          float(w.v_scale))
            assert torch.equal(torch.cat(gathered_k, dim=2), fk)
            assert torch.equal(torch.cat(gathered_v, dim=2), fv)
            open(os.path.join(out_dir, "ok"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_two_ranks_head_sharding(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert (tmp_path / "ok").read_text() == "ok"


def test_shard_heads_rejects_uneven_split():
    import pytest
    import workloads
    w = workloads.c1()
    with pytest.raises(ValueError):
        workloads.shard_heads(w, 0, 3)
    parts = [workloads.shard_heads(w, r, 4) for r in range(4)]
    assert torch.equal(torch.cat([p.key for p in parts], dim=1), w.key)
    assert all(p.slot_mapping is w.slot_mapping for p in parts)


def _failing_worker(rank: int, world: int, port: int, out_dir: str) -> None:
    """Rank 1 leaves between steps (no collective in flight); rank 0's next reduction must end with an
    error within the process-group timeout instead of hanging."""
    import datetime
    import time
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    if here not in sys.path:
        sys.path.insert(0, here)
    import bench
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    assert bench.max_over_ranks(dist, float(rank), device="cpu") == 1.0  # one healthy step first
    if rank == 1:
        os._exit(0)  # the rank disappears without a goodbye
    time.sleep(1.0)
    t0 = time.monotonic()
    try:
        bench.max_over_ranks(dist, 5.0, device="cpu")
        outcome = "no error"
    except Exception as e:  # noqa: BLE001  (gloo reports a closed connection or a timeout)
        outcome = "detected: " + type(e).__name__
    took = time.monotonic() - t0
    with open(os.path.join(out_dir, "outcome"), "w") as f:
        f.write(f"{outcome} after {took:.1f}s")
    os._exit(0)  # skip the process-group teardown, which would wait for the missing rank


def test_missing_rank_is_detected_not_waited_for(tmp_path):
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_failing_worker, args=(r, 2, port, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=60)
    assert all(not p.is_alive() for p in procs), "a rank hung"
    text = (tmp_path / "outcome").read_text()
    assert text.startswith("detected"), text
    assert float(text.rsplit("after ", 1)[1][:-1]) < 30.0
