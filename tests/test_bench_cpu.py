"""The CPU-only parts of the measurement harness: the reference arm prints one well-formed JSON line,
and every benchmark script at least compiles."""
import json
import os
import py_compile
import subprocess
import sys

from tests.conftest import PKG_ROOT, REPO


def test_reference_arm_prints_one_json_line():
    r = subprocess.run([sys.executable, os.path.join(REPO, "bench.py"), "--impl", "reference", "--steps", "2",
                        "--warmup", "1", "--workload", "C2"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    lines = [ln for ln in r.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["unit"] == "tokens/s" and d["value"] > 0
    assert d["metric"] == "reshape_and_cache_flash_fp8_tokens_per_s" and d["higher_is_better"] is True
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"] == {"value": d["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert d["steps"] == 2 and d["warmup"] == 1 and d["gpu_launches"] == 0


def test_reference_arm_of_the_op_workloads():
    """The ops around the cache write have the same reference arm (CPU oracle, bounded sample per step)."""
    for workload, metric in (("rope", "rotary_embedding_tokens_per_s"), ("gather", "gather_cache_tokens_per_s")):
        r = subprocess.run([sys.executable, os.path.join(REPO, "bench.py"), "--impl", "reference", "--steps", "2",
                            "--warmup", "1", "--workload", workload], capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr
        lines = [ln for ln in r.stdout.splitlines() if ln.strip()]
        assert len(lines) == 1
        d = json.loads(lines[0])
        assert d["impl"] == "reference" and d["metric"] == metric and d["value"] > 0 and d["gpu_launches"] == 0
        assert d["cpu_baseline"]["value"] == d["value"] and d["e2e"]["h2d_bytes_per_step"] == 0


def test_non_zero_ranks_of_the_reference_arm_do_nothing():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    r = subprocess.run([sys.executable, os.path.join(REPO, "bench.py"), "--impl", "reference", "--gpus", "2",
                        "--steps", "2", "--warmup", "1"], capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and r.stdout.strip() == ""


def test_benchmark_scripts_compile():
    bench_dir = os.path.join(PKG_ROOT, "benchmark")
    for fn in sorted(os.listdir(bench_dir)):
        if fn.endswith(".py"):
            py_compile.compile(os.path.join(bench_dir, fn), doraise=True)
    py_compile.compile(os.path.join(REPO, "bench.py"), doraise=True)
    py_compile.compile(os.path.join(REPO, "__graft_entry__.py"), doraise=True)


def test_b200_arm_refuses_to_run_without_a_gpu():
    import torch
    if torch.cuda.is_available():
        return
    r = subprocess.run([sys.executable, os.path.join(REPO, "bench.py"), "--steps", "2", "--warmup", "1"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode != 0 and "no CPU path" in (r.stderr + r.stdout)
