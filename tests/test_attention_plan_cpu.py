"""The launch planner of the paged attention (pure host code, runs without a GPU): a windowed call never needs
more workspace than the window-less size query reports, and its splits always cover every tile a CTA of the
decode kernel has to walk, for every sequence length of a tile period."""
import json
import os
import subprocess
import sys

import pytest

from tests.conftest import PKG_ROOT

SCRIPT = r"""
import json, sys
sys.path.insert(0, sys.argv[1])
import torch
from vllm_xpu_kernels import cabi
L = cabi.lib()
bad = []
count = 0
for kv in ("auto", "fp8"):
    for D in (64, 128, 256):
        for (S, hq, hk) in ((1, 64, 8), (4, 64, 8), (32, 8, 8), (3, 16, 2), (256, 64, 8), (1, 8, 1)):
            for max_len in (300, 1153, 4096, 8192, 16000, 65536):
                for q in (1, 2, 4, 16):
                    if q * (hq // hk) > 16:
                        continue
                    ws = L.kvc_paged_attention_workspace_bytes(S, S * q, q, hq, hk, D, max_len, 2, cabi.parse_kv_cache_dtype(kv))
                    for window in ((63, 0), (127, 127), (1023, -1), (1024, -1), (4095, -1), (4096, 0), (8000, 100)):
                        for causal in (True, False):
                            p = cabi.paged_attention_plan(S, S * q, q, hq, hk, D, max_len, causal, window,
                                                          torch.bfloat16, kv)
                            count += 1
                            if p["workspace_bytes"] > ws:
                                bad.append(("workspace", kv, D, S, hq, hk, max_len, q, window, causal, p, ws))
                            # tiles a CTA may have to walk: its first row's start to its last row's end
                            closed = window[0] >= 0 and (causal or window[1] >= 0)
                            if not closed:
                                continue
                            TN, g = p["tile_tokens"], hq // hk
                            tokens_in_cta = min(q, 16)
                            right = 0 if causal else window[1]
                            for n in range(max(q, max_len - 2 * TN), max_len + 1):
                                pos0, pos1 = n - q, n - q + tokens_in_cta - 1
                                lo = max(0, pos0 - window[0])
                                hi = min(n, pos1 + right + 1)
                                need = (hi + TN - 1) // TN - lo // TN
                                if need > p["splits"] * p["tiles_per_split"]:
                                    bad.append(("tiles", kv, D, S, hq, hk, max_len, q, window, causal, n, need, p))
                                    break
print(json.dumps({"checked": count, "bad": bad[:5], "n_bad": len(bad)}))
"""


@pytest.mark.parametrize("slots", [148, 444, 592])
def test_windowed_plan_fits_the_size_query_and_covers_its_tiles(slots):
    """KVC_TEST_DECODE_SLOTS stands in for the device's size (CTAs it holds at once: 148 SMs x 1, 3 or 4), which
    the cost model depends on and which no GPU is here to tell."""
    env = dict(os.environ, KVC_TEST_DECODE_SLOTS=str(slots))
    r = subprocess.run([sys.executable, "-c", SCRIPT, PKG_ROOT], capture_output=True, text=True, timeout=900, env=env)
    assert r.returncode == 0, r.stderr[-2000:]
    d = json.loads(r.stdout.strip().splitlines()[-1])
    assert d["checked"] > 5000
    assert d["n_bad"] == 0, d["bad"]


def test_plan_cases_that_used_to_disagree():
    """One sequence x 8 kv heads, 8192 cached tokens, window 4096 on 444 or 592 CTA slots: planning on the
    window alone asks for 66 splits where the size query allowed for 64."""
    script = (
        "import sys; sys.path.insert(0, sys.argv[1]); import torch\n"
        "from vllm_xpu_kernels import cabi\n"
        "ws = cabi.lib().kvc_paged_attention_workspace_bytes(1, 1, 1, 64, 8, 128, 8192, 2, 0)\n"
        "p = cabi.paged_attention_plan(1, 1, 1, 64, 8, 128, 8192, True, (4096, -1))\n"
        "q = cabi.paged_attention_plan(1, 1, 1, 64, 8, 128, 8192, True, (-1, -1))\n"
        "assert q['workspace_bytes'] == ws, (q, ws)\n"
        "assert p['workspace_bytes'] <= ws and p['splits'] <= q['splits'], (p, q, ws)\n"
        "assert p['splits'] * p['tiles_per_split'] * p['tile_tokens'] >= 4097, p\n")
    for slots in (444, 592):
        env = dict(os.environ, KVC_TEST_DECODE_SLOTS=str(slots))
        r = subprocess.run([sys.executable, "-c", script, PKG_ROOT], capture_output=True, text=True, timeout=300, env=env)
        assert r.returncode == 0, r.stderr[-2000:]
