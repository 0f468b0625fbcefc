#!/usr/bin/env python
"""A small, self-ending run of one KV-cache write kernel, meant to be wrapped by a profiler.

    python profile_case.py --layout flash --kv fp8 --tokens 32768 --launches 6

Holds well under a few GB on the device (inputs of two rotating batches plus a cache just
large enough for them), yet each batch is larger than the 126 MB L2 so DRAM counters mean
something.  Prints the mean launch time measured with CUDA events, which is only meaningful
when the script is NOT running under a profiler.
"""
from __future__ import annotations

import argparse
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

import torch  # noqa: E402

from vllm_xpu_kernels import cabi  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layout", choices=["flash", "paged", "mla", "gather", "quant-static", "quant-dynamic", "quant-token",
                                         "rope", "rope-cache", "rope-then-cache", "decode", "prefill"], default="flash",
                    help="mla: concat_and_cache_mla (512 + 64 wide entries); gather: gather_cache of such entries; "
                         "rope: rotary_embedding; rope-cache: the fused rotary_embedding_and_cache_flash; "
                         "rope-then-cache: the two separate ops back to back (what the fused op replaces)")
    ap.add_argument("--seqs", type=int, default=64, help="decode: sequences in the batch (one query token each)")
    ap.add_argument("--seq-len", type=int, default=4096, help="decode: cached tokens per sequence")
    ap.add_argument("--q-heads", type=int, default=64, help="query heads of the rope layouts (--heads are kv heads)")
    ap.add_argument("--rot-dim", type=int, default=0, help="rotary dim of the rope layouts (0: head size)")
    ap.add_argument("--gptj", action="store_true", help="interleaved pairs instead of the NeoX halves")
    ap.add_argument("--no-write-back", action="store_true", help="rope-cache: leave key un-rotated")
    ap.add_argument("--kv", choices=["auto", "fp8", "fp8_e5m2"], default="fp8")
    ap.add_argument("--dtype", choices=["bfloat16", "half", "float"], default="bfloat16")
    ap.add_argument("--tokens", type=int, default=32768)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--head-size", type=int, default=128)
    ap.add_argument("--block-size", type=int, default=64)
    ap.add_argument("--slots", choices=["runs", "random"], default="runs",
                    help="runs: whole blocks in random order (a prefill); random: distinct random slots")
    ap.add_argument("--skip-frac", type=float, default=0.0, help="fraction of slots set to -1")
    ap.add_argument("--strided", action="store_true", help="key/value are slices of a fused qkv tensor")
    ap.add_argument("--launches", type=int, default=6)
    ap.add_argument("--nbuf", type=int, default=2)
    ns = ap.parse_args()

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    torch.manual_seed(0)
    if ns.layout in ("mla", "gather"):
        run_mla_or_gather(ns, dev)
        return
    if ns.layout.startswith("quant"):
        run_quant(ns, dev)
        return
    if ns.layout.startswith("rope"):
        run_rope(ns, dev)
        return
    if ns.layout == "decode":
        run_decode(ns, dev)
        return
    if ns.layout == "prefill":
        run_prefill(ns, dev)
        return
    dt = {"bfloat16": torch.bfloat16, "half": torch.float16, "float": torch.float32}[ns.dtype]
    T, H, D, bs = ns.tokens, ns.heads, ns.head_size, ns.block_size
    nb = 2 * ((T + bs - 1) // bs)
    es_out = 1 if ns.kv != "auto" else torch.empty((), dtype=dt).element_size()
    cdt = dt if ns.kv == "auto" else torch.uint8
    if ns.layout == "flash":
        kc = torch.zeros(nb, bs, H, D, dtype=cdt, device=dev)
        vc = torch.zeros(nb, bs, H, D, dtype=cdt, device=dev)
    else:
        x = 16 // es_out
        kc = torch.zeros(nb, H, D // x, bs, x, dtype=cdt, device=dev)
        vc = torch.zeros(nb, H, D, bs, dtype=cdt, device=dev)
    sets = []
    for b in range(ns.nbuf):
        if ns.strided:
            qkv = torch.randn(T, 3 * H * D, device=dev).to(dt)
            key = qkv[:, H * D:2 * H * D].view(T, H, D)
            value = qkv[:, 2 * H * D:].view(T, H, D)
        else:
            key = torch.randn(T, H, D, device=dev).to(dt)
            value = torch.randn(T, H, D, device=dev).to(dt)
        if ns.slots == "runs":
            perm = torch.randperm(nb, device=dev)[:(T + bs - 1) // bs]
            slots = (perm[:, None] * bs + torch.arange(bs, device=dev)[None, :]).flatten()[:T].contiguous()
        else:
            slots = torch.randperm(nb * bs, device=dev)[:T]
        if ns.skip_frac > 0:
            slots[torch.rand(T, device=dev) < ns.skip_frac] = -1
        sets.append((key, value, slots))
    ks = torch.tensor(0.02, device=dev)
    vs = torch.tensor(0.02, device=dev)
    fn = cabi.reshape_and_cache_flash if ns.layout == "flash" else cabi.reshape_and_cache
    active = int((sets[0][2] >= 0).sum())
    es_in = torch.empty((), dtype=dt).element_size()
    alg_bytes = 8 * T + active * H * D * 2 * (es_in + es_out)

    evs = []
    for i in range(ns.launches):
        key, value, slots = sets[i % ns.nbuf]
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn(key, value, kc, vc, slots, ns.kv, ks, vs)
        b.record()
        evs.append((a, b))
    torch.cuda.synchronize()
    times = [a.elapsed_time(b) * 1e3 for a, b in evs]
    best = min(times[1:]) if len(times) > 1 else times[0]
    print(f"layout={ns.layout} kv={ns.kv} dtype={ns.dtype} T={T} H={H} D={D} bs={bs} slots={ns.slots} "
          f"algorithmic_bytes={alg_bytes} launches={ns.launches} event_us={['%.1f' % t for t in times]} "
          f"best_GBps={alg_bytes / best / 1e3:.0f}")


def run_mla_or_gather(ns, dev) -> None:
    dt = {"bfloat16": torch.bfloat16, "half": torch.float16, "float": torch.float32}[ns.dtype]
    T, bs, R, P = ns.tokens, ns.block_size, 512, 64
    nb = 2 * ((T + bs - 1) // bs)
    es_in = torch.empty((), dtype=dt).element_size()
    es_out = 1 if ns.kv != "auto" else es_in
    cache = torch.zeros(nb, bs, R + P, dtype=dt if ns.kv == "auto" else torch.uint8, device=dev)
    scale = torch.tensor(0.02, device=dev)
    sets = []
    for b in range(ns.nbuf):
        perm = torch.randperm(nb, device=dev)[:(T + bs - 1) // bs]
        if ns.layout == "mla":
            kv_c = torch.randn(T, R, device=dev).to(dt)
            k_pe = torch.randn(T, P, device=dev).to(dt)
            slots = (perm[:, None] * bs + torch.arange(bs, device=dev)[None, :]).flatten()[:T].contiguous()
            if ns.slots == "random":
                slots = torch.randperm(nb * bs, device=dev)[:T]
            sets.append((kv_c, k_pe, slots))
        else:
            batch = 64
            per = T // batch
            cu = torch.arange(batch + 1, device=dev, dtype=torch.int32) * per
            table = perm[:batch * ((per + bs - 1) // bs)].view(batch, -1).to(torch.int32).contiguous()
            dst = torch.zeros(batch * per, R + P, dtype=cache.dtype, device=dev)
            sets.append((dst, table, cu, batch))
    if ns.layout == "gather":
        cache.view(torch.uint8).random_(0, 120)
    alg = T * (R + P) * (es_in + es_out) + 8 * T if ns.layout == "mla" else 2 * sets[0][0].numel() * es_out
    evs = []
    for i in range(ns.launches):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        if ns.layout == "mla":
            kv_c, k_pe, slots = sets[i % ns.nbuf]
            cabi.concat_and_cache_mla(kv_c, k_pe, cache, slots, ns.kv, scale)
        else:
            dst, table, cu, batch = sets[i % ns.nbuf]
            cabi.gather_cache(cache, dst, table, cu, batch)
        b.record()
        evs.append((a, b))
    torch.cuda.synchronize()
    times = [a.elapsed_time(b) * 1e3 for a, b in evs]
    best = min(times[1:]) if len(times) > 1 else times[0]
    print(f"layout={ns.layout} kv={ns.kv} dtype={ns.dtype} T={T} entry=576 bs={bs} algorithmic_bytes={alg} "
          f"launches={ns.launches} event_us={['%.1f' % t for t in times]} best_GBps={alg / best / 1e3:.0f}")


def run_quant(ns, dev) -> None:
    """fp8 activation quantisation of a [tokens, heads * head_size] activation."""
    dt = {"bfloat16": torch.bfloat16, "half": torch.float16, "float": torch.float32}[ns.dtype]
    T, hidden = ns.tokens, ns.heads * ns.head_size
    f8 = torch.float8_e5m2 if ns.kv == "fp8_e5m2" else torch.float8_e4m3fn
    xs = [torch.randn(T, hidden, device=dev).to(dt) for _ in range(ns.nbuf)]
    out = torch.empty(T, hidden, dtype=f8, device=dev)
    scale = torch.tensor([0.02], device=dev)
    scales = torch.zeros(T, 1, device=dev)
    es = xs[0].element_size()
    n = T * hidden
    alg = {"quant-static": n * (es + 1), "quant-dynamic": n * (2 * es + 1), "quant-token": n * (es + 1) + 4 * T}[ns.layout]
    evs = []
    for i in range(ns.launches):
        x = xs[i % ns.nbuf]
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if ns.layout == "quant-dynamic":
            scale.zero_()
        a.record()
        if ns.layout == "quant-static":
            cabi.static_scaled_fp8_quant(out, x, scale)
        elif ns.layout == "quant-dynamic":
            cabi.dynamic_scaled_fp8_quant(out, x, scale)
        else:
            cabi.dynamic_per_token_scaled_fp8_quant(out, x, scales)
        b.record()
        evs.append((a, b))
    torch.cuda.synchronize()
    times = [a.elapsed_time(b) * 1e3 for a, b in evs]
    best = min(times[1:]) if len(times) > 1 else times[0]
    print(f"layout={ns.layout} fp8={ns.kv} dtype={ns.dtype} T={T} hidden={hidden} algorithmic_bytes={alg} "
          f"launches={ns.launches} event_us={['%.1f' % t for t in times]} best_GBps={alg / best / 1e3:.0f}")


def run_rope(ns, dev) -> None:
    """Rotary embedding of a fused qkv projection output [T, (Hq + 2 Hkv) * D], alone, fused with the cache
    write, or followed by the separate cache write."""
    dt = {"bfloat16": torch.bfloat16, "half": torch.float16, "float": torch.float32}[ns.dtype]
    T, hq, hk, D, bs = ns.tokens, ns.q_heads, ns.heads, ns.head_size, ns.block_size
    R = ns.rot_dim or D
    neox = not ns.gptj
    es = torch.empty((), dtype=dt).element_size()
    es_out = 1 if ns.kv != "auto" else es
    max_pos = 8192
    inv_freq = 1.0 / (10000.0 ** (torch.arange(0, R, 2, dtype=torch.float) / R))
    freqs = torch.einsum("i,j -> ij", torch.arange(max_pos, dtype=torch.float), inv_freq)
    table = torch.cat((freqs.cos(), freqs.sin()), dim=-1).to(dt).to(dev)
    nb = 2 * ((T + bs - 1) // bs)
    cdt = dt if ns.kv == "auto" else torch.uint8
    with_cache = ns.layout != "rope"
    if with_cache:
        kc = torch.zeros(nb, bs, hk, D, dtype=cdt, device=dev)
        vc = torch.zeros(nb, bs, hk, D, dtype=cdt, device=dev)
    sets = []
    for b in range(ns.nbuf):
        qkv = torch.randn(T, (hq + 2 * hk) * D, device=dev).to(dt)
        q = qkv[:, :hq * D].view(T, hq, D)
        k = qkv[:, hq * D:(hq + hk) * D].view(T, hk, D)
        v = qkv[:, (hq + hk) * D:].view(T, hk, D)
        positions = torch.arange(T, device=dev) % max_pos
        perm = torch.randperm(nb, device=dev)[:(T + bs - 1) // bs]
        slots = (perm[:, None] * bs + torch.arange(bs, device=dev)[None, :]).flatten()[:T].contiguous()
        sets.append((positions, q, k, v, slots))
    ks = torch.tensor(0.05, device=dev)
    vs = torch.tensor(0.05, device=dev)
    rope_bytes = 2 * T * (hq + hk) * R * es + T * R * es + 8 * T
    if with_cache:
        wb = 0 if (ns.layout == "rope-cache" and ns.no_write_back) else T * hk * R * es
        alg = (2 * T * hq * R * es + T * R * es + 16 * T + T * hk * D * es + wb + T * hk * D * es_out
               + T * hk * D * (es + es_out))
    else:
        alg = rope_bytes
    evs = []
    for i in range(ns.launches):
        positions, q, k, v, slots = sets[i % ns.nbuf]
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        if ns.layout == "rope":
            cabi.rotary_embedding(positions, q, k, D, table, neox)
        elif ns.layout == "rope-cache":
            cabi.rotary_embedding_and_cache_flash(positions, q, k, v, D, table, neox, kc, vc, slots, ns.kv, ks, vs,
                                                  write_back_key=not ns.no_write_back)
        else:
            cabi.rotary_embedding(positions, q, k, D, table, neox)
            cabi.reshape_and_cache_flash(k, v, kc, vc, slots, ns.kv, ks, vs)
        b.record()
        evs.append((a, b))
    torch.cuda.synchronize()
    times = [a.elapsed_time(b) * 1e3 for a, b in evs]
    best = min(times[1:]) if len(times) > 1 else times[0]
    print(f"layout={ns.layout} kv={ns.kv} dtype={ns.dtype} T={T} Hq={hq} Hkv={hk} D={D} rot_dim={R} "
          f"style={'neox' if neox else 'gptj'} algorithmic_bytes={alg} launches={ns.launches} "
          f"event_us={['%.1f' % t for t in times]} best_GBps={alg / best / 1e3:.0f}")


def run_decode(ns, dev) -> None:
    """Paged decode attention: --seqs sequences of --seq-len cached tokens, --q-heads query heads over --heads kv
    heads.  Every launch streams the whole cache (larger than L2 at the default size), so one buffer set is enough."""
    dt = {"bfloat16": torch.bfloat16, "half": torch.float16}[ns.dtype]
    S, L, hq, hk, D, bs = ns.seqs, ns.seq_len, ns.q_heads, ns.heads, ns.head_size, ns.block_size
    blocks_per_seq = (L + bs - 1) // bs
    nb = S * blocks_per_seq
    es = 2 if ns.kv == "auto" else 1
    if ns.kv == "auto":
        kc = torch.randn(nb, bs, hk, D, device=dev).to(dt)
        vc = torch.randn(nb, bs, hk, D, device=dev).to(dt)
    else:
        kc = torch.randint(0, 120, (nb, bs, hk, D), device=dev, dtype=torch.uint8)
        vc = torch.randint(0, 120, (nb, bs, hk, D), device=dev, dtype=torch.uint8)
    table = torch.randperm(nb, device=dev).view(S, blocks_per_seq).to(torch.int32)
    lens = torch.full((S,), L, dtype=torch.int32, device=dev)
    query = torch.randn(S, hq, D, device=dev).to(dt)
    out = torch.empty_like(query)
    ds = torch.tensor(0.05, device=dev)
    alg = 2 * S * L * hk * D * es + 2 * S * hq * D * 2 + 4 * S * blocks_per_seq + 4 * S
    evs = []
    for i in range(ns.launches):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        cabi.paged_decode_attention(query, kc, vc, table, lens, D ** -0.5, L, ns.kv, ds, ds, out=out)
        b.record()
        evs.append((a, b))
    torch.cuda.synchronize()
    times = [a.elapsed_time(b) * 1e3 for a, b in evs]
    best = min(times[1:]) if len(times) > 1 else times[0]
    print(f"layout=decode kv={ns.kv} dtype={ns.dtype} seqs={S} seq_len={L} Hq={hq} Hkv={hk} D={D} bs={bs} "
          f"algorithmic_bytes={alg} launches={ns.launches} event_us={['%.1f' % t for t in times]} "
          f"best_GBps={alg / best / 1e3:.0f}")


def run_prefill(ns, dev) -> None:
    """Causal attention of whole prompts over their own paged keys/values: --seqs prompts of --seq-len tokens
    (query length = cached length).  Compute-bound: reports TFLOP/s of the 4 * L^2 / 2 * Hq * D useful flops."""
    dt = {"bfloat16": torch.bfloat16, "half": torch.float16}[ns.dtype]
    S, L, hq, hk, D, bs = ns.seqs, ns.seq_len, ns.q_heads, ns.heads, ns.head_size, ns.block_size
    blocks_per_seq = (L + bs - 1) // bs
    nb = S * blocks_per_seq
    if ns.kv == "auto":
        kc = torch.randn(nb, bs, hk, D, device=dev).to(dt)
        vc = torch.randn(nb, bs, hk, D, device=dev).to(dt)
    else:
        kc = torch.randint(0, 120, (nb, bs, hk, D), device=dev, dtype=torch.uint8)
        vc = torch.randint(0, 120, (nb, bs, hk, D), device=dev, dtype=torch.uint8)
    table = torch.randperm(nb, device=dev).view(S, blocks_per_seq).to(torch.int32)
    lens = torch.full((S,), L, dtype=torch.int32, device=dev)
    cu = (torch.arange(S + 1, device=dev, dtype=torch.int32) * L)
    query = torch.randn(S * L, hq, D, device=dev).to(dt)
    out = torch.empty_like(query)
    ds = torch.tensor(0.05, device=dev)
    flops = 4.0 * S * (L * (L + 1) / 2) * hq * D
    evs = []
    for i in range(ns.launches):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        cabi.paged_attention(query, kc, vc, table, lens, cu, L, D ** -0.5, L, True, ns.kv, ds, ds, out=out)
        b.record()
        evs.append((a, b))
    torch.cuda.synchronize()
    times = [a.elapsed_time(b) * 1e3 for a, b in evs]
    best = min(times[1:]) if len(times) > 1 else times[0]
    print(f"layout=prefill kv={ns.kv} dtype={ns.dtype} seqs={S} seq_len={L} Hq={hq} Hkv={hk} D={D} bs={bs} "
          f"useful_flops={flops:.3e} launches={ns.launches} event_us={['%.1f' % t for t in times]} "
          f"best_TFLOPs={flops / best / 1e6:.1f}")


if __name__ == "__main__":
    main()
