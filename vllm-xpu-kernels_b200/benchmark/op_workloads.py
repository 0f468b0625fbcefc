"""Seeded synthetic workloads for the ops around the KV-cache write: MLA concat, gather, fp8 activation
quantisation, rotary embedding (alone and fused with the cache write) and paged decode attention.

Each workload knows how to build its device buffers, run one step through the C ABI, count the bytes one
step must move, and run the same op on the CPU oracle for a bounded sample, so that ``bench.py --workload
<name>`` reports the same kind of line as for the cache-write configurations.  A "unit" is a token (for
decode attention: a cached token that the step attends over).
"""
from __future__ import annotations

import dataclasses
import time
from typing import Callable

import torch


@dataclasses.dataclass
class OpWorkload:
    name: str
    metric: str
    describe: str
    units_per_step: int            # tokens one step processes
    algorithmic_bytes: int         # bytes one step must move
    launches_per_step: int
    make_steps: Callable           # (device, nbuf) -> (step(i), e2e_step(i), h2d_bytes, d2h_bytes)
    cpu_run: Callable              # (units) -> (run(), units_done, threads)
    arithmetic: str = "f32"
    flops: float = 0.0             # > 0: the step is compute-bound; useful floating-point operations of one step


def _rope_table(max_pos: int, rot_dim: int, dtype: torch.dtype) -> torch.Tensor:
    inv_freq = 1.0 / (10000.0 ** (torch.arange(0, rot_dim, 2, dtype=torch.float) / rot_dim))
    freqs = torch.einsum("i,j -> ij", torch.arange(max_pos, dtype=torch.float), inv_freq)
    return torch.cat((freqs.cos(), freqs.sin()), dim=-1).to(dtype)


def _block_runs(nb: int, bs: int, T: int, device) -> torch.Tensor:
    """Slots of a prefill: whole blocks in random order."""
    perm = torch.randperm(nb, device=device)[:(T + bs - 1) // bs]
    return (perm[:, None] * bs + torch.arange(bs, device=device)[None, :]).flatten()[:T].contiguous()


def _oracle_threads() -> int:
    import oracle
    return oracle.max_threads()


# ---------------------------------------------------------------------------------------------- MLA
def mla(kv: str = "fp8") -> OpWorkload:
    T, R, P, bs = 131072, 512, 64, 64
    es_out = 1 if kv != "auto" else 2

    def make_steps(dev, nbuf):
        from vllm_xpu_kernels import cabi
        torch.manual_seed(10)
        nb = 2 * (T // bs)
        cache = torch.zeros(nb, bs, R + P, dtype=torch.uint8 if kv != "auto" else torch.bfloat16, device=dev)
        scale = torch.tensor(0.02, device=dev)
        sets = [(torch.randn(T, R, device=dev).to(torch.bfloat16), torch.randn(T, P, device=dev).to(torch.bfloat16),
                 _block_runs(nb, bs, T, dev)) for _ in range(nbuf)]
        host = [(a.cpu().pin_memory(), b.cpu().pin_memory(), s.cpu().pin_memory()) for a, b, s in sets[:2]]
        probe = torch.empty(R + P, dtype=cache.dtype).pin_memory()

        def step(i):
            a, b, s = sets[i % nbuf]
            cabi.concat_and_cache_mla(a, b, cache, s, kv, scale)

        def e2e_step(i):
            a, b, s = host[i % 2]
            sd = s.to(dev, non_blocking=True)
            cabi.concat_and_cache_mla(a.to(dev, non_blocking=True), b.to(dev, non_blocking=True), cache, sd, kv, scale)
            probe.copy_(cache.view(nb * bs, R + P)[int(s[-1])], non_blocking=True)

        return step, e2e_step, T * (R + P) * 2 + 8 * T, probe.numel() * probe.element_size()

    def cpu_run(units):
        from oracle import torch_views
        torch.manual_seed(10)
        n = max(bs, units - units % bs)
        a, b = torch.randn(n, R).to(torch.bfloat16), torch.randn(n, P).to(torch.bfloat16)
        nb = n // bs
        cache = torch.zeros(nb, bs, R + P, dtype=torch.uint8 if kv != "auto" else torch.bfloat16)
        cview = cache.view(torch.float8_e4m3fn) if kv != "auto" else cache
        slots = _block_runs(nb, bs, n, "cpu")
        return (lambda: torch_views.run_mla(a, b, cview, slots, kv, 0.02)), n, 1

    return OpWorkload(
        f"mla-{kv}", "concat_and_cache_mla_fp8_tokens_per_s" if kv != "auto" else "concat_and_cache_mla_tokens_per_s",
        f"concat_and_cache_mla bfloat16->{kv}, T={T}, kv_lora_rank={R}, pe_dim={P}, block_size={bs}, whole-block slot runs",
        T, T * (R + P) * (2 + es_out) + 8 * T, 1, make_steps, cpu_run)


# ---------------------------------------------------------------------------------------------- gather
def gather() -> OpWorkload:
    batch, per, bs, E = 64, 2048, 64, 576
    T = batch * per

    def build(device, n_batch):
        nb = 2 * n_batch * (per // bs)
        cache = torch.randn(nb, bs, E, device=device).to(torch.bfloat16)
        perm = torch.randperm(nb, device=device)[:n_batch * (per // bs)]
        table = perm.view(n_batch, -1).to(torch.int32).contiguous()
        cu = (torch.arange(n_batch + 1, device=device, dtype=torch.int32) * per)
        dst = torch.zeros(n_batch * per, E, dtype=torch.bfloat16, device=device)
        return cache, table, cu, dst

    def make_steps(dev, nbuf):
        from vllm_xpu_kernels import cabi
        torch.manual_seed(11)
        cache, _, cu, _ = build(dev, batch)
        nb = cache.shape[0]
        tables = [torch.randperm(nb, device=dev)[:batch * (per // bs)].view(batch, -1).to(torch.int32).contiguous()
                  for _ in range(nbuf)]
        dsts = [torch.zeros(T, E, dtype=torch.bfloat16, device=dev) for _ in range(2)]
        host_tables = [t.cpu().pin_memory() for t in tables[:2]]
        host_cu = cu.cpu().pin_memory()
        out_host = torch.empty(T, E, dtype=torch.bfloat16).pin_memory()

        def step(i):
            cabi.gather_cache(cache, dsts[i % 2], tables[i % nbuf], cu, batch)

        def e2e_step(i):  # tables go up, the gathered rows come back
            t = host_tables[i % 2].to(dev, non_blocking=True)
            c = host_cu.to(dev, non_blocking=True)
            cabi.gather_cache(cache, dsts[i % 2], t, c, batch)
            out_host.copy_(dsts[i % 2], non_blocking=True)

        return step, e2e_step, host_tables[0].numel() * 4 + host_cu.numel() * 4, T * E * 2

    def cpu_run(units):
        from oracle import torch_views
        torch.manual_seed(11)
        n_batch = max(1, min(batch, units // per))
        cache, table, cu, dst = build("cpu", n_batch)
        return (lambda: torch_views.run_gather(cache, dst, table, cu, n_batch)), n_batch * per, 1

    return OpWorkload("gather", "gather_cache_tokens_per_s",
                      f"gather_cache bfloat16 entries of {E}, {batch} sequences x {per} tokens, block_size={bs}",
                      T, 2 * T * E * 2 + T // bs * 4, 1, make_steps, cpu_run, arithmetic="u8")


# ---------------------------------------------------------------------------------------------- fp8 quant
def quant(kind: str) -> OpWorkload:
    T, hidden = 16384, 4096
    n = T * hidden

    def make_steps(dev, nbuf):
        from vllm_xpu_kernels import cabi
        torch.manual_seed(12)
        xs = [torch.randn(T, hidden, device=dev).to(torch.bfloat16) for _ in range(nbuf)]
        out = torch.empty(T, hidden, dtype=torch.float8_e4m3fn, device=dev)
        scale = torch.tensor([0.02], device=dev)
        scales = torch.zeros(T, 1, device=dev)
        host = [x.cpu().pin_memory() for x in xs[:2]]
        probe = torch.empty(hidden, dtype=torch.uint8).pin_memory()

        def run(x):
            if kind == "static":
                cabi.static_scaled_fp8_quant(out, x, scale)
            else:
                cabi.dynamic_per_token_scaled_fp8_quant(out, x, scales)

        def step(i):
            run(xs[i % nbuf])

        def e2e_step(i):
            run(host[i % 2].to(dev, non_blocking=True))
            probe.copy_(out.view(torch.uint8)[T - 1], non_blocking=True)

        return step, e2e_step, n * 2, hidden

    def cpu_run(units):
        import oracle
        torch.manual_seed(12)
        rows = max(1, units)
        x = torch.randn(rows, hidden).to(torch.bfloat16).view(torch.int16).numpy().view("uint16")
        if kind == "static":
            return (lambda: oracle.static_scaled_fp8_quant(x, 0.02, "bf16", "fp8_e4m3")), rows, 1
        return (lambda: oracle.per_token_fp8_quant(x, "bf16", "fp8_e4m3")), rows, 1

    name = "static_scaled_fp8_quant" if kind == "static" else "dynamic_per_token_scaled_fp8_quant"
    return OpWorkload(f"quant-{kind}", f"{name}_tokens_per_s", f"{name} bfloat16->fp8_e4m3, {T} tokens x {hidden}",
                      T, n * 3 + (4 * T if kind != "static" else 0), 1, make_steps, cpu_run)


# ---------------------------------------------------------------------------------------------- rope
def rope(fused: bool) -> OpWorkload:
    T, hq, hk, D, bs, max_pos = 8192, 64, 8, 128, 64, 8192
    rope_bytes = 2 * T * (hq + hk) * D * 2 + T * D * 2 + 8 * T
    fused_bytes = (2 * T * hq * D * 2 + T * D * 2 + 16 * T + T * hk * D * 2 + T * hk * D * 2 + T * hk * D
                   + T * hk * D * (2 + 1))

    def make_steps(dev, nbuf):
        from vllm_xpu_kernels import cabi
        torch.manual_seed(13)
        table = _rope_table(max_pos, D, torch.bfloat16).to(dev)
        nb = 2 * (T // bs)
        cache = torch.zeros(nb, 2, bs, hk, D, dtype=torch.uint8, device=dev) if fused else None
        ks, vs = torch.tensor(0.05, device=dev), torch.tensor(0.05, device=dev)
        sets = []
        for _ in range(nbuf):
            qkv = torch.randn(T, (hq + 2 * hk) * D, device=dev).to(torch.bfloat16)
            sets.append((qkv, torch.arange(T, device=dev) % max_pos, _block_runs(nb, bs, T, dev)))
        split = lambda t: (t[:, :hq * D].view(T, hq, D), t[:, hq * D:(hq + hk) * D].view(T, hk, D),
                           t[:, (hq + hk) * D:].view(T, hk, D))
        host = [(q.cpu().pin_memory(), p.cpu().pin_memory(), s.cpu().pin_memory()) for q, p, s in sets[:2]]
        probe = torch.empty(hq * D, dtype=torch.bfloat16).pin_memory()

        def run(qkv, pos, slots):
            q, k, v = split(qkv)
            if fused:
                cabi.rotary_embedding_and_cache_flash(pos, q, k, v, D, table, True, cache[:, 0], cache[:, 1], slots, "fp8",
                                                      ks, vs)
            else:
                cabi.rotary_embedding(pos, q, k, D, table, True)

        def step(i):
            run(*sets[i % nbuf])

        def e2e_step(i):
            hqkv, hpos, hslots = host[i % 2]
            d = hqkv.to(dev, non_blocking=True)
            run(d, hpos.to(dev, non_blocking=True), hslots.to(dev, non_blocking=True))
            probe.copy_(d[T - 1, :hq * D], non_blocking=True)

        return step, e2e_step, T * (hq + 2 * hk) * D * 2 + 16 * T, probe.numel() * 2

    def cpu_run(units):
        from oracle import torch_views
        torch.manual_seed(13)
        n = max(bs, units - units % bs)
        table = _rope_table(max_pos, D, torch.bfloat16)
        q = torch.randn(n, hq, D).to(torch.bfloat16)
        k = torch.randn(n, hk, D).to(torch.bfloat16)
        v = torch.randn(n, hk, D).to(torch.bfloat16)
        pos = torch.arange(n) % max_pos
        nb = n // bs
        cache = torch.zeros(nb, 2, bs, hk, D, dtype=torch.uint8).view(torch.float8_e4m3fn)
        slots = _block_runs(nb, bs, n, "cpu")

        def run():
            torch_views.run_rope(pos, q, k, D, table, True)
            if fused:
                torch_views.run("flash", k, v, cache[:, 0], cache[:, 1], slots, "fp8", 0.05, 0.05, threads=_oracle_threads())

        return run, n, _oracle_threads()

    if fused:
        return OpWorkload("rope-cache-fp8", "rotary_embedding_and_cache_flash_fp8_tokens_per_s",
                          f"rotary_embedding_and_cache_flash bfloat16->fp8_e4m3, T={T}, {hq} q / {hk} kv heads x {D}, "
                          f"full rotation (NeoX), block_size={bs}", T, fused_bytes, 1, make_steps, cpu_run)
    return OpWorkload("rope", "rotary_embedding_tokens_per_s",
                      f"rotary_embedding bfloat16, T={T}, {hq} q / {hk} kv heads x {D}, full rotation (NeoX)",
                      T, rope_bytes, 1, make_steps, cpu_run)


# ---------------------------------------------------------------------------------------------- decode attention
def decode(kv: str) -> OpWorkload:
    S, L, hq, hk, D, bs = 64, 4096, 64, 8, 128, 64
    es = 2 if kv == "auto" else 1
    blocks_per_seq = L // bs

    def make_steps(dev, nbuf):
        from vllm_xpu_kernels import cabi
        torch.manual_seed(14)
        nb = S * blocks_per_seq
        if kv == "auto":
            kc = torch.randn(nb, bs, hk, D, device=dev).to(torch.bfloat16)
            vc = torch.randn(nb, bs, hk, D, device=dev).to(torch.bfloat16)
        else:
            kc = torch.randint(0, 120, (nb, bs, hk, D), device=dev, dtype=torch.uint8)
            vc = torch.randint(0, 120, (nb, bs, hk, D), device=dev, dtype=torch.uint8)
        tables = [torch.randperm(nb, device=dev).view(S, blocks_per_seq).to(torch.int32) for _ in range(nbuf)]
        lens = torch.full((S,), L, dtype=torch.int32, device=dev)
        queries = [torch.randn(S, hq, D, device=dev).to(torch.bfloat16) for _ in range(nbuf)]
        out = torch.empty(S, hq, D, dtype=torch.bfloat16, device=dev)
        ds = torch.tensor(0.05, device=dev)
        host = [(q.cpu().pin_memory(), t.cpu().pin_memory()) for q, t in zip(queries[:2], tables[:2])]
        host_lens = lens.cpu().pin_memory()
        out_host = torch.empty(S, hq, D, dtype=torch.bfloat16).pin_memory()

        def step(i):
            cabi.paged_decode_attention(queries[i % nbuf], kc, vc, tables[i % nbuf], lens, D ** -0.5, L, kv, ds, ds, out=out)

        def e2e_step(i):  # a decode step's inputs go up (queries, tables, lengths), its output comes back
            hq_, ht = host[i % 2]
            cabi.paged_decode_attention(hq_.to(dev, non_blocking=True), kc, vc, ht.to(dev, non_blocking=True),
                                        host_lens.to(dev, non_blocking=True), D ** -0.5, L, kv, ds, ds, out=out)
            out_host.copy_(out, non_blocking=True)

        return step, e2e_step, S * hq * D * 2 + S * blocks_per_seq * 4 + S * 4, S * hq * D * 2

    def cpu_run(units):
        from oracle import torch_views
        torch.manual_seed(14)
        n_seq = max(1, min(S, units // L))
        nb = n_seq * blocks_per_seq
        if kv == "auto":
            kc, vc = torch.randn(nb, bs, hk, D).to(torch.bfloat16), torch.randn(nb, bs, hk, D).to(torch.bfloat16)
        else:
            kc = torch.randint(0, 120, (nb, bs, hk, D), dtype=torch.uint8).view(torch.float8_e4m3fn)
            vc = torch.randint(0, 120, (nb, bs, hk, D), dtype=torch.uint8).view(torch.float8_e4m3fn)
        table = torch.randperm(nb).view(n_seq, blocks_per_seq).to(torch.int32)
        lens = torch.full((n_seq,), L, dtype=torch.int32)
        q = torch.randn(n_seq, hq, D).to(torch.bfloat16)
        name = "auto" if kv == "auto" else "fp8"
        return (lambda: torch_views.run_paged_decode_attention(q, kc, vc, table, lens, D ** -0.5, name, 0.05, 0.05)), \
            n_seq * L, _oracle_threads()

    tag = "bf16" if kv == "auto" else "fp8"
    return OpWorkload(
        f"decode-{tag}", f"paged_decode_attention_{tag}_cache_kv_tokens_per_s",
        f"paged decode attention, {S} sequences x {L} cached tokens, {hq} q / {hk} kv heads x {D}, "
        f"cache {'bfloat16' if kv == 'auto' else 'fp8_e4m3'}, block_size={bs}",
        S * L, 2 * S * L * hk * D * es + 2 * S * hq * D * 2 + 4 * S * blocks_per_seq + 4 * S, 2, make_steps, cpu_run)


# ---------------------------------------------------------------------------------------------- prefill attention
def prefill(kv: str, S: int = 4, L: int = 2048, D: int = 128) -> OpWorkload:
    """Causal attention of S whole prompts of L tokens over their own paged keys/values (query length = cached
    length): the many-rows path of paged attention.  Compute-bound, unlike everything else here."""
    # 8 kv heads; the q heads shrink with the head size so that a token's query row stays 8192 elements wide
    hq, hk, bs = {64: 64, 128: 64, 192: 48, 256: 32}[D], 8, 64
    es = 2 if kv == "auto" else 1
    blocks_per_seq = L // bs

    def build(device, n_seq):
        nb = n_seq * blocks_per_seq
        if kv == "auto":
            kc = torch.randn(nb, bs, hk, D, device=device).to(torch.bfloat16)
            vc = torch.randn(nb, bs, hk, D, device=device).to(torch.bfloat16)
        else:
            kc = torch.randint(0, 120, (nb, bs, hk, D), device=device, dtype=torch.uint8)
            vc = torch.randint(0, 120, (nb, bs, hk, D), device=device, dtype=torch.uint8)
        table = torch.randperm(nb, device=device).view(n_seq, blocks_per_seq).to(torch.int32)
        lens = torch.full((n_seq,), L, dtype=torch.int32, device=device)
        cu = torch.arange(n_seq + 1, device=device, dtype=torch.int32) * L
        return kc, vc, table, lens, cu

    def make_steps(dev, nbuf):
        from vllm_xpu_kernels import cabi
        torch.manual_seed(15)
        kc, vc, table, lens, cu = build(dev, S)
        queries = [torch.randn(S * L, hq, D, device=dev).to(torch.bfloat16) for _ in range(nbuf)]
        out = torch.empty(S * L, hq, D, dtype=torch.bfloat16, device=dev)
        ds = torch.tensor(0.05, device=dev)
        host = [q.cpu().pin_memory() for q in queries[:2]]
        out_host = torch.empty(S * L, hq, D, dtype=torch.bfloat16).pin_memory()

        def step(i):
            cabi.paged_attention(queries[i % nbuf], kc, vc, table, lens, cu, L, D ** -0.5, L, True, kv, ds, ds, out=out)

        def e2e_step(i):
            cabi.paged_attention(host[i % 2].to(dev, non_blocking=True), kc, vc, table, lens, cu, L, D ** -0.5, L, True,
                                 kv, ds, ds, out=out)
            out_host.copy_(out, non_blocking=True)

        return step, e2e_step, S * L * hq * D * 2, S * L * hq * D * 2

    def cpu_run(units):
        from oracle import torch_views
        torch.manual_seed(15)
        # the oracle is quadratic in the prompt length: a short prompt of the same head geometry
        n = max(16, min(256, units))
        nb = (n + bs - 1) // bs
        kc = torch.randn(nb, bs, hk, D).to(torch.bfloat16)
        vc = torch.randn(nb, bs, hk, D).to(torch.bfloat16)
        if kv != "auto":
            kc, vc = kc.to(torch.float8_e4m3fn), vc.to(torch.float8_e4m3fn)
        table = torch.arange(nb, dtype=torch.int32)[None, :]
        lens = torch.tensor([n], dtype=torch.int32)
        cu = torch.tensor([0, n], dtype=torch.int32)
        q = torch.randn(n, hq, D).to(torch.bfloat16)
        name = "auto" if kv == "auto" else "fp8"
        return (lambda: torch_views.run_paged_decode_attention(q, kc, vc, table, lens, D ** -0.5, name, 0.05, 0.05,
                                                               cu_seqlens_q=cu, causal=True)), n, _oracle_threads()

    tag = "bf16" if kv == "auto" else "fp8"
    return OpWorkload(
        f"prefill-{tag}" + ("" if (S, L) == (4, 2048) else f"-{L // 1024}k") + ("" if D == 128 else f"-d{D}"),
        f"paged_attention_prefill_{tag}_cache_tokens_per_s",
        f"causal paged attention of {S} whole prompts of {L} tokens, {hq} q / {hk} kv heads x {D}, cache "
        f"{'bfloat16' if kv == 'auto' else 'fp8_e4m3'}, block_size={bs} (CPU oracle: a {256}-token prompt)",
        S * L, 2 * S * L * hk * D * es + 2 * S * L * hq * D * 2, 1, make_steps, cpu_run,
        flops=4.0 * S * (L * (L + 1) / 2) * hq * D)


BY_NAME: dict[str, Callable[[], OpWorkload]] = {
    "mla-fp8": lambda: mla("fp8"),
    "gather": gather,
    "quant-static": lambda: quant("static"),
    "quant-token": lambda: quant("token"),
    "rope": lambda: rope(False),
    "rope-cache-fp8": lambda: rope(True),
    "decode-bf16": lambda: decode("auto"),
    "decode-fp8": lambda: decode("fp8"),
    "prefill-bf16": lambda: prefill("auto"),
    "prefill-fp8": lambda: prefill("fp8"),
    "prefill-bf16-8k": lambda: prefill("auto", 1, 8192),
    "prefill-fp8-8k": lambda: prefill("fp8", 1, 8192),
    "prefill-bf16-8k-d64": lambda: prefill("auto", 1, 8192, 64),
    "prefill-bf16-8k-d192": lambda: prefill("auto", 1, 8192, 192),
    "prefill-bf16-8k-d256": lambda: prefill("auto", 1, 8192, 256),
}


def cpu_rate(w: OpWorkload, budget_s: float):
    """(units/s, threads, units per pass, passes, seconds) of the CPU oracle on a sample sized for the budget."""
    probe_units = max(64, w.units_per_step // 256)
    run, n, threads = w.cpu_run(probe_units)
    t0 = time.perf_counter()
    run()
    rate0 = n / max(1e-6, time.perf_counter() - t0)
    units = int(max(probe_units, min(w.units_per_step, rate0 * budget_s / 4)))
    run, n, threads = w.cpu_run(units)
    run()
    passes, t0 = 0, time.perf_counter()
    while True:
        run()
        passes += 1
        dt = time.perf_counter() - t0
        if dt >= budget_s:
            break
    return n * passes / dt, threads, n, passes, dt
