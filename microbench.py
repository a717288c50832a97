"""Time one kernel of the library alone, at a given shape.

    python microbench.py linear --m 8 --n 6144 --k 4096 [--variant gemm_skinny]
    python microbench.py attention_decode --batch 8 --context 8192
    python microbench.py attention_prefill --tokens 2048
    python microbench.py rmsnorm --m 8 --k 4096
    python microbench.py sample --batch 8 --n 128256 [--temperature 0.7]
    python microbench.py delta_rule --batch 1 --tokens 2048 --heads 32 --kv-heads 16 --head-dim 128
    python microbench.py gated_recurrence --batch 1 --tokens 2048 --k 4096
    python microbench.py routed_experts --m 2048 --k 4096 --n 1792 --experts 32 --top 8 [--variant narrow|wide128]
    python microbench.py norm_add --m 2048 --k 4096 --top 8
    LLMB_NVCC_FLAGS=-DLLMB_TRACE python microbench.py linear --m 8 --n 6144 --k 4096 --timeline
    LLMB_NVCC_FLAGS=-DLLMB_TRACE python microbench.py attention_prefill --tokens 2048 --timeline

Each call is timed inside a CUDA graph of `--reps` back-to-back launches (so that
the host's launch cost is not in the number), with CUDA events, after warm-up.
Weights rotate over enough copies to exceed L2, so every launch streams from
HBM. `--once` runs a single plain launch after warm-up instead (for a profiler).
Default sizes are those of a Llama-3.1-8B layer. The per-kernel table that
MythEclipse/llm prints with LLM_PROFILE=1 (apps/engine/src/cuda/mod.rs:1917-1972)
is the precedent; this tool isolates one kernel instead of wrapping every launch.
`--timeline` (tcgen05 product and decode attention, a build with -DLLMB_TRACE) prints when
the blocks of the last launch passed the phases the kernel stamps with the GPU's global timer;
for attention_prefill it prints the SM clock cycles that a softmax thread and the product thread
spend in each phase of a key block (the phases are too short for the global timer's steps).
"""
from __future__ import annotations

import argparse
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent))

from llm_b200.ops import attention, linear, rmsnorm, rope_cache_write, swiglu, tactics  # noqa: E402

DEV = "cuda:0"


def time_in_graph(fn, reps: int, rounds: int = 10) -> float:
    """Microseconds per call of fn, from `rounds` replays of a graph of `reps` calls."""
    fn()
    fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(reps):
            fn()
    graph.replay()
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(rounds):
        graph.replay()
    end.record()
    torch.cuda.synchronize()
    return begin.elapsed_time(end) / (rounds * reps) * 1e3


def run(fn, args, work_bytes=0.0, work_flops=0.0, label=""):
    if args.once:
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        fn()
        torch.cuda.synchronize()
        print(f"{label}: one launch done")
        return
    us = time_in_graph(fn, args.reps)
    line = f"{label}: {us:.1f} us"
    if work_bytes:
        line += f", {work_bytes / us / 1e6:.2f} TB/s"
    if work_flops:
        line += f", {work_flops / us / 1e6:.1f} TFLOP/s"
    print(line)


PHASES = {
    "gemm_tc": ["block started", "set-up done", "predecessor complete", "first tiles landed",
                "last product issued", "partial written and fenced", "counter answered",
                "summed and stored (last arriver)"],
    "attention_decode": ["block started", "predecessor complete", "first pages landed", "keys done",
                         "partial written"],
}


def timeline(fn, label: str, library: str = "gemm_tc") -> int:
    """Back-to-back launches of fn, then the global-timer stamps of the last one, in microseconds
    after its first block started: earliest, median and latest block for every phase."""
    import ctypes
    from llm_b200.ops.build import load_library
    lib = load_library(library)
    read = getattr(lib, f"llmb_{library}_trace")
    rows, slots = 296, 12
    stamps = (ctypes.c_ulonglong * (rows * slots))()
    for _ in range(20):
        fn()
    torch.cuda.synchronize()
    if read(stamps, 1) != 0:
        print("this build has no stamps: set LLMB_NVCC_FLAGS=-DLLMB_TRACE", file=sys.stderr)
        return 1
    for _ in range(3):                       # the chain that is measured: the last of three launches
        fn()
    torch.cuda.synchronize()
    read(stamps, 0)
    table = torch.tensor(list(stamps), dtype=torch.float64).view(rows, slots)
    table = table[table[:, 0] > 0]
    # every block of every launch overwrites its row: what is left belongs to the last launch,
    # except phases that only some blocks reach (they may be older): those are cut at the start
    start = table[:, 0].min()
    print(f"{label}: {table.shape[0]} blocks; microseconds after the first block started")
    for slot, name in enumerate(PHASES[library]):
        column = table[:, slot]
        column = column[column >= start]
        if column.numel():
            relative = (column - start) / 1e3
            print(f"  {name:34s}{relative.min():8.2f}{relative.median():8.2f}{relative.max():8.2f}"
                  f"   ({column.numel()} blocks)")
    return 0


def phase_sums(fn, label: str) -> int:
    """attention_prefill, a build with -DLLMB_TRACE: mean SM clock cycles per key block that a softmax
    thread and the product thread of a block spend in each phase (over the launch's first 296 blocks)."""
    import ctypes
    from llm_b200.ops.build import load_library
    lib = load_library("attention_prefill_tc")
    rows, slots = 296, 12
    sums = (ctypes.c_ulonglong * (rows * slots))()
    for _ in range(5):
        fn()
    torch.cuda.synchronize()
    if lib.llmb_attention_prefill_tc_trace(sums, 1) != 0:
        print("this build has no phase sums: set LLMB_NVCC_FLAGS=-DLLMB_TRACE", file=sys.stderr)
        return 1
    fn()
    torch.cuda.synchronize()
    lib.llmb_attention_prefill_tc_trace(sums, 0)
    table = torch.tensor(list(sums), dtype=torch.float64).view(rows, slots)
    table = table[table[:, slots - 1] > 0]
    key_blocks = table[:, slots - 1].sum()
    names = ["softmax thread: waiting for S", "  reading S, the row's maximum", None,
             "  waiting for O, rescaling", "  exponentials, writing P", "  releasing P",
             "product thread: waiting for P", "  waiting for V", "  issuing P V", "  waiting for K, issuing Q K^T",
             "  the first two Q K^T"]
    print(f"{label}: {table.shape[0]} blocks, {int(key_blocks)} key blocks; mean SM cycles per key block")
    for slot, name in enumerate(names):
        if name:
            print(f"  {name:36s}{float(table[:, slot].sum() / key_blocks):9.0f}")
    return 0


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    p.add_argument("op", choices=["delta_rule", "gated_recurrence", "state_space", "routed_experts", "norm_add",
                                  "linear", "attention_decode", "attention_prefill", "rmsnorm",
                                  "swiglu", "rope", "sample"])
    p.add_argument("--m", type=int, default=8, help="rows (tokens)")
    p.add_argument("--n", type=int, default=6144)
    p.add_argument("--k", type=int, default=4096)
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--context", type=int, default=8192)
    p.add_argument("--tokens", type=int, default=2048)
    p.add_argument("--heads", type=int, default=32)
    p.add_argument("--kv-heads", type=int, default=8)
    p.add_argument("--head-dim", type=int, default=128)
    p.add_argument("--variant", default=None, help="force a kernel variant by disabling higher ranks")
    p.add_argument("--residual", action="store_true", help="linear: add into a 32-bit residual")
    p.add_argument("--norm", action="store_true", help="linear: with a folded norm (32 partial sums a row)")
    p.add_argument("--emit", action="store_true", help="linear (with --residual): leave the next norm's input")
    p.add_argument("--rope", action="store_true",
                   help="linear: the q/k/v product with rotation and cache write (n = (heads + 2 kv heads) * head dim)")
    p.add_argument("--glu", action="store_true", help="linear: the gated epilogue (n = 2 x the feed-forward width)")
    p.add_argument("--yardstick", action="store_true",
                   help="linear: also time torch.matmul (cuBLAS) on the same operands in the same harness: a "
                        "yardstick only, the library never calls it")
    p.add_argument("--temperature", type=float, default=0.0,
                   help="sample: 0 is greedy; above it the default chain (top-k 40, top-p 0.75, min-p 0.25, "
                        "repeat penalty 1.1 over the last 64) runs")
    p.add_argument("--experts", type=int, default=32)
    p.add_argument("--top", type=int, default=8, help="routed_experts: chosen experts; norm_add: rows a token")
    p.add_argument("--reps", type=int, default=20)
    p.add_argument("--once", action="store_true")
    p.add_argument("--timeline", action="store_true",
                   help="linear, attention_decode: phases of the last launch's blocks; attention_prefill: cycles "
                        "per key block and phase (builds with -DLLMB_TRACE)")
    args = p.parse_args(argv)
    torch.manual_seed(0)
    bf16 = torch.bfloat16

    if args.op == "linear":
        if args.variant:
            table = tactics.rows("linear")
            wanted = [r for r in table if r.name == args.variant][0]
            for row in table:
                if row.rank > wanted.rank:
                    tactics.disable(row.name)
        m, n, k = args.m, args.n, args.k
        copies = 1 if args.once else max(2, int(300e6 / (n * k * 2)) + 1)
        ws = [torch.randn(n, k, device=DEV, dtype=bf16) * 0.02 for _ in range(copies)]
        x = torch.randn(m, k, device=DEV, dtype=bf16)
        res = torch.zeros(m, n, device=DEV, dtype=torch.float32) if args.residual else None
        out = None if args.residual else torch.empty(m, n, device=DEV, dtype=bf16)
        turn = [0]

        import llm_b200.ops as ops
        norm = emit = rope = None
        if args.norm:
            norm = ops.FoldedNorm(x, torch.rand(m, ops.SUMSQ_LD, device=DEV) * k / 32, 32, 1e-5, k)
        if args.emit:
            emit = ops.Emit(torch.empty(m, n, device=DEV, dtype=bf16), torch.empty(m, ops.SUMSQ_LD, device=DEV))
        if args.rope:
            hq, hkv, d = args.heads, args.kv_heads, args.head_dim
            assert n == (hq + 2 * hkv) * d, "--n must be (heads + 2 kv heads) * head dim"
            if m <= 64:                      # a decode step: m sequences, each at its context's last position
                pages = (args.context + 63) // 64
                kc = torch.zeros(m * pages, hkv, 64, d, device=DEV, dtype=bf16)
                vc = torch.zeros_like(kc)
                rope = ops.RopeWrite(torch.rand(args.context, d, device=DEV),
                                     torch.full((m,), args.context - 1, dtype=torch.int32, device=DEV),
                                     torch.arange(m, dtype=torch.int32, device=DEV),
                                     torch.arange(m * pages, dtype=torch.int32, device=DEV).view(m, pages), pages,
                                     kc, vc, hq, hkv, d)
            else:                            # a prefill: one sequence of m tokens
                pages = (m + 63) // 64
                kc = torch.zeros(pages, hkv, 64, d, device=DEV, dtype=bf16)
                vc = torch.zeros_like(kc)
                rope = ops.RopeWrite(torch.rand(m, d, device=DEV), torch.arange(m, dtype=torch.int32, device=DEV),
                                     torch.zeros(m, dtype=torch.int32, device=DEV),
                                     torch.arange(pages, dtype=torch.int32, device=DEV).view(1, pages), pages,
                                     kc, vc, hq, hkv, d)
        if args.glu:
            out = torch.empty(m, n // 2, device=DEV, dtype=bf16)

        def fn():
            linear(x, ws[turn[0] % copies], residual=res, out=out, norm=norm, emit=emit, rope=rope, glu=args.glu)
            turn[0] += 1
        args.reps = max(args.reps, copies * 2) if not args.once else args.reps
        name = tactics.choose_linear(m, n, k, bf16, bf16, k)
        if args.timeline:
            return timeline(fn, f"linear {name} M={m} N={n} K={k}")
        run(fn, args, n * k * 2, 2.0 * m * n * k, f"linear {name} M={m} N={n} K={k}")
        if args.yardstick and not args.once:
            plain_out = torch.empty(m, n, device=DEV, dtype=bf16)

            def library():
                torch.matmul(x, ws[turn[0] % copies].t(), out=plain_out)
                turn[0] += 1
            run(library, args, n * k * 2, 2.0 * m * n * k, f"torch.matmul (cuBLAS) M={m} N={n} K={k}")
    elif args.op in ("attention_decode", "attention_prefill"):
        hq, hkv, d = args.heads, args.kv_heads, args.head_dim
        decode = args.op == "attention_decode"
        batch = args.batch if decode else 1
        ctx = args.context if decode else args.tokens
        pages_per = (ctx + 63) // 64
        n_pages = batch * pages_per
        kc = torch.randn(n_pages, hkv, 64, d, device=DEV, dtype=bf16)
        vc = torch.randn(n_pages, hkv, 64, d, device=DEV, dtype=bf16)
        table = torch.arange(n_pages, dtype=torch.int32, device=DEV).view(batch, pages_per)
        lens = torch.full((batch,), ctx, dtype=torch.int32, device=DEV)
        if decode:
            qkv = torch.randn(batch, (hq + 2 * hkv) * d, device=DEV, dtype=bf16)
            pos = torch.full((batch,), ctx - 1, dtype=torch.int32, device=DEV)
            seq = torch.arange(batch, dtype=torch.int32, device=DEV)
            fn = lambda: attention(qkv, kc, vc, table, pages_per, pos, seq, hq, hkv, d, d ** -0.5, 0,
                                   decode=True, seq_lens=lens, max_len=ctx)
            if args.timeline:
                return timeline(fn, f"attention_decode batch={batch} context={ctx} heads={hq}/{hkv} D={d}",
                                "attention_decode")
            run(fn, args, batch * ctx * hkv * d * 2 * 2, 0.0,
                f"attention_decode batch={batch} context={ctx} heads={hq}/{hkv} D={d}")
        else:
            qkv = torch.randn(ctx, (hq + 2 * hkv) * d, device=DEV, dtype=bf16)
            pos = torch.arange(ctx, dtype=torch.int32, device=DEV)
            seq = torch.zeros(ctx, dtype=torch.int32, device=DEV)
            cu = torch.tensor([0, ctx], dtype=torch.int32, device=DEV)
            fn = lambda: attention(qkv, kc, vc, table, pages_per, pos, seq, hq, hkv, d, d ** -0.5, 0,
                                   seq_lens=lens, max_len=ctx, cu_seqlens=cu, max_new=ctx)
            args.reps = min(args.reps, 5)
            if args.timeline:
                return phase_sums(fn, f"attention_prefill tokens={ctx} heads={hq}/{hkv} D={d}")
            run(fn, args, 0.0, 2.0 * 2.0 * ctx * ctx / 2 * d * hq,
                f"attention_prefill tokens={ctx} heads={hq}/{hkv} D={d} (causal flops)")
    elif args.op == "sample":
        from llm_b200.sampling import BatchSampler, SamplingParams
        vocab, rows = args.n, list(range(args.batch))
        sampler = BatchSampler([SamplingParams(temperature=args.temperature)] * args.batch, vocab, DEV)
        base = torch.randn(args.batch, vocab, device=DEV)
        logits = base.clone()

        def fn():
            logits.copy_(base)                      # the penalty changes logits in place
            sampler.sample(logits, rows)
        run(fn, args, 0.0, 0.0, f"sample (with a copy of the logits) rows={args.batch} vocab={vocab} "
                                f"temperature={args.temperature}")
    elif args.op == "rmsnorm":
        x = torch.randn(args.m, args.k, device=DEV)
        g = torch.ones(args.k, device=DEV)
        run(lambda: rmsnorm(x, g, 1e-5, bf16), args, args.m * args.k * 6, 0.0, f"rmsnorm {args.m}x{args.k}")
    elif args.op == "swiglu":
        gu = torch.randn(args.m, 2 * args.n, device=DEV, dtype=bf16)
        run(lambda: swiglu(gu), args, args.m * args.n * 6, 0.0, f"swiglu {args.m}x{args.n}")
    elif args.op == "rope":
        hq, hkv, d, b = args.heads, args.kv_heads, args.head_dim, args.batch
        pages_per = (args.context + 63) // 64
        kc = torch.zeros(b * pages_per, hkv, 64, d, device=DEV, dtype=bf16)
        vc = torch.zeros_like(kc)
        table = torch.arange(b * pages_per, dtype=torch.int32, device=DEV).view(b, pages_per)
        qkv = torch.randn(b, (hq + 2 * hkv) * d, device=DEV, dtype=bf16)
        pos = torch.full((b,), args.context - 1, dtype=torch.int32, device=DEV)
        seq = torch.arange(b, dtype=torch.int32, device=DEV)
        angles = torch.randn(args.context, d, device=DEV)
        run(lambda: rope_cache_write(qkv, angles, pos, seq, table, pages_per, kc, vc, hq, hkv, d), args,
            0.0, 0.0, f"rope_cache_write batch={b}")
    elif args.op in ("delta_rule", "gated_recurrence"):
        # `--batch` sequences bring `--tokens` tokens each (1: a decode step); the state of every sequence is read and written
        from llm_b200 import ops
        b, t = args.batch, args.tokens
        n = b * t
        seq = torch.arange(b, dtype=torch.int32, device=DEV).repeat_interleave(t)
        cu = torch.arange(b + 1, dtype=torch.int32, device=DEV) * t
        slots = torch.arange(b, dtype=torch.int32, device=DEV)
        if args.op == "delta_rule":
            H, G, D, V, K = args.heads, args.kv_heads, args.head_dim, args.head_dim, 4
            C = 2 * G * D + H * V
            proj = torch.randn(n, (C + H * V + 2 * H + 7) // 8 * 8, device=DEV).to(bf16)
            taps = torch.randn(C, K, device=DEV) / 2
            state = torch.zeros(b, (K - 1) * C + H * D * V, device=DEV)
            rate, dt_bias, weight = -torch.ones(H, device=DEV), torch.zeros(H, device=DEV), torch.ones(V, device=DEV)
            work = torch.empty(n, ops.delta_rule_work_width(H, G, D, V), device=DEV)
            o, mixed = torch.empty(n, H * V, device=DEV), torch.empty(n, H * V, device=DEV, dtype=bf16)
            moved = proj.numel() * 2 + work.numel() * 8 + o.numel() * 8 + mixed.numel() * 2 + state.numel() * 8
            run(lambda: ops.delta_rule(proj, taps, state, seq, cu, slots, rate, dt_bias, 1e-6, weight, 1e-5, work, o, mixed,
                                       H, G, D, V), args, moved, 6.0 * n * H * D * V,
                f"delta_rule {b} x {t} tokens, {H}/{G} heads of {D}")
        else:
            channels, blocks, K = args.k, 16, 4
            part = channels // blocks
            wide = torch.randn(n, 2 * channels, device=DEV).to(bf16)
            conv_w, conv_b = torch.randn(channels, K, device=DEV) / 2, torch.zeros(channels, device=DEV)
            gate = torch.randn(blocks, part, part, device=DEV) / part ** 0.5
            zeros, rate = torch.zeros(channels, device=DEV), -torch.ones(channels, device=DEV)
            state = torch.zeros(b, K, channels, device=DEV)
            out, work = torch.empty(n, channels, device=DEV, dtype=bf16), torch.empty(3, n, channels, device=DEV)
            moved = wide.numel() * 2 + out.numel() * 2 + work.numel() * 8 + state.numel() * 8
            run(lambda: ops.gated_recurrence(wide[:, :channels], wide[:, channels:], conv_w, conv_b, gate, zeros, gate, zeros,
                                             rate, state, seq, cu, slots, out, 1.0, work,
                                             single_tokens=t == 1), args, moved, 4.0 * n * channels * part,
                f"gated_recurrence {b} x {t} tokens, {channels} channels in {blocks} blocks")
    elif args.op == "state_space":
        # `--batch` sequences bring `--tokens` tokens each (1: a decode step): `--heads` heads of `--head-dim` values with
        # states of `--n` rows in `--kv-heads` groups, four taps
        from llm_b200 import ops
        b, t = args.batch, args.tokens
        n = b * t
        seq = torch.arange(b, dtype=torch.int32, device=DEV).repeat_interleave(t)
        cu = torch.arange(b + 1, dtype=torch.int32, device=DEV) * t
        slots = torch.arange(b, dtype=torch.int32, device=DEV)
        H, G, N, V, K = args.heads, args.kv_heads, args.n, args.head_dim, 4
        inner = H * V
        C = inner + 2 * G * N
        proj = torch.randn(n, (inner + C + H + 7) // 8 * 8, device=DEV).to(bf16)
        taps, conv_b = torch.randn(C, K, device=DEV) / 2, torch.zeros(C, device=DEV)
        state = torch.zeros(b, (K - 1) * C + H * N * V, device=DEV)
        rate, dt_bias, skip = -torch.ones(H, device=DEV), torch.zeros(H, device=DEV), torch.ones(H, device=DEV)
        weight = torch.ones(inner, device=DEV)
        work = torch.empty(n, ops.state_space_work_width(H, G, N, V), device=DEV)
        y, mixed = torch.empty(n, inner, device=DEV), torch.empty(n, inner, device=DEV, dtype=bf16)
        moved = proj.numel() * 2 + work.numel() * 8 + y.numel() * 8 + mixed.numel() * 2 + state.numel() * 8
        run(lambda: ops.state_space(proj, taps, conv_b, state, seq, cu, slots, rate, dt_bias, skip, weight, 1e-5, 8, 1.0, work, y,
                                    mixed, H, G, N, V), args, moved, 5.0 * n * H * N * V,
            f"state_space {b} x {t} tokens, {H} heads of {V} with states of {N} in {G} groups")
    elif args.op == "routed_experts":
        # `--m` tokens, width `--k`, `--experts` experts of `--n`, `--top` chosen; weights rotate only across experts
        from llm_b200 import ops
        n, hidden, F, E, top = args.m, args.k, args.n, args.experts, args.top
        h = torch.randn(n, hidden, device=DEV).to(bf16)
        router = torch.randn(E, hidden, device=DEV)
        w_up = (torch.randn(E, 2 * F, hidden, device=DEV) * 0.02).to(bf16)
        w_down = (torch.randn(E, hidden, F, device=DEV) * 0.02).to(bf16)
        a = n * top
        ids, order = torch.zeros(a, dtype=torch.int32, device=DEV), torch.zeros(a, dtype=torch.int32, device=DEV)
        weights = torch.zeros(a, device=DEV)
        plan = torch.zeros(ops.routed_experts_plan_ints(n, top, E), dtype=torch.int32, device=DEV)
        act, y = torch.zeros(a, F, device=DEV, dtype=bf16), torch.zeros(a, hidden, device=DEV)
        gathered = torch.zeros(a, hidden, device=DEV, dtype=bf16)
        if args.variant == "narrow":
            tactics.disable("routed_experts_wide")
        if args.variant == "wide128":
            tactics.disable("routed_experts_wide256")
        ops.routed_experts(h, router, None, w_up, w_down, top, ids, weights, order, plan, act, y, gathered)
        used = int(torch.unique(ids).numel())
        moved = used * 3 * hidden * F * 2 + a * (hidden * 2 + F * 4 + hidden * 4)
        run(lambda: ops.routed_experts(h, router, None, w_up, w_down, top, ids, weights, order, plan, act, y, gathered), args,
            moved, 6.0 * a * hidden * F, f"routed_experts {n} tokens, {top} of {E} experts of {F} ({used} used), width {hidden}")
    elif args.op == "norm_add":
        from llm_b200 import ops
        x, y = torch.randn(args.m, args.k, device=DEV), torch.randn(args.m * args.top, args.k, device=DEV)
        g = torch.ones(args.k, device=DEV)
        out = torch.empty(args.m, args.k, device=DEV, dtype=bf16)
        run(lambda: ops.norm_add_(x, y, g, 1e-5, args.top, g, 1e-5, out=out, out_dtype=bf16), args,
            args.m * args.k * (4 * args.top + 10), 0.0, f"norm_add {args.m}x{args.k}, {args.top} rows a token")
    return 0


if __name__ == "__main__":
    sys.exit(main())
