"""Kernel microbenchmarks: one kernel at a time, on shapes given on the command line.

    python -m tandem_b200.kernels.microbench gemm --m 8 --n 24576 --k 4096
    python -m tandem_b200.kernels.microbench decode-attention --batch 64 --context 2048
    python -m tandem_b200.kernels.microbench prefill-attention --tokens 2048
    python -m tandem_b200.kernels.microbench tokenwise --tokens 2048
    python -m tandem_b200.kernels.microbench norm-gemm --m 8 --n 6144 --k 4096
    python -m tandem_b200.kernels.microbench dispatch [--shapes 8b|14b|32b]
    python -m tandem_b200.kernels.microbench step-timeline --batch 8 --layers 4
    python -m tandem_b200.kernels.microbench sink-attention --tokens 2048 --window 1024 --keep-first 4
    python -m tandem_b200.kernels.microbench recurrence --tokens 2048 --heads 32 --head-dim 128
    python -m tandem_b200.kernels.microbench post-norm --tokens 2048 --hidden 4096 --taps 4 --results 8
    python -m tandem_b200.kernels.microbench window-attention --tokens 2048 --window 1024 --taps 4 --width 4096

Timing follows 12vivi/tandem's kernel benchmarks (benchmarks/bench_gemv.py:3-6,35-56): the calls are
captured in one CUDA graph so that launch cost does not count, and weights or caches are rotated
through copies that together exceed L2, so every call streams from HBM.  ``--no-graph --iters N``
runs N plain launches instead (what a profiler is pointed at).
"""

from __future__ import annotations

import argparse
import math

import torch

L2_BYTES = 126 << 20


def time_calls(fn, iters: int, graph: bool) -> float:
    """Microseconds per call of fn(i), i = 0 .. iters-1."""
    for i in range(min(3, iters)):
        fn(i)
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(iters):
                fn(i)
        g.replay()
        torch.cuda.synchronize()
        start.record()
        g.replay()
        stop.record()
    else:
        start.record()
        for i in range(iters):
            fn(i)
        stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / iters * 1000.0


def copies_for(nbytes: int) -> int:
    return max(2, 3 * L2_BYTES // max(1, nbytes) + 1)


def bench_gemm(args) -> None:
    from tandem_b200.kernels import gemm_bf16

    M, N, K = args.m, args.n, args.k
    ws = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(copies_for(N * K * 2))]
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    out = torch.float32 if args.f32_out else torch.bfloat16
    rows = []
    if gemm_bf16.skinny_applies(M, N, K) and args.impl in ("both", "skinny"):
        rows.append(("tcgen05 skinny kernel", time_calls(lambda i: gemm_bf16.skinny(x, ws[i % len(ws)], out), args.iters, args.graph)))
    if gemm_bf16.gemv_applies(M, N, K) and args.impl in ("both", "gemv"):
        rows.append(("mma.sync streaming kernel", time_calls(lambda i: gemm_bf16.gemv(x, ws[i % len(ws)], out), args.iters, args.graph)))
    if args.impl in ("both", "wide") and M > gemm_bf16.SKINNY_MAX_ROWS and gemm_bf16.wide_applies(M, N, K):
        rows.append(("tcgen05 wide kernel", time_calls(lambda i: gemm_bf16.wide(x, ws[i % len(ws)], out), args.iters, args.graph)))
    if args.impl in ("both", "pair") and M > gemm_bf16.SKINNY_MAX_ROWS and gemm_bf16.wide_applies(M, N, K):
        rows.append(("tcgen05 pair kernel", time_calls(lambda i: gemm_bf16.wide_pair(x, ws[i % len(ws)], out), args.iters, args.graph)))
    if args.impl in ("both", "library"):
        rows.append(("library (cuBLAS)", time_calls(lambda i: gemm_bf16._library(x, ws[i % len(ws)], out), args.iters, args.graph)))
    if args.gated and M > gemm_bf16.SKINNY_MAX_ROWS:
        from tandem_b200.kernels import ops

        rows.append(("wide kernel, silu*up fused", time_calls(lambda i: gemm_bf16.wide(x, ws[i % len(ws)], out, gated=True), args.iters, args.graph)))
        rows.append(("pair kernel, silu*up fused", time_calls(lambda i: gemm_bf16.wide_pair(x, ws[i % len(ws)], out, gated=True), args.iters, args.graph)))
        rows.append(("library + silu_mul kernel", time_calls(lambda i: ops.silu_mul(gemm_bf16._library(x, ws[i % len(ws)], out)), args.iters, args.graph)))
    for name, us in rows:
        print(f"gemm M={M} N={N} K={K}  {name:24s} {us:8.1f} us  {N * K * 2 / us / 1e3:7.0f} GB/s weights  "
              f"{2.0 * M * N * K / us / 1e6:7.1f} TFLOP/s")


def bench_norm_gemm(args) -> None:
    """add_rmsnorm followed by the matrix product that reads its output, as a block runs them
    (TANDEM_PDL=0 shows what the programmatic dependent launch between the two is worth)."""
    from tandem_b200.kernels import gemm_bf16, ops

    M, N, K = args.m, args.n, args.k
    ws = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(copies_for(N * K * 2))]
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    res, w = torch.randn(M, K, device="cuda"), torch.ones(K, device="cuda")
    for impl, gemm in (("tcgen05 skinny kernel", gemm_bf16.skinny), ("library (cuBLAS)", gemm_bf16._library)):
        if impl.startswith("tcgen05") and not gemm_bf16.skinny_applies(M, N, K):
            continue

        def step(i):
            gemm(ops.add_rmsnorm(x, res, w, 1e-6, torch.bfloat16), ws[i % len(ws)], torch.bfloat16)

        alone = time_calls(lambda i: gemm(x, ws[i % len(ws)], torch.bfloat16), args.iters, args.graph)
        norm = time_calls(lambda i: ops.add_rmsnorm(x, res, w, 1e-6, torch.bfloat16), args.iters, args.graph)
        both = time_calls(step, args.iters, args.graph)
        print(f"norm + gemm M={M} N={N} K={K}  {impl:24s} {both:8.1f} us  (alone: gemm {alone:.1f} us, norm {norm:.1f} us)")


LAYER_SHAPES = {  # (name, N, K) of the products of a layer and the output head
    "8b": [("qkv", 6144, 4096), ("o", 4096, 4096), ("gate_up", 24576, 4096), ("down", 4096, 12288), ("head", 151936, 4096)],
    "14b": [("qkv", 7168, 5120), ("o", 5120, 5120), ("gate_up", 34816, 5120), ("down", 5120, 17408), ("head", 151936, 5120)],
    "32b": [("qkv", 10240, 5120), ("o", 5120, 8192), ("gate_up", 51200, 5120), ("down", 5120, 25600), ("head", 151936, 5120)],
}


def bench_dispatch(args) -> None:
    """Every kernel that takes a shape, timed on the products of a layer at each class of rows, next
    to what the fixed rule of ``gemm_bf16.choose`` picks: the table its thresholds are read off."""
    from tandem_b200.kernels import gemm_bf16, ops

    bf = torch.bfloat16
    for name, N, K in LAYER_SHAPES[args.shapes]:
        ws = [torch.randn(N, K, device="cuda", dtype=bf) * 0.02 for _ in range(copies_for(N * K * 2))]
        out = torch.float32 if name == "head" else bf
        winners = {}
        for M in gemm_bf16.ROW_CLASSES:
            x = torch.randn(M, K, device="cuda", dtype=bf)
            times = {"library": time_calls(lambda i: gemm_bf16._library(x, ws[i % len(ws)], out), args.iters, args.graph)}
            if gemm_bf16.skinny_applies(M, N, K):
                times["skinny"] = time_calls(lambda i: gemm_bf16.skinny(x, ws[i % len(ws)], out), args.iters, args.graph)
            if gemm_bf16.gemv_applies(M, N, K):
                times["gemv"] = time_calls(lambda i: gemm_bf16.gemv(x, ws[i % len(ws)], out), args.iters, args.graph)
            rule, best = gemm_bf16.choose(M, N, K), min(times, key=times.get)
            # this package's kernels are kept where they are within 2 % of the fastest (gemv before skinny)
            winners[M] = next((k for k in ("gemv", "skinny") if k in times and times[k] <= 1.02 * times[best]), best)
            cells = "  ".join(f"{k} {v:7.1f} us" for k, v in times.items())
            print(f"{name:8s} M={M:3d} N={N:6d} K={K:5d} ({N * K * 2 >> 20:4d} MiB)  {cells}  rule: {rule}"
                  + ("" if rule == best else f"  (fastest: {best}, {times[rule] / times[best]:.2f}x)"))
        print(f"    ({N}, {K}): {winners},")
        if name == "gate_up" or args.many_rows:
            gated = name == "gate_up"
            for M in (96, 128, 192, 256, 384, 512, 768, 1024, 1536, 2048, 3072, 4096, 8192):
                x = torch.randn(M, K, device="cuda", dtype=bf)
                if gated:
                    times = {"wide": time_calls(lambda i: gemm_bf16.wide(x, ws[i % len(ws)], bf, gated=True), args.iters, args.graph),
                             "pair": time_calls(lambda i: gemm_bf16.wide_pair(x, ws[i % len(ws)], bf, gated=True), args.iters, args.graph),
                             "product": time_calls(lambda i: ops.silu_mul(gemm_bf16._library(x, ws[i % len(ws)], bf)), args.iters, args.graph)}
                    rule = gemm_bf16.choose_gated(M, N, K)
                else:
                    times = {"pair": time_calls(lambda i: gemm_bf16.wide_pair(x, ws[i % len(ws)], out), args.iters, args.graph),
                             "library": time_calls(lambda i: gemm_bf16._library(x, ws[i % len(ws)], out), args.iters, args.graph)}
                    rule = gemm_bf16.choose(M, N, K)
                best = min(times, key=times.get)
                cells = "  ".join(f"{k} {v:8.1f} us" for k, v in times.items())
                print(f"{name:8s} M={M:4d}{' gated' if gated else ''}: {cells}  rule: {rule}"
                      + ("" if rule == best else f"  (fastest: {best}, {times[rule] / times[best]:.2f}x)"))
        del ws


def bench_step_timeline(args) -> None:
    """When every kernel of one decode step (a CUDA graph replay) starts and ends on the device, from
    the profiler's activity records: what lies on the critical path and what hides behind a neighbour."""
    from torch.profiler import ProfilerActivity, profile

    from tandem_b200.config.engine_config import EngineConfig
    from tandem_b200.engine.core import random_model
    from tandem_b200.engine.llm_engine import LLMEngine
    from tandem_b200.kernels import ops
    from tandem_b200.sampling.params import SamplingParams

    H = {"8b": 4096, "14b": 5120, "32b": 5120}[args.shapes]
    heads = {"8b": 32, "14b": 40, "32b": 64}[args.shapes]
    inter = {"8b": 12288, "14b": 17408, "32b": 25600}[args.shapes]
    config = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=args.layers, hidden_size=H,
                  num_attention_heads=heads, num_key_value_heads=8, head_dim=128, intermediate_size=inter, vocab_size=151936,
                  rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=args.context + 256)
    with torch.inference_mode(False):
        decoder, cfg = random_model(config, seed=0, dtype="bfloat16")
        pages = args.batch * (-(-(args.context + 64) // 16)) + 8
        eng = LLMEngine(EngineConfig(model="", dtype="bfloat16", block_size=16, num_kv_blocks=pages, max_num_seqs=args.batch,
                                     max_model_len=args.context + 256, cuda_graph_max_bs=args.batch),
                        decoder=decoder, model_config=cfg, load_tokenizer=False)
        g = torch.Generator().manual_seed(args.batch)
        sp = SamplingParams(max_tokens=64, temperature=0.0, ignore_eos=True)
        for _ in range(args.batch):
            eng.add_request(torch.randint(10, 100000, (args.context,), generator=g).tolist(), sp)
        while eng.scheduler.waiting or any(not r.is_decoding for r in eng.requests.values()):
            eng.step()
        for _ in range(8):
            eng.step()
        eng.drain()
        entries = eng.entries_of(eng.scheduler.schedule())
        for e in entries:
            e.want = [0]
        for _ in range(5):
            ops.argmax(eng.graphs.run(entries))
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            ops.argmax(eng.graphs.run(entries))
            torch.cuda.synchronize()
    events = sorted((e for e in prof.events() if e.device_time_total > 0 and "Memcpy" not in e.name), key=lambda e: e.time_range.start)
    t0 = events[0].time_range.start
    print(f"decode step, batch {args.batch}, context {args.context}, {args.layers} layers of Qwen3-{args.shapes} sizes: start, duration, end (us)")
    for e in events:
        start = e.time_range.start - t0
        print(f"{start:9.1f} +{e.device_time_total:7.1f} = {start + e.device_time_total:9.1f}  {e.name[:70]}")


def _cache(pages: int, nkv: int, ps: int, hd: int):
    return (torch.randn(pages, nkv, ps, hd, device="cuda", dtype=torch.bfloat16),
            torch.randn(pages, nkv, ps, hd, device="cuda", dtype=torch.bfloat16))


def bench_decode_attention(args) -> None:
    from tandem_b200.kernels import attention as A
    from tandem_b200.parts.base import KVView

    B, L, nh, nkv, hd, ps = args.batch, args.context, args.heads, args.kv_heads, args.head_dim, args.page_size
    pages_per_seq = -(-L // ps)
    kv_bytes = B * L * nkv * hd * 2 * 2
    copies = copies_for(kv_bytes)
    views = []
    for _ in range(copies):
        k, v = _cache(B * pages_per_seq, nkv, ps, hd)
        table = torch.randperm(B * pages_per_seq, device="cuda").to(torch.int32).view(B, pages_per_seq)
        views.append(KVView(k, v, table, None, ps, True))
    items = A.plan_decode([(b, b, L - 1) for b in range(B)], None, nkv, *([args.pieces * B * nkv] if args.pieces else []))
    spare = args.spare_items  # a CUDA graph's item array has room for the largest plan of its bucket: blocks without an item
    flat = torch.tensor([x for it in items for x in it] + [0] * (A.ITEM_INTS * spare), dtype=torch.int32, device="cuda")
    count = torch.tensor([len(items)], dtype=torch.int32, device="cuda")
    qkv = torch.randn(B, (nh + 2 * nkv) * hd, device="cuda", dtype=torch.bfloat16)
    us = time_calls(lambda i: A.paged_attention_decode(qkv, views[i % copies], flat, count, nh, nkv, hd, hd ** -0.5),
                    args.iters, args.graph)
    print(f"decode attention B={B} context={L} heads={nh}/{nkv} hd={hd} page={ps} items={len(items)}  {us:8.1f} us  "
          f"{kv_bytes / us / 1e3:7.0f} GB/s of keys and values")


def bench_prefill_attention(args) -> None:
    from tandem_b200.kernels import attention as A
    from tandem_b200.parts.base import KVView

    T, start, nh, nkv, hd, ps = args.tokens, args.start, args.heads, args.kv_heads, args.head_dim, args.page_size
    pages = -(-(start + T) // ps)
    k, v = _cache(pages, nkv, ps, hd)
    table = torch.randperm(pages, device="cuda").to(torch.int32).view(1, pages)
    kv = KVView(k, v, table, None, ps, True)
    flat = A.prefill_plan([(0, 0, start, T)], nh, nkv, hd, ps, None, "cuda")
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, device="cuda", dtype=torch.bfloat16)
    us = time_calls(lambda i: A.paged_attention_prefill(qkv, kv, flat, nh, nkv, hd, None, hd ** -0.5), args.iters, args.graph)
    flops = 4.0 * nh * hd * (T * start + T * (T + 1) / 2)
    which = "tcgen05" if A.tcgen05_prefill_applies(hd, ps) else "mma.sync"
    print(f"prefill attention ({which}) tokens={T} start={start} heads={nh}/{nkv} hd={hd} page={ps} plan={tuple(flat.shape)}  {us:8.1f} us  "
          f"{flops / us / 1e6:7.1f} TFLOP/s")


def sink_attention_case(tokens: int, batch: int, context: int, nh: int, nkv: int, dk: int, dv: int, ps: int, window: int,
                        keep_first: int, iters: int, graph: bool) -> dict:
    """The windowed attention with a sink: a prompt of ``tokens`` tokens on the tensor-core kernel, and a
    decode step of ``batch`` requests at ``context`` tokens on the kernel of one warp per token and head."""
    from tandem_b200.kernels import sink_attention as S
    from tandem_b200.parts.base import KVView

    class Ctx:
        pass

    scale, cap = dk ** -0.5, 30.0
    bias = torch.randn(129, nh, device="cuda") * 0.1
    sink = torch.randn(nh, device="cuda")
    out = {}
    # prompt
    pages = -(-tokens // ps)
    k = torch.randn(pages, nkv, ps, dk, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(pages, nkv, ps, dv, device="cuda", dtype=torch.bfloat16)
    kv = KVView(k, v, torch.randperm(pages, device="cuda").to(torch.int32).view(1, pages), None, ps, True)
    q = torch.randn(tokens, (nh + nkv) * dk + nkv * dv, device="cuda")
    tiles = torch.tensor(S.plan_tiles([0], [tokens], nh // nkv), dtype=torch.int32, device="cuda")
    us = time_calls(lambda i: S.attend_tiles(q, kv, tiles, nh, nkv, dk, dv, window, keep_first, scale, cap, bias, sink), iters, graph)
    seen = sum(min(p + 1, window) + min(keep_first, max(0, p - window + 1)) for p in range(tokens)) if window else tokens * (tokens + 1) // 2
    out["prefill_us"], out["prefill_tflops"] = us, 2.0 * nh * (dk + dv) * seen / us / 1e6
    # decode
    per_seq = -(-context // ps)
    live = min(context, (window + keep_first) if window else context)
    kv_bytes = batch * live * nkv * (dk + dv) * 2
    copies = copies_for(batch * context * nkv * (dk + dv) * 2)
    views = []
    for _ in range(copies):
        views.append(KVView(torch.randn(batch * per_seq, nkv, ps, dk, device="cuda", dtype=torch.bfloat16),
                            torch.randn(batch * per_seq, nkv, ps, dv, device="cuda", dtype=torch.bfloat16),
                            torch.randperm(batch * per_seq, device="cuda").to(torch.int32).view(batch, per_seq), None, ps, True))
    ctx = Ctx()
    ctx.positions = torch.full((batch,), context - 1, dtype=torch.int32, device="cuda")
    ctx.seq_of_token = torch.arange(batch, dtype=torch.int32, device="cuda")
    qd = torch.randn(batch, (nh + nkv) * dk + nkv * dv, device="cuda")
    decode = S.attend_split if S.split_applies(torch.bfloat16, dk, dv, nh // nkv, qd.shape[1]) else S.attend
    us = time_calls(lambda i: decode(qd, views[i % copies], ctx, nh, nkv, dk, dv, window, keep_first, scale, cap, bias, sink), iters, graph)
    out["decode_us"], out["decode_gbs"] = us, kv_bytes / us / 1e3
    return out


def bench_sink_attention(args) -> None:
    r = sink_attention_case(args.tokens, args.batch, args.context, args.heads, args.kv_heads, args.head_dim, args.value_dim or args.head_dim,
                            args.page_size, args.window, args.keep_first, args.iters, args.graph)
    print(f"sink attention heads={args.heads}/{args.kv_heads} dk={args.head_dim} dv={args.value_dim or args.head_dim} window={args.window}+{args.keep_first}: "
          f"prompt of {args.tokens} tokens {r['prefill_us']:8.1f} us {r['prefill_tflops']:7.1f} TFLOP/s;  decode B={args.batch} context={args.context} "
          f"{r['decode_us']:8.1f} us {r['decode_gbs']:7.0f} GB/s of visible keys and values")


def recurrence_case(tokens: int, batch: int, H: int, dk: int, dv: int, iters: int, graph: bool) -> dict:
    """The decay recurrence: one prompt of ``tokens`` tokens, and a decode step of ``batch`` requests (state read and written)."""
    from tandem_b200.kernels import recurrence as R

    decay = torch.full((H,), 0.99, device="cuda")
    cols = 2 * H * dk + 2 * H * dv
    out = {}
    proj = torch.randn(tokens, cols, device="cuda") * 0.1
    state = torch.zeros(2, H, dk, dv, device="cuda")
    cu = torch.tensor([0, tokens], dtype=torch.int32, device="cuda")
    slot = torch.zeros(1, dtype=torch.int32, device="cuda")
    us = time_calls(lambda i: R.scan(proj, cu, slot, 1, state, decay, H, dk, dv), iters, graph)
    out["prefill_us"], out["prefill_tflops"] = us, 4.0 * tokens * H * dk * dv / us / 1e6
    state_bytes = batch * H * dk * dv * 4
    copies = copies_for(state_bytes)
    states = [torch.zeros(batch + 1, H, dk, dv, device="cuda") for _ in range(copies)]
    projd = torch.randn(batch, cols, device="cuda") * 0.1
    cud = torch.arange(batch + 1, dtype=torch.int32, device="cuda")
    slots = torch.arange(batch, dtype=torch.int32, device="cuda")
    us = time_calls(lambda i: R.scan(projd, cud, slots, batch, states[i % copies], decay, H, dk, dv), iters, graph)
    out["decode_us"], out["decode_gbs"] = us, 2 * state_bytes / us / 1e3
    return out


def selective_case(tokens: int, batch: int, H: int, G: int, N: int, P: int, iters: int, graph: bool) -> dict:
    """The same scan with a decay per token and q and k shared by groups of heads, in the row layout of the selective
    layer ([x | B | C | dt x]): one prompt of ``tokens`` tokens, and a decode step of ``batch`` requests."""
    from tandem_b200.kernels import recurrence as R

    inner, gn = H * P, G * N
    cols = 2 * inner + 2 * gn
    out = {}

    def run(rows, decay, cu, slots, n, state):
        return R.scan_general(rows, cu, slots, n, state, None, decay, H, G, N, P, inner + gn, inner, inner + 2 * gn)

    rows = torch.randn(tokens, cols, device="cuda") * 0.1
    decay = torch.rand(tokens, H, device="cuda") * 0.1 + 0.9
    state = torch.zeros(2, inner * N + 64, device="cuda")
    cu = torch.tensor([0, tokens], dtype=torch.int32, device="cuda")
    slot = torch.zeros(1, dtype=torch.int32, device="cuda")
    us = time_calls(lambda i: run(rows, decay, cu, slot, 1, state), iters, graph)
    out["prefill_us"], out["prefill_tflops"] = us, 4.0 * tokens * H * N * P / us / 1e6
    state_bytes = batch * inner * N * 4
    copies = copies_for(state_bytes)
    states = [torch.zeros(batch + 1, inner * N + 64, device="cuda") for _ in range(copies)]
    rowsd = torch.randn(batch, cols, device="cuda") * 0.1
    decayd = torch.rand(batch, H, device="cuda") * 0.1 + 0.9
    cud = torch.arange(batch + 1, dtype=torch.int32, device="cuda")
    slots = torch.arange(batch, dtype=torch.int32, device="cuda")
    us = time_calls(lambda i: run(rowsd, decayd, cud, slots, batch, states[i % copies]), iters, graph)
    out["decode_us"], out["decode_gbs"] = us, 2 * state_bytes / us / 1e3
    return out


def experts_case(tokens: int, batch: int, hidden: int, inner: int, experts: int, top: int, iters: int, graph: bool,
                 gated: bool = True, identity: int = 0, activation: str = "gelu") -> dict:
    """Routed experts (bfloat16): ``tokens`` tokens through the sorted tiles, ``batch`` tokens through the kernel of one warp
    per output.  Gated experts have three matrices (FLOPs = 6 slots hidden inner), experts without a gate two (4 slots
    hidden inner; slots of the ``identity`` router outputs behind the experts cost nothing and are not counted); bytes of
    a decode step = the weights of the experts its slots use."""
    from tandem_b200.kernels import moe

    bf = torch.bfloat16
    mats = 3 if gated else 2
    gate_up = torch.randn(experts, (mats - 1) * inner, hidden, device="cuda", dtype=bf) * 0.02
    down = torch.randn(experts, hidden, inner, device="cuda", dtype=bf) * 0.02
    out = {}
    for name, T in (("prefill", tokens), ("decode", batch)):
        x = torch.randn(T, hidden, device="cuda", dtype=bf)
        if gated:
            ids, weights = moe.route(torch.randn(T, experts + identity, device="cuda"), top, "sigmoid", True, 1.0)
        else:
            ids, weights = moe.route(torch.randn(T, experts + identity, device="cuda"), top, "softmax", False, 1.0,
                                     torch.zeros(experts + identity, device="cuda"))
        us = time_calls(lambda i: moe.experts(x, gate_up, down, ids, weights, gated=gated, num_router_outputs=experts + identity,
                                              activation=activation), iters, graph)
        chosen = ids.flatten().tolist()
        slots = sum(1 for e in chosen if e < experts)
        out[f"{name}_us"] = us
        out[f"{name}_tflops"] = 2.0 * mats * slots * hidden * inner / us / 1e6
        used = len(set(e for e in chosen if e < experts))
        out[f"{name}_gbs"] = used * mats * hidden * inner * 2 / us / 1e3
    return out


class _Batch:
    """The device arrays of a step that the kernels between sublayers read: ``requests`` equal requests of ``each`` new
    tokens that stand ``before`` tokens into their sequences."""

    def __init__(self, requests: int, each: int, before: int) -> None:
        i32 = dict(dtype=torch.int32, device="cuda")
        self.num_seqs = requests
        self.seq_of_token = torch.arange(requests, **i32).repeat_interleave(each)
        self.positions = (before + torch.arange(each, **i32)).repeat(requests)
        self.seq_starts = torch.full((requests,), before, **i32)
        self.state_slots = torch.arange(requests, **i32)
        self.cu_seqlens = torch.arange(requests + 1, **i32) * each


def window_attention_case(tokens: int, batch: int, context: int, width: int, nh: int, nkv: int, dk: int, dv: int, ps: int, window: int,
                          taps: int, iters: int, graph: bool) -> dict:
    """What a window-attention mixer and its sandwich of norms add to the package's windowed attention, on ``tokens`` rows of one
    prompt and on ``batch`` single tokens at ``context`` tokens: the prepare kernel in three dressings ("whole": biases, a norm
    over all heads, the keys for values; "head": a weighted norm per head; "conv": a convolution of ``taps`` taps with its state
    update), each reading the float32 projection once and writing float32 queries and bfloat16 keys and values, beside the
    like kernel of the package's other windowed attention (bias + unit norm + cache write, in place); the attention kernels
    with a sink and a gate per head; and norm + add + norm (4 or 2 bytes of the output read, 8 of the stream, 2 of the
    normed rows written per number) beside the add + RMSNorm of the pre-norm models (12 bytes)."""
    from tandem_b200.kernels import ops, post_norm
    from tandem_b200.kernels import sink_attention as S
    from tandem_b200.parts.base import KVView

    f32, bf = dict(device="cuda", dtype=torch.float32), dict(device="cuda", dtype=torch.bfloat16)
    out = {}
    freq = torch.tensor([1e4 ** (-2.0 * i / dk) for i in range(dk // 2)], **f32)
    for name, T, each, before in (("prefill", tokens, tokens, 0), ("decode", batch, 1, context)):
        requests = T // each
        b = _Batch(requests, each, before)
        per_seq = -(-(before + each) // ps)
        pages = requests * per_seq

        def view(value_dim):
            table = torch.randperm(pages, device="cuda").to(torch.int32).view(requests, per_seq)
            slots = (table[b.seq_of_token.long(), (b.positions // ps).long()] * ps + b.positions % ps).to(torch.int32)
            return KVView(torch.zeros(pages, nkv, ps, dk, **bf), torch.zeros(pages, nkv, ps, value_dim, **bf), table, slots, ps, True)

        q_cols, k_cols, v_cols = nh * dk, nkv * dk, nkv * dv
        dressings = {
            "whole": dict(cols=q_cols + k_cols, dv=dk, kw=dict(bias=torch.randn(q_cols + k_cols, **f32), qk_norm="whole",
                                                               q_weight=torch.rand(q_cols, **f32), k_weight=torch.rand(k_cols, **f32),
                                                               freq=freq, values_from_keys=True)),
            "head": dict(cols=q_cols + k_cols + v_cols, dv=dv, kw=dict(qk_norm="head", q_weight=torch.rand(dk, **f32),
                                                                       k_weight=torch.rand(dk, **f32), freq=freq)),
            "conv": dict(cols=q_cols + k_cols + v_cols, dv=dv, kw=dict(taps=torch.randn(taps, q_cols + k_cols + v_cols, **f32), freq=freq)),
        }
        for label, d in dressings.items():
            cols = d["cols"]
            copies = copies_for(T * cols * 4)
            projs = [torch.randn(T, cols + nh, **f32) for _ in range(copies)]
            kv = view(d["dv"])
            kw = dict(d["kw"])
            state = None
            if label == "conv":
                state = torch.zeros(requests + 1, taps - 1, cols, **f32)
                kw["state"] = state

            def run(i, kv=kv, kw=kw, projs=projs, state=state, cols=cols, dvv=d["dv"]):
                S.prepare_rows(projs[i % len(projs)], kv, b, nh, nkv, dk, dvv, **kw)
                if state is not None:
                    post_norm.short_conv_state(projs[i % len(projs)], state, b, taps, width=cols)

            us = time_calls(run, iters, graph)
            moved = T * (cols * 4 + q_cols * 4 + (k_cols + nkv * d["dv"]) * 2)
            out[f"{name}_prepare_{label}_us"], out[f"{name}_prepare_{label}_gbs"] = us, moved / us / 1e3
        # the like kernel of the package's other windowed attention: bias + unit norm + cache write, queries left in place
        cols = q_cols + k_cols + v_cols
        projs = [torch.randn(T, cols, **f32) for _ in range(copies_for(T * cols * 4))]
        kv, bias = view(dv), torch.randn(cols, **f32)
        us = time_calls(lambda i: S.prepare(projs[i % len(projs)], bias, None, None, kv, nh, nkv, dk, dv, True, 1e-6), iters, graph)
        out[f"{name}_prep_unit_us"], out[f"{name}_prep_unit_gbs"] = us, T * (cols * 4 + q_cols * 4 + (k_cols + v_cols) * 2) / us / 1e3
        # norm + add + norm beside add + RMSNorm
        copies = copies_for(T * width * 14)
        ys = [torch.randn(T, width, **f32) for _ in range(copies)]
        xs = [torch.randn(T, width, **bf) for _ in range(copies)]
        streams = [torch.randn(T, width, **f32) for _ in range(copies)]
        w1, w2 = torch.rand(width, **f32), torch.rand(width, **f32)
        us = time_calls(lambda i: ops.norm_add_norm(ys[i % copies], w1, 1e-6, streams[i % copies], w2, 1e-6, torch.bfloat16), iters, graph)
        out[f"{name}_norm_add_norm_us"], out[f"{name}_norm_add_norm_gbs"] = us, T * width * 14 / us / 1e3
        us = time_calls(lambda i: ops.add_rmsnorm(xs[i % copies], streams[i % copies], w2, 1e-6, torch.bfloat16), iters, graph)
        out[f"{name}_add_rmsnorm_us"], out[f"{name}_add_rmsnorm_gbs"] = us, T * width * 12 / us / 1e3
    # the attention itself with a sink and a gate per head: the tile kernel on the prompt, the split kernel on single tokens
    scale, cap = dk ** -0.5, 30.0
    sink = torch.zeros(nh, **f32)
    pages = -(-tokens // ps)
    kv = KVView(torch.randn(pages, nkv, ps, dk, **bf), torch.randn(pages, nkv, ps, dv, **bf),
                torch.randperm(pages, device="cuda").to(torch.int32).view(1, pages), None, ps, True)
    q, gate = torch.randn(tokens, nh * dk, **f32), torch.randn(tokens, nh, **f32)
    tiles = torch.tensor(S.plan_tiles([0], [tokens], nh // nkv), dtype=torch.int32, device="cuda")
    us = time_calls(lambda i: S.attend_tiles(q, kv, tiles, nh, nkv, dk, dv, window, 0, scale, cap, None, sink, gate=gate), iters, graph)
    seen = sum(min(p + 1, window) for p in range(tokens)) if window else tokens * (tokens + 1) // 2
    out["prefill_attention_us"], out["prefill_attention_tflops"] = us, 2.0 * nh * (dk + dv) * seen / us / 1e6
    per_seq = -(-context // ps)
    live = min(context, window) if window else context
    copies = copies_for(batch * context * nkv * (dk + dv) * 2)
    views = [KVView(torch.randn(batch * per_seq, nkv, ps, dk, **bf), torch.randn(batch * per_seq, nkv, ps, dv, **bf),
                    torch.randperm(batch * per_seq, device="cuda").to(torch.int32).view(batch, per_seq), None, ps, True) for _ in range(copies)]
    b = _Batch(batch, 1, context - 1)
    qd, gd = torch.randn(batch, nh * dk, **f32), torch.randn(batch, nh, **f32)
    decode = S.attend_split if S.split_applies(torch.bfloat16, dk, dv, nh // nkv, qd.shape[1]) else S.attend
    us = time_calls(lambda i: decode(qd, views[i % copies], b, nh, nkv, dk, dv, window, 0, scale, cap, None, sink, gate=gd), iters, graph)
    out["decode_attention_us"], out["decode_attention_gbs"] = us, batch * live * nkv * (dk + dv) * 2 / us / 1e3
    return out


def bench_window_attention(args) -> None:
    r = window_attention_case(args.tokens, args.batch, args.context, args.width, args.heads, args.kv_heads, args.head_dim,
                              args.value_dim or args.head_dim, args.page_size, args.window, args.taps, args.iters, args.graph)
    for k in sorted(r):
        if k.endswith("_us"):
            rate = r.get(k[:-3] + "_gbs")
            print(f"{k[:-3]:36s} {r[k]:9.1f} us" + (f" {rate:8.0f} GB/s" if rate is not None else f" {r[k[:-3] + '_tflops']:8.1f} TFLOP/s"))


def post_norm_case(tokens: int, batch: int, width: int, groups: int, taps: int, results: int, iters: int, graph: bool) -> dict:
    """What stands between the sublayers of a layer with its norms on the sublayers' output, on ``tokens`` rows of one
    prompt and on ``batch`` single tokens: the link behind the mixer (stream + normed output, and the convolved
    bfloat16 input of the feed-forward: 12 + 2 bytes per number), the link behind the feed-forward with the weighted
    sum over ``results`` earlier results (4 (results + 4) bytes per number), the convolution alone in front of a mixer (6 bytes)
    and the state update.  Beside them the package's add + RMSNorm kernel for norms in front of sublayers (12 bytes)."""
    from tandem_b200.kernels import ops, post_norm

    bf = torch.bfloat16
    out = {}
    w = torch.rand(width, device="cuda") + 0.5
    tap_w = torch.randn(width, taps, device="cuda") * 0.3
    coeff = torch.rand(results + 1, device="cuda")
    for name, T, ctx in (("prefill", tokens, _Batch(1, tokens, 0)), ("decode", batch, _Batch(batch, 1, tokens))):
        copies = copies_for(T * width * 4 * (results + 4))
        xs = [torch.randn(T, width, device="cuda") for _ in range(copies)]
        ys = [torch.randn(T, width, device="cuda") for _ in range(copies)]
        seconds = [torch.empty(T, width, device="cuda") for _ in range(copies)]
        planes = [torch.randn(results + 1, T, width, device="cuda") for _ in range(copies)]
        state = torch.zeros(ctx.num_seqs, (taps - 1) * width, device="cuda")
        n = T * width
        us = time_calls(lambda i: post_norm.link(xs[i % copies], ys[i % copies], w, groups, 1e-5, seconds[i % copies], taps=tap_w,
                                                 state=state, ctx=ctx, out_dtype=bf), iters, graph)
        out[f"{name}_link_conv_us"], out[f"{name}_link_conv_gbs"] = us, n * 14 / us / 1e3
        us = time_calls(lambda i: post_norm.link(seconds[i % copies], ys[i % copies], w, groups, 1e-5, xs[i % copies],
                                                 planes=planes[i % copies], coeff=coeff, n_planes=results), iters, graph)
        out[f"{name}_link_average_us"], out[f"{name}_link_average_gbs"] = us, n * 4 * (results + 4) / us / 1e3
        us = time_calls(lambda i: post_norm.short_conv(xs[i % copies], tap_w, state, ctx, bf), iters, graph)
        out[f"{name}_conv_us"], out[f"{name}_conv_gbs"] = us, n * 6 / us / 1e3
        us = time_calls(lambda i: post_norm.short_conv_state(xs[i % copies], state, ctx, taps), iters, graph)
        out[f"{name}_conv_state_us"] = us
        hs = [torch.randn(T, width, device="cuda", dtype=bf) for _ in range(copies)]
        us = time_calls(lambda i: ops.add_rmsnorm(hs[i % copies], xs[i % copies], w, 1e-6, bf), iters, graph)
        out[f"{name}_add_rmsnorm_us"], out[f"{name}_add_rmsnorm_gbs"] = us, n * 12 / us / 1e3
    return out


def bench_post_norm(args) -> None:
    r = post_norm_case(args.tokens, args.batch, args.hidden, args.groups, args.taps, args.results, args.iters, args.graph)
    for name, T in (("prefill", args.tokens), ("decode", args.batch)):
        print(f"{name} T={T} W={args.hidden}: link + convolution {r[name + '_link_conv_us']:7.1f} us {r[name + '_link_conv_gbs']:6.0f} GB/s;  "
              f"link + average over {args.results} {r[name + '_link_average_us']:7.1f} us {r[name + '_link_average_gbs']:6.0f} GB/s;  "
              f"convolution {r[name + '_conv_us']:7.1f} us {r[name + '_conv_gbs']:6.0f} GB/s;  state {r[name + '_conv_state_us']:6.1f} us;  "
              f"add_rmsnorm {r[name + '_add_rmsnorm_us']:7.1f} us {r[name + '_add_rmsnorm_gbs']:6.0f} GB/s")


def bench_recurrence(args) -> None:
    r = recurrence_case(args.tokens, args.batch, args.heads, args.head_dim, args.value_dim or args.head_dim, args.iters, args.graph)
    print(f"decay recurrence heads={args.heads} dk={args.head_dim} dv={args.value_dim or args.head_dim}: prompt of {args.tokens} tokens "
          f"{r['prefill_us']:8.1f} us {r['prefill_tflops']:6.2f} TFLOP/s (4 T H dk dv);  decode B={args.batch} {r['decode_us']:8.1f} us "
          f"{r['decode_gbs']:7.0f} GB/s of state read and written")


def bench_tokenwise(args) -> None:
    from tandem_b200.kernels import ops

    T, H, I = args.tokens, args.hidden, args.intermediate
    bf = torch.bfloat16
    x, res, w = torch.randn(T, H, device="cuda", dtype=bf), torch.randn(T, H, device="cuda"), torch.ones(H, device="cuda")
    us = time_calls(lambda i: ops.add_rmsnorm(x, res, w, 1e-6, bf), args.iters, args.graph)
    print(f"add_rmsnorm T={T} H={H}  {us:8.1f} us  {T * H * 12 / us / 1e3:7.0f} GB/s")
    gu = torch.randn(T, 2 * I, device="cuda", dtype=bf)
    us = time_calls(lambda i: ops.silu_mul(gu), args.iters, args.graph)
    print(f"silu_mul    T={T} I={I}  {us:8.1f} us  {T * I * 6 / us / 1e3:7.0f} GB/s")
    nh, nkv, hd, ps = 32, 8, 128, 16
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, device="cuda", dtype=bf)
    pages = -(-T // ps)
    kc, vc = _cache(pages, nkv, ps, hd)
    cs = torch.randn(max(T, 16), hd, device="cuda")
    pos = torch.arange(T, dtype=torch.int32, device="cuda")
    qw = torch.ones(hd, device="cuda")
    us = time_calls(lambda i: ops.qk_norm_rope_kv(qkv, pos, pos, qw, qw, cs, kc, vc, nh, nkv, hd, hd, ps, 1e-6), args.iters, args.graph)
    print(f"qk_norm_rope_kv T={T} heads={nh}/{nkv} hd={hd}  {us:8.1f} us  {T * (nh + 2 * nkv) * hd * 2 * 2 / us / 1e3:7.0f} GB/s")
    table = torch.randn(32768, H, device="cuda", dtype=bf)
    ids = torch.randint(0, 32768, (T,), device="cuda", dtype=torch.int32)
    us = time_calls(lambda i: ops.embedding(ids, table), args.iters, args.graph)
    print(f"embedding   T={T} H={H}  {us:8.1f} us  {T * H * 6 / us / 1e3:7.0f} GB/s")
    logits = torch.randn(min(T, 64), 151936, device="cuda")
    us = time_calls(lambda i: ops.argmax(logits), args.iters, args.graph)
    print(f"argmax      R={logits.shape[0]} V=151936  {us:8.1f} us  {logits.numel() * 4 / us / 1e3:7.0f} GB/s")


def bench_sampling(args) -> None:
    """From logits [rows, vocabulary] to tokens: argmax and the filters of temperature sampling, one by one
    and together, against one pass over the logits at memory speed."""
    from tandem_b200.kernels import ops

    R, V = args.rows, args.vocab
    logits = [torch.randn(R, V, device="cuda") * 3 for _ in range(copies_for(R * V * 4))]
    u = torch.rand(R, device="cuda")

    def opts(temperature=1.0, top_k=0, top_p=1.0, min_p=0.0):
        f = lambda v: torch.full((R,), v, device="cuda", dtype=torch.float32)
        return f(temperature), torch.full((R,), top_k, device="cuda", dtype=torch.int32), f(top_p), f(min_p)

    cases = [("argmax", None), ("temperature 0.8", opts(0.8)), ("top_k 50", opts(0.8, top_k=50)), ("top_p 0.9", opts(0.8, top_p=0.9)),
             ("min_p 0.05", opts(0.8, min_p=0.05)), ("top_k 50, top_p 0.9, min_p 0.05", opts(0.8, 50, 0.9, 0.05))]
    for name, o in cases:
        if o is None:
            us = time_calls(lambda i: ops.argmax(logits[i % len(logits)]), args.iters, args.graph)
        else:
            t, k, tp, mp = o
            any_k, any_p = bool(k[0] > 0), bool(tp[0] < 1)
            us = time_calls(lambda i: ops.sample(logits[i % len(logits)], t, k, tp, mp, u, any_top_k=any_k, any_top_p=any_p),
                            args.iters, args.graph)
        print(f"sampling R={R} V={V}  {name:32s} {us:8.1f} us  ({R * V * 4 / us / 1e3:6.0f} GB/s if it were one pass)")


def main(argv=None) -> None:
    p = argparse.ArgumentParser(prog="python -m tandem_b200.kernels.microbench")
    sub = p.add_subparsers(dest="case", required=True)
    common = argparse.ArgumentParser(add_help=False)
    common.add_argument("--iters", type=int, default=20)
    common.add_argument("--no-graph", dest="graph", action="store_false")
    g = sub.add_parser("gemm", parents=[common])
    g.add_argument("--m", type=int, default=8)
    g.add_argument("--n", type=int, default=24576)
    g.add_argument("--k", type=int, default=4096)
    g.add_argument("--f32-out", action="store_true")
    g.add_argument("--gated", action="store_true", help="also time the product with the SiLU * up epilogue (rows of W = [gate | up])")
    g.add_argument("--impl", choices=["both", "skinny", "gemv", "wide", "pair", "library"], default="both")
    g.set_defaults(fn=bench_gemm)
    ng = sub.add_parser("norm-gemm", parents=[common])
    ng.add_argument("--m", type=int, default=8)
    ng.add_argument("--n", type=int, default=6144)
    ng.add_argument("--k", type=int, default=4096)
    ng.set_defaults(fn=bench_norm_gemm)
    shape = argparse.ArgumentParser(add_help=False)
    shape.add_argument("--heads", type=int, default=32)
    shape.add_argument("--kv-heads", type=int, default=8)
    shape.add_argument("--head-dim", type=int, default=128)
    shape.add_argument("--page-size", type=int, default=16)
    d = sub.add_parser("decode-attention", parents=[common, shape])
    d.add_argument("--batch", type=int, default=64)
    d.add_argument("--context", type=int, default=2048)
    d.add_argument("--pieces", type=int, default=0, help="cut every request's keys into this many items instead of what the rule picks")
    d.add_argument("--spare-items", type=int, default=0, help="room in the item array beyond the plan, as in a CUDA graph's bucket")
    d.set_defaults(fn=bench_decode_attention)
    f = sub.add_parser("prefill-attention", parents=[common, shape])
    f.add_argument("--tokens", type=int, default=2048)
    f.add_argument("--start", type=int, default=0)
    f.set_defaults(fn=bench_prefill_attention)
    for name, fn in (("sink-attention", bench_sink_attention), ("recurrence", bench_recurrence), ("window-attention", bench_window_attention)):
        c = sub.add_parser(name, parents=[common, shape])
        c.add_argument("--tokens", type=int, default=2048)
        c.add_argument("--batch", type=int, default=8)
        c.add_argument("--context", type=int, default=2048)
        c.add_argument("--value-dim", type=int, default=0)
        c.add_argument("--window", type=int, default=1024)
        c.add_argument("--keep-first", type=int, default=4)
        c.add_argument("--width", type=int, default=4096)
        c.add_argument("--taps", type=int, default=4)
        c.set_defaults(fn=fn)
    t = sub.add_parser("tokenwise", parents=[common])
    t.add_argument("--tokens", type=int, default=2048)
    t.add_argument("--hidden", type=int, default=4096)
    t.add_argument("--intermediate", type=int, default=12288)
    t.set_defaults(fn=bench_tokenwise)
    pn = sub.add_parser("post-norm", parents=[common])
    pn.add_argument("--tokens", type=int, default=2048)
    pn.add_argument("--batch", type=int, default=8)
    pn.add_argument("--hidden", type=int, default=4096)
    pn.add_argument("--groups", type=int, default=4)
    pn.add_argument("--taps", type=int, default=4)
    pn.add_argument("--results", type=int, default=8, help="earlier results in the weighted sum")
    pn.set_defaults(fn=bench_post_norm)
    sa = sub.add_parser("sampling", parents=[common])
    sa.add_argument("--rows", type=int, default=64)
    sa.add_argument("--vocab", type=int, default=151936)
    sa.set_defaults(fn=bench_sampling)
    dp = sub.add_parser("dispatch", parents=[common])
    dp.add_argument("--shapes", choices=sorted(LAYER_SHAPES), default="8b")
    dp.add_argument("--many-rows", action="store_true", help="also the pair kernel against the library at 96 to 8,192 rows, every product")
    dp.set_defaults(fn=bench_dispatch)
    tl = sub.add_parser("step-timeline", parents=[common])
    tl.add_argument("--batch", type=int, default=8)
    tl.add_argument("--context", type=int, default=2048)
    tl.add_argument("--layers", type=int, default=4)
    tl.add_argument("--shapes", choices=sorted(LAYER_SHAPES), default="8b")
    tl.set_defaults(fn=bench_step_timeline)
    args = p.parse_args(argv)
    with torch.inference_mode():
        args.fn(args)


if __name__ == "__main__":
    main()
