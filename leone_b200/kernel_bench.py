"""Times single kernels at given sizes and relates them to the measured rooflines.

    python -m leone_b200.kernel_bench gemm --m 8 --n 4096 --k 12288 [--splits S] [--epilogue E]
    python -m leone_b200.kernel_bench decode-attention --batch 8 --context 2048
    python -m leone_b200.kernel_bench prefill-attention --tokens 2048
    python -m leone_b200.kernel_bench layer-shapes --m 8          # every product of a Qwen3-8B layer

The reference's ``--profile-decode`` prints per-operation microseconds and GEMV GB/s by shape
(crates/leone-cli/src/main.rs:2918-2995); this is the same kind of table for this engine's
kernels.  Inputs are larger than the 126 MB L2, or a buffer larger than L2 is written between
timed launches (``--flush``), so DRAM figures mean something.  Timing is by CUDA events on the
launching stream around a CUDA graph of the launches, after warm-up launches.
"""
from __future__ import annotations

import argparse
import json
import math
import sys
import types

import torch

from .benchmark import measured_peaks

DEV = "cuda:0"


def _time(fn, reps: int, warmup: int, flush=None, per_graph: int = 1) -> float:
    """Median device time of one launch, in ms.  ``per_graph`` launches (each on its own copy
    of the operands, together larger than L2) are captured into a CUDA graph and the graph's
    time is divided by their number, so the time is the kernels', not the Python calls'."""
    for _ in range(max(warmup, 1) * per_graph):
        fn()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for _ in range(per_graph):
                fn()
    torch.cuda.current_stream().wait_stream(side)
    times = []
    for _ in range(reps):
        if flush is not None:
            flush.add_(1.0)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        graph.replay()
        stop.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(stop) / per_graph)
    times.sort()
    return times[len(times) // 2]


def bench_gemm(ops, m, n, k, splits, epilogue, reps, warmup, flush, trace=False, cluster=False, norm="none",
               token_major=None):
    fast = ops.fast
    x = torch.randn((m, k), device=DEV).to(torch.bfloat16)
    # several copies of the weight so successive launches do not hit L2
    copies = max(1, min(16, int(400e6 // (n * k * 2)) + 1))
    ws = [(torch.randn((n, k), device=DEV) * 0.02).to(torch.bfloat16) for _ in range(copies)]
    out_cols = n // 2 if epilogue == 3 else n
    out = torch.empty((m, out_cols), device=DEV, dtype=torch.bfloat16 if epilogue in (0, 3) else torch.float32)
    res = out if epilogue == 2 else None
    if epilogue == 2:
        out.zero_()
    state = {"i": 0}
    full_tiles = 0
    pairs = token_major is None and splits is None and fast.in_pairs(m, n, k)    # gemm_pair.cu: no form is forced
    if pairs:
        pass
    elif token_major is None and splits is None and norm == "none":
        token_major, splits, full_tiles, cluster = fast.plan_product(m, n, k)
    elif token_major:
        splits = splits or 1
        cluster = splits > 1
    elif splits is None:
        splits, full_tiles, cluster = fast.choose_splits(m, n, k)

    # an RMSNorm folded into this product: "out" = it is the product before the norm, "in" = after
    norm_out = norm_in = None
    if norm == "out":
        norm_out = (torch.empty((m, n), device=DEV, dtype=torch.bfloat16), torch.ones(n, device=DEV),
                    torch.empty((fast.norm_parts(m, n), m), device=DEV))
    elif norm == "in":
        parts = fast.norm_parts(m, k)
        norm_in = (torch.rand((parts, m), device=DEV), parts, 1e-6)

    def run():
        w = ws[state["i"] % copies]
        state["i"] += 1
        fast._gemm(x, w, out, epilogue, res, n, splits=splits, full_tiles=full_tiles, cluster=cluster,
                   norm_in=norm_in, norm_out=norm_out, token_major=token_major)

    ms = _time(run, reps, warmup, flush, per_graph=copies)
    if trace:
        _print_trace(ops, run, copies)
    bytes_ = n * k * 2 + m * k * 2 + out.numel() * out.element_size()
    flops = 2.0 * m * n * k
    if pairs:
        ps = fast.pair_split(m, n, k) if norm == "none" else 1
        return dict(kernel="gemm_pair", m=m, n=n, k=k, norm=norm, splits=ps, full_tiles=0, cluster=ps > 1, token_major=True,
                    width=256 if ps > 1 else fast.pair_width(m, n, epilogue == 3), epilogue=epilogue, us=ms * 1e3,
                    gbs=bytes_ / ms / 1e6, tflops=flops / ms / 1e9)
    return dict(kernel="gemm_tc", m=m, n=n, k=k, norm=norm, splits=splits, full_tiles=full_tiles, cluster=bool(cluster), token_major=bool(token_major), epilogue=epilogue, us=ms * 1e3,
                gbs=bytes_ / ms / 1e6, tflops=flops / ms / 1e9)


def _print_trace(ops, run, copies):
    """Phase stamps of launches replayed back to back from a CUDA graph, the way the engine
    runs them (see leone_gemm_tc_set_trace).  Times are relative to the first instruction of
    the first block of the launch before the last; both launches are shown."""
    import ctypes
    n = max(copies, 4)
    stride = 600 * 8
    buf = torch.zeros((n, 600, 8), dtype=torch.int64, device=DEV)
    ops.fast.lib.leone_gemm_tc_set_trace(ctypes.c_void_p(buf.data_ptr()), ctypes.c_longlong(stride))
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for _ in range(n):
                run()
    torch.cuda.current_stream().wait_stream(side)
    ops.fast.lib.leone_gemm_tc_set_trace(ctypes.c_void_p(0), ctypes.c_longlong(0))
    graph.replay()
    torch.cuda.synchronize()
    buf.zero_()
    graph.replay()
    torch.cuda.synchronize()
    names = ["setup done", "early weights issued", "predecessor done", "first stage landed",
             "last mma issued", "accumulator done", "block done", "first instruction"]
    t0 = None
    for launch in (n - 2, n - 1):
        t = buf[launch]
        t = t[t[:, 6] > 0].cpu().double()
        if t.numel() == 0:
            continue
        if t0 is None:
            t0 = t[:, 7].min()
        print(f"  launch {launch} ({t.shape[0]} blocks)")
        for i in (7, 0, 1, 2, 3, 4, 5, 6):
            col = (t[:, i] - t0) / 1e3
            print(f"    {names[i]:22s} min {col.min():7.2f}  median {col.median():7.2f}  max {col.max():7.2f} us")


def bench_decode_attention(ops, batch, context, n_q, n_kv, d, page_tokens, reps, warmup, flush, prep="none"):
    """``prep``: "none" times attention over final q rows; "kernel" adds the q/k norm + rotary +
    cache-write kernel before it; "fused" lets the attention kernel do that work itself."""
    blocks = -(-context // page_tokens)
    per_copy = batch * blocks
    bytes_ = 2.0 * batch * context * n_kv * d * 2
    copies = max(1, min(64, int(400e6 // bytes_) + 1))       # successive launches read different pages
    pages = per_copy * copies
    k_pool = torch.randn((pages, n_kv, page_tokens, d), device=DEV).to(torch.bfloat16)
    v_pool = torch.randn((pages, n_kv, page_tokens, d), device=DEV).to(torch.bfloat16)
    tables = torch.randperm(pages, device=DEV).to(torch.int32).view(copies, batch, blocks)
    qkv = torch.randn((batch, (n_q + 2 * n_kv) * d), device=DEV).to(torch.bfloat16)
    out = torch.empty((batch, n_q * d), device=DEV, dtype=torch.bfloat16)
    ctx = types.SimpleNamespace(
        q_start=torch.arange(batch + 1, device=DEV, dtype=torch.int32),
        ctx_len=torch.full((batch,), context, device=DEV, dtype=torch.int32),
        status=torch.zeros(4, device=DEV, dtype=torch.int32), n_seqs=batch, max_q_len=1,
        max_ctx_len=context, decode_only=True)
    state = {"i": 0}
    ctx.positions = ctx.ctx_len - 1
    ctx.seq_of_token = torch.arange(batch, device=DEV, dtype=torch.int32)
    ctx.n_tokens = batch
    from .parts.rotary import build_rotary_table
    rope = build_rotary_table(context + 1, d, 1e6).to(DEV)
    qw = torch.ones(d, device=DEV)
    kw = torch.ones(d, device=DEV)

    def run():
        cache = types.SimpleNamespace(k_pool=k_pool, v_pool=v_pool,
                                      block_table=tables[state["i"] % copies], page_tokens=page_tokens)
        state["i"] += 1
        fuse = None
        if prep == "kernel":
            ops.qk_norm_rope_write(ctx, qkv, n_q, n_kv, d, qw, kw, 1e-6, rope, d, cache)
        elif prep == "fused":
            fuse = dict(q_w=qw, k_w=kw, eps=1e-6, rope=rope, write_cache=True)
        ops.fast.attention(ctx, qkv, out, n_q, n_kv, d, 1 / math.sqrt(d), None, cache, fuse)

    ms = _time(run, reps, warmup, flush, per_graph=copies)
    return dict(kernel="attention_decode", batch=batch, context=context, prep=prep,
                clusters=ops.fast.use_clusters, us=ms * 1e3,
                splits=ops.fast.decode_splits(batch, n_kv, n_q // n_kv, context), gbs=bytes_ / ms / 1e6)


def bench_prefill_attention(ops, tokens, n_q, n_kv, d, page_tokens, reps, warmup):
    blocks = -(-tokens // page_tokens)
    k_pool = torch.randn((blocks, n_kv, page_tokens, d), device=DEV).to(torch.bfloat16)
    v_pool = torch.randn((blocks, n_kv, page_tokens, d), device=DEV).to(torch.bfloat16)
    table = torch.randperm(blocks, device=DEV).to(torch.int32).view(1, blocks)
    qkv = torch.randn((tokens, (n_q + 2 * n_kv) * d), device=DEV).to(torch.bfloat16)
    out = torch.empty((tokens, n_q * d), device=DEV, dtype=torch.bfloat16)
    ctx = types.SimpleNamespace(
        q_start=torch.tensor([0, tokens], device=DEV, dtype=torch.int32),
        ctx_len=torch.tensor([tokens], device=DEV, dtype=torch.int32),
        status=torch.zeros(4, device=DEV, dtype=torch.int32), n_seqs=1, max_q_len=tokens,
        max_ctx_len=tokens, decode_only=False)
    cache = types.SimpleNamespace(k_pool=k_pool, v_pool=v_pool, block_table=table, page_tokens=page_tokens)
    ms = _time(lambda: ops.fast.attention(ctx, qkv, out, n_q, n_kv, d, 1 / math.sqrt(d), None, cache),
               reps, warmup)
    flops = 2.0 * n_q * d * tokens * tokens       # causal half of QK^T and PV
    return dict(kernel="attention_prefill", tokens=tokens, us=ms * 1e3, tflops=flops / ms / 1e9)


def bench_sampling(ops, rows, vocab, stages, reps, warmup):
    """The sampler's truncation pipeline (sort, stages, draw) on ``rows`` rows of ``vocab`` logits;
    wall time with a synchronize on both sides (the call makes dozens of small launches)."""
    import time
    from .sampling.sampler import TRUNCATION_STAGES
    logits = torch.randn((rows, vocab), device=DEV) * 3
    numbered = [(TRUNCATION_STAGES[n], v) for n, v in stages]
    args = (logits, [0.8] * rows, list(range(rows)), list(range(rows)), numbered)
    for _ in range(warmup):
        ops.sample_truncated(*args)
    torch.cuda.synchronize()
    t = time.perf_counter()
    for _ in range(reps):
        ops.sample_truncated(*args)
    torch.cuda.synchronize()
    return dict(kernel="sample_truncated", rows=rows, vocab=vocab, stages=[f"{n}={v}" for n, v in stages],
                us=(time.perf_counter() - t) / reps * 1e6)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m leone_b200.kernel_bench")
    ap.add_argument("what", choices=["gemm", "decode-attention", "prefill-attention", "layer-shapes", "sampling"])
    ap.add_argument("--stages", default="top_k=40,top_p=0.95",
                    help="sampling: truncation stages in order, e.g. top_k=40,typical=0.9")
    ap.add_argument("--vocab", type=int, default=151936)
    ap.add_argument("--m", type=int, default=8)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--splits", type=int, default=None)
    ap.add_argument("--epilogue", type=int, default=0)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--page-tokens", type=int, default=16)
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--flush", action="store_true", help="write a 256 MB buffer between timed launches")
    ap.add_argument("--token-major", choices=["auto", "0", "1"], default="auto",
                    help="gemm, layer-shapes: force the token-major (1) or the swapped (0) form up to 256 tokens")
    ap.add_argument("--trace", action="store_true", help="gemm: print the kernel's phase time stamps")
    ap.add_argument("--prep", choices=["none", "kernel", "fused"], default="none",
                    help="decode-attention: where q/k norm, rotary and cache write are done")
    ap.add_argument("--norm", choices=["none", "in", "out"], default="none",
                    help="gemm: fold an RMSNorm after (out) or before (in) the product into it")
    ap.add_argument("--cluster", action="store_true",
                    help="gemm with --splits: sum the splits inside thread-block clusters")
    ap.add_argument("--decode-splits", type=int, default=0,
                    help="decode-attention: split every sequence's keys this many ways (0: the dispatcher's choice)")
    ap.add_argument("--max-cluster", type=int, default=8, help="largest thread-block cluster the dispatchers may use")
    ap.add_argument("--l2-ahead", type=int, default=None,
                    help="gemm, layer-shapes: k-blocks of weights a decode-sized product asks the L2 for ahead of its stages")
    ap.add_argument("--pair-width", type=int, default=0,
                    help="gemm: tile width of the products on pairs of SMs (0: the dispatcher's choice)")
    ap.add_argument("--pair-padding", type=float, default=None,
                    help="gemm: what a pair's half tile may cost against a single block's tile (0: pairs at any size)")
    ap.add_argument("--pairs-from", type=int, default=None,
                    help="gemm: tokens from which products run on pairs of SMs")
    ap.add_argument("--decode-cluster-rounds", type=int, default=1,
                    help="decode-attention: rounds of blocks that a launch of clusters may take")
    ap.add_argument("--gemm-splits", default="",
                    help='layer-shapes: forced splits by product, "6144x4096:4,4096x12288:c8" (c: inside a cluster)')
    args = ap.parse_args(argv)
    from .ops.cuda import CudaOps
    ops = CudaOps(DEV, torch.bfloat16)
    ops.fast.force_decode_splits = args.decode_splits
    ops.fast.max_cluster = args.max_cluster
    ops.fast.decode_cluster_rounds = args.decode_cluster_rounds
    ops.fast.pair_width_override = args.pair_width
    if args.pairs_from is not None:
        ops.fast.pairs_from = args.pairs_from
    if args.pair_padding is not None:
        ops.fast.pair_padding = args.pair_padding
    if args.l2_ahead is not None:
        ops.fast.lib.leone_gemm_tc_set_l2_ahead(args.l2_ahead)
    for item in filter(None, args.gemm_splits.split(",")):
        shape, _, how = item.partition(":")
        n_, _, k_ = shape.partition("x")
        ops.fast.split_override = {**ops.fast.split_override,      # (assigned, not changed in place: forgets the plans)
                                   (int(n_), int(k_)): (int(how.lstrip("c")), how.startswith("c"))}
    peaks = measured_peaks()
    flush = torch.zeros(64 << 20, device=DEV) if args.flush else None
    rows = []
    if args.what == "gemm":
        rows.append(bench_gemm(ops, args.m, args.n, args.k, args.splits, args.epilogue, args.reps, args.warmup, flush,
                               args.trace, args.cluster, args.norm,
                               None if args.token_major == "auto" else args.token_major == "1"))
    elif args.what == "layer-shapes":
        h, inter, qkv = 4096, 12288, (args.heads + 2 * args.kv_heads) * args.head_dim
        for name, n, k, epi in (("qkv", qkv, h, 0), ("o_proj", h, args.heads * args.head_dim, 2),
                                ("gate_up", 2 * inter, h, 3), ("down", h, inter, 2), ("lm_head", 151936, h, 1)):
            r = bench_gemm(ops, args.m, n, k, None, epi, args.reps, args.warmup, flush,
                           token_major=None if args.token_major == "auto" else args.token_major == "1")
            r["name"] = name
            rows.append(r)
    elif args.what == "sampling":
        stages = [(n, float(v)) for n, v in (item.split("=") for item in args.stages.split(",") if item)]
        rows.append(bench_sampling(ops, args.batch, args.vocab, stages, args.reps, args.warmup))
    elif args.what == "decode-attention":
        rows.append(bench_decode_attention(ops, args.batch, args.context, args.heads, args.kv_heads,
                                           args.head_dim, args.page_tokens, args.reps, args.warmup, flush, args.prep))
    else:
        rows.append(bench_prefill_attention(ops, args.tokens, args.heads, args.kv_heads, args.head_dim,
                                            args.page_tokens, args.reps, args.warmup))
    for r in rows:
        if "gbs" in r:
            r["hbm_frac"] = r["gbs"] / peaks["hbm_gbs"]
        if "tflops" in r:
            r["tensor_frac"] = r["tflops"] / peaks["bf16_tflops"]
        print(json.dumps({k: (round(v, 4) if isinstance(v, float) else v) for k, v in r.items()}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
