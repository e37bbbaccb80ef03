"""Per-kernel micro-benchmarks with roofline fractions.

    python -m tensorrt_edge_llm_b200.benchmarks.kernel_bench gemm --dtype bf16 --shapes 8192x24576x4096 64x4096x4096
    python -m tensorrt_edge_llm_b200.benchmarks.kernel_bench attention --batch 64 --past 1024 --q 1

Timing: CUDA events on the launching stream, ``--warmup`` untimed runs, a 256 MiB buffer written
between timed runs so nothing is served from L2 unless the kernel itself re-reads it.  Fractions
are reported against ``MEASURED_PEAKS.json`` at the repository root when present ("of measured"),
else against 6.65 TB/s and 1.59 PFLOP/s ("of fallback").

Counterpart of the reference's kernel benchmark programs (``unittests`` perf modes and
``examples/cpp/llm_bench.cpp``), restricted to single kernels.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import torch


def peaks():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"] * 1e9, d["bf16_tflops"] * 1e12, "of measured"
    return 6.65e12, 1.59e15, "of fallback"


def time_fn(fn, warmup=3, iters=10, flush=None, graph_reps=0):
    """Median / best seconds per call.  ``graph_reps > 0`` captures that many back-to-back calls in
    a CUDA graph and times the replay (per-call GPU time without host launch cost, but with the
    operands L2-warm after the first call: use it for latency-bound decode-size kernels)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if graph_reps > 0:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(graph_reps):
                fn()
        inner = fn
        fn = g.replay
        scale = 1.0 / graph_reps
    else:
        scale = 1.0
    ts = []
    for _ in range(iters):
        if flush is not None:
            flush.fill_(1)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e-3 * scale)
    return statistics.median(ts), min(ts)


def bench_gemm(args):
    from ..ops import cuda as cu
    from ..ops import reference as ref
    bw, fl, tag = peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for shp in args.shapes:
        m, n, k = (int(v) for v in shp.lower().split("x"))
        g = torch.Generator(device="cuda").manual_seed(0)
        if args.dtype == "nvfp4":
            x = torch.randn(m, k, device="cuda", generator=g).half()
            wq = torch.randint(0, 256, (n, k // 2), device="cuda", generator=g, dtype=torch.uint8)
            wsf = torch.randint(40, 60, (n, k // 16), device="cuda", generator=g, dtype=torch.uint8)
            atoms = cu.nvfp4_swizzle_scales(wsf)
            gs = torch.full((1,), 1.0 / 448, device="cuda")
            alpha = torch.ones(n, device="cuda")
            xq, xsf = cu.nvfp4_quantize(x, gs)
            fn = lambda: cu.gemm_nvfp4(xq, xsf, wq, atoms, alpha, torch.float16)
            wbytes = n * k * 0.5625
            abytes = m * k * 0.5625
        else:
            dt = torch.bfloat16 if args.dtype == "bf16" else torch.float16
            x = torch.randn(m, k, device="cuda", generator=g).to(dt)
            w = (torch.randn(n, k, device="cuda", generator=g) * 0.05).to(dt)
            fn = lambda: cu.gemm(x, w)
            wbytes, abytes = n * k * 2, m * k * 2
        med, best = time_fn(fn, args.warmup, args.iters, flush, args.graph if m <= 128 else 0)
        flops = 2.0 * m * n * k
        byts = wbytes + abytes + m * n * 2
        roof = max(flops / fl, byts / bw)
        print(json.dumps({"kernel": f"gemm_{args.dtype}", "M": m, "N": n, "K": k, "median_us": round(med * 1e6, 2),
                          "best_us": round(best * 1e6, 2), "tflops": round(flops / med / 1e12, 1),
                          "gbs": round(byts / med / 1e9, 1), "roofline_us": round(roof * 1e6, 2),
                          "fraction": round(roof / med, 3), "basis": tag + " (bf16 cuBLAS / copy)"}))
    cu.Workspace.get(torch.device("cuda", 0)).check_status()


def bench_attention(args):
    from ..ops import build_step_meta
    from ..ops import cuda as cu
    bw, fl, tag = peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    b, past, q = args.batch, args.past, args.q
    hq, hkv, d, page = args.hq, args.hkv, 128, 64
    pages_per = (past + q + page - 1) // page
    table = torch.arange(b * pages_per, dtype=torch.int32).view(b, pages_per)
    kv = torch.randn(b * pages_per, 2, hkv, page, d, device="cuda").bfloat16()
    kv_alt = kv.clone()          # graph timing alternates two pools so a replay never re-reads L2-resident K/V
    meta = build_step_meta([q] * b, [past] * b, table, page, device="cuda")
    qt = torch.randn(b * q, hq, d, device="cuda").bfloat16()
    if args.variant >= 0:
        if q > 4:
            cu._check(cu.lib().telb_set_attn_variant(args.variant), "set_attn_variant", 0)
        else:
            cu._check(cu.lib().telb_set_decode_variant(args.variant), "set_decode_variant", 0)
    flip = [0]

    def fn():
        flip[0] ^= 1
        return cu.paged_attention(qt, kv if flip[0] else kv_alt, meta, d ** -0.5, splits=args.splits or None)

    out = fn()
    if args.check:      # numerics against the fp32 statement of the op
        from ..ops import reference as ref
        want = ref.paged_attention(qt, kv, meta, d ** -0.5)
        err = ((out.float() - want.float()).norm() / want.float().norm()).item()
        assert err < 8e-3, err
    # a single launch timed with events also counts the host time to encode descriptors and launch: decode-size
    # calls are therefore timed as a captured chain of launches
    med, best = time_fn(fn, args.warmup, args.iters, flush, (args.graph or 8) if q <= 4 else 0)
    if args.trace:      # per-tile timeline of the first CTA (ns since it started)
        tr = torch.zeros(3, 64, 4, dtype=torch.int64, device="cuda")
        cu.paged_attention(qt, kv, meta, d ** -0.5, splits=args.splits or None, trace=tr)
        torch.cuda.synchronize()
        tiles = min(64, args.trace_tiles or (past + q + 127) // 128)
        names = {0: ("k_slot_free", "v_slot_free"), 1: ("issue_S", "issue_PV"), 2: ("S_ready", "max_exchanged", "P_published")}
        for role, evs in names.items():
            for e, nm in enumerate(evs):
                print(f"trace {nm:>14}: " + " ".join(f"{int(tr[role, j, e]):6d}" for j in range(tiles)))
    kv_bytes = b * (past + q) * hkv * d * 2 * 2
    flops = 4.0 * b * hq * d * (q * past + q * (q + 1) / 2)
    roof = max(flops / fl, kv_bytes / bw)
    print(json.dumps({"kernel": "paged_attention", "batch": b, "past": past, "q": q, "median_us": round(med * 1e6, 2),
                      "best_us": round(best * 1e6, 2), "kv_gbs": round(kv_bytes / med / 1e9, 1),
                      "tflops": round(flops / med / 1e12, 1), "roofline_us": round(roof * 1e6, 2),
                      "fraction": round(roof / med, 3), "basis": tag, "variant": args.variant, "splits": args.splits}))
    cu.Workspace.get(torch.device("cuda", 0)).check_status()


def main():
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--dtype", default="bf16", choices=["bf16", "fp16", "nvfp4"])
    g.add_argument("--shapes", nargs="+", default=["8192x24576x4096", "8192x4096x12288", "64x24576x4096", "64x4096x4096", "1x4096x4096"])
    a = sub.add_parser("attention")
    a.add_argument("--batch", type=int, default=64)
    a.add_argument("--past", type=int, default=1024)
    a.add_argument("--q", type=int, default=1)
    a.add_argument("--hq", type=int, default=32)
    a.add_argument("--hkv", type=int, default=8)
    a.add_argument("--variant", type=int, default=-1, help="decode kernel ring / residency variant (see telb_set_decode_variant)")
    a.add_argument("--splits", type=int, default=0, help="KV splits (0 = heuristic)")
    a.add_argument("--check", action="store_true", help="compare with the fp32 reference first")
    a.add_argument("--trace", action="store_true", help="print the per-tile timeline of the first CTA of the decode kernel")
    a.add_argument("--trace-tiles", type=int, default=0, help="tiles of the first CTA to print (it walks several items)")
    for p in (g, a):
        p.add_argument("--warmup", type=int, default=3)
        p.add_argument("--iters", type=int, default=10)
        p.add_argument("--graph", type=int, default=0, help="time decode-size calls as N captured launches per replay")
    args = ap.parse_args()
    {"gemm": bench_gemm, "attention": bench_attention}[args.cmd](args)


if __name__ == "__main__":
    main()
