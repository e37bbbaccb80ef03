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

    fp8 = getattr(args, "kv_dtype", "model") == "fp8"
    if fp8:                 # E4M3 pages read in place by the decode kernel (decode-shaped steps only)
        kv, kv_alt = kv.to(torch.float8_e4m3fn), kv_alt.to(torch.float8_e4m3fn)
        q8 = qt.to(torch.float8_e4m3fn)
        kv_scales = torch.ones(2, device="cuda")

    def fn():
        flip[0] ^= 1
        if fp8:
            return cu.paged_attention_decode_fp8(q8, kv if flip[0] else kv_alt, meta, d ** -0.5, None, kv_scales, torch.bfloat16,
                                                 splits=args.splits or None)
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
    kv_bytes = b * (past + q) * hkv * d * 2 * (1 if fp8 else 2)
    flops = 4.0 * b * hq * d * (q * past + q * (q + 1) / 2)
    roof = max(flops / fl, kv_bytes / bw)
    print(json.dumps({"kernel": "paged_attention", "batch": b, "past": past, "q": q, "median_us": round(med * 1e6, 2),
                      "best_us": round(best * 1e6, 2), "kv_gbs": round(kv_bytes / med / 1e9, 1),
                      "tflops": round(flops / med / 1e12, 1), "roofline_us": round(roof * 1e6, 2),
                      "fraction": round(roof / med, 3), "basis": tag, "variant": args.variant, "splits": args.splits}))
    cu.Workspace.get(torch.device("cuda", 0)).check_status()


def bench_ops(args):
    """Bandwidth-bound and recurrent kernels at prefill size (``--tokens`` rows of the Qwen3-8B / hybrid shapes): achieved
    bytes per second over the algorithmic bytes, against the measured copy bandwidth."""
    from ..ops import build_step_meta
    from ..ops import cuda as cu
    bw, _, tag = peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    t, h, inter = args.tokens, 4096, 12288
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(t, h, device="cuda", generator=g).bfloat16()
    res = torch.randn(t, h, device="cuda", generator=g).bfloat16()
    w = torch.ones(h, device="cuda").bfloat16()
    gs = torch.full((1,), 1.0 / 448, device="cuda")
    gu = torch.randn(t, 2 * inter, device="cuda", generator=g).bfloat16()
    nf = 0.5625                                                         # NVFP4 bytes per element incl. block scales
    cases = {
        "add_rmsnorm": (lambda: cu.add_rmsnorm(x, res, w, 1e-6), t * h * 2 * 4),
        "add_rmsnorm_quant": (lambda: cu.rmsnorm_quant(x, res, w, 1e-6, gs), t * h * (2 * 3 + nf)),
        "swiglu_quant": (lambda: cu.swiglu_quant(gu, gs), t * inter * (4 + nf)),
        "nvfp4_quantize": (lambda: cu.nvfp4_quantize(x, gs), t * h * (2 + nf)),
    }
    # RoPE + q/k norm + paged KV write (32 q / 8 kv heads of 128)
    hq, hkv, d, page = 32, 8, 128, 64
    seqs = max(t // 1024, 1)
    per = t // seqs
    pages_per = (per + page - 1) // page
    table = torch.arange(seqs * pages_per, dtype=torch.int32).view(seqs, pages_per)
    meta = build_step_meta([per] * seqs, [0] * seqs, table, page, device="cuda")
    kvp = torch.zeros(seqs * pages_per, 2, hkv, page, d, device="cuda", dtype=torch.bfloat16)
    qkv = torch.randn(seqs * per, (hq + 2 * hkv) * d, device="cuda", generator=g).bfloat16()
    from ..ops import reference as ref
    cs = ref.rope_cos_sin(per + 8, d, 1e6, None, device="cuda")
    nw = torch.ones(d, device="cuda").bfloat16()
    cases["rope_qknorm_kv_write"] = (lambda: cu.rope_kv_write(qkv, kvp, meta, cs, hq, hkv, d, nw, nw, 1e-6),
                                     seqs * per * ((hq + 2 * hkv) * d * 2 + (hq + 2 * hkv) * d * 2))
    # Mamba2 segmented scan (64 heads of 64, state 128, 8 groups) and gated DeltaNet (16 / 32 heads of 128)
    nh, hd, ns, ng = 64, 64, 128, 8
    xs = torch.randn(seqs * per, nh, hd, device="cuda", generator=g).bfloat16()
    dt = torch.randn(seqs * per, nh, device="cuda", generator=g).bfloat16()
    A = -torch.rand(nh, device="cuda", generator=g) - 0.5
    Bm = torch.randn(seqs * per, ng, ns, device="cuda", generator=g).bfloat16()
    Cm = torch.randn(seqs * per, ng, ns, device="cuda", generator=g).bfloat16()
    Dv, dtb = torch.ones(nh, device="cuda"), torch.zeros(nh, device="cuda")
    st = torch.zeros(seqs, nh, hd, ns, device="cuda")
    cases["ssm_scan_prefill"] = (lambda: cu.ssm_scan(xs, dt, A, Bm, Cm, Dv, dtb, st, meta),
                                 seqs * per * (nh * hd * 2 * 2 + nh * 2 + 2 * ng * ns * 2) + seqs * nh * hd * ns * 4 * 2)
    hk, hv, dk = 16, 32, 128
    qg = torch.randn(seqs * per, hk, dk, device="cuda", generator=g).bfloat16()
    kg = torch.nn.functional.normalize(torch.randn(seqs * per, hk, dk, device="cuda", generator=g), dim=-1).bfloat16()
    vg = torch.randn(seqs * per, hv, dk, device="cuda", generator=g).bfloat16()
    ag = torch.randn(seqs * per, hv, device="cuda", generator=g).bfloat16()
    bg = torch.randn(seqs * per, hv, device="cuda", generator=g).bfloat16()
    gst = torch.zeros(seqs, hv, dk, dk, device="cuda")
    cases["gated_delta_rule_prefill"] = (lambda: cu.gated_delta_rule(qg, kg, vg, ag, bg, torch.zeros(hv, device="cuda"), torch.zeros(hv, device="cuda"),
                                                                     gst, meta),
                                         seqs * per * (2 * hk * dk * 2 + 2 * hv * dk * 2 + 2 * hv * 2) + seqs * hv * dk * dk * 4 * 2)
    # sampling over the Qwen3 vocabulary
    logits = torch.randn(64, 151936, device="cuda", generator=g).bfloat16()
    cases["argmax_b64"] = (lambda: cu.argmax(logits), 64 * 151936 * 2)
    u = torch.rand(64, device="cuda")
    tk = torch.full((64,), 50, dtype=torch.int32, device="cuda")
    cases["sample_topk_topp_b64"] = (lambda: cu.sample(logits, torch.full((64,), 0.8, device="cuda"), tk, torch.full((64,), 0.9, device="cuda"), u),
                                     64 * 151936 * 2)
    want = set(args.only) if args.only else None
    for name, (fn, byts) in cases.items():
        if want and name not in want:
            continue
        med, best = time_fn(fn, args.warmup, args.iters, flush)
        print(json.dumps({"kernel": name, "tokens": t, "median_us": round(med * 1e6, 2), "best_us": round(best * 1e6, 2),
                          "algorithmic_mb": round(byts / 1e6, 1), "gbs": round(byts / med / 1e9, 1),
                          "fraction": round(byts / med / bw, 3), "basis": tag + " (copy bandwidth)"}))
    cu.Workspace.get(torch.device("cuda", 0)).check_status()


def bench_moe(args):
    """One Qwen3-30B-A3B-shape NVFP4 MoE block (128 experts, top-8, H 2048, I 768) at ``--tokens`` rows, as a whole and
    kernel by kernel.  Calls are timed as captured chains; the whole-block figure rotates over three weight sets (340 MB
    each) so the expert weights come from HBM as they do in a decode step."""
    from ..config import QuantConfig, qwen3_30b_a3b_config
    from ..models.qwen3_moe import MoEBlock
    from ..ops import cuda as cu

    def chain_us(fns):
        for f in fns:
            f()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for f in fns:
                f()
        ts = []
        for _ in range(args.iters):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3 / len(fns))
        return round(statistics.median(ts), 2)

    cfg = qwen3_30b_a3b_config(num_hidden_layers=1)
    cfg.quant = QuantConfig(quant_type="nvfp4", group_size=16, excluded=["*self_attn*", "*mlp.gate", "lm_head"])
    blocks = []
    for i in range(3):
        b = MoEBlock(cfg, "model.layers.0.mlp").cuda()
        b.random_init(torch.Generator().manual_seed(i), std=0.05)
        b.finalize()
        blocks.append(b)
    m = args.tokens
    x = torch.randn(m, cfg.hidden_size, device="cuda", generator=torch.Generator(device="cuda").manual_seed(0)).bfloat16()
    print(json.dumps({"kernel": "moe_block", "tokens": m, "us": chain_us([(lambda b=b: b(x)) for b in blocks]),
                      "expert_weight_mb": round(sum(t.numel() for t in (blocks[0].w13, blocks[0].w2)) * 1.125 / 1e6, 1)}))
    b = blocks[0]
    e, k = cfg.num_experts, cfg.num_experts_per_tok
    logits = b.gate(x)
    w, idx = cu.moe_route_softmax_topk(logits, k, True)
    ws = cu.moe_align(idx, e, 0, e)
    a = cu.moe_gather(x, ws, k, b.input_scale)
    a2 = b.expert_fc1(a, ws)
    y = cu.gemm_grouped(a2, b.w2, ws, e, alpha=b.w2_alpha, w_sf=b._w2_sf)
    parts = {"gate": lambda: b.gate(x), "route": lambda: cu.moe_route_softmax_topk(logits, k, True),
             "align": lambda: cu.moe_align(idx, e, 0, e), "gather_quant": lambda: cu.moe_gather(x, ws, k, b.input_scale),
             "fc1_swiglu_quant": lambda: b.expert_fc1(a, ws),
             "fc2": lambda: cu.gemm_grouped(a2, b.w2, ws, e, alpha=b.w2_alpha, w_sf=b._w2_sf),
             "combine": lambda: cu.moe_combine(y, ws, w)}
    print(json.dumps({"kernel": "moe_parts_us", "tokens": m, "tiles_in_use": int(ws.counts.item()) // 128,
                      **{name: chain_us([f] * 8) for name, f in parts.items()}}))
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
    a.add_argument("--kv-dtype", default="model", choices=["model", "fp8"], help="fp8: E4M3 cache pages read in place (decode shapes)")
    a.add_argument("--trace", action="store_true", help="print the per-tile timeline of the first CTA of the decode kernel")
    a.add_argument("--trace-tiles", type=int, default=0, help="tiles of the first CTA to print (it walks several items)")
    o = sub.add_parser("ops")
    o.add_argument("--tokens", type=int, default=8192)
    o.add_argument("--only", nargs="*", default=None)
    mo = sub.add_parser("moe")
    mo.add_argument("--tokens", type=int, default=32)
    for p in (g, a, o, mo):
        p.add_argument("--warmup", type=int, default=3)
        p.add_argument("--iters", type=int, default=10)
        p.add_argument("--graph", type=int, default=0, help="time decode-size calls as N captured launches per replay")
    args = ap.parse_args()
    {"gemm": bench_gemm, "attention": bench_attention, "ops": bench_ops, "moe": bench_moe}[args.cmd](args)


if __name__ == "__main__":
    main()
