"""Scans the launch arguments of the fused-MoE expert kernels and writes moe_dispatch_arg.csv.

    python -m muxi_native_layout_kernels_b200.kernel_args_scan.moe_scan [--config mixtral|fine|both] [--tokens ...]

Role of the reference's kernel_args_scan/muxi_moe_args_scan.py.  For every token count a coordinate search is run:
token tiles per work item x (GEMM1 row warps, split-K), then (GEMM2 row groups, row warps, split-K) with the best
GEMM1 setting.  Each candidate is the whole layer captured in a CUDA graph over 8 different activation batches and
timed with CUDA events; a candidate must agree with the automatic setting's output within 1e-2 (combined bound).
"""
from __future__ import annotations

import argparse
import csv
import itertools

import torch

import muxi_native_layout_kernels_b200 as mlk
from muxi_native_layout_kernels_b200._lib import MlkError
from muxi_native_layout_kernels_b200.kernel_args_scan.moe_bench import CONFIGS, NBATCH, build
from muxi_native_layout_kernels_b200.muxi_moe_planC import _MOE_TABLE_FILE, fused_moe

HEADER = ["E", "topk", "H", "I", "fp8", "T", "nt", "wm1", "sk1", "rg2", "wm2", "sk2"]


def time_layer(call, iters=3):
    graph = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        with torch.cuda.graph(graph, stream=s):
            for i in range(NBATCH):
                call(i)
    torch.cuda.current_stream().wait_stream(s)
    graph.replay()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) * 1e3 / NBATCH)
    return best


def scan_case(cfg, T, w1, w2, wg, g, dev):
    E, H, I, topk, fp8 = cfg["E"], cfg["H"], cfg["I"], cfg["topk"], cfg["fp8"]
    xs = [torch.randn(T, H, generator=g, device=dev).to(torch.bfloat16) for _ in range(NBATCH)]
    logits = [(x.float() @ wg.float().t()).to(torch.bfloat16) for x in xs]
    kw = dict(block_shape=[128, 128], soft_fp8=True, fp8_repacked=True) if fp8 else {}
    want = fused_moe(xs[0], w1, w2, logits[0], topk, True, tune=(0, 0, 0, 0, 0, 0), **kw).float()
    tol = 1e-2 * max(1.0, float(want.pow(2).mean().sqrt()))

    def try_args(args):
        try:
            got = fused_moe(xs[0], w1, w2, logits[0], topk, True, tune=args, **kw).float()
        except MlkError:
            return None
        if not bool(((got - want).abs() <= tol + 1e-2 * want.abs()).all()):
            return None
        return time_layer(lambda i: fused_moe(xs[i], w1, w2, logits[i], topk, True, tune=args, **kw))

    best_args, best_us = (0, 0, 0, 0, 0, 0), try_args((0, 0, 0, 0, 0, 0))
    print(f"  T={T}: library default {best_us:.1f} us", flush=True)
    nts = [n for n in (1, 2, 4, 8) if n * 8 <= max(8, 2 * T)]
    # few routed slots leave few work items: deeper split-K is then the only source of CTAs
    few = T * topk <= 64
    for nt in nts:
        g1_best, g1_us = None, float("inf")
        for wm1, sk1 in itertools.product([1, 2, 4], [1, 2, 4, 8] if few else [1, 2]):
            us = try_args((nt, wm1, sk1, 0, 0, 0))
            if us is not None and us < g1_us:
                g1_best, g1_us = (wm1, sk1), us
        if g1_best is None:
            continue
        for rg2, wm2, sk2 in itertools.product([1, 2], [1, 2, 4], [1, 2, 4, 8] if few else [1, 2, 4]):
            args = (nt, g1_best[0], g1_best[1], rg2, wm2, sk2)
            us = try_args(args)
            if us is not None and us < best_us:
                best_args, best_us = args, us
    if H % 128 == 0 and I % 128 == 0:
        # tcgen05 expert GEMMs (16-bit or e4m3 weights): wm = 100 + ring stages, sk = CTAs per cluster
        for nt in [n for n in (1, 2, 4, 8) + (() if fp8 else (16,)) if n * 8 <= max(8, 2 * T)]:
            g1_best, g1_us = None, float("inf")
            for st1, ck1 in itertools.product([2, 3, 4], [1, 2, 4, 8] if few else [1, 2, 4]):
                us = try_args((nt, 100 + st1, ck1, 0, 103, 4))
                if us is not None and us < g1_us:
                    g1_best, g1_us = (100 + st1, ck1), us
            if g1_best is None:
                continue
            for st2, ck2 in itertools.product([2, 3, 4, 6], [1, 2, 4, 8]):
                args = (nt, g1_best[0], g1_best[1], 0, 100 + st2, ck2)
                us = try_args(args)
                if us is not None and us < best_us:
                    best_args, best_us = args, us
    if fp8 and H % 128 == 0 and I % 128 == 0:
        # native-e4m3 tcgen05 expert GEMMs (weights undecoded into the 8-bit MMA): wm = 200 + ring stages
        for nt in [n for n in (2, 4, 8) if n * 8 <= max(16, 2 * T)]:
            g1_best, g1_us = None, float("inf")
            # (240 + stages: 128 k per stage, built for 64-slot tiles without a cluster)
            for st1, ck1 in itertools.chain(itertools.product([2, 3, 4, 6], [1, 2, 4, 8] if few else [1, 2, 4]),
                                            [(42, 1), (43, 1)] if (nt == 8 and H % 128 == 0) else []):
                us = try_args((nt, 200 + st1, ck1, 0, 203, 2))
                if us is not None and us < g1_us:
                    g1_best, g1_us = (200 + st1, ck1), us
            if g1_best is None:
                continue
            # second GEMM: CTAs per cluster, or 10 + row tiles per CTA (no cluster)
            # (240 + stages: 128 k per stage, for the form without clusters)
            for st2, ck2 in itertools.chain(itertools.product([2, 3, 4, 6], [1, 2, 4, 11, 12, 14, 16, 18]),
                                            itertools.product([42, 43, 44], [11, 12, 14, 16, 18] if I % 128 == 0 else [])):
                args = (nt, g1_best[0], g1_best[1], 0, 200 + st2, ck2)
                us = try_args(args)
                if us is not None and us < best_us:
                    best_args, best_us = args, us
    if T <= 8 and T * topk <= 64:
        # decode batches as one cooperative kernel (weights through a shared-memory ring): wm = 300 in both fields
        args = (1, 300, 1, 0, 300, 1)
        us = try_args(args)
        if us is not None:
            print(f"    decode kernel {args}: {us:.1f} us", flush=True)
        if us is not None and us < best_us:
            best_args, best_us = args, us
    return best_args, best_us


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="both", choices=["mixtral", "fine", "both"])
    ap.add_argument("--tokens", default=None)
    ap.add_argument("--out", default=str(_MOE_TABLE_FILE))
    ap.add_argument("--experts", type=int, default=None,
                    help="expert count to scan instead of the configuration's: the rows an expert-parallel rank with that "
                         "many local experts looks up (with tokens = global tokens x local / global experts)")
    a = ap.parse_args(argv)
    dev = torch.device("cuda")
    mlk.set_static_weights(True)
    rows = {}
    try:
        with open(a.out) as f:
            r = csv.reader(f)
            next(r, None)
            for row in r:
                if len(row) == 12:
                    rows[tuple(int(v) for v in row[:6])] = [int(v) for v in row[6:]]
    except FileNotFoundError:
        pass
    for name in (["mixtral", "fine"] if a.config == "both" else [a.config]):
        cfg = dict(CONFIGS[name])
        if a.experts is not None:
            cfg["E"] = a.experts
        w1, w2, wg, g = build(cfg, dev)
        for T in ([int(t) for t in a.tokens.split(",")] if a.tokens else cfg["tokens"]):
            args, us = scan_case(cfg, T, w1, w2, wg, g, dev)
            rows[(cfg["E"], cfg["topk"], cfg["H"], cfg["I"], int(cfg["fp8"]), T)] = list(args)
            with open(a.out, "w", newline="") as f:
                w = csv.writer(f)
                w.writerow(HEADER)
                for k in sorted(rows):
                    w.writerow(list(k) + rows[k])
            print(f"{name} T={T}: best {args} {us:.1f} us", flush=True)
        del w1, w2
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
