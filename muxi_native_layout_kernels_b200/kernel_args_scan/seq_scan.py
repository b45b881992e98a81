"""Tunes the `layoutA_gemm` table for a whole sequence of launches instead of one launch at a time.

    python -m muxi_native_layout_kernels_b200.kernel_args_scan.seq_scan --shapes 4096x4096,14336x4096,4096x14336 \
           --tokens 1,2,4,8,16,32,64 [--passes 2] [--out DIR]

Why: with programmatic dependent launch the kernels of a stream overlap -- the next kernel's CTAs become resident
and fill their weight rings while the previous kernel is still finishing, if its shared memory and registers leave
room.  The cost of a launch therefore depends on its neighbours, and the best arguments found by timing one kernel
back to back with itself (scan.py) are not always the best inside a model's real sequence (measured: 1.6 % of a
21-launch step).  This tool starts from the current table and does
coordinate descent: for one (m, n, k) key at a time it tries every candidate of scan.candidates() inside the full
sequence -- the sequence is captured in a CUDA graph and replayed, every matrix having its own weights, ordered so
that other matrices stream between two uses of one matrix -- and keeps the candidate that makes the whole sequence
fastest.  The sequence is `for n in tokens: for (m, k) in shapes`, the order of a decoder layer's projections.
The reference has no counterpart (its kernel_args_scan scripts time single kernels).
"""
from __future__ import annotations

import argparse
from pathlib import Path

import torch

import muxi_native_layout_kernels_b200 as mlk
from muxi_native_layout_kernels_b200._lib import MlkError, PKG_DIR
from muxi_native_layout_kernels_b200.kernel_args_scan.scan import (GEMM_HEADER, TABLES, candidates, close_enough,
                                                                  read_table, write_table)


def time_sequence(calls, reps: int = 3, replays: int = 10) -> float:
    """Device time (us) of one pass over `calls` (zero-argument launchers): the sequence is captured in a CUDA graph,
    the graph is replayed `replays` times back to back between two events (so the last launch of one pass overlaps
    the first of the next, as in a serving loop), best of `reps` such measurements."""
    for c in calls:
        c()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        with torch.cuda.graph(graph, stream=s):
            for c in calls:
                c()
    torch.cuda.current_stream().wait_stream(s)
    graph.replay()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(replays):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) * 1e3 / replays)
    return best


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", required=True, help="comma list of MxK (weight rows x reduction)")
    ap.add_argument("--tokens", default="1,2,4,8,16,32,64")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16"])
    ap.add_argument("--passes", type=int, default=2)
    ap.add_argument("--out", default=str(PKG_DIR), help="directory of the table file")
    a = ap.parse_args(argv)
    mlk.set_static_weights(True)
    dev = torch.device("cuda")
    dtype = torch.float16 if a.dtype == "fp16" else torch.bfloat16
    fname, kind = TABLES["layoutA_gemm"]
    path = Path(a.out) / fname
    rows = read_table(path, 3)
    shapes = [tuple(int(v) for v in s.split("x")) for s in a.shapes.split(",")]
    tokens = [int(t) for t in a.tokens.split(",")]
    order = [(n, m, k) for n in tokens for (m, k) in shapes]

    g = torch.Generator(device=dev).manual_seed(1)
    W, A, X, want = {}, {}, {}, {}
    for (m, k) in shapes:
        W[(m, k)] = (torch.randn(m, k, generator=g, device=dev) * 0.02).to(dtype)
        A[(m, k)] = mlk.layoutA(W[(m, k)])
    for n in tokens:
        for kk in sorted({k for (_, k) in shapes}):
            X[(n, kk)] = torch.randn(n, kk, generator=g, device=dev).to(dtype)
    for (n, m, k) in order:
        want[(n, m, k)] = (X[(n, k)].float() @ W[(m, k)].float().t()).to(dtype)

    def launcher(n, m, k, c):
        return lambda: mlk.gemm_layoutA_wapper(A[(m, k)], X[(n, k)], m, n, k, kernelParam1=c[1], kernelParam2=c[2],
                                               kernelParam3=c[3], kernelId=c[0])

    choice = {}
    for (n, m, k) in order:
        if (m, n, k) not in rows:
            raise SystemExit(f"table {path} has no row for m={m} n={n} k={k}: run scan.py first")
        choice[(n, m, k)] = tuple(rows[(m, n, k)])
    base = time_sequence([launcher(*key, choice[key]) for key in order])
    print(f"start: {base:.1f} us per sequence of {len(order)} launches", flush=True)
    for ps in range(a.passes):
        changed = 0
        for key in order:
            n, m, k = key
            best_c, best_t = choice[key], base
            for c in candidates(kind, m, n, k):
                if c == choice[key]:
                    continue
                try:
                    got = launcher(n, m, k, c)()
                except MlkError:
                    continue
                if not close_enough(got, want[key]):
                    continue
                t = time_sequence([launcher(*kk, c if kk == key else choice[kk]) for kk in order], reps=2)
                if t < best_t - 0.5:          # ignore gains below the timing noise
                    best_c, best_t = c, t
            if best_c != choice[key]:
                # confirm against a fresh measurement of the incumbent before switching
                t_old = time_sequence([launcher(*kk, choice[kk]) for kk in order])
                t_new = time_sequence([launcher(*kk, best_c if kk == key else choice[kk]) for kk in order])
                if t_new < t_old - 0.5:
                    print(f"pass {ps} m={m} n={n} k={k}: {choice[key]} -> {best_c}  {t_old:.1f} -> {t_new:.1f} us", flush=True)
                    choice[key], base = best_c, t_new
                    rows[(m, n, k)] = list(best_c)
                    write_table(path, GEMM_HEADER, rows)
                    changed += 1
                else:
                    base = t_old
        print(f"pass {ps}: {changed} rows changed, {base:.1f} us per sequence", flush=True)
        if changed == 0:
            break


if __name__ == "__main__":
    main()
