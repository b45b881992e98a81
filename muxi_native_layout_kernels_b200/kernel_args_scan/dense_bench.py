"""Times every dense configuration of the weight-streaming path, one row per (operator, dtype, shape, token count).

    python -m muxi_native_layout_kernels_b200.kernel_args_scan.dense_bench [--json]

C1  bf16 GeMV 4096 x 4096 through gemv_layoutA.
C2  narrow GEMM, tokens {1,2,4,8,16,32,64} x {(4096,4096), (14336,4096), (4096,14336)}: fp16 through gemm_layoutA, bf16
    through gemm_layoutAB_ContinuousC and gemm_layoutABC (activations prepared with layoutB; token counts below 16 are
    zero-padded to 16 rows as that operator requires, bytes are counted with the true token count).  The bf16
    gemm_layoutA grid is the headline step of bench.py and is not repeated here.
F3  many-token GEMM muxi_hgemm_layoutA, bf16, 128 and 1024 tokens (TFLOP/s against the dense bf16 peak).
C3  soft-FP8: gemv_layoutA and gemm_layoutA_soft_fp8 with e4m3 weights, tokens {1, 8, 32} x {(28672,8192),
    (8192,28672), (8192,8192)}.
Role of the reference's benchmark_and_test/gemv_benchmark.py and gemm_benchmark.py (same traffic formula, :111).
Every case is a CUDA graph of back-to-back launches that cycle through enough weight copies for more than three L2
sizes to stream between two uses of a copy; device time from CUDA events; the table-driven entry points are used.
"""
from __future__ import annotations

import argparse
import json

import torch

import muxi_native_layout_kernels_b200 as mlk

L2_BYTES = 126 << 20
TOKENS = [1, 2, 4, 8, 16, 32, 64]
SHAPES_8B = [(4096, 4096), (14336, 4096), (4096, 14336)]
SHAPES_70B = [(28672, 8192), (8192, 28672), (8192, 8192)]
NOMINAL_HBM_GBS = 8000.0


def _time(fn_of_weight, pool, iters=5):
    reps = max(len(pool) * 2, 8)
    for i in range(min(3, len(pool))):
        fn_of_weight(pool[i])
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        fn_of_weight(pool[0])            # per-stream scratch is set up outside the capture
        with torch.cuda.graph(graph, stream=s):
            for i in range(reps):
                fn_of_weight(pool[i % len(pool)])
    torch.cuda.current_stream().wait_stream(s)
    graph.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) * 1e3 / reps)
    times.sort()
    return times[len(times) // 2]


def _pool(W):
    copies = max(2, (3 * L2_BYTES) // (W.numel() * W.element_size()) + 1)
    first = mlk.layoutA(W)
    return [first] + [first.clone() for _ in range(copies - 1)]


def _row(config, op, dtype, N, K, n, us, wbytes, peak):
    nbytes = N * K * wbytes + 2 * (n * K + n * N)
    gbs = nbytes / us / 1e3
    return {"config": config, "op": op, "dtype": dtype, "N": N, "K": K, "tokens": n, "us": round(us, 2),
            "gbs": round(gbs, 1), "frac_measured": round(gbs / peak, 3), "frac_nominal_8TBs": round(gbs / NOMINAL_HBM_GBS, 3)}


def run(dev=None, peak=6450.0, rank=0, world=1, configs=("C1", "C2", "C3", "F3"), tensor_peak=1633.9):
    """Rows for this rank's row shard of every weight matrix (rank g owns rows [g N / world, (g + 1) N / world))."""
    dev = dev or torch.device("cuda")
    mlk.set_static_weights(True)
    rows = []

    def shard(W):
        r = W.shape[0] // world
        return W[rank * r:(rank + 1) * r].contiguous()

    if "C1" in configs:
        g = torch.Generator().manual_seed(0)
        W = shard((torch.randn(4096, 4096, generator=g) * 0.02).to(torch.bfloat16)).to(dev)
        x = torch.randn(1, 4096, generator=g).to(torch.bfloat16).to(dev)
        pool = _pool(W)
        rows.append(_row("C1", "gemv_layoutA", "bf16", W.shape[0], 4096, 1, _time(lambda A: mlk.gemv_layoutA(A, x), pool), 2, peak))
        del pool
    if "C2" in configs:
        g = torch.Generator().manual_seed(1)
        for (N, K) in SHAPES_8B:
            W = shard((torch.randn(N, K, generator=g) * 0.02)).to(dev)
            p16, pbf = _pool(W.to(torch.float16)), _pool(W.to(torch.bfloat16))
            for n in TOKENS:
                X = torch.randn(n, K, generator=g)
                Xh = X.to(torch.float16).to(dev)
                rows.append(_row("C2", "gemm_layoutA", "fp16", W.shape[0], K, n, _time(lambda A: mlk.gemm_layoutA(A, Xh), p16), 2, peak))
                npad = max(16, n)
                Xp = torch.zeros(npad, K, dtype=torch.bfloat16)
                Xp[:n] = X.to(torch.bfloat16)
                XB = mlk.layoutB(Xp.to(dev))
                rows.append(_row("C2", "gemm_layoutAB_ContinuousC", "bf16", W.shape[0], K, n,
                                 _time(lambda A: mlk.gemm_layoutAB_ContinuousC(A, XB), pbf), 2, peak))
                rows.append(_row("C2", "gemm_layoutABC", "bf16", W.shape[0], K, n, _time(lambda A: mlk.gemm_layoutABC(A, XB), pbf), 2, peak))
            del p16, pbf
            torch.cuda.empty_cache()
    if "C3" in configs:
        g = torch.Generator().manual_seed(2)
        for (N, K) in SHAPES_70B:
            W8 = shard((torch.randn(N, K, generator=g) * 0.5).to(torch.float8_e4m3fn)).to(dev)
            raw = W8.view(torch.uint8)
            assert not bool(((raw & 0x7F) == 0x7F).any()), "NaN encoding in generated e4m3 weights"
            pool = _pool(W8)
            x = torch.randn(1, K, generator=g).to(torch.bfloat16).to(dev)
            rows.append(_row("C3", "gemv_layoutA", "e4m3", W8.shape[0], K, 1, _time(lambda A: mlk.gemv_layoutA(A, x), pool), 1, peak))
            for n in (1, 8, 32):
                X = torch.randn(n, K, generator=g).to(torch.bfloat16).to(dev)
                rows.append(_row("C3", "gemm_layoutA_soft_fp8", "e4m3", W8.shape[0], K, n,
                                 _time(lambda A: mlk.gemm_layoutA_soft_fp8(A, None, X), pool), 1, peak))
            del pool
            torch.cuda.empty_cache()
    if "F3" in configs:
        # many-token GEMM on the same prepacked weights (muxi_hgemm_layoutA): tensor-core bound, TFLOP/s against the
        # measured dense bf16 peak
        g = torch.Generator().manual_seed(5)
        for (N, K) in [(4096, 4096), (14336, 4096), (8192, 8192)]:
            W = shard((torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16)).to(dev)
            pool = _pool(W)
            for n in (128, 1024):
                X = torch.randn(n, K, generator=g).to(torch.bfloat16).to(dev)
                us = _time(lambda A: mlk.muxi_hgemm_layoutA(A, X), pool)
                tf = 2.0 * W.shape[0] * n * K / us / 1e6
                rows.append({"config": "F3", "op": "muxi_hgemm_layoutA", "dtype": "bf16", "N": W.shape[0], "K": K, "tokens": n,
                             "us": round(us, 2), "tflops": round(tf, 1), "frac_measured_tensor": round(tf / tensor_peak, 3)})
            del pool
            torch.cuda.empty_cache()
    return rows


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--json", action="store_true")
    ap.add_argument("--configs", default="C1,C2,C3,F3")
    a = ap.parse_args()
    out = run(configs=tuple(a.configs.split(",")))
    if a.json:
        print(json.dumps(out))
    else:
        for r in out:
            print(r, flush=True)
