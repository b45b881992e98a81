"""Runs one dense op on one shape a few times and prints its device time: the small, self-ending case to put
under a profiler, or to try launch arguments by hand.

    python -m muxi_native_layout_kernels_b200.kernel_args_scan.run_one --op gemm_layoutA --shape 14336x4096 \
           --tokens 8 [--dtype bf16|fp16|fp8] [--args 1,2,4] [--iters 5] [--copies 3]

--args: kernelParam1,kernelParam2,kernelParam3[,kernelId] (GEMM) or blockDimX,kernelId,kernelParam1,kernelParam2 (gemv);
without it the packaged dispatch table decides.  --copies weight copies are cycled so that consecutive launches
read different HBM lines.
"""
from __future__ import annotations

import argparse

import torch

import muxi_native_layout_kernels_b200 as mlk


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="gemm_layoutA", choices=["gemm_layoutA", "gemv", "gemm_layoutAB_ContinuousC", "gemm_layoutABC"])
    ap.add_argument("--shape", default="4096x4096", help="MxK: weight rows x reduction")
    ap.add_argument("--tokens", type=int, default=1)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16", "fp8"])
    ap.add_argument("--args", default=None)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--copies", type=int, default=3)
    ap.add_argument("--static-weights", action="store_true")
    ap.add_argument("--scales", action="store_true", help="fp8: pass a block-scale tensor (all ones)")
    a = ap.parse_args(argv)
    mlk.set_static_weights(a.static_weights)
    m, k = (int(v) for v in a.shape.split("x"))
    n = 1 if a.op == "gemv" else a.tokens
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    adt = torch.float16 if a.dtype == "fp16" else torch.bfloat16
    if a.dtype == "fp8":
        W = (torch.randn(m, k, generator=g, device=dev) * 0.5).to(torch.float8_e4m3fn)
    else:
        W = (torch.randn(m, k, generator=g, device=dev) * 0.02).to(adt)
    pool = [mlk.layoutA(W) for _ in range(a.copies)]
    X = torch.randn(n, k, generator=g, device=dev).to(adt)
    XB = mlk.layoutB(X) if a.op in ("gemm_layoutAB_ContinuousC", "gemm_layoutABC") else None
    args = [int(v) for v in a.args.split(",")] if a.args else None
    S = torch.ones((m + 127) // 128, (k + 127) // 128, device=dev) if (a.scales and a.dtype == "fp8") else None

    def call(A):
        if a.op == "gemv":
            if args:
                return mlk.gemv_layoutA_wapper(A, X, m, k, blockDimX=args[0], kernelId=args[1], kernelParam1=args[2], kernelParam2=args[3],
                                               scale_matrix=S)
            return mlk.gemv_layoutA(A, X, scale_matrix=S)
        if a.dtype == "fp8":
            if args:
                return mlk.gemm_layoutA_soft_fp8_wapper(A, S, X, m, n, k, kernelParam1=args[0], kernelParam2=args[1], kernelParam3=args[2],
                                                        kernelId=args[3] if len(args) > 3 else 1)
            return mlk.gemm_layoutA_soft_fp8(A, S, X)
        fn = getattr(mlk, a.op + ("_wapper" if args else ""))
        xin = XB if XB is not None else X
        if args:
            return fn(A, xin, m, n, k, kernelParam1=args[0], kernelParam2=args[1], kernelParam3=args[2],
                      kernelId=args[3] if len(args) > 3 else 1)
        return fn(A, xin)

    want = (X.float() @ W.float().t()).to(adt)
    got = call(pool[0])
    if a.op == "gemm_layoutABC":
        got = mlk.reLayoutC(got)
    err = (got.float() - want.float()).abs()
    ok = bool((err <= 1e-2 + 1e-2 * want.float().abs()).all())
    times = []
    for i in range(a.iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        call(pool[i % len(pool)])
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) * 1e3)
    wbytes = 1 if a.dtype == "fp8" else 2
    nbytes = m * k * wbytes + 2 * n * (m + k)
    best = min(times)
    print(f"{a.op} m={m} n={n} k={k} {a.dtype}: parity {'ok' if ok else 'FAIL'} max_abs {float(err.max()):.4g}; "
          f"event times us {[round(t, 2) for t in times]}; best {nbytes / best / 1e3:.0f} GB/s (single launches include launch latency)")


if __name__ == "__main__":
    main()
