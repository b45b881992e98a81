"""Generates the golden fixtures of this directory from the reference checkout.

Run once, on a machine that has the reference tree, from any directory:
    python tests/golden/make_golden.py /path/to/reference
It imports the reference's own torch functions (muxi_layout_kernels/utils.py: fused_moe, scale_tensor,
scale_whole_tensor) with an empty stand-in for its compiled extension, and applies the reference's layout recipes
(view/permute lines quoted below) to seeded inputs.  Inputs and outputs are stored together, so the tests never
need the reference tree.  Files written: layouts.npz, dequant.pt, moe_*.pt, dense.pt.
"""
from __future__ import annotations

import os
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def import_reference(ref_root: str):
    # the repository root holds a same-named drop-in package: make sure the reference wins
    sys.path = [p for p in sys.path if os.path.abspath(p or ".") != str(HERE.parent.parent)]
    sys.path.insert(0, ref_root)
    sys.modules["muxi_layout_kernels_ext"] = types.ModuleType("muxi_layout_kernels_ext")
    import muxi_layout_kernels.utils as ref_utils
    assert os.path.abspath(ref_utils.__file__).startswith(os.path.abspath(ref_root)), ref_utils.__file__
    return ref_utils


def golden_layouts():
    g = torch.Generator().manual_seed(100)
    out = {}
    # layout A: benchmark_and_test/gemm_benchmark.py:41-42
    for name, (m, k) in {"a16": (32, 64), "a8": (48, 40)}.items():
        A = torch.randint(-30000, 30000, (m, k), generator=g, dtype=torch.int16)
        out[f"{name}_in"] = A.numpy()
        out[f"{name}_out"] = A.view(m // 16, 16, k // 8, 8).permute(0, 2, 1, 3).contiguous().numpy()
    # layout B: benchmark_and_test/transposeB_bench.py:10-11
    n, k = 32, 96
    B = torch.randint(-30000, 30000, (n, k), generator=g, dtype=torch.int16)
    out["b_in"] = B.numpy()
    out["b_out"] = B.view(n // 16, 16, k // 32, 4, 8).permute(2, 0, 3, 1, 4).contiguous().numpy()
    # layout C -> row-major: benchmark_and_test/gemm_benchmark.py:74-76
    m, n = 64, 32
    C5 = torch.randint(-30000, 30000, (m // 32, n // 16, 4, 16, 8), generator=g, dtype=torch.int16)
    out["c_in"] = C5.numpy()
    out["c_out"] = C5.permute(1, 3, 0, 2, 4).contiguous().view(n, m).numpy()
    # fp8 repack: csrc/fp8_weight_repack.cu:35-36, evaluated on 32-bit words exactly as written there
    raw = torch.randint(0, 256, (8, 64), generator=g, dtype=torch.int64).to(torch.uint8).numpy()
    words = raw.view(np.uint32)
    rep = (words & np.uint32(0xFF0000FF)) | ((words & np.uint32(0x00FF0000)) >> np.uint32(8)) | (
        (words & np.uint32(0x0000FF00)) << np.uint32(8))
    out["repack_in"] = raw
    out["repack_out"] = rep.view(np.uint8)
    # e4m3 -> float: torch's own cast for every finite byte
    allb = torch.arange(256, dtype=torch.int64).to(torch.uint8)
    out["e4m3_bytes"] = allb.numpy()
    out["e4m3_float"] = allb.view(torch.float8_e4m3fn).to(torch.float32).numpy()
    np.savez_compressed(HERE / "layouts.npz", **out)


def golden_dequant(ref_utils):
    g = torch.Generator().manual_seed(101)
    w8 = (torch.randn(256, 384, generator=g) * 0.5).to(torch.float8_e4m3fn)
    sc = torch.rand(2, 3, generator=g) * 2
    out = ref_utils.scale_tensor(w8.to(torch.bfloat16), sc)
    we = (torch.randn(3, 128, 256, generator=g) * 0.5).to(torch.float8_e4m3fn)
    se = torch.rand(3, 1, 2, generator=g) * 2
    oute = ref_utils.scale_whole_tensor(we, se)
    torch.save({"w8": w8.view(torch.uint8), "scale": sc, "out": out,
                "we": we.view(torch.uint8), "se": se, "oute": oute}, HERE / "dequant.pt")


def moe_case(ref_utils, name, seed, T, E, topk, H, I, dtype, score_func, groups, topk_group, use_bias, fp8, renorm=True):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, H, generator=g).to(dtype)
    if fp8:
        w1 = (torch.randn(E, 2 * I, H, generator=g) * 0.5).to(torch.float8_e4m3fn)
        w2 = (torch.randn(E, H, I, generator=g) * 0.5).to(torch.float8_e4m3fn)
        w1_ref, w2_ref = w1.to(dtype), w2.to(dtype)
    else:
        w1 = (torch.randn(E, 2 * I, H, generator=g) * 0.05).to(dtype)
        w2 = (torch.randn(E, H, I, generator=g) * 0.05).to(dtype)
        w1_ref, w2_ref = w1, w2
    logits = torch.randn(T, E, generator=g).to(dtype)
    bias = (torch.randn(E, generator=g) * 0.1).to(dtype) if use_bias else None
    y = ref_utils.fused_moe(x, w1_ref, w2_ref, logits, topk, groups, topk_group, global_num_experts=E,
                            renormalize=renorm, e_score_correction_bias=bias, score_func=score_func)
    torch.save({"x": x, "w1": w1.view(torch.uint8) if fp8 else w1, "w2": w2.view(torch.uint8) if fp8 else w2,
                "logits": logits, "bias": bias, "y": y, "topk": topk, "groups": groups, "topk_group": topk_group,
                "score_func": score_func, "renormalize": renorm, "fp8": fp8}, HERE / f"moe_{name}.pt")


def golden_dense():
    """Dense expected values by the math the reference's benchmarks compare with (fp32 product, one rounding;
    csrc/gemm_ex.cu:40-43 with COMPUTE_32F), bias added afterwards in 16-bit as gemv_benchmark.py:41 does."""
    g = torch.Generator().manual_seed(102)
    out = {}
    for dt_name, dt in (("bf16", torch.bfloat16), ("fp16", torch.float16)):
        W = (torch.randn(128, 256, generator=g) * 0.02).to(dt)
        X = torch.randn(5, 256, generator=g).to(dt)
        bias = torch.randn(128, generator=g).to(dt)
        out[dt_name] = {"W": W, "X": X, "bias": bias,
                        "C": (X.float() @ W.float().t()).to(dt),
                        "C_bias": (X.float() @ W.float().t()).to(dt) + bias}
    torch.save(out, HERE / "dense.pt")


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path to a checkout of the reference project>")
    ref_root = sys.argv[1]
    ref_utils = import_reference(ref_root)
    torch.set_num_threads(1)   # fixed summation order inside torch's CPU GEMM
    golden_layouts()
    golden_dequant(ref_utils)
    golden_dense()
    moe_case(ref_utils, "softmax_top2", 200, T=5, E=8, topk=2, H=128, I=64, dtype=torch.bfloat16,
             score_func="softmax", groups=1, topk_group=1, use_bias=False, fp8=False)
    moe_case(ref_utils, "sigmoid_grouped_bias", 201, T=7, E=16, topk=4, H=128, I=64, dtype=torch.bfloat16,
             score_func="sigmoid", groups=4, topk_group=2, use_bias=True, fp8=False)
    moe_case(ref_utils, "fp16_softmax", 202, T=3, E=8, topk=2, H=64, I=32, dtype=torch.float16,
             score_func="softmax", groups=1, topk_group=1, use_bias=False, fp8=False, renorm=False)
    moe_case(ref_utils, "fp8_top8", 203, T=4, E=32, topk=8, H=128, I=128, dtype=torch.bfloat16,
             score_func="softmax", groups=1, topk_group=1, use_bias=False, fp8=True)
    for f in sorted(HERE.iterdir()):
        print(f.name, f.stat().st_size)


if __name__ == "__main__":
    main()
