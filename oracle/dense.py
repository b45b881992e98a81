"""TEST INFRASTRUCTURE -- CPU oracle for GeMV / narrow GEMM / soft-FP8 dequantisation.

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline leg may import this package.

The reference checks its dense kernels against its vendor GEMM (csrc/gemm_ex.cu:33-58: C[n,m] = alpha * B A^T,
fp32 compute for bf16, csrc/utils.cuh:125-127), whose source is not in the tree; bias is added afterwards by the
benchmark scripts (benchmark_and_test/gemv_benchmark.py:41).  The math is restated here with torch on the
un-permuted weight: fp32 product, one rounding to the 16-bit output type.  Parity for the dense path is
"unpinned" in the sense that the reference holds no stored expected outputs for it (it prints max-abs-diff
against the vendor GEMM and never asserts, gemv_benchmark.py:79-106); what pins this file are the golden
vectors of tests/golden/ (generated with the reference's layout recipes and its scale_tensor helper).
"""
from __future__ import annotations

from typing import Optional

import torch

BLOCK = 128


def gemm_ref(X: torch.Tensor, W: torch.Tensor, alpha: float = 1.0, bias: Optional[torch.Tensor] = None,
             out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """C[n,m] = alpha * X[n,k] W[m,k]^T (+ bias[m]) in fp32, rounded once to `out_dtype` (default X.dtype)."""
    out_dtype = out_dtype or X.dtype
    acc = X.to(torch.float32) @ W.to(torch.float32).t()
    acc = acc * alpha
    if bias is not None:
        acc = acc + bias.to(torch.float32).reshape(1, -1)
    return acc.to(out_dtype)


def gemm_ref_f64(X: torch.Tensor, W: torch.Tensor, alpha: float = 1.0, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Same product in float64, not rounded: the yardstick for "which of two 16-bit results is closer"."""
    acc = X.to(torch.float64) @ W.to(torch.float64).t() * alpha
    if bias is not None:
        acc = acc + bias.to(torch.float64).reshape(1, -1)
    return acc


def dequant_block_scaled(W8: torch.Tensor, scale: Optional[torch.Tensor]) -> torch.Tensor:
    """e4m3 weight [m,k] (+ fp32 [ceil(m/128), ceil(k/128)] block scales) -> bf16, following the reference helper
    scale_tensor (muxi_layout_kernels/utils.py:14-25): the bf16 weight block is multiplied in place by a 0-dim fp32
    tensor, which torch evaluates as one fp32 product with the unrounded factor, rounded once to bf16 (checked
    against the imported reference function; pinned by tests/golden/dequant_*.pt).
    Without scales the conversion e4m3 -> bf16 is exact."""
    w = W8.to(torch.bfloat16)
    if scale is None:
        return w
    m, k = w.shape
    full = scale.repeat_interleave(BLOCK, dim=0)[:m].repeat_interleave(BLOCK, dim=1)[:, :k]
    return _mul_like_reference(w, full)


def _mul_like_reference(w_bf16: torch.Tensor, scale_full_f32: torch.Tensor) -> torch.Tensor:
    return (w_bf16.to(torch.float32) * scale_full_f32.to(torch.float32)).to(torch.bfloat16)


def dequant_exact_scale(W8: torch.Tensor, scale: Optional[torch.Tensor]) -> torch.Tensor:
    """fp32 weight times the *unrounded* fp32 block scale, no rounding: what the CUDA kernels effectively use
    (they apply the scale to the fp32 partial sums of each 128-wide K block)."""
    w = W8.to(torch.float32)
    if scale is None:
        return w
    m, k = w.shape
    full = scale.repeat_interleave(BLOCK, dim=0)[:m].repeat_interleave(BLOCK, dim=1)[:, :k]
    return w * full


def error_report(got: torch.Tensor, want: torch.Tensor, atol: float = 1e-2, rtol: float = 1e-2,
                 scale_atol: bool = False) -> dict:
    """Combined-tolerance check |got - want| <= atol + rtol * |want| plus the raw figures (max abs, max rel over
    non-tiny entries).  scale_atol=True multiplies atol by max(1, rms(want)): used where outputs are far larger
    than 1 (soft-FP8 MoE outputs reach 1e3, where one bf16 ulp is already 4-8)."""
    g = got.to(torch.float64).flatten()
    w = want.to(torch.float64).flatten()
    diff = (g - w).abs()
    if scale_atol and w.numel():
        atol = atol * max(1.0, float(w.pow(2).mean().sqrt()))
    tol = atol + rtol * w.abs()
    big = w.abs() >= 1e-2 * max(float(w.abs().max()), 1e-30)
    rel = (diff[big] / w.abs()[big]).max().item() if bool(big.any()) else 0.0
    return {
        "ok": bool((diff <= tol).all()),
        "max_abs": float(diff.max()) if diff.numel() else 0.0,
        "max_rel": float(rel),
        "worst_excess": float((diff - tol).max()) if diff.numel() else 0.0,
        "n": int(diff.numel()),
    }
