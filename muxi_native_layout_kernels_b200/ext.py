"""Operator surface of the reference extension module ``muxi_layout_kernels_ext`` (csrc/ffi.cu:32-144).

Same function names, argument names, defaults, return conventions and error behaviour (a violated
precondition raises ``RuntimeError``).  Each function checks its tensors, allocates the result with torch,
looks up the current CUDA stream and calls the C-ABI library; nothing is computed in Python or by torch.

Extensions over the reference surface (all optional, defaults keep reference behaviour):
  * ``layoutA`` / ``layoutA_inverse`` device ops (the reference builds layout A with view/permute in Python);
  * ``fp8_repacked=`` keyword on the soft-FP8 ops, for weights that went through ``fp8_weight_repack``.
"""
from __future__ import annotations

from typing import List, Optional

import torch

import ctypes

from ._lib import MlkAux, MlkError, check, lib

__all__ = [
    "set_static_weights", "set_pdl", "set_full_scales", "kernel_status",
    "layoutA", "layoutA_inverse", "layoutB", "reLayoutC", "fp8_weight_repack",
    "gemv_layoutA", "gemv_layoutA_wapper",
    "gemm_layoutA", "gemm_layoutA_wapper", "gemm_layoutA_soft_fp8", "gemm_layoutA_soft_fp8_wapper",
    "gemm_layoutA_linear", "gemm_layoutAB_ContinuousC", "gemm_layoutAB_ContinuousC_wapper",
    "gemm_layoutABC", "gemm_layoutABC_wapper",
    "fused_routing_gate", "fused_router_gemm_gate", "batched_routed_activation_indexed_to_expert_block_indexed",
    "fused_experts_compute",
    "gemmEx", "muxi_hgemm", "muxi_hgemm_layout", "muxi_hgemm_layoutA", "muxi_hgemm_layoutC", "routing_gate",
    "experts_compute", "MlkError",
]

_FP8_DTYPES = tuple(getattr(torch, n) for n in ("float8_e4m3fn", "uint8", "int8") if hasattr(torch, n))


def set_static_weights(enabled: bool) -> None:
    """Promise that weight tensors are not written by kernels of the calling stream while ops of this library are
    in flight (weights prepacked once, then only read).  The dense kernels then begin streaming weights while the
    preceding kernel is still draining.  Off by default."""
    check(lib.mlk_set_option(1, int(bool(enabled))))


def set_full_scales(enabled: bool) -> None:
    """How the tcgen05 e4m3 kernels apply 128x128 block scales: False (default) rounds the scale to bf16 and folds it
    into the decode at no cost; True keeps 16 significant bits of the scale (two more packed instructions per weight
    pair; the result is the weight the reference's torch recipe dequantises to, rne_bf16(w * s))."""
    check(lib.mlk_set_option(2, int(bool(enabled))))


def set_pdl(enabled: bool) -> None:
    """Programmatic dependent launch for all kernels of this library (on by default)."""
    check(lib.mlk_set_option(0, int(bool(enabled))))


def _chk(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _cuda_contig(t: torch.Tensor, name: str) -> None:
    _chk(t.is_cuda, f"{name} must be a CUDA tensor")
    _chk(t.is_contiguous(), f"{name} must be contiguous")


def _act_code(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return 0
    if t.dtype == torch.float16:
        return 1
    raise RuntimeError("Unsupported data type")


def _dense_code(A: torch.Tensor, B: torch.Tensor) -> int:
    """dtype code of a dense op: 16-bit weights must match the activations; 1-byte weights need bf16 activations
    (reference: csrc/gemv_layout_a.cu:30-66)."""
    if A.element_size() == 1:
        _chk(B.dtype == torch.bfloat16, "Unsupported data type")
        return 2
    _chk(A.dtype == B.dtype, "A and B must have the same data type")
    return _act_code(B)


def _layoutA_dims(A: torch.Tensor):
    _chk(A.dim() == 4, "A must be a 4D tensor")
    _chk(A.size(2) == 16, "A.shape[2] must be 16")
    _chk(A.size(3) == 8, "A.shape[3] must be 8")
    return A.size(0) * 16, A.size(1) * 8


def _layoutB_dims(B: torch.Tensor):
    _chk(B.dim() == 5, "B must be a 5D tensor")
    _chk(B.size(2) == 4 and B.size(3) == 16 and B.size(4) == 8, "B trailing dims must be (4, 16, 8)")
    return B.size(1) * 16, B.size(0) * 32


def _bias_ptr(bias: Optional[torch.Tensor], like: torch.Tensor, m: int):
    if bias is None:
        return None
    _cuda_contig(bias, "bias")
    _chk(bias.dtype == like.dtype, "bias must have the activation data type")
    _chk(bias.numel() == m, "bias must hold m elements")
    return bias.data_ptr()


def _scale_ptr(scale: Optional[torch.Tensor], m: int, k: int):
    if scale is None:
        return None
    _cuda_contig(scale, "scale_matrix")
    _chk(scale.dtype == torch.float32, "scale_matrix must be float32")
    _chk(scale.numel() == ((m + 127) // 128) * ((k + 127) // 128), "scale_matrix must be [ceil(m/128), ceil(k/128)]")
    return scale.data_ptr()


# ---------------------------------------------------------------------------------------------------
# prepack ops
# ---------------------------------------------------------------------------------------------------

def layoutA(W: torch.Tensor) -> torch.Tensor:
    """``W[m,k]`` -> layout A ``[m/16, k/8, 16, 8]`` (= ``W.view(m/16,16,k/8,8).permute(0,2,1,3)``,
    benchmark_and_test/gemm_benchmark.py:41-42).  3-D input ``[E,m,k]`` is converted expert by expert and keeps
    its shape, like the MoE weight loop of benchmark_and_test/test_muxi_moe.py:73-81."""
    _cuda_contig(W, "W")
    _chk(W.dim() in (2, 3), "W must be a 2D or 3D tensor")
    _chk(W.element_size() in (1, 2), "Unsupported data type")
    m, k = W.shape[-2], W.shape[-1]
    _chk(m % 16 == 0 and k % 8 == 0, "layoutA needs m % 16 == 0 and k % 8 == 0")
    batch = W.shape[0] if W.dim() == 3 else 1
    out = torch.empty_like(W) if W.dim() == 3 else torch.empty((m // 16, k // 8, 16, 8), dtype=W.dtype, device=W.device)
    # consecutive experts are consecutive 16-row groups of one [batch*m, k] matrix
    check(lib.mlk_layoutA(W.data_ptr(), out.data_ptr(), batch * m, k, W.element_size(), 0, _stream(W)))
    return out


def layoutA_inverse(A: torch.Tensor) -> torch.Tensor:
    """Layout A ``[m/16, k/8, 16, 8]`` -> ``W[m,k]``."""
    _cuda_contig(A, "A")
    m, k = _layoutA_dims(A)
    out = torch.empty((m, k), dtype=A.dtype, device=A.device)
    check(lib.mlk_layoutA(A.data_ptr(), out.data_ptr(), m, k, A.element_size(), 1, _stream(A)))
    return out


def layoutB(B: torch.Tensor) -> torch.Tensor:
    """``B[n,k]`` -> ``[k/32, n/16, 4, 16, 8]`` (csrc/layout_b.cu:65-99)."""
    _cuda_contig(B, "B")
    _chk(B.dim() == 2, "B must be a 2D tensor")
    n, k = B.shape
    _chk(n % 16 == 0, "n must be a multiple of 16")
    _chk(k % 32 == 0, "k must be a multiple of 32")
    _act_code(B)
    out = torch.empty((k // 32, n // 16, 4, 16, 8), dtype=B.dtype, device=B.device)
    check(lib.mlk_layoutB(B.data_ptr(), out.data_ptr(), n, k, _stream(B)))
    return out


def reLayoutC(C_in: torch.Tensor) -> torch.Tensor:
    """``[m/32, n/16, 4, 16, 8]`` -> ``C[n,m]`` (csrc/re_layout_c.cu:63-95)."""
    _cuda_contig(C_in, "C_in")
    _chk(C_in.dim() == 5, "C_in must be a 5D tensor")
    _chk(C_in.size(2) == 4, "C_in.shape[2] must be 4")
    _chk(C_in.size(3) == 16, "C_in.shape[3] must be 16")
    _chk(C_in.size(4) == 8, "C_in.shape[4] must be 8")
    _act_code(C_in)
    m, n = C_in.size(0) * 32, C_in.size(1) * 16
    out = torch.empty((n, m), dtype=C_in.dtype, device=C_in.device)
    check(lib.mlk_reLayoutC(C_in.data_ptr(), out.data_ptr(), m, n, _stream(C_in)))
    return out


def fp8_weight_repack(weight: torch.Tensor) -> torch.Tensor:
    """Swaps bytes 1 and 2 of every 32-bit word of a 2-D or 3-D e4m3 tensor; shape preserved
    (csrc/fp8_weight_repack.cu:44-67).  Applying it twice gives the input back."""
    _cuda_contig(weight, "weight")
    _chk(weight.element_size() == 1, "weight must be a 1-byte (e4m3) tensor")
    _chk(weight.dim() in (2, 3, 4), "weight must be a 2D or 3D tensor")
    out = torch.empty_like(weight)
    check(lib.mlk_fp8_weight_repack(weight.data_ptr(), out.data_ptr(), weight.numel(), _stream(weight)))
    return out


# ---------------------------------------------------------------------------------------------------
# GeMV
# ---------------------------------------------------------------------------------------------------

def _gemv_checks(A, B, scale_matrix, bias):
    _chk(A.is_cuda, "A must be a CUDA tensor")
    _chk(B.is_cuda, "B must be a CUDA tensor")
    _chk(A.is_contiguous(), "A must be contiguous")
    _chk(B.is_contiguous(), "B must be contiguous")
    m, A_k = _layoutA_dims(A)
    _chk(B.dim() == 2 and B.size(0) == 1, "B must be a vector")
    _chk(A_k == B.size(1), "A and B must have the same k")
    _chk(m % 16 == 0, "GEMV m % 16(at least) must be 0")
    _chk(A_k % 32 == 0, "GEMV k % 32(at least) must be 0")
    code = _dense_code(A, B)
    _chk(code == 2 or scale_matrix is None, "scale_matrix needs 1-byte weights")
    return m, A_k, code


def gemv_layoutA(A, B, alpha: float = 1, beta: float = 0, scale_matrix=None, bias=None, *, fp8_repacked: bool = False):
    """``y[1,m] = alpha * A x (+ bias)``; table-driven (csrc/gemv_layout_a.cu:73-150).  ``beta`` is ignored, as by
    the reference kernels.  For e4m3 weights ``scale_matrix=None`` means unit scales."""
    m, k, code = _gemv_checks(A, B, scale_matrix, bias)
    C = torch.empty((1, m), dtype=B.dtype, device=B.device)
    aux, _keep = _aux(B, m, 1, k, stream_k=False)
    check(lib.mlk_gemv_layoutA(A.data_ptr(), B.data_ptr(), C.data_ptr(), m, k, code, alpha, beta,
                               _scale_ptr(scale_matrix, m, k), _bias_ptr(bias, B, m), int(fp8_repacked),
                               ctypes.byref(aux), _stream(B)))
    return C


def gemv_layoutA_wapper(A, B, m: int, k: int, alpha: float = 1, beta: float = 0, blockDimX: int = 256,
                        kernelId: int = 1, kernelParam1: int = 1, kernelParam2: int = 1, scale_matrix=None, bias=None,
                        *, fp8_repacked: bool = False):
    """Tuner hook with explicit launch arguments (csrc/gemv_layout_a.cu:17-71)."""
    m2, k2, code = _gemv_checks(A, B, scale_matrix, bias)
    _chk(m == m2 and k == k2, "m, k do not match the tensors")
    C = torch.empty((1, m), dtype=B.dtype, device=B.device)
    aux, _keep = _aux(B, m, 1, k, stream_k=False)
    check(lib.mlk_gemv_layoutA_wapper(A.data_ptr(), B.data_ptr(), C.data_ptr(), m, k, code, alpha, beta, blockDimX,
                                      kernelId, kernelParam1, kernelParam2, _scale_ptr(scale_matrix, m, k),
                                      _bias_ptr(bias, B, m), int(fp8_repacked), ctypes.byref(aux), _stream(B)))
    return C


# ---------------------------------------------------------------------------------------------------
# narrow GEMM
# ---------------------------------------------------------------------------------------------------

def _gemm_checks(A, B, b_layout: bool):
    _chk(A.is_cuda, "A must be a CUDA tensor")
    _chk(B.is_cuda, "B must be a CUDA tensor")
    _chk(A.is_contiguous(), "A must be contiguous")
    _chk(B.is_contiguous(), "B must be contiguous")
    m, A_k = _layoutA_dims(A)
    if b_layout:
        n, B_k = _layoutB_dims(B)
    else:
        _chk(B.dim() == 2, "B must be a 2D tensor")
        n, B_k = B.shape
    _chk(A_k == B_k, "A and B must have the same k")
    _chk(m % 128 == 0, "m must be a multiple of 128")
    _chk(A_k % 128 == 0, "k must be a multiple of 128")
    return m, n, A_k


_SYNC_BUFFERS = {}   # (device index, stream handle) -> [counters, status, workspace, MlkAux]
_WS_BYTES = {}       # (device index, m, n-tile, k) -> workspace bytes of the tcgen05 kernel
_MIN_WS_FLOATS = 1 << 20
_RETIRED = []        # workspaces replaced during a stream capture: CUDA graphs may still reference them


def _stream_bufs(device: torch.device, stream: int, tiles: int = 0):
    key = (device.index, stream)
    bufs = _SYNC_BUFFERS.get(key)
    if bufs is None or bufs[0].numel() < tiles:
        bufs = [torch.zeros(max(4096, tiles), dtype=torch.int32, device=device),
                torch.zeros(1, dtype=torch.int32, device=device) if bufs is None else bufs[1],
                None if bufs is None else bufs[2], None]
        _SYNC_BUFFERS[key] = bufs
    return bufs


def _status_ptr(t: torch.Tensor) -> int:
    """Device address of the sticky status word of the current stream of `t`'s device."""
    return _stream_bufs(t.device, _stream(t))[1].data_ptr()


def _aux(B: torch.Tensor, m: int, n: int, k: int, stream_k: bool = True):
    """Scratch lent to the tcgen05 kernels, kept per (device, stream): a block of counters that every kernel leaves
    zeroed, the sticky status word of the kernels' bounded waits, and an fp32 workspace that only grows (partial tiles
    of the persistent stream-K grid; per-token scales of the native-FP8 kernels).  Successive launches of one stream
    may share it: a kernel touches it only after the preceding kernel of the stream has completed
    (griddepcontrol.wait), and kernels of one stream never run concurrently otherwise; another stream gets its own.
    A CUDA graph captures these addresses: replay graphs that were captured on the same stream one at a time.
    stream_k=False: the call cannot use the persistent stream-K grid (e4m3 weights, GeMV) and needs no more than the
    minimum workspace.  Returns (MlkAux, tensor that keeps the workspace alive)."""
    stream = _stream(B)
    bufs = _stream_bufs(B.device, stream, m // 128)
    nbytes = 0
    if not stream_k:
        nbytes = 1024 + 2 * k * min(n, 64)       # what mlk_soft_fp8_workspace_bytes(n, k) reports
    elif n <= 64 and m % 128 == 0 and k % 64 == 0:
        npad = 16 if n <= 16 else (32 if n <= 32 else 64)
        wkey = (B.device.index, m, npad, k)
        nbytes = _WS_BYTES.get(wkey)
        if nbytes is None:
            with torch.cuda.device(B.device):
                nbytes = _WS_BYTES[wkey] = int(lib.mlk_gemm_workspace_bytes(m, n, k))
    ws = bufs[2]
    if ws is None or ws.numel() * 4 < nbytes:
        # the old buffer may still be in use by kernels already queued on this stream: torch's allocator keeps a freed
        # block stream-ordered, so dropping the reference here is safe -- except while the stream is being captured:
        # graphs captured earlier hold the old address, so the old buffer is then kept alive for good
        if ws is not None and torch.cuda.is_current_stream_capturing():
            _RETIRED.append(ws)
        ws = bufs[2] = torch.empty(max(nbytes // 4, _MIN_WS_FLOATS), dtype=torch.float32, device=B.device)
        bufs[3] = None
    if bufs[3] is None:
        bufs[3] = MlkAux(ws.data_ptr(), ws.numel() * 4, bufs[0].data_ptr(), bufs[0].numel(), bufs[1].data_ptr())
    return bufs[3], ws


def kernel_status(device=None, reset: bool = False) -> int:
    """Sticky status word of the bounded waits inside the tcgen05 kernels for the current stream of `device`
    (0 = no wait ever expired).  Synchronises the stream.  A kernel that gave up leaves its output unwritten and, in
    the persistent stream-K mode, may leave tile counters behind; ``reset=True`` clears the word and the counters so
    that the stream can be used again."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = (dev.index if dev.index is not None else torch.cuda.current_device(), torch.cuda.current_stream(dev).cuda_stream)
    bufs = _SYNC_BUFFERS.get(key)
    if bufs is None:
        return 0
    value = int(bufs[1].item())
    if reset and value != 0:
        bufs[0].zero_()
        bufs[1].zero_()
    return value


def _alloc_c(B, m, n, c_layout: bool):
    if c_layout:
        return torch.empty((m // 32, n // 16, 4, 16, 8), dtype=B.dtype, device=B.device)
    return torch.empty((n, m), dtype=B.dtype, device=B.device)


def gemm_layoutA(A, B, alpha: float = 1, beta: float = 0, bias=None):
    """``C[n,m] = alpha * B A^T (+ bias)``, A layout A, B and C row-major (csrc/gemm_layout_A.cu:752-787)."""
    m, n, k = _gemm_checks(A, B, False)
    code = _dense_code(A, B)
    _chk(code != 2, "Unsupported data type")
    C = _alloc_c(B, m, n, False)
    aux, _keep = _aux(B, m, n, k)
    check(lib.mlk_gemm_layoutA(A.data_ptr(), B.data_ptr(), C.data_ptr(), m, n, k, code, alpha, beta,
                               _bias_ptr(bias, B, m), ctypes.byref(aux), _stream(B)))
    return C


def gemm_layoutA_wapper(A, B, m: int, n: int, k: int, alpha: float = 1, beta: float = 0, kernelParam1: int = 1,
                        kernelParam2: int = 1, kernelParam3: int = 1, kernelId: int = 1, bias=None):
    """Tuner hook (csrc/gemm_layout_A.cu:684-750)."""
    m2, n2, k2 = _gemm_checks(A, B, False)
    _chk((m, n, k) == (m2, n2, k2), "m, n, k do not match the tensors")
    code = _dense_code(A, B)
    _chk(code != 2, "Unsupported data type")
    C = _alloc_c(B, m, n, False)
    aux, _keep = _aux(B, m, n, k)
    check(lib.mlk_gemm_layoutA_wapper(A.data_ptr(), B.data_ptr(), C.data_ptr(), m, n, k, code, alpha, beta,
                                      kernelParam1, kernelParam2, kernelParam3, kernelId, _bias_ptr(bias, B, m),
                                      ctypes.byref(aux), _stream(B)))
    return C


def gemm_layoutA_soft_fp8(A, A_Scale, B, alpha: float = 1, beta: float = 0, bias=None, *, fp8_repacked: bool = False):
    """e4m3 A with fp32 128x128 block scales, bf16 B/C (csrc/gemm_layout_A_soft_fp8.cu:825).  ``A_Scale=None``
    means unit scales."""
    m, n, k = _gemm_checks(A, B, False)
    _chk(_dense_code(A, B) == 2, "Unsupported data type")
    C = _alloc_c(B, m, n, False)
    aux, _keep = _aux(B, m, n, k, stream_k=False)
    check(lib.mlk_gemm_layoutA_soft_fp8(A.data_ptr(), _scale_ptr(A_Scale, m, k), B.data_ptr(), C.data_ptr(), m, n, k,
                                        alpha, beta, _bias_ptr(bias, B, m), int(fp8_repacked), ctypes.byref(aux),
                                        _stream(B)))
    return C


def gemm_layoutA_soft_fp8_wapper(A, A_Scale, B, m: int, n: int, k: int, alpha: float = 1, beta: float = 0,
                                 kernelParam1: int = 1, kernelParam2: int = 1, kernelParam3: int = 1,
                                 kernelId: int = 1, bias=None, *, fp8_repacked: bool = False):
    """Tuner hook (csrc/gemm_layout_A_soft_fp8.cu:749)."""
    m2, n2, k2 = _gemm_checks(A, B, False)
    _chk((m, n, k) == (m2, n2, k2), "m, n, k do not match the tensors")
    _chk(_dense_code(A, B) == 2, "Unsupported data type")
    C = _alloc_c(B, m, n, False)
    aux, _keep = _aux(B, m, n, k, stream_k=False)
    check(lib.mlk_gemm_layoutA_soft_fp8_wapper(A.data_ptr(), _scale_ptr(A_Scale, m, k), B.data_ptr(), C.data_ptr(),
                                               m, n, k, alpha, beta, kernelParam1, kernelParam2, kernelParam3,
                                               kernelId, _bias_ptr(bias, B, m), int(fp8_repacked), ctypes.byref(aux),
                                               _stream(B)))
    return C


def gemm_layoutA_linear(A, B, alpha: float = 1, beta: float = 0, scale_matrix=None, bias=None):
    """Routes on the presence of ``scale_matrix`` (csrc/gemm_layoutA_linear.cu:8-19)."""
    if scale_matrix is not None:
        return gemm_layoutA_soft_fp8(A, scale_matrix, B, alpha, beta, bias)
    return gemm_layoutA(A, B, alpha, beta, bias)


def muxi_hgemm_layoutA(A, B, alpha: float = 1, beta: float = 0, scale_matrix=None, bias=None, *, fp8_repacked: bool = False):
    """``C[n,m] = alpha * B A^T (+ bias)`` for any token count n, A in layout A (16-bit, or e4m3 with optional 128x128
    block scales), B and C row-major (csrc/muxi_hgemm_layoutA.cu:12-217): the prefill-side consumer of the weights the
    GeMV / narrow-GEMM operators stream.  ``beta`` is ignored (the reference applies it to its own uninitialised C)."""
    _chk(A.is_cuda, "A must be a CUDA tensor")
    _chk(B.is_cuda, "B must be a CUDA tensor")
    _chk(A.is_contiguous(), "A must be contiguous")
    _chk(B.is_contiguous(), "B must be contiguous")
    m, A_k = _layoutA_dims(A)
    _chk(B.dim() == 2, "B must be a 2D tensor")
    n, B_k = B.shape
    _chk(A_k == B_k, "A and B must have the same k")
    _chk(m % 128 == 0, "m must be a multiple of 128")
    _chk(A_k % 128 == 0, "k must be a multiple of 128")
    code = _dense_code(A, B)
    _chk(code == 2 or scale_matrix is None, "scale_matrix needs 1-byte weights")
    C = torch.empty((n, m), dtype=B.dtype, device=B.device)
    aux, _keep = _aux(B, m, min(n, 64), A_k, stream_k=(code != 2))
    check(lib.mlk_muxi_hgemm_layoutA(A.data_ptr(), _scale_ptr(scale_matrix, m, A_k), B.data_ptr(), C.data_ptr(), m, n, A_k,
                                     code, alpha, beta, _bias_ptr(bias, B, m), int(fp8_repacked), ctypes.byref(aux),
                                     _stream(B)))
    return C


def gemm_layoutAB_ContinuousC(A, B, alpha: float = 1, beta: float = 0, bias=None):
    """A layout A, B layout B (from ``layoutB``), C row-major (csrc/gemm_layout_ab_continuous_c.cu:1051)."""
    m, n, k = _gemm_checks(A, B, True)
    code = _dense_code(A, B)
    _chk(code != 2, "Unsupported data type")
    C = _alloc_c(B, m, n, False)
    aux, _keep = _aux(B, m, n, k)
    check(lib.mlk_gemm_layoutAB_ContinuousC(A.data_ptr(), B.data_ptr(), C.data_ptr(), m, n, k, code, alpha, beta,
                                            _bias_ptr(bias, B, m), ctypes.byref(aux), _stream(B)))
    return C


def gemm_layoutAB_ContinuousC_wapper(A, B, m: int, n: int, k: int, alpha: float = 1, beta: float = 0,
                                     kernelParam1: int = 1, kernelParam2: int = 1, kernelParam3: int = 1,
                                     kernelId: int = 1, bias=None):
    """Tuner hook (csrc/gemm_layout_ab_continuous_c.cu:982)."""
    m2, n2, k2 = _gemm_checks(A, B, True)
    _chk((m, n, k) == (m2, n2, k2), "m, n, k do not match the tensors")
    code = _dense_code(A, B)
    _chk(code != 2, "Unsupported data type")
    C = _alloc_c(B, m, n, False)
    aux, _keep = _aux(B, m, n, k)
    check(lib.mlk_gemm_layoutAB_ContinuousC_wapper(A.data_ptr(), B.data_ptr(), C.data_ptr(), m, n, k, code, alpha,
                                                   beta, kernelParam1, kernelParam2, kernelParam3, kernelId,
                                                   _bias_ptr(bias, B, m), ctypes.byref(aux), _stream(B)))
    return C


def gemm_layoutABC(A, B, alpha: float = 1, beta: float = 0, bias=None):
    """A layout A, B layout B, result in layout C ``[m/32, n/16, 4, 16, 8]`` (csrc/gemm_layout_abc.cu:754)."""
    m, n, k = _gemm_checks(A, B, True)
    code = _dense_code(A, B)
    _chk(code != 2, "Unsupported data type")
    C = _alloc_c(B, m, n, True)
    aux, _keep = _aux(B, m, n, k)
    check(lib.mlk_gemm_layoutABC(A.data_ptr(), B.data_ptr(), C.data_ptr(), m, n, k, code, alpha, beta,
                                 _bias_ptr(bias, B, m), ctypes.byref(aux), _stream(B)))
    return C


def gemm_layoutABC_wapper(A, B, m: int, n: int, k: int, alpha: float = 1, beta: float = 0, kernelParam1: int = 1,
                          kernelParam2: int = 1, kernelParam3: int = 1, kernelId: int = 1, bias=None):
    """Tuner hook (csrc/gemm_layout_abc.cu:685)."""
    m2, n2, k2 = _gemm_checks(A, B, True)
    _chk((m, n, k) == (m2, n2, k2), "m, n, k do not match the tensors")
    code = _dense_code(A, B)
    _chk(code != 2, "Unsupported data type")
    C = _alloc_c(B, m, n, True)
    aux, _keep = _aux(B, m, n, k)
    check(lib.mlk_gemm_layoutABC_wapper(A.data_ptr(), B.data_ptr(), C.data_ptr(), m, n, k, code, alpha, beta,
                                        kernelParam1, kernelParam2, kernelParam3, kernelId, _bias_ptr(bias, B, m),
                                        ctypes.byref(aux), _stream(B)))
    return C


# ---------------------------------------------------------------------------------------------------
# fused MoE
# ---------------------------------------------------------------------------------------------------

def fused_router_gemm_gate(hidden_states, gate_weight, score_fun: int, n_groups: int, topK_groups: int, experts_ids,
                           selected_experts_weights, topK: int, load_balance_bias=None, *, renormalize: bool = False,
                           logits_out=None) -> None:
    """Router GEMM fused with the routing: ``logits = hidden_states @ gate_weight.T`` (fp32 sums rounded once to the
    activation dtype) followed by ``fused_routing_gate``; writes ``experts_ids`` and ``selected_experts_weights`` in
    place and, if given, the rounded logits into ``logits_out`` [T, E].  No counterpart in the reference, whose layer
    starts from ``gating_output``; meant for decode batches."""
    _cuda_contig(hidden_states, "hidden_states")
    _cuda_contig(gate_weight, "gate_weight")
    _cuda_contig(experts_ids, "experts_ids")
    _cuda_contig(selected_experts_weights, "selected_experts_weights")
    _chk(hidden_states.dim() == 2 and gate_weight.dim() == 2 and hidden_states.size(1) == gate_weight.size(1),
         "hidden_states [T, H] and gate_weight [E, H] must share H")
    _chk(gate_weight.dtype == hidden_states.dtype and selected_experts_weights.dtype == hidden_states.dtype,
         "hidden_states, gate_weight and selected_experts_weights must have the same data type.")
    _chk(experts_ids.dtype == torch.int32, "experts_ids must be of type torch::kInt32.")
    T, H = hidden_states.shape
    E = gate_weight.size(0)
    _chk(experts_ids.numel() == T * topK and selected_experts_weights.numel() == T * topK,
         "experts_ids / selected_experts_weights must be [batch_size, topK]")
    code = _act_code(hidden_states)
    if load_balance_bias is not None:
        _cuda_contig(load_balance_bias, "load_balance_bias")
        _chk(load_balance_bias.dtype == hidden_states.dtype and load_balance_bias.numel() == E,
             "load_balance_bias must be [E] in the gating dtype")
    if logits_out is not None:
        _cuda_contig(logits_out, "logits_out")
        _chk(logits_out.dtype == hidden_states.dtype and tuple(logits_out.shape) == (T, E), "logits_out must be [T, E]")
    check(lib.mlk_fused_router_gemm_gate(hidden_states.data_ptr(), gate_weight.data_ptr(), score_fun, T, H, E, n_groups,
                                         topK_groups, experts_ids.data_ptr(), selected_experts_weights.data_ptr(), topK,
                                         None if load_balance_bias is None else load_balance_bias.data_ptr(), code,
                                         int(bool(renormalize)), None if logits_out is None else logits_out.data_ptr(),
                                         _stream(hidden_states)))


def fused_routing_gate(gating_output, score_fun: int, batch_size: int, hidden_size: int, n_groups: int,
                       topK_groups: int, experts_ids, selected_experts_weights, topK: int,
                       load_balance_bias=None, *, renormalize: bool = False) -> None:
    """Router: softmax (0) / sigmoid (1) + optional bias + group-limited top-k; writes ``experts_ids`` (int32) and
    ``selected_experts_weights`` in place (csrc/moe_kernels/fused_gating.cu:5-67).  ``hidden_size`` is unused, as
    in the reference.  Extension: ``renormalize=True`` also divides every token's weights by their sum (in the logits'
    dtype), which saves the two torch ops the reference orchestrator spends on it."""
    _cuda_contig(gating_output, "gating_output")
    _cuda_contig(experts_ids, "experts_ids")
    _cuda_contig(selected_experts_weights, "selected_experts_weights")
    _chk(gating_output.dim() == 2 and gating_output.size(0) == batch_size, "gating_output must be [batch_size, E]")
    _chk(experts_ids.dtype == torch.int32, "experts_ids must be of type torch::kInt32.")
    _chk(selected_experts_weights.dtype == gating_output.dtype,
         "gating_output and selected_experts_weights must have the same data type.")
    _chk(experts_ids.numel() == batch_size * topK and selected_experts_weights.numel() == batch_size * topK,
         "experts_ids / selected_experts_weights must be [batch_size, topK]")
    code = _act_code(gating_output)
    E = gating_output.size(1)
    if load_balance_bias is not None:
        _cuda_contig(load_balance_bias, "load_balance_bias")
        _chk(load_balance_bias.dtype == gating_output.dtype and load_balance_bias.numel() == E,
             "load_balance_bias must be [E] in the gating dtype")
    check(lib.mlk_fused_routing_gate_renorm(gating_output.data_ptr(), score_fun, batch_size, E, n_groups, topK_groups,
                                            experts_ids.data_ptr(), selected_experts_weights.data_ptr(), topK,
                                            _ptr(load_balance_bias), code, int(bool(renormalize)),
                                            _stream(gating_output)))


def _map_args(experts_map):
    if experts_map is None:
        return None, 0
    _cuda_contig(experts_map, "experts_map")
    _chk(experts_map.dtype == torch.int32, "experts_map must be of type torch::kInt32.")
    return experts_map.data_ptr(), experts_map.numel()


def batched_routed_activation_indexed_to_expert_block_indexed(batchSize: int, expertCount: int, topK: int,
                                                              microBatchSize: int, expertsIds, dev_sorted_token_ids,
                                                              dev_cumsum_buffer, dev_padded_num_experts,
                                                              dev_experts_ids, experts_map=None) -> None:
    """Token alignment (csrc/moe_kernels/fused_experts_compute.cu:6-48); all outputs are written in place."""
    for t, name in ((expertsIds, "expertsIds"), (dev_sorted_token_ids, "dev_sorted_token_ids"),
                    (dev_cumsum_buffer, "dev_cumsum_buffer"), (dev_padded_num_experts, "dev_padded_num_experts"),
                    (dev_experts_ids, "dev_experts_ids")):
        _cuda_contig(t, name)
        _chk(t.dtype == torch.int32, f"{name} must be of type torch::kInt32.")
    _chk(expertsIds.numel() == batchSize * topK, "expertsIds must be [batchSize, topK]")
    _chk(dev_sorted_token_ids.numel() >= batchSize * topK + expertCount * (microBatchSize - 1),
         "dev_sorted_token_ids is too small")
    _chk(dev_cumsum_buffer.numel() >= expertCount + 1, "dev_cumsum_buffer is too small")
    mp, ml = _map_args(experts_map)
    check(lib.mlk_moe_align(batchSize, expertCount, topK, microBatchSize, expertsIds.data_ptr(),
                            dev_sorted_token_ids.data_ptr(), dev_cumsum_buffer.data_ptr(),
                            dev_padded_num_experts.data_ptr(), dev_experts_ids.data_ptr(), mp, ml,
                            _stream(expertsIds)))


def fused_experts_compute(experts_weights_matrix1, experts_weights_matrix2, activations, batch_size: int,
                          expert_count: int, dynamic_experts_per_act: int, topk_ids, actived_experts_weights,
                          sorted_token_ids, cumsum_buffer, padded_num_experts, experts_ids, C, y, *args, **kwargs) -> None:
    """Expert compute of the fused MoE; writes ``y`` (must be zero on entry) in place.

    Two call forms, told apart by their arguments exactly like the two pybind overloads (csrc/ffi.cu:112-143):
      * 16-bit weights:  ``..., C, y, APerWarp=2, splitK=3, tile_m_2=128, tile_n_2=16, tile_k_2=128,
        block_dim_x_gemm=256, microBatchSize=16, experts_map=None``
      * e4m3 weights:    ``..., C, y, w1_scale, w2_scale, block_shape, soft_fp8=False, microBatchSize=16,
        experts_map=None``  (block_shape must be [128,128] and soft_fp8 True; scales may be None = unit scales)
    The tile arguments of the first form describe the reference's MetaX kernels; here only ``APerWarp`` (row groups
    per warp of the second GEMM: 1 or 2, other values = automatic) is used, split-K is chosen from the shape.
    Extra keywords: ``fp8_repacked`` marks e4m3 weights that went through ``fp8_weight_repack``;
    ``deterministic`` (default True) sums each token's expert outputs in fp32 in a fixed order with one rounding,
    False uses 16-bit atomic adds into ``y`` as the reference does; a float32 ``y`` (deterministic only) receives the
    un-rounded sums; ``tune`` = six launch integers (token tiles per
    work item, GEMM1 row warps, GEMM1 split-K, GEMM2 row groups per warp, GEMM2 row warps, GEMM2 split-K; 0 = automatic);
    ``routing`` = (gating_output, score_fun, n_groups, topK_groups, gating_bias, renormalize) runs ``fused_routing_gate``
    in front inside the same library call (``topk_ids`` and ``actived_experts_weights`` become outputs): for decode
    batches with the single-kernel tuning (300) the whole layer is then one launch.
    """
    w1, w2, x = experts_weights_matrix1, experts_weights_matrix2, activations
    fp8_form = (len(args) > 0 and not isinstance(args[0], int)) or any(
        k_ in kwargs for k_ in ("w1_scale", "w2_scale", "block_shape", "soft_fp8"))
    fp8_repacked = bool(kwargs.pop("fp8_repacked", False))
    deterministic = bool(kwargs.pop("deterministic", True))
    out_fp32 = y.dtype == torch.float32 and activations.dtype != torch.float32
    tune = kwargs.pop("tune", None)
    routing = kwargs.pop("routing", None)
    if fp8_form:
        names = ["w1_scale", "w2_scale", "block_shape", "soft_fp8", "microBatchSize", "experts_map"]
        vals = {"soft_fp8": False, "microBatchSize": 16, "experts_map": None}
    else:
        names = ["APerWarp", "splitK", "tile_m_2", "tile_n_2", "tile_k_2", "block_dim_x_gemm", "microBatchSize",
                 "experts_map"]
        vals = {"APerWarp": 2, "splitK": 3, "tile_m_2": 128, "tile_n_2": 16, "tile_k_2": 128,
                "block_dim_x_gemm": 256, "microBatchSize": 16, "experts_map": None}
    _chk(len(args) <= len(names), "fused_experts_compute(): incompatible function arguments")
    for n_, v in zip(names, args):
        vals[n_] = v
    for k_, v in kwargs.items():
        _chk(k_ in names, f"fused_experts_compute(): unexpected keyword argument '{k_}'")
        vals[k_] = v

    for t, name in ((w1, "experts_weights_matrix1"), (w2, "experts_weights_matrix2"), (x, "activations"),
                    (topk_ids, "topk_ids"), (actived_experts_weights, "actived_experts_weights"),
                    (sorted_token_ids, "sorted_token_ids"), (cumsum_buffer, "cumsum_buffer"),
                    (padded_num_experts, "padded_num_experts"), (experts_ids, "experts_ids"), (C, "C"), (y, "y")):
        _cuda_contig(t, name)
    _chk(w1.dtype == w2.dtype, "experts_weights_matrix1 and experts_weights_matrix2 must have the same data type.")
    _chk(topk_ids.dtype == torch.int32, "expertsIds must be of type torch::kInt32.")
    _chk(x.dtype == actived_experts_weights.dtype,
         "activations and activedExpertsWeights must have the same data type.")
    _chk(x.dtype in (torch.float16, torch.bfloat16),
         "activations must be of type torch::kFloat16 or torch::kBFloat16.")
    _chk(w1.dim() == 3 and w2.dim() == 3, "expert weights must be 3D tensors [E, rows, cols]")
    E, m1, k1 = w1.shape
    E2, m2, k2 = w2.shape
    _chk(E == E2 and m1 == 2 * k2 and m2 == k1, "w1 must be [E, 2I, H] and w2 [E, H, I]")
    _chk(x.dim() == 2 and x.size(0) == batch_size and x.size(1) == k1, "activations must be [batch_size, H]")
    topK = dynamic_experts_per_act
    _chk(topk_ids.numel() == batch_size * topK, "topk_ids must be [batch_size, topK]")
    _chk(C.numel() >= topK * m1 * batch_size and C.dtype == x.dtype, "C must hold topK * 2I * batch_size elements")
    _chk(y.shape == x.shape and (y.dtype == x.dtype or (out_fp32 and deterministic)),
         "y must look like activations (or be their float32 twin, with deterministic=True)")
    w1s = w2s = None
    if fp8_form:
        _chk(w1.element_size() == 1, "experts_weights_matrix1 must be a 1-byte (float8_e4m3fn) tensor.")
        _chk(x.dtype == torch.bfloat16, "Weight date type and activation date type are not supported.")
        bs = list(vals["block_shape"]) if vals.get("block_shape") is not None else None
        _chk(bs is not None and len(bs) == 2, "block_shape must have size 2.")
        _chk(bs[0] == 128 and bs[1] == 128, "block_shape must be (128, 128) for float8_e4m3fn.")
        _chk(bool(vals["soft_fp8"]), "soft_fp8 must be true for float8_e4m3fn.")
        w1s, w2s = vals.get("w1_scale"), vals.get("w2_scale")
        _chk((w1s is None) == (w2s is None), "give both block scales or neither")
        if w1s is not None:
            _cuda_contig(w1s, "w1_scale")
            _cuda_contig(w2s, "w2_scale")
            _chk(w1s.dtype == torch.float32 and w2s.dtype == torch.float32, "w1_scale and w2_scale must be float32.")
            _chk(w1s.numel() == E * ((m1 + 127) // 128) * ((k1 + 127) // 128) and
                 w2s.numel() == E * ((m2 + 127) // 128) * ((k2 + 127) // 128),
                 "scales must be [E, rows/128, cols/128]")
        code, rg = 2, 0
    else:
        _chk(w1.dtype in (torch.float16, torch.bfloat16),
             "experts_weights_matrix1 must be of type torch::kFloat16 or torch::kBFloat16.")
        _chk(w1.dtype == x.dtype, "Weight date type and activation date type are not supported.")
        code = _act_code(x)
        rg = vals["APerWarp"] if vals["APerWarp"] in (1, 2) else 0
    mp, ml = _map_args(vals["experts_map"])
    t6 = [0, 0, 0, rg, 0, 0]
    if tune is not None:
        _chk(len(tune) == 6, "tune must hold six integers")
        t6 = [int(v) for v in tune]
    tune_arr = (ctypes.c_int32 * 6)(*t6)
    # fp32 [slots, H] buffer for the fixed-order combine (torch's caching allocator makes this a pointer bump)
    scratch = torch.empty((batch_size * topK, k1), dtype=torch.float32, device=x.device) if deterministic else None
    tail = (w1.data_ptr(), w2.data_ptr(), x.data_ptr(), batch_size, E, topK, k1, k2, topk_ids.data_ptr(),
            actived_experts_weights.data_ptr(), sorted_token_ids.data_ptr(), cumsum_buffer.data_ptr(),
            padded_num_experts.data_ptr(), experts_ids.data_ptr(), C.data_ptr(), y.data_ptr(), _ptr(w1s), _ptr(w2s), code,
            int(fp8_repacked), int(vals["microBatchSize"]), mp, ml, _ptr(scratch),
            0 if scratch is None else scratch.numel() * 4, tune_arr, _status_ptr(x), int(out_fp32), _stream(x))
    if routing is None:
        check(lib.mlk_fused_experts_compute(*tail))
        return
    # routing fused in front: (gating_output, score_fun, n_groups, topK_groups, gating_bias, renormalize); topk_ids and
    # actived_experts_weights are then outputs
    gating, score_fun, n_groups, topk_groups, gbias, renorm = routing
    _cuda_contig(gating, "gating_output")
    _chk(gating.dtype == x.dtype and gating.dim() == 2 and gating.size(0) == batch_size,
         "gating_output must be [batch_size, num_experts] in the activation dtype")
    if gbias is not None:
        _cuda_contig(gbias, "gating_bias")
        _chk(gbias.dtype == gating.dtype and gbias.numel() == gating.size(1), "gating_bias must be [num_experts] in the logits' dtype")
    check(lib.mlk_fused_routing_experts_compute(gating.data_ptr(), gating.size(1), int(score_fun), int(n_groups),
                                                int(topk_groups), _ptr(gbias), int(bool(renorm)), *tail))


# ---------------------------------------------------------------------------------------------------
# names the reference module also exports but that are outside the weight-streaming path
# ---------------------------------------------------------------------------------------------------

def _out_of_scope(name: str, why: str):
    def f(*_a, **_k):
        raise NotImplementedError(f"{name} is not part of this library: {why}")
    f.__name__ = name
    f.__doc__ = f"Not implemented: {why}"
    return f


gemmEx = _out_of_scope("gemmEx", "it wraps the vendor GEMM of the reference platform (csrc/gemm_ex.cu); use torch.matmul")
muxi_hgemm = _out_of_scope("muxi_hgemm", "large-n prefill GEMM family (csrc/muxi_hgemm.cu)")
muxi_hgemm_layout = _out_of_scope("muxi_hgemm_layout", "large-n prefill GEMM family (csrc/muxi_hgemm_layout.cu)")
muxi_hgemm_layoutC = _out_of_scope("muxi_hgemm_layoutC", "large-n prefill GEMM family (csrc/muxi_hgemm_layoutC.cu)")
routing_gate = _out_of_scope("routing_gate", "legacy split MoE, superseded by fused_routing_gate (csrc/moe_kernels/routing_gate.cu)")
experts_compute = _out_of_scope("experts_compute", "legacy host-synchronous MoE, superseded by fused_experts_compute (csrc/moe_kernels/experts_compute.cu)")
