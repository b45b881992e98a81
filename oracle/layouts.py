"""TEST INFRASTRUCTURE -- CPU oracle for the layout permutations and the e4m3 bit format.

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline leg may import this package; the product
(muxi_native_layout_kernels_b200) never does.

Every function is an element-index restatement (numpy fancy indexing, no view/permute tricks) of a layout the
reference defines through torch view/permute recipes or device index arithmetic:
  layout A   benchmark_and_test/gemm_benchmark.py:41-42, csrc/moe_kernels/layout.h:80-97
  layout B   csrc/layout_b.cu:34-60,73; benchmark_and_test/transposeB_bench.py:10-11
  layout C   benchmark_and_test/gemm_benchmark.py:74-76; csrc/re_layout_c.cu:67-72
  repack     csrc/fp8_weight_repack.cu:35-36
  e4m3       csrc/utils.cuh:232-251 (decode), OCP FP8 E4M3 "fn" format (bias 7, no infinity, S.1111.111 = NaN)
Pinned against golden vectors produced by the reference's own recipes: tests/golden/make_golden.py.
"""
from __future__ import annotations

import numpy as np


def layout_a(W: np.ndarray) -> np.ndarray:
    """A4[g, o, r, e] = W[16g + r, 8o + e]."""
    m, k = W.shape
    assert m % 16 == 0 and k % 8 == 0
    g, o, r, e = np.meshgrid(np.arange(m // 16), np.arange(k // 8), np.arange(16), np.arange(8), indexing="ij")
    return W[16 * g + r, 8 * o + e]


def layout_a_inverse(A4: np.ndarray) -> np.ndarray:
    G, O, R, E = A4.shape
    assert R == 16 and E == 8
    row, col = np.meshgrid(np.arange(G * 16), np.arange(O * 8), indexing="ij")
    return A4[row // 16, col // 8, row % 16, col % 8]


def layout_b(B: np.ndarray) -> np.ndarray:
    """B5[c, nb, q, r, e] = B[16nb + r, 32c + 8q + e]."""
    n, k = B.shape
    assert n % 16 == 0 and k % 32 == 0
    c, nb, q, r, e = np.meshgrid(np.arange(k // 32), np.arange(n // 16), np.arange(4), np.arange(16), np.arange(8),
                                 indexing="ij")
    return B[16 * nb + r, 32 * c + 8 * q + e]


def layout_c(C: np.ndarray) -> np.ndarray:
    """C5[mb, nb, q, r, e] = C[16nb + r, 32mb + 8q + e] for C of shape [n, m]."""
    n, m = C.shape
    assert n % 16 == 0 and m % 32 == 0
    mb, nb, q, r, e = np.meshgrid(np.arange(m // 32), np.arange(n // 16), np.arange(4), np.arange(16), np.arange(8),
                                  indexing="ij")
    return C[16 * nb + r, 32 * mb + 8 * q + e]


def layout_c_inverse(C5: np.ndarray) -> np.ndarray:
    MB, NB, Q, R, E = C5.shape
    assert (Q, R, E) == (4, 16, 8)
    tok, row = np.meshgrid(np.arange(NB * 16), np.arange(MB * 32), indexing="ij")
    return C5[row // 32, tok // 16, (row % 32) // 8, tok % 16, row % 8]


def fp8_repack(raw: np.ndarray) -> np.ndarray:
    """Bytes [b0,b1,b2,b3] of every aligned 32-bit word -> [b0,b2,b1,b3]; input is a uint8 array whose size is a
    multiple of 4 (shape preserved)."""
    flat = raw.reshape(-1, 4)
    return flat[:, [0, 2, 1, 3]].reshape(raw.shape)


def e4m3_decode_table() -> np.ndarray:
    """float32 value of each of the 256 e4m3fn bytes; the two NaN encodings decode to +-480 as in the
    reference's bit trick (there is no special case for them), not to NaN."""
    out = np.zeros(256, dtype=np.float32)
    for b in range(256):
        s = -1.0 if b & 0x80 else 1.0
        e = (b >> 3) & 0xF
        mant = b & 0x7
        if e == 0:
            v = mant / 8.0 * 2.0 ** -6
        else:
            v = (1.0 + mant / 8.0) * 2.0 ** (e - 7)
        out[b] = s * v
    return out
