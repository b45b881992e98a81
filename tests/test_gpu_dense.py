"""GeMV / narrow GEMM / soft-FP8 on the GPU (through the C ABI) against the CPU oracle.

Tolerance: |got - want| <= 1e-2 + 1e-2 * |want| on the 16-bit outputs (fp32 accumulation on both sides), the
combined form of the "max-abs / max-rel <= 1e-2" bar: a bf16 value of magnitude 4..8 has a unit in the last place
of 0.031, so a pure absolute bound cannot hold for correct results, and a pure relative one blows up near zero.
"""
import ctypes
import itertools

import pytest
import torch

import muxi_native_layout_kernels_b200 as mlk
from oracle import dense as odense
from oracle import layouts as olay
from tests.gpu_util import DT, assert_close, rand_e4m3, randn, require_gpu

pytestmark = pytest.mark.gpu


def _weights(m, k, seed, dtype, dev, scale=0.02):
    W = randn((m, k), seed, scale, dtype)
    return W, mlk.layoutA(W.to(dev))


# ----------------------------------------------------------------------------------------------------
# e4m3 decode: every byte value, both byte orders, exact
# ----------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("repacked", [False, True])
def test_e4m3_decode_is_exact_for_all_256_bytes(repacked):
    dev = require_gpu()
    table = torch.from_numpy(olay.e4m3_decode_table())
    raw = (torch.arange(128 * 128, dtype=torch.int64) * 37 % 256).to(torch.uint8).reshape(128, 128)
    assert raw.unique().numel() == 256
    w8 = raw.view(torch.float8_e4m3fn).to(dev)
    A = mlk.layoutA(w8)
    if repacked:
        A = mlk.fp8_weight_repack(A)
    want = table[raw.long()]                      # [m, k] fp32, NaN bytes -> +-480
    for half in range(2):                         # 64 one-hot tokens per call
        X = torch.zeros(64, 128, dtype=torch.bfloat16)
        X[torch.arange(64), half * 64 + torch.arange(64)] = 1.0
        for (rg, wm, sk) in [(1, 1, 1), (2, 4, 2)]:
            C = mlk.gemm_layoutA_soft_fp8_wapper(A, None, X.to(dev), 128, 64, 128, kernelParam1=rg, kernelParam2=wm,
                                                 kernelParam3=sk, fp8_repacked=repacked)
            got = C.float().cpu()                 # [token j, row] = W[row, half*64 + j]
            assert torch.equal(got, want[:, half * 64:(half + 1) * 64].t().contiguous())


# ----------------------------------------------------------------------------------------------------
# GeMV
# ----------------------------------------------------------------------------------------------------

GEMV_SHAPES = [(16, 32), (64, 160), (128, 1024), (272, 352), (512, 4096)]


@pytest.mark.parametrize("dt", ["bf16", "fp16"])
@pytest.mark.parametrize("kernel_id", [1, 2])
def test_gemv_all_launch_parameters(dt, kernel_id):
    dev = require_gpu()
    for (m, k) in GEMV_SHAPES:
        W, A = _weights(m, k, 10 + m, DT[dt], dev, 0.05)
        x = randn((1, k), 11 + k, 1.0, DT[dt])
        want = odense.gemm_ref(x, W)
        for threads, rg, sk in itertools.product([64, 128, 256], [1, 2], [1, 2, 4, 8]):
            if m % (16 * rg):
                continue
            y = mlk.gemv_layoutA_wapper(A, x.to(dev), m, k, blockDimX=threads, kernelId=kernel_id, kernelParam1=rg,
                                        kernelParam2=sk)
            assert y.shape == (1, m) and y.dtype == DT[dt]
            assert_close(y, want, f"gemv {dt} id={kernel_id} m={m} k={k} threads={threads} rg={rg} sk={sk}")


def test_gemv_alpha_bias_and_table_path():
    dev = require_gpu()
    m, k = 256, 512
    for dt in ("bf16", "fp16"):
        W, A = _weights(m, k, 20, DT[dt], dev, 0.05)
        x = randn((1, k), 21, 1.0, DT[dt])
        bias = randn((1, m), 22, 1.0, DT[dt])
        y = mlk.gemv_layoutA(A, x.to(dev), alpha=0.5, beta=3.0, bias=bias.to(dev))   # beta is ignored
        assert_close(y, odense.gemm_ref(x, W, alpha=0.5, bias=bias), f"gemv table {dt}")
        for kid in (1, 2):
            y = mlk.gemv_layoutA_wapper(A, x.to(dev), m, k, alpha=2.0, kernelId=kid, bias=bias.to(dev))
            assert_close(y, odense.gemm_ref(x, W, alpha=2.0, bias=bias), f"gemv wapper {dt} {kid}")


@pytest.mark.parametrize("repacked", [False, True])
def test_gemv_soft_fp8(repacked):
    dev = require_gpu()
    for (m, k) in [(128, 128), (256, 1024), (384, 4096)]:
        W8 = rand_e4m3((m, k), 30 + m)
        A = mlk.layoutA(W8.to(dev))
        if repacked:
            A = mlk.fp8_weight_repack(A)
        x = randn((1, k), 31, 1.0, torch.bfloat16)
        want = odense.gemm_ref(x, W8.to(torch.bfloat16))
        for threads, rg, sk in itertools.product([128, 256], [1, 2], [1, 2, 8]):
            y = mlk.gemv_layoutA_wapper(A, x.to(dev), m, k, blockDimX=threads, kernelParam1=rg, kernelParam2=sk,
                                        fp8_repacked=repacked)
            assert_close(y, want, f"gemv fp8 m={m} k={k} threads={threads} rg={rg} sk={sk}")
        # block scales: compared with fp32 weight * fp32 scale (what the kernel applies, to the fp32 block sums)
        scale = (torch.rand((m + 127) // 128, (k + 127) // 128, generator=torch.Generator().manual_seed(32)) * 2).float()
        y = mlk.gemv_layoutA(A, x.to(dev), scale_matrix=scale.to(dev), fp8_repacked=repacked)
        want_s = (x.float() @ odense.dequant_exact_scale(W8, scale).t()).to(torch.bfloat16)
        assert_close(y, want_s, f"gemv fp8 scaled m={m} k={k}")
        # and within tolerance of the reference's own dequantise-then-GEMM recipe (weights rounded to bf16 first)
        want_r = odense.gemm_ref(x, odense.dequant_block_scaled(W8, scale))
        assert_close(y, want_r, f"gemv fp8 scaled vs reference recipe m={m} k={k}", scale_atol=True)


def test_gemv_kernel2_rejects_what_it_cannot_do():
    dev = require_gpu()
    W8 = rand_e4m3((128, 128), 40)
    A = mlk.layoutA(W8.to(dev))
    x = randn((1, 128), 41).to(dev)
    with pytest.raises(RuntimeError, match="no e4m3 variant"):
        mlk.gemv_layoutA_wapper(A, x, 128, 128, kernelId=2)
    with pytest.raises(RuntimeError, match="kernelId"):
        mlk.gemv_layoutA_wapper(A, x, 128, 128, kernelId=5)
    with pytest.raises(RuntimeError, match="same k"):
        mlk.gemv_layoutA(A, randn((1, 256), 42).to(dev))


# ----------------------------------------------------------------------------------------------------
# narrow GEMM, three layout variants
# ----------------------------------------------------------------------------------------------------

GEMM_CONFIGS = [(1, 1, 1), (1, 1, 8), (2, 1, 2), (1, 2, 1), (2, 2, 4), (1, 4, 2), (2, 4, 1), (1, 8, 1), (2, 8, 2)]
TOKENS = [1, 2, 3, 8, 9, 16, 17, 32, 33, 64, 65, 128, 200, 256]


@pytest.mark.parametrize("dt", ["bf16", "fp16"])
def test_gemm_layoutA_tokens_and_configs(dt):
    dev = require_gpu()
    for (m, k) in [(256, 128), (512, 640), (384, 2048)]:
        W, A = _weights(m, k, 50 + m, DT[dt], dev, 0.05)
        for n in TOKENS:
            X = randn((n, k), 51 + n, 1.0, DT[dt])
            want = odense.gemm_ref(X, W)
            for (rg, wm, sk) in GEMM_CONFIGS:
                if m % (16 * rg * wm):
                    continue
                C = mlk.gemm_layoutA_wapper(A, X.to(dev), m, n, k, kernelParam1=rg, kernelParam2=wm, kernelParam3=sk)
                assert C.shape == (n, m)
                assert_close(C, want, f"gemm_layoutA {dt} m={m} k={k} n={n} rg={rg} wm={wm} sk={sk}")
            assert_close(mlk.gemm_layoutA(A, X.to(dev)), want, f"gemm_layoutA table {dt} m={m} k={k} n={n}")


@pytest.mark.parametrize("dt", ["bf16", "fp16"])
def test_gemm_layoutB_variants(dt):
    dev = require_gpu()
    for (m, k) in [(256, 256), (512, 1024)]:
        W, A = _weights(m, k, 60 + m, DT[dt], dev, 0.05)
        bias = randn((1, m), 61, 1.0, DT[dt])
        for n in [16, 32, 48, 64, 128, 256]:
            X = randn((n, k), 62 + n, 1.0, DT[dt])
            XB = mlk.layoutB(X.to(dev))
            want = odense.gemm_ref(X, W, alpha=1.5, bias=bias)
            for (rg, wm, sk) in [(1, 1, 1), (2, 2, 2), (2, 4, 4), (1, 8, 1)]:
                C = mlk.gemm_layoutAB_ContinuousC_wapper(A, XB, m, n, k, alpha=1.5, kernelParam1=rg, kernelParam2=wm,
                                                         kernelParam3=sk, bias=bias.to(dev))
                assert_close(C, want, f"ContinuousC {dt} m={m} k={k} n={n} {(rg, wm, sk)}")
                C5 = mlk.gemm_layoutABC_wapper(A, XB, m, n, k, alpha=1.5, kernelParam1=rg, kernelParam2=wm,
                                               kernelParam3=sk, bias=bias.to(dev))
                assert C5.shape == (m // 32, n // 16, 4, 16, 8)
                assert_close(mlk.reLayoutC(C5), want, f"ABC {dt} m={m} k={k} n={n} {(rg, wm, sk)}")
                # the reference's own un-permute recipe (benchmark_and_test/gemm_benchmark.py:74-76)
                assert torch.equal(C5.permute(1, 3, 0, 2, 4).reshape(n, m), mlk.reLayoutC(C5))
            if n <= 64:
                # kernelId 2: the tcgen05 kernel reads layout-B activations through a 5-D tensor map
                for (cps, stages, ck) in [(1, 2, 0), (2, 4, 0), (1, 3, 2), (1, 4, 4)]:
                    C = mlk.gemm_layoutAB_ContinuousC_wapper(A, XB, m, n, k, alpha=1.5, kernelParam1=cps, kernelParam2=stages,
                                                             kernelParam3=ck, kernelId=2, bias=bias.to(dev))
                    assert_close(C, want, f"ContinuousC tcgen05 {dt} m={m} k={k} n={n} {(cps, stages, ck)}")
                    C5 = mlk.gemm_layoutABC_wapper(A, XB, m, n, k, alpha=1.5, kernelParam1=cps, kernelParam2=stages,
                                                   kernelParam3=ck, kernelId=2, bias=bias.to(dev))
                    assert_close(mlk.reLayoutC(C5), want, f"ABC tcgen05 {dt} m={m} k={k} n={n} {(cps, stages, ck)}")
            assert_close(mlk.gemm_layoutAB_ContinuousC(A, XB, alpha=1.5, bias=bias.to(dev)), want, "ContinuousC table")
            assert_close(mlk.reLayoutC(mlk.gemm_layoutABC(A, XB, alpha=1.5, bias=bias.to(dev))), want, "ABC table")


@pytest.mark.parametrize("repacked", [False, True])
def test_gemm_soft_fp8(repacked):
    dev = require_gpu()
    for (m, k) in [(256, 256), (512, 1024)]:
        W8 = rand_e4m3((m, k), 70 + m)
        A = mlk.layoutA(W8.to(dev))
        if repacked:
            A = mlk.fp8_weight_repack(A)
        scale = (torch.rand(m // 128, k // 128, generator=torch.Generator().manual_seed(71)) * 2).float()
        for n in [1, 5, 8, 16, 24, 32, 64, 100]:
            X = randn((n, k), 72 + n, 1.0, torch.bfloat16)
            want = odense.gemm_ref(X, W8.to(torch.bfloat16))
            want_s = (X.float() @ odense.dequant_exact_scale(W8, scale).t()).to(torch.bfloat16)
            for (rg, wm, sk) in [(1, 1, 1), (2, 1, 2), (2, 2, 1), (1, 4, 2), (2, 8, 1)]:
                C = mlk.gemm_layoutA_soft_fp8_wapper(A, None, X.to(dev), m, n, k, kernelParam1=rg, kernelParam2=wm,
                                                     kernelParam3=sk, fp8_repacked=repacked)
                assert_close(C, want, f"fp8 gemm m={m} k={k} n={n} {(rg, wm, sk)}")
                Cs = mlk.gemm_layoutA_soft_fp8_wapper(A, scale.to(dev), X.to(dev), m, n, k, kernelParam1=rg,
                                                      kernelParam2=wm, kernelParam3=sk, fp8_repacked=repacked)
                assert_close(Cs, want_s, f"fp8 scaled gemm m={m} k={k} n={n} {(rg, wm, sk)}")
            # table-driven entry points: these shapes have no row, so 2..64 tokens run on the tcgen05 kernel, which
            # rounds the scaled weight to bf16 (as the reference does): tolerance relative to the output scale
            _close_rel(mlk.gemm_layoutA_soft_fp8(A, scale.to(dev), X.to(dev), fp8_repacked=repacked), want_s, "fp8 table")
            if not repacked:
                _close_rel(mlk.gemm_layoutA_linear(A, X.to(dev), scale_matrix=scale.to(dev)), want_s, "linear fp8")


@pytest.mark.parametrize("repacked", [False, True])
def test_soft_fp8_tcgen05_pipeline(repacked):
    """kernelId 2 (GEMM) / 3 (GeMV) with e4m3 weights: TMA -> decode in shared memory -> tcgen05, cluster split-K."""
    dev = require_gpu()
    for (m, k) in [(128, 128), (256, 384), (512, 1024), (1024, 4096)]:
        W8 = rand_e4m3((m, k), 170 + m)
        A = mlk.layoutA(W8.to(dev))
        if repacked:
            A = mlk.fp8_weight_repack(A)
        bias = randn((1, m), 171, 1.0, torch.bfloat16)
        for n in [1, 7, 16, 17, 32, 48, 64]:
            X = randn((n, k), 172 + n, 1.0, torch.bfloat16)
            want = odense.gemm_ref(X, W8.to(torch.bfloat16))
            for stages, ck in [(2, 1), (3, 2), (4, 4), (6, 3), (8, 8)]:
                if ck > k // 64:
                    continue
                C = mlk.gemm_layoutA_soft_fp8_wapper(A, None, X.to(dev), m, n, k, kernelParam1=1, kernelParam2=stages,
                                                     kernelParam3=ck, kernelId=2, fp8_repacked=repacked)
                assert_close(C, want, f"fp8 tcgen05 m={m} k={k} n={n} stages={stages} cluster={ck}")
            C = mlk.gemm_layoutA_soft_fp8_wapper(A, None, X.to(dev), m, n, k, alpha=0.5, kernelParam2=4, kernelParam3=2,
                                                 kernelId=2, bias=bias.to(dev), fp8_repacked=repacked)
            assert_close(C, odense.gemm_ref(X, W8.to(torch.bfloat16), alpha=0.5, bias=bias), f"fp8 tcgen05 bias m={m} n={n}")
        x = randn((1, k), 173, 1.0, torch.bfloat16)
        for stages, ck in [(2, 2), (4, 1), (8, 2)]:
            y = mlk.gemv_layoutA_wapper(A, x.to(dev), m, k, kernelId=3, kernelParam1=stages, kernelParam2=ck,
                                        fp8_repacked=repacked)
            assert_close(y, odense.gemm_ref(x, W8.to(torch.bfloat16)), f"gemv fp8 tcgen05 m={m} k={k} {stages},{ck}")
    # bit-identical from run to run
    X = randn((40, 4096), 174, 1.0, torch.bfloat16).to(dev)
    ref = mlk.gemm_layoutA_soft_fp8_wapper(A, None, X, 1024, 40, 4096, kernelParam2=4, kernelParam3=4, kernelId=2, fp8_repacked=repacked)
    for _ in range(3):
        assert torch.equal(ref, mlk.gemm_layoutA_soft_fp8_wapper(A, None, X, 1024, 40, 4096, kernelParam2=4, kernelParam3=4,
                                                                 kernelId=2, fp8_repacked=repacked))
    # unit block scales change nothing, bit for bit
    ones = torch.ones(8, 32, device=dev)
    assert torch.equal(ref, mlk.gemm_layoutA_soft_fp8_wapper(A, ones, X, 1024, 40, 4096, kernelParam2=4, kernelParam3=4,
                                                             kernelId=2, fp8_repacked=repacked))


@pytest.mark.parametrize("repacked", [False, True])
def test_soft_fp8_native_tensor_core_kernel(repacked):
    """kernelId 9 (GEMM) / 4 (GeMV): e4m3 weights undecoded into tcgen05.mma.kind::f8f6f4, activations split into two
    e4m3 terms under a per-token power-of-two scale.  Same oracle and tolerance as the decode kernels."""
    dev = require_gpu()
    for (m, k) in [(128, 128), (256, 384), (512, 1024), (1024, 4096)]:
        W8 = rand_e4m3((m, k), 270 + m)
        A = mlk.layoutA(W8.to(dev))
        if repacked:
            A = mlk.fp8_weight_repack(A)
        bias = randn((1, m), 271, 1.0, torch.bfloat16)
        for n in [1, 7, 16, 17, 32, 48, 64]:
            X = randn((n, k), 272 + n, 1.0, torch.bfloat16)
            want = odense.gemm_ref(X, W8.to(torch.bfloat16))
            for bk, stages, ck in [(64, 2, 1), (64, 3, 2), (128, 4, 4), (64, 6, 3), (64, 8, 8), (128, 6, 8), (128, 2, 1)]:
                if ck > k // bk or k % bk:
                    continue
                C = mlk.gemm_layoutA_soft_fp8_wapper(A, None, X.to(dev), m, n, k, kernelParam1=bk, kernelParam2=stages,
                                                     kernelParam3=ck, kernelId=9, fp8_repacked=repacked)
                assert_close(C, want, f"fp8 native m={m} k={k} n={n} bk={bk} stages={stages} cluster={ck}")
            C = mlk.gemm_layoutA_soft_fp8_wapper(A, None, X.to(dev), m, n, k, alpha=0.5, kernelParam1=64, kernelParam2=4,
                                                 kernelParam3=2, kernelId=9, bias=bias.to(dev), fp8_repacked=repacked)
            assert_close(C, odense.gemm_ref(X, W8.to(torch.bfloat16), alpha=0.5, bias=bias), f"fp8 native bias m={m} n={n}")
        x = randn((1, k), 273, 1.0, torch.bfloat16)
        for bk, stages, ck in [(64, 2, 2), (128, 4, 1), (256, 3, 2)]:
            if k % min(bk, 128) or ck > k // min(bk, 128):
                continue
            y = mlk.gemv_layoutA_wapper(A, x.to(dev), m, k, blockDimX=bk, kernelId=4, kernelParam1=stages, kernelParam2=ck,
                                        fp8_repacked=repacked)
            assert_close(y, odense.gemm_ref(x, W8.to(torch.bfloat16)), f"gemv fp8 native m={m} k={k} {bk},{stages},{ck}")
    # bit-identical from run to run
    X = randn((40, 4096), 274, 1.0, torch.bfloat16).to(dev)
    call = lambda: mlk.gemm_layoutA_soft_fp8_wapper(A, None, X, 1024, 40, 4096, kernelParam1=64, kernelParam2=4,
                                                    kernelParam3=4, kernelId=9, fp8_repacked=repacked)
    ref = call()
    for _ in range(3):
        assert torch.equal(ref, call())
    assert mlk.kernel_status() == 0
    # block scales are not this kernel's business
    with pytest.raises(RuntimeError, match="block scales"):
        mlk.gemm_layoutA_soft_fp8_wapper(A, torch.ones(8, 32, device=dev), X, 1024, 40, 4096, kernelParam1=64,
                                         kernelParam2=4, kernelParam3=4, kernelId=9, fp8_repacked=repacked)


def test_soft_fp8_native_kernel_exactness_and_ranges():
    """Properties of the two-term activation split: every finite e4m3 byte is multiplied exactly; rows of very
    different magnitude in one call keep their precision (per-token scale); tiny and huge activations; zero rows."""
    dev = require_gpu()
    table = torch.from_numpy(olay.e4m3_decode_table())
    raw = (torch.arange(128 * 128, dtype=torch.int64) * 37 % 256).to(torch.uint8).reshape(128, 128)
    raw = torch.where((raw & 0x7F) == 0x7F, torch.zeros_like(raw), raw)          # the two NaN encodings -> 0
    A = mlk.layoutA(raw.view(torch.float8_e4m3fn).to(dev))
    want = table[raw.long()]
    for half in range(2):                         # 64 one-hot tokens per call: C[j, row] = W[row, half * 64 + j]
        X = torch.zeros(64, 128, dtype=torch.bfloat16)
        X[torch.arange(64), half * 64 + torch.arange(64)] = 1.0
        C = mlk.gemm_layoutA_soft_fp8_wapper(A, None, X.to(dev), 128, 64, 128, kernelParam1=64, kernelParam2=2,
                                             kernelParam3=1, kernelId=9)
        assert torch.equal(C.float().cpu(), want[:, half * 64:(half + 1) * 64].t().contiguous())
    # tokens of magnitudes 1e-30 ... 1e30 in one batch, plus an all-zero token
    m, k = 256, 1024
    W8 = rand_e4m3((m, k), 280)
    A = mlk.layoutA(W8.to(dev))
    X = randn((16, k), 281, 1.0, torch.float32)
    mags = torch.tensor([1e-30, 1e-20, 1e-10, 1e-5, 1e-3, 0.1, 1.0, 10.0, 1e3, 1e5, 1e10, 1e20, 1e30, 3.0, 0.0, 1.0])
    X = (X * mags[:, None]).to(torch.bfloat16)
    C = mlk.gemm_layoutA_soft_fp8_wapper(A, None, X.to(dev), m, 16, k, kernelParam1=128, kernelParam2=3, kernelParam3=2,
                                         kernelId=9).float().cpu()
    ref = X.double() @ W8.to(torch.bfloat16).double().t()
    for t in range(16):
        scale = float(ref[t].abs().max()) or 1.0
        err = float((C[t].double() - ref[t]).abs().max()) / scale
        assert err < 6e-3, f"token {t} (magnitude {float(mags[t])}): error {err} of the row's largest output"
    assert bool((C[14] == 0).all())
    # an element 2^-14 of its token's maximum: still resolved to 2^-17 of the maximum
    X = torch.zeros(1, k, dtype=torch.bfloat16)
    X[0, 0] = 1024.0
    X[0, 1] = 1024.0 * 2.0 ** -14 * 1.4375
    y = mlk.gemv_layoutA_wapper(A, X.to(dev), m, k, blockDimX=64, kernelId=4, kernelParam1=2, kernelParam2=1).double().cpu()
    ref = X.double() @ W8.to(torch.bfloat16).double().t()
    bound = 2.0 ** -17 * 1024.0 * float(W8.float()[:, 1].abs().max()) + 2.0 ** -8 * ref.abs()
    assert bool(((y - ref).abs() <= bound + 1e-6).all())


def _close_rel(got, want, what, tol=1e-2):
    """|got - want| <= tol * (rms(want) + |want|): the absolute part follows the output scale, which block scales
    move by orders of magnitude."""
    rms = float(want.double().pow(2).mean().sqrt())
    rep = odense.error_report(got.detach().cpu(), want, atol=tol * rms, rtol=tol)
    assert rep["ok"], f"{what}: {rep}"


@pytest.fixture
def full_scales(request):
    mlk.set_full_scales(request.param)
    yield request.param
    mlk.set_full_scales(False)


@pytest.mark.parametrize("full_scales", [False, True], indirect=True)
@pytest.mark.parametrize("repacked", [False, True])
def test_soft_fp8_tcgen05_block_scales(repacked, full_scales):
    """Block scales in the decode.  Default: the scale rounded to bf16, rne_bf16(w * bf16(s)), inside the parity
    tolerance of the path.  Full scales: rne_bf16(w * s), so the GEMM equals, to accumulation order and the final
    rounding (one bf16 ulp, 2^-8), a bf16 GEMM on the weights the reference's torch recipe dequantises to
    (muxi_layout_kernels/utils.py:14-25)."""
    dev = require_gpu()
    # default: up to one bf16 ulp per weight (2^-8) on top of the rounding of the output, measured against the output
    # scale (these outputs are far below 1, where the path's absolute bar of 1e-2 says nothing)
    # full scales: the two bf16 outputs may still sit on either side of a rounding boundary (one ulp = 2^-7 of the value)
    tol = 8e-3 if full_scales else 2e-2
    g = torch.Generator().manual_seed(177)
    for (m, k) in [(128, 128), (256, 1024), (1024, 4096), (384, 4224)]:
        W8 = rand_e4m3((m, k), 175 + m)
        A = mlk.layoutA(W8.to(dev))
        if repacked:
            A = mlk.fp8_weight_repack(A)
        sm, sk_ = (m + 127) // 128, (k + 127) // 128
        scales = {
            "quant": torch.rand(sm, sk_, generator=g) * 0.01 + 1e-4,                  # amax / 448 style
            "wide": torch.exp2(torch.randint(-40, 20, (sm, sk_), generator=g).float()) * (1 + torch.rand(sm, sk_, generator=g)),
            "signed": (torch.rand(sm, sk_, generator=g) - 0.5) * 4,
        }
        # values outside the folded range of the decode: huge, tiny, zero
        edge = torch.rand(sm, sk_, generator=g) + 0.5
        edge.view(-1)[0::3] *= 2.0 ** 20
        edge.view(-1)[1::3] *= 2.0 ** -130
        if edge.numel() > 4:
            edge.view(-1)[4] = 0.0
        scales["edge"] = edge
        for name, scale in scales.items():
            scale = scale.float().contiguous()
            Wd = odense.dequant_block_scaled(W8, scale)
            for n in (1, 8, 24, 64):
                X = randn((n, k), 176 + n, 1.0, torch.bfloat16)
                want = odense.gemm_ref(X, Wd)
                for stages, ck in [(2, 1), (4, 2), (6, 1)]:
                    if ck > k // 64:
                        continue
                    C = mlk.gemm_layoutA_soft_fp8_wapper(A, scale.to(dev), X.to(dev), m, n, k, kernelParam2=stages,
                                                         kernelParam3=ck, kernelId=2, fp8_repacked=repacked)
                    _close_rel(C, want, f"fp8 tcgen05 scaled[{name}] m={m} k={k} n={n} stages={stages} cluster={ck}", tol)
            x = randn((1, k), 178, 1.0, torch.bfloat16)
            y = mlk.gemv_layoutA_wapper(A, x.to(dev), m, k, kernelId=3, kernelParam1=4, kernelParam2=2,
                                        scale_matrix=scale.to(dev), fp8_repacked=repacked)
            _close_rel(y, odense.gemm_ref(x, Wd), f"gemv fp8 tcgen05 scaled[{name}] m={m} k={k}", tol)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_many_token_gemm_tile_kernel(dt):
    """muxi_hgemm_layoutA / kernelId 10: 128 x 128 and 128 x 256 (weight rows x tokens) tcgen05 tiles, whole k per CTA,
    any token count; also gemm_layoutA above 64 tokens, which runs on it by default."""
    dev = require_gpu()
    for (m, k) in [(128, 128), (384, 512), (1024, 4096)]:
        W, A = _weights(m, k, 300 + m, dt, dev)
        bias = randn((1, m), 301, 1.0, dt)
        for n in [65, 128, 200, 256, 257, 700, 1024]:
            X = randn((n, k), 302 + n, 1.0, dt)
            want = odense.gemm_ref(X, W)
            assert_close(mlk.muxi_hgemm_layoutA(A, X.to(dev)), want, f"hgemm m={m} k={k} n={n} {dt}")
            for nt, stages in [(128, 2), (128, 6), (256, 3), (256, 4)]:
                C = mlk.gemm_layoutA_wapper(A, X.to(dev), m, n, k, kernelParam1=nt, kernelParam2=stages, kernelId=10)
                assert_close(C, want, f"hgemm tile m={m} k={k} n={n} nt={nt} stages={stages} {dt}")
            if n <= 256:
                assert_close(mlk.gemm_layoutA(A, X.to(dev)), want, f"gemm_layoutA above 64 tokens m={m} n={n}")
        X = randn((300, k), 303, 1.0, dt)
        C = mlk.muxi_hgemm_layoutA(A, X.to(dev), alpha=0.5, bias=bias.to(dev))
        assert_close(C, odense.gemm_ref(X, W, alpha=0.5, bias=bias), f"hgemm alpha bias m={m}")
        # few tokens: the narrow kernels
        X = randn((40, k), 304, 1.0, dt)
        assert_close(mlk.muxi_hgemm_layoutA(A, X.to(dev)), odense.gemm_ref(X, W), f"hgemm 40 tokens m={m}")
    assert mlk.kernel_status() == 0


def test_many_token_gemm_e4m3_weights():
    """muxi_hgemm_layoutA with e4m3 weights (with and without block scales): the narrow kernels, 64 tokens at a time."""
    dev = require_gpu()
    m, k, n = 512, 1024, 200
    W8 = rand_e4m3((m, k), 310)
    A = mlk.layoutA(W8.to(dev))
    X = randn((n, k), 311, 1.0, torch.bfloat16)
    assert_close(mlk.muxi_hgemm_layoutA(A, X.to(dev)), odense.gemm_ref(X, W8.to(torch.bfloat16)), "hgemm e4m3")
    scale = (torch.rand(m // 128, k // 128, generator=torch.Generator().manual_seed(312)) * 2).float()
    want_s = (X.float() @ odense.dequant_exact_scale(W8, scale).t()).to(torch.bfloat16)
    _close_rel(mlk.muxi_hgemm_layoutA(A, X.to(dev), scale_matrix=scale.to(dev)), want_s, "hgemm e4m3 scaled")


def test_gemm_errors_and_determinism():
    dev = require_gpu()
    W, A = _weights(256, 256, 80, torch.bfloat16, dev)
    X = randn((16, 256), 81).to(dev)
    with pytest.raises(RuntimeError, match="multiple of 128"):
        mlk.gemm_layoutA(mlk.layoutA(randn((144, 256), 82).to(dev)), X)
    with pytest.raises(RuntimeError, match="same k"):
        mlk.gemm_layoutA(A, randn((16, 128), 83).to(dev))
    with pytest.raises(RuntimeError, match="kernelId"):
        mlk.gemm_layoutA_wapper(A, X, 256, 16, 256, kernelId=9)
    with pytest.raises(RuntimeError, match="row tile"):
        A128 = mlk.layoutA(randn((128, 256), 84).to(dev))
        mlk.gemm_layoutA_wapper(A128, X, 128, 16, 256, kernelParam1=2, kernelParam2=8, kernelParam3=1)
    with pytest.raises(RuntimeError, match="same data type"):
        mlk.gemm_layoutA(A, X.to(torch.float16))
    # split-K partial sums are reduced in a fixed order: bit-identical from run to run
    ref = mlk.gemm_layoutA_wapper(A, X, 256, 16, 256, kernelParam1=1, kernelParam2=1, kernelParam3=8)
    for _ in range(5):
        assert torch.equal(ref, mlk.gemm_layoutA_wapper(A, X, 256, 16, 256, kernelParam1=1, kernelParam2=1, kernelParam3=8))


@pytest.mark.parametrize("dt", ["bf16", "fp16"])
def test_gemm_tcgen05_tile_kernel(dt):
    """kernelId 2: TMA-fed tcgen05 tile kernel (tokens are the UMMA N dimension), all split-K / stage settings."""
    dev = require_gpu()
    for (m, k) in [(128, 128), (256, 384), (512, 640), (1024, 4096)]:
        W, A = _weights(m, k, 95 + m, DT[dt], dev, 0.05)
        bias = randn((1, m), 96, 1.0, DT[dt])
        for n in [1, 7, 16, 17, 32, 33, 48, 64]:
            X = randn((n, k), 97 + n, 1.0, DT[dt])
            want = odense.gemm_ref(X, W)
            want_b = odense.gemm_ref(X, W, alpha=0.5, bias=bias)
            for sk, stages in [(1, 2), (1, 8), (2, 4), (3, 6), (4, 2), (1, 3), (2, 5)]:
                C = mlk.gemm_layoutA_wapper(A, X.to(dev), m, n, k, kernelParam1=sk, kernelParam2=stages, kernelId=2)
                assert_close(C, want, f"tcgen05 {dt} m={m} k={k} n={n} sk={sk} stages={stages}")
            # thread-block-cluster split-K: partial tiles are added through distributed shared memory
            for ck, stages in [(2, 4), (3, 2), (4, 6), (8, 8), (16, 3)]:
                if ck > k // 64:
                    continue
                C = mlk.gemm_layoutA_wapper(A, X.to(dev), m, n, k, kernelParam1=1, kernelParam2=stages, kernelParam3=ck,
                                            kernelId=2)
                assert_close(C, want, f"tcgen05 cluster {dt} m={m} k={k} n={n} cluster={ck} stages={stages}")
            C = mlk.gemm_layoutA_wapper(A, X.to(dev), m, n, k, alpha=0.5, kernelParam1=2, kernelParam2=4, kernelId=2,
                                        bias=bias.to(dev))
            assert_close(C, want_b, f"tcgen05 bias {dt} m={m} k={k} n={n}")
    # split-K partial tiles are added in a fixed order: bit-identical from run to run
    X = randn((40, 4096), 98, 1.0, DT[dt]).to(dev)
    ref = mlk.gemm_layoutA_wapper(A, X, 1024, 40, 4096, kernelParam1=2, kernelParam2=4, kernelId=2)
    for _ in range(5):
        assert torch.equal(ref, mlk.gemm_layoutA_wapper(A, X, 1024, 40, 4096, kernelParam1=2, kernelParam2=4, kernelId=2))
    refc = mlk.gemm_layoutA_wapper(A, X, 1024, 40, 4096, kernelParam1=1, kernelParam2=4, kernelParam3=4, kernelId=2)
    for _ in range(3):
        assert torch.equal(refc, mlk.gemm_layoutA_wapper(A, X, 1024, 40, 4096, kernelParam1=1, kernelParam2=4, kernelParam3=4, kernelId=2))
    assert mlk.kernel_status() == 0, "a bounded wait inside the tcgen05 kernel expired"
    with pytest.raises(RuntimeError, match="stages"):
        mlk.gemm_layoutA_wapper(A, X, 1024, 40, 4096, kernelParam1=1, kernelParam2=7, kernelId=2)


@pytest.mark.parametrize("dt", ["bf16", "fp16"])
def test_gemm_cuda_core_kernel_up_to_four_tokens(dt):
    """kernelId 5/6/7: the CUDA-core FMA kernel behind the GEMM entry point for 1..4 tokens."""
    dev = require_gpu()
    for (m, k) in [(128, 128), (512, 640), (384, 2048)]:
        W, A = _weights(m, k, 85 + m, DT[dt], dev, 0.05)
        bias = randn((1, m), 86, 1.0, DT[dt])
        for n in [1, 2, 3, 4]:
            X = randn((n, k), 87 + n, 1.0, DT[dt])
            want = odense.gemm_ref(X, W, alpha=0.75, bias=bias)
            for kid, rg, sk in itertools.product([5, 6, 7], [1, 2], [1, 2, 8]):
                C = mlk.gemm_layoutA_wapper(A, X.to(dev), m, n, k, alpha=0.75, kernelParam1=rg, kernelParam3=sk,
                                            kernelId=kid, bias=bias.to(dev))
                assert_close(C, want, f"cuda-core gemm {dt} m={m} k={k} n={n} kid={kid} rg={rg} sk={sk}")
    with pytest.raises(RuntimeError, match="1..4 tokens"):
        mlk.gemm_layoutA_wapper(A, randn((8, 2048), 88, 1.0, DT[dt]).to(dev), 384, 8, 2048, kernelId=5)


def test_static_weights_and_pdl_modes_give_identical_results():
    """Launch options change when loads are issued, never what is computed: bit-identical outputs."""
    dev = require_gpu()
    W, A = _weights(1024, 2048, 90, torch.bfloat16, dev)
    torch.cuda.synchronize()           # the weights are complete before any launch under the static promise
    outs = {}
    try:
        for pdl, static in [(True, False), (True, True), (False, False)]:
            mlk.set_pdl(pdl)
            mlk.set_static_weights(static)
            res = []
            x = randn((1, 2048), 91).to(dev)
            for it in range(20):       # a dependent chain: each output feeds the next activation
                y = mlk.gemv_layoutA_wapper(A, x, 1024, 2048, kernelId=1 + it % 2, kernelParam1=1 + it % 2, kernelParam2=2)
                C = mlk.gemm_layoutA_wapper(A, torch.cat([x, x * 0.5]).contiguous(), 1024, 2, 2048, kernelParam1=1,
                                            kernelParam2=2, kernelParam3=2)
                C16 = mlk.gemm_layoutA_wapper(A, x.expand(16, 2048).contiguous(), 1024, 16, 2048, kernelParam1=2,
                                              kernelParam2=2, kernelParam3=1)
                res += [y, C, C16]
                x = torch.cat([y, y], dim=1).contiguous()
            torch.cuda.synchronize()
            outs[(pdl, static)] = [r.cpu() for r in res]
    finally:
        mlk.set_pdl(True)
        mlk.set_static_weights(False)
    base = outs[(False, False)]
    for k_, v in outs.items():
        assert all(torch.equal(a, b) for a, b in zip(v, base)), k_


# ----------------------------------------------------------------------------------------------------
# the benchmark configurations at full size
# ----------------------------------------------------------------------------------------------------

def test_config_gemv_4096_bf16():
    """bf16 GeMV, N=K=4096, W ~ N(0, 0.02^2), x ~ N(0,1), seed 0; oracle = fp32 matmul on the CPU, cast to bf16."""
    dev = require_gpu()
    W = randn((4096, 4096), 0, 0.02)
    x = randn((1, 4096), 1000, 1.0)
    A = mlk.layoutA(W.to(dev))
    want = odense.gemm_ref(x, W)
    assert_close(mlk.gemv_layoutA(A, x.to(dev)), want, "C1 table path")
    for kid, rg, sk in [(1, 1, 1), (1, 2, 4), (2, 1, 2), (2, 2, 8)]:
        y = mlk.gemv_layoutA_wapper(A, x.to(dev), 4096, 4096, kernelId=kid, kernelParam1=rg, kernelParam2=sk)
        rep = assert_close(y, want, f"C1 id={kid} rg={rg} sk={sk}")
    print("C1", rep)


@pytest.mark.parametrize("N,K", [(4096, 4096), (14336, 4096), (4096, 14336)])
def test_config_narrow_gemm_llama8b(N, K):
    dev = require_gpu()
    for dt in ("bf16", "fp16"):
        W = randn((N, K), 1, 0.02, DT[dt])
        A = mlk.layoutA(W.to(dev))
        Wf = W.float()
        for n in [1, 2, 4, 8, 16, 32, 64]:
            X = randn((n, K), 1000 + n, 1.0, DT[dt])
            want = (X.float() @ Wf.t()).to(DT[dt])
            assert_close(mlk.gemm_layoutA(A, X.to(dev)), want, f"C2 layoutA {dt} {(N, K)} n={n}")
            Xp = torch.zeros(max(16, (n + 15) // 16 * 16), K, dtype=DT[dt])
            Xp[:n] = X                             # the layout-B variants need n % 16 == 0: zero-pad, then slice
            XB = mlk.layoutB(Xp.to(dev))
            assert_close(mlk.gemm_layoutAB_ContinuousC(A, XB)[:n], want, f"C2 ContinuousC {dt} {(N, K)} n={n}")
            assert_close(mlk.reLayoutC(mlk.gemm_layoutABC(A, XB))[:n], want, f"C2 ABC {dt} {(N, K)} n={n}")


@pytest.mark.parametrize("N,K", [(28672, 8192), (8192, 28672), (8192, 8192)])
def test_config_soft_fp8_llama70b(N, K):
    dev = require_gpu()
    W8 = rand_e4m3((N, K), 2)
    A = mlk.layoutA(W8.to(dev))
    Wf = W8.float()
    x = randn((1, K), 2000, 1.0)
    assert_close(mlk.gemv_layoutA(A, x.to(dev)), (x.float() @ Wf.t()).to(torch.bfloat16), f"C3 gemv {(N, K)}")
    A_rep = mlk.fp8_weight_repack(A)
    for n in [1, 8, 32]:
        X = randn((n, K), 2000 + n, 1.0)
        want = (X.float() @ Wf.t()).to(torch.bfloat16)
        assert_close(mlk.gemm_layoutA_soft_fp8(A, None, X.to(dev)), want, f"C3 gemm {(N, K)} n={n}")
        assert_close(mlk.gemm_layoutA_soft_fp8(A_rep, None, X.to(dev), fp8_repacked=True), want, f"C3 repacked n={n}")


def test_offline_tuner_writes_rows_the_library_uses(tmp_path):
    """The offline tuner on two tiny keys (role of the reference's kernel_args_scan/gemv_kernel_args_scan.py:135-157):
    it must write a row per key into a table file of the reference's format, the library must load that file and
    return exactly those rows, and the table-driven entry point must give the oracle's result with them."""
    import csv
    from muxi_native_layout_kernels_b200._lib import lib, load_tables
    from muxi_native_layout_kernels_b200.kernel_args_scan import scan
    dev = require_gpu()
    try:
        scan.main(["--table", "layoutA_gemm", "--shapes", "256x256", "--tokens", "16", "--out", str(tmp_path)])
        scan.main(["--table", "layout_gemv_bf16", "--shapes", "256x256", "--out", str(tmp_path)])
        for t, name, key in ((2, "layoutA_gemm_dispatch_arg.csv", (256, 16, 256)), (5, "layout_gemv_bf16_dispatch_arg.csv", (256, 256))):
            rows = list(csv.reader(open(tmp_path / name)))
            assert rows[0] == (scan.GEMM_HEADER if t == 2 else scan.GEMV_HEADER)
            assert len(rows) == 2 and tuple(int(v) for v in rows[1][:len(key)]) == key
            assert lib.mlk_table_load(t, str(tmp_path / name).encode()) == 0
            out, hit = (ctypes.c_int * 4)(), ctypes.c_int(0)
            assert lib.mlk_table_lookup(t, key[0], key[1] if t == 2 else 1, key[-1], out, ctypes.byref(hit)) == 0
            assert hit.value == 1 and list(out) == [int(v) for v in rows[1][len(key):]]
        W, A = _weights(256, 256, 400, torch.bfloat16, dev)
        X = randn((16, 256), 401, 1.0, torch.bfloat16)
        assert_close(mlk.gemm_layoutA(A, X.to(dev)), odense.gemm_ref(X, W), "gemm with the tuner's row")
        assert_close(mlk.gemv_layoutA(A, X[:1].to(dev)), odense.gemm_ref(X[:1], W), "gemv with the tuner's row")
        log = list(csv.reader(open(tmp_path / "layoutA_gemm_scan_result.csv")))
        assert len(log) > 10 and all(r[-1] != "WRONG" for r in log)
    finally:
        load_tables()     # the packaged tables again
