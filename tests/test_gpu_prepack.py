"""Prepack ops on the GPU against the index-formula oracle (bit-exact) and round trips at full sizes."""
import numpy as np
import pytest
import torch

from oracle import layouts as olay
from tests.gpu_util import require_gpu

pytestmark = pytest.mark.gpu


def _rand_bits(shape, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    if dtype == torch.uint8:
        return torch.randint(0, 256, shape, generator=g, dtype=torch.int64).to(torch.uint8)
    return torch.randint(-32768, 32767, shape, generator=g, dtype=torch.int64).to(torch.int16)


@pytest.mark.parametrize("m,k", [(16, 8), (16, 32), (32, 64), (48, 40), (256, 1000), (4096, 512)])
@pytest.mark.parametrize("esz", [1, 2])
def test_layoutA_matches_oracle_and_inverts(m, k, esz):
    import muxi_native_layout_kernels_b200 as mlk
    dev = require_gpu()
    bits = _rand_bits((m, k), 1, torch.uint8 if esz == 1 else torch.int16)
    t = bits.view(torch.float8_e4m3fn) if esz == 1 else bits.view(torch.bfloat16)
    A4 = mlk.layoutA(t.to(dev))
    assert A4.shape == (m // 16, k // 8, 16, 8)
    got = A4.cpu().view(bits.dtype).numpy()
    assert np.array_equal(got, olay.layout_a(bits.numpy()))
    back = mlk.layoutA_inverse(A4).cpu().view(bits.dtype)
    assert torch.equal(back, bits)


def test_layoutA_golden_and_batched(golden_dir):
    import muxi_native_layout_kernels_b200 as mlk
    dev = require_gpu()
    g = np.load(golden_dir / "layouts.npz")
    a = torch.from_numpy(g["a16_in"]).view(torch.float16).to(dev)
    assert np.array_equal(mlk.layoutA(a).cpu().view(torch.int16).numpy(), g["a16_out"])
    # 3-D [E,m,k]: every expert permuted on its own, shape kept (benchmark_and_test/test_muxi_moe.py:73-81)
    bits = _rand_bits((3, 32, 64), 5, torch.int16)
    out = mlk.layoutA(bits.view(torch.bfloat16).to(dev)).cpu().view(torch.int16)
    assert out.shape == (3, 32, 64)
    for e in range(3):
        assert np.array_equal(out[e].numpy().reshape(2, 8, 16, 8), olay.layout_a(bits[e].numpy()))


@pytest.mark.parametrize("n,k", [(16, 32), (32, 96), (64, 4096), (256, 14336)])
def test_layoutB_matches_oracle(n, k):
    import muxi_native_layout_kernels_b200 as mlk
    dev = require_gpu()
    bits = _rand_bits((n, k), 2, torch.int16)
    got = mlk.layoutB(bits.view(torch.bfloat16).to(dev))
    assert got.shape == (k // 32, n // 16, 4, 16, 8)
    assert np.array_equal(got.cpu().view(torch.int16).numpy(), olay.layout_b(bits.numpy()))


@pytest.mark.parametrize("n,m", [(16, 32), (32, 64), (64, 4096), (256, 14336)])
def test_reLayoutC_matches_oracle(n, m):
    import muxi_native_layout_kernels_b200 as mlk
    dev = require_gpu()
    bits = _rand_bits((m // 32, n // 16, 4, 16, 8), 3, torch.int16)
    got = mlk.reLayoutC(bits.view(torch.float16).to(dev))
    assert got.shape == (n, m)
    assert np.array_equal(got.cpu().view(torch.int16).numpy(), olay.layout_c_inverse(bits.numpy()))


def test_prepack_golden_b_c_repack(golden_dir):
    import muxi_native_layout_kernels_b200 as mlk
    dev = require_gpu()
    g = np.load(golden_dir / "layouts.npz")
    b = torch.from_numpy(g["b_in"]).view(torch.bfloat16).to(dev)
    assert np.array_equal(mlk.layoutB(b).cpu().view(torch.int16).numpy(), g["b_out"])
    c = torch.from_numpy(g["c_in"]).view(torch.bfloat16).to(dev)
    assert np.array_equal(mlk.reLayoutC(c).cpu().view(torch.int16).numpy(), g["c_out"])
    r = torch.from_numpy(g["repack_in"]).view(torch.float8_e4m3fn).to(dev)
    assert np.array_equal(mlk.fp8_weight_repack(r).cpu().view(torch.uint8).numpy(), g["repack_out"])


@pytest.mark.parametrize("shape", [(256, 256), (3, 256, 512), (5, 36)])
def test_fp8_repack_matches_oracle_and_is_involution(shape):
    import muxi_native_layout_kernels_b200 as mlk
    dev = require_gpu()
    bits = _rand_bits(shape, 4, torch.uint8)
    w = bits.view(torch.float8_e4m3fn).to(dev)
    rep = mlk.fp8_weight_repack(w)
    assert rep.shape == w.shape
    assert np.array_equal(rep.cpu().view(torch.uint8).numpy(), olay.fp8_repack(bits.numpy()))
    assert torch.equal(mlk.fp8_weight_repack(rep).view(torch.uint8), w.view(torch.uint8))


def test_full_size_round_trips():
    """Size-independent properties at the largest BASELINE shapes: inverse(layoutA(W)) == W, repack twice == id,
    and repack commutes with layout A (it acts inside the 8-byte chunks that layout A moves whole)."""
    import muxi_native_layout_kernels_b200 as mlk
    dev = require_gpu()
    g = torch.Generator(device=dev).manual_seed(7)
    w8 = torch.randint(0, 255, (28672, 8192), generator=g, device=dev, dtype=torch.int32).to(torch.uint8).view(torch.float8_e4m3fn)
    a = mlk.layoutA(w8)
    assert torch.equal(mlk.layoutA_inverse(a).view(torch.uint8), w8.view(torch.uint8))
    r1 = mlk.fp8_weight_repack(a.view(28672, 8192))
    r2 = mlk.layoutA(mlk.fp8_weight_repack(w8)).view(28672, 8192)
    assert torch.equal(r1.view(torch.uint8), r2.view(torch.uint8))
    assert torch.equal(mlk.fp8_weight_repack(r1).view(torch.uint8), a.view(28672, 8192).view(torch.uint8))
    w16 = torch.randn(14336, 4096, generator=g, device=dev).to(torch.bfloat16)
    assert torch.equal(mlk.layoutA_inverse(mlk.layoutA(w16)), w16)
    x = torch.randn(64, 14336, generator=g, device=dev).to(torch.float16)
    b5 = mlk.layoutB(x)
    assert torch.equal(b5.permute(1, 3, 0, 2, 4).reshape(64, 14336), x)


def test_prepack_argument_errors():
    import muxi_native_layout_kernels_b200 as mlk
    dev = require_gpu()
    with pytest.raises(RuntimeError, match="multiple of 16"):
        mlk.layoutB(torch.zeros(10, 32, dtype=torch.bfloat16, device=dev))
    with pytest.raises(RuntimeError, match="multiple of 32"):
        mlk.layoutB(torch.zeros(16, 48, dtype=torch.bfloat16, device=dev))
    with pytest.raises(RuntimeError, match="5D"):
        mlk.reLayoutC(torch.zeros(16, 48, dtype=torch.bfloat16, device=dev))
    with pytest.raises(RuntimeError, match="contiguous"):
        mlk.layoutB(torch.zeros(32, 64, dtype=torch.bfloat16, device=dev).t())
