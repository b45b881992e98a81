"""The expert-compute entry point that allocates nothing (mlk_fused_experts_compute_static), called through the
C ABI, against the regular entry point with a caller-provided combine buffer.

Who needs it: hosts that may not allocate device memory on the request path -- a plugin living inside another
runtime's memory pool, a serving loop with a frozen memory budget.  For them the fp32 combine
buffer is an 8 MiB array built into the library.  This file is named so that pytest collects it last.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(dev, seed, T, E, topk, H, I, plain=False):
    import muxi_native_layout_kernels_b200 as mlk
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).to(dev)
    w1_plain = (torch.randn(E, 2 * I, H, generator=g) * 0.05).to(torch.bfloat16)
    w2_plain = (torch.randn(E, H, I, generator=g) * 0.05).to(torch.bfloat16)
    w1 = mlk.layoutA(w1_plain.to(dev))
    w2 = mlk.layoutA(w2_plain.to(dev))
    ids = torch.stack([torch.randperm(E, generator=g)[:topk] for _ in range(T)]).to(torch.int32).to(dev)
    wts = torch.rand(T, topk, generator=g).to(torch.bfloat16).to(dev)
    if plain:
        return x, w1, w2, ids, wts, w1_plain, w2_plain
    return x, w1, w2, ids, wts


def _call(static, x, w1, w2, ids, wts, E, topk, H, I, emap=None, tune=None):
    from muxi_native_layout_kernels_b200._lib import check, lib
    T = x.shape[0]
    dev = x.device
    n = T * topk + E * 15
    sorted_ids = torch.full((n,), T * topk, dtype=torch.int32, device=dev)
    cumsum = torch.empty(E + 1, dtype=torch.int32, device=dev)
    nblk = torch.empty(1, dtype=torch.int32, device=dev)
    blk = torch.empty((n + 15) // 16, dtype=torch.int32, device=dev)
    C = torch.empty(topk * 2 * I * T, dtype=torch.bfloat16, device=dev)
    y = torch.zeros(T, H, dtype=torch.bfloat16, device=dev)
    status_word = torch.zeros(1, dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    e_local = w1.shape[0]
    common = (w1.data_ptr(), w2.data_ptr(), x.data_ptr(), T, e_local, topk, H, I, ids.data_ptr(), wts.data_ptr(),
              sorted_ids.data_ptr(), cumsum.data_ptr(), nblk.data_ptr(), blk.data_ptr(), C.data_ptr(), y.data_ptr(),
              None, None, 0, 0, 16, None if emap is None else emap.data_ptr(), 0 if emap is None else emap.numel())
    tune_arr = None if tune is None else (ctypes.c_int32 * 6)(*tune)
    if static:
        status = lib.mlk_fused_experts_compute_static(*common, tune_arr, status_word.data_ptr(), 0, stream)
    else:
        scratch = torch.empty(T * topk * H, dtype=torch.float32, device=dev)
        status = lib.mlk_fused_experts_compute(*common, scratch.data_ptr(), scratch.numel() * 4, tune_arr,
                                               status_word.data_ptr(), 0, stream)
    torch.cuda.synchronize()
    assert int(status_word.item()) == 0
    return status, y


def test_static_scratch_entry_point_matches_regular_one_twice_in_a_row():
    assert torch.cuda.is_available()
    dev = torch.device("cuda:0")
    E, topk, H, I = 16, 4, 256, 128
    # two different calls in a row: the second must not be disturbed by what the first left in the built-in array
    for seed, T in ((1234, 37), (4321, 12)):
        x, w1, w2, ids, wts = _inputs(dev, seed, T, E, topk, H, I)
        st_ref, y_ref = _call(False, x, w1, w2, ids, wts, E, topk, H, I)
        st_new, y_new = _call(True, x, w1, w2, ids, wts, E, topk, H, I)
        assert st_ref == 0 and st_new == 0
        assert bool(y_ref.float().abs().max() > 0)
        # same kernels, same fixed summation order: the two entry points agree bit for bit (well inside the
        # |diff| <= 1e-2 + 1e-2*|want| bar of the other MoE tests)
        assert torch.equal(y_new, y_ref), float((y_new.float() - y_ref.float()).abs().max())


def test_static_scratch_entry_point_other_kernel_families_and_the_oracle():
    """The built-in scratch under the warp-level kernels (an intermediate size that the 128-row tensor-core tiles do
    not divide), with explicit launch arguments, and with an expert map; one case is also held against the CPU
    oracle directly, not only against the other entry point."""
    from oracle import dense as odense
    from oracle import moe as omoe
    assert torch.cuda.is_available()
    dev = torch.device("cuda:0")
    # warp-level path: I = 96
    E, topk, H, I, T = 8, 2, 256, 96, 21
    x, w1, w2, ids, wts, w1_plain, w2_plain = _inputs(dev, 77, T, E, topk, H, I, plain=True)
    for tune in (None, (2, 2, 1, 1, 2, 1)):
        st_ref, y_ref = _call(False, x, w1, w2, ids, wts, E, topk, H, I, tune=tune)
        st_new, y_new = _call(True, x, w1, w2, ids, wts, E, topk, H, I, tune=tune)
        assert st_ref == 0 and st_new == 0 and torch.equal(y_new, y_ref)
    want = omoe.experts_ref(x.cpu(), w1_plain, w2_plain, ids.cpu().long(), wts.cpu(), compute_dtype=torch.float32)
    rep = odense.error_report(y_new.cpu(), want, scale_atol=True)
    assert rep["ok"], rep
    # expert map: only the odd experts are local (4 local experts); explicit tcgen05 launch arguments
    E, topk, H, I, T = 8, 2, 256, 128, 19
    x, w1, w2, ids, wts = _inputs(dev, 78, T, E, topk, H, I)
    emap = torch.tensor([-1, 0, -1, 1, -1, 2, -1, 3], dtype=torch.int32, device=dev)
    w1l = w1[1::2].contiguous()
    w2l = w2[1::2].contiguous()
    for tune in (None, (2, 103, 2, 0, 103, 2)):
        st_ref, y_ref = _call(False, x, w1l, w2l, ids, wts, E, topk, H, I, emap=emap, tune=tune)
        st_new, y_new = _call(True, x, w1l, w2l, ids, wts, E, topk, H, I, emap=emap, tune=tune)
        assert st_ref == 0 and st_new == 0 and torch.equal(y_new, y_ref)
        assert bool(y_ref.float().abs().max() > 0)


def test_static_scratch_entry_point_rejects_oversized_problem():
    from muxi_native_layout_kernels_b200._lib import lib
    assert torch.cuda.is_available()
    one = ctypes.c_void_p(256)    # never dereferenced: the size check comes before any launch
    # 4096 tokens x top-8 x 2048 hidden = 64 Mi floats > 2 Mi
    st = lib.mlk_fused_experts_compute_static(one, one, one, 4096, 128, 8, 2048, 768, one, one, one, one, one, one, one,
                                              one, None, None, 0, 0, 16, None, 0, None, None, 0, None)
    assert st == 1
    assert b"exceeds the built-in scratch" in lib.mlk_last_error()
