"""Fused MoE on the GPU (through the C ABI) against the CPU oracle.

Three comparisons per case, as the arithmetic demands: kernel vs the fp32 evaluation with the same routing
decisions (the pass/fail bar: |diff| <= atol + 1e-2*|want| with atol = 1e-2 * max(1, rms(want))); kernel vs the
16-bit oracle (the reference's arithmetic, five intermediate roundings); 16-bit oracle vs fp32 (its own noise
floor).  The kernel must not be further from the 16-bit oracle than that floor plus the bar.  Expert ids must
match the oracle exactly; rows whose k-th and (k+1)-th scores are equal are compared as sets and counted.
"""
import pytest
import torch

import muxi_native_layout_kernels_b200 as mlk
from muxi_native_layout_kernels_b200.muxi_moe_planC import fused_moe as planC_moe
from oracle import dense as odense
from oracle import moe as omoe
from tests.gpu_util import DT, assert_close, rand_e4m3, randn, require_gpu

pytestmark = pytest.mark.gpu


# ----------------------------------------------------------------------------------------------------
# router
# ----------------------------------------------------------------------------------------------------

ROUTER_CASES = [
    # E, topk, groups, kept, bias, score
    (8, 2, 1, 1, False, "softmax"),
    (128, 8, 1, 1, False, "softmax"),
    (128, 8, 8, 4, False, "sigmoid"),
    (256, 8, 8, 4, True, "sigmoid"),
    (256, 8, 8, 4, True, "softmax"),
    (16, 4, 4, 2, True, "sigmoid"),
    (64, 6, 1, 1, False, "sigmoid"),
    (96, 5, 3, 2, False, "softmax"),
    (8, 8, 1, 1, False, "softmax"),
]


@pytest.mark.parametrize("dt", ["bf16", "fp16"])
@pytest.mark.parametrize("case", ROUTER_CASES)
def test_router_matches_oracle(case, dt):
    dev = require_gpu()
    E, topk, G, KG, use_bias, score = case
    for T in (1, 7, 64, 513):
        logits = randn((T, E), 300 + T + E, 1.0, DT[dt])
        bias = randn((E,), 301, 0.1, DT[dt]) if use_bias else None
        ids = torch.empty(T, topk, dtype=torch.int32, device=dev)
        w = torch.empty(T, topk, dtype=DT[dt], device=dev)
        mlk.fused_routing_gate(logits.to(dev), 0 if score == "softmax" else 1, T, 0, G, KG, ids, w, topk,
                               None if bias is None else bias.to(dev))
        ids_ref, w_ref, masked = omoe.router_ref(logits, topk, G, KG, bias, score)
        rep = omoe.compare_topk(ids.cpu(), ids_ref, masked)
        assert rep["mismatch_rows"] == 0, (case, T, rep)
        # weights travel with ids: compare per (row, expert) where the sets agree
        got = torch.zeros(T, E).scatter_(1, ids.cpu().long(), w.float().cpu())
        want = torch.zeros(T, E).scatter_(1, ids_ref, w_ref.float())
        same = (torch.sort(ids.cpu().long(), -1)[0] == torch.sort(ids_ref, -1)[0]).all(-1)
        assert_close(got[same], want[same], f"router weights {case} T={T}", atol=1e-3, rtol=1e-2)
        # output order: ascending expert id for softmax (csrc/moe_kernels/fused_topK.h:294-306)
        if score == "softmax":
            assert bool((ids[:, 1:] > ids[:, :-1]).all()) or topk == 1


@pytest.mark.parametrize("dt", ["bf16", "fp16"])
@pytest.mark.parametrize("T,E,H,topk,groups,kept,score", [(1, 8, 4096, 2, 1, 1, 0), (5, 128, 2048, 8, 8, 4, 1),
                                                         (33, 64, 512, 6, 1, 1, 0), (130, 256, 256, 8, 4, 2, 1)])
def test_router_gemm_fused_with_routing(dt, T, E, H, topk, groups, kept, score):
    """fused_router_gemm_gate: the logits it produces are the fp32 dot products rounded once (within one ulp of the exact
    products summed in float64 on the host), and its routing is bit-identical to fused_routing_gate applied
    to those logits."""
    dev = require_gpu()
    x = randn((T, H), 950 + T, 1.0, DT[dt]).to(dev)
    wg = randn((E, H), 951, 0.05, DT[dt]).to(dev)
    bias = (randn((E,), 952, 0.1, DT[dt]).to(dev)) if score == 1 else None
    ids = torch.empty(T, topk, dtype=torch.int32, device=dev)
    wts = torch.empty(T, topk, dtype=DT[dt], device=dev)
    logits = torch.empty(T, E, dtype=DT[dt], device=dev)
    mlk.fused_router_gemm_gate(x, wg, score, groups, kept, ids, wts, topk, bias, renormalize=True, logits_out=logits)
    want = x.cpu().double() @ wg.cpu().double().t()     # exact products on the host: no device library in the check
    ulp = 2.0 ** (-7 if dt == "bf16" else -10)      # spacing of the 16-bit type relative to the value
    # one rounding to the 16-bit type, plus what an fp32 sum over H terms may differ from the exact one
    assert bool(((logits.cpu().double() - want).abs() <= ulp * want.abs().clamp_min(2.0 ** -14) * 1.01 + 2e-5).all())
    ids2 = torch.empty_like(ids)
    wts2 = torch.empty_like(wts)
    mlk.fused_routing_gate(logits, score, T, H, groups, kept, ids2, wts2, topk, bias, renormalize=True)
    torch.cuda.synchronize()
    assert torch.equal(ids, ids2) and torch.equal(wts, wts2)


def test_fused_moe_with_gate_weight_matches_layer_on_its_logits():
    dev = require_gpu()
    E, topk, H, I, T = 16, 4, 256, 128, 21
    x = randn((T, H), 960, 1.0).to(dev)
    wg = randn((E, H), 961, 0.05).to(dev)
    w1 = mlk.layoutA(randn((E, 2 * I, H), 962, 0.05).to(dev))
    w2 = mlk.layoutA(randn((E, H, I), 963, 0.05).to(dev))
    ids = torch.empty(T, topk, dtype=torch.int32, device=dev)
    wts = torch.empty(T, topk, dtype=torch.bfloat16, device=dev)
    logits = torch.empty(T, E, dtype=torch.bfloat16, device=dev)
    mlk.fused_router_gemm_gate(x, wg, 0, 1, 1, ids, wts, topk, renormalize=True, logits_out=logits)
    y_fused = planC_moe(x, w1, w2, None, topk, True, gate_weight=wg)
    y_plain = planC_moe(x, w1, w2, logits, topk, True)
    torch.cuda.synchronize()
    assert torch.equal(y_fused, y_plain)


def test_router_ties_prefer_lower_id():
    dev = require_gpu()
    logits = torch.zeros(3, 64, dtype=torch.bfloat16)
    logits[1, 40:] = 1.0
    logits[2, ::2] = 2.0
    for score in (0, 1):
        ids = torch.empty(3, 4, dtype=torch.int32, device=dev)
        w = torch.empty(3, 4, dtype=torch.bfloat16, device=dev)
        mlk.fused_routing_gate(logits.to(dev), score, 3, 0, 1, 1, ids, w, 4)
        assert ids.cpu().tolist() == [[0, 1, 2, 3], [40, 41, 42, 43], [0, 2, 4, 6]]


def test_router_errors():
    dev = require_gpu()
    logits = torch.zeros(2, 64, dtype=torch.bfloat16, device=dev)
    ids = torch.empty(2, 4, dtype=torch.int32, device=dev)
    w = torch.empty(2, 4, dtype=torch.bfloat16, device=dev)
    with pytest.raises(RuntimeError, match="n_groups"):
        mlk.fused_routing_gate(logits, 0, 2, 0, 5, 1, ids, w, 4)
    with pytest.raises(RuntimeError, match="score_fun"):
        mlk.fused_routing_gate(logits, 3, 2, 0, 1, 1, ids, w, 4)
    with pytest.raises(RuntimeError, match="kInt32"):
        mlk.fused_routing_gate(logits, 0, 2, 0, 1, 1, ids.to(torch.int64), w, 4)


# ----------------------------------------------------------------------------------------------------
# token alignment
# ----------------------------------------------------------------------------------------------------

def _run_align(ids, E, mbs, emap, dev):
    T, topk = ids.shape
    n = T * topk + E * (mbs - 1)
    sorted_ids = torch.full((n,), T * topk, dtype=torch.int32, device=dev)
    cumsum = torch.empty(E + 1, dtype=torch.int32, device=dev)
    nblk = torch.empty(1, dtype=torch.int32, device=dev)
    blk = torch.full(((n + mbs - 1) // mbs,), -7, dtype=torch.int32, device=dev)
    mlk.batched_routed_activation_indexed_to_expert_block_indexed(T, E, topk, mbs, ids.to(dev), sorted_ids, cumsum, nblk,
                                                                  blk, None if emap is None else emap.to(dev))
    return sorted_ids.cpu(), cumsum.cpu(), int(nblk.item()), blk.cpu()


@pytest.mark.parametrize("T,E,topk,mbs", [(1, 8, 2, 16), (64, 8, 2, 16), (37, 128, 8, 16), (512, 128, 8, 16),
                                          (2048, 256, 8, 16), (5, 4, 1, 4), (300, 1024, 4, 16)])
def test_align_contract(T, E, topk, mbs):
    dev = require_gpu()
    g = torch.Generator().manual_seed(400 + T)
    ids = torch.stack([torch.randperm(E, generator=g)[:topk] for _ in range(T)]).to(torch.int32)
    for emap in (None, torch.where(torch.arange(E) % 2 == 0, torch.arange(E) // 2, torch.full((E,), -1)).to(torch.int32)):
        E_loc = E if emap is None else (E + 1) // 2
        s, cumsum, nblk, blk = _run_align(ids, E_loc if emap is not None else E, mbs, emap, dev)
        r = omoe.align_ref(ids, E_loc, mbs, emap)
        assert nblk == r["num_blocks"]
        assert blk[:nblk].tolist() == r["block_expert"].tolist()
        assert bool((blk[nblk:] == 0).all())                      # zero-filled beyond the used blocks
        assert cumsum.tolist() == r["cumsum_after"].tolist()
        for e in range(E_loc):
            st, c = int(r["starts"][e]), int(r["counts"][e])
            assert sorted(s[st:st + c].tolist()) == r["slots_of"][e].tolist()      # any order inside an expert
            pad_end = st + (c + mbs - 1) // mbs * mbs
            assert bool((s[st + c:pad_end] == T * topk).all())                     # padding keeps the sentinel
        assert bool((s[r["padded_total"]:] == T * topk).all())


def test_align_reference_smoke_vector():
    """Same problem shape as the reference's print-only driver (csrc/moe_kernels/test_moe_align_tokens.cc: 8 tokens
    x top-8 over 16 experts, ids generated here); the driver records no expected output, so the contract is checked."""
    dev = require_gpu()
    ids = (torch.arange(64, dtype=torch.int32).reshape(8, 8) * 5 + 3) % 16
    ids = torch.stack([torch.sort(r)[0] for r in ids])
    s, cumsum, nblk, blk = _run_align(ids, 16, 16, None, dev)
    r = omoe.align_ref(ids, 16, 16)
    assert nblk == r["num_blocks"] and cumsum.tolist() == r["cumsum_after"].tolist()


# ----------------------------------------------------------------------------------------------------
# whole layer
# ----------------------------------------------------------------------------------------------------

def _kernel_routing(x, logits, topk, renorm, groups, kept, bias, score, dev):
    """Router kernel output, checked (tie-aware) against the oracle's routing and then used for the expert-compute
    oracle, so that a tie at the top-k cut cannot turn into a spurious output mismatch."""
    T = x.shape[0]
    ids = torch.empty(T, topk, dtype=torch.int32, device=dev)
    w = torch.empty(T, topk, dtype=x.dtype, device=dev)
    mlk.fused_routing_gate(logits.to(dev), 0 if score == "softmax" else 1, T, x.shape[1], groups, kept, ids, w, topk,
                           None if bias is None else bias.to(dev))
    ids_ref, _, masked = omoe.router_ref(logits, topk, groups, kept, bias, score)
    rep = omoe.compare_topk(ids.cpu(), ids_ref, masked)
    assert rep["mismatch_rows"] == 0, rep
    w = w.cpu()
    if renorm:
        w = w / w.sum(dim=-1, keepdim=True)      # in the activation dtype, as planC does
    return ids.cpu().long(), w


def _moe_compare(x, w1, w2, logits, topk, what, renorm=True, groups=1, kept=1, bias=None, score="softmax", fp8=False,
                 scales=None, repack=False, dev=None, tune=None):
    dev = dev or require_gpu()
    E = w1.shape[0]
    w1d, w2d = mlk.layoutA(w1.to(dev)), mlk.layoutA(w2.to(dev))
    if repack:
        w1d, w2d = mlk.fp8_weight_repack(w1d), mlk.fp8_weight_repack(w2d)
    s1 = s2 = None
    if scales is not None:
        s1, s2 = scales[0].to(dev), scales[1].to(dev)
    y = planC_moe(x.to(dev), w1d, w2d, logits.to(dev), topk, renorm, use_grouped_topk=groups > 1,
                  num_expert_group=groups, topk_group=kept, w1_scale=s1, w2_scale=s2,
                  block_shape=[128, 128] if fp8 else None, gating_bias=None if bias is None else bias.to(dev),
                  score_func=score, soft_fp8=fp8, fp8_repacked=repack, tune=tune)
    torch.cuda.synchronize()
    # oracle weights: e4m3 (+ scales) dequantised as the reference's test does (scale_whole_tensor)
    if fp8 and scales is not None:
        w1o = torch.stack([odense.dequant_block_scaled(w1[e], scales[0][e]) for e in range(E)])
        w2o = torch.stack([odense.dequant_block_scaled(w2[e], scales[1][e]) for e in range(E)])
        # the fp32 yardstick uses the unrounded product weight * scale (the kernels scale fp32 block sums)
        w1x = torch.stack([odense.dequant_exact_scale(w1[e], scales[0][e]) for e in range(E)])
        w2x = torch.stack([odense.dequant_exact_scale(w2[e], scales[1][e]) for e in range(E)])
    else:
        w1o, w2o, w1x, w2x = w1, w2, w1, w2
    ids, w = _kernel_routing(x, logits, topk, renorm, groups, kept, bias, score, dev)
    y16 = omoe.experts_ref(x, w1o, w2o, ids, w)
    y32 = omoe.experts_ref(x, w1x, w2x, ids, w, compute_dtype=torch.float32)
    floor = odense.error_report(y16, y32, scale_atol=True)
    rep32 = odense.error_report(y.cpu(), y32, scale_atol=True)
    rep16 = odense.error_report(y.cpu(), y16, scale_atol=True)
    print(what, "kernel-vs-fp32", rep32, "kernel-vs-16bit", rep16, "floor", floor)
    # within the path's tolerance of the fp32 yardstick, or (kernels that round the block-scaled weights to bf16, as the
    # reference's do) at least as close to it as the reference's own 16-bit recipe is
    assert rep32["ok"] or rep32["max_abs"] <= 1.1 * floor["max_abs"], (what, rep32, floor)
    assert rep16["max_abs"] <= floor["max_abs"] * 1.5 + 1e-2 * max(1.0, float(y32.abs().max())), (what, rep16, floor)
    return y


@pytest.mark.parametrize("name", ["softmax_top2", "sigmoid_grouped_bias", "fp16_softmax", "fp8_top8"])
def test_moe_golden_fixtures(golden_dir, name):
    """The fused layer against outputs of the reference's own torch fused_moe (tests/golden/make_golden.py)."""
    dev = require_gpu()
    g = torch.load(golden_dir / f"moe_{name}.pt")
    w1, w2 = g["w1"], g["w2"]
    if g["fp8"]:
        w1, w2 = w1.view(torch.float8_e4m3fn), w2.view(torch.float8_e4m3fn)
    y = _moe_compare(g["x"], w1, w2, g["logits"], g["topk"], name, g["renormalize"], g["groups"], g["topk_group"],
                     g["bias"], g["score_func"], g["fp8"], dev=dev)
    # the stored reference output itself, with the reference test's own tolerance (test_muxi_moe.py:111)
    # (its atol 0.1 / rtol 0.05 are meant for outputs well below 1; the absolute part is scaled with the output rms)
    rep = odense.error_report(y.cpu(), g["y"], atol=0.1, rtol=0.05, scale_atol=True)
    assert rep["ok"], rep


@pytest.mark.parametrize("dt", ["bf16", "fp16"])
@pytest.mark.parametrize("T", [1, 3, 8, 16, 33, 64, 100, 257])
def test_moe_16bit_random(dt, T):
    E, topk, H, I = 16, 4, 256, 160
    x = randn((T, H), 500 + T, 1.0, DT[dt])
    w1 = randn((E, 2 * I, H), 501, 0.05, DT[dt])
    w2 = randn((E, H, I), 502, 0.05, DT[dt])
    logits = randn((T, E), 503 + T, 1.0, DT[dt])
    _moe_compare(x, w1, w2, logits, topk, f"moe {dt} T={T}")


@pytest.mark.parametrize("dt", ["bf16", "fp16"])
@pytest.mark.parametrize("T", [40, 64, 100, 257, 600])
def test_moe_16bit_tcgen05_expert_gemms(dt, T):
    """tune = (token tiles, 100 + stages, cluster, -, 100 + stages, cluster): the tcgen05 expert GEMMs (gathered token
    rows, gate/up tile pair with fused SiLU*up, routing-weighted fp32 rows), same oracle and tolerance."""
    E, topk, H, I = 8, 2, 256, 384
    x = randn((T, H), 700 + T, 1.0, DT[dt])
    w1 = randn((E, 2 * I, H), 701, 0.05, DT[dt])
    w2 = randn((E, H, I), 702, 0.05, DT[dt])
    logits = randn((T, E), 703 + T, 1.0, DT[dt])
    for tune in [(2, 102, 1, 0, 102, 1), (4, 103, 2, 0, 104, 3), (8, 104, 4, 0, 106, 6), (1, 102, 2, 0, 103, 2),
                 (16, 102, 2, 0, 103, 2)]:
        y = _moe_compare(x, w1, w2, logits, topk, f"moe tcgen05 {dt} T={T} tune={tune}", tune=tune)
        y0 = _moe_compare(x, w1, w2, logits, topk, f"moe warp-level {dt} T={T}", tune=(min(tune[0], 8), 2, 1, 1, 2, 1))
        # both paths sum the same fp32 products in different orders: results agree to rounding
        assert_close(y, y0.cpu(), f"tcgen05 vs warp-level {dt} T={T} tune={tune}", scale_atol=True)


@pytest.mark.parametrize("T", [1, 8, 32, 130, 520])
@pytest.mark.parametrize("repack", [False, True])
def test_moe_soft_fp8_tcgen05_expert_gemms(T, repack):
    """e4m3 experts with unit scales on the tcgen05 kernels (decode into tensor memory), against the same oracle
    and against the warp-level kernels."""
    E, topk, H, I = 32, 8, 256, 128
    x = randn((T, H), 800 + T, 1.0)
    w1 = rand_e4m3((E, 2 * I, H), 801, 0.25)
    w2 = rand_e4m3((E, H, I), 802, 0.25)
    logits = randn((T, E), 803 + T, 1.0)
    for tune in [(1, 102, 1, 0, 102, 1), (2, 103, 2, 0, 104, 2), (4, 104, 4, 0, 106, 1), (8, 102, 2, 0, 103, 2)]:
        y = _moe_compare(x, w1, w2, logits, topk, f"moe fp8 tcgen05 T={T} repack={repack} tune={tune}", fp8=True,
                         repack=repack, tune=tune)
        y0 = _moe_compare(x, w1, w2, logits, topk, f"moe fp8 warp-level T={T}", fp8=True, repack=repack,
                          tune=(tune[0], 2, 1, 1, 2, 1))
        assert_close(y, y0.cpu(), f"fp8 tcgen05 vs warp-level T={T} tune={tune}", scale_atol=True)


@pytest.mark.parametrize("T", [1, 8, 32, 130, 520])
@pytest.mark.parametrize("repack", [False, True])
def test_moe_soft_fp8_native_tensor_core_expert_gemms(T, repack):
    """e4m3 experts on the native-e4m3 tcgen05 kernels (tuning values 200 + stages: weight bytes undecoded into the
    8-bit MMA, activation rows as two e4m3 terms, the activation of the first GEMM split in place), against the same
    oracle and against the warp-level kernels; with an expert map; and with block scales, where the same tuning
    arguments must run the decode kernels instead."""
    E, topk, H, I = 32, 8, 256, 128
    x = randn((T, H), 900 + T, 1.0)
    w1 = rand_e4m3((E, 2 * I, H), 901, 0.25)
    w2 = rand_e4m3((E, H, I), 902, 0.25)
    logits = randn((T, E), 903 + T, 1.0)
    for tune in [(1, 202, 1, 0, 202, 1), (2, 203, 2, 0, 204, 2), (4, 204, 4, 0, 206, 1), (8, 202, 2, 0, 203, 2),
                 (2, 203, 1, 0, 203, 12), (4, 203, 2, 0, 202, 11), (8, 204, 1, 0, 204, 18),
                 (2, 203, 1, 0, 243, 11), (4, 204, 1, 0, 242, 12), (8, 203, 1, 0, 244, 14),
                 (8, 242, 1, 0, 203, 12), (8, 243, 1, 0, 242, 14)]:
        y = _moe_compare(x, w1, w2, logits, topk, f"moe fp8 native T={T} repack={repack} tune={tune}", fp8=True,
                         repack=repack, tune=tune)
        y0 = _moe_compare(x, w1, w2, logits, topk, f"moe fp8 warp-level T={T}", fp8=True, repack=repack,
                          tune=(tune[0], 2, 1, 1, 2, 1))
        assert_close(y, y0.cpu(), f"fp8 native vs warp-level T={T} tune={tune}", scale_atol=True)
    g = torch.Generator().manual_seed(904)
    scales = (torch.rand(E, 2 * I // 128, H // 128, generator=g) * 0.5 + 0.01,
              torch.rand(E, H // 128, I // 128, generator=g) * 0.5 + 0.01)
    _moe_compare(x, w1, w2, logits, topk, f"moe fp8 native tuning with scales T={T}", fp8=True, scales=scales, repack=repack,
                 tune=(2, 203, 2, 0, 203, 2))


@pytest.mark.parametrize("T", [1, 2, 5, 8])
@pytest.mark.parametrize("kind", ["bf16", "fp16", "fp8", "fp8_repacked", "fp8_scaled"])
def test_moe_decode_single_kernel(kind, T):
    """Tuning values of 300 in both row-warp fields: the whole expert compute of a decode batch (at most 8 tokens, 64
    routed slots) as one cooperative kernel with the weights streamed through a shared-memory ring by bulk copies.
    Against the oracle and the warp-level three-launch path; replays must agree bit for bit (fixed summation orders,
    and the kernel's counters must come back to zero between launches)."""
    dev = require_gpu()
    E, topk, H, I = 32, 8, 256, 128
    fp8 = kind.startswith("fp8")
    dt = torch.float16 if kind == "fp16" else torch.bfloat16
    x = randn((T, H), 1000 + T, 1.0, dt)
    logits = randn((T, E), 1003 + T, 1.0, dt)
    scales = None
    if fp8:
        w1 = rand_e4m3((E, 2 * I, H), 1001, 0.25)
        w2 = rand_e4m3((E, H, I), 1002, 0.25)
        if kind == "fp8_scaled":
            g = torch.Generator().manual_seed(1004)
            scales = (torch.rand(E, 2 * I // 128, H // 128, generator=g) * 0.5 + 0.01,
                      torch.rand(E, H // 128, I // 128, generator=g) * 0.5 + 0.01)
    else:
        w1 = randn((E, 2 * I, H), 1001, 0.05, dt)
        w2 = randn((E, H, I), 1002, 0.05, dt)
    repack = kind == "fp8_repacked"
    y0 = _moe_compare(x, w1, w2, logits, topk, f"moe warp-level {kind} T={T}", fp8=fp8, scales=scales, repack=repack,
                      tune=(1, 2, 1, 1, 2, 1))
    tune = (1, 300, 1, 0, 300, 1)
    first = None
    for rep in range(4):
        y = _moe_compare(x, w1, w2, logits, topk, f"moe decode {kind} T={T}", fp8=fp8, scales=scales, repack=repack, tune=tune)
        assert_close(y, y0.float().cpu(), f"decode kernel vs warp-level {kind} T={T}", scale_atol=True)
        first = y if first is None else first
        assert torch.equal(y, first), (kind, T, rep)
    assert mlk.kernel_status() == 0


@pytest.mark.parametrize("kind", ["bf16", "fp8", "fp8_scaled"])
@pytest.mark.parametrize("T,E,topk,H,I", [(1, 8, 2, 1024, 3584), (3, 16, 4, 2048, 768), (8, 64, 8, 512, 1536), (2, 8, 8, 96, 160)])
def test_moe_decode_single_kernel_shapes(kind, T, E, topk, H, I):
    """Shapes that exercise the ring: more segments per unit than consumer warps (K = 3584 in 16-bit = 14 segments),
    segment counts that do not divide the warps (3, 5, 6), several laps of the ring, K not a multiple of 128."""
    if kind == "fp8_scaled" and (H % 128 or I % 128):
        pytest.skip("block scales need multiples of 128")
    fp8 = kind.startswith("fp8")
    x = randn((T, H), 1300 + T, 1.0)
    logits = randn((T, E), 1303 + T, 1.0)
    scales = None
    if fp8:
        w1 = rand_e4m3((E, 2 * I, H), 1301, 0.25)
        w2 = rand_e4m3((E, H, I), 1302, 0.25)
        if kind == "fp8_scaled":
            g = torch.Generator().manual_seed(1304)
            scales = (torch.rand(E, 2 * I // 128, H // 128, generator=g) * 0.5 + 0.01,
                      torch.rand(E, H // 128, I // 128, generator=g) * 0.5 + 0.01)
    else:
        w1 = randn((E, 2 * I, H), 1301, 0.03)
        w2 = randn((E, H, I), 1302, 0.03)
    _moe_compare(x, w1, w2, logits, topk, f"moe decode {kind} {(T, E, topk, H, I)}", fp8=fp8, scales=scales,
                 tune=(1, 300, 1, 0, 300, 1))
    assert mlk.kernel_status() == 0


def test_moe_decode_single_kernel_expert_map_and_fallback():
    dev = require_gpu()
    E, topk, H, I, T = 16, 4, 128, 128, 6
    x = randn((T, H), 1100).to(dev)
    w1 = mlk.layoutA(randn((E, 2 * I, H), 1101, 0.05).to(dev))
    w2 = mlk.layoutA(randn((E, H, I), 1102, 0.05).to(dev))
    logits = randn((T, E), 1103).to(dev)
    tune = (1, 300, 1, 0, 300, 1)
    full = planC_moe(x, w1, w2, logits, topk, True, tune=tune)
    assert_close(full, planC_moe(x, w1, w2, logits, topk, True, tune=(1, 2, 1, 1, 2, 1)).float().cpu(), 'decode vs warp-level')
    assert torch.equal(planC_moe(x[:1], w1, w2, logits[:1], topk, True, tune=tune), full[:1])
    acc = torch.zeros(T, H, dtype=torch.float32, device=dev)
    for rank in range(4):
        lo = rank * 4
        emap = torch.full((E,), -1, dtype=torch.int32)
        emap[lo:lo + 4] = torch.arange(4, dtype=torch.int32)
        part = planC_moe(x, w1[lo:lo + 4].contiguous(), w2[lo:lo + 4].contiguous(), logits, topk, True,
                         experts_map=emap.to(dev), tune=tune, out_dtype=torch.float32)
        assert part.dtype == torch.float32
        acc += part
    assert_close(acc.to(torch.bfloat16), full.float().cpu(), "decode kernel, EP shares", atol=2e-2, rtol=2e-2)
    # 40 tokens are more than the kernel takes: the same tuning row runs the library's own choice
    T2 = 40
    x2, l2 = randn((T2, H), 1104).to(dev), randn((T2, E), 1105).to(dev)
    assert_close(planC_moe(x2, w1, w2, l2, topk, True, tune=tune), planC_moe(x2, w1, w2, l2, topk, True).float().cpu(),
                 "decode tuning on a large batch", atol=2e-2, rtol=2e-2)
    assert mlk.kernel_status() == 0


@pytest.mark.parametrize("case", ROUTER_CASES)
@pytest.mark.parametrize("T", [1, 4, 8])
def test_moe_decode_single_kernel_routes_like_the_router_kernel(case, T):
    """With the routing fused in front (one launch for the whole layer) topk_ids / topk_weights must equal the router
    kernel's bit for bit, and the layer must equal the two-call form bit for bit, for every routing configuration."""
    dev = require_gpu()
    E, topk, G, KG, use_bias, score = case
    if T * topk > 64:
        pytest.skip("more routed slots than the single-kernel path takes")
    H, I = 128, 64
    x = randn((T, H), 1400 + T).to(dev)
    logits = randn((T, E), 1401 + T + E).to(dev)
    bias = randn((E,), 1402, 0.1).to(dev) if use_bias else None
    w1 = mlk.layoutA(randn((E, 2 * I, H), 1403, 0.05).to(dev))
    w2 = mlk.layoutA(randn((E, H, I), 1404, 0.05).to(dev))
    sf = 0 if score == "softmax" else 1
    ids0 = torch.empty(T, topk, dtype=torch.int32, device=dev)
    wts0 = torch.empty(T, topk, dtype=torch.bfloat16, device=dev)
    mlk.fused_routing_gate(logits, sf, T, H, G, KG, ids0, wts0, topk, bias, renormalize=True)
    mbs = 16
    n = T * topk + E * (mbs - 1)

    def run(routing, ids, wts):
        bufs = [torch.empty(n, dtype=torch.int32, device=dev), torch.empty(E + 1, dtype=torch.int32, device=dev),
                torch.empty(1, dtype=torch.int32, device=dev), torch.empty((n + mbs - 1) // mbs, dtype=torch.int32, device=dev)]
        C = torch.empty(T * topk * 2 * I, dtype=torch.bfloat16, device=dev)
        y = torch.zeros(T, H, dtype=torch.bfloat16, device=dev)
        mlk.fused_experts_compute(w1, w2, x, T, E, topk, ids, wts, *bufs, C, y, microBatchSize=mbs,
                                  tune=(1, 300, 1, 0, 300, 1), routing=routing)
        return y

    y0 = run(None, ids0, wts0)
    ids1 = torch.full_like(ids0, -5)
    wts1 = torch.zeros_like(wts0)
    y1 = run((logits, sf, G, KG, bias, True), ids1, wts1)
    torch.cuda.synchronize()
    assert torch.equal(ids1, ids0) and torch.equal(wts1, wts0), case
    assert torch.equal(y1, y0), case
    # the same call with a tuning row of another family: router kernel + expert kernels inside the one library call
    ids2 = torch.full_like(ids0, -5)
    wts2 = torch.zeros_like(wts0)
    bufs = [torch.empty(n, dtype=torch.int32, device=dev), torch.empty(E + 1, dtype=torch.int32, device=dev),
            torch.empty(1, dtype=torch.int32, device=dev), torch.empty((n + mbs - 1) // mbs, dtype=torch.int32, device=dev)]
    y2 = torch.zeros(T, H, dtype=torch.bfloat16, device=dev)
    mlk.fused_experts_compute(w1, w2, x, T, E, topk, ids2, wts2, *bufs, torch.empty(T * topk * 2 * I, dtype=torch.bfloat16, device=dev),
                              y2, microBatchSize=mbs, tune=(1, 2, 1, 1, 2, 1), routing=(logits, sf, G, KG, bias, True))
    torch.cuda.synchronize()
    assert torch.equal(ids2, ids0) and torch.equal(wts2, wts0), case
    assert_close(y2, y0.float().cpu(), f"routed call, warp-level kernels {case}")
    assert mlk.kernel_status() == 0


@pytest.mark.parametrize("T,E,topk,mapped", [(1, 8, 2, False), (8, 128, 8, False), (5, 16, 4, True)])
def test_moe_decode_single_kernel_leaves_the_alignment_outputs(T, E, topk, mapped):
    """The single-kernel path fills sorted_token_ids / cumsum_buffer / padded_num_experts / experts_ids as the
    stand-alone alignment op does (slot order inside an expert is unspecified in the contract)."""
    dev = require_gpu()
    H, I, mbs = 128, 64, 16
    g = torch.Generator().manual_seed(1200 + T)
    ids = torch.stack([torch.randperm(E, generator=g)[:topk] for _ in range(T)]).to(torch.int32)
    emap = None
    n_local = E
    if mapped:
        n_local = E // 2
        emap = torch.full((E,), -1, dtype=torch.int32)
        emap[::2] = torch.arange(n_local, dtype=torch.int32)
    want_sorted, want_cumsum, want_nblk, want_blk = _run_align(ids, n_local, mbs, emap, dev)
    x = randn((T, H), 1201).to(dev)
    w1 = mlk.layoutA(randn((n_local, 2 * I, H), 1202, 0.05).to(dev))
    w2 = mlk.layoutA(randn((n_local, H, I), 1203, 0.05).to(dev))
    wts = torch.full((T, topk), 1.0 / topk, dtype=torch.bfloat16, device=dev)
    n = T * topk + n_local * (mbs - 1)
    sorted_ids = torch.full((n,), -3, dtype=torch.int32, device=dev)
    cumsum = torch.full((n_local + 1,), -3, dtype=torch.int32, device=dev)
    nblk = torch.full((1,), -3, dtype=torch.int32, device=dev)
    blk = torch.full(((n + mbs - 1) // mbs,), -3, dtype=torch.int32, device=dev)
    C = torch.empty(T * topk * 2 * I, dtype=torch.bfloat16, device=dev)
    y = torch.zeros(T, H, dtype=torch.bfloat16, device=dev)
    mlk.fused_experts_compute(w1, w2, x, T, n_local, topk, ids.to(dev), wts, sorted_ids, cumsum, nblk, blk, C, y,
                              microBatchSize=mbs, experts_map=None if emap is None else emap.to(dev),
                              tune=(1, 300, 1, 0, 300, 1))
    torch.cuda.synchronize()
    assert torch.equal(cumsum.cpu(), want_cumsum) and int(nblk.item()) == want_nblk
    assert torch.equal(blk.cpu(), want_blk)
    got_sorted = sorted_ids.cpu()
    start = 0
    for e in range(n_local):
        end = int(want_cumsum[e])
        padded_end = start + ((end - start + mbs - 1) // mbs) * mbs
        assert sorted(got_sorted[start:end].tolist()) == sorted(want_sorted[start:end].tolist())
        assert bool((got_sorted[end:padded_end] == T * topk).all())
        start = padded_end
    assert bool((got_sorted[start:] == T * topk).all())


@pytest.mark.parametrize("T", [1, 32, 130])
@pytest.mark.parametrize("repack", [False, True])
def test_moe_soft_fp8_tcgen05_block_scales(T, repack):
    """e4m3 experts WITH 128x128 block scales on the tcgen05 kernels: the decode yields rne_bf16(w * s), the weights
    the reference's torch recipe dequantises to; compared with the oracle and with the warp-level kernels."""
    E, topk, H, I = 32, 8, 256, 256
    x = randn((T, H), 810 + T, 1.0)
    w1 = rand_e4m3((E, 2 * I, H), 811, 0.25)
    w2 = rand_e4m3((E, H, I), 812, 0.25)
    logits = randn((T, E), 813 + T, 1.0)
    g = torch.Generator().manual_seed(814)
    scales = (torch.rand(E, 2 * I // 128, H // 128, generator=g) * 0.5 + 0.01,
              torch.rand(E, H // 128, I // 128, generator=g) * 0.5 + 0.01)
    for tune in [(1, 102, 1, 0, 102, 1), (2, 103, 2, 0, 104, 2), (8, 104, 4, 0, 103, 2)]:
        y = _moe_compare(x, w1, w2, logits, topk, f"moe fp8 tcgen05 scaled T={T} repack={repack} tune={tune}", fp8=True,
                         scales=scales, repack=repack, tune=tune)
        y0 = _moe_compare(x, w1, w2, logits, topk, f"moe fp8 warp-level scaled T={T}", fp8=True, scales=scales,
                          repack=repack, tune=(tune[0], 2, 1, 1, 2, 1))
        assert_close(y, y0.cpu(), f"fp8 tcgen05 vs warp-level, scaled, T={T} tune={tune}", scale_atol=True)


@pytest.mark.parametrize("T", [1, 8, 32, 130])
@pytest.mark.parametrize("repack", [False, True])
def test_moe_soft_fp8_random(T, repack):
    E, topk, H, I = 32, 8, 256, 128
    x = randn((T, H), 600 + T, 1.0)
    w1 = rand_e4m3((E, 2 * I, H), 601, 0.25)
    w2 = rand_e4m3((E, H, I), 602, 0.25)
    logits = randn((T, E), 603 + T, 1.0)
    _moe_compare(x, w1, w2, logits, topk, f"moe fp8 T={T} repack={repack}", fp8=True, repack=repack)
    g = torch.Generator().manual_seed(604)
    scales = (torch.rand(E, 2 * I // 128, H // 128, generator=g) * 2, torch.rand(E, H // 128, I // 128, generator=g) * 2)
    _moe_compare(x, w1, w2, logits, topk, f"moe fp8 scaled T={T} repack={repack}", fp8=True, scales=scales, repack=repack,
                 groups=8, kept=4, score="sigmoid")


def test_graphed_fused_moe_replays_bit_exactly():
    """GraphedFusedMoE: the layer captured once, replayed on new inputs, equals the eager call bit for bit."""
    from muxi_native_layout_kernels_b200.muxi_moe_planC import GraphedFusedMoE
    dev = require_gpu()
    E, topk, H, I, T = 16, 4, 256, 128, 24
    w1 = mlk.layoutA(randn((E, 2 * I, H), 901, 0.05).to(dev))
    w2 = mlk.layoutA(randn((E, H, I), 902, 0.05).to(dev))
    layer = GraphedFusedMoE(w1, w2, T, E, topk, True)
    from muxi_native_layout_kernels_b200 import muxi_moe_planC
    muxi_moe_planC.set_nvtx(True)        # opt-in NVTX ranges around the stages: same results, only markers
    for seed in (903, 904, 905):
        x = randn((T, H), seed, 1.0).to(dev)
        logits = randn((T, E), seed + 10, 1.0).to(dev)
        want = planC_moe(x, w1, w2, logits, topk, True)
        got = layer(x, logits)
        torch.cuda.synchronize()
        assert torch.equal(got, want)
    muxi_moe_planC.set_nvtx(False)
    with pytest.raises(ValueError, match="captured for"):
        layer(x[:3], logits[:3])


@pytest.mark.parametrize("tune", [None, (2, 102, 2, 0, 103, 2)])
def test_moe_expert_parallel_map_sums_to_full_layer(tune):
    """experts_map is the reference's only multi-GPU hook (csrc/moe_kernels/moe_align_tokens.h:46-49): each rank
    computes its local experts' share of y; the shares add up to the full layer (warp-level and tcgen05 kernels)."""
    dev = require_gpu()
    E, topk, H, I, T = 16, 4, 128, 128, 40
    x = randn((T, H), 700).to(dev)
    w1 = mlk.layoutA(randn((E, 2 * I, H), 701, 0.05).to(dev))
    w2 = mlk.layoutA(randn((E, H, I), 702, 0.05).to(dev))
    logits = randn((T, E), 703).to(dev)
    full = planC_moe(x, w1, w2, logits, topk, True).float()
    acc = torch.zeros_like(full)
    for rank in range(4):
        lo = rank * 4
        emap = torch.full((E,), -1, dtype=torch.int32)
        emap[lo:lo + 4] = torch.arange(4, dtype=torch.int32)
        part = planC_moe(x, w1[lo:lo + 4].contiguous(), w2[lo:lo + 4].contiguous(), logits, topk, True,
                         experts_map=emap.to(dev), tune=tune)
        acc += part.float()
    assert_close(acc, full.cpu(), "EP shares", atol=2e-2, rtol=2e-2)


def test_moe_errors():
    dev = require_gpu()
    E, topk, H, I, T = 4, 2, 64, 32, 3
    x = randn((T, H), 800).to(dev)
    w1 = mlk.layoutA(randn((E, 2 * I, H), 801).to(dev))
    w2 = mlk.layoutA(randn((E, H, I), 802).to(dev))
    logits = randn((T, E), 803).to(dev)
    with pytest.raises(ValueError, match="num_expert_group"):
        planC_moe(x, w1, w2, logits, topk, True, use_grouped_topk=False, num_expert_group=2)
    with pytest.raises(ValueError, match="scoring"):
        planC_moe(x, w1, w2, logits, topk, True, score_func="relu")
    with pytest.raises(RuntimeError, match="w1 must be"):
        planC_moe(x, w1, w1, logits, topk, True)
    with pytest.raises(RuntimeError, match="soft_fp8 must be true"):
        w8 = mlk.layoutA(rand_e4m3((E, 2 * I, H), 804).to(dev))
        w8b = mlk.layoutA(rand_e4m3((E, H, I), 805).to(dev))
        ids = torch.zeros(T, topk, dtype=torch.int32, device=dev)
        ww = torch.zeros(T, topk, dtype=torch.bfloat16, device=dev)
        buf = torch.zeros(64, dtype=torch.int32, device=dev)
        mlk.fused_experts_compute(w8, w8b, x, T, E, topk, ids, ww, torch.zeros(T * topk + E * 15, dtype=torch.int32, device=dev),
                                  buf, buf, buf, torch.zeros(topk * 2 * I * T, dtype=torch.bfloat16, device=dev),
                                  torch.zeros_like(x), None, None, [128, 128], False)


# ----------------------------------------------------------------------------------------------------
# the benchmark configurations at full size
# ----------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("T", [1, 16, 64, 256])
def test_config_moe_mixtral_bf16(T):
    """E=8, top-2, H=4096, I=14336, gated SiLU, W ~ N(0, 0.02^2), seed 3; router softmax + renormalise."""
    dev = require_gpu()
    g = torch.Generator(device=dev).manual_seed(3)
    E, H, I = 8, 4096, 14336
    w1 = (torch.randn(E, 2 * I, H, generator=g, device=dev) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, generator=g, device=dev) * 0.02).to(torch.bfloat16)
    wg = (torch.randn(E, H, generator=g, device=dev) * 0.02).to(torch.bfloat16)
    x = torch.randn(T, H, generator=g, device=dev).to(torch.bfloat16)
    logits = (x.float() @ wg.float().t()).to(torch.bfloat16)
    y = planC_moe(x, mlk.layoutA(w1), mlk.layoutA(w2), logits, 2, True)
    torch.cuda.synchronize()
    ids, w = _kernel_routing(x.cpu(), logits.cpu(), 2, True, 1, 1, None, "softmax", dev)
    y16 = omoe.experts_ref(x.cpu(), w1.cpu(), w2.cpu(), ids, w)
    y32 = omoe.experts_ref(x.cpu(), w1.cpu(), w2.cpu(), ids, w, compute_dtype=torch.float32)
    rep = assert_close(y, y32, f"C4 T={T}", scale_atol=True)
    print("C4", T, rep, "floor", odense.error_report(y16, y32, scale_atol=True))


@pytest.mark.parametrize("T,skew", [(1, False), (32, False), (128, True), (512, False), (512, True)])
def test_config_moe_fine_grained_fp8(T, skew):
    """E=128, top-8, H=2048, I=768, e4m3 weights through layout A and fp8_weight_repack, seed 4; the skewed
    variant adds +2.0 to the logits of 8 hot experts."""
    dev = require_gpu()
    g = torch.Generator(device=dev).manual_seed(4)
    E, H, I = 128, 2048, 768
    w1 = (torch.randn(E, 2 * I, H, generator=g, device=dev) * 0.5).to(torch.float8_e4m3fn)
    w2 = (torch.randn(E, H, I, generator=g, device=dev) * 0.5).to(torch.float8_e4m3fn)
    wg = (torch.randn(E, H, generator=g, device=dev) * 0.02).to(torch.bfloat16)
    x = torch.randn(T, H, generator=g, device=dev).to(torch.bfloat16)
    logits = (x.float() @ wg.float().t())
    if skew:
        hot = torch.randperm(E, generator=torch.Generator().manual_seed(44))[:8]
        logits[:, hot.to(dev)] += 2.0
    logits = logits.to(torch.bfloat16)
    w1d = mlk.fp8_weight_repack(mlk.layoutA(w1))
    w2d = mlk.fp8_weight_repack(mlk.layoutA(w2))
    y = planC_moe(x, w1d, w2d, logits, 8, True, block_shape=[128, 128], soft_fp8=True, fp8_repacked=True)
    torch.cuda.synchronize()
    ids, w = _kernel_routing(x.cpu(), logits.cpu(), 8, True, 1, 1, None, "softmax", dev)
    y16 = omoe.experts_ref(x.cpu(), w1.cpu(), w2.cpu(), ids, w)
    y32 = omoe.experts_ref(x.cpu(), w1.cpu(), w2.cpu(), ids, w, compute_dtype=torch.float32)
    rep = assert_close(y, y32, f"C5 T={T} skew={skew}", scale_atol=True)
    print("C5", T, skew, rep, "floor", odense.error_report(y16, y32, scale_atol=True))


def test_ep_reduce_shares_single_rank():
    """mlk_ep_reduce_shares with a world of one (its flags are exchanged with itself): rounding, row ownership, the epoch
    that lets a CUDA graph replay the launch.  More ranks need more GPUs: tests/ep_worker.py."""
    dev = require_gpu()
    from muxi_native_layout_kernels_b200 import ext
    from muxi_native_layout_kernels_b200._lib import check, lib
    T, H = 37, 256
    share = torch.randn(T, H, device=dev) * 100
    out = torch.zeros(T, H, dtype=torch.bfloat16, device=dev)
    flags = torch.zeros(int(lib.mlk_ep_reduce_flag_bytes()) // 4, dtype=torch.int32, device=dev)
    ptrs = [torch.tensor([t.data_ptr()], dtype=torch.int64, device=dev) for t in (share, out, flags)]

    def launch():
        check(lib.mlk_ep_reduce_shares(ptrs[0].data_ptr(), ptrs[1].data_ptr(), ptrs[2].data_ptr(), None, 0, 1, T, H, 0,
                                       ext._status_ptr(share), ext._stream(share)))

    for rep in range(3):
        launch()
        torch.cuda.synchronize()
        assert torch.equal(out, share.to(torch.bfloat16))
        assert int(flags[0].item()) == rep + 1 and int(flags[1].item()) == 0
        share.mul_(-0.5)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            launch()
    torch.cuda.current_stream().wait_stream(side)
    for rep in range(3):
        share.add_(1.0)
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, share.to(torch.bfloat16))
    assert mlk.kernel_status() == 0
    with pytest.raises(RuntimeError):
        check(lib.mlk_ep_reduce_shares(ptrs[0].data_ptr(), ptrs[1].data_ptr(), ptrs[2].data_ptr(), None, 3, 2, T, H, 0, None, None))


def test_ep_reduce_shares_reports_a_peer_that_never_arrives():
    """The expiry path of a bounded wait, end to end: a world of two in which the second rank never launches (its
    buffers are local stand-ins that nothing writes).  With a small poll budget the kernel must give up, record its
    status code, end by itself and leave the context usable."""
    dev = require_gpu()
    from muxi_native_layout_kernels_b200 import ext
    from muxi_native_layout_kernels_b200._lib import check, lib
    T, H = 600, 512                      # 307200 elements: the two-exchange form
    nflags = int(lib.mlk_ep_reduce_flag_bytes()) // 4
    share = [torch.ones(T, H, device=dev), torch.ones(T, H, device=dev)]
    out = [torch.zeros(T, H, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    flags = [torch.zeros(nflags, dtype=torch.int32, device=dev) for _ in range(2)]
    ptrs = [torch.tensor([a.data_ptr(), b.data_ptr()], dtype=torch.int64, device=dev) for a, b in (share, out, flags)]
    mlk.kernel_status(reset=True)
    check(lib.mlk_set_option(3, 12))     # 4096 polls instead of 2^24
    try:
        check(lib.mlk_ep_reduce_shares(ptrs[0].data_ptr(), ptrs[1].data_ptr(), ptrs[2].data_ptr(), None, 0, 2, T, H, 0,
                                       ext._status_ptr(share[0]), ext._stream(share[0])))
        torch.cuda.synchronize()
    finally:
        check(lib.mlk_set_option(3, 0))
    assert mlk.kernel_status(reset=True) == 0x0E000001
    assert mlk.kernel_status() == 0
    # small shares, the one-pass form: the pairs of the missing rank never land
    Ts = 4
    recv_bytes = int(lib.mlk_ep_reduce_recv_bytes(2, Ts, H))
    assert recv_bytes == 2 * 2 * Ts * H * 8
    recv = [torch.zeros(recv_bytes // 4, dtype=torch.int32, device=dev) for _ in range(2)]
    flags2 = [torch.zeros(nflags, dtype=torch.int32, device=dev) for _ in range(2)]
    p2 = [torch.tensor([a.data_ptr(), b.data_ptr()], dtype=torch.int64, device=dev) for a, b in (share, out, flags2, recv)]
    check(lib.mlk_set_option(3, 12))
    try:
        check(lib.mlk_ep_reduce_shares(p2[0].data_ptr(), p2[1].data_ptr(), p2[2].data_ptr(), p2[3].data_ptr(), 0, 2, Ts, H, 0,
                                       ext._status_ptr(share[0]), ext._stream(share[0])))
        torch.cuda.synchronize()
    finally:
        check(lib.mlk_set_option(3, 0))
    assert mlk.kernel_status(reset=True) == 0x0E000001
    # the context is intact: an ordinary call still works
    y = mlk.gemv_layoutA(mlk.layoutA(torch.ones(64, 64, dtype=torch.bfloat16, device=dev)), torch.ones(1, 64, dtype=torch.bfloat16, device=dev))
    torch.cuda.synchronize()
    assert float(y[0, 0]) == 64.0 and mlk.kernel_status() == 0


def test_fused_moe_writes_into_a_given_output_tensor():
    """out= (extension): the result lands in the caller's tensor, 16-bit or the un-rounded fp32 sums."""
    dev = require_gpu()
    E, topk, H, I, T = 16, 4, 256, 128, 19
    x = randn((T, H), 1500).to(dev)
    w1 = mlk.layoutA(randn((E, 2 * I, H), 1501, 0.05).to(dev))
    w2 = mlk.layoutA(randn((E, H, I), 1502, 0.05).to(dev))
    logits = randn((T, E), 1503).to(dev)
    want = planC_moe(x, w1, w2, logits, topk, True)
    buf = torch.full((T, H), 7.0, dtype=torch.bfloat16, device=dev)
    got = planC_moe(x, w1, w2, logits, topk, True, out=buf)
    assert got.data_ptr() == buf.data_ptr() and torch.equal(buf, want)
    buf32 = torch.full((T, H), 7.0, dtype=torch.float32, device=dev)
    got32 = planC_moe(x, w1, w2, logits, topk, True, out_dtype=torch.float32, out=buf32)
    assert got32.data_ptr() == buf32.data_ptr() and torch.equal(buf32.to(torch.bfloat16), want)
    with pytest.raises(ValueError):
        planC_moe(x, w1, w2, logits, topk, True, out=buf32)
