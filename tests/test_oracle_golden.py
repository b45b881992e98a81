"""The CPU oracle against the golden vectors generated from the reference (tests/golden/make_golden.py)."""
import numpy as np
import torch

from oracle import dense as odense
from oracle import layouts as olay
from oracle import moe as omoe


def test_layout_a_matches_reference_recipe(golden_dir):
    g = np.load(golden_dir / "layouts.npz")
    for name in ("a16", "a8"):
        assert np.array_equal(olay.layout_a(g[f"{name}_in"]), g[f"{name}_out"])
        assert np.array_equal(olay.layout_a_inverse(g[f"{name}_out"]), g[f"{name}_in"])


def test_layout_b_matches_reference_recipe(golden_dir):
    g = np.load(golden_dir / "layouts.npz")
    assert np.array_equal(olay.layout_b(g["b_in"]), g["b_out"])


def test_layout_c_matches_reference_recipe(golden_dir):
    g = np.load(golden_dir / "layouts.npz")
    assert np.array_equal(olay.layout_c_inverse(g["c_in"]), g["c_out"])
    assert np.array_equal(olay.layout_c(g["c_out"]), g["c_in"])


def test_fp8_repack_matches_reference_word_formula(golden_dir):
    g = np.load(golden_dir / "layouts.npz")
    assert np.array_equal(olay.fp8_repack(g["repack_in"]), g["repack_out"])
    assert np.array_equal(olay.fp8_repack(olay.fp8_repack(g["repack_in"])), g["repack_in"])   # involution


def test_e4m3_table_matches_torch_cast(golden_dir):
    g = np.load(golden_dir / "layouts.npz")
    table = olay.e4m3_decode_table()
    want = g["e4m3_float"]
    finite = ~np.isnan(want)
    assert finite.sum() == 254
    assert np.array_equal(table[finite], want[finite])
    # the two NaN encodings decode to +-480 under the reference's bit trick (csrc/utils.cuh:232-251)
    assert table[0x7F] == 480.0 and table[0xFF] == -480.0


def test_dequant_matches_reference_scale_tensor(golden_dir):
    g = torch.load(golden_dir / "dequant.pt")
    w8 = g["w8"].view(torch.float8_e4m3fn)
    assert torch.equal(odense.dequant_block_scaled(w8, g["scale"]), g["out"])
    we = g["we"].view(torch.float8_e4m3fn)
    got = torch.stack([odense.dequant_block_scaled(we[e], g["se"][e]) for e in range(we.shape[0])])
    assert torch.equal(got, g["oute"])
    # unit scale is exact
    assert torch.equal(odense.dequant_block_scaled(w8, None).float(), w8.float())


def test_dense_oracle_matches_golden(golden_dir):
    g = torch.load(golden_dir / "dense.pt")
    for name in ("bf16", "fp16"):
        d = g[name]
        assert torch.equal(odense.gemm_ref(d["X"], d["W"]), d["C"])
        # the oracle adds the bias in fp32 before the single rounding; the benchmark recipe adds it after
        # rounding: at most one output ulp apart
        rep = odense.error_report(odense.gemm_ref(d["X"], d["W"], bias=d["bias"]), d["C_bias"])
        assert rep["ok"], rep


def _load_moe(golden_dir, name):
    g = torch.load(golden_dir / f"moe_{name}.pt")
    if g["fp8"]:
        g["w1"] = g["w1"].view(torch.float8_e4m3fn)
        g["w2"] = g["w2"].view(torch.float8_e4m3fn)
    return g


def _check_moe(golden_dir, name):
    torch.set_num_threads(1)
    g = _load_moe(golden_dir, name)
    y, ids, w, masked = omoe.fused_moe_ref(g["x"], g["w1"], g["w2"], g["logits"], g["topk"],
                                            renormalize=g["renormalize"], num_expert_group=g["groups"],
                                            topk_group=g["topk_group"], bias=g["bias"], score_func=g["score_func"],
                                            dense=True)
    # no ties at the cut in these fixtures -> the restatement must reproduce the reference bit for bit
    srt = torch.sort(masked.float(), dim=-1, descending=True)[0]
    assert bool((srt[:, g["topk"] - 1] > srt[:, g["topk"]]).all()), "fixture has a tie at the top-k cut"
    assert torch.equal(y, g["y"]), (y.float() - g["y"].float()).abs().max()
    # the sparse evaluation (only routed tokens) and the fp32 evaluation stay within tolerance of it
    y_sparse = omoe.experts_ref(g["x"], g["w1"], g["w2"], ids, w)
    assert odense.error_report(y_sparse, g["y"])["ok"]
    y32 = omoe.experts_ref(g["x"], g["w1"], g["w2"], ids, w, compute_dtype=torch.float32)
    # (this is the noise floor of the 16-bit oracle itself: five intermediate roundings)
    assert odense.error_report(y32, g["y"], atol=3e-2, rtol=3e-2, scale_atol=True)["ok"]


def test_moe_oracle_softmax_top2(golden_dir):
    _check_moe(golden_dir, "softmax_top2")


def test_moe_oracle_sigmoid_grouped_bias(golden_dir):
    _check_moe(golden_dir, "sigmoid_grouped_bias")


def test_moe_oracle_fp16(golden_dir):
    _check_moe(golden_dir, "fp16_softmax")


def test_moe_oracle_fp8(golden_dir):
    _check_moe(golden_dir, "fp8_top8")


def test_align_ref_contract():
    ids = torch.tensor([[0, 3], [3, 1], [3, 0], [2, 3]], dtype=torch.int32)
    r = omoe.align_ref(ids, 4, mbs=4)
    assert r["counts"].tolist() == [2, 1, 1, 4]
    assert r["starts"].tolist() == [0, 4, 8, 12]
    assert r["num_blocks"] == 4 and r["block_expert"].tolist() == [0, 1, 2, 3]
    assert r["cumsum_after"].tolist() == [2, 5, 9, 16, 16]
    emap = torch.tensor([-1, 0, -1, 1], dtype=torch.int32)
    r = omoe.align_ref(ids, 2, mbs=4, experts_map=emap)
    assert r["counts"].tolist() == [1, 4] and r["slots_of"][1].tolist() == [1, 2, 4, 7]


def test_router_tie_rule_lower_id_wins():
    logits = torch.zeros(1, 8, dtype=torch.bfloat16)   # all scores equal
    ids, w, _ = omoe.router_ref(logits, 3)
    assert ids.tolist() == [[0, 1, 2]]
    assert torch.allclose(w.float(), torch.full((1, 3), 0.125))
