"""CPU-side checks of the C-ABI library and the host logic above it (no kernel is launched here)."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


def _declared_symbols():
    text = (ROOT / "include" / "mlk_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mlk_[A-Za-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from muxi_native_layout_kernels_b200 import _lib
    names = _declared_symbols()
    assert len(names) >= 20
    raw = ctypes.CDLL(str(_lib.LIB_PATH))
    for n in names:
        assert hasattr(raw, n), f"{n} is declared in include/mlk_b200.h but not exported"
    # and the ctypes prototypes cover the header exactly, argument count included
    assert sorted(_lib.PROTOTYPES) == names
    text = re.sub(r"/\*.*?\*/", "", (ROOT / "include" / "mlk_b200.h").read_text(), flags=re.S)
    for name, params in re.findall(r"\b(mlk_[A-Za-z0-9_]+)\s*\(([^;{]*)\)\s*;", text):
        params = params.strip()
        count = 0 if params in ("", "void") else params.count(",") + 1
        assert count == len(_lib.PROTOTYPES[name][1]), f"{name}: header has {count} parameters, ctypes {len(_lib.PROTOTYPES[name][1])}"


def test_status_strings_and_build_info():
    from muxi_native_layout_kernels_b200._lib import lib
    assert lib.mlk_status_string(0) == b"ok"
    assert lib.mlk_status_string(1) == b"invalid argument"
    assert b"sm_100a" in lib.mlk_build_info()


def test_table_load_lookup_and_miss_default(tmp_path, capfd):
    from muxi_native_layout_kernels_b200._lib import lib
    p = tmp_path / "t.csv"
    p.write_text("m,n,k,kernelId,kernelParam1,kernelParam2,kernelParam3\n"
                 "4096,16,4096,1,2,4,2\n"
                 "bad,line\n"
                 "4096,16,4096,1,1,2,8\n"          # later duplicate wins (reference: arg_selector.cu:49)
                 "128,32,256,1,2,1,1\n")
    assert lib.mlk_table_load(2, str(p).encode()) == 0
    out = (ctypes.c_int * 4)()
    hit = ctypes.c_int(-1)
    assert lib.mlk_table_lookup(2, 4096, 16, 4096, out, ctypes.byref(hit)) == 0
    assert list(out) == [1, 1, 2, 8] and hit.value == 1
    assert "Invalid line" in capfd.readouterr().err
    # miss: warns once, returns a runnable default, then remembers it
    assert lib.mlk_table_lookup(2, 8192, 8, 1024, out, ctypes.byref(hit)) == 0
    first = list(out)
    # 128-row tiles, 2..64 tokens: the tcgen05 tile kernel, cluster mode (ring stages, CTAs per cluster)
    assert hit.value == 0 and first[0] == 2 and first[2] in (3, 4) and 2 <= first[3] <= 8
    assert "No matching arguments" in capfd.readouterr().err
    # any other shape: the warp-level kernel
    assert lib.mlk_table_lookup(2, 8192 + 16, 8, 1024, out, ctypes.byref(hit)) == 0
    w = list(out)
    assert hit.value == 0 and w[0] == 1 and w[1] in (1, 2) and w[2] in (1, 2, 4, 8) and w[3] in (1, 2, 4, 8)
    # more than 64 tokens on 128-row tiles: the many-token tcgen05 tile kernel; layout-B variants stay warp-level
    assert lib.mlk_table_lookup(2, 8192, 128, 1024, out, ctypes.byref(hit)) == 0 and list(out)[0] == 10
    assert lib.mlk_table_lookup(1, 8192, 128, 1024, out, ctypes.byref(hit)) == 0 and list(out)[0] == 1
    capfd.readouterr()
    assert lib.mlk_table_lookup(2, 8192, 8, 1024, out, ctypes.byref(hit)) == 0
    assert list(out) == first and hit.value == 1
    assert capfd.readouterr().err == ""
    # GeMV tables are keyed by (m, k) with six columns
    q = tmp_path / "v.csv"
    q.write_text("m,k,BLOCK_DIM_X,KernelId,KernelParam1,KernelParam2\n4096,4096,128,2,1,4\n")
    assert lib.mlk_table_load(5, str(q).encode()) == 0
    assert lib.mlk_table_lookup(5, 4096, 999, 4096, out, ctypes.byref(hit)) == 0
    assert list(out) == [128, 2, 1, 4] and hit.value == 1
    # missing file: I/O status, lookups still answer with defaults
    assert lib.mlk_table_load(5, b"/nonexistent/file.csv") == 4
    assert lib.mlk_table_lookup(5, 4096, 1, 4096, out, ctypes.byref(hit)) == 0 and hit.value == 0
    assert lib.mlk_table_lookup(9, 1, 1, 1, out, ctypes.byref(hit)) == 1
    from muxi_native_layout_kernels_b200 import _lib
    _lib.load_tables()   # restore the packaged tables for the other tests


def test_packaged_tables_exist_with_reference_headers():
    from muxi_native_layout_kernels_b200._lib import PKG_DIR, lib
    gemm_hdr = "m,n,k,kernelId,kernelParam1,kernelParam2,kernelParam3"
    gemv_hdr = "m,k,BLOCK_DIM_X,KernelId,KernelParam1,KernelParam2"
    for t in range(7):
        f = PKG_DIR / lib.mlk_table_file_name(t).decode()
        assert f.exists(), f
        assert f.read_text().splitlines()[0].strip() == (gemv_hdr if t >= 4 else gemm_hdr)


def test_packaged_table_rows_name_launches_the_library_accepts():
    """Every row of the packaged tables must pass the validity rules of the table-driven entry points (a row that
    fails them silently falls back to the shape-based default and loses the tuned performance)."""
    import csv
    pkg = Path(__file__).resolve().parents[1] / "muxi_native_layout_kernels_b200"

    def rows(name):
        with open(pkg / name) as f:
            r = csv.reader(f)
            next(r)
            return [[int(v) for v in row] for row in r if row]

    for name, fp8, layout_a in [("layout_gemm_dispatch_arg.csv", False, False), ("continuous_gemm_dispatch_arg.csv", False, False),
                                ("layoutA_gemm_dispatch_arg.csv", False, True), ("layoutA_Soft_Fp8_gemm_dispatch_arg.csv", True, True)]:
        table = rows(name)
        assert table, name
        for m, n, k, kid, p1, p2, p3 in table:
            what = (name, m, n, k, kid, p1, p2, p3)
            assert m % 128 == 0 and k % 128 == 0 and 1 <= n <= 256, what
            if kid in (1, 3, 4):
                assert p1 in (1, 2) and p2 in (1, 2, 4, 8) and p2 <= {1: 8, 3: 4, 4: 2}[kid] and p3 in (1, 2, 4, 8), what
                assert m % (16 * p1 * p2) == 0, what
            elif kid == 2 and not fp8:
                assert n <= 64 and 1 <= p1 <= 4 and p2 in (2, 3, 4, 5, 6, 8) and 0 <= p3 <= 16, what
                assert layout_a or (n % 16 == 0 and p3 >= 2), what     # layout-B variants pass no scratch: cluster mode
                assert p3 < 2 or p3 <= k // 64, what
            elif kid == 2 and fp8:
                assert n <= 64 and p2 in (2, 3, 4, 6, 8) and 1 <= p3 <= min(8, k // 64), what
            elif kid == 9:       # e4m3 weights undecoded into the 8-bit MMA: k per stage, ring stages, cluster size
                assert fp8 and n <= 64 and p1 in (64, 128) and k % p1 == 0 and p2 in (2, 3, 4, 6, 8), what
                assert 1 <= p3 <= min(8, k // p1), what
                np_ = 16 if n <= 16 else (32 if n <= 32 else 64)
                assert p2 * (128 * p1 + (p1 // 64) * np_ * 128) + 1024 <= 227 * 1024, what
            elif kid in (5, 6, 7):
                assert layout_a and not fp8 and n <= 4 and p1 in (1, 2) and p3 in (1, 2, 4, 8) and m % (16 * p1) == 0, what
            else:
                raise AssertionError(what)
    for name, fp8 in [("layout_gemv_dispatch_arg.csv", False), ("layout_gemv_bf16_dispatch_arg.csv", False),
                      ("layout_gemv_soft_fp8_dispatch_arg.csv", True)]:
        table = rows(name)
        assert table, name
        for m, k, block, kid, p1, p2 in table:
            what = (name, m, k, block, kid, p1, p2)
            if kid == 3:
                assert fp8 and m % 128 == 0 and k % 64 == 0 and p1 in (2, 3, 4, 6, 8) and 1 <= p2 <= 8, what
            elif kid == 4:
                bk = 64 if block == 64 else 128
                assert fp8 and block in (64, 128, 256) and m % 128 == 0 and k % bk == 0 and p1 in (2, 3, 4, 6, 8), what
                assert 1 <= p2 <= min(8, k // bk), what
            else:
                assert block in (64, 128, 256) and (kid == 1 or (kid == 2 and not fp8)), what
                assert p1 in (1, 2) and p2 in (1, 2, 4, 8) and m % (16 * p1) == 0, what
    for E, topk, H, I, fp8, T, nt, wm1, sk1, rg2, wm2, sk2 in rows("moe_dispatch_arg.csv"):
        what = (E, topk, H, I, fp8, T, nt, wm1, sk1, rg2, wm2, sk2)
        assert nt in (1, 2, 4, 8) or (nt == 16 and wm1 >= 100 and not fp8), what
        assert (wm1 >= 100) == (wm2 >= 100), what
        if wm1 >= 300:       # decode batches as one cooperative kernel
            assert wm2 >= 300 and T <= 8 and T * topk <= 64 and H % 32 == 0 and I % 32 == 0, what
        elif wm1 >= 100:     # tcgen05 expert GEMMs: 100 (decode) or 200 (native e4m3) + ring stages, CTAs per cluster
            fam = 200 if wm1 >= 200 else 100
            assert H % 128 == 0 and I % 128 == 0 and (fam == 100 or fp8) and (wm2 >= 200) == (wm1 >= 200), what
            assert (wm1 - fam in (2, 3, 4, 6) and 1 <= sk1 <= min(8, H // 64)) or \
                   (fam == 200 and wm1 - fam in (42, 43) and nt == 8 and sk1 == 1 and H % 128 == 0), what      # 128 k per stage
            assert wm2 - fam in (2, 3, 4, 6) or (fam == 200 and wm2 - fam in (42, 43, 44, 46) and 11 <= sk2 <= 18), what    # 240 + stages: 128 k per stage
            assert 1 <= sk2 <= min(8, I // 64) or (fam == 200 and 11 <= sk2 <= 18), what      # 10 + row tiles per CTA
        else:
            assert wm1 in (1, 2, 4, 8) and wm2 in (1, 2, 4, 8) and sk1 in (1, 2, 4, 8) and sk2 in (1, 2, 4, 8) and rg2 in (1, 2), what


def test_argument_errors_surface_as_runtime_error_without_a_gpu():
    import muxi_native_layout_kernels_b200 as mlk
    A = torch.zeros(8, 16, 16, 8, dtype=torch.bfloat16)
    B = torch.zeros(1, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="A must be a CUDA tensor"):
        mlk.gemv_layoutA(A, B)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        mlk.layoutB(torch.zeros(16, 32, dtype=torch.bfloat16))
    with pytest.raises(NotImplementedError):
        mlk.gemmEx(A, B)
    with pytest.raises(NotImplementedError):
        mlk.muxi_hgemm(A, B)


def test_c_abi_rejects_bad_shapes_before_touching_the_device():
    from muxi_native_layout_kernels_b200._lib import lib
    one = ctypes.c_void_p(16)   # never dereferenced: the shape check comes first
    assert lib.mlk_gemm_layoutA(one, one, one, 100, 16, 128, 0, 1.0, 0.0, None, None, None) == 1
    assert b"multiple of 128" in lib.mlk_last_error()
    assert lib.mlk_gemv_layoutA_wapper(one, one, one, 40, 64, 0, 1.0, 0.0, 256, 1, 1, 1, None, None, 0, None, None) == 1
    assert lib.mlk_gemv_layoutA_wapper(one, one, one, 64, 64, 0, 1.0, 0.0, 256, 7, 1, 1, None, None, 0, None, None) == 2
    assert lib.mlk_gemm_layoutA_wapper(one, one, one, 128, 16, 128, 0, 1.0, 0.0, 3, 1, 1, 1, None, None, None) == 1
    assert lib.mlk_layoutB(one, one, 10, 32, None) == 1
    assert lib.mlk_fp8_weight_repack(one, one, 6, None) == 1
    assert lib.mlk_fused_routing_gate(one, 0, 4, 300, 1, 1, one, one, 2, None, 0, None) == 2
    assert lib.mlk_fused_routing_gate(one, 0, 4, 64, 3, 1, one, one, 2, None, 0, None) == 1


def test_drop_in_alias_package_exposes_reference_names():
    import muxi_layout_kernels
    from muxi_layout_kernels.muxi_moe_planC import fused_moe as planC  # noqa: F401
    from muxi_layout_kernels.utils import fused_moe, scale_tensor, scale_whole_tensor  # noqa: F401
    for name in ("layoutB", "reLayoutC", "gemm_layoutABC", "gemm_layoutA_linear", "gemm_layoutA",
                 "gemm_layoutA_soft_fp8", "gemm_layoutAB_ContinuousC", "gemv_layoutA", "gemm_layoutABC_wapper",
                 "gemm_layoutA_wapper", "gemm_layoutA_soft_fp8_wapper", "gemm_layoutAB_ContinuousC_wapper",
                 "gemv_layoutA_wapper", "fp8_weight_repack", "fused_routing_gate",
                 "batched_routed_activation_indexed_to_expert_block_indexed", "fused_experts_compute",
                 "gemmEx", "muxi_hgemm", "routing_gate", "experts_compute"):
        assert hasattr(muxi_layout_kernels, name), name


def test_package_utils_match_reference_helpers(golden_dir):
    """The package's own torch helpers (public API of the reference package) against the golden vectors."""
    from muxi_native_layout_kernels_b200 import utils
    g = torch.load(golden_dir / "dequant.pt")
    assert torch.equal(utils.scale_tensor(g["w8"].view(torch.float8_e4m3fn).to(torch.bfloat16), g["scale"]), g["out"])
    assert torch.equal(utils.scale_whole_tensor(g["we"].view(torch.float8_e4m3fn), g["se"]), g["oute"])
    torch.set_num_threads(1)
    m = torch.load(golden_dir / "moe_softmax_top2.pt")
    y = utils.fused_moe(m["x"], m["w1"], m["w2"], m["logits"], m["topk"], m["groups"], m["topk_group"],
                        global_num_experts=m["logits"].shape[1], renormalize=m["renormalize"])
    assert torch.equal(y, m["y"])


def test_moe_table_lookup_rules():
    """lookup_moe_args: the row of the smallest tabulated token count >= T, the last row beyond the table, decode rows
    (tuning values >= 300) only where the caller can use them, nothing for an unknown geometry."""
    from muxi_native_layout_kernels_b200.muxi_moe_planC import lookup_moe_args
    fine = (128, 8, 2048, 768, True)
    assert lookup_moe_args(*fine, 1)[1] >= 300 and lookup_moe_args(*fine, 2)[1] >= 300
    assert lookup_moe_args(*fine, 3) == lookup_moe_args(*fine, 4) and lookup_moe_args(*fine, 4)[1] < 300
    assert lookup_moe_args(*fine, 100) == lookup_moe_args(*fine, 128)
    assert lookup_moe_args(*fine, 100000) == lookup_moe_args(*fine, 512)
    # an expert-parallel rank with 16 local experts looks its row up by (16, tokens x 16 / 128); with 32 global tokens
    # the decode rows (T_eff = 4) cannot be used (the batch is larger than 8) and the next row applies
    ep = (16, 8, 2048, 768, True)
    assert lookup_moe_args(*ep, 4)[1] >= 300
    assert lookup_moe_args(*ep, 4, allow_decode=False)[1] < 300
    assert lookup_moe_args(*ep, 4, allow_decode=False) == lookup_moe_args(*ep, 16)
    assert lookup_moe_args(7, 3, 640, 320, False, 5) is None


def test_ep_reduce_buffer_sizes_follow_the_one_pass_bound():
    """mlk_ep_reduce_recv_bytes: two sets of (value, epoch) pairs from every rank for shares that take the one-pass
    form, 0 for shares past its bound -- min(256 Ki, 1 Mi / world) elements, since that form moves world x the data
    of the two-exchange form -- and for a single rank."""
    from muxi_native_layout_kernels_b200._lib import lib
    assert lib.mlk_ep_reduce_flag_bytes() > 0
    n = 64 * 4096                                   # 256 Ki elements
    for world in (2, 4):
        assert lib.mlk_ep_reduce_recv_bytes(world, 64, 4096) == 2 * world * n * 8
        assert lib.mlk_ep_reduce_recv_bytes(world, 65, 4096) == 0
    assert lib.mlk_ep_reduce_recv_bytes(8, 64, 4096) == 0
    assert lib.mlk_ep_reduce_recv_bytes(8, 32, 4096) == 2 * 8 * (n // 2) * 8
    assert lib.mlk_ep_reduce_recv_bytes(8, 0, 4096) == 0
    assert lib.mlk_ep_reduce_recv_bytes(1, 8, 4096) == 0


def test_bench_arms_share_one_config():
    """bench.py: the line of the library's arm and the line of the reference arm carry the same `config` (one function
    builds it from the rank count alone), and the reference arm prints it."""
    import importlib.util
    import json
    import subprocess
    import sys
    spec = importlib.util.spec_from_file_location("bench_module", ROOT / "bench.py")
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    c1, c8 = bench.step_config(1), bench.step_config(8)
    assert c1["launches_per_step"] == 21 and c1["sharding"] == "rows/1" and c8["sharding"] == "rows/8"
    assert "partly L2-resident" in c8["l2"] and "partly L2-resident" not in c1["l2"]
    src = (ROOT / "bench.py").read_text()
    assert src.count('"config": step_config(world)') == 2
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=600, cwd=str(ROOT))
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["config"] == json.loads(json.dumps(c1))
    assert line["cpu_baseline"]["kind"] == "port" and line["e2e"]["h2d_bytes_per_step"] == 0
