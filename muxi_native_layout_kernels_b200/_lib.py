"""ctypes binding of libmlk_b200.so (declarations in include/mlk_b200.h).

The library is the only compute path of this package: if it cannot be loaded the import raises,
there is no eager/torch fallback.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
LIB_PATH = PKG_DIR / "libmlk_b200.so"

c_int, c_i64, c_f32, c_vp, c_cp = C.c_int, C.c_int64, C.c_float, C.c_void_p, C.c_char_p

# name -> (restype, argtypes); mirrors include/mlk_b200.h line by line
PROTOTYPES = {
    "mlk_status_string": (c_cp, [c_int]),
    "mlk_last_error": (c_cp, []),
    "mlk_build_info": (c_cp, []),
    "mlk_set_option": (c_int, [c_int, c_int]),
    "mlk_get_option": (c_int, [c_int]),
    "mlk_gemm_workspace_bytes": (c_i64, [c_int, c_int, c_int]),
    "mlk_soft_fp8_workspace_bytes": (c_i64, [c_int, c_int]),
    "mlk_table_load": (c_int, [c_int, c_cp]),
    "mlk_table_lookup": (c_int, [c_int, c_int, c_int, c_int, C.POINTER(c_int), C.POINTER(c_int)]),
    "mlk_table_file_name": (c_cp, [c_int]),
    "mlk_layoutA": (c_int, [c_vp, c_vp, c_i64, c_i64, c_int, c_int, c_vp]),
    "mlk_layoutB": (c_int, [c_vp, c_vp, c_int, c_int, c_vp]),
    "mlk_reLayoutC": (c_int, [c_vp, c_vp, c_int, c_int, c_vp]),
    "mlk_fp8_weight_repack": (c_int, [c_vp, c_vp, c_i64, c_vp]),
    "mlk_gemv_layoutA_wapper": (c_int, [c_vp, c_vp, c_vp, c_int, c_int, c_int, c_f32, c_f32, c_int, c_int, c_int,
                                        c_int, c_vp, c_vp, c_int, c_vp, c_vp]),
    "mlk_gemv_layoutA": (c_int, [c_vp, c_vp, c_vp, c_int, c_int, c_int, c_f32, c_f32, c_vp, c_vp, c_int, c_vp, c_vp]),
    "mlk_gemm_layoutA_wapper": (c_int, [c_vp, c_vp, c_vp, c_int, c_int, c_int, c_int, c_f32, c_f32, c_int, c_int,
                                        c_int, c_int, c_vp, c_vp, c_vp]),
    "mlk_gemm_layoutA": (c_int, [c_vp, c_vp, c_vp, c_int, c_int, c_int, c_int, c_f32, c_f32, c_vp, c_vp, c_vp]),
    "mlk_gemm_layoutA_soft_fp8_wapper": (c_int, [c_vp, c_vp, c_vp, c_vp, c_int, c_int, c_int, c_f32, c_f32, c_int,
                                                 c_int, c_int, c_int, c_vp, c_int, c_vp, c_vp]),
    "mlk_gemm_layoutA_soft_fp8": (c_int, [c_vp, c_vp, c_vp, c_vp, c_int, c_int, c_int, c_f32, c_f32, c_vp, c_int,
                                          c_vp, c_vp]),
    "mlk_muxi_hgemm_layoutA": (c_int, [c_vp, c_vp, c_vp, c_vp, c_int, c_int, c_int, c_int, c_f32, c_f32, c_vp, c_int, c_vp,
                                       c_vp]),
    "mlk_gemm_layoutAB_ContinuousC_wapper": (c_int, [c_vp, c_vp, c_vp, c_int, c_int, c_int, c_int, c_f32, c_f32,
                                                     c_int, c_int, c_int, c_int, c_vp, c_vp, c_vp]),
    "mlk_gemm_layoutAB_ContinuousC": (c_int, [c_vp, c_vp, c_vp, c_int, c_int, c_int, c_int, c_f32, c_f32, c_vp,
                                              c_vp, c_vp]),
    "mlk_gemm_layoutABC_wapper": (c_int, [c_vp, c_vp, c_vp, c_int, c_int, c_int, c_int, c_f32, c_f32, c_int, c_int,
                                          c_int, c_int, c_vp, c_vp, c_vp]),
    "mlk_gemm_layoutABC": (c_int, [c_vp, c_vp, c_vp, c_int, c_int, c_int, c_int, c_f32, c_f32, c_vp, c_vp, c_vp]),
    "mlk_fused_routing_gate": (c_int, [c_vp, c_int, c_int, c_int, c_int, c_int, c_vp, c_vp, c_int, c_vp, c_int,
                                       c_vp]),
    "mlk_fused_router_gemm_gate": (c_int, [c_vp, c_vp, c_int, c_int, c_int, c_int, c_int, c_int, c_vp, c_vp, c_int, c_vp,
                                           c_int, c_int, c_vp, c_vp]),
    "mlk_fused_routing_gate_renorm": (c_int, [c_vp, c_int, c_int, c_int, c_int, c_int, c_vp, c_vp, c_int, c_vp, c_int,
                                              c_int, c_vp]),
    "mlk_moe_align": (c_int, [c_int, c_int, c_int, c_int, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_vp]),
    "mlk_fused_experts_compute_static": (c_int, [c_vp, c_vp, c_vp, c_int, c_int, c_int, c_int, c_int, c_vp, c_vp, c_vp,
                                                 c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_int, c_int, c_vp,
                                                 c_int, C.POINTER(C.c_int32), c_vp, c_int, c_vp]),
    "mlk_moe_gather_rows": (c_int, [c_vp, c_vp, c_vp, c_i64, c_int, c_i64, c_vp]),
    "mlk_moe_unpermute_sum": (c_int, [c_vp, c_vp, c_vp, c_i64, c_int, c_int, c_i64, c_int, c_vp]),
    "mlk_fused_experts_compute": (c_int, [c_vp, c_vp, c_vp, c_int, c_int, c_int, c_int, c_int, c_vp, c_vp, c_vp,
                                          c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_int, c_int, c_vp,
                                          c_int, c_vp, c_i64, C.POINTER(C.c_int32), c_vp, c_int, c_vp]),
    "mlk_ep_reduce_flag_bytes": (c_i64, []),
    "mlk_ep_reduce_recv_bytes": (c_i64, [c_int, c_i64, c_int]),
    "mlk_ep_reduce_shares": (c_int, [c_vp, c_vp, c_vp, c_vp, c_int, c_int, c_i64, c_int, c_int, c_vp, c_vp]),
    "mlk_fused_routing_experts_compute": (c_int, [c_vp, c_int, c_int, c_int, c_int, c_vp, c_int,
                                                  c_vp, c_vp, c_vp, c_int, c_int, c_int, c_int, c_int, c_vp, c_vp, c_vp,
                                                  c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_int, c_int, c_vp,
                                                  c_int, c_vp, c_i64, C.POINTER(C.c_int32), c_vp, c_int, c_vp]),
}


class MlkAux(C.Structure):
    """struct mlk_aux of include/mlk_b200.h."""
    _fields_ = [("workspace", c_vp), ("workspace_bytes", c_i64), ("counters", c_vp), ("n_counters", C.c_int32),
                ("status", c_vp)]


class MlkError(RuntimeError):
    """Raised when a library call returns a non-zero status (the reference raises RuntimeError via TORCH_CHECK)."""


def _load() -> C.CDLL:
    path = os.environ.get("MLK_B200_LIB", str(LIB_PATH))
    if not os.path.exists(path):
        raise ImportError(
            f"{path} is missing: build it with `python muxi_native_layout_kernels_b200/build.py` "
            "(needs nvcc; there is no non-CUDA fallback)"
        )
    lib = C.CDLL(path)
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)   # AttributeError here means header and library disagree
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def check(status: int) -> None:
    if status != 0:
        msg = lib.mlk_last_error().decode() or lib.mlk_status_string(status).decode()
        raise MlkError(msg)


def load_tables(directory: os.PathLike | str | None = None) -> None:
    """Loads the seven packaged dispatch tables (reference: first use of each selector, arg_selector.cu:75-87)."""
    d = Path(directory) if directory is not None else PKG_DIR
    for t in range(7):
        name = lib.mlk_table_file_name(t).decode()
        lib.mlk_table_load(t, str(d / name).encode())   # a missing file only warns, as in the reference


load_tables()
