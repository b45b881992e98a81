"""B200-native (sm_100a) implementation of the weight-streaming operators of ``muxi_layout_kernels``.

``from muxi_native_layout_kernels_b200 import *`` gives the operator names of the reference extension module
(csrc/ffi.cu); the submodules ``muxi_moe_planC`` and ``utils`` mirror the reference package's Python modules.
Importing fails if the CUDA library has not been built: there is no fallback path.
"""
from .ext import *  # noqa: F401,F403
from .ext import __all__ as _ext_all
from . import ext, muxi_moe_planC, parallel, utils  # noqa: F401

__all__ = list(_ext_all) + ["ext", "muxi_moe_planC", "parallel", "utils"]
