"""Drop-in alias: lets code written against the reference package (``import muxi_layout_kernels``,
``from muxi_layout_kernels.muxi_moe_planC import fused_moe``) run on the B200 implementation unchanged."""
import sys as _sys

import muxi_native_layout_kernels_b200 as _impl
from muxi_native_layout_kernels_b200 import *  # noqa: F401,F403
from muxi_native_layout_kernels_b200 import muxi_moe_planC, utils  # noqa: F401

_sys.modules[__name__ + ".muxi_moe_planC"] = muxi_moe_planC
_sys.modules[__name__ + ".utils"] = utils
__all__ = _impl.__all__
