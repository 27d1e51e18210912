"""B200-native expert-parallel MoE layer behind the `mega_moe` operator API.

Same public names as the reference package (src/mega_moe/__init__.py:4-27); the kernels
underneath are hand-written sm_100a CUDA reached through a C ABI (see `_native.py`).
"""

from .config import MoEForwardConfig
from .ops.backward import MegaMoEBackwardFunction, moe_backward_triton
from .ops.forward import DispatchFC1Result, FusedMoEForward, pack_gate_up_weights
from .ops.function import MegaMoEFunction
from .ops.router import router_topk
from .runtime.routing import MoERoutingPlan

__all__ = [
    "router_topk",
    "FusedMoEForward",
    "DispatchFC1Result",
    "pack_gate_up_weights",
    "MegaMoEBackwardFunction",
    "MegaMoEFunction",
    "moe_backward_triton",
    "MoEForwardConfig",
    "MoERoutingPlan",
]
