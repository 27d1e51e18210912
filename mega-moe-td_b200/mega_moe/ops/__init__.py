"""Operator layer (mirrors src/mega_moe/ops/__init__.py:9-24 of the reference)."""

from .backward import MegaMoEBackwardFunction, moe_backward_triton
from .forward import DispatchFC1Result, FusedMoEForward, pack_gate_up_weights
from .function import MegaMoEFunction

__all__ = [
    "DispatchFC1Result",
    "FusedMoEForward",
    "MegaMoEBackwardFunction",
    "MegaMoEFunction",
    "moe_backward_triton",
    "pack_gate_up_weights",
]
