"""MoonEP planning tables B.0-B.3: which routes leave an overloaded home rank, and which
logical experts every rank must hold a replica of.

Same names, argument meaning and errors as the reference's host planner
(src/mega_moe/runtime/moonep_planning.py:21-322): :func:`plan_moonep_b0_b3` takes the CPU
``[R, E]`` count matrix and returns ``alloc_cumsum [E, R]`` and ``experts_to_copy [R, E/R]``.
The arithmetic runs in the shared library: ``mm_moonep_plan_host`` for CPU tensors and
``mm_moonep_plan`` (one kernel launch, :func:`launch_moonep_b0_b3`) for the count cube that
``mm_count_exchange`` leaves on the device; both compile the same planning code
(``csrc/moonep_core.h``).  There is no Python implementation of the plan in this package.

The tables are not yet consumed by ``FusedMoEForward`` (``enable_moonep=True`` still raises
``NotImplementedError``): replica weight transport and the replica gradient reduce are missing.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import _native as N

_INT32_MAX = (1 << 31) - 1

# MM_PLAN_* of include/mega_moe_b200.h
PLAN_OK, PLAN_BAD_COUNT, PLAN_UNEQUAL_ROWS, PLAN_NOT_DROPLESS, PLAN_TOO_LARGE = 0, 1, 2, 3, 4
PLAN_FILL_FAILED, PLAN_CUT_FAILED, PLAN_REPLICA_BUDGET = 5, 6, 7
MAX_WORLD = 64
MAX_EXPERTS = 4096


@dataclass(frozen=True)
class MoonEPPlanningResult:
    """``alloc_cumsum[e, d]``: routes of logical expert ``e`` executed on ranks ``0..d``
    (inclusive prefix).  ``experts_to_copy[d, b]``: logical expert in replica slot ``b`` of
    rank ``d``, ``-1`` for an empty slot; a rank has ``E/R`` replica slots
    (reference: runtime/moonep_planning.py:21-72)."""

    alloc_cumsum: torch.Tensor
    experts_to_copy: torch.Tensor

    def __post_init__(self) -> None:
        for name in ("alloc_cumsum", "experts_to_copy"):
            t = getattr(self, name)
            if t.device.type != "cpu":
                raise ValueError(f"{name} must be a CPU tensor")
            if t.dtype != torch.int32:
                raise TypeError(f"{name} must have dtype torch.int32")
            if t.ndim != 2 or not t.is_contiguous():
                raise ValueError(f"{name} must be a contiguous rank-2 tensor")
        num_experts, world = self.alloc_cumsum.shape
        if world <= 0 or num_experts <= 0:
            raise ValueError("planning table dimensions must be positive")
        if self.experts_to_copy.shape[0] != world:
            raise ValueError("planning tables disagree on world_size")
        if num_experts % world:
            raise ValueError("num_experts must be divisible by world_size")
        if self.experts_to_copy.shape[1] != num_experts // world:
            raise ValueError("replica budget must equal experts_per_rank")

    @property
    def replica_slot_high_water(self) -> int:
        """One past the highest replica slot in use on any rank."""
        used = (self.experts_to_copy >= 0).any(dim=0).nonzero()
        return int(used.max()) + 1 if used.numel() else 0


def _raise_for(reason: int, row_totals: Optional[torch.Tensor] = None) -> None:
    if reason == PLAN_OK:
        return
    if reason == PLAN_BAD_COUNT:
        raise ValueError("tpe_all counts must be non-negative")
    if reason == PLAN_UNEQUAL_ROWS:
        raise ValueError("MoonEP B.0-B.3 currently requires equal route counts per source rank")
    if reason == PLAN_NOT_DROPLESS:
        raise ValueError("MoonEP load balancing currently requires dropless valid routes "
                         "and equal route counts on every EP rank")
    if reason == PLAN_TOO_LARGE:
        if row_totals is not None and int(row_totals.max()) > _INT32_MAX:
            raise ValueError("routes per source rank must fit in int32")
        raise ValueError("global route count for each expert must fit in int32")
    if reason == PLAN_FILL_FAILED:
        raise RuntimeError("MoonEP B.1 failed to balance destination capacities")
    if reason == PLAN_CUT_FAILED:
        raise RuntimeError("MoonEP B.2 could not satisfy a transfer quota")
    if reason == PLAN_REPLICA_BUDGET:
        raise RuntimeError("fixed replica budget cannot cover all remote allocated experts")
    raise RuntimeError(f"MoonEP planning failed with reason {reason}")


def plan_moonep_b0_b3(tpe_all: torch.Tensor) -> MoonEPPlanningResult:
    """Plan for a contiguous CPU int32/int64 ``[R, E]`` count matrix whose rows have equal sums
    (dropless routing); ``E`` divisible by ``R`` (reference:
    runtime/moonep_planning.py:239-276, input checks :75-109)."""
    if not isinstance(tpe_all, torch.Tensor):
        raise TypeError("tpe_all must be a torch.Tensor")
    if tpe_all.device.type != "cpu":
        raise ValueError("tpe_all must be a CPU tensor")
    if tpe_all.dtype not in (torch.int32, torch.int64):
        raise TypeError("tpe_all must have dtype torch.int32 or torch.int64")
    if tpe_all.ndim != 2:
        raise ValueError("tpe_all must have shape [world_size, num_experts]")
    if not tpe_all.is_contiguous():
        raise ValueError("tpe_all must be contiguous")
    world, experts = (int(v) for v in tpe_all.shape)
    if world <= 0 or experts <= 0:
        raise ValueError("world_size and num_experts must be positive")
    if experts % world:
        raise ValueError("num_experts must be divisible by world_size")
    if world > MAX_WORLD or experts > MAX_EXPERTS:
        raise ValueError(f"the planner handles at most {MAX_WORLD} ranks and {MAX_EXPERTS} experts")
    if tpe_all.dtype == torch.int64:
        if bool((tpe_all < 0).any()):
            raise ValueError("tpe_all counts must be non-negative")
        if bool((tpe_all > _INT32_MAX).any()):
            raise ValueError("each tpe_all count must fit in int32")
    counts = tpe_all.to(torch.int32).contiguous()
    epr = experts // world
    allocation = torch.empty((world, experts), dtype=torch.int32)
    alloc_cumsum = torch.empty((experts, world), dtype=torch.int32)
    experts_to_copy = torch.empty((world, epr), dtype=torch.int32)
    inverse = torch.empty((world, experts), dtype=torch.int32)
    replica_counts = torch.empty((world,), dtype=torch.int32)
    stats = torch.zeros((4,), dtype=torch.int32)
    N.check(N.lib().mm_moonep_plan_host(
        counts.data_ptr(), experts, world, experts, -1, allocation.data_ptr(),
        alloc_cumsum.data_ptr(), experts_to_copy.data_ptr(), inverse.data_ptr(),
        replica_counts.data_ptr(), stats.data_ptr()), "mm_moonep_plan_host")
    _raise_for(int(stats[1]), counts.to(torch.int64).sum(dim=1))
    return MoonEPPlanningResult(alloc_cumsum=alloc_cumsum, experts_to_copy=experts_to_copy)


def build_inverse_experts_to_copy(experts_to_copy: torch.Tensor, num_experts: int) -> torch.Tensor:
    """``inverse[d, e]`` = replica slot of expert ``e`` on rank ``d`` or ``-1``
    (reference: runtime/moonep_planning.py:279-322)."""
    if not isinstance(experts_to_copy, torch.Tensor):
        raise TypeError("experts_to_copy must be a torch.Tensor")
    if experts_to_copy.device.type != "cpu":
        raise ValueError("experts_to_copy must be a CPU tensor")
    if experts_to_copy.dtype != torch.int32:
        raise TypeError("experts_to_copy must have dtype torch.int32")
    if experts_to_copy.ndim != 2 or not experts_to_copy.is_contiguous():
        raise ValueError("experts_to_copy must be a contiguous rank-2 tensor")
    if type(num_experts) is not int or num_experts <= 0:
        raise ValueError("num_experts must be a positive integer")
    world, budget = (int(v) for v in experts_to_copy.shape)
    if world <= 0 or num_experts % world:
        raise ValueError("num_experts must be divisible by world_size")
    epr = num_experts // world
    if budget != epr:
        raise ValueError("replica budget must equal experts_per_rank")
    etc = experts_to_copy.to(torch.int64)
    used = etc != -1
    if bool((used & ((etc < 0) | (etc >= num_experts))).any()):
        raise ValueError("experts_to_copy contains an invalid expert id")
    ranks = torch.arange(world).unsqueeze(1).expand_as(etc)
    if bool((used & (torch.div(etc, epr, rounding_mode="floor") == ranks)).any()):
        raise ValueError("experts_to_copy must contain only remote experts")
    slots = torch.arange(budget, dtype=torch.int32).unsqueeze(0).expand_as(etc)
    inverse = torch.full((world, num_experts), -1, dtype=torch.int32)
    hits = torch.zeros((world, num_experts), dtype=torch.int32)
    hits.index_put_((ranks[used], etc[used]), torch.ones(int(used.sum()), dtype=torch.int32),
                    accumulate=True)
    if bool((hits > 1).any()):
        raise ValueError("experts_to_copy contains duplicate experts in a row")
    inverse[ranks[used], etc[used]] = slots[used]
    return inverse


def launch_moonep_b0_b3(tpe_all: torch.Tensor, allocation: torch.Tensor,
                        alloc_cumsum: torch.Tensor, experts_to_copy: torch.Tensor,
                        inverse_experts_to_copy: torch.Tensor, replica_counts: torch.Tensor,
                        plan_stats: torch.Tensor, *, world_size: int, num_experts: int,
                        experts_per_rank: int, row_stride: int, total_bin: int = -1,
                        status: Optional[torch.Tensor] = None) -> None:
    """Queue the device planner on the current stream (reference:
    kernels/moonep_planning.py:365-460, four launches there, one here).  ``tpe_all`` is the
    replicated ``[R, row_stride]`` int32 count cube on the device; ``total_bin`` names the
    column with each rank's unfiltered route count, if the cube has one.  Nothing is read back:
    an input the planner rejects leaves ``plan_stats[1] != 0``, status code 4 and the plan that
    keeps every expert at home."""
    if num_experts % world_size or experts_per_rank != num_experts // world_size:
        raise ValueError("MoonEP requires E to be divisible by world size")
    expected = {
        "tpe_all": (tpe_all, (world_size, row_stride)),
        "allocation": (allocation, (world_size, num_experts)),
        "alloc_cumsum": (alloc_cumsum, (num_experts, world_size)),
        "experts_to_copy": (experts_to_copy, (world_size, experts_per_rank)),
        "inverse_experts_to_copy": (inverse_experts_to_copy, (world_size, num_experts)),
        "replica_counts": (replica_counts, (world_size,)),
        "plan_stats": (plan_stats, (4,)),
    }
    device = tpe_all.device
    if device.type != "cuda":
        raise ValueError("launch_moonep_b0_b3 takes device tensors; use plan_moonep_b0_b3 on the host")
    for name, (t, shape) in expected.items():
        if tuple(t.shape) != shape or t.dtype != torch.int32:
            raise ValueError(f"{name} must have shape {shape} and dtype torch.int32")
        if t.device != device or not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous on {device}")
    N.check(N.lib().mm_moonep_plan(
        tpe_all.data_ptr(), row_stride, world_size, num_experts, total_bin,
        allocation.data_ptr(), alloc_cumsum.data_ptr(), experts_to_copy.data_ptr(),
        inverse_experts_to_copy.data_ptr(), replica_counts.data_ptr(), plan_stats.data_ptr(),
        N.ptr(status), N.stream_ptr(device)), "mm_moonep_plan")
    N.count_launches(1)


__all__ = [
    "MoonEPPlanningResult",
    "build_inverse_experts_to_copy",
    "launch_moonep_b0_b3",
    "plan_moonep_b0_b3",
]
