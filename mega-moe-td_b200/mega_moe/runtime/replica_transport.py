"""MoonEP replica transport: replica weight tables in symmetric memory, the owner-push of
expert weights into them and the owner-pull of replica weight gradients.

Counterparts in the reference: ``ReplicaWeightBuffers`` and its allocation
(src/mega_moe/runtime/replica_weight_prefetch.py:105-310), the owner-push kernels
(src/mega_moe/kernels/replica_weight_prefetch.py:17-180) and the owner-pull reduction
(src/mega_moe/kernels/replica_grad_reduce.py:62-190, src/mega_moe/runtime/replica_grad_transport.py).
As in the reference, the backward reuses the replica *weight* tables as the landing zone of the
replica weight gradients, so one pair of symmetric tables serves both directions.

The byte movers are ``mm_moonep_push_replicas`` / ``mm_moonep_pull_replica_grads`` of the shared
library.  Ordering between ranks is the caller's: a rank barrier after the push (before a
destination reads its slots), one before the pull (after every rank has written its replica
gradients) and one after it (before the slots are written again).

``FusedMoEForward`` does not use this module yet; ``enable_moonep=True`` raises
``NotImplementedError``.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch

from .. import _native as N
from .workspace import SymmetricBlock


@dataclass
class ReplicaWeightBuffers:
    """Per rank ``E/R`` replica slots for the two weight tables of an expert:
    ``gate_up [E/R, H, 2F]`` and ``down [E/R, F, H]`` (any per-expert shape works; the transport
    moves bytes).  ``gate_up_peers`` / ``down_peers``: device int64 tensors with every rank's base
    pointer of that table."""

    symm: SymmetricBlock
    gate_up: torch.Tensor
    down: torch.Tensor
    gate_up_peers: torch.Tensor
    down_peers: torch.Tensor
    experts_per_rank: int

    def free(self) -> None:
        self.symm.free()


def allocate_replica_weight_buffers(gate_up_weight: torch.Tensor, down_weight: torch.Tensor, *,
                                    rank: int, world_size: int, group=None
                                    ) -> ReplicaWeightBuffers:
    """Symmetric replica tables shaped like this rank's home weights ``[E/R, ...]`` (reference:
    runtime/replica_weight_prefetch.py:236-310).  Collective over ``group`` when
    ``world_size > 1`` (the CUDA-IPC handles are exchanged)."""
    for name, w in (("gate_up_weight", gate_up_weight), ("down_weight", down_weight)):
        if w.device.type != "cuda":
            raise ValueError(f"{name} must be a CUDA tensor")
        if w.dtype != torch.bfloat16:
            raise TypeError(f"{name} must have dtype torch.bfloat16")
        if w.ndim < 2:
            raise ValueError(f"{name} must have a leading expert dimension")
    if gate_up_weight.shape[0] != down_weight.shape[0]:
        raise ValueError("the two weight tables disagree on the number of local experts")
    epr = int(gate_up_weight.shape[0])
    sizes = {"gate_up": gate_up_weight[0].numel() * 2 * epr, "down": down_weight[0].numel() * 2 * epr}
    for name, size in sizes.items():
        if (size // epr) % 16:
            raise ValueError(f"one expert of the {name} table must be a multiple of 16 bytes")
    symm = SymmetricBlock(sizes, rank, world_size, group, gate_up_weight.device)
    return ReplicaWeightBuffers(
        symm=symm,
        gate_up=symm.local("gate_up", torch.bfloat16).view(gate_up_weight.shape),
        down=symm.local("down", torch.bfloat16).view(down_weight.shape),
        gate_up_peers=symm.peer_table("gate_up"),
        down_peers=symm.peer_table("down"),
        experts_per_rank=epr,
    )


def _table(local: torch.Tensor, peers: torch.Tensor, name: str) -> N.ReplicaTable:
    """Descriptor of one ``[E/R, ...]`` table whose experts are contiguous blocks (the table
    itself may be strided along the expert dimension)."""
    per_expert = local[0]
    if not per_expert.is_contiguous():
        raise ValueError(f"{name}: every expert's block must be contiguous")
    if local.dtype != torch.bfloat16:
        raise TypeError(f"{name} must have dtype torch.bfloat16")
    return N.ReplicaTable(local.data_ptr(), local.stride(0) * 2 if local.shape[0] > 1 else
                          per_expert.numel() * 2, per_expert.numel() * 2, peers.data_ptr())


def push_replica_weights(experts_to_copy: torch.Tensor, gate_up_weight: torch.Tensor,
                         down_weight: Optional[torch.Tensor], buffers: ReplicaWeightBuffers, *,
                         rank: int, world_size: int, grid_limit: int = 0) -> None:
    """Queue the owner-push on the current stream: every expert of this rank that
    ``experts_to_copy [R, E/R]`` (device int32, from the planner) places in a replica slot of
    another rank is stored into that slot."""
    if experts_to_copy.dtype != torch.int32 or not experts_to_copy.is_contiguous():
        raise TypeError("experts_to_copy must be a contiguous int32 tensor")
    if tuple(experts_to_copy.shape) != (world_size, buffers.experts_per_rank):
        raise ValueError("experts_to_copy must have shape [R, E/R]")
    t0 = _table(gate_up_weight, buffers.gate_up_peers, "gate_up_weight")
    t1 = _table(down_weight, buffers.down_peers, "down_weight") if down_weight is not None else None
    N.check(N.lib().mm_moonep_push_replicas(
        experts_to_copy.data_ptr(), rank, world_size, buffers.experts_per_rank, C.byref(t0),
        C.byref(t1) if t1 is not None else None, grid_limit,
        N.stream_ptr(experts_to_copy.device)), "mm_moonep_push_replicas")
    N.count_launches(1)


def pull_replica_weight_grads(inverse_experts_to_copy: torch.Tensor, grad_gate_up: torch.Tensor,
                              grad_down: Optional[torch.Tensor], buffers: ReplicaWeightBuffers, *,
                              rank: int, world_size: int, grid_limit: int = 0) -> None:
    """Queue the owner-pull on the current stream: the gradients that other ranks left in the
    replica slots holding this rank's experts are added, in fp32 and in ascending rank order,
    onto ``grad_gate_up`` / ``grad_down`` (``[E/R, ...]`` bf16, updated in place)."""
    inv = inverse_experts_to_copy
    if inv.dtype != torch.int32 or not inv.is_contiguous():
        raise TypeError("inverse_experts_to_copy must be a contiguous int32 tensor")
    if tuple(inv.shape) != (world_size, world_size * buffers.experts_per_rank):
        raise ValueError("inverse_experts_to_copy must have shape [R, E]")
    t0 = _table(grad_gate_up, buffers.gate_up_peers, "grad_gate_up")
    t1 = _table(grad_down, buffers.down_peers, "grad_down") if grad_down is not None else None
    N.check(N.lib().mm_moonep_pull_replica_grads(
        inv.data_ptr(), rank, world_size, buffers.experts_per_rank, C.byref(t0),
        C.byref(t1) if t1 is not None else None, grid_limit, N.stream_ptr(inv.device)),
        "mm_moonep_pull_replica_grads")
    N.count_launches(1)


__all__ = [
    "ReplicaWeightBuffers",
    "allocate_replica_weight_buffers",
    "pull_replica_weight_grads",
    "push_replica_weights",
]
