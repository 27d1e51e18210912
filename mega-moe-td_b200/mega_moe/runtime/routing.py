"""Stable route filtering, count exchange and typed dispatch metadata.

Counterpart of the reference's ``runtime/routing.py`` (MoERoutingPlan at lines 21-54,
build_routing_plan at 621-768).  The metadata is produced by CUDA kernels
(``mm_route_local`` / ``mm_route_finalize``); between them every rank stores its count row
into all ranks' count cubes (``mm_count_exchange``: peer stores behind an epoch flag, like the
reference's in-kernel publication, kernels/fused_forward.py:158-238), so that every rank holds
the whole ``[world, bins]`` count cube, which ``send_bucket_dst_starts`` needs (it sums *other*
sources' counts to a destination).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import _native as N
from .workspace import MoEForwardContext


@dataclass
class MoERoutingPlan:
    """Single-in-flight routing metadata shared by dispatch and combine.

    Invalid expert ids are represented by ``valid_route_mask`` and are omitted from all
    communication.  The remaining routes are stable-sorted by global expert id, preserving
    the exact inverse-order contract used by combine.
    """

    num_input_tokens: int
    num_received_routes: int
    selected_experts: torch.Tensor
    send_token_indices: torch.Tensor
    send_bucket_starts: torch.Tensor
    send_bucket_receive_offsets: torch.Tensor
    send_counts_by_rank_expert: torch.Tensor
    num_sent_routes: int
    received_routes_per_expert: torch.Tensor
    received_expert_offsets: torch.Tensor
    receive_counts_by_source_expert: torch.Tensor
    stable_sort_indices: torch.Tensor
    valid_route_mask: torch.Tensor
    physical_experts_per_rank: int = 0
    active_physical_experts_per_rank: int = 0
    experts_to_copy: torch.Tensor | None = None
    send_route_indices: torch.Tensor | None = None
    experts_to_copy_cpu: torch.Tensor | None = None
    owner_token: object | None = None
    generation: int = 0
    selected_experts_version: int = -1


def launch_routing_metadata(context: MoEForwardContext, selected_experts: torch.Tensor) -> None:
    """Enqueue the metadata kernels for ``selected_experts``; no host synchronisation.

    Afterwards the context tables hold: send order (``send_route_indices``,
    ``send_token_indices``, ``send_bucket``), ``route_to_send``, the count cube, all offset
    tables, the 128-row tile table and the per-received-row source tables.
    """
    lib = N.lib()
    ctx = context
    num_routes = selected_experts.numel()
    stream = N.stream_ptr()
    from ..ops import _launch as L
    timer = L._timed("routing_metadata")
    timer.__enter__()
    N.check(lib.mm_route_local(
        selected_experts.data_ptr(), num_routes, ctx.top_k, ctx.num_experts,
        ctx.metadata_num_bins, ctx.send_route_indices.data_ptr(),
        ctx.send_token_indices.data_ptr(), ctx.send_bucket.data_ptr(),
        ctx.route_to_send.data_ptr(), ctx.metadata_count_row.data_ptr(),
        ctx.metadata_local_stats.data_ptr(), ctx.route_scratch.data_ptr(),
        ctx.route_scratch.numel(), stream), "mm_route_local")
    bins = ctx.metadata_num_bins
    # Count exchange: the row goes into every rank's cube by peer stores behind an epoch flag
    # (no collective library call on the path); two cubes alternate so that a rank that is
    # already one launch ahead never writes into the cube a slower rank still reads.
    ctx.count_epoch += 1
    if ctx.count_epoch >= 2**31 - 1:
        raise RuntimeError("count-exchange epoch exhausted; recreate the operator")
    parity = ctx.count_epoch & 1
    ctx.metadata_counts_mem = ctx.count_cubes[parity]
    N.check(lib.mm_count_exchange(
        ctx.metadata_count_row.data_ptr(), bins, ctx.rank, ctx.world_size,
        ctx.symm.peer_table("count_cubes").data_ptr(), parity * ctx.world_size * bins,
        ctx.symm.peer_table("count_flags").data_ptr(), ctx.count_flags.data_ptr(),
        ctx.count_epoch, ctx.status.data_ptr(), stream), "mm_count_exchange")
    N.check(lib.mm_route_finalize(
        ctx.metadata_counts_mem.data_ptr(), ctx.rank, ctx.world_size, ctx.experts_per_rank, bins,
        ctx.max_received_routes,
        ctx.metadata_send_bucket_starts.data_ptr(), ctx.metadata_send_bucket_dst_starts.data_ptr(),
        ctx.metadata_recv_counts_re.data_ptr(), ctx.metadata_recv_per_expert.data_ptr(),
        ctx.metadata_recv_expert_offs.data_ptr(), ctx.metadata_recv_seg_starts.data_ptr(),
        ctx.metadata_pull_dst_start.data_ptr(), ctx.metadata_stats.data_ptr(),
        ctx.mtile_group.data_ptr(), ctx.mtile_row0.data_ptr(), ctx.num_mtiles.data_ptr(),
        ctx.mtile2_group.data_ptr(), ctx.mtile2_row0.data_ptr(), ctx.num_mtiles2.data_ptr(),
        ctx.row_src_rank.data_ptr(), ctx.row_src_pos.data_ptr(),
        ctx.disp_order_prefix.data_ptr(), ctx.disp_bucket_done.data_ptr(),
        ctx.row_arrival.data_ptr(), ctx.arrival_row.data_ptr(),
        ctx.status.data_ptr(), stream),
        "mm_route_finalize")
    timer.__exit__()
    N.count_launches(6)  # histogram, scan, scatter, count exchange, offsets, row tables


def check_receive_capacity(context: MoEForwardContext) -> None:
    """Raise ``ValueError`` like the reference (runtime/routing.py:738-744) on overflow."""
    if context.receive_capacity_factor < context.world_size:
        required = int(context.metadata_stats[1].item())
        if required > context.max_received_routes:
            context.reset_status()
            raise ValueError(
                f"peer buffer capacity {context.max_received_routes} routes is smaller than "
                f"the required receive size {required}")


def build_routing_plan(context: MoEForwardContext, selected_experts: torch.Tensor,
                       **_unused) -> MoERoutingPlan:
    """Build one stable, compact routing plan for dispatch and combine."""
    world_size = context.world_size
    experts_per_rank = context.experts_per_rank
    num_experts = context.num_experts
    launch_routing_metadata(context, selected_experts)
    flat_experts = selected_experts.reshape(-1)
    valid_route_mask = (flat_experts >= 0) & (flat_experts < num_experts)
    num_valid = int(context.metadata_local_stats[0].item())
    num_received_routes = int(context.metadata_stats[0].item())
    check_receive_capacity(context)
    send_route_indices = context.send_route_indices[:num_valid]
    send_token_indices = context.send_token_indices[:num_valid]
    # Position of each send row among the kept (valid) routes: the stable argsort the
    # reference computes with torch.argsort (runtime/routing.py:648-650).
    kept_rank = torch.cumsum(valid_route_mask.to(torch.int64), 0) - 1
    stable_sort_indices = kept_rank[send_route_indices.long()]
    bins = context.metadata_num_bins
    local_count_start = context.rank * bins
    send_counts = context.metadata_counts_mem[
        local_count_start:local_count_start + num_experts].view(world_size, experts_per_rank)
    return MoERoutingPlan(
        num_input_tokens=selected_experts.shape[0],
        num_received_routes=num_received_routes,
        selected_experts=selected_experts,
        send_token_indices=send_token_indices,
        send_route_indices=send_route_indices,
        send_bucket_starts=context.metadata_send_bucket_starts,
        send_bucket_receive_offsets=context.metadata_send_bucket_dst_starts,
        send_counts_by_rank_expert=send_counts,
        num_sent_routes=num_valid,
        received_routes_per_expert=context.metadata_recv_per_expert,
        received_expert_offsets=context.metadata_recv_expert_offs,
        receive_counts_by_source_expert=context.metadata_recv_counts_re,
        stable_sort_indices=stable_sort_indices,
        valid_route_mask=valid_route_mask,
        physical_experts_per_rank=experts_per_rank,
        active_physical_experts_per_rank=experts_per_rank,
        experts_to_copy=None,
    )


__all__ = ["MoERoutingPlan", "build_routing_plan", "launch_routing_metadata"]
