"""MoonEP-balanced routing metadata: every route's physical bucket and the offset tables of
the balanced dispatch.

Same names and contract as the reference's ``build_balanced_routing_metadata``
(src/mega_moe/runtime/balanced_routing.py:24-55, 545-805): routes are numbered per logical
expert in stable (token, top-k slot) order across the source ranks; the rank whose allocation
interval holds a route's number executes it, in the expert's home slot or in its replica slot
there; ``bucket = rank * 2 * E/R + physical slot``; the send order is bucket-major and stable;
the receive side stores rows slot-major and, inside a slot, by increasing source rank.

Where the numbers are computed:

* the balanced count cube, the per-expert tables and the placement of every route: the shared
  library (``mm_moonep_count_cube`` / ``mm_moonep_map_routes`` on the device, their ``*_host``
  twins for CPU tensors; one implementation, ``csrc/moonep_core.h``);
* on the device the remaining offset tables come from ``mm_route_finalize`` run on the balanced
  cube with ``2 * E/R`` slots per rank (:func:`launch_balanced_routing`); for CPU tensors they are
  four prefix sums of the cube, written here in torch.

``FusedMoEForward`` does not consume these tables yet (``enable_moonep=True`` raises
``NotImplementedError``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import _native as N

_INT32_MAX = (1 << 31) - 1


@dataclass(frozen=True)
class BalancedRoutingMetadata:
    """Field for field the reference's record (runtime/balanced_routing.py:24-55).
    ``final_order``: original flattened route ids in send order; ``balanced_buckets``: bucket of
    each send row; ``balanced_counts[source, bucket]``: the whole group's cube."""

    rank: int
    world_size: int
    num_experts: int
    experts_per_rank: int
    replica_slots_per_rank: int
    physical_slots_per_rank: int
    num_input_tokens: int
    num_valid_routes: int
    valid_route_mask: torch.Tensor
    final_order: torch.Tensor
    send_token_indices: torch.Tensor
    send_route_indices: torch.Tensor
    balanced_buckets: torch.Tensor
    balanced_counts: torch.Tensor
    send_bucket_starts: torch.Tensor
    send_bucket_receive_offsets: torch.Tensor
    receive_counts_by_source_slot: torch.Tensor
    received_routes_per_slot: torch.Tensor
    received_slot_offsets: torch.Tensor


def _require_integral(name: str, t: torch.Tensor, ndim: int) -> None:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if t.dtype not in (torch.int32, torch.int64):
        raise TypeError(f"{name} must have dtype torch.int32 or torch.int64")
    if t.ndim != ndim:
        raise ValueError(f"{name} must be rank {ndim}")


def _validate(selected, tpe_all, alloc_cumsum, inverse, rank) -> None:
    """Input contract of runtime/balanced_routing.py:72-154."""
    _require_integral("selected_experts", selected, 2)
    _require_integral("tpe_all", tpe_all, 2)
    _require_integral("alloc_cumsum", alloc_cumsum, 2)
    _require_integral("inverse_experts_to_copy", inverse, 2)
    for name, t in (("tpe_all", tpe_all), ("alloc_cumsum", alloc_cumsum),
                    ("inverse_experts_to_copy", inverse)):
        if t.device != selected.device:
            raise ValueError(f"{name} must be on {selected.device}")
    world, experts = (int(v) for v in tpe_all.shape)
    if world <= 0 or experts <= 0:
        raise ValueError("world_size and num_experts must be positive")
    if experts % world:
        raise ValueError("num_experts must be divisible by world_size")
    if type(rank) is not int or not 0 <= rank < world:
        raise ValueError("rank must identify a source rank in the EP group")
    if selected.shape[1] <= 0:
        raise ValueError("selected_experts top-k dimension must be positive")
    if tuple(alloc_cumsum.shape) != (experts, world):
        raise ValueError("alloc_cumsum must have shape [E, R]")
    if tuple(inverse.shape) != (world, experts):
        raise ValueError("inverse_experts_to_copy must have shape [R, E]")
    tpe = tpe_all.to(torch.int64)
    alloc = alloc_cumsum.to(torch.int64)
    inv = inverse.to(torch.int64)
    if bool((tpe < 0).any()):
        raise ValueError("tpe_all counts must be non-negative")
    if bool((alloc < 0).any()):
        raise ValueError("alloc_cumsum must be non-negative")
    if world > 1 and bool((alloc[:, 1:] < alloc[:, :-1]).any()):
        raise ValueError("alloc_cumsum must be monotone along destination rank")
    if not torch.equal(alloc[:, -1], tpe.sum(dim=0)):
        raise ValueError("alloc_cumsum must conserve every logical expert")
    epr = experts // world
    if bool(((inv < -1) | (inv >= epr)).any()):
        raise ValueError("inverse replica slots must be -1 or in [0, E/R)")
    owner = torch.arange(experts, device=inv.device) // epr
    at_home = owner.unsqueeze(0) == torch.arange(world, device=inv.device).unsqueeze(1)
    if bool((at_home & (inv != -1)).any()):
        raise ValueError("inverse table must not assign slots to home experts")
    per_slot = torch.zeros((world, epr), dtype=torch.int64, device=inv.device)
    taken = inv >= 0
    per_slot.index_put_((taken.nonzero()[:, 0], inv[taken]),
                        torch.ones(int(taken.sum()), dtype=torch.int64, device=inv.device),
                        accumulate=True)
    if bool((per_slot > 1).any()):
        raise ValueError("inverse table contains duplicate replica slots")
    executed = torch.diff(alloc, dim=1, prepend=torch.zeros_like(alloc[:, :1])).t()  # [R, E]
    if bool(((executed > 0) & ~at_home & (inv < 0)).any()):
        raise ValueError("a remote allocation is missing its replica slot")


def experts_to_copy_from_inverse(inverse: torch.Tensor, experts_per_rank: int) -> torch.Tensor:
    """The ``[R, E/R]`` replica list behind an ``[R, E]`` inverse table, ``-1`` for empty slots
    (reference: runtime/balanced_routing.py:157-173)."""
    world, experts = inverse.shape
    etc = torch.full((world, experts_per_rank), -1, dtype=torch.int32, device=inverse.device)
    where = (inverse >= 0).nonzero()
    etc[where[:, 0], inverse[where[:, 0], where[:, 1]].long()] = where[:, 1].to(torch.int32)
    return etc


def _i32(name: str, t: torch.Tensor, validate: bool) -> torch.Tensor:
    if validate and t.numel() and int(t.max()) > _INT32_MAX:
        raise ValueError(f"{name} exceeds the int32 metadata range")
    return t.to(torch.int32).contiguous()


def build_balanced_routing_metadata(
    selected_experts: torch.Tensor,
    tpe_all: torch.Tensor,
    alloc_cumsum: torch.Tensor,
    inverse_experts_to_copy: torch.Tensor,
    rank: int,
    *,
    validate: bool = True,
    expert_order: Optional[torch.Tensor] = None,
    sorted_experts: Optional[torch.Tensor] = None,
    use_direct_bucket_scatter: bool = False,
    use_fused_count_cube: bool = True,
) -> BalancedRoutingMetadata:
    """Balanced dispatch metadata of source rank ``rank`` for host tensors (reference:
    runtime/balanced_routing.py:545-805).  Routes are always placed directly by interval
    arithmetic, which the reference proves equal to its stable bucket sort;
    ``use_direct_bucket_scatter`` and ``use_fused_count_cube`` are accepted for compatibility and
    change nothing.  Device tensors go through :func:`launch_balanced_routing`."""
    for name, flag in (("validate", validate),
                       ("use_direct_bucket_scatter", use_direct_bucket_scatter),
                       ("use_fused_count_cube", use_fused_count_cube)):
        if type(flag) is not bool:
            raise TypeError(f"{name} must be a bool")
    if isinstance(selected_experts, torch.Tensor) and selected_experts.device.type != "cpu":
        raise ValueError("build_balanced_routing_metadata takes host tensors; the device path is "
                         "launch_balanced_routing")
    if validate:
        _validate(selected_experts, tpe_all, alloc_cumsum, inverse_experts_to_copy, rank)
    world, experts = (int(v) for v in tpe_all.shape)
    epr = experts // world
    slots = 2 * epr
    buckets = world * slots
    top_k = int(selected_experts.shape[1])
    num_flat = int(selected_experts.numel())
    if num_flat > _INT32_MAX:
        raise ValueError("flattened route ids exceed the int32 metadata range")
    if (expert_order is None) != (sorted_experts is None):
        raise ValueError("expert_order and sorted_experts must either both be provided or "
                         "both be omitted")

    flat = selected_experts.reshape(-1).to(torch.int64)
    valid_mask = (flat >= 0) & (flat < experts)
    if expert_order is not None:
        for name, t in (("expert_order", expert_order), ("sorted_experts", sorted_experts)):
            _require_integral(name, t, 1)
            if t.numel() != num_flat:
                raise ValueError(f"{name} must contain every route in the dropless input")
        if validate and not bool(valid_mask.all()):
            raise ValueError("precomputed expert order is only valid for dropless routes")
        if validate:
            want = torch.argsort(flat, stable=True)
            if not torch.equal(expert_order.to(torch.int64), want):
                raise ValueError("expert_order is not Mega's stable expert order")
            if not torch.equal(sorted_experts.to(torch.int64), flat[want]):
                raise ValueError("sorted_experts does not match selected_experts[expert_order]")
        route_in = expert_order.to(torch.int32).contiguous()
        expert_in = sorted_experts.to(torch.int32).contiguous()
    else:
        ids = valid_mask.nonzero().reshape(-1)
        order = torch.argsort(flat[ids], stable=True)
        route_in = ids[order].to(torch.int32).contiguous()
        expert_in = flat[ids][order].to(torch.int32).contiguous()
    num_valid = int(route_in.numel())
    if validate and not torch.equal(torch.bincount(expert_in.long(), minlength=experts),
                                    tpe_all[rank].to(torch.int64)):
        raise ValueError("the valid selected_experts histogram must equal tpe_all[rank]")

    counts = tpe_all.to(torch.int32).contiguous()
    prefix = alloc_cumsum.to(torch.int32).contiguous()
    inverse = inverse_experts_to_copy.to(torch.int32).contiguous()
    etc = experts_to_copy_from_inverse(inverse, epr).contiguous()
    cube = torch.empty((world, buckets), dtype=torch.int32)
    expert_start = torch.empty((experts,), dtype=torch.int32)
    below = torch.empty((experts,), dtype=torch.int32)
    lib = N.lib()
    N.check(lib.mm_moonep_count_cube_host(
        counts.data_ptr(), experts, rank, world, experts, prefix.data_ptr(), etc.data_ptr(),
        cube.data_ptr(), buckets, expert_start.data_ptr(), below.data_ptr()),
        "mm_moonep_count_cube_host")
    cube64 = cube.to(torch.int64)
    if validate and not torch.equal(cube64.sum(dim=1), tpe_all.to(torch.int64).sum(dim=1)):
        raise RuntimeError("balanced count construction lost source routes")

    own = cube64[rank]
    send_bucket_starts = own.cumsum(0) - own
    send_route = torch.full((num_valid,), -1, dtype=torch.int32)
    send_token = torch.full((num_valid,), -1, dtype=torch.int32)
    send_bucket = torch.full((num_valid,), -1, dtype=torch.int32)
    route_to_send = torch.full((max(num_flat, 1),), -1, dtype=torch.int32)
    misplaced = torch.zeros((1,), dtype=torch.int32)
    starts32 = _i32("send_bucket_starts", send_bucket_starts, validate)
    if num_valid:
        N.check(lib.mm_moonep_map_routes_host(
            route_in.data_ptr(), expert_in.data_ptr(), num_valid, num_flat, top_k, world, experts,
            expert_start.data_ptr(), below.data_ptr(), prefix.data_ptr(), inverse.data_ptr(),
            starts32.data_ptr(), send_route.data_ptr(), send_token.data_ptr(),
            send_bucket.data_ptr(), route_to_send.data_ptr(), misplaced.data_ptr()),
            "mm_moonep_map_routes_host")
    if int(misplaced):
        raise RuntimeError("a route has no destination allocation or no replica slot")
    if validate and num_valid:
        if bool((send_route < 0).any()):
            raise RuntimeError("direct balanced bucket scatter produced duplicate or "
                               "out-of-range positions")
        if not torch.equal(torch.bincount(send_bucket.long(), minlength=buckets), own):
            raise RuntimeError("local route buckets disagree with balanced counts")

    by_dest_slot = cube64.view(world, world, slots)
    per_dest_slot = by_dest_slot.sum(dim=0)
    slot_starts = per_dest_slot.cumsum(dim=1) - per_dest_slot
    receive_offsets = slot_starts.reshape(-1) + cube64[:rank].sum(dim=0)
    received = by_dest_slot[:, rank, :]
    per_slot = received.sum(dim=0)
    slot_offsets = torch.cat((torch.zeros(1, dtype=torch.int64), per_slot.cumsum(0)))

    return BalancedRoutingMetadata(
        rank=rank, world_size=world, num_experts=experts, experts_per_rank=epr,
        replica_slots_per_rank=epr, physical_slots_per_rank=slots,
        num_input_tokens=int(selected_experts.shape[0]), num_valid_routes=num_valid,
        valid_route_mask=valid_mask.contiguous(),
        final_order=send_route.to(torch.int64),
        send_token_indices=send_token,
        send_route_indices=send_route,
        balanced_buckets=send_bucket,
        balanced_counts=cube,
        send_bucket_starts=starts32,
        send_bucket_receive_offsets=_i32("send_bucket_receive_offsets", receive_offsets, validate),
        receive_counts_by_source_slot=_i32("receive_counts_by_source_slot", received, validate),
        received_routes_per_slot=_i32("received_routes_per_slot", per_slot, validate),
        received_slot_offsets=_i32("received_slot_offsets", slot_offsets, validate),
    )


def launch_balanced_routing(*, count_cube: torch.Tensor, rank: int, world_size: int,
                            num_experts: int, top_k: int, alloc_cumsum: torch.Tensor,
                            experts_to_copy: torch.Tensor, inverse_experts_to_copy: torch.Tensor,
                            expert_major_routes: torch.Tensor, expert_major_experts: torch.Tensor,
                            local_stats: torch.Tensor, balanced_cube: torch.Tensor,
                            expert_start: torch.Tensor, below: torch.Tensor,
                            finalize, send_bucket_starts: torch.Tensor,
                            send_route: torch.Tensor, send_token: torch.Tensor,
                            send_bucket: torch.Tensor, route_to_send: torch.Tensor,
                            status: Optional[torch.Tensor] = None) -> None:
    """Queue the device side of the balanced routing on the current stream (reference:
    ``build_balanced_routing_metadata_inplace``, runtime/balanced_routing.py:372-541):

    1. ``mm_moonep_count_cube``: ``count_cube [R, stride]`` + plan -> ``balanced_cube
       [R, >= 2E]``, ``expert_start [E]``, ``below [E]``;
    2. ``finalize(balanced_cube)``: the caller's ``mm_route_finalize`` launch on that cube with
       ``epr = 2 * E/R``; it fills ``send_bucket_starts`` and every receive-side table;
    3. ``mm_moonep_map_routes``: ``expert_major_routes`` / ``expert_major_experts`` (the
       ``send_route`` / ``send_bucket`` of ``mm_route_local``) -> bucket-major ``send_route``,
       ``send_token``, ``send_bucket``; ``route_to_send`` updated in place.
    """
    device = count_cube.device
    if device.type != "cuda":
        raise ValueError("launch_balanced_routing takes device tensors")
    lib = N.lib()
    stream = N.stream_ptr(device)
    N.check(lib.mm_moonep_count_cube(
        count_cube.data_ptr(), count_cube.stride(0), rank, world_size, num_experts,
        alloc_cumsum.data_ptr(), experts_to_copy.data_ptr(), balanced_cube.data_ptr(),
        balanced_cube.stride(0), expert_start.data_ptr(), below.data_ptr(), stream),
        "mm_moonep_count_cube")
    finalize(balanced_cube)
    N.check(lib.mm_moonep_map_routes(
        expert_major_routes.data_ptr(), expert_major_experts.data_ptr(), local_stats.data_ptr(),
        int(expert_major_routes.numel()), top_k, world_size, num_experts,
        expert_start.data_ptr(), below.data_ptr(), alloc_cumsum.data_ptr(),
        inverse_experts_to_copy.data_ptr(), send_bucket_starts.data_ptr(),
        send_route.data_ptr(), send_token.data_ptr(), send_bucket.data_ptr(),
        route_to_send.data_ptr(), N.ptr(status), stream), "mm_moonep_map_routes")
    N.count_launches(2)


def launch_physical_relabel(*, count_cube: torch.Tensor, rank: int, world_size: int,
                            num_experts: int, alloc_cumsum: torch.Tensor,
                            experts_to_copy: torch.Tensor, inverse_experts_to_copy: torch.Tensor,
                            expert_major_routes: torch.Tensor, expert_major_experts: torch.Tensor,
                            route_to_send: torch.Tensor, local_stats: torch.Tensor,
                            balanced_cube: torch.Tensor, expert_start: torch.Tensor,
                            below: torch.Tensor, physical: torch.Tensor,
                            status: Optional[torch.Tensor] = None) -> None:
    """Queue MoonEP as a re-labelling on the current stream: ``physical[route]`` (int32, one
    entry per flattened ``(token, top-k slot)``) receives the bucket ``rank * 2 * E/R + slot``
    that executes the route, ``-1`` for dropped routes.  Feeding ``physical`` as the expert ids
    of a layer with ``2 * E`` experts (``2 * E/R`` per rank: home slots, then replica slots) to
    the ordinary routing gives the balanced send order, cube and offsets, so dispatch, GEMMs,
    combine and backward run unchanged over the physical slots.  ``balanced_cube`` is written
    too (a by-product of the per-expert tables)."""
    device = count_cube.device
    if device.type != "cuda":
        raise ValueError("launch_physical_relabel takes device tensors")
    lib = N.lib()
    stream = N.stream_ptr(device)
    N.check(lib.mm_moonep_count_cube(
        count_cube.data_ptr(), count_cube.stride(0), rank, world_size, num_experts,
        alloc_cumsum.data_ptr(), experts_to_copy.data_ptr(), balanced_cube.data_ptr(),
        balanced_cube.stride(0), expert_start.data_ptr(), below.data_ptr(), stream),
        "mm_moonep_count_cube")
    N.check(lib.mm_moonep_relabel_routes(
        expert_major_routes.data_ptr(), expert_major_experts.data_ptr(),
        route_to_send.data_ptr(), local_stats.data_ptr(), int(physical.numel()), world_size,
        num_experts, expert_start.data_ptr(), below.data_ptr(), alloc_cumsum.data_ptr(),
        inverse_experts_to_copy.data_ptr(), physical.data_ptr(), N.ptr(status), stream),
        "mm_moonep_relabel_routes")
    N.count_launches(2)


__all__ = [
    "BalancedRoutingMetadata",
    "build_balanced_routing_metadata",
    "experts_to_copy_from_inverse",
    "launch_balanced_routing",
    "launch_physical_relabel",
]
