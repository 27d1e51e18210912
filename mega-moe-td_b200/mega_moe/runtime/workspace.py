"""Symmetric (peer-mapped) buffers and reusable metadata workspaces of one MoE operator.

Counterpart of the reference's ``runtime/workspace.py`` (MoEForwardContext,
create_moe_forward_context: src/mega_moe/runtime/workspace.py:11-314).  The ACLSHMEM
symmetric heap becomes one ``cudaMalloc`` block per rank whose CUDA-IPC handle is exchanged
once over the EP process group; every rank then holds a table of ``world`` base pointers per
region and kernels store straight into a peer's memory over NVLink.
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Optional

import torch
import torch.distributed as dist

from .. import _native as N


# Routing tables of one metadata launch that a saved dict carries to the backward.
PLAN_FIELDS = (
    "send_token_indices", "send_route_indices", "send_bucket", "route_to_send",
    "metadata_send_bucket_starts", "metadata_send_bucket_dst_starts", "metadata_local_stats",
    "metadata_stats", "metadata_recv_expert_offs", "metadata_recv_counts_re",
    "metadata_recv_per_expert", "mtile_group", "mtile_row0", "num_mtiles", "row_src_rank",
    "row_src_pos", "metadata_count_row", "disp_order_prefix", "mtile2_group", "mtile2_row0",
    "num_mtiles2", "row_arrival", "arrival_row",
)


def carve_plan(arena: torch.Tensor, layout) -> dict:
    """Views of the plan tables inside an int32 arena laid out by ``layout``."""
    return {name: arena[off:off + numel].view(shape) for name, off, numel, shape in layout}


def next_power_of_2(n: int) -> int:
    return 1 if n <= 1 else 1 << (n - 1).bit_length()


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


class SymmetricBlock:
    """One same-sized device allocation per rank, mapped into every rank's address space.

    ``regions`` maps a name to a byte size; each region starts at a 256-byte aligned offset
    that is identical on all ranks.  ``local(name, dtype)`` is a torch view of this rank's
    region, ``peer_table(name)`` a device int64 tensor of ``world`` base pointers.
    """

    def __init__(self, regions: dict[str, int], rank: int, world_size: int, group, device):
        self.rank = rank
        self.world_size = world_size
        self.device = device
        self.offsets: dict[str, int] = {}
        self.sizes: dict[str, int] = {}
        off = 0
        for name, size in regions.items():
            self.offsets[name] = off
            self.sizes[name] = size
            off += _align(max(size, 16))
        self.nbytes = off
        lib = N.lib()
        base = C.c_void_p()
        handle = C.create_string_buffer(64)
        N.check(lib.mm_symm_alloc(self.nbytes, C.byref(base), handle), "mm_symm_alloc")
        self.base = base.value
        self.peer_bases = [0] * world_size
        self.peer_bases[rank] = self.base
        self._opened: list[int] = []
        if world_size > 1:
            handles: list = [None] * world_size
            dist.all_gather_object(handles, handle.raw, group=group)
            for r, h in enumerate(handles):
                if r == rank:
                    continue
                p = C.c_void_p()
                N.check(lib.mm_symm_open(h, C.byref(p)), f"mm_symm_open(rank {r})")
                self.peer_bases[r] = p.value
                self._opened.append(p.value)
        self._tables: dict[str, torch.Tensor] = {}

    def local(self, name: str, dtype: torch.dtype) -> torch.Tensor:
        return N.tensor_from_ptr(self.base + self.offsets[name], self.sizes[name], dtype,
                                 self.device)

    def peer_table(self, name: str) -> torch.Tensor:
        if name not in self._tables:
            ptrs = [b + self.offsets[name] for b in self.peer_bases]
            self._tables[name] = torch.tensor(ptrs, dtype=torch.int64, device=self.device)
        return self._tables[name]

    def free(self):
        lib = N.lib()
        for p in self._opened:
            lib.mm_symm_close(p)
        self._opened = []
        if self.base:
            lib.mm_symm_free(self.base)
            self.base = 0


@dataclass
class MoEForwardContext:
    """Single-in-flight symmetric buffers and reusable routing workspaces.

    Field names follow the reference context (runtime/workspace.py:11-59); the ``combine_*``,
    ``send_*``, ``mtile_*`` and ``row_src_*`` members are workspaces of the CUDA pipeline.
    A routing plan must be consumed before the next plan is built because the metadata
    tensors are reused in place.
    """

    hidden_size: int
    num_experts: int
    experts_per_rank: int
    replica_budget: int
    physical_experts_per_rank: int
    world_size: int
    rank: int
    receive_capacity_factor: float
    max_source_tiles: int
    top_k: int = 0
    max_tokens_per_rank: int = 0
    max_received_routes: int = 0

    symm: Optional[SymmetricBlock] = None
    peer_mem: Optional[torch.Tensor] = None
    routing_weight_mem: Optional[torch.Tensor] = None
    signal_mem: Optional[torch.Tensor] = None
    combine_mem: Optional[torch.Tensor] = None
    combine_gate_mem: Optional[torch.Tensor] = None
    row_token_indices: Optional[torch.Tensor] = None
    row_route_indices: Optional[torch.Tensor] = None
    metadata_counts_mem: Optional[torch.Tensor] = None
    metadata_num_bins: int = 0
    metadata_send_bucket_starts: Optional[torch.Tensor] = None
    metadata_send_bucket_dst_starts: Optional[torch.Tensor] = None
    metadata_recv_counts_re: Optional[torch.Tensor] = None
    metadata_recv_seg_starts: Optional[torch.Tensor] = None
    metadata_recv_per_expert: Optional[torch.Tensor] = None
    metadata_recv_expert_offs: Optional[torch.Tensor] = None
    metadata_stats: Optional[torch.Tensor] = None
    metadata_pull_dst_start: Optional[torch.Tensor] = None
    metadata_local_stats: Optional[torch.Tensor] = None
    metadata_count_row: Optional[torch.Tensor] = None
    send_token_indices: Optional[torch.Tensor] = None
    send_route_indices: Optional[torch.Tensor] = None
    send_bucket: Optional[torch.Tensor] = None
    route_to_send: Optional[torch.Tensor] = None
    route_scratch: Optional[torch.Tensor] = None
    mtile_group: Optional[torch.Tensor] = None
    mtile_row0: Optional[torch.Tensor] = None
    num_mtiles: Optional[torch.Tensor] = None
    mtile2_group: Optional[torch.Tensor] = None
    mtile2_row0: Optional[torch.Tensor] = None
    num_mtiles2: Optional[torch.Tensor] = None
    row_src_rank: Optional[torch.Tensor] = None
    row_src_pos: Optional[torch.Tensor] = None
    status: Optional[torch.Tensor] = None
    dispatch_flags: Optional[torch.Tensor] = None
    peer_grad_mem: Optional[torch.Tensor] = None
    recv_weights_bf16: Optional[torch.Tensor] = None
    row_arrival: Optional[torch.Tensor] = None
    arrival_row: Optional[torch.Tensor] = None
    plan_arena: Optional[torch.Tensor] = None
    plan_layout: Optional[list] = None
    redispatch_mem: Optional[torch.Tensor] = None
    disp_order_prefix: Optional[torch.Tensor] = None
    disp_bucket_done: Optional[torch.Tensor] = None
    count_cubes: Optional[torch.Tensor] = None
    count_flags: Optional[torch.Tensor] = None
    count_epoch: int = 0
    dispatch_epoch: int = 0
    barrier_epoch: int = 0
    ep_group: object = None
    _extra: dict = field(default_factory=dict)

    # ---- device helpers -------------------------------------------------------------
    def _barrier(self, phase: int) -> None:
        N.check(N.lib().mm_rank_barrier(
            self.symm.peer_table("flags").data_ptr(), self.rank, self.world_size,
            self.barrier_epoch, phase, self.status.data_ptr(), N.stream_ptr()), "mm_rank_barrier")
        N.count_launches(1)

    def _next_epoch(self) -> None:
        self.barrier_epoch += 1
        if self.barrier_epoch >= 2**31 - 1:
            raise RuntimeError("barrier epoch exhausted; recreate the operator")

    def rank_barrier(self) -> None:
        """All ranks' earlier stores into this rank's symmetric memory are visible after it."""
        if self.world_size == 1:
            return
        self._next_epoch()
        self._barrier(0)

    def rank_signal(self) -> None:
        """First half of a barrier: announce that this rank's earlier stores are done."""
        if self.world_size == 1:
            return
        self._next_epoch()
        self._barrier(1)

    def rank_wait(self) -> None:
        """Second half: wait until every rank has announced the epoch of `rank_signal`."""
        if self.world_size == 1:
            return
        self._barrier(2)

    def next_dispatch_epoch(self) -> int:
        """Epoch of the next fused dispatch; arrival flags only ever grow."""
        self.dispatch_epoch += 1
        if self.dispatch_epoch >= 2**31 - 1:
            raise RuntimeError("dispatch epoch exhausted; recreate the operator")
        return self.dispatch_epoch

    def read_status(self) -> N.StatusRecord:
        rec = N.StatusRecord()
        N.check(N.lib().mm_status_read(self.status.data_ptr(), C.byref(rec), N.stream_ptr()),
                "mm_status_read")
        return rec

    def reset_status(self) -> None:
        N.check(N.lib().mm_status_reset(self.status.data_ptr(), N.stream_ptr()),
                "mm_status_reset")

    def finalize(self):
        """Release the symmetric allocation and drop ordinary workspaces."""
        if self.symm is not None:
            torch.cuda.synchronize()
            unregister_context(self)
            self.symm.free()
            self.symm = None
        for name in list(self.__dataclass_fields__):
            if isinstance(getattr(self, name), torch.Tensor):
                setattr(self, name, None)


# peer_mem data pointer -> context, so that moe_backward_triton(saved, dy, peer_mem) can find
# the symmetric workspaces that belong to the buffer it was handed.
_CONTEXTS: dict[int, MoEForwardContext] = {}


def register_context(ctx: MoEForwardContext) -> None:
    _CONTEXTS[ctx.peer_mem.data_ptr()] = ctx


def unregister_context(ctx: MoEForwardContext) -> None:
    if ctx.peer_mem is not None:
        _CONTEXTS.pop(ctx.peer_mem.data_ptr(), None)


def context_of(peer_mem: torch.Tensor) -> MoEForwardContext:
    ctx = _CONTEXTS.get(peer_mem.data_ptr())
    if ctx is None:
        raise ValueError(
            "peer_mem is not the symmetric receive buffer of a live MoE operator context")
    return ctx


def saved_recompute_enabled() -> bool:
    """``MOE_SAVED_RECOMPUTE=1`` (reference: ops/backward.py:135): the backward re-dispatches the
    forward's input rows and recomputes the weighted activation instead of reading the saved
    ``recv_hidden_sorted`` / ``swiglu_out_weighted``.  Read when the operator is constructed
    (the symmetric re-dispatch slab is part of its allocation) and by every backward call."""
    import os
    return os.environ.get("MOE_SAVED_RECOMPUTE", "0") == "1"


def create_moe_forward_context(
    *,
    max_tokens_per_rank: int,
    hidden_size: int,
    top_k: int,
    num_experts: int,
    rank: int,
    world_size: int,
    receive_capacity_factor: float,
    dispatch_fc1_block_size_m: int,
    single_kernel_dispatch_block_size_m: Optional[int] = None,
    enable_moonep: bool = False,
    ep_group=None,
    device=None,
) -> MoEForwardContext:
    """Allocate the symmetric block and the metadata tables (reference lines 105-314).

    Sizes follow the reference: ``max_received_routes = int(max_tokens * top_k * factor)``
    rows of ``hidden_size`` bf16 in ``peer_mem``, one fp32 routing weight per row, a
    ``[world, next_pow2(world * epr)]`` int32 count cube.  The symmetric block also holds the
    combine buffer (``max_tokens * top_k`` rows returned by FC2 or by the FC1 input
    gradient), a bf16 gate-gradient channel and the barrier flag words.
    """
    if type(enable_moonep) is not bool:
        raise TypeError("enable_moonep must be a bool")
    if enable_moonep:
        raise NotImplementedError("MoonEP is not implemented in the B200 build")
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    experts_per_rank = num_experts // world_size
    max_received_routes = int(max_tokens_per_rank * top_k * receive_capacity_factor)
    if max_received_routes >= torch.iinfo(torch.int32).max:
        raise ValueError("dispatch receive offsets exceed int32 range")
    source_tile_m = dispatch_fc1_block_size_m
    if single_kernel_dispatch_block_size_m is not None:
        source_tile_m = min(source_tile_m, single_kernel_dispatch_block_size_m)
    num_routes = max_tokens_per_rank * top_k
    max_source_tiles = (num_routes + source_tile_m - 1) // source_tile_m
    ctx = MoEForwardContext(
        hidden_size=hidden_size,
        num_experts=num_experts,
        experts_per_rank=experts_per_rank,
        replica_budget=0,
        physical_experts_per_rank=experts_per_rank,
        world_size=world_size,
        rank=rank,
        receive_capacity_factor=receive_capacity_factor,
        max_source_tiles=max_source_tiles,
        top_k=top_k,
        max_tokens_per_rank=max_tokens_per_rank,
        max_received_routes=max_received_routes,
        ep_group=ep_group,
    )
    regions = {
        "flags": 4096,
        "peer_mem": max_received_routes * hidden_size * 2,
        # receive buffer of the backward's dy rows: the forward's rows stay readable in
        # peer_mem until the next forward, so the FC1 weight gradient needs no copy of them
        "peer_grad_mem": max_received_routes * hidden_size * 2,
        "routing_weight_mem": max_received_routes * 4,
        "combine_mem": num_routes * hidden_size * 2,
        "combine_gate_mem": num_routes * 2,
        "dispatch_flags": world_size * experts_per_rank * 4,
        # two count cubes [world, bins] used alternately, and one epoch flag per source rank
        "count_cubes": 2 * world_size * next_power_of_2(world_size * experts_per_rank) * 4,
        "count_flags": world_size * 4,
    }
    if saved_recompute_enabled():
        # re-dispatch slab of the recompute backward (reference: kernels/mega_bwd.py:2962-3030):
        # the forward's input rows are pushed again into it instead of being saved
        regions["redispatch_mem"] = max_received_routes * hidden_size * 2
    ctx.symm = SymmetricBlock(regions, rank, world_size, ep_group, device)
    ctx.peer_mem = ctx.symm.local("peer_mem", torch.bfloat16)
    ctx.routing_weight_mem = ctx.symm.local("routing_weight_mem", torch.float32)
    ctx.signal_mem = ctx.symm.local("flags", torch.int32)
    ctx.combine_mem = ctx.symm.local("combine_mem", torch.bfloat16).view(num_routes, hidden_size)
    ctx.combine_gate_mem = ctx.symm.local("combine_gate_mem", torch.bfloat16)
    ctx.dispatch_flags = ctx.symm.local("dispatch_flags", torch.int32)
    ctx.peer_grad_mem = ctx.symm.local("peer_grad_mem", torch.bfloat16)
    ctx.redispatch_mem = (ctx.symm.local("redispatch_mem", torch.bfloat16)
                          if "redispatch_mem" in regions else None)

    num_buckets = world_size * experts_per_rank
    bins = next_power_of_2(num_buckets)
    ctx.metadata_num_bins = bins
    i32 = dict(dtype=torch.int32, device=device)
    ctx.count_cubes = ctx.symm.local("count_cubes", torch.int32).view(2, world_size * bins)
    ctx.count_flags = ctx.symm.local("count_flags", torch.int32)
    ctx.metadata_counts_mem = ctx.count_cubes[0]
    ctx.metadata_recv_seg_starts = torch.empty((experts_per_rank, world_size + 1), **i32)
    ctx.metadata_pull_dst_start = torch.empty(experts_per_rank * world_size, **i32)
    ctx.row_token_indices = torch.arange(num_routes, **i32) // top_k
    ctx.row_route_indices = torch.arange(num_routes, **i32)
    scratch_bytes = N.lib().mm_route_scratch_bytes(num_routes, bins)
    ctx.route_scratch = torch.empty(max(scratch_bytes, 16), dtype=torch.uint8, device=device)
    max_tiles = max_received_routes // 128 + experts_per_rank + 1
    max_tiles2 = max_received_routes // 256 + experts_per_rank + 1
    cap_rows = max(max_received_routes, 1)
    # Every table a saved dict has to keep (PLAN_FIELDS) is a slice of one int32 arena, so a
    # snapshot of the plan is a single device copy.
    shapes = {
        "send_token_indices": (num_routes,), "send_route_indices": (num_routes,),
        "send_bucket": (num_routes,), "route_to_send": (num_routes,),
        "metadata_send_bucket_starts": (num_buckets,),
        "metadata_send_bucket_dst_starts": (num_buckets,),
        "metadata_local_stats": (2,), "metadata_stats": (2 + world_size,),
        "metadata_recv_expert_offs": (experts_per_rank + 1,),
        "metadata_recv_counts_re": (world_size, experts_per_rank),
        "metadata_recv_per_expert": (experts_per_rank,),
        "mtile_group": (max_tiles,), "mtile_row0": (max_tiles,), "num_mtiles": (1,),
        "row_src_rank": (cap_rows,), "row_src_pos": (cap_rows,),
        "metadata_count_row": (bins,), "disp_order_prefix": (num_buckets + 1,),
        "mtile2_group": (max_tiles2,), "mtile2_row0": (max_tiles2,), "num_mtiles2": (1,),
        "row_arrival": (cap_rows,), "arrival_row": (cap_rows,),
    }
    assert tuple(shapes) == PLAN_FIELDS
    layout, off = [], 0
    for name in PLAN_FIELDS:
        numel = 1
        for d in shapes[name]:
            numel *= d
        layout.append((name, off, numel, shapes[name]))
        off += (numel + 3) // 4 * 4            # 16-byte aligned tables
    ctx.plan_arena = torch.zeros(max(off, 4), **i32)
    ctx.plan_layout = layout
    for name, view in carve_plan(ctx.plan_arena, layout).items():
        setattr(ctx, name, view)
    ctx.route_to_send.fill_(-1)
    ctx.status = torch.zeros(8, **i32)
    ctx.disp_bucket_done = torch.zeros(num_buckets, **i32)
    ctx.recv_weights_bf16 = torch.zeros(cap_rows, dtype=torch.bfloat16, device=device)
    register_context(ctx)
    return ctx


__all__ = ["MoEForwardContext", "SymmetricBlock", "create_moe_forward_context", "context_of"]
