"""BF16 post-routing MoE forward on B200 (API of the reference's ``ops/forward.py``).

The public boundary starts with selected experts and FP32 routing weights; router matmul,
softmax and top-k selection are outside it (reference: src/mega_moe/ops/forward.py:1-6).

Pipeline of one ``forward`` call, all on the caller's CUDA stream and without host
synchronisation unless ``return_saved`` or a reduced receive capacity asks for one:

    routing metadata (CUDA kernels + one NCCL all-gather of the count row)
    -> dispatch: rows pushed by P2P stores into the owning rank's receive buffer
    -> rank barrier (flag words in symmetric memory)
    -> FC1 grouped GEMM (tcgen05) with bf16 rounding + weighted gated activation fused
    -> FC2 grouped GEMM whose epilogue stores each row into the source rank's combine buffer
    -> rank barrier -> top-k gather-sum
"""

from __future__ import annotations

import os
import types
import weakref
from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.distributed

from ..config import MoEForwardConfig
from ..runtime.routing import (
    MoERoutingPlan,
    build_routing_plan,
    check_receive_capacity,
    launch_routing_metadata,
)
from ..runtime.workspace import carve_plan, create_moe_forward_context
from .. import _native as N
from . import _launch as L


@dataclass
class DispatchFC1Result:
    """Outputs and route identity produced by the dispatch plus FC1 stage."""

    routing_plan: MoERoutingPlan
    fc1_output: torch.Tensor
    dispatched_tokens: torch.Tensor
    received_routing_weights: torch.Tensor
    send_route_indices: torch.Tensor


def snapshot_plan(context, copy: bool = True) -> types.SimpleNamespace:
    """The routing tables of the last metadata launch as one object.

    All tables are slices of one int32 arena (a few MB), so a snapshot is a single device
    copy; ``copy=False`` returns views of the live tables (valid until the next metadata
    launch on the operator).
    """
    arena = context.plan_arena.clone() if copy else context.plan_arena
    return types.SimpleNamespace(**carve_plan(arena, context.plan_layout))


class FusedMoEForward(torch.nn.Module):
    """Fused EP all-to-all + grouped GEMM MoE operator for B200.

    Same constructor, attributes and ``forward`` contract as the reference class
    (src/mega_moe/ops/forward.py:68-243,1884-2109).  Instances are single-in-flight and
    single-stream because their workspaces are reused; they are not thread-safe.
    """

    def __init__(
        self,
        ep_group: Optional[torch.distributed.ProcessGroup],
        *,
        max_tokens_per_rank: int,
        hidden_size: int,
        top_k: int,
        num_experts: int,
        config: Optional[MoEForwardConfig] = None,
    ):
        super().__init__()
        if max_tokens_per_rank <= 0:
            raise ValueError("max_tokens_per_rank must be positive")
        if hidden_size <= 0:
            raise ValueError("hidden_size must be positive")
        if top_k <= 0:
            raise ValueError("top_k must be positive")
        if num_experts <= 0:
            raise ValueError("num_experts must be positive")
        if config is not None and not isinstance(config, MoEForwardConfig):
            raise TypeError("config must be a MoEForwardConfig instance or None")

        self.ep_group = ep_group
        if ep_group is not None:
            self.rank = ep_group.rank()
            self.world_size = ep_group.size()
        elif torch.distributed.is_available() and torch.distributed.is_initialized():
            self.rank = torch.distributed.get_rank()
            self.world_size = torch.distributed.get_world_size()
        else:
            self.rank = 0
            self.world_size = 1
        if num_experts % self.world_size:
            raise ValueError("num_experts must be divisible by the EP world size")
        if hidden_size % 8:
            raise ValueError("hidden_size must be a multiple of 8 (16-byte rows)")

        self.max_tokens_per_rank = max_tokens_per_rank
        self.hidden_size = hidden_size
        self.top_k = top_k
        self.num_experts = num_experts
        self.experts_per_rank = num_experts // self.world_size
        self.activation_dtype = torch.bfloat16
        self.config = config if config is not None else MoEForwardConfig()
        self.enable_moonep = self.config.enable_moonep
        self.enable_single_kernel_forward = self.config.enable_single_kernel_forward
        self.replica_budget = 0
        self.physical_experts_per_rank = self.experts_per_rank
        self.receive_capacity_factor = self.config.resolved_receive_capacity_factor(
            self.world_size)
        self.num_aicore_programs = self.config.num_aicore_programs
        self.num_aivector_programs = self.config.num_aivector_programs
        self._save_fc1_dtype = self.config.save_fc1_dtype
        self.activation = self.config.activation
        self.situ_beta = self.config.situ_beta
        self.situ_linear_beta = self.config.situ_linear_beta
        self.clamp_limit = self.config.clamp_limit

        self._tile_signal_epoch = 1
        self._routing_owner_token = object()
        self._routing_generation = 0
        self.context = create_moe_forward_context(
            max_tokens_per_rank=max_tokens_per_rank,
            hidden_size=hidden_size,
            top_k=top_k,
            num_experts=num_experts,
            rank=self.rank,
            world_size=self.world_size,
            receive_capacity_factor=self.receive_capacity_factor,
            dispatch_fc1_block_size_m=self.config.dispatch_fc1_block_size_m,
            single_kernel_dispatch_block_size_m=(
                self.config.single_kernel_dispatch_block_size_m
                if self.enable_single_kernel_forward else None),
            enable_moonep=self.enable_moonep,
            ep_group=self.ep_group,
        )
        self.context._extra["operator"] = weakref.ref(self)
        self._route_to_send = self.context.route_to_send
        self._forward_stream = None
        self._act_buf = None
        self._fc1_buf = None
        self._routing_weights_keepalive = None
        self._fwd_timing_last = None
        # When True, the backward writes the expert-weight gradients into buffers that are
        # allocated once and handed out again every step (the caller must consume or
        # accumulate them before the next backward), like the fixed-address saved-activation
        # workspace of the reference (ops/forward.py:246-282).  Off by default.
        self.persistent_weight_grads = False
        self._grad_ws = None
        # When True, `forward` never waits for the device: the receive-capacity check is
        # deferred (an overflow raises ValueError from the next call, `sync()` or
        # `finalize()` instead of from the call that overflowed), and the saved dict carries
        # capacity-sized activation buffers with the row counts left on the device
        # (`saved["M"]`, `total_recv`, `total_send` are None).  The default (False) keeps the
        # reference's behaviour: immediate ValueError and exact-size saved tensors, at the
        # price of host synchronisations inside every call.
        self.host_sync_free = False
        # When True, `saved["fc1_output"]` / `saved["swiglu_out_weighted"]` are views of this
        # operator's fixed buffers instead of copies (valid until its next forward), like the
        # reference's fixed-address saved workspace (ops/forward.py:246-282).
        self.saved_views = False
        self._pending_check = []
        self._host_stats_ring = [torch.zeros(2, dtype=torch.int32).pin_memory() for _ in range(8)]
        self._host_stats_next = 0

        # All ranks must observe zeroed symmetric buffers before first use.
        torch.cuda.synchronize()
        if self.world_size > 1:
            torch.distributed.barrier(group=self.ep_group)

    def _fc1_scale_group(self, ffn: int) -> int:
        """Columns per fp8 scale of a saved FC1 row: half the FC1 tile width of the
        configuration, as in the reference (ops/forward.py:612-613)."""
        group = self.config.fc1_gemm_block_size_n // 2
        if group <= 0 or (2 * ffn) % group or group % 2:
            raise ValueError(f"save_fc1_dtype='fp8' needs fc1_gemm_block_size_n // 2 (= {group}) "
                             f"to divide 2 * ffn (= {2 * ffn})")
        return group

    # ===================== buffer management =====================
    def _ensure_activation_buffers(self, ffn: int, need_fc1: bool):
        cap = max(self.context.max_received_routes, 1)
        dev = self.context.peer_mem.device
        if self._act_buf is None or self._act_buf.shape[1] != ffn:
            self._act_buf = torch.empty(cap, ffn, dtype=torch.bfloat16, device=dev)
            self._fc1_buf = None
        if need_fc1 and self._fc1_buf is None:
            self._fc1_buf = torch.empty(cap, 2 * ffn, dtype=torch.bfloat16, device=dev)

    def _get_grad_workspace(self, ffn: int):
        if self._grad_ws is None or self._grad_ws["grad_fc2"].shape[2] != ffn:
            dev = self.context.peer_mem.device
            self._grad_ws = {
                "grad_fc1": torch.empty(self.experts_per_rank, 2 * ffn, self.hidden_size,
                                        dtype=torch.bfloat16, device=dev),
                "grad_fc2": torch.empty(self.experts_per_rank, self.hidden_size, ffn,
                                        dtype=torch.bfloat16, device=dev),
            }
        return self._grad_ws

    def _check_pending_capacity(self, wait: bool) -> None:
        """Raise the deferred receive-capacity error of an earlier sync-free forward."""
        while self._pending_check:
            host_stats, event = self._pending_check[0]
            if wait:
                event.synchronize()
            elif not event.query():
                return
            self._pending_check.pop(0)
            required = int(host_stats[1])
            if (self.receive_capacity_factor < self.world_size
                    and required > self.context.max_received_routes):
                self._pending_check.clear()
                self.context.reset_status()
                raise ValueError(
                    f"peer buffer capacity {self.context.max_received_routes} routes is "
                    f"smaller than the required receive size {required}")

    def _defer_capacity_check(self) -> None:
        """Queue an asynchronous copy of {M, max required rows} for a later host-side check."""
        if len(self._pending_check) >= len(self._host_stats_ring):
            self._check_pending_capacity(wait=True)
        slot = self._host_stats_ring[self._host_stats_next % len(self._host_stats_ring)]
        self._host_stats_next += 1
        slot.copy_(self.context.metadata_stats[:2], non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        self._pending_check.append((slot, event))

    def sync(self):
        torch.cuda.synchronize()
        self._check_pending_capacity(wait=True)

    def finalize(self):
        """Drain the device, then release the symmetric block and all workspaces."""
        if self.context.peer_mem is not None:
            torch.cuda.synchronize(self.context.peer_mem.device)
        self._pending_check = []
        if self.world_size > 1 and self.context.symm is not None:
            torch.distributed.barrier(group=self.ep_group)
        self._act_buf = None
        self._fc1_buf = None
        self._grad_ws = None
        self._route_to_send = None
        self._forward_stream = None
        self._routing_weights_keepalive = None
        self.context.finalize()

    def read_last_forward_phase_timing(self):
        """Device time of each phase of the last forward, recorded under ``MOE_FWD_TIMING=1``
        (the reference's switch, ops/forward.py:1555-1570; there the products are SYS_CNT
        ticks per Ascend core, here CUDA-event times on the caller's stream).

        Returns ``{"phase_ms": {phase: ms}, "total_ms": ms, "acc": {...}, "acc_slots": (...)}``
        with the phases ``routing_metadata``, ``dispatch_fc1_activation`` (dispatch, FC1 and
        the weighted activation are one launch, or a chain without gaps), ``fc2_combine``,
        ``rank_barrier`` and ``topk_reduce``.  ``acc`` is the counterpart of the reference's
        issue-stream busy ticks: when the instrumented library is built
        (``python mega-moe-td_b200/build.py --profile``) and the switch was set before the
        first call into the library, every grouped-GEMM launch since the forward began
        (backward launches included) has an int64 ``[160, 16]`` device tensor of SM clocks per
        CTA and warp role, columns named by ``acc_slots``; otherwise ``acc`` is empty.  Waits
        for the last stamp.  Raises ``RuntimeError`` when no forward has run with the switch set.
        """
        if self._fwd_timing_last is None:
            raise RuntimeError("no forward has run on this operator with MOE_FWD_TIMING=1")
        phases = self._fwd_timing_last.phase_ms()
        return {"phase_ms": phases, "total_ms": sum(phases.values()),
                "acc": dict(N.role_counters), "acc_slots": N.ROLE_COUNTER_SLOTS}

    # ===================== validation =====================
    def _validate_topk_indices(self, selected_experts: torch.Tensor):
        if selected_experts.ndim != 2:
            raise ValueError(
                "selected_experts must have shape [tokens, top_k], got "
                f"{tuple(selected_experts.shape)}")
        if selected_experts.shape[1] != self.top_k:
            raise ValueError(
                f"selected_experts must have top_k={self.top_k}, got shape "
                f"{tuple(selected_experts.shape)}")
        if selected_experts.dtype != torch.int32:
            raise TypeError(
                f"selected_experts must use torch.int32, got {selected_experts.dtype}")
        if selected_experts.device != self.context.peer_mem.device:
            raise ValueError("selected_experts must be on the operator's CUDA device")
        if not selected_experts.is_contiguous():
            raise ValueError("selected_experts must be contiguous")
        if selected_experts.shape[0] > self.max_tokens_per_rank:
            raise ValueError(
                f"input has {selected_experts.shape[0]} tokens, exceeding "
                f"max_tokens_per_rank={self.max_tokens_per_rank}")

    def _validate_dispatch_inputs(self, hidden_states, selected_experts):
        self._validate_topk_indices(selected_experts)
        if hidden_states.ndim != 2:
            raise ValueError(
                f"hidden_states must have shape [tokens, hidden], got {tuple(hidden_states.shape)}")
        expected_shape = (selected_experts.shape[0], self.hidden_size)
        if hidden_states.shape != expected_shape:
            raise ValueError(
                f"hidden_states must have shape {expected_shape}, got {tuple(hidden_states.shape)}")
        if hidden_states.dtype != self.activation_dtype:
            raise TypeError(
                f"hidden_states must use {self.activation_dtype}, got {hidden_states.dtype}")
        if hidden_states.device != selected_experts.device:
            raise ValueError("hidden_states and selected_experts must be on the same device")
        if not hidden_states.is_contiguous():
            raise ValueError("hidden_states must be contiguous")

    def _validate_gate_up_weight(self, gate_up_weight, device):
        if gate_up_weight.ndim != 3:
            raise ValueError("gate_up_weight must have shape [experts_per_rank, hidden, 2F]")
        if gate_up_weight.shape[0] != self.experts_per_rank:
            raise ValueError(
                f"gate_up_weight has {gate_up_weight.shape[0]} local experts, "
                f"expected {self.experts_per_rank}")
        if gate_up_weight.shape[1] != self.hidden_size:
            raise ValueError(
                "gate_up_weight must use [experts_per_rank, hidden, 2F] layout "
                f"with hidden_size={self.hidden_size}, got {tuple(gate_up_weight.shape)}")
        packed_output_size = gate_up_weight.shape[2]
        if packed_output_size <= 0 or packed_output_size % 2:
            raise ValueError("gate_up_weight output dimension must be a positive even value (2F)")
        if gate_up_weight.dtype != self.activation_dtype:
            raise TypeError(
                f"gate_up_weight must use {self.activation_dtype}, got {gate_up_weight.dtype}")
        if gate_up_weight.device != device:
            raise ValueError("gate_up_weight and hidden_states must be on the same device")
        if not gate_up_weight.is_contiguous():
            raise ValueError("gate_up_weight must be contiguous and pre-packed before forward")

    def _check_stream(self, device):
        current_stream = torch.cuda.current_stream(device)
        if self._forward_stream is None:
            self._forward_stream = current_stream
        elif self._forward_stream != current_stream:
            raise RuntimeError(
                "FusedMoEForward is single-stream; recreate the operator for "
                "a different caller stream")

    # ===================== routing metadata =========================
    def build_routing_plan(self, selected_experts: torch.Tensor, *,
                           moonep_plan_hook: Optional[Callable] = None) -> MoERoutingPlan:
        """Build stable dispatch/count metadata for one set of selected experts."""
        self._validate_topk_indices(selected_experts)
        self._routing_generation += 1
        generation = self._routing_generation
        plan = build_routing_plan(self.context, selected_experts)
        plan.owner_token = self._routing_owner_token
        plan.generation = generation
        plan.selected_experts_version = selected_experts._version
        return plan

    # ===================== dispatch + FC1 ===========================
    def dispatch_fc1(
        self,
        hidden_states: torch.Tensor,
        selected_experts: torch.Tensor,
        routing_plan: MoERoutingPlan,
        fc1_weight: torch.Tensor,
        fc1_output: Optional[torch.Tensor] = None,
        *,
        routing_weights: torch.Tensor,
        final_barrier: bool = True,
        **_moonep_unused,
    ) -> DispatchFC1Result:
        """Dispatch routes and run the local experts' FC1 (no activation).

        ``fc1_weight`` uses the contiguous ``[expert, K, N]`` layout (reference:
        ops/forward.py:928-1320); ``fc1_output`` is ``[num_received_routes, N]`` bf16.
        """
        self._validate_dispatch_inputs(hidden_states, selected_experts)
        if routing_plan.selected_experts is not selected_experts:
            raise ValueError("routing_plan must be built from this exact selected_experts tensor")
        if (routing_plan.owner_token is not self._routing_owner_token
                or routing_plan.generation != self._routing_generation):
            raise RuntimeError("routing plan belongs to another or superseded operator")
        if routing_plan.num_input_tokens != hidden_states.shape[0]:
            raise ValueError("routing plan token count does not match hidden_states")
        if fc1_weight.ndim != 3:
            raise ValueError("fc1_weight must be a 3D local-expert weight tensor")
        if fc1_weight.shape[0] != self.experts_per_rank:
            raise ValueError(
                f"fc1_weight has {fc1_weight.shape[0]} local experts, "
                f"expected {self.experts_per_rank}")
        if fc1_weight.shape[1] != self.hidden_size:
            raise ValueError("fc1_weight must use [expert, hidden, N] layout")
        if fc1_weight.dtype != self.activation_dtype:
            raise TypeError(f"fc1_weight must use {self.activation_dtype}")
        if (routing_weights.shape != selected_experts.shape
                or routing_weights.dtype != torch.float32
                or not routing_weights.is_contiguous()):
            raise ValueError(
                "routing_weights must be contiguous FP32 with the same shape as selected_experts")
        ctx = self.context
        m = routing_plan.num_received_routes
        n_out = fc1_weight.shape[2]
        if fc1_output is None:
            fc1_output = torch.empty(m, n_out, dtype=self.activation_dtype,
                                     device=hidden_states.device)
        elif fc1_output.shape != (m, n_out) or fc1_output.dtype != self.activation_dtype:
            raise ValueError(f"fc1_output must be BF16 with shape {(m, n_out)}")
        # dispatch runs inside the GEMM launch (it must run even when this rank receives
        # nothing: its rows are someone else's input)
        recv = ctx.peer_mem.view(ctx.max_received_routes, self.hidden_size)
        desc = L.make_desc(ctx, recv, ctx.max_received_routes, self.hidden_size, fc1_weight,
                           k_dim=1, n_dim=2, n_out=n_out, k_extent=self.hidden_size)
        if L.fused_dispatch_enabled(ctx):
            disp = L.make_dispatch_desc(ctx, hidden_states, routing_weights)
        else:
            disp = None
            L.dispatch_rows(ctx, hidden_states, routing_weights, selected_experts.numel())
            ctx.rank_barrier()
        out_buf = fc1_output if m > 0 else torch.empty(
            1, n_out, dtype=self.activation_dtype, device=hidden_states.device)
        L.grouped_gemm(desc, out_buf, dispatch=disp)
        if final_barrier:
            ctx.rank_barrier()
        recv_rows = ctx.peer_mem.view(ctx.max_received_routes, self.hidden_size)[:m]
        return DispatchFC1Result(
            routing_plan=routing_plan,
            fc1_output=fc1_output,
            dispatched_tokens=recv_rows,
            received_routing_weights=ctx.routing_weight_mem[:m],
            send_route_indices=routing_plan.send_route_indices,
        )

    # ===================== full forward ================================
    def forward(
        self,
        hidden_states: torch.Tensor,
        selected_experts: torch.Tensor,
        gate_up_weight: torch.Tensor,
        down_weight: torch.Tensor,
        routing_weights: torch.Tensor,
        *,
        return_saved: bool = False,
    ):
        """Run the complete BF16 post-routing MoE forward.

        Shapes: ``hidden_states [T, H]`` bf16, ``selected_experts [T, k]`` int32,
        ``gate_up_weight [EPR, H, 2F]`` bf16 (gate columns first), ``down_weight [EPR, H, F]``
        bf16 (contiguous or a transposed view of ``[EPR, F, H]``), ``routing_weights [T, k]``
        fp32.  Returns ``out [T, H]`` bf16, or ``(out, saved)`` with the intermediates the
        five-stage backward consumes.
        """
        self._validate_dispatch_inputs(hidden_states, selected_experts)
        self._validate_gate_up_weight(gate_up_weight, hidden_states.device)
        self._check_stream(hidden_states.device)
        if (routing_weights.shape != selected_experts.shape
                or routing_weights.dtype != torch.float32
                or routing_weights.device != hidden_states.device
                or not routing_weights.is_contiguous()):
            raise ValueError(
                "routing_weights must be contiguous FP32 with the same shape "
                "and device as selected_experts")
        ffn_size = gate_up_weight.shape[2] // 2
        expected_down_shape = (self.experts_per_rank, self.hidden_size, ffn_size)
        if (down_weight.ndim != 3
                or tuple(down_weight.shape) != expected_down_shape
                or down_weight.dtype != self.activation_dtype
                or down_weight.device != hidden_states.device):
            raise ValueError(
                "down_weight must be BF16 with shape "
                f"{expected_down_shape} on the input device (a strided "
                "natural-layout [E, F, H] view flows through unstaged)")
        if (gate_up_weight.shape[2] % self.config.fc1_gemm_block_size_n
                or self.hidden_size % self.config.fc1_gemm_block_size_k
                or self.hidden_size % self.config.fc2_gemm_block_size_n
                or ffn_size % self.config.fc2_gemm_block_size_k):
            raise ValueError("configured FC1/FC2 N and K tiles must divide the weight dimensions")
        if ffn_size % 128:
            raise ValueError("expert FFN size must be a multiple of 128")

        ctx = self.context
        self._check_pending_capacity(wait=False)
        tokens = hidden_states.shape[0]
        num_routes = tokens * self.top_k
        hidden = self.hidden_size
        cap = ctx.max_received_routes
        # Skinny tiles run FC1 in two steps (plain GEMM into the raw gate|up buffer, then the
        # activation pass), so they need the raw buffer even when nothing is saved.
        two_step_fc1 = L.gemm_tile_mode(ctx) == L.TILE_SKINNY
        self._ensure_activation_buffers(ffn_size, need_fc1=return_saved or two_step_fc1)
        out = torch.empty(tokens, hidden, dtype=self.activation_dtype, device=hidden_states.device)
        stamps = _PhaseStamps() if N.forward_timing_enabled() else None
        if stamps:
            N.role_counters.clear()

        launch_routing_metadata(ctx, selected_experts)
        if stamps:
            stamps.mark("routing_metadata")
        self._routing_generation += 1
        self._routing_weights_keepalive = routing_weights
        # Dispatch is fused into the FC1 launch: extra warps push the rows while the GEMM
        # consumes each expert as soon as every source has flagged it complete.
        recv = ctx.peer_mem.view(cap, hidden)
        fc1_desc = L.make_desc(ctx, recv, cap, hidden, gate_up_weight, k_dim=1, n_dim=2,
                               n_out=ffn_size, k_extent=hidden)
        if L.fused_dispatch_enabled(ctx):
            disp = L.make_dispatch_desc(ctx, hidden_states, routing_weights)
        else:
            disp = None
            L.dispatch_rows(ctx, hidden_states, routing_weights, num_routes)
            ctx.rank_barrier()
        # The received routing weights live in symmetric memory that the next forward's
        # dispatch rewrites; FC1 leaves the bf16 copy the backward reads in a private buffer.
        L.fc1_swiglu(ctx, fc1_desc, self._act_buf,
                     self._fc1_buf if (return_saved or two_step_fc1) else None,
                     ctx.routing_weight_mem, self.activation, self.situ_beta,
                     self.situ_linear_beta, self.clamp_limit, dispatch=disp,
                     weight_bf16_out=ctx.recv_weights_bf16 if return_saved else None)
        if stamps:
            stamps.mark("dispatch_fc1_activation")
        fc2_desc = L.make_desc(ctx, self._act_buf, cap, ffn_size, down_weight, k_dim=2, n_dim=1,
                               n_out=hidden, k_extent=ffn_size)
        L.grouped_gemm_scatter(ctx, fc2_desc, "combine_mem", hidden, name="fc2_combine")
        if stamps:
            stamps.mark("fc2_combine")
        ctx.rank_barrier()
        if stamps:
            stamps.mark("rank_barrier")
        L.topk_reduce(ctx.combine_mem, ctx.route_to_send, tokens, self.top_k, hidden, out)
        if stamps:
            stamps.mark("topk_reduce")
            self._fwd_timing_last = stamps
        if self.host_sync_free:
            self._defer_capacity_check()
        else:
            check_receive_capacity(ctx)
        if not return_saved:
            return out

        if self.host_sync_free:
            num_received_routes = num_sent_routes = None
            m = cap
            sent = num_routes
        else:
            num_received_routes = int(ctx.metadata_stats[0].item())
            num_sent_routes = int(ctx.metadata_local_stats[0].item())
            m = num_received_routes
            sent = num_sent_routes
            if num_sent_routes != num_routes:
                # reference: ops/_single_saved_adapter.py:116-121
                raise ValueError(
                    "droless routing required for the single-kernel backward "
                    f"contract: {num_sent_routes} routes kept of {num_routes} — raise "
                    "receive_capacity_factor to >= world_size")
        # With saved_views the saved tensors are views of this operator's buffers, valid until
        # its next forward: the backward's dy rows land in a second receive region, so the
        # forward's received rows stay in place.  Otherwise every saved tensor is a copy and a
        # later forward on the same operator does not disturb it (reference: clone-out at
        # ops/forward.py:2074-2080 and the full-snapshot marker of the saved adapter).
        views = self.saved_views
        keep = (lambda t: t) if views else (lambda t: t.clone())
        plan = snapshot_plan(ctx, copy=not views)
        save_fmt = self.config.save_fc1_dtype
        fc1_scale = None
        if save_fmt == "bf16":
            fc1_output = keep(self._fc1_buf[:m])
        else:
            # Saved-format pass (reference: quantise leg of the FC1 epilogue,
            # kernels/fused_forward.py:877-949): the raw bf16 rows stay in the operator's
            # workspace, the saved tensor is the fp16 copy or fp8 E4M3 + per-group scales.
            dt = torch.float16 if save_fmt == "fp16" else torch.float8_e4m3fn
            fc1_output = torch.empty(m, 2 * ffn_size, dtype=dt, device=out.device)
            if save_fmt == "fp8":
                fc1_scale = torch.empty(m, 2 * ffn_size // self._fc1_scale_group(ffn_size),
                                        dtype=torch.float32, device=out.device)
            if m > 0:
                L.fc1_save_convert(self._fc1_buf, ctx.metadata_stats, m, save_fmt,
                                   self._fc1_scale_group(ffn_size), fc1_output, fc1_scale)
        saved = {
            # minimal contract of the reference's single-launch forward
            # (ops/forward.py:1813-1873)
            "fc1_output": fc1_output,
            "recv_weights_sorted": keep(ctx.recv_weights_bf16[:m]),
            "hidden_states": hidden_states,
            "selected_experts": selected_experts,
            "routing_weights": routing_weights,
            "recv_expert_offsets": plan.metadata_recv_expert_offs,
            "recv_counts_by_source_expert": plan.metadata_recv_counts_re,
            "send_token_indices": plan.send_token_indices[:sent],
            "send_route_indices": plan.send_route_indices[:sent],
            "total_send": num_sent_routes,
            "total_recv": num_received_routes,
            "M": num_received_routes,
            "_routing_generation": self._routing_generation,
            "_owner_token": id(self._routing_owner_token),
            "_single_kernel_snapshot": not views,
            "_saved_views": views,
            # activation section and scalars of the full backward contract
            # (ops/_torch_forward.py:294-320)
            "recv_hidden_sorted": keep(recv[:m]),
            "swiglu_out_weighted": keep(self._act_buf[:m]),
            "gate": fc1_output[:, :ffn_size],
            "up": fc1_output[:, ffn_size:],
            "expert_counts": plan.metadata_recv_per_expert,
            "split_size_cum_per_expert": plan.metadata_recv_expert_offs,
            "batch_size": tokens, "hidden_dim": hidden, "ffn_dim": ffn_size,
            "num_experts": self.num_experts, "experts_per_rank": self.experts_per_rank,
            "topk": self.top_k, "world_size": self.world_size, "ep_rank": self.rank,
            "ep_group": self.ep_group,
            "activation": self.activation, "situ_beta": self.situ_beta,
            "situ_linear_beta": self.situ_linear_beta, "clamp_limit": self.clamp_limit,
            # weight references: [E, 2F, H] / [E, F, H] views of the packed table
            "fc1_combined": gate_up_weight.transpose(1, 2),
            "fc1_1": gate_up_weight[:, :, :ffn_size].transpose(1, 2),
            "fc1_2": gate_up_weight[:, :, ffn_size:].transpose(1, 2),
            "fc2": down_weight,
            "output": out, "dy": None,
            "_plan": plan,
        }
        saved.update(self._saved_index_section(plan, m, sent, num_received_routes is not None))
        if fc1_scale is not None:
            saved["fc1_output_scale"] = fc1_scale
            saved["fc1_scale_group_size"] = self._fc1_scale_group(ffn_size)
        if self.persistent_weight_grads:
            saved["_grad_workspace"] = self._get_grad_workspace(ffn_size)
        return out, saved

    def _saved_index_section(self, plan, m: int, sent: int, host_values: bool) -> dict:
        """Index keys of the saved contract after the reference's enrichment
        (ops/_single_saved_adapter.py:247-340), all from the routing tables of this forward.

        ``sort_idxs`` is the forward's own send order and ``inv_sort`` its inverse
        (= ``route_to_send`` for dropless routes); ``local_sort_idxs`` / ``inv_local`` map
        between the receive order (expert-major, then source) and the source-major arrival
        order of an all-to-all (written by the metadata kernel).  The per-rank split lists and
        the 64-row tile tables of the reference's grouped GEMMs need host values, so they are
        ``None`` in ``host_sync_free`` mode (``host_values`` False).
        """
        out = {
            "forward_send_route": plan.send_route_indices[:sent],
            "sort_idxs": plan.send_route_indices[:sent],
            "inv_sort": plan.route_to_send[:sent],
            "local_sort_idxs": plan.row_arrival[:m],
            "inv_local": plan.arrival_row[:m],
        }
        keys = ("splits_send_list", "splits_recv_list", "num_tiles_total", "meta_expert_ids",
                "meta_split_cum", "meta_tile_num", "meta_tile_num_cum")
        if not host_values:
            out.update({k: None for k in keys})
            return out
        counts = plan.metadata_recv_counts_re.cpu().to(torch.int64)          # [W, EPR]
        send_row = plan.metadata_count_row[:self.num_experts].cpu().to(torch.int64)
        out["splits_send_list"] = send_row.view(self.world_size, -1).sum(1).tolist()
        out["splits_recv_list"] = counts.sum(1).tolist()
        per_expert = counts.sum(0)
        tile_rows = 64                       # BLOCK_SIZE_M of the reference's metadata builder
        tiles = (per_expert + tile_rows - 1) // tile_rows
        row_starts = per_expert.cumsum(0) - per_expert
        tile_starts = tiles.cumsum(0) - tiles
        total = int(tiles.sum())
        dev = plan.metadata_recv_counts_re.device
        i32 = lambda t: t.to(torch.int32).to(dev)
        out["num_tiles_total"] = i32(torch.tensor([total]))
        out["meta_expert_ids"] = i32(torch.repeat_interleave(torch.arange(tiles.numel()), tiles))
        out["meta_split_cum"] = i32(torch.repeat_interleave(row_starts, tiles))
        out["meta_tile_num_cum"] = i32(torch.repeat_interleave(tile_starts, tiles))
        out["meta_tile_num"] = i32(torch.arange(total) - torch.repeat_interleave(tile_starts, tiles))
        return out


class _PhaseStamps:
    """CUDA events at the phase boundaries of one forward (``MOE_FWD_TIMING=1``)."""

    def __init__(self):
        self.names = []
        self.events = [self._now()]

    @staticmethod
    def _now():
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        return ev

    def mark(self, name: str) -> None:
        self.names.append(name)
        self.events.append(self._now())

    def phase_ms(self) -> dict:
        self.events[-1].synchronize()
        return {n: self.events[i].elapsed_time(self.events[i + 1])
                for i, n in enumerate(self.names)}


def pack_gate_up_weights(gate_weight_local: torch.Tensor,
                         up_weight_local: torch.Tensor) -> torch.Tensor:
    """Pack local BF16 gate/up projections as contiguous ``[E, H, 2F]``."""
    if gate_weight_local.ndim != 3 or up_weight_local.ndim != 3:
        raise ValueError(
            "gate and up weights must have shape [experts_per_rank, ffn_size, hidden_size]")
    if gate_weight_local.shape != up_weight_local.shape:
        raise ValueError(
            "gate and up weight shapes must match, got "
            f"{gate_weight_local.shape} and {up_weight_local.shape}")
    if gate_weight_local.dtype != torch.bfloat16 or up_weight_local.dtype != torch.bfloat16:
        raise TypeError("gate and up weights must both use torch.bfloat16")
    if gate_weight_local.device != up_weight_local.device:
        raise ValueError("gate and up weights must be on the same device")
    return torch.cat(
        (gate_weight_local.transpose(1, 2), up_weight_local.transpose(1, 2)), dim=2
    ).contiguous()
