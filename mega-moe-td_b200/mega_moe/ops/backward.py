"""Five-stage MoE backward on B200 (API of the reference's ``ops/backward.py``).

Given ``dy [T, H]`` the stages are the reference's (src/mega_moe/ops/backward.py:27-34):

1. dispatch ``dy`` rows to the expert ranks (same routes as the forward) and compute the
   FC2 input gradient ``grad_swiglu = recv_dy @ fc2[e]``;
2. gated-activation backward -> ``grad_fc1_output``, ``grad_gate``;
3. FC2 weight gradient ``grad_fc2[e] = recv_dy^T @ swiglu_out_weighted``;
4. FC1 input gradient, each row stored straight into the source rank's combine buffer
   together with its gate gradient, then the top-k gather-sum -> ``grad_hidden``,
   ``grad_routing_weights``;
5. FC1 weight gradient ``grad_fc1[e] = grad_fc1_output^T @ recv_hidden_sorted``.

All GEMMs run on the tcgen05 grouped-GEMM kernel; the name ``moe_backward_triton`` is kept
only because callers import it.  ``MOE_BWD_MEGA=1`` (reference: ops/backward.py:100-224, one
launch for all stages on Ascend) is accepted and selects this same chain of launches on one
stream: on this hardware the stages already run back to back without host synchronisation,
and the results are identical by construction.

Execution order on the stream (the numbering above is the reference's): 1, 2, 4 (GEMM +
stores to the source ranks), 5, barrier signal, 3, barrier wait, gather-sum of 4.  The dy
rows are received in a second symmetric region (``peer_grad_mem``), so the forward's received
rows in ``peer_mem`` stay readable until the next forward; stage 5 reads them and therefore
runs before this rank signals (a peer that has seen every signal may start its next forward
and overwrite them), while stage 3 reads only the dy rows, which no peer rewrites before the
next backward, and absorbs the ranks' skew between the two halves of the barrier.
"""

from __future__ import annotations

import torch

from ..runtime.routing import launch_routing_metadata
from ..runtime.workspace import context_of, saved_recompute_enabled
from . import _launch as L
from .forward import snapshot_plan


def _plan_for(saved, ctx):
    """Routing tables for ``saved``: the forward's snapshot, or a rebuild from the experts.

    A saved dict produced by the Torch functional forward carries no device routing tables;
    they are a pure function of ``selected_experts``, so they are rebuilt here.
    """
    plan = saved.get("_plan")
    if plan is not None:
        return plan
    selected = saved["selected_experts"]
    if selected.dtype != torch.int32:
        selected = selected.to(torch.int32)
    selected = selected.contiguous()
    launch_routing_metadata(ctx, selected)
    plan = snapshot_plan(ctx)
    saved["_plan"] = plan
    return plan


def moe_backward_triton(saved, dy, peer_mem, grad_transport=None, hidden_states=None):
    """Run the five backward stages; returns the reference's dict of gradients.

    ``saved`` is either the dict returned by ``FusedMoEForward.forward(return_saved=True)``
    or the 39-key dict of the Torch functional forward (``ops/_torch_forward.py:294-320`` of
    the reference).  ``peer_mem`` must be the symmetric receive buffer of a live operator
    context; it is reused as the receive buffer of the ``dy`` dispatch.
    """
    if grad_transport is not None:
        raise ValueError("grad_transport requires a MoonEP saved_phys, which is not implemented")
    recompute = saved_recompute_enabled()
    recv_hidden_sorted = saved.get("recv_hidden_sorted")
    if recompute:
        # reference: ops/backward.py:135-145, kernels/mega_bwd.py:3211-3230
        if hidden_states is None:
            hidden_states = saved.get("hidden_states")
        if hidden_states is None:
            raise ValueError("MOE_SAVED_RECOMPUTE=1 needs the forward input hidden_states "
                             "(saved['hidden_states'] or the hidden_states argument)")
    else:
        if recv_hidden_sorted is None:
            raise ValueError(
                "saved is missing recv_hidden_sorted; the fused backward requires "
                "the activation section (replay saved or return_saved=True)")
        if (recv_hidden_sorted.data_ptr() == peer_mem.data_ptr()
                and not saved.get("_saved_views")):
            raise ValueError(
                "saved['recv_hidden_sorted'] aliases peer_mem; the receive buffer "
                "is single-in-flight and was overwritten after dispatch")
    ctx = context_of(peer_mem)
    if recompute and ctx.redispatch_mem is None:
        raise RuntimeError("MOE_SAVED_RECOMPUTE=1 must be set before the operator is constructed: "
                           "its symmetric allocation holds the re-dispatch slab")
    dtype = saved["fc1_1"].dtype
    dy = dy.to(dtype).contiguous()
    tokens, hidden = dy.shape
    top_k = int(saved["topk"])
    fc1_output = saved["fc1_output"]
    m = fc1_output.shape[0]
    ffn = fc1_output.shape[1] // 2
    epr = int(saved["experts_per_rank"])
    fc1_combined = saved["fc1_combined"]   # [E, 2F, H]
    fc2 = saved["fc2"]                      # [E, H, F]
    device = dy.device
    plan = _plan_for(saved, ctx)
    cap = ctx.max_received_routes
    num_routes = tokens * top_k
    group_offs = plan.metadata_recv_expert_offs
    tiles = dict(plan=plan)

    fc1_scale = saved.get("fc1_output_scale")
    scale_group = saved.get("fc1_scale_group_size") or 0
    activation = saved.get("activation", "swiglu") or "swiglu"
    act_args = (activation, saved.get("situ_beta"), saved.get("situ_linear_beta"),
                saved.get("clamp_limit"))

    if recompute:
        # Re-dispatch the forward's input rows into the slab (same maps as the forward
        # dispatch, so the rows land in the receive layout the FC1 weight gradient expects);
        # the barrier of stage 1 publishes them together with the dy rows.
        L.dispatch_rows(ctx, hidden_states.to(dtype).contiguous(), None, num_routes, plan=plan,
                        region="redispatch_mem")
        recv_hidden_sorted = ctx.redispatch_mem.view(cap, hidden)[:m]

    # ---- stage 1: dispatch dy + FC2 input gradient ------------------------------------
    # The dy dispatch is fused into the GEMM launch (it runs even when this rank received
    # nothing, because its rows are other ranks' input).
    recv_dy = ctx.peer_grad_mem.view(cap, hidden)
    grad_swiglu = torch.empty(max(m, 1), ffn, dtype=dtype, device=device)[:m]
    desc = L.make_desc(ctx, recv_dy, cap, hidden, fc2, k_dim=1, n_dim=2, n_out=ffn,
                       k_extent=hidden, **tiles)
    if L.fused_dispatch_enabled(ctx) and not recompute:
        disp = L.make_dispatch_desc(ctx, dy, None, plan=plan, region="peer_grad_mem")
    else:
        disp = None
        L.dispatch_rows(ctx, dy, None, num_routes, plan=plan, region="peer_grad_mem")
        ctx.rank_barrier()
    L.grouped_gemm(desc, grad_swiglu if m > 0 else grad_swiglu.new_empty(1, ffn),
                   name="fc2_dgrad", dispatch=disp)
    grad_fc2_out_sorted = recv_dy[:m]

    # ---- stage 2: gated-activation backward (+ gate gradient pushed to the source) -----
    grad_fc1_output = torch.empty(m, 2 * ffn, dtype=dtype, device=device)
    grad_gate = torch.empty(m, dtype=dtype, device=device)
    if m > 0:
        L.swiglu_bwd(ctx, grad_swiglu, fc1_output, saved["recv_weights_sorted"], ffn,
                     plan.metadata_stats, m, grad_fc1_output, grad_gate, *act_args, plan=plan,
                     fc1_scale=fc1_scale, scale_group=scale_group)

    # ---- stage 4: FC1 input gradient -> source ranks ------------------------------------
    if m > 0:
        desc = L.make_desc(ctx, grad_fc1_output, m, 2 * ffn, fc1_combined, k_dim=1, n_dim=2,
                           n_out=hidden, k_extent=2 * ffn, **tiles)
        L.grouped_gemm_scatter(ctx, desc, "combine_mem", hidden, plan=plan, name="fc1_dgrad_combine")

    # ---- stage 5: FC1 weight gradient (reads the forward's received rows, which a peer may
    #      overwrite once it has seen this rank's signal) ---------------------------------
    grad_ws = saved.get("_grad_workspace")
    if m > 0:
        grad_fc1 = (grad_ws["grad_fc1"] if grad_ws is not None
                    else torch.empty(epr, 2 * ffn, hidden, dtype=dtype, device=device))
        L.grouped_wgrad(ctx, grad_fc1_output, recv_hidden_sorted, m, group_offs, epr, grad_fc1,
                        name="fc1_wgrad")
    else:
        grad_fc1 = torch.zeros(epr, 2 * ffn, hidden, dtype=dtype, device=device)

    # Peers may read what this rank stored as soon as it has signalled.
    ctx.rank_signal()

    # ---- stage 3: FC2 weight gradient, between the two halves of the barrier ------------
    if recompute:
        # weighted activation rows from the saved FC1 rows and the saved bf16 routing weights
        act = torch.empty(max(m, 1), ffn, dtype=dtype, device=device)[:m]
        if m > 0:
            L.swiglu_recompute(fc1_output, saved["recv_weights_sorted"], ffn, plan.metadata_stats,
                               m, act, *act_args, fc1_scale=fc1_scale, scale_group=scale_group)
    else:
        act = saved["swiglu_out_weighted"]
    if m > 0:
        grad_fc2 = (grad_ws["grad_fc2"] if grad_ws is not None
                    else torch.empty(epr, hidden, ffn, dtype=dtype, device=device))
        L.grouped_wgrad(ctx, recv_dy, act, m, group_offs, epr, grad_fc2, name="fc2_wgrad")
    else:
        grad_fc2 = torch.zeros(epr, hidden, ffn, dtype=dtype, device=device)

    ctx.rank_wait()
    grad_hidden = torch.empty(tokens, hidden, dtype=dtype, device=device)
    grad_routing_weights = torch.empty(tokens, top_k, dtype=dtype, device=device)
    # the same values as fp32 for the autograd wrappers (routing weights are fp32 inputs)
    grad_routing_weights_f32 = torch.empty(tokens, top_k, dtype=torch.float32, device=device)
    L.topk_reduce(ctx.combine_mem, plan.route_to_send, tokens, top_k, hidden, grad_hidden,
                  gate_in=ctx.combine_gate_mem, gate_out=grad_routing_weights,
                  gate_out_f32=grad_routing_weights_f32)

    grad_fc1_1, grad_fc1_2 = torch.chunk(grad_fc1, 2, dim=1)
    return dict(
        grad_hidden=grad_hidden, grad_routing_weights=grad_routing_weights,
        grad_fc1_1=grad_fc1_1, grad_fc1_2=grad_fc1_2, grad_fc2=grad_fc2,
        grad_swiglu=grad_swiglu, grad_fc1_output=grad_fc1_output, grad_gate=grad_gate,
        grad_fc2_out_sorted=grad_fc2_out_sorted, grad_fc1=grad_fc1,
        _grad_routing_weights_f32=grad_routing_weights_f32,
    )


class MegaMoEBackwardFunction(torch.autograd.Function):
    """EP-MoE whose forward is this package's fused operator and whose backward is the
    five-stage CUDA backward.

    Signature of the reference class (ops/backward.py:405-455):
    ``apply(hidden_states, routing_weights, selected_experts, fc1_1, fc1_2, fc2, ep_group,
    topk, peer_mem)`` with ``fc1_1`` / ``fc1_2`` ``[E_local, F, H]`` and ``fc2``
    ``[E_local, H, F]``.  The reference runs a Torch functional forward here; this build has
    no Torch compute path, so the forward goes through the operator that owns ``peer_mem``.
    """

    @staticmethod
    def forward(ctx, hidden_states, routing_weights, selected_experts, fc1_1, fc1_2, fc2,
                ep_group, topk, peer_mem):
        from .forward import pack_gate_up_weights
        context = context_of(peer_mem)
        op_ref = context._extra.get("operator")
        op = op_ref() if op_ref is not None else None
        if op is None:
            raise ValueError("peer_mem does not belong to a live FusedMoEForward operator")
        with torch.no_grad():
            gate_up = pack_gate_up_weights(fc1_1, fc1_2)
            out, saved = op.forward(
                hidden_states, selected_experts.to(torch.int32).contiguous(), gate_up, fc2,
                routing_weights.float().contiguous(), return_saved=True)
        saved = dict(saved)
        saved["output"] = None   # see MegaMoEFunction.forward: avoids a node <-> output cycle
        ctx.saved = saved
        ctx.peer_mem = peer_mem
        ctx.rw_dtype = routing_weights.dtype
        return out

    @staticmethod
    def backward(ctx, dy):
        grads = moe_backward_triton(ctx.saved, dy, ctx.peer_mem)
        return (
            grads["grad_hidden"],
            (grads["_grad_routing_weights_f32"] if ctx.rw_dtype == torch.float32
             else grads["grad_routing_weights"].to(ctx.rw_dtype)),
            None,
            grads["grad_fc1_1"],
            grads["grad_fc1_2"],
            grads["grad_fc2"],
            None,
            None,
            None,
        )


__all__ = ["MegaMoEBackwardFunction", "moe_backward_triton"]
