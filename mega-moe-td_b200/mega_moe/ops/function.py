"""The autograd.Function layer of the MoE operator (reference: src/mega_moe/ops/function.py).

``MegaMoEFunction.forward`` runs :class:`FusedMoEForward` with ``return_saved=True`` so that
the backward's saved values are captured inside the fused pass; ``backward`` runs
:func:`moe_backward_triton` on that dict behind the same owner / generation gates as the
reference (function.py:135-151).
"""

import torch

from .backward import moe_backward_triton


class MegaMoEFunction(torch.autograd.Function):
    """One-pass fused EP-MoE whose backward runs on the native saved dict.

    ``apply(op, hidden_states, routing_weights, selected_experts, gate_up_weight,
    down_weight, peer_mem, state)``; gradients come back for ``hidden_states``,
    ``routing_weights``, ``gate_up_weight`` (packed ``[E, H, 2F]``) and ``down_weight``.
    ``peer_mem`` must be passed explicitly (``None`` raises ``ValueError``); ``state`` is a
    caller-owned namespace that receives ``signal_mem`` / ``epoch`` / ``mega_persistent``
    after the backward, like the reference writes them back (function.py:199-205).
    """

    @staticmethod
    def forward(ctx, op, hidden_states, routing_weights, selected_experts,
                gate_up_weight, down_weight, peer_mem, state):
        if peer_mem is None:
            raise ValueError(
                "peer_mem must be passed explicitly: the backward symmetric "
                "buffer cannot default to op.context.peer_mem")
        with torch.no_grad():
            output, saved = op.forward(
                hidden_states,
                selected_experts,
                gate_up_weight,
                down_weight,
                routing_weights,
                return_saved=True,
            )
        # The output tensor becomes the autograd node's own result: keeping it inside the
        # node's saved dict would close a reference cycle (node -> saved -> output -> node)
        # that only the cyclic garbage collector could free, pinning every step's activations.
        saved = dict(saved)
        saved["output"] = None
        ctx.op = op
        ctx.saved = saved
        ctx.peer_mem = peer_mem
        ctx.state = state
        ctx.hidden_states = hidden_states
        return output

    @staticmethod
    def backward(ctx, dy):
        op = ctx.op
        saved = ctx.saved
        if saved.get("_owner_token") != id(op._routing_owner_token):
            raise RuntimeError(
                "the saved dict belongs to another operator instance; run "
                "the forward and backward on the same operator")
        if (saved.get("_routing_generation") != op._routing_generation
                and not saved.get("_single_kernel_snapshot")):
            raise RuntimeError(
                "the saved dict belongs to a routing plan this operator "
                "has already superseded; run backward before the next "
                "forward on the operator")
        grads = moe_backward_triton(saved, dy, ctx.peer_mem,
                                    hidden_states=getattr(ctx, "hidden_states", None))
        if ctx.state is not None:
            ctx.state.signal_mem = op.context.signal_mem
            ctx.state.epoch = op.context.barrier_epoch
            ctx.state.mega_persistent = {}
        # The weight-gradient halves are [E, F, H]; merge back into the packed
        # [E, H, 2F] layout of the gate_up_weight input.
        grad_gate_up = grads["grad_fc1"].transpose(1, 2)
        return (
            None,
            grads["grad_hidden"],
            grads["_grad_routing_weights_f32"],
            None,
            grad_gate_up,
            grads["grad_fc2"],
            None,
            None,
        )
