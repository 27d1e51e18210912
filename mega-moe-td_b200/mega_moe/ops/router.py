"""Router in front of the layer: top-k of the router logits and their softmax.

The reference keeps the router on the caller's side; its own benchmark and tests build the
layer's post-router inputs as ``topk(logits, k)`` followed by ``softmax(topk_logits)`` in fp32
(reference: benchmark/layer/bench_moe_suite.py:487-497).  ``router_topk`` does both in one
kernel and returns tensors in exactly the form ``FusedMoEForward.forward`` takes.
"""
from __future__ import annotations

import torch

from .. import _native as N


def router_topk(router_logits: torch.Tensor, top_k: int):
    """``selected_experts [T, k] int32`` (descending logits, ties to the lower expert id) and
    ``routing_weights [T, k] fp32`` = softmax over the selected logits."""
    if router_logits.dim() != 2:
        raise ValueError("router_logits must be [tokens, experts]")
    if router_logits.dtype != torch.float32:
        raise TypeError("router_logits must be FP32")
    if not router_logits.is_cuda:
        raise ValueError("router_logits must live on a CUDA device")
    if router_logits.stride(1) != 1:
        router_logits = router_logits.contiguous()
    tokens, experts = router_logits.shape
    if type(top_k) is not int or not 1 <= top_k <= min(experts, 32):
        raise ValueError("top_k must be an int in [1, min(experts, 32)]")
    selected = torch.empty(tokens, top_k, dtype=torch.int32, device=router_logits.device)
    weights = torch.empty(tokens, top_k, dtype=torch.float32, device=router_logits.device)
    if tokens == 0:
        return selected, weights
    N.check(N.lib().mm_router_topk(router_logits.data_ptr(), router_logits.stride(0), tokens,
                                   experts, top_k, selected.data_ptr(), weights.data_ptr(),
                                   N.stream_ptr()), "mm_router_topk")
    N.count_launches(1)
    return selected, weights
