"""CPU checks of the oracle's router: it must equal torch.topk + softmax (what the reference's
benchmark feeds the layer, benchmark/layer/bench_moe_suite.py:487-497) and break ties towards
the lower expert id."""
import torch
import torch.nn.functional as F

from oracle import moe_oracle as O


def test_router_equals_topk_softmax():
    g = torch.Generator().manual_seed(0)
    logits = torch.randn(300, 128, generator=g)
    sel, w = O.router_topk(logits, 8)
    top_vals, top_idx = torch.topk(logits, k=8, dim=-1)
    assert torch.equal(sel, top_idx.to(torch.int32))
    torch.testing.assert_close(w, F.softmax(top_vals, dim=-1), rtol=0, atol=0)
    assert sel.dtype == torch.int32 and w.dtype == torch.float32


def test_router_ties():
    logits = torch.zeros(3, 10)
    logits[:, 7] = 1.0
    logits[:, 2] = 1.0
    sel, w = O.router_topk(logits, 3)
    assert sel[0].tolist() == [2, 7, 0]
    torch.testing.assert_close(w.sum(-1), torch.ones(3))
