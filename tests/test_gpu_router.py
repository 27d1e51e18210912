"""GPU parity of the router kernel (top-k + softmax over the selected logits) with the oracle:
expert ids bit-exact (ties included), weights within fp32 rounding of the softmax; and the
layer driven from logits end to end."""
import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("tokens,experts,top_k", [(1, 8, 1), (77, 8, 2), (512, 128, 8),
                                                  (8192, 896, 16), (33, 1024, 32), (5, 40, 40 - 8)])
def test_router_topk_matches_oracle(tokens, experts, top_k):
    import mega_moe
    g = torch.Generator().manual_seed(tokens + experts)
    logits = torch.randn(tokens, experts, generator=g)
    want_sel, want_w = O.router_topk(logits, top_k)
    sel, w = mega_moe.router_topk(logits.to(DEV), top_k)
    assert sel.dtype == torch.int32 and w.dtype == torch.float32
    assert torch.equal(sel.cpu(), want_sel)
    torch.testing.assert_close(w.cpu(), want_w, rtol=1e-5, atol=1e-7)
    torch.testing.assert_close(w.sum(-1).cpu(), torch.ones(tokens), rtol=1e-5, atol=1e-6)


def test_router_ties_go_to_the_lower_expert_and_strides_are_honoured():
    import mega_moe
    logits = torch.zeros(9, 70)
    logits[:, 11] = 2.0
    logits[:, 43] = 2.0
    logits[:, 5] = 1.0
    want_sel, want_w = O.router_topk(logits, 4)
    wide = torch.full((9, 96), 100.0)          # padded rows: the columns past 70 must be ignored
    wide[:, :70] = logits
    sel, w = mega_moe.router_topk(wide.to(DEV)[:, :70], 4)
    assert sel[0].tolist() == [11, 43, 5, 0]
    assert torch.equal(sel.cpu(), want_sel)
    torch.testing.assert_close(w.cpu(), want_w, rtol=1e-5, atol=1e-7)


def test_router_masked_and_nan_logits_follow_a_stable_descending_sort():
    """Rows with fewer than k finite logits (masked experts) still select k distinct real experts,
    -inf ties in expert order; a NaN logit ranks first, as in torch.sort / torch.topk."""
    import mega_moe
    g = torch.Generator().manual_seed(5)
    logits = torch.randn(6, 40, generator=g)
    logits[0, 3:] = float("-inf")              # 3 finite logits, k = 6
    logits[1, :] = float("-inf")               # nothing finite
    logits[2, 17] = float("nan")
    logits[3, 5] = float("inf")
    logits[3, 9] = float("-inf")
    logits[4, 0] = 0.0
    logits[4, 1] = -0.0                        # equal: expert 0 before expert 1
    logits[4, 2:] = -1.0
    want_sel, want_w = O.router_topk(logits, 6)
    sel, w = mega_moe.router_topk(logits.to(DEV), 6)
    assert torch.equal(sel.cpu(), want_sel)
    assert sel[0].tolist()[3:] == [3, 4, 5] and sel[1].tolist() == [0, 1, 2, 3, 4, 5]
    assert int(sel[2, 0]) == 17 and sel[4].tolist()[:2] == [0, 1]
    assert int(sel.min()) >= 0 and int(sel.max()) < 40
    torch.testing.assert_close(w.cpu(), want_w, rtol=1e-5, atol=1e-7, equal_nan=True)
    assert torch.isnan(w[1]).all() and torch.isnan(w[2]).all()      # softmax arithmetic
    torch.testing.assert_close(w[0, :3].sum().cpu(), torch.tensor(1.0), rtol=1e-5, atol=1e-6)


def test_router_validation():
    import mega_moe
    x = torch.randn(4, 16, device=DEV)
    with pytest.raises(TypeError):
        mega_moe.router_topk(x.to(torch.bfloat16), 2)
    with pytest.raises(ValueError):
        mega_moe.router_topk(x, 0)
    with pytest.raises(ValueError):
        mega_moe.router_topk(x, 17)
    with pytest.raises(ValueError):
        mega_moe.router_topk(x[0], 2)
    with pytest.raises(RuntimeError):
        mega_moe.router_topk(torch.randn(2, 2048, device=DEV), 2)   # more than 1024 experts
    sel, w = mega_moe.router_topk(torch.empty(0, 16, device=DEV), 2)
    assert sel.shape == (0, 2) and w.shape == (0, 2)


def test_layer_from_logits_matches_oracle():
    import mega_moe
    from test_gpu_operator import _check_out, _make_op
    tokens, hidden, ffn, experts, top_k = 256, 256, 128, 16, 4
    inp = O.make_inputs(1, tokens, hidden, ffn, experts, top_k, seed=21, weight_std=0.05)
    logits = torch.randn(tokens, experts, generator=torch.Generator().manual_seed(4))
    sel, w = O.router_topk(logits, top_k)
    want = O.forward_golden(inp["hidden"], [w], [sel], inp["w_gate"], inp["w_up"], inp["w_down"],
                            experts)[0]
    op = _make_op(tokens, hidden, top_k, experts)
    try:
        gsel, gw = mega_moe.router_topk(logits.to(DEV), top_k)
        gate_up = mega_moe.pack_gate_up_weights(inp["w_gate"][0].to(DEV), inp["w_up"][0].to(DEV))
        out = op(inp["hidden"][0].to(DEV), gsel, gate_up, inp["w_down"][0].to(DEV), gw)
        _check_out(out, want)
    finally:
        op.finalize()


def test_one_operator_shared_by_two_layers():
    """A host framework may share one operator between same-shape layers: the saved dict of a
    forward is a full snapshot, so the backward of the first layer still works after the second
    layer's forward ran on the same operator (reference: ops/function.py:152-158)."""
    import mega_moe
    from test_gpu_operator import _check_grad, _make_op
    tokens, hidden, ffn, experts, top_k = 192, 256, 128, 8, 2
    layers = [O.make_inputs(1, tokens, hidden, ffn, experts, top_k, seed=31 + i, weight_std=0.05)
              for i in range(2)]
    op = _make_op(tokens, hidden, top_k, experts)
    try:
        saved = []
        for inp in layers:
            gate_up = mega_moe.pack_gate_up_weights(inp["w_gate"][0].to(DEV), inp["w_up"][0].to(DEV))
            _, s = op(inp["hidden"][0].to(DEV), inp["selected"][0].to(DEV), gate_up,
                      inp["w_down"][0].to(DEV), inp["routing_weights"][0].to(DEV),
                      return_saved=True)
            saved.append(s)
        for inp, s in reversed(list(zip(layers, saved))):
            _, gold_saved = O.forward_saved(inp["hidden"], inp["routing_weights"], inp["selected"],
                                            inp["w_gate"], inp["w_up"], inp["w_down"], top_k)
            want = O.backward(gold_saved, inp["dy"])[0]
            got = mega_moe.moe_backward_triton(s, inp["dy"][0].to(DEV), op.context.peer_mem)
            for k in ("grad_hidden", "grad_routing_weights", "grad_fc1_1", "grad_fc1_2", "grad_fc2"):
                _check_grad(k, got[k], want[k])
    finally:
        op.finalize()
