"""GPU parity of the `mega_moe` operator (single rank) against the CPU oracle.

Tolerances are the reference's (tests/_numeric.py:24-34): layout exact, FC1 / activation
2e-2, full output 4e-2, gradients |d| <= 1e-2 + 2e-2 * max|gold|; plus cosine >= 0.9999.
"""
import types

import numpy as np
import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


# (name, MOE_GEMM_MODE, MOE_WGRAD_MODE, MOE_FUSED_DISPATCH): every operator test runs with the
# automatic choice of a single rank (transposed "skinny" tiles and the unit walk at these rows
# per expert, separate row-push kernel), with the 128-row single-CTA tiles, with CTA pairs, and
# with the dispatch warps fused into the GEMM launches -- the form every multi-GPU run uses
# (on one GPU all peer pointers are local, the arrival flags and the per-expert waits run
# unchanged).
MODES = [
    ("auto", "auto", "auto", None),
    ("single", "single", "single", "0"),
    ("pair", "pair", "pair", None),
    ("auto-fused", "auto", "auto", "1"),
    ("single-fused", "single", "single", "1"),
    ("pair-fused-unit", "pair", "unit", "1"),
]


@pytest.fixture(autouse=True, params=MODES, ids=[m[0] for m in MODES])
def tile_mode(request, monkeypatch):
    name, gemm, wgrad, fused = request.param
    monkeypatch.setenv("MOE_GEMM_MODE", gemm)
    monkeypatch.setenv("MOE_WGRAD_MODE", wgrad)
    if fused is None:
        monkeypatch.delenv("MOE_FUSED_DISPATCH", raising=False)
    else:
        monkeypatch.setenv("MOE_FUSED_DISPATCH", fused)
    return name


def _pow2_divisor(n, cap):
    d = 16
    while d * 2 <= cap and n % (d * 2) == 0:
        d *= 2
    return d


def _make_op(tokens, hidden, top_k, experts, ffn=None, **cfg):
    """Operator whose (reference-validated) tile fields divide the test's small dimensions."""
    import mega_moe
    cfg.setdefault("fc1_gemm_block_size_k", _pow2_divisor(hidden, 128))
    cfg.setdefault("fc2_gemm_block_size_n", _pow2_divisor(hidden, 256))
    config = mega_moe.MoEForwardConfig(**cfg)
    return mega_moe.FusedMoEForward(None, max_tokens_per_rank=tokens, hidden_size=hidden,
                                    top_k=top_k, num_experts=experts, config=config)


def _check_out(got, want):
    got = got.cpu()
    assert got.dtype == torch.bfloat16 and got.shape == want.shape
    assert torch.isfinite(got.float()).all()
    torch.testing.assert_close(got.float(), want.float(), rtol=O.OUTPUT_RTOL, atol=O.OUTPUT_ATOL)
    if want.float().abs().max() > 0:
        assert O.cosine(got, want) > O.MIN_COSINE


def _check_grad(name, got, want):
    ok, max_d, rel, n_bad = O.cmp_grad(got.cpu(), want)
    assert ok, f"{name}: max_abs={max_d:.3e} rel={rel:.3e} mismatches={n_bad}"
    if want.float().abs().max() > 0:
        assert O.cosine(got.cpu(), want) > O.MIN_COSINE, name


FWD_CASES = [
    # tokens, hidden, ffn, experts, top_k, drop, zipf
    (64, 128, 128, 8, 2, 0.0, None),
    (512, 256, 128, 8, 2, 0.0, None),          # the CPU-plumbing configuration, in bf16
    (300, 256, 384, 16, 4, 0.3, None),
    (1024, 512, 256, 32, 8, 0.0, 1.2),
    (130, 128, 128, 4, 3, 1.0, None),          # every route dropped -> zeros
    (512, 256, 128, 64, 4, 0.0, None),         # 64 buckets: the dispatch warps' bucket search
                                               # takes two 32-way steps
]


@pytest.mark.parametrize("tokens,hidden,ffn,experts,top_k,drop,zipf", FWD_CASES)
def test_forward_matches_oracle(tokens, hidden, ffn, experts, top_k, drop, zipf):
    import mega_moe
    bias = O.zipf_expert_bias(experts, zipf) if zipf else None
    inp = O.make_inputs(1, tokens, hidden, ffn, experts, top_k, seed=tokens, expert_bias=bias,
                        drop_frac=drop, weight_std=0.05)
    want = O.forward_golden(inp["hidden"], inp["routing_weights"], inp["selected"],
                            inp["w_gate"], inp["w_up"], inp["w_down"], experts)[0]
    op = _make_op(tokens, hidden, top_k, experts)
    try:
        gate_up = mega_moe.pack_gate_up_weights(inp["w_gate"][0].to(DEV), inp["w_up"][0].to(DEV))
        x, sel, rw = (inp[k][0].to(DEV) for k in ("hidden", "selected", "routing_weights"))
        out = op(x, sel, gate_up, inp["w_down"][0].to(DEV), rw)
        _check_out(out, want)
        # second call on the same operator, with the down weight as a transposed [E, F, H] view
        down_t = inp["w_down"][0].to(DEV).transpose(1, 2).contiguous().transpose(1, 2)
        assert not down_t.is_contiguous()
        out2 = op(x, sel, gate_up, down_t, rw)
        assert torch.equal(out2, out)
        assert op.context.read_status().code == 0
    finally:
        op.finalize()


def test_forward_matches_reference_fixture():
    """Same inputs as the reference run stored in tests/golden/w1_e8_k2.npz."""
    import mega_moe
    from conftest import Golden
    g = Golden("w1_e8_k2")
    op = _make_op(g.tokens, g.hidden, g.top_k, g.experts)
    try:
        gate_up = mega_moe.pack_gate_up_weights(g.get(0, "in_w_gate").to(DEV),
                                                g.get(0, "in_w_up").to(DEV))
        out = op(g.get(0, "in_hidden").to(DEV), g.get(0, "in_selected").to(DEV), gate_up,
                 g.get(0, "in_w_down").to(DEV), g.get(0, "in_routing_weights").to(DEV))
        _check_out(out, g.get(0, "fwd_golden"))
    finally:
        op.finalize()


@pytest.mark.parametrize("activation", ["clamp_swiglu", "situglu"])
def test_forward_other_activations(activation):
    import mega_moe
    tokens, hidden, ffn, experts, top_k = 256, 256, 256, 8, 2
    kw = dict(activation=activation, situ_beta=1.5, situ_linear_beta=2.0, clamp_limit=0.5)
    inp = O.make_inputs(1, tokens, hidden, ffn, experts, top_k, seed=9, weight_std=0.08)
    want = O.forward_golden(inp["hidden"], inp["routing_weights"], inp["selected"], inp["w_gate"],
                            inp["w_up"], inp["w_down"], experts, **kw)[0]
    op = _make_op(tokens, hidden, top_k, experts, **kw)
    try:
        gate_up = mega_moe.pack_gate_up_weights(inp["w_gate"][0].to(DEV), inp["w_up"][0].to(DEV))
        out = op(inp["hidden"][0].to(DEV), inp["selected"][0].to(DEV), gate_up,
                 inp["w_down"][0].to(DEV), inp["routing_weights"][0].to(DEV))
        _check_out(out, want)
    finally:
        op.finalize()


def test_routing_plan_and_dispatch_fc1_stage_api():
    """build_routing_plan + dispatch_fc1 vs the dispatch+FC1 golden (layout exact)."""
    tokens, hidden, ffn, experts, top_k = 200, 128, 256, 8, 3
    inp = O.make_inputs(1, tokens, hidden, ffn, experts, top_k, seed=4, drop_frac=0.3,
                        weight_std=0.1)
    w1 = torch.cat([inp["w_gate"][0], inp["w_up"][0]], dim=1)           # logical [E, N, H]
    fc1, eg, xg = O.dispatch_fc1_golden(inp["hidden"], inp["selected"], [w1], experts)[0]
    meta = O.routing_metadata([inp["selected"][0].numpy()], experts)[0]
    op = _make_op(tokens, hidden, top_k, experts)
    try:
        sel = inp["selected"][0].to(DEV)
        plan = op.build_routing_plan(sel)
        assert plan.num_received_routes == meta["num_received_routes"]
        assert plan.num_sent_routes == meta["num_sent_routes"]
        np.testing.assert_array_equal(plan.send_route_indices.cpu().numpy(),
                                      meta["send_route_indices"])
        np.testing.assert_array_equal(plan.send_token_indices.cpu().numpy(),
                                      meta["send_token_indices"])
        np.testing.assert_array_equal(plan.stable_sort_indices.cpu().numpy(),
                                      meta["stable_sort_indices"])
        np.testing.assert_array_equal(op._route_to_send[:tokens * top_k].cpu().numpy(),
                                      meta["route_to_send"])
        weight = w1.transpose(1, 2).contiguous().to(DEV)                # [E, K, N] model layout
        res = op.dispatch_fc1(inp["hidden"][0].to(DEV), sel, plan, weight,
                              routing_weights=torch.ones(tokens, top_k, device=DEV))
        kernel_exp = torch.repeat_interleave(torch.arange(experts, dtype=torch.int32),
                                             plan.received_routes_per_expert.cpu())
        assert torch.equal(kernel_exp, eg)
        assert torch.equal(res.dispatched_tokens.cpu(), xg)
        torch.testing.assert_close(res.fc1_output.cpu().float(), fc1.float(),
                                   rtol=O.APPROX_RTOL, atol=O.APPROX_ATOL)
    finally:
        op.finalize()


def _to_dev(saved):
    out = {}
    for k, v in saved.items():
        out[k] = v.to(DEV) if isinstance(v, torch.Tensor) else v
    return out


BWD_CASES = [(64, 128, 128, 8, 2, None), (512, 256, 128, 8, 2, None), (700, 256, 384, 16, 4, 1.2),
             (600, 128, 128, 64, 4, 1.2)]      # 64 buckets, some of them empty


@pytest.mark.parametrize("tokens,hidden,ffn,experts,top_k,zipf", BWD_CASES)
def test_backward_on_oracle_saved_dict(tokens, hidden, ffn, experts, top_k, zipf):
    """moe_backward_triton must accept the 39-key saved dict of the Torch functional forward."""
    import mega_moe
    bias = O.zipf_expert_bias(experts, zipf) if zipf else None
    inp = O.make_inputs(1, tokens, hidden, ffn, experts, top_k, seed=tokens + 1, expert_bias=bias,
                        weight_std=0.05)
    _, saved = O.forward_saved(inp["hidden"], inp["routing_weights"], inp["selected"],
                               inp["w_gate"], inp["w_up"], inp["w_down"], top_k)
    want = O.backward(saved, inp["dy"])[0]
    op = _make_op(tokens, hidden, top_k, experts)
    try:
        got = mega_moe.moe_backward_triton(_to_dev(saved[0]), inp["dy"][0].to(DEV),
                                           op.context.peer_mem)
        for k in ("grad_fc2_out_sorted", "grad_swiglu", "grad_fc1_output", "grad_gate",
                  "grad_hidden", "grad_routing_weights", "grad_fc1_1", "grad_fc1_2", "grad_fc2"):
            _check_grad(k, got[k], want[k])
        assert op.context.read_status().code == 0
    finally:
        op.finalize()


@pytest.mark.parametrize("tokens,hidden,ffn,experts,top_k,zipf", BWD_CASES)
def test_autograd_function_end_to_end(tokens, hidden, ffn, experts, top_k, zipf):
    """MegaMoEFunction: fused forward with native saved dict + five-stage backward."""
    import mega_moe
    bias = O.zipf_expert_bias(experts, zipf) if zipf else None
    inp = O.make_inputs(1, tokens, hidden, ffn, experts, top_k, seed=tokens + 2, expert_bias=bias,
                        weight_std=0.05)
    want_out = O.forward_golden(inp["hidden"], inp["routing_weights"], inp["selected"],
                                inp["w_gate"], inp["w_up"], inp["w_down"], experts)[0]
    _, saved = O.forward_saved(inp["hidden"], inp["routing_weights"], inp["selected"],
                               inp["w_gate"], inp["w_up"], inp["w_down"], top_k)
    want = O.backward(saved, inp["dy"])[0]
    op = _make_op(tokens, hidden, top_k, experts)
    try:
        x = inp["hidden"][0].to(DEV).requires_grad_(True)
        rw = inp["routing_weights"][0].to(DEV).requires_grad_(True)
        gate_up = mega_moe.pack_gate_up_weights(
            inp["w_gate"][0].to(DEV), inp["w_up"][0].to(DEV)).requires_grad_(True)
        down = inp["w_down"][0].to(DEV).requires_grad_(True)
        state = types.SimpleNamespace()
        out = mega_moe.MegaMoEFunction.apply(op, x, rw, inp["selected"][0].to(DEV), gate_up, down,
                                             op.context.peer_mem, state)
        _check_out(out.detach(), want_out)
        out.backward(inp["dy"][0].to(DEV))
        _check_grad("grad_hidden", x.grad, want["grad_hidden"])
        _check_grad("grad_routing_weights", rw.grad, want["grad_routing_weights"])
        _check_grad("grad_down", down.grad, want["grad_fc2"])
        want_gate_up = torch.cat((want["grad_fc1_1"], want["grad_fc1_2"]), dim=1).transpose(1, 2)
        _check_grad("grad_gate_up", gate_up.grad, want_gate_up)
        assert hasattr(state, "epoch")
        with pytest.raises(ValueError):
            mega_moe.MegaMoEFunction.apply(op, x, rw, inp["selected"][0].to(DEV), gate_up, down,
                                           None, None)
    finally:
        op.finalize()


def test_backward_matches_reference_fixture():
    import mega_moe
    from conftest import Golden
    g = Golden("w1_e8_k2")
    _, saved = O.forward_saved(g.per_rank("in_hidden"), g.per_rank("in_routing_weights"),
                               g.per_rank("sel_dropless"), g.per_rank("in_w_gate"),
                               g.per_rank("in_w_up"), g.per_rank("in_w_down"), g.top_k)
    op = _make_op(g.tokens, g.hidden, g.top_k, g.experts)
    try:
        got = mega_moe.moe_backward_triton(_to_dev(saved[0]), g.get(0, "in_dy").to(DEV),
                                           op.context.peer_mem)
        for k in ("grad_hidden", "grad_routing_weights", "grad_fc1_1", "grad_fc1_2", "grad_fc2"):
            _check_grad(k, got[k], g.get(0, "bwd_" + k))
    finally:
        op.finalize()


def test_validation_errors_and_capacity_overflow():
    import mega_moe
    tokens, hidden, ffn, experts, top_k = 64, 128, 128, 8, 2
    inp = O.make_inputs(1, tokens, hidden, ffn, experts, top_k, seed=3)
    op = _make_op(tokens, hidden, top_k, experts)
    try:
        gate_up = mega_moe.pack_gate_up_weights(inp["w_gate"][0].to(DEV), inp["w_up"][0].to(DEV))
        x, sel, rw = (inp[k][0].to(DEV) for k in ("hidden", "selected", "routing_weights"))
        down = inp["w_down"][0].to(DEV)
        with pytest.raises(TypeError):
            op(x.float(), sel, gate_up, down, rw)
        with pytest.raises(TypeError):
            op(x, sel.long(), gate_up, down, rw)
        with pytest.raises(ValueError):
            op(x[:, :64], sel, gate_up, down, rw)
        with pytest.raises(ValueError):
            op(x, sel, gate_up, down, rw.double())
        with pytest.raises(ValueError):
            op(x, sel, gate_up, down[:, :, :64], rw)
        with pytest.raises(ValueError):
            op(torch.cat([x, x]), torch.cat([sel, sel]), gate_up, down, rw)
        with torch.cuda.stream(torch.cuda.Stream()):
            pass
        out = op(x, sel, gate_up, down, rw)
        with pytest.raises(RuntimeError):
            with torch.cuda.stream(torch.cuda.Stream()):
                op(x, sel, gate_up, down, rw)
        assert out.shape == (tokens, hidden)
    finally:
        op.finalize()
    # World size 1 always fits its own routes (factor 1.0 == world size), so overflow is
    # exercised at the C ABI level in test_gpu_kernels.py::test_routing_capacity_overflow_sets_status.


def test_host_sync_free_mode_matches_and_defers_capacity_error():
    """host_sync_free + saved_views: same results without host waits inside the call."""
    import mega_moe
    tokens, hidden, ffn, experts, top_k = 384, 256, 256, 8, 2
    inp = O.make_inputs(1, tokens, hidden, ffn, experts, top_k, seed=21, weight_std=0.05)
    want_out = O.forward_golden(inp["hidden"], inp["routing_weights"], inp["selected"],
                                inp["w_gate"], inp["w_up"], inp["w_down"], experts)[0]
    _, saved = O.forward_saved(inp["hidden"], inp["routing_weights"], inp["selected"],
                               inp["w_gate"], inp["w_up"], inp["w_down"], top_k)
    want = O.backward(saved, inp["dy"])[0]
    op = _make_op(tokens, hidden, top_k, experts)
    op.host_sync_free = True
    op.saved_views = True
    op.persistent_weight_grads = True
    try:
        for _ in range(3):  # repeated steps reuse every workspace
            x = inp["hidden"][0].to(DEV).requires_grad_(True)
            rw = inp["routing_weights"][0].to(DEV).requires_grad_(True)
            gate_up = mega_moe.pack_gate_up_weights(
                inp["w_gate"][0].to(DEV), inp["w_up"][0].to(DEV)).requires_grad_(True)
            down = inp["w_down"][0].to(DEV).requires_grad_(True)
            out = mega_moe.MegaMoEFunction.apply(op, x, rw, inp["selected"][0].to(DEV), gate_up,
                                                 down, op.context.peer_mem, None)
            gx, grw, ggu, gd = torch.autograd.grad(out, [x, rw, gate_up, down],
                                                   inp["dy"][0].to(DEV))
            _check_out(out.detach(), want_out)
            _check_grad("grad_hidden", gx, want["grad_hidden"])
            _check_grad("grad_routing_weights", grw, want["grad_routing_weights"])
            _check_grad("grad_down", gd, want["grad_fc2"])
            _check_grad("grad_gate_up", ggu, torch.cat(
                (want["grad_fc1_1"], want["grad_fc1_2"]), dim=1).transpose(1, 2))
        op.sync()
        assert op.context.read_status().code == 0
    finally:
        op.finalize()


def test_forward_with_the_reference_benchmarks_skewed_routes():
    """Deterministic skewed routes of the reference's benchmark (restated in the oracle and
    pinned by digests): forward and backward parity on one rank."""
    import mega_moe
    tokens, hidden, ffn, experts, top_k = 256, 256, 128, 32, 8
    inp = O.make_inputs(1, tokens, hidden, ffn, experts, top_k, seed=78, weight_std=0.05)
    routes = [O.kimi_skewed_routes(tokens, experts, top_k, 0)]
    want_out = O.forward_golden(inp["hidden"], inp["routing_weights"], routes, inp["w_gate"],
                                inp["w_up"], inp["w_down"], experts)[0]
    _, saved = O.forward_saved(inp["hidden"], inp["routing_weights"], routes, inp["w_gate"],
                               inp["w_up"], inp["w_down"], top_k)
    want = O.backward(saved, inp["dy"])[0]
    op = _make_op(tokens, hidden, top_k, experts)
    try:
        gate_up = mega_moe.pack_gate_up_weights(inp["w_gate"][0].to(DEV), inp["w_up"][0].to(DEV))
        out, dev_saved = op(inp["hidden"][0].to(DEV), routes[0].to(DEV), gate_up,
                            inp["w_down"][0].to(DEV), inp["routing_weights"][0].to(DEV),
                            return_saved=True)
        _check_out(out, want_out)
        got = mega_moe.moe_backward_triton(dev_saved, inp["dy"][0].to(DEV), op.context.peer_mem)
        for k in ("grad_hidden", "grad_routing_weights", "grad_fc1_1", "grad_fc1_2", "grad_fc2"):
            _check_grad(k, got[k], want[k])
    finally:
        op.finalize()
