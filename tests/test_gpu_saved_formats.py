"""GPU parity of the saved-FC1 formats (`save_fc1_dtype` = fp16 / fp8) and of the recompute
backward (`MOE_SAVED_RECOMPUTE=1`) against the CPU oracle.

The forward's saved tensor must be bit-identical to the oracle's conversion of the same raw
bf16 rows and must respect the bounds of the reference's own tests
(tests/layer/test_moe_suite.py:665-735); the backward on such a saved dict must match the
oracle backward fed with the dequantised values, within the reference's gradient tolerance
(|d| <= 1e-2 + 2e-2 * max|gold|, cosine >= 0.9999).
"""
import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
GRAD_KEYS = ("grad_fc2_out_sorted", "grad_swiglu", "grad_fc1_output", "grad_gate", "grad_hidden",
             "grad_routing_weights", "grad_fc1_1", "grad_fc1_2", "grad_fc2")


def _make_op(tokens, hidden, top_k, experts, **cfg):
    import mega_moe
    from test_gpu_operator import _pow2_divisor
    cfg.setdefault("fc1_gemm_block_size_k", _pow2_divisor(hidden, 128))
    cfg.setdefault("fc2_gemm_block_size_n", _pow2_divisor(hidden, 256))
    return mega_moe.FusedMoEForward(None, max_tokens_per_rank=tokens, hidden_size=hidden,
                                    top_k=top_k, num_experts=experts,
                                    config=mega_moe.MoEForwardConfig(**cfg))


def _to_dev(saved):
    return {k: (v.to(DEV) if isinstance(v, torch.Tensor) else v) for k, v in saved.items()}


def _check_grad(name, got, want):
    ok, max_d, rel, n_bad = O.cmp_grad(got.cpu(), want)
    assert ok, f"{name}: max_abs={max_d:.3e} rel={rel:.3e} mismatches={n_bad}"
    if want.float().abs().max() > 0:
        assert O.cosine(got.cpu(), want) > O.MIN_COSINE, name


def _inputs(tokens, hidden, ffn, experts, top_k, seed):
    return O.make_inputs(1, tokens, hidden, ffn, experts, top_k, seed=seed, weight_std=0.05)


@pytest.mark.parametrize("fmt", ["fp16", "fp8"])
def test_forward_saves_fc1_in_the_requested_format(fmt):
    import mega_moe
    tokens, hidden, ffn, experts, top_k = 300, 256, 256, 8, 4
    inp = _inputs(tokens, hidden, ffn, experts, top_k, seed=5)
    _, gold_saved = O.forward_saved(inp["hidden"], inp["routing_weights"], inp["selected"],
                                    inp["w_gate"], inp["w_up"], inp["w_down"], top_k)
    op = _make_op(tokens, hidden, top_k, experts, save_fc1_dtype=fmt)
    try:
        gate_up = mega_moe.pack_gate_up_weights(inp["w_gate"][0].to(DEV), inp["w_up"][0].to(DEV))
        x, sel, rw = (inp[k][0].to(DEV) for k in ("hidden", "selected", "routing_weights"))
        _, saved = op(x, sel, gate_up, inp["w_down"][0].to(DEV), rw, return_saved=True)
        m = int(saved["M"])
        raw = op._fc1_buf[:m].cpu()                      # the bf16 rows the save was made from
        ref = gold_saved[0]["fc1_output"].float()
        got = saved["fc1_output"].cpu()
        assert got.shape == (m, 2 * ffn)
        if fmt == "fp16":
            assert got.dtype == torch.float16 and "fc1_output_scale" not in saved
            assert torch.equal(got, O.convert_fc1_fp16(raw))
            err = (got.float() - ref).abs()
            assert bool((err <= 0.15 * ref.abs() + 1e-3).all())
        else:
            group = int(saved["fc1_scale_group_size"])
            assert group == op.config.fc1_gemm_block_size_n // 2
            scale = saved["fc1_output_scale"].cpu()
            assert got.dtype == torch.float8_e4m3fn and scale.dtype == torch.float32
            assert scale.shape == (m, 2 * ffn // group)
            q, s = O.quantize_fc1_fp8(raw, group)
            assert torch.equal(got.view(torch.uint8), q.view(torch.uint8))
            assert torch.equal(scale, s)
            deq = O.dequantize_fc1(got, scale, group)
            amax = ref.view(m, -1, group).abs().amax(-1)
            err = (deq - ref).abs().view(m, -1, group)
            assert bool((err <= 0.15 * amax[:, :, None] + 1e-3).all())
            expected = torch.where(amax > 1e-3, amax, torch.ones_like(amax)) / 448.0
            torch.testing.assert_close(scale, expected, rtol=1e-1, atol=1e-3)
        assert op.context.read_status().code == 0
    finally:
        op.finalize()


@pytest.mark.parametrize("fmt", ["fp16", "fp8"])
@pytest.mark.parametrize("activation", ["swiglu", "situglu"])
def test_backward_reads_saved_fc1_formats(fmt, activation):
    import mega_moe
    tokens, hidden, ffn, experts, top_k, group = 256, 256, 128, 8, 2, 128
    inp = _inputs(tokens, hidden, ffn, experts, top_k, seed=9)
    kw = dict(activation=activation)
    if activation == "situglu":
        kw.update(situ_beta=1.5, situ_linear_beta=2.0)
    _, saved = O.forward_saved(inp["hidden"], inp["routing_weights"], inp["selected"],
                               inp["w_gate"], inp["w_up"], inp["w_down"], top_k, **kw)
    s = saved[0]
    raw = s["fc1_output"]
    if fmt == "fp16":
        stored, scale = O.convert_fc1_fp16(raw), None
    else:
        stored, scale = O.quantize_fc1_fp8(raw, group)
    deq = O.dequantize_fc1(stored, scale, group)
    gold = dict(s, gate=deq[:, :ffn], up=deq[:, ffn:])
    want = O.backward([gold], inp["dy"])[0]
    op = _make_op(tokens, hidden, top_k, experts)
    try:
        dev_saved = _to_dev(dict(s, fc1_output=stored))
        if scale is not None:
            dev_saved["fc1_output_scale"] = scale.to(DEV)
            dev_saved["fc1_scale_group_size"] = group
        got = mega_moe.moe_backward_triton(dev_saved, inp["dy"][0].to(DEV), op.context.peer_mem)
        for k in GRAD_KEYS:
            _check_grad(k, got[k], want[k])
        assert op.context.read_status().code == 0
    finally:
        op.finalize()


@pytest.mark.parametrize("fmt", ["bf16", "fp8"])
def test_recompute_backward(fmt, monkeypatch):
    """MOE_SAVED_RECOMPUTE=1: no saved receive rows, no saved activation; the input rows are
    dispatched again and the activation is rebuilt from the saved FC1 rows."""
    import mega_moe
    monkeypatch.setenv("MOE_SAVED_RECOMPUTE", "1")
    tokens, hidden, ffn, experts, top_k, group = 320, 256, 128, 8, 2, 128
    inp = _inputs(tokens, hidden, ffn, experts, top_k, seed=13)
    _, saved = O.forward_saved(inp["hidden"], inp["routing_weights"], inp["selected"],
                               inp["w_gate"], inp["w_up"], inp["w_down"], top_k)
    s = saved[0]
    if fmt == "fp8":
        stored, scale = O.quantize_fc1_fp8(s["fc1_output"], group)
    else:
        stored, scale = s["fc1_output"], None
    deq = O.dequantize_fc1(stored, scale, group)
    act = O.recompute_act(deq[:, :ffn], deq[:, ffn:], s["recv_weights_sorted"])
    gold = dict(s, gate=deq[:, :ffn], up=deq[:, ffn:], swiglu_out_weighted=act)
    want = O.backward([gold], inp["dy"])[0]
    op = _make_op(tokens, hidden, top_k, experts)
    try:
        assert op.context.redispatch_mem is not None
        dev_saved = _to_dev(dict(s, fc1_output=stored))
        del dev_saved["recv_hidden_sorted"], dev_saved["swiglu_out_weighted"]
        if scale is not None:
            dev_saved["fc1_output_scale"] = scale.to(DEV)
            dev_saved["fc1_scale_group_size"] = group
        got = mega_moe.moe_backward_triton(dev_saved, inp["dy"][0].to(DEV), op.context.peer_mem,
                                           hidden_states=inp["hidden"][0].to(DEV))
        for k in GRAD_KEYS:
            _check_grad(k, got[k], want[k])
        assert op.context.read_status().code == 0
    finally:
        op.finalize()


def test_recompute_needs_the_slab_and_the_input(monkeypatch):
    import mega_moe
    tokens, hidden, ffn, experts, top_k = 64, 128, 128, 8, 2
    inp = _inputs(tokens, hidden, ffn, experts, top_k, seed=17)
    _, saved = O.forward_saved(inp["hidden"], inp["routing_weights"], inp["selected"],
                               inp["w_gate"], inp["w_up"], inp["w_down"], top_k)
    op = _make_op(tokens, hidden, top_k, experts)        # constructed without the switch
    try:
        monkeypatch.setenv("MOE_SAVED_RECOMPUTE", "1")
        dev_saved = _to_dev(saved[0])
        with pytest.raises(RuntimeError):
            mega_moe.moe_backward_triton(dev_saved, inp["dy"][0].to(DEV), op.context.peer_mem,
                                         hidden_states=inp["hidden"][0].to(DEV))
        assert "hidden_states" not in dev_saved
        with pytest.raises(ValueError):
            mega_moe.moe_backward_triton(dev_saved, inp["dy"][0].to(DEV), op.context.peer_mem)
    finally:
        op.finalize()
