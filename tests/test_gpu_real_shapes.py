"""GPU parity at the real hidden / FFN sizes of the benchmark configurations.

The full layers hold tens of GB of expert weights, so each case is a *slice*: the real H and
F, the real rows per expert, but few experts, sized so that the CPU oracle finishes in
seconds.  Every case checks the forward output, every backward intermediate and all five
gradients against the oracle (tolerances of the reference's tests/_numeric.py:24-34 plus
cosine >= 0.9999), in the tile modes the benchmark uses at that rows-per-expert.

* headline layer (H 7168, F 2048): 146 / 292 / 585 / 1170 rows per expert = the per-expert
  load at 1 / 2 / 4 / 8 GPUs (8192 tokens x top-16 over 896 experts);
* Qwen3-30B-A3B-like (H 2048, F 768, top-8), E32-skewed (H 7168, F 2048, Zipf 1.2, top-8) and
  Qwen3-235B-A22B-like (H 4096, F 1536, Zipf 1.0, top-8; also 128 tokens) slices.
"""
import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

INTERMEDIATES = ("grad_fc2_out_sorted", "grad_swiglu", "grad_fc1_output", "grad_gate")
GRADS = ("grad_hidden", "grad_routing_weights", "grad_fc1_1", "grad_fc1_2", "grad_fc2")


def _check_grad(name, got, want):
    ok, max_d, rel, n_bad = O.cmp_grad(got.cpu(), want)
    assert ok, f"{name}: max_abs={max_d:.3e} rel={rel:.3e} mismatches={n_bad}"
    if want.float().abs().max() > 0:
        assert O.cosine(got.cpu(), want) > O.MIN_COSINE, name


def _exact_rows_routes(tokens, experts):
    """Every token selects every expert once (top_k = experts), in a rotated order: each
    expert receives exactly `tokens` rows."""
    base = torch.arange(experts, dtype=torch.int32)
    return torch.stack([(base + t) % experts for t in range(tokens)]).contiguous()


def _run_case(monkeypatch, modes, tokens, hidden, ffn, experts, top_k, zipf, exact_rows, seed):
    import mega_moe
    gemm, wgrad, fused = modes
    monkeypatch.setenv("MOE_GEMM_MODE", gemm)
    monkeypatch.setenv("MOE_WGRAD_MODE", wgrad)
    monkeypatch.setenv("MOE_FUSED_DISPATCH", fused)
    bias = O.zipf_expert_bias(experts, zipf) if zipf else None
    inp = O.make_inputs(1, tokens, hidden, ffn, experts, top_k, seed=seed, expert_bias=bias,
                        weight_std=0.02)
    selected = [_exact_rows_routes(tokens, experts)] if exact_rows else inp["selected"]
    want_out = O.forward_golden(inp["hidden"], inp["routing_weights"], selected, inp["w_gate"],
                                inp["w_up"], inp["w_down"], experts)[0]
    _, gsaved = O.forward_saved(inp["hidden"], inp["routing_weights"], selected, inp["w_gate"],
                                inp["w_up"], inp["w_down"], top_k)
    want = O.backward(gsaved, inp["dy"])[0]
    op = mega_moe.FusedMoEForward(None, max_tokens_per_rank=tokens, hidden_size=hidden,
                                  top_k=top_k, num_experts=experts)
    try:
        gate_up = mega_moe.pack_gate_up_weights(inp["w_gate"][0].to(DEV), inp["w_up"][0].to(DEV))
        out, saved = op(inp["hidden"][0].to(DEV), selected[0].to(DEV), gate_up,
                        inp["w_down"][0].to(DEV), inp["routing_weights"][0].to(DEV),
                        return_saved=True)
        got_out = out.cpu()
        assert torch.isfinite(got_out.float()).all()
        torch.testing.assert_close(got_out.float(), want_out.float(), rtol=O.OUTPUT_RTOL,
                                   atol=O.OUTPUT_ATOL)
        assert O.cosine(got_out, want_out) > O.MIN_COSINE
        # saved activations of the forward against the differentiable-forward restatement
        for key in ("fc1_output", "swiglu_out_weighted"):
            torch.testing.assert_close(saved[key].cpu().float(), gsaved[0][key].float(),
                                       rtol=O.APPROX_RTOL, atol=O.APPROX_ATOL, msg=key)
            assert O.cosine(saved[key].cpu(), gsaved[0][key]) > O.MIN_COSINE, key
        assert torch.equal(saved["recv_hidden_sorted"].cpu(), gsaved[0]["recv_hidden_sorted"])
        got = mega_moe.moe_backward_triton(saved, inp["dy"][0].to(DEV), op.context.peer_mem)
        for key in INTERMEDIATES + GRADS:
            _check_grad(key, got[key], want[key])
        assert op.context.read_status().code == 0
    finally:
        op.finalize()


# rows per expert -> (tile modes the benchmark uses at that load, plus the fused dispatch that
# every multi-GPU run uses)
HEADLINE = [
    # rows/expert, experts, modes (gemm, wgrad, fused dispatch)
    (146, 8, ("auto", "auto", "0")),        # 1 GPU: skinny tiles, unit walk, row-push kernel
    (146, 8, ("single", "single", "1")),
    (292, 8, ("auto", "auto", "1")),        # 2 GPUs
    (585, 4, ("auto", "auto", "1")),        # 4 GPUs
    (1170, 4, ("auto", "auto", "1")),       # 8 GPUs: 9 full row tiles and an 18-row tail
    (1170, 4, ("pair", "pair", "1")),
]


@pytest.mark.parametrize("rows,experts,modes", HEADLINE,
                         ids=[f"rows{r}-e{e}-{'-'.join(m)}" for r, e, m in HEADLINE])
def test_headline_layer_slice(monkeypatch, rows, experts, modes):
    _run_case(monkeypatch, modes, tokens=rows, hidden=7168, ffn=2048, experts=experts,
              top_k=experts, zipf=None, exact_rows=True, seed=rows)


OTHER = [
    # name, tokens, hidden, ffn, experts, top_k, zipf
    ("qwen3_30b_slice", 1024, 2048, 768, 16, 8, None),
    ("e32_skewed_slice", 1024, 7168, 2048, 8, 4, 1.2),
    ("qwen3_235b_slice", 1024, 4096, 1536, 16, 8, 1.0),
    ("qwen3_235b_small_batch", 128, 4096, 1536, 16, 8, 1.0),
]


@pytest.mark.parametrize("name,tokens,hidden,ffn,experts,top_k,zipf", OTHER,
                         ids=[c[0] for c in OTHER])
@pytest.mark.parametrize("fused", ["0", "1"])
def test_other_configuration_slices(monkeypatch, name, tokens, hidden, ffn, experts, top_k, zipf,
                                    fused):
    _run_case(monkeypatch, ("auto", "auto", fused), tokens, hidden, ffn, experts, top_k, zipf,
              exact_rows=False, seed=len(name))
