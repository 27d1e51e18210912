"""CPU checks of the oracle's saved-FC1 formats against the bounds of the reference's own
tests (tests/layer/test_moe_suite.py:665-735): dequantised fp8 within 0.15 x group amax + 1e-3,
scale = group amax / 448 with the 1 / 448 sentinel for empty groups, fp16 a plain copy."""
import torch

from oracle import moe_oracle as O


def _raw(rows=37, cols=512, seed=3):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(rows, cols, generator=g) * 1.7).to(torch.bfloat16)
    x[5, 128:256] = 0          # an all-zero group
    x[7, :] = 0                # an all-zero row
    x[9, 3] = 300.0            # an outlier dominates its group
    return x


def test_fp8_save_respects_the_reference_bounds():
    group = 128
    raw = _raw()
    q, scale = O.quantize_fc1_fp8(raw, group)
    assert q.dtype == torch.float8_e4m3fn and q.shape == raw.shape
    assert scale.dtype == torch.float32 and scale.shape == (raw.shape[0], raw.shape[1] // group)
    ref = raw.float()
    amax = ref.view(ref.shape[0], -1, group).abs().amax(-1)
    deq = O.dequantize_fc1(q, scale, group)
    err = (deq - ref).abs().view(ref.shape[0], -1, group)
    assert bool((err <= 0.15 * amax[:, :, None] + 1e-3).all())
    # E4M3 round-to-nearest keeps every element within 1/16 of the group's largest value
    assert bool((err <= amax[:, :, None] / 16 + 1e-6).all())
    expected = torch.where(amax > 0, amax, torch.ones_like(amax)) / 448.0
    torch.testing.assert_close(scale, expected, rtol=1e-6, atol=0)
    assert float(scale[5, 1]) == float(torch.tensor(1.0) / torch.tensor(448.0)) and bool((q[5, 128:256].float() == 0).all())
    assert bool((deq[7] == 0).all())
    assert torch.isfinite(q.float()).all()


def test_fp16_save_is_a_plain_copy():
    raw = _raw()
    h = O.convert_fc1_fp16(raw)
    assert h.dtype == torch.float16
    # bf16 values in fp16's normal range convert without loss
    torch.testing.assert_close(h.float(), raw.float(), rtol=0, atol=0)
    assert O.dequantize_fc1(h).dtype == torch.float32


def test_recompute_matches_forward_activation_up_to_the_weight_rounding():
    g = torch.Generator().manual_seed(11)
    gate = torch.randn(64, 96, generator=g).to(torch.bfloat16)
    up = torch.randn(64, 96, generator=g).to(torch.bfloat16)
    w = torch.rand(64, generator=g)
    fwd = (O.gated_activation(gate, up) * w.unsqueeze(-1)).to(torch.bfloat16)
    rec = O.recompute_act(gate, up, w.to(torch.bfloat16))
    torch.testing.assert_close(rec.float(), fwd.float(), rtol=2e-2, atol=2e-2)
    for act, kw in (("clamp_swiglu", dict(clamp_limit=1.0)),
                    ("situglu", dict(situ_beta=1.5, situ_linear_beta=2.0))):
        rec = O.recompute_act(gate, up, w.to(torch.bfloat16), act, **kw)
        fwd = (O.gated_activation(gate, up, act, **kw) * w.unsqueeze(-1)).to(torch.bfloat16)
        torch.testing.assert_close(rec.float(), fwd.float(), rtol=2e-2, atol=2e-2)
