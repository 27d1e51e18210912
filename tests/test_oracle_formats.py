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


# ---- pinned by the reference's own source text (tests/golden/make_golden_saved.py) ----------
def _fixture(name):
    import numpy as np
    from conftest import GOLDEN_DIR
    with np.load(GOLDEN_DIR / name) as z:
        return {k: z[k] for k in z.files}


def _bf16(a):
    return torch.from_numpy(a.copy()).view(torch.bfloat16)


def test_saved_formats_reproduce_the_reference_save_leg_bit_exactly():
    """fp16 / fp8 save of raw FC1 rows: the reference's store statement
    (kernels/fused_forward.py:891-949) executed on the same rows."""
    z = _fixture("saved_formats.npz")
    rows, ffn, group = (int(v) for v in z["meta"])
    raw = _bf16(z["in_raw"])
    assert torch.equal(_bf16(z["save_bf16"]), raw)
    h = O.convert_fc1_fp16(raw)
    assert torch.equal(h.view(torch.int16), torch.from_numpy(z["save_fp16"].copy()))
    q, scale = O.quantize_fc1_fp8(raw, group)
    assert torch.equal(q.view(torch.uint8), torch.from_numpy(z["save_fp8"].copy()))
    assert torch.equal(scale, torch.from_numpy(z["save_fp8_scale"].copy()))


def test_recompute_reproduces_the_reference_helper_bit_exactly():
    """_recompute_act_rows (kernels/mega_bwd.py:1414-1465) on bf16 and fp8 saved rows."""
    z = _fixture("saved_formats.npz")
    rows, ffn, group = (int(v) for v in z["meta"])
    raw = _bf16(z["in_raw"])
    w = _bf16(z["in_weights"])
    q = torch.from_numpy(z["save_fp8"].copy()).view(torch.float8_e4m3fn)
    scale = torch.from_numpy(z["save_fp8_scale"].copy())
    acts = {"swiglu": ("swiglu", {}),
            "situglu": ("situglu", dict(situ_beta=1.5, situ_linear_beta=2.0)),
            "situglu_plain_up": ("situglu", dict(situ_beta=0.75, situ_linear_beta=None)),
            "clamp_swiglu": ("clamp_swiglu", dict(clamp_limit=0.5))}
    for fmt in ("bf16", "fp8"):
        vals = raw.float() if fmt == "bf16" else O.dequantize_fc1(q, scale, group)
        for name, (act, kw) in acts.items():
            got = O.recompute_act(vals[:, :ffn], vals[:, ffn:], w, act, **kw)
            want = _bf16(z[f"recompute_{fmt}_{name}"])
            assert torch.equal(got.view(torch.int16), want.view(torch.int16)), (fmt, name)


def test_saved_contract_tables_reproduce_the_reference_helpers():
    """prepare_moe_metadata and _arrival_to_slot_permutation of the reference on seeded counts."""
    import numpy as np
    z = _fixture("saved_tables.npz")
    for i, (world, epr) in enumerate(z["cases"]):
        counts = z[f"c{i}_counts"]
        per_expert = counts.sum(0)
        perm = O.arrival_to_slot_permutation(counts, np.cumsum(per_expert) - per_expert)
        np.testing.assert_array_equal(perm, z[f"c{i}_local_sort_idxs"])
        meta = O.tile_metadata(per_expert)
        for key, val in meta.items():
            np.testing.assert_array_equal(val, z[f"c{i}_{key}"], err_msg=key)
