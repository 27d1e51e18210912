"""GPU parity of the saved dict ``FusedMoEForward.forward(return_saved=True)`` returns, checked
by key class like the reference's native-saved test (tests/layer/test_moe_suite.py:3092-3173):
index keys bitwise against the oracle's tables, the received-row copy bitwise, computed
activations at 2e-2, weight references as zero-copy views; plus the "dropless required"
error, the reference's save leg / recompute helper through the C ABI on the fixture pinned by
the reference's own source text, and the device-time phase record of ``MOE_FWD_TIMING=1``.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

BITWISE_KEYS = ("expert_counts", "split_size_cum_per_expert", "meta_expert_ids", "meta_split_cum",
                "meta_tile_num", "meta_tile_num_cum", "num_tiles_total")
SCALAR_KEYS = ("batch_size", "hidden_dim", "ffn_dim", "topk", "world_size", "ep_rank",
               "experts_per_rank", "M", "total_send", "total_recv", "splits_send_list",
               "splits_recv_list")


def _make_op(tokens, hidden, top_k, experts, **cfg):
    import mega_moe
    from test_gpu_operator import _pow2_divisor
    cfg.setdefault("fc1_gemm_block_size_k", _pow2_divisor(hidden, 128))
    cfg.setdefault("fc2_gemm_block_size_n", _pow2_divisor(hidden, 256))
    return mega_moe.FusedMoEForward(None, max_tokens_per_rank=tokens, hidden_size=hidden,
                                    top_k=top_k, num_experts=experts,
                                    config=mega_moe.MoEForwardConfig(**cfg))


@pytest.mark.parametrize("views", [False, True])
@pytest.mark.parametrize("tokens,hidden,ffn,experts,top_k,zipf", [
    (64, 128, 128, 8, 2, None), (700, 256, 384, 16, 4, 1.2)])
def test_saved_dict_by_key_class(tokens, hidden, ffn, experts, top_k, zipf, views):
    import mega_moe
    bias = O.zipf_expert_bias(experts, zipf) if zipf else None
    inp = O.make_inputs(1, tokens, hidden, ffn, experts, top_k, seed=tokens + 7, expert_bias=bias,
                        weight_std=0.05)
    _, gold = O.forward_saved(inp["hidden"], inp["routing_weights"], inp["selected"],
                              inp["w_gate"], inp["w_up"], inp["w_down"], top_k)
    gold = gold[0]
    meta = O.routing_metadata([inp["selected"][0].numpy()], experts)[0]
    tables = O.saved_contract_tables(meta, inp["selected"][0].numpy(), 1)
    op = _make_op(tokens, hidden, top_k, experts)
    op.saved_views = views
    try:
        gate_up = mega_moe.pack_gate_up_weights(inp["w_gate"][0].to(DEV), inp["w_up"][0].to(DEV))
        down = inp["w_down"][0].to(DEV)
        x, sel, rw = (inp[k][0].to(DEV) for k in ("hidden", "selected", "routing_weights"))
        _, saved = op(x, sel, gate_up, down, rw, return_saved=True)
        # index keys: bitwise
        for key in BITWISE_KEYS + ("sort_idxs", "inv_sort", "local_sort_idxs", "inv_local",
                                   "forward_send_route"):
            np.testing.assert_array_equal(saved[key].cpu().numpy().astype(np.int64),
                                          np.asarray(tables[key]).astype(np.int64), err_msg=key)
        assert torch.equal(saved["selected_experts"], sel)
        # each permutation pair is a pair of inverses, and the receive order it describes
        # gathers exactly the oracle's received rows
        for a, b in (("sort_idxs", "inv_sort"), ("local_sort_idxs", "inv_local")):
            pa, pb = saved[a].long(), saved[b].long()
            assert torch.equal(pa[pb], torch.arange(pa.numel(), device=DEV)), (a, b)
        # scalars and split lists
        want_scalars = dict(gold, M=gold["M"], total_recv=gold["total_recv"],
                            splits_send_list=tables["splits_send_list"],
                            splits_recv_list=tables["splits_recv_list"])
        for key in SCALAR_KEYS:
            assert saved[key] == want_scalars[key], key
        # received rows: bitwise (same receive order as the replay with one source rank)
        assert torch.equal(saved["recv_hidden_sorted"].cpu(), gold["recv_hidden_sorted"])
        # computed activations: the reference grants 2e-2
        for key in ("fc1_output", "swiglu_out_weighted", "recv_weights_sorted"):
            assert saved[key].dtype == torch.bfloat16, key
            torch.testing.assert_close(saved[key].cpu().float(), gold[key].float(),
                                       rtol=O.APPROX_RTOL, atol=O.APPROX_ATOL, msg=key)
        assert torch.equal(saved["recv_weights_sorted"].cpu(), gold["recv_weights_sorted"])
        # weight references: zero-copy views of the forward's inputs
        assert saved["fc1_combined"].data_ptr() == gate_up.data_ptr()
        assert saved["fc1_1"].data_ptr() == gate_up.data_ptr()
        assert saved["fc1_2"].data_ptr() == gate_up[:, :, ffn:].data_ptr()
        assert saved["fc2"].data_ptr() == down.data_ptr()
        for key, ref in (("fc1_1", inp["w_gate"][0]), ("fc1_2", inp["w_up"][0]),
                         ("fc2", inp["w_down"][0])):
            assert torch.equal(saved[key].cpu(), ref), key
        # activation tensors: views of the operator's buffers only when asked for
        is_view = saved["recv_hidden_sorted"].data_ptr() == op.context.peer_mem.data_ptr()
        assert is_view == views
        assert (saved["swiglu_out_weighted"].data_ptr() == op._act_buf.data_ptr()) == views
        # the backward accepts the dict in both forms
        _, gsaved = O.forward_saved(inp["hidden"], inp["routing_weights"], inp["selected"],
                                    inp["w_gate"], inp["w_up"], inp["w_down"], top_k)
        want = O.backward(gsaved, inp["dy"])[0]
        got = mega_moe.moe_backward_triton(saved, inp["dy"][0].to(DEV), op.context.peer_mem)
        for key in ("grad_hidden", "grad_routing_weights", "grad_fc1_1", "grad_fc1_2", "grad_fc2"):
            ok, max_d, rel, n_bad = O.cmp_grad(got[key].cpu(), want[key])
            assert ok, f"{key}: max_abs={max_d:.3e} rel={rel:.3e} mismatches={n_bad}"
        assert op.context.read_status().code == 0
    finally:
        op.finalize()


def test_saved_contract_requires_dropless_routes():
    """reference: ops/_single_saved_adapter.py:116-121."""
    import mega_moe
    tokens, hidden, ffn, experts, top_k = 64, 128, 128, 8, 2
    inp = O.make_inputs(1, tokens, hidden, ffn, experts, top_k, seed=1, drop_frac=0.3)
    op = _make_op(tokens, hidden, top_k, experts)
    try:
        gate_up = mega_moe.pack_gate_up_weights(inp["w_gate"][0].to(DEV), inp["w_up"][0].to(DEV))
        args = (inp["hidden"][0].to(DEV), inp["selected"][0].to(DEV), gate_up,
                inp["w_down"][0].to(DEV), inp["routing_weights"][0].to(DEV))
        with pytest.raises(ValueError, match="droless routing required"):
            op(*args, return_saved=True)
        out = op(*args)                         # the forward alone supports dropped routes
        assert out.shape == (tokens, hidden)
    finally:
        op.finalize()


def test_saved_snapshot_survives_a_later_forward_and_views_do_not_claim_to():
    """A full snapshot (default) stays valid when another forward runs on the operator first,
    as a host sharing one operator between layers needs (reference: ops/function.py:152-158);
    with saved_views the autograd gate refuses the superseded dict."""
    import types

    import mega_moe
    tokens, hidden, ffn, experts, top_k = 128, 128, 128, 8, 2
    a = O.make_inputs(1, tokens, hidden, ffn, experts, top_k, seed=31, weight_std=0.05)
    b = O.make_inputs(1, tokens, hidden, ffn, experts, top_k, seed=32, weight_std=0.05)
    _, gsaved = O.forward_saved(a["hidden"], a["routing_weights"], a["selected"], a["w_gate"],
                                a["w_up"], a["w_down"], top_k)
    want = O.backward(gsaved, a["dy"])[0]
    op = _make_op(tokens, hidden, top_k, experts)
    try:
        def run(inp, views):
            op.saved_views = views
            x = inp["hidden"][0].to(DEV).requires_grad_(True)
            rw = inp["routing_weights"][0].to(DEV).requires_grad_(True)
            gu = mega_moe.pack_gate_up_weights(inp["w_gate"][0].to(DEV),
                                               inp["w_up"][0].to(DEV)).requires_grad_(True)
            dn = inp["w_down"][0].to(DEV).requires_grad_(True)
            out = mega_moe.MegaMoEFunction.apply(op, x, rw, inp["selected"][0].to(DEV), gu, dn,
                                                 op.context.peer_mem, types.SimpleNamespace())
            return out, x
        out_a, x_a = run(a, False)
        run(b, False)                            # a later layer's forward on the same operator
        out_a.backward(a["dy"][0].to(DEV))
        ok, max_d, rel, n_bad = O.cmp_grad(x_a.grad.cpu(), want["grad_hidden"])
        assert ok, f"grad_hidden after a later forward: max_abs={max_d:.3e} mismatches={n_bad}"
        out_v, _ = run(a, True)
        run(b, True)
        with pytest.raises(RuntimeError, match="superseded"):
            out_v.backward(a["dy"][0].to(DEV))
    finally:
        op.finalize()


def _fixture():
    from conftest import GOLDEN_DIR
    with np.load(GOLDEN_DIR / "saved_formats.npz") as z:
        return {k: z[k] for k in z.files}


def test_save_convert_and_recompute_match_the_reference_source_bit_exactly():
    """mm_fc1_save_convert / mm_swiglu_recompute on the rows of tests/golden/saved_formats.npz,
    whose outputs were produced by executing the reference's own kernel source."""
    from mega_moe import _native as N
    z = _fixture()
    rows, ffn, group = (int(v) for v in z["meta"])
    raw = torch.from_numpy(z["in_raw"].copy()).view(torch.bfloat16).to(DEV)
    w = torch.from_numpy(z["in_weights"].copy()).view(torch.bfloat16).to(DEV)
    n_rows = torch.tensor([rows], dtype=torch.int32, device=DEV)
    lib = N.lib()
    h = torch.zeros(rows, 2 * ffn, dtype=torch.float16, device=DEV)
    N.check(lib.mm_fc1_save_convert(raw.data_ptr(), raw.stride(0), 2 * ffn, n_rows.data_ptr(),
                                    rows, N.FC1_FORMAT_IDS["fp16"], 0, h.data_ptr(), h.stride(0),
                                    None, N.stream_ptr()), "fp16")
    assert torch.equal(h.cpu().view(torch.int16), torch.from_numpy(z["save_fp16"].copy()))
    q = torch.zeros(rows, 2 * ffn, dtype=torch.uint8, device=DEV)
    scale = torch.zeros(rows, 2 * ffn // group, dtype=torch.float32, device=DEV)
    N.check(lib.mm_fc1_save_convert(raw.data_ptr(), raw.stride(0), 2 * ffn, n_rows.data_ptr(),
                                    rows, N.FC1_FORMAT_IDS["fp8"], group, q.data_ptr(),
                                    q.stride(0), scale.data_ptr(), N.stream_ptr()), "fp8")
    assert torch.equal(q.cpu(), torch.from_numpy(z["save_fp8"].copy()))
    assert torch.equal(scale.cpu(), torch.from_numpy(z["save_fp8_scale"].copy()))
    acts = {"swiglu": (0, 1.0, 0.0, 7.0), "situglu": (1, 1.5, 2.0, 7.0),
            "situglu_plain_up": (1, 0.75, 0.0, 7.0), "clamp_swiglu": (2, 1.0, 0.0, 0.5)}
    for fmt, src, sc, grp in (("bf16", raw, None, 0), ("fp8", q, scale, group)):
        for name, (act_id, beta, lbeta, clamp) in acts.items():
            out = torch.zeros(rows, ffn, dtype=torch.bfloat16, device=DEV)
            N.check(lib.mm_swiglu_recompute(
                src.data_ptr(), src.stride(0), N.FC1_FORMAT_IDS[fmt], N.ptr(sc), grp,
                w.data_ptr(), ffn, n_rows.data_ptr(), rows, out.data_ptr(), out.stride(0), act_id,
                beta, lbeta, clamp, N.stream_ptr()), "recompute")
            want = torch.from_numpy(z[f"recompute_{fmt}_{name}"].copy()).view(torch.bfloat16)
            # the device's sigmoid / tanh differ from the host's in the last bits: one bf16
            # step at most on a small fraction of the elements
            got = out.cpu().float()
            diff = (got - want.float()).abs()
            assert bool((diff <= 2.0 ** -7 * want.float().abs() + 1e-30).all()), (fmt, name)
            assert float((diff > 0).float().mean()) < 0.05, (fmt, name)


def test_forward_phase_timing_follows_the_reference_switch(monkeypatch):
    import mega_moe
    tokens, hidden, ffn, experts, top_k = 256, 256, 128, 8, 2
    inp = O.make_inputs(1, tokens, hidden, ffn, experts, top_k, seed=2)
    op = _make_op(tokens, hidden, top_k, experts)
    try:
        gate_up = mega_moe.pack_gate_up_weights(inp["w_gate"][0].to(DEV), inp["w_up"][0].to(DEV))
        args = (inp["hidden"][0].to(DEV), inp["selected"][0].to(DEV), gate_up,
                inp["w_down"][0].to(DEV), inp["routing_weights"][0].to(DEV))
        op(*args)
        with pytest.raises(RuntimeError):
            op.read_last_forward_phase_timing()
        monkeypatch.setenv("MOE_FWD_TIMING", "1")
        op(*args)
        rec = op.read_last_forward_phase_timing()
        assert list(rec["phase_ms"]) == ["routing_metadata", "dispatch_fc1_activation",
                                         "fc2_combine", "rank_barrier", "topk_reduce"]
        assert all(v >= 0 for v in rec["phase_ms"].values()) and rec["total_ms"] > 0
    finally:
        op.finalize()
