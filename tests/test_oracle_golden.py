"""Pin the CPU oracle to the reference: every function of oracle/moe_oracle.py is compared
with outputs the reference itself produced (fixtures of tests/golden/make_golden.py)."""
import numpy as np
import torch

from oracle import moe_oracle as O


def _eq(a, b):
    assert a.shape == b.shape, (a.shape, b.shape)
    assert torch.equal(a, b), float((a.float() - b.float()).abs().max())


def test_forward_golden_matches_reference(golden):
    g = golden
    outs = O.forward_golden(g.per_rank("in_hidden"), g.per_rank("in_routing_weights"),
                            g.per_rank("in_selected"), g.per_rank("in_w_gate"),
                            g.per_rank("in_w_up"), g.per_rank("in_w_down"), g.experts)
    for r in range(g.world):
        _eq(outs[r], g.get(r, "fwd_golden"))


def test_dispatch_fc1_golden_matches_reference(golden):
    g = golden
    w1 = [torch.cat([a, b], dim=1) for a, b in zip(g.per_rank("in_w_gate"), g.per_rank("in_w_up"))]
    res = O.dispatch_fc1_golden(g.per_rank("in_hidden"), g.per_rank("in_selected"), w1, g.experts)
    for r in range(g.world):
        fc1, eg, xg = res[r]
        _eq(eg, g.get(r, "dfc1_experts"))
        _eq(xg, g.get(r, "dfc1_tokens"))
        _eq(fc1, g.get(r, "dfc1_out"))


def _saved(g):
    return O.forward_saved(g.per_rank("in_hidden"), g.per_rank("in_routing_weights"),
                           g.per_rank("sel_dropless"), g.per_rank("in_w_gate"),
                           g.per_rank("in_w_up"), g.per_rank("in_w_down"), g.top_k)


def test_forward_saved_matches_reference(golden):
    g = golden
    outs, saved = _saved(g)
    for r in range(g.world):
        _eq(outs[r], g.get(r, "mf_output"))
        for k in ("sort_idxs", "local_sort_idxs", "inv_local", "inv_sort", "expert_counts",
                  "split_size_cum_per_expert", "recv_hidden_sorted", "fc1_output",
                  "swiglu_out_weighted", "recv_weights_sorted", "fc2_out"):
            _eq(saved[r][k], g.get(r, "saved_" + k))
        assert saved[r]["splits_send_list"] == g.raw[f"r{r}_saved_splits_send"].tolist()
        assert saved[r]["splits_recv_list"] == g.raw[f"r{r}_saved_splits_recv"].tolist()


def test_backward_matches_reference(golden):
    g = golden
    _, saved = _saved(g)
    grads = O.backward(saved, g.per_rank("in_dy"))
    for r in range(g.world):
        for k in ("grad_hidden", "grad_routing_weights", "grad_fc1_1", "grad_fc1_2", "grad_fc2",
                  "grad_fc2_out_sorted", "grad_swiglu", "grad_fc1_output", "grad_gate",
                  "grad_recv_hidden_sorted"):
            _eq(grads[r][k], g.get(r, "bwd_" + k))


def test_routing_metadata_reproduces_reference_receive_order(golden):
    """The receive order implied by the routing tables (expert-major, source-major, stable
    route order) must gather exactly the rows the reference's forward received."""
    g = golden
    sel = [s.numpy() for s in g.per_rank("sel_dropless")]
    meta = O.routing_metadata(sel, g.experts)
    src = O.receive_sources(meta)
    xs = g.per_rank("in_hidden")
    for r in range(g.world):
        ranks, routes = src[r]
        rows = torch.stack([xs[s][route // g.top_k] for s, route in zip(ranks, routes)]) \
            if len(ranks) else torch.zeros(0, g.hidden, dtype=torch.bfloat16)
        _eq(rows, g.get(r, "saved_recv_hidden_sorted"))
        assert meta[r]["recv_per_expert"].tolist() == g.get(r, "saved_expert_counts").tolist()
        assert meta[r]["recv_expert_offs"].tolist() == \
            g.get(r, "saved_split_size_cum_per_expert").tolist()


def test_routing_metadata_with_drops_matches_dispatch_golden(golden):
    g = golden
    sel = [s.numpy() for s in g.per_rank("in_selected")]
    meta = O.routing_metadata(sel, g.experts)
    src = O.receive_sources(meta)
    xs = g.per_rank("in_hidden")
    for r in range(g.world):
        ranks, routes = src[r]
        rows = torch.stack([xs[s][route // g.top_k] for s, route in zip(ranks, routes)]) \
            if len(ranks) else torch.zeros(0, g.hidden, dtype=torch.bfloat16)
        _eq(rows, g.get(r, "dfc1_tokens"))
        eg = np.repeat(np.arange(g.experts // g.world), meta[r]["recv_per_expert"])
        assert eg.tolist() == g.get(r, "dfc1_experts").tolist()


def test_routing_closed_forms():
    """Closed forms the reference's host tests assert
    (tests/function/test_single_kernel_routing_metadata.py:138-194, stable scatter
    tests/function/test_single_kernel_stable_scatter.py:51-59)."""
    rng = np.random.default_rng(5)
    world, epr, k, tokens = 4, 6, 3, 40
    experts = world * epr
    sel = [rng.integers(-2, experts + 3, size=(tokens, k)).astype(np.int32) for _ in range(world)]
    meta = O.routing_metadata(sel, experts)
    cube = meta[0]["count_cube"]
    for r in range(world):
        m = meta[r]
        flat = sel[r].reshape(-1)
        valid = [i for i in range(flat.size) if 0 <= flat[i] < experts]
        expect = sorted(valid, key=lambda i: flat[i])  # Python's sort is stable
        assert m["send_route_indices"].tolist() == expect
        assert m["send_token_indices"].tolist() == [i // k for i in expect]
        inv = np.full(flat.size, -1)
        inv[expect] = np.arange(len(expect))
        assert m["route_to_send"].tolist() == inv.tolist()
        row = cube[r, :experts]
        assert m["send_bucket_starts"].tolist() == (np.cumsum(row) - row).tolist()
        for d in range(world):
            block = cube[:, d * epr:(d + 1) * epr]
            sums = block.sum(0)
            assert m["send_bucket_dst_starts"][d * epr:(d + 1) * epr].tolist() == \
                ((np.cumsum(sums) - sums) + block[:r].sum(0)).tolist()
            assert m["stats"][2 + d] == sums.sum()
        local_recv = cube[:, r * epr:(r + 1) * epr]
        assert m["recv_counts_re"].tolist() == local_recv.tolist()
        assert m["recv_expert_offs"].tolist() == np.r_[0, np.cumsum(local_recv.sum(0))].tolist()
        assert m["stats"][0] == local_recv.sum()
        assert m["recv_seg_starts"].tolist() == np.column_stack(
            (np.zeros(epr), np.cumsum(local_recv.T, axis=1))).astype(int).tolist()
        for s in range(world):
            excl = np.cumsum(cube[s]) - cube[s]
            assert m["pull_dst_start"].reshape(epr, world)[:, s].tolist() == \
                excl[r * epr:(r + 1) * epr].tolist()


def test_topk_reduce_masks_dropped_routes():
    """tests/function/test_single_kernel_reduce.py:41-77 of the reference."""
    rng = np.random.default_rng(3)
    tokens, k, hidden = 7, 5, 17
    rows = torch.from_numpy(rng.integers(-3, 4, size=(tokens * k, hidden)).astype(np.float32))
    routes = rng.permutation(tokens * k).astype(np.int32)
    routes[::3] = -1
    out = O.topk_reduce(rows.to(torch.bfloat16), routes, tokens, k).float()
    expect = torch.zeros(tokens, hidden)
    for t in range(tokens):
        for r in routes[t * k:(t + 1) * k]:
            if r >= 0:
                expect[t] += rows[r]
    assert torch.equal(out, expect)


# Activation variants (fixtures written by act_worker of tests/golden/make_golden.py).
ACT_FIXTURES = {
    "act_situglu_w2": (dict(activation="situglu", situ_beta=1.5, situ_linear_beta=2.0), True),
    "act_situglu_plain_up_w1": (dict(activation="situglu", situ_beta=0.75,
                                     situ_linear_beta=None), True),
    "act_clamp_swiglu_w1": (dict(activation="clamp_swiglu", clamp_limit=0.5), False),
}


def test_activation_variants_match_reference():
    """Forward (saved tensors, output) with situglu / clamp_swiglu and the situglu backward are
    bit-identical to what the reference's Torch functional path produced."""
    from conftest import Golden
    for name, (kw, has_bwd) in ACT_FIXTURES.items():
        g = Golden(name)
        outs, saved = O.forward_saved(g.per_rank("in_hidden"), g.per_rank("in_routing_weights"),
                                      g.per_rank("in_selected"), g.per_rank("in_w_gate"),
                                      g.per_rank("in_w_up"), g.per_rank("in_w_down"), g.top_k,
                                      **kw)
        for r in range(g.world):
            _eq(outs[r], g.get(r, "mf_output"))
            for k in ("fc1_output", "swiglu_out_weighted", "recv_weights_sorted", "fc2_out"):
                _eq(saved[r][k], g.get(r, "saved_" + k))
        if has_bwd:
            grads = O.backward(saved, g.per_rank("in_dy"))
            for r in range(g.world):
                for k in ("grad_hidden", "grad_routing_weights", "grad_fc1_1", "grad_fc1_2",
                          "grad_fc2", "grad_fc1_output", "grad_gate"):
                    _eq(grads[r][k], g.get(r, "bwd_" + k))


def test_kimi_skewed_routes_match_reference_digests():
    """The restated skew generator reproduces the reference's routes (SHA-256 known answers
    written by tests/golden/make_golden.py) and keeps its invariants."""
    import hashlib
    import json
    from conftest import GOLDEN_DIR
    digests = json.loads((GOLDEN_DIR / "kimi_routes_digests.json").read_text())
    assert len(digests) == 15
    for key, want in digests.items():
        tokens, experts, top_k, rank = (int(p[1:]) for p in key.split("_"))
        routes = O.kimi_skewed_routes(tokens, experts, top_k, rank)
        assert routes.dtype == torch.int32 and routes.shape == (tokens, top_k)
        assert hashlib.sha256(routes.numpy().tobytes()).hexdigest() == want, key
        # no token repeats an expert; owner loads follow the profile
        assert all(len(set(row.tolist())) == top_k for row in routes[:64])
        owners = torch.bincount((routes // (experts // 8)).flatten(), minlength=8)
        assert owners.tolist() == [c * tokens * top_k // 128 for c in O.KIMI_OWNER_LOADS]
    for bad in ((64, 896, 4, 0), (60, 896, 16, 0), (64, 900, 16, 0)):
        try:
            O.kimi_skewed_routes(*bad)
        except ValueError:
            continue
        raise AssertionError(bad)
