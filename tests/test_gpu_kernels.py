"""GPU parity tests of the individual C-ABI entry points (routing bit-exact, GEMMs vs fp32)."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _route_local(sel_np, num_experts, top_k):
    from mega_moe import _native as N
    from mega_moe.runtime.workspace import next_power_of_2
    lib = N.lib()
    sel = torch.tensor(sel_np, dtype=torch.int32, device=DEV).contiguous()
    n = sel.numel()
    bins = next_power_of_2(num_experts)
    i32 = dict(dtype=torch.int32, device=DEV)
    outs = dict(send_route=torch.full((max(n, 1),), -7, **i32),
                send_token=torch.full((max(n, 1),), -7, **i32),
                send_bucket=torch.full((max(n, 1),), -7, **i32),
                route_to_send=torch.full((max(n, 1),), -7, **i32),
                count_row=torch.full((bins,), -7, **i32), local_stats=torch.full((2,), -7, **i32))
    nbytes = lib.mm_route_scratch_bytes(n, bins)
    scratch = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=DEV)
    N.check(lib.mm_route_local(sel.data_ptr(), n, top_k, num_experts, bins,
                               outs["send_route"].data_ptr(), outs["send_token"].data_ptr(),
                               outs["send_bucket"].data_ptr(), outs["route_to_send"].data_ptr(),
                               outs["count_row"].data_ptr(), outs["local_stats"].data_ptr(),
                               scratch.data_ptr(), scratch.numel(), N.stream_ptr()),
            "mm_route_local")
    torch.cuda.synchronize()
    return {k: v.cpu().numpy() for k, v in outs.items()}, bins


def _finalize(cube_np, rank, world, epr, bins, capacity, tile_tail=0):
    """Run mm_route_finalize on fresh tables.  ``tile_tail`` extra entries are appended to the
    four row-tile tables (the documented size is capacity / tile rows + epr) so a caller can
    check that nothing is written past the documented end."""
    from mega_moe import _native as N
    lib = N.lib()
    i32 = dict(dtype=torch.int32, device=DEV)
    nb = world * epr
    cube = torch.tensor(cube_np.reshape(-1), **i32)
    t = dict(send_bucket_starts=torch.full((nb,), -7, **i32),
             send_bucket_dst_starts=torch.full((nb,), -7, **i32),
             recv_counts_re=torch.full((world * epr,), -7, **i32),
             recv_per_expert=torch.full((epr,), -7, **i32),
             recv_expert_offs=torch.zeros(epr + 1, **i32),
             recv_seg_starts=torch.full((epr * (world + 1),), -7, **i32),
             pull_dst_start=torch.full((epr * world,), -7, **i32),
             stats=torch.full((2 + world,), -7, **i32),
             mtile_group=torch.full((capacity // 128 + epr + tile_tail,), -7, **i32),
             mtile_row0=torch.full((capacity // 128 + epr + tile_tail,), -7, **i32),
             num_mtiles=torch.full((1,), -7, **i32),
             mtile2_group=torch.full((capacity // 256 + epr + tile_tail,), -7, **i32),
             mtile2_row0=torch.full((capacity // 256 + epr + tile_tail,), -7, **i32),
             num_mtiles2=torch.full((1,), -7, **i32),
             row_src_rank=torch.full((max(capacity, 1),), -7, **i32),
             row_src_pos=torch.full((max(capacity, 1),), -7, **i32),
             order_prefix=torch.full((nb + 1,), -7, **i32),
             bucket_done=torch.full((nb,), -7, **i32),
             row_arrival=torch.full((max(capacity, 1),), -7, **i32),
             arrival_row=torch.full((max(capacity, 1),), -7, **i32))
    status = torch.zeros(8, **i32)
    order = ["send_bucket_starts", "send_bucket_dst_starts", "recv_counts_re", "recv_per_expert",
             "recv_expert_offs", "recv_seg_starts", "pull_dst_start", "stats", "mtile_group",
             "mtile_row0", "num_mtiles", "mtile2_group", "mtile2_row0", "num_mtiles2",
             "row_src_rank", "row_src_pos", "order_prefix",
             "bucket_done", "row_arrival", "arrival_row"]
    N.check(lib.mm_route_finalize(cube.data_ptr(), rank, world, epr, bins, capacity,
                                  *[t[k].data_ptr() for k in order], status.data_ptr(),
                                  N.stream_ptr()), "mm_route_finalize")
    torch.cuda.synchronize()
    return {k: v.cpu().numpy() for k, v in t.items()}, status.cpu().numpy()


ROUTE_CASES = [
    # tokens, top_k, experts, world, drop fraction
    (64, 2, 8, 1, 0.0),
    (300, 3, 24, 4, 0.3),
    (8192, 16, 896, 8, 0.0),
    (4096, 8, 128, 2, 0.05),
    (1000, 4, 32, 8, 1.0),   # every route dropped
    (1, 1, 4, 2, 0.0),
]


@pytest.mark.parametrize("tokens,top_k,experts,world,drop", ROUTE_CASES)
def test_routing_metadata_bit_exact(tokens, top_k, experts, world, drop):
    rng = np.random.default_rng(tokens + experts)
    epr = experts // world
    sels = []
    for r in range(world):
        s = rng.integers(0, experts, size=(tokens, top_k)).astype(np.int32)
        if drop > 0:
            bad = rng.random((tokens, top_k)) < drop
            s[bad] = rng.choice([-1, experts, experts + 5], size=int(bad.sum()))
        sels.append(s)
    meta = O.routing_metadata(sels, experts)
    rows = []
    for r in range(world):
        got, bins = _route_local(sels[r], experts, top_k)
        want = meta[r]
        n = want["num_sent_routes"]
        assert got["local_stats"][0] == n
        np.testing.assert_array_equal(got["send_route"][:n], want["send_route_indices"])
        np.testing.assert_array_equal(got["send_token"][:n], want["send_token_indices"])
        np.testing.assert_array_equal(got["send_bucket"][:n], want["send_bucket"])
        np.testing.assert_array_equal(got["route_to_send"][:tokens * top_k], want["route_to_send"])
        np.testing.assert_array_equal(got["count_row"], want["count_cube"][r])
        rows.append(got["count_row"])
    cube = np.stack(rows)
    capacity = int(meta[0]["stats"][1]) + 5
    for r in range(world):
        got, status = _finalize(cube, r, world, epr, bins, capacity)
        want = meta[r]
        assert status[0] == 0
        for k in ("send_bucket_starts", "send_bucket_dst_starts", "recv_per_expert",
                  "recv_expert_offs", "pull_dst_start", "stats"):
            np.testing.assert_array_equal(got[k], want[k].reshape(-1), err_msg=k)
        np.testing.assert_array_equal(got["recv_counts_re"], want["recv_counts_re"].reshape(-1))
        np.testing.assert_array_equal(got["recv_seg_starts"], want["recv_seg_starts"].reshape(-1))
        m = want["num_received_routes"]
        np.testing.assert_array_equal(got["row_src_rank"][:m], want["row_src_rank"])
        np.testing.assert_array_equal(got["row_src_pos"][:m], want["row_src_pos"])
        exp_groups, exp_rows = [], []
        for e in range(epr):
            for r0 in range(0, int(want["recv_per_expert"][e]), 128):
                exp_groups.append(e)
                exp_rows.append(int(want["recv_expert_offs"][e]) + r0)
        # dispatch order: local expert slot outermost, destinations rotated by the rank
        order = [((r + 1 + dd) % world) * epr + le for le in range(epr) for dd in range(world)]
        local_row = cube[r, :world * epr]
        np.testing.assert_array_equal(got["order_prefix"],
                                      np.r_[0, np.cumsum(local_row[order])])
        assert (got["bucket_done"] == 0).all()
        nt = int(got["num_mtiles"][0])
        assert nt == len(exp_groups)
        np.testing.assert_array_equal(got["mtile_group"][:nt], exp_groups)
        np.testing.assert_array_equal(got["mtile_row0"][:nt], exp_rows)
        g2, r2 = [], []
        for e in range(epr):
            for r0 in range(0, int(want["recv_per_expert"][e]), 256):
                g2.append(e)
                r2.append(int(want["recv_expert_offs"][e]) + r0)
        assert int(got["num_mtiles2"][0]) == len(g2)
        np.testing.assert_array_equal(got["mtile2_group"][:len(g2)], g2)
        np.testing.assert_array_equal(got["mtile2_row0"][:len(g2)], r2)


def test_routing_capacity_overflow_sets_status():
    rng = np.random.default_rng(0)
    sel = rng.integers(0, 8, size=(256, 2)).astype(np.int32)
    meta = O.routing_metadata([sel], 8)
    got, bins = _route_local(sel, 8, 2)
    out, status = _finalize(got["count_row"][None, :], 0, 1, 8, bins, 100)
    assert status[0] == 2 and status[3] == 100 and status[4] == 512
    assert out["num_mtiles"][0] == 0 and out["num_mtiles2"][0] == 0
    assert out["stats"][1] == meta[0]["stats"][1]


@pytest.mark.parametrize("world,epr,rows_per_bucket,capacity", [
    (1, 8, 4000, 100),        # 32 000 rows into room for 100: 250 tiles against 8 entries
    (8, 112, 300, 20000),     # headline bucket count, 2.1x the capacity of every rank
    (4, 2, 70000, 128),
])
def test_routing_capacity_overflow_writes_no_tile_entry(world, epr, rows_per_bucket, capacity):
    """A receive total far above capacity_rows must leave the row-tile tables untouched: they are
    sized for capacity_rows, and entries past them would land in someone else's memory."""
    from mega_moe.runtime.workspace import next_power_of_2
    nb = world * epr
    bins = next_power_of_2(nb)
    cube = np.zeros((world, bins), dtype=np.int32)
    cube[:, :nb] = rows_per_bucket // world
    tail = 8192
    for rank in range(world):
        out, status = _finalize(cube, rank, world, epr, bins, capacity, tile_tail=tail)
        assert status[0] == 2 and status[3] == capacity
        assert status[4] == (rows_per_bucket // world) * world * epr
        assert out["num_mtiles"][0] == 0 and out["num_mtiles2"][0] == 0
        for key in ("mtile_group", "mtile_row0", "mtile2_group", "mtile2_row0"):
            assert (out[key] == -7).all(), key
        # the per-row tables are guarded by capacity_rows as before
        assert out["row_src_rank"].shape[0] == capacity


@pytest.fixture(params=[1, 0, 2], ids=["pair", "single", "skinny"])
def gemm_mode(request):
    """Run a GEMM test in every tile mode: CTA pairs (cta_group::2), single CTAs, and the
    transposed product for groups with few rows."""
    import _gpu_util
    old = _gpu_util.PAIR
    _gpu_util.PAIR = request.param
    yield request.param
    _gpu_util.PAIR = old


GEMM_CASES = [
    # counts per group, K, N
    ([128], 64, 256),
    ([128, 128], 128, 256),
    ([37, 0, 200, 129], 192, 512),
    ([300, 5], 256, 128),
    ([1000, 24, 0, 0, 511], 1024, 768),
]


@pytest.mark.parametrize("counts,K,N", GEMM_CASES)
@pytest.mark.parametrize("layout", ["k_major", "mn_major"])
def test_grouped_gemm_matches_fp32(counts, K, N, layout, gemm_mode):
    from _gpu_util import ref_grouped, rel_err, run_grouped_gemm
    g = torch.Generator(device="cpu").manual_seed(K + N)
    rows = sum(counts)
    a = (torch.randn(rows + 3, K, generator=g) * 0.5).to(torch.bfloat16).to(DEV)
    groups = len(counts)
    if layout == "k_major":
        w = (torch.randn(groups, N, K, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
        k_dim, n_dim = 2, 1
    else:
        w = (torch.randn(groups, K, N, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
        k_dim, n_dim = 1, 2
    out = run_grouped_gemm(a, w, k_dim, n_dim, counts)
    ref = ref_grouped(a, w, k_dim, n_dim, counts)
    assert torch.isfinite(out[:rows].float()).all()
    assert rel_err(out[:rows], ref[:rows]) < 1e-2
    # rows past the last group are never written
    assert torch.isnan(out[rows:].float()).all()


@pytest.mark.parametrize("counts,H,F", [([128], 64, 128), ([70, 200, 0, 129], 256, 256),
                                        ([513, 31], 512, 384)])
@pytest.mark.parametrize("activation", ["swiglu", "clamp_swiglu", "situglu"])
def test_fc1_swiglu_matches_oracle_rounding(counts, H, F, activation, gemm_mode):
    from _gpu_util import rel_err, run_fc1_swiglu
    g = torch.Generator(device="cpu").manual_seed(H + F)
    rows = sum(counts)
    a = (torch.randn(rows, H, generator=g)).to(torch.bfloat16)
    w = (torch.randn(len(counts), H, 2 * F, generator=g) * 0.2).to(torch.bfloat16)
    rw = torch.rand(rows, generator=g) + 0.1
    kw = dict(activation=activation, beta=1.5, linear_beta=2.0 if activation == "situglu" else None,
              clamp=1.0)
    act, raw = run_fc1_swiglu(a.to(DEV), w.to(DEV), rw.to(DEV), counts, **kw)
    ref_raw = torch.zeros(rows, 2 * F)
    start = 0
    for e, c in enumerate(counts):
        ref_raw[start:start + c] = a[start:start + c].float() @ w[e].float()
        start += c
    ref_raw = ref_raw.to(torch.bfloat16)
    assert rel_err(raw.cpu(), ref_raw) < 1e-2
    # activation computed from the kernel's own bf16 gate/up must match the oracle's formula
    gate, up = raw.cpu()[:, :F], raw.cpu()[:, F:]
    ref_act = (O.gated_activation(gate, up, activation, 1.5,
                                  2.0 if activation == "situglu" else None, 1.0)
               * rw[:, None]).to(torch.bfloat16)
    torch.testing.assert_close(act.cpu().float(), ref_act.float(), rtol=O.APPROX_RTOL,
                               atol=O.APPROX_ATOL)
    assert O.cosine(act.cpu(), ref_act) > O.MIN_COSINE


@pytest.mark.parametrize("counts,Mw,Nw", [([64], 128, 256), ([128, 70], 256, 256),
                                          ([5, 0, 300, 64, 1], 384, 128),
                                          ([1000, 0, 37], 512, 768)])
def test_grouped_wgrad_matches_fp32(counts, Mw, Nw, gemm_mode):
    from _gpu_util import rel_err, run_wgrad
    g = torch.Generator(device="cpu").manual_seed(Mw + Nw)
    rows = sum(counts)
    go = (torch.randn(rows + 2, Mw, generator=g) * 0.3).to(torch.bfloat16).to(DEV)
    oi = (torch.randn(rows, Nw, generator=g) * 0.3).to(torch.bfloat16).to(DEV)
    # poison the rows after the last group: they must not leak into the last group's sum
    go[rows:] = float("nan")
    out = run_wgrad(go, oi, counts)
    start = 0
    for e, c in enumerate(counts):
        ref = (go[start:start + c].float().T @ oi[start:start + c].float()).to(torch.bfloat16)
        if c == 0:
            assert (out[e] == 0).all()
        else:
            assert rel_err(out[e], ref) < 1e-2, (e, c)
        start += c
