"""MoonEP planning and balanced routing of the package on host tensors, through the C ABI
(``mm_moonep_*_host`` run the same code as the device kernels), against fixtures written by the
reference's own host code and the known answers of its tests
(tests/function/test_moonep_planning.py, tests/function/test_balanced_routing.py)."""

from __future__ import annotations

import hashlib
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

REPO = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(REPO / "mega-moe-td_b200"))

from mega_moe import _native as N  # noqa: E402
from mega_moe.runtime.balanced_routing import (  # noqa: E402
    build_balanced_routing_metadata, experts_to_copy_from_inverse)
from mega_moe.runtime.moonep_planning import (  # noqa: E402
    MoonEPPlanningResult, build_inverse_experts_to_copy, plan_moonep_b0_b3)
from oracle import moonep_oracle as M  # noqa: E402

GOLDEN = Path(__file__).resolve().parent / "golden" / "moonep_tables.npz"
FIELDS = (
    "final_order", "send_token_indices", "send_route_indices", "balanced_buckets",
    "balanced_counts", "send_bucket_starts", "send_bucket_receive_offsets",
    "receive_counts_by_source_slot", "received_routes_per_slot", "received_slot_offsets",
)


def digest(a: np.ndarray) -> str:
    a = np.ascontiguousarray(a)
    return hashlib.sha256(str(a.dtype).encode() + str(a.shape).encode() + a.tobytes()).hexdigest()


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN)


def names(golden, routed=None):
    all_names = sorted({k.split("/")[0] for k in golden.files})
    if routed is None:
        return all_names
    return [n for n in all_names if (f"{n}/selected_0" in golden.files) == routed]


def test_plan_matches_the_reference(golden):
    for name in names(golden):
        tpe = torch.from_numpy(golden[f"{name}/tpe_all"])
        for dtype in (torch.int32, torch.int64):
            plan = plan_moonep_b0_b3(tpe.to(dtype).contiguous())
            assert isinstance(plan, MoonEPPlanningResult)
            np.testing.assert_array_equal(plan.alloc_cumsum.numpy(), golden[f"{name}/alloc_cumsum"])
            np.testing.assert_array_equal(plan.experts_to_copy.numpy(),
                                          golden[f"{name}/experts_to_copy"])
            assert plan.alloc_cumsum.dtype == torch.int32 and plan.alloc_cumsum.is_contiguous()
            assert plan.replica_slot_high_water == int(golden[f"{name}/high_water"])
        inverse = build_inverse_experts_to_copy(plan.experts_to_copy, tpe.shape[1])
        np.testing.assert_array_equal(inverse.numpy(), golden[f"{name}/inverse"])
        np.testing.assert_array_equal(
            experts_to_copy_from_inverse(inverse, tpe.shape[1] // tpe.shape[0]).numpy(),
            golden[f"{name}/experts_to_copy"])


def test_balanced_metadata_matches_the_reference(golden):
    for name in names(golden, routed=True):
        tpe = torch.from_numpy(golden[f"{name}/tpe_all"])
        alloc = torch.from_numpy(golden[f"{name}/alloc_cumsum"])
        inverse = torch.from_numpy(golden[f"{name}/inverse"])
        full = bool(golden[f"{name}/full"])
        for rank in range(tpe.shape[0]):
            sel = torch.from_numpy(golden[f"{name}/selected_{rank}"])
            got = build_balanced_routing_metadata(sel, tpe, alloc, inverse, rank)
            assert got.num_valid_routes == int(golden[f"{name}/r{rank}/num_valid_routes"])
            assert got.physical_slots_per_rank == 2 * got.experts_per_rank
            for f in FIELDS:
                have = getattr(got, f).numpy()
                want = golden[f"{name}/r{rank}/{f}"]
                if full:
                    assert have.dtype == want.dtype, (name, rank, f)
                    np.testing.assert_array_equal(have, want, f"{name} r{rank} {f}")
                else:
                    assert digest(have) == str(want), (name, rank, f)


def test_precomputed_expert_order_gives_the_same_tables(golden):
    name = "zipf_w4_e16_k4"
    tpe = torch.from_numpy(golden[f"{name}/tpe_all"])
    alloc = torch.from_numpy(golden[f"{name}/alloc_cumsum"])
    inverse = torch.from_numpy(golden[f"{name}/inverse"])
    for rank in range(4):
        sel = torch.from_numpy(golden[f"{name}/selected_{rank}"])
        flat = sel.reshape(-1).long()
        order = torch.argsort(flat, stable=True)
        a = build_balanced_routing_metadata(sel, tpe, alloc, inverse, rank)
        b = build_balanced_routing_metadata(sel, tpe, alloc, inverse, rank, expert_order=order,
                                            sorted_experts=flat[order], validate=False,
                                            use_direct_bucket_scatter=True)
        for f in FIELDS:
            assert torch.equal(getattr(a, f), getattr(b, f)), f
        with pytest.raises(ValueError, match="stable expert order"):
            build_balanced_routing_metadata(sel, tpe, alloc, inverse, rank,
                                            expert_order=order.flip(0), sorted_experts=flat[order])


def test_known_answers_of_the_reference_tests():
    plan = plan_moonep_b0_b3(torch.tensor([[2, 2, 0, 0], [0, 0, 2, 2]], dtype=torch.int32))
    assert plan.alloc_cumsum.tolist() == [[2, 2], [2, 2], [0, 2], [0, 2]]
    assert plan.experts_to_copy.tolist() == [[-1, -1], [-1, -1]]
    assert plan.replica_slot_high_water == 0

    tpe = torch.tensor([[4, 0, 0, 0], [4, 0, 0, 0]], dtype=torch.int64)
    plan = plan_moonep_b0_b3(tpe)
    assert plan.alloc_cumsum.tolist() == [[4, 8], [0, 0], [0, 0], [0, 0]]
    assert plan.experts_to_copy.tolist() == [[-1, -1], [0, -1]]
    assert plan.replica_slot_high_water == 1
    inverse = build_inverse_experts_to_copy(plan.experts_to_copy, 4)
    assert int(inverse[1, 0]) == 0 and int((inverse >= 0).sum()) == 1

    sel = torch.zeros((2, 2), dtype=torch.int32)
    t = [build_balanced_routing_metadata(sel, tpe, plan.alloc_cumsum, inverse, r) for r in (0, 1)]
    for r in (0, 1):
        assert t[r].balanced_counts.tolist() == [[4, 0, 0, 0, 0, 0, 0, 0], [0, 0, 0, 0, 0, 0, 4, 0]]
    assert t[0].received_slot_offsets.tolist() == [0, 4, 4, 4, 4]
    assert t[1].received_slot_offsets.tolist() == [0, 0, 0, 4, 4]
    assert t[1].balanced_buckets.tolist() == [6, 6, 6, 6]
    assert t[0].send_bucket_receive_offsets.tolist() == [0, 4, 4, 4, 0, 0, 0, 4]
    assert t[1].send_bucket_receive_offsets.tolist() == [4, 4, 4, 4, 0, 0, 0, 4]

    row = [1, 1, 1, 1, 2, 0, 0, 0, 2, 0, 0, 0, 0, 0, 0, 0]
    plan = plan_moonep_b0_b3(torch.tensor([row] * 4, dtype=torch.int32))
    assert plan.experts_to_copy[3].tolist() == [1, 0, -1, -1]
    assert plan.replica_slot_high_water == 2


@pytest.mark.parametrize("tpe, error, message", [
    (torch.zeros((2, 4), dtype=torch.float32), TypeError, "dtype"),
    (torch.zeros((4, 2), dtype=torch.int32).t(), ValueError, "contiguous"),
    (torch.zeros((2, 3), dtype=torch.int32), ValueError, "divisible"),
    (torch.tensor([[1, 0, 0, 0], [0, 0, 0, 0]], dtype=torch.int32), ValueError,
     "equal route counts"),
    (torch.tensor([[0, -1], [0, -1]], dtype=torch.int32), ValueError, "non-negative"),
    (torch.tensor([[(1 << 31) - 1, 0], [(1 << 31) - 1, 0]], dtype=torch.int64), ValueError,
     "global route count"),
    (torch.tensor([[1 << 31, 0], [1 << 31, 0]], dtype=torch.int64), ValueError,
     "each tpe_all count"),
])
def test_invalid_planner_inputs_are_rejected(tpe, error, message):
    with pytest.raises(error, match=message):
        plan_moonep_b0_b3(tpe)


def test_inverse_rejects_home_and_duplicate_experts():
    with pytest.raises(ValueError, match="remote"):
        build_inverse_experts_to_copy(torch.tensor([[0, -1], [-1, -1]], dtype=torch.int32), 4)
    with pytest.raises(ValueError, match="duplicate"):
        build_inverse_experts_to_copy(torch.tensor([[2, 2], [-1, -1]], dtype=torch.int32), 4)
    with pytest.raises(ValueError, match="invalid expert id"):
        build_inverse_experts_to_copy(torch.tensor([[9, -1], [-1, -1]], dtype=torch.int32), 4)


def test_balanced_metadata_input_contract():
    tpe = torch.tensor([[4, 0, 0, 0], [4, 0, 0, 0]], dtype=torch.int32)
    plan = plan_moonep_b0_b3(tpe)
    inverse = build_inverse_experts_to_copy(plan.experts_to_copy, 4)
    sel = torch.zeros((2, 2), dtype=torch.int32)
    with pytest.raises(ValueError, match="histogram"):
        build_balanced_routing_metadata(torch.ones((2, 2), dtype=torch.int32), tpe,
                                        plan.alloc_cumsum, inverse, 0)
    with pytest.raises(ValueError, match="monotone"):
        build_balanced_routing_metadata(sel, tpe, plan.alloc_cumsum.flip(1).contiguous(), inverse, 0)
    with pytest.raises(ValueError, match="missing its replica slot"):
        build_balanced_routing_metadata(sel, tpe, plan.alloc_cumsum, torch.full_like(inverse, -1), 0)
    with pytest.raises(ValueError, match="home experts"):
        bad = inverse.clone()
        bad[0, 0] = 0
        build_balanced_routing_metadata(sel, tpe, plan.alloc_cumsum, bad, 0)
    with pytest.raises(ValueError, match="rank must identify"):
        build_balanced_routing_metadata(sel, tpe, plan.alloc_cumsum, inverse, 2)
    with pytest.raises(TypeError, match="validate"):
        build_balanced_routing_metadata(sel, tpe, plan.alloc_cumsum, inverse, 0, validate=1)


def _plan_host(counts: np.ndarray, experts: int, total_bin: int = -1):
    world, stride = counts.shape
    epr = experts // world
    out = dict(allocation=np.empty((world, experts), np.int32),
               alloc_cumsum=np.empty((experts, world), np.int32),
               experts_to_copy=np.empty((world, epr), np.int32),
               inverse=np.empty((world, experts), np.int32),
               replica_counts=np.empty((world,), np.int32),
               plan_stats=np.zeros((4,), np.int32))
    counts = np.ascontiguousarray(counts, np.int32)
    rc = N.lib().mm_moonep_plan_host(counts.ctypes.data, stride, world, experts, total_bin,
                                     *[out[k].ctypes.data for k in out])
    return rc, out


def test_c_abi_planner_reports_a_reason_and_plans_every_expert_at_home():
    # unequal rows
    rc, out = _plan_host(np.array([[3, 0, 0, 0], [1, 0, 0, 0]]), 4)
    assert rc == 0 and out["plan_stats"][1] == 2
    assert out["alloc_cumsum"].tolist() == [[4, 4], [0, 0], [0, 0], [0, 0]]
    assert (out["experts_to_copy"] == -1).all() and (out["inverse"] == -1).all()
    # the unfiltered route count in column 4 disagrees with rank 1's histogram
    rc, out = _plan_host(np.array([[4, 0, 0, 0, 4, 0], [4, 0, 0, 0, 5, 0]]), 4, total_bin=4)
    assert rc == 0 and out["plan_stats"][1] == 3
    assert out["alloc_cumsum"].tolist() == [[8, 8], [0, 0], [0, 0], [0, 0]]
    # the same cube with matching totals is balanced: half of expert 0 moves to rank 1
    rc, out = _plan_host(np.array([[4, 0, 0, 0, 4, 0], [4, 0, 0, 0, 4, 0]]), 4, total_bin=4)
    assert rc == 0 and out["plan_stats"].tolist() == [4, 0, 1, 0]
    assert out["alloc_cumsum"].tolist() == [[4, 8], [0, 0], [0, 0], [0, 0]]
    assert out["allocation"].tolist() == [[4, 0, 0, 0], [4, 0, 0, 0]]
    assert out["replica_counts"].tolist() == [0, 1]
    # argument errors
    rc, _ = _plan_host(np.zeros((2, 3)), 3)
    assert rc == -1 and b"bad sizes" in N.lib().mm_last_error()


def test_c_abi_route_placement_counts_routes_without_a_slot():
    tpe = np.array([[4, 0, 0, 0], [4, 0, 0, 0]], np.int32)
    plan = M.plan_tables(tpe)
    inverse = np.full((2, 4), -1, np.int32)            # replica slot of expert 0 on rank 1 missing
    starts = np.zeros(8, np.int32)
    expert_start = np.zeros(4, np.int32)
    below = np.array([4, 0, 0, 0], np.int32)             # rank 1
    route_in = np.arange(4, dtype=np.int32)
    expert_in = np.zeros(4, np.int32)
    outs = [np.full(4, -1, np.int32) for _ in range(4)]
    bad = np.zeros(1, np.int32)
    rc = N.lib().mm_moonep_map_routes_host(
        route_in.ctypes.data, expert_in.ctypes.data, 4, 4, 2, 2, 4, expert_start.ctypes.data,
        below.ctypes.data, plan.alloc_cumsum.ctypes.data, inverse.ctypes.data, starts.ctypes.data,
        *[o.ctypes.data for o in outs], bad.ctypes.data)
    assert rc == 0 and bad[0] == 4 and all((o == -1).all() for o in outs)


def test_random_plans_agree_with_the_oracle():
    rng = np.random.default_rng(7)
    for world, experts, cap in ((2, 8, 31), (4, 16, 97), (8, 64, 500), (16, 64, 333), (8, 384, 4096)):
        for _ in range(6):
            skew = rng.dirichlet(np.full(experts, 0.3))
            tpe = np.stack([rng.multinomial(cap, skew) for _ in range(world)]).astype(np.int32)
            want = M.plan_tables(tpe)
            got = plan_moonep_b0_b3(torch.from_numpy(tpe))
            np.testing.assert_array_equal(got.alloc_cumsum.numpy(), want.alloc_cumsum)
            np.testing.assert_array_equal(got.experts_to_copy.numpy(), want.experts_to_copy)


def _plans(selected, experts):
    tpe = torch.stack([torch.bincount(s.reshape(-1)[(s.reshape(-1) >= 0) & (s.reshape(-1) < experts)]
                                      .long(), minlength=experts).to(torch.int32)
                       for s in selected]).contiguous()
    plan = plan_moonep_b0_b3(tpe)
    inverse = build_inverse_experts_to_copy(plan.experts_to_copy, experts)
    return tpe, plan, inverse, [build_balanced_routing_metadata(s, tpe, plan.alloc_cumsum, inverse, r)
                                for r, s in enumerate(selected)]


def test_invalid_routes_are_left_out_and_route_ids_keep_their_numbers():
    # known answer of tests/function/test_balanced_routing.py:120-152
    selected = [torch.tensor([[0, -1], [4, 0]], dtype=torch.int32),
                torch.tensor([[0, 0]], dtype=torch.int32)]
    _, _, _, plans = _plans(selected, 4)
    assert plans[0].valid_route_mask.tolist() == [True, False, False, True]
    assert plans[0].final_order.tolist() == [0, 3] and plans[0].final_order.dtype == torch.int64
    assert plans[0].send_route_indices.tolist() == [0, 3]
    assert plans[0].send_token_indices.tolist() == [0, 1]
    assert plans[0].num_valid_routes == 2 and plans[0].num_input_tokens == 2


def test_empty_input_gives_empty_tables():
    selected = [torch.empty((0, 2), dtype=torch.int32)] * 2
    _, _, _, plans = _plans(selected, 4)
    for plan in plans:
        assert plan.num_valid_routes == 0 and plan.final_order.numel() == 0
        assert plan.balanced_counts.tolist() == [[0] * 8] * 2
        assert plan.received_slot_offsets.tolist() == [0] * 5


def test_send_order_is_bucket_major_and_agrees_with_the_cube():
    # the invariants of tests/function/test_balanced_routing.py:175-212
    selected = [torch.tensor([[3, 0], [1, 0], [3, 0], [1, 0]], dtype=torch.int32),
                torch.tensor([[3, 0], [3, 0], [3, 0], [1, 0]], dtype=torch.int32)]
    _, _, _, plans = _plans(selected, 4)
    for plan in plans:
        assert torch.equal(plan.balanced_counts, plans[0].balanced_counts)
        assert bool((plan.balanced_buckets[1:] >= plan.balanced_buckets[:-1]).all())
        assert torch.equal(torch.bincount(plan.balanced_buckets.long(), minlength=8).to(torch.int32),
                           plan.balanced_counts[plan.rank])
        assert torch.sort(plan.final_order).values.tolist() == list(range(plan.num_valid_routes))
        cube = plan.balanced_counts.view(2, 2, 4).long()
        totals = cube.sum(dim=0)
        want = (totals.cumsum(dim=1) - totals + cube[:plan.rank].sum(dim=0)).reshape(-1)
        assert plan.send_bucket_receive_offsets.tolist() == want.tolist()


def test_flags_must_be_bools():
    args = (torch.tensor([[0, 1]], dtype=torch.int32), torch.tensor([[1, 1]], dtype=torch.int32),
            torch.tensor([[1], [1]], dtype=torch.int32), torch.full((1, 2), -1, dtype=torch.int32))
    with pytest.raises(TypeError, match="use_direct_bucket_scatter"):
        build_balanced_routing_metadata(*args, rank=0, use_direct_bucket_scatter=1)
    plan = build_balanced_routing_metadata(*args, rank=0)
    assert plan.balanced_buckets.tolist() == [0, 1] and plan.physical_slots_per_rank == 4


# ------------------------------------------------------------------------------------------
# world_size-2 gloo ranks: every rank plans from the gathered counts and gets the same plan
# ------------------------------------------------------------------------------------------
def _gloo_moonep_worker(rank, world, port, q):
    import os
    import torch.distributed as dist
    sys.path[:0] = [str(REPO), str(REPO / "mega-moe-td_b200")]
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    experts, tokens, top_k = 8, 40, 2
    gen = torch.Generator().manual_seed(100 + rank)
    hot = torch.zeros(tokens, 1, dtype=torch.int32)                     # every token picks expert 0
    other = torch.randint(1, experts, (tokens, 1), generator=gen, dtype=torch.int32)
    selected = torch.cat([hot, other], dim=1).contiguous()
    row = torch.bincount(selected.reshape(-1).long(), minlength=experts).to(torch.int32)
    cube = torch.zeros(world * experts, dtype=torch.int32)
    dist.all_gather_into_tensor(cube, row)
    tpe = cube.view(world, experts).contiguous()
    plan = plan_moonep_b0_b3(tpe)
    inverse = build_inverse_experts_to_copy(plan.experts_to_copy, experts)
    mine = build_balanced_routing_metadata(selected, tpe, plan.alloc_cumsum, inverse, rank)
    # the plans of all ranks are identical, and so are their views of the whole cube
    tables = torch.cat([plan.alloc_cumsum.reshape(-1), plan.experts_to_copy.reshape(-1),
                        mine.balanced_counts.reshape(-1)])
    gathered = [torch.zeros_like(tables) for _ in range(world)]
    dist.all_gather(gathered, tables)
    ok = all(torch.equal(g, tables) for g in gathered)
    # what this rank sends to rank d is what rank d expects from it
    sent = mine.balanced_counts[rank].view(world, -1)
    expect = [torch.zeros_like(mine.receive_counts_by_source_slot) for _ in range(world)]
    dist.all_gather(expect, mine.receive_counts_by_source_slot)
    ok &= all(torch.equal(sent[d], expect[d][rank]) for d in range(world))
    ok &= int(mine.received_slot_offsets[-1]) == tokens * top_k          # balanced: equal loads
    ok &= bool((plan.experts_to_copy >= 0).any())                        # a replica was needed
    q.put((rank, bool(ok)))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_derive_the_same_plan_and_matching_counts():
    import os
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    world = 2
    port = 29750 + (os.getpid() % 40)
    procs = [ctx.Process(target=_gloo_moonep_worker, args=(r, world, port, q)) for r in range(world)]
    for proc in procs:
        proc.start()
    results = dict(q.get(timeout=120) for _ in range(world))
    for proc in procs:
        proc.join(timeout=60)
        assert proc.exitcode == 0
    assert results == {0: True, 1: True}
