"""The numpy oracle of the MoonEP tables against fixtures written by the reference's own host
code (tests/golden/make_golden_moonep.py) and against the known answers of the reference's
tests (tests/function/test_moonep_planning.py:57-127, test_balanced_routing.py:69-120)."""

from __future__ import annotations

import hashlib
from pathlib import Path

import numpy as np
import pytest

from oracle import moonep_oracle as M

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


def case_names(golden, routed=None):
    names = sorted({k.split("/")[0] for k in golden.files})
    if routed is None:
        return names
    return [n for n in names if (f"{n}/selected_0" in golden.files) == routed]


def test_fixture_has_planned_and_routed_cases(golden):
    assert len(case_names(golden, routed=False)) >= 4
    assert len(case_names(golden, routed=True)) >= 12


def test_planning_tables_match_the_reference(golden):
    for name in case_names(golden):
        tpe = golden[f"{name}/tpe_all"]
        plan = M.plan_tables(tpe)
        assert plan.alloc_cumsum.dtype == np.int32 and plan.experts_to_copy.dtype == np.int32
        np.testing.assert_array_equal(plan.alloc_cumsum, golden[f"{name}/alloc_cumsum"], name)
        np.testing.assert_array_equal(plan.experts_to_copy, golden[f"{name}/experts_to_copy"], name)
        inverse = M.inverse_experts_to_copy(plan.experts_to_copy, tpe.shape[1])
        np.testing.assert_array_equal(inverse, golden[f"{name}/inverse"], name)
        assert plan.replica_slot_high_water == int(golden[f"{name}/high_water"])
        # invariants the reference's tests assert (test_moonep_planning.py:21-54)
        assert (plan.allocation >= 0).all()
        np.testing.assert_array_equal(plan.allocation.sum(axis=0), tpe.sum(axis=0))
        np.testing.assert_array_equal(plan.allocation.sum(axis=1), tpe.sum(axis=1))


def test_balanced_routing_tables_match_the_reference(golden):
    for name in case_names(golden, routed=True):
        tpe = golden[f"{name}/tpe_all"]
        full = bool(golden[f"{name}/full"])
        world = tpe.shape[0]
        for rank in range(world):
            got = M.balanced_routing_tables(golden[f"{name}/selected_{rank}"], tpe,
                                            golden[f"{name}/alloc_cumsum"],
                                            golden[f"{name}/inverse"], rank)
            assert got.num_valid_routes == int(golden[f"{name}/r{rank}/num_valid_routes"])
            for f in FIELDS:
                want = golden[f"{name}/r{rank}/{f}"]
                have = getattr(got, f)
                if full:
                    assert have.dtype == want.dtype, (name, rank, f)
                    np.testing.assert_array_equal(have, want, f"{name} r{rank} {f}")
                else:
                    assert digest(have) == str(want), (name, rank, f)


def test_receive_ranges_tile_the_receive_buffer(golden):
    """Every receive row is written by exactly one (source, route), rows of one slot are
    contiguous, and a slot holds only routes of its logical expert."""
    for name in case_names(golden, routed=True):
        if not bool(golden[f"{name}/full"]):
            continue
        tpe = golden[f"{name}/tpe_all"]
        world, experts = tpe.shape
        epr = experts // world
        etc = golden[f"{name}/experts_to_copy"]
        tables = [M.balanced_routing_tables(golden[f"{name}/selected_{r}"], tpe,
                                            golden[f"{name}/alloc_cumsum"],
                                            golden[f"{name}/inverse"], r) for r in range(world)]
        rows = M.logical_to_physical_rows(tables)
        for dest in range(world):
            offs = tables[dest].received_slot_offsets
            assert offs[-1] == tpe.sum(axis=1)[0]          # every rank ends at the common capacity
            for slot in range(2 * epr):
                logical = dest * epr + slot if slot < epr else int(etc[dest, slot - epr])
                for src, route in rows[dest][offs[slot]:offs[slot + 1]]:
                    sel = golden[f"{name}/selected_{src}"].reshape(-1)
                    assert sel[route] == logical


# ---- known answers written out in the reference's tests ---------------------------------

def test_known_answer_balanced_input_stays_home():
    plan = M.plan_tables(np.array([[2, 2, 0, 0], [0, 0, 2, 2]], np.int32))
    np.testing.assert_array_equal(plan.alloc_cumsum, [[2, 2], [2, 2], [0, 2], [0, 2]])
    np.testing.assert_array_equal(plan.experts_to_copy, np.full((2, 2), -1))
    assert plan.replica_slot_high_water == 0


def test_known_answer_hot_expert_is_split():
    plan = M.plan_tables(np.array([[4, 0, 0, 0], [4, 0, 0, 0]], np.int64))
    np.testing.assert_array_equal(plan.alloc_cumsum, [[4, 8], [0, 0], [0, 0], [0, 0]])
    np.testing.assert_array_equal(plan.experts_to_copy, [[-1, -1], [0, -1]])
    assert plan.replica_slot_high_water == 1
    inverse = M.inverse_experts_to_copy(plan.experts_to_copy, 4)
    assert inverse[1, 0] == 0 and (inverse >= 0).sum() == 1


def test_known_answer_replica_tie_takes_larger_expert_id():
    row = [1, 1, 1, 1, 2, 0, 0, 0, 2, 0, 0, 0, 0, 0, 0, 0]
    plan = M.plan_tables(np.array([row] * 4, np.int32))
    np.testing.assert_array_equal(plan.experts_to_copy[3], [1, 0, -1, -1])
    inverse = M.inverse_experts_to_copy(plan.experts_to_copy, 16)
    assert inverse[3, 1] == 0 and inverse[3, 0] == 1


def test_known_answer_hot_expert_routing():
    selected = [np.zeros((2, 2), np.int32)] * 2
    tpe = np.array([[4, 0, 0, 0], [4, 0, 0, 0]], np.int32)
    plan = M.plan_tables(tpe)
    inverse = M.inverse_experts_to_copy(plan.experts_to_copy, 4)
    t = [M.balanced_routing_tables(selected[r], tpe, plan.alloc_cumsum, inverse, r) for r in (0, 1)]
    want_counts = [[4, 0, 0, 0, 0, 0, 0, 0], [0, 0, 0, 0, 0, 0, 4, 0]]
    for r in (0, 1):
        np.testing.assert_array_equal(t[r].balanced_counts, want_counts)
    np.testing.assert_array_equal(t[0].received_routes_per_slot, [4, 0, 0, 0])
    np.testing.assert_array_equal(t[1].received_routes_per_slot, [0, 0, 4, 0])
    np.testing.assert_array_equal(t[0].received_slot_offsets, [0, 4, 4, 4, 4])
    np.testing.assert_array_equal(t[1].received_slot_offsets, [0, 0, 0, 4, 4])
    np.testing.assert_array_equal(t[0].balanced_buckets, [0, 0, 0, 0])
    np.testing.assert_array_equal(t[1].balanced_buckets, [6, 6, 6, 6])
    np.testing.assert_array_equal(t[0].send_bucket_receive_offsets, [0, 4, 4, 4, 0, 0, 0, 4])
    np.testing.assert_array_equal(t[1].send_bucket_receive_offsets, [4, 4, 4, 4, 0, 0, 0, 4])


@pytest.mark.parametrize("tpe, error, message", [
    (np.zeros((2, 4), np.float32), TypeError, "dtype"),
    (np.zeros((2, 3), np.int32), ValueError, "divisible"),
    (np.array([[1, 0, 0, 0], [0, 0, 0, 0]], np.int32), ValueError, "equal route counts"),
    (np.array([[0, -1], [0, -1]], np.int32), ValueError, "non-negative"),
    (np.array([[(1 << 31) - 1, 0], [(1 << 31) - 1, 0]], np.int64), ValueError, "global route count"),
])
def test_invalid_planner_inputs_are_rejected(tpe, error, message):
    with pytest.raises(error, match=message):
        M.plan_tables(tpe)


def test_inverse_rejects_home_and_duplicate_experts():
    with pytest.raises(ValueError, match="remote"):
        M.inverse_experts_to_copy(np.array([[0, -1], [-1, -1]], np.int32), 4)
    with pytest.raises(ValueError, match="duplicate"):
        M.inverse_experts_to_copy(np.array([[2, 2], [-1, -1]], np.int32), 4)


def test_random_dropless_counts_keep_routes_and_capacity():
    rng = np.random.default_rng(20260821)
    for _ in range(20):
        routes = rng.integers(0, 16, size=(4, 97))
        tpe = np.stack([np.bincount(r, minlength=16) for r in routes]).astype(np.int32)
        plan = M.plan_tables(tpe)
        np.testing.assert_array_equal(plan.allocation.sum(axis=0), tpe.sum(axis=0))
        np.testing.assert_array_equal(plan.allocation.sum(axis=1), tpe.sum(axis=1))
        for dest in range(4):
            remote = plan.allocation[dest].copy()
            remote[dest * 4:(dest + 1) * 4] = 0
            assert set(np.nonzero(remote)[0]) == set(plan.experts_to_copy[dest][
                plan.experts_to_copy[dest] >= 0])


def test_offset_tables_of_the_balanced_cube_are_the_balanced_tables(golden):
    """The offset formulas of the unbalanced routing, applied to the balanced cube with
    2 * E/R slots per rank, give the reference's balanced send / receive tables: the device path
    reuses its offset kernel for MoonEP on the strength of this identity."""
    from oracle import moe_oracle as O

    pairs = (("send_bucket_starts", "send_bucket_starts"),
             ("send_bucket_dst_starts", "send_bucket_receive_offsets"),
             ("recv_counts_re", "receive_counts_by_source_slot"),
             ("recv_per_expert", "received_routes_per_slot"),
             ("recv_expert_offs", "received_slot_offsets"))
    for name in case_names(golden, routed=True):
        tpe = golden[f"{name}/tpe_all"]
        world, experts = tpe.shape
        full = bool(golden[f"{name}/full"])
        cube = M.balanced_count_cube(tpe, golden[f"{name}/alloc_cumsum"], golden[f"{name}/inverse"])
        for rank in range(world):
            t = O.offset_tables_from_cube(cube, rank, 2 * experts // world)
            for mine, theirs in pairs:
                have = np.ascontiguousarray(t[mine]).astype(np.int32)
                want = golden[f"{name}/r{rank}/{theirs}"]
                if full:
                    np.testing.assert_array_equal(have, want, f"{name} r{rank} {mine}")
                else:
                    assert digest(have) == str(want), (name, rank, mine)


@pytest.mark.parametrize("world, experts, top_k, tokens, zipf", [
    (2, 8, 3, 24, 1.2), (4, 16, 4, 20, 1.2), (8, 32, 4, 12, 1.5)])
def test_forward_over_physical_slots_equals_the_logical_forward(world, experts, top_k, tokens, zipf):
    """Routing every row through the balanced tables and computing replica slots with copies of
    the home weights gives the same layer output as the forward over logical experts."""
    from oracle import moe_oracle as O

    inp = O.make_inputs(world, tokens, 64, 64, experts, top_k, seed=world,
                        expert_bias=O.zipf_expert_bias(experts, zipf))
    want = O.forward_golden(inp["hidden"], inp["routing_weights"], inp["selected"], inp["w_gate"],
                            inp["w_up"], inp["w_down"], experts)
    got, tables, plan = M.forward_over_physical_slots(
        inp["hidden"], inp["routing_weights"], inp["selected"], inp["w_gate"], inp["w_up"],
        inp["w_down"], experts)
    assert (plan.experts_to_copy >= 0).any(), "the case must exercise a replica slot"
    loads = [int(t.received_slot_offsets[-1]) for t in tables]
    assert len(set(loads)) == 1                      # every rank executes the same number of rows
    for r in range(world):
        O_ = want[r].float()
        diff = (got[r].float() - O_).abs().max().item()
        assert diff <= O.LAYOUT_ATOL + 2.0 ** -7 * O_.abs().max().item(), (r, diff)


def test_relabelled_routes_through_the_ordinary_routing_give_the_balanced_tables(golden):
    """Replace every route's logical expert by its physical bucket and run the ordinary routing
    (stable sort by expert id, count cube, offsets) with 2E experts: send order, buckets, cube
    and receive offsets are the reference's balanced tables.  MoonEP is therefore a re-labelling
    in front of the unchanged pipeline."""
    from oracle import moe_oracle as O

    for name in case_names(golden, routed=True):
        if not bool(golden[f"{name}/full"]):
            continue
        tpe = golden[f"{name}/tpe_all"]
        world, experts = tpe.shape
        relabelled = []
        for rank in range(world):
            sel = golden[f"{name}/selected_{rank}"]
            phys = np.full(sel.size, -1, np.int32)
            phys[golden[f"{name}/r{rank}/final_order"]] = golden[f"{name}/r{rank}/balanced_buckets"]
            relabelled.append(phys.reshape(sel.shape))
        if relabelled[0].size == 0:
            continue
        meta = O.routing_metadata(relabelled, 2 * experts)
        for rank in range(world):
            m = meta[rank]
            n = m["num_sent_routes"]
            assert n == int(golden[f"{name}/r{rank}/num_valid_routes"])
            np.testing.assert_array_equal(m["send_route_indices"],
                                          golden[f"{name}/r{rank}/send_route_indices"])
            np.testing.assert_array_equal(m["send_token_indices"],
                                          golden[f"{name}/r{rank}/send_token_indices"])
            np.testing.assert_array_equal(m["send_bucket"], golden[f"{name}/r{rank}/balanced_buckets"])
            np.testing.assert_array_equal(m["count_cube"][:, :2 * experts],
                                          golden[f"{name}/r{rank}/balanced_counts"])
            np.testing.assert_array_equal(m["send_bucket_dst_starts"],
                                          golden[f"{name}/r{rank}/send_bucket_receive_offsets"])
            np.testing.assert_array_equal(m["recv_expert_offs"],
                                          golden[f"{name}/r{rank}/received_slot_offsets"])
