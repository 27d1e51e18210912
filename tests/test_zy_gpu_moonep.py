"""GPU tests of the MoonEP table kernels through the C ABI: ``mm_moonep_plan``,
``mm_moonep_count_cube`` and ``mm_moonep_map_routes``, alone and chained with
``mm_route_local`` and ``mm_route_finalize`` into the balanced routing of one rank, bit-exact
against fixtures written by the reference's host planner and balanced routing
(tests/golden/make_golden_moonep.py).  All ranks of a case run one after another on one GPU;
the tables need no communication once the count cube is known.

The file sorts after the operator tests on purpose: these entry points feed no other test.
"""
from __future__ import annotations

import hashlib
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
GOLDEN = Path(__file__).resolve().parent / "golden" / "moonep_tables.npz"
I32 = dict(dtype=torch.int32, device=DEV)


def digest(a: np.ndarray) -> str:
    a = np.ascontiguousarray(a)
    return hashlib.sha256(str(a.dtype).encode() + str(a.shape).encode() + a.tobytes()).hexdigest()


@pytest.fixture(scope="module")
def tables():
    return np.load(GOLDEN)


def names(tables, routed=None):
    all_names = sorted({k.split("/")[0] for k in tables.files})
    if routed is None:
        return all_names
    return [n for n in all_names if (f"{n}/selected_0" in tables.files) == routed]


def dev(a) -> torch.Tensor:
    return torch.tensor(np.ascontiguousarray(a), **I32).contiguous()


def plan_on_device(cube: torch.Tensor, experts: int, total_bin: int = -1):
    from mega_moe.runtime.moonep_planning import launch_moonep_b0_b3
    world, stride = cube.shape
    epr = experts // world
    out = dict(allocation=torch.full((world, experts), 77, **I32),
               alloc_cumsum=torch.full((experts, world), 77, **I32),
               experts_to_copy=torch.full((world, epr), 77, **I32),
               inverse_experts_to_copy=torch.full((world, experts), 77, **I32),
               replica_counts=torch.full((world,), 77, **I32),
               plan_stats=torch.full((4,), 77, **I32))
    status = torch.zeros(8, **I32)
    launch_moonep_b0_b3(cube, world_size=world, num_experts=experts, experts_per_rank=epr,
                        row_stride=stride, total_bin=total_bin, status=status, **out)
    torch.cuda.synchronize()
    return out, status.cpu().numpy()


def test_plan_kernel_matches_the_reference(tables):
    for name in names(tables):
        tpe = tables[f"{name}/tpe_all"]
        world, experts = tpe.shape
        wide = np.zeros((world, experts + 3), np.int32)
        wide[:, :experts] = tpe
        wide[:, experts] = tpe.sum(axis=1)
        wide[:, experts + 1:] = 12345
        for counts, total_bin in ((tpe, -1), (wide, experts)):
            out, status = plan_on_device(dev(counts), experts, total_bin)
            assert status[0] == 0, (name, status)
            got = {k: v.cpu().numpy() for k, v in out.items()}
            np.testing.assert_array_equal(got["alloc_cumsum"], tables[f"{name}/alloc_cumsum"], name)
            np.testing.assert_array_equal(got["experts_to_copy"],
                                          tables[f"{name}/experts_to_copy"], name)
            np.testing.assert_array_equal(got["inverse_experts_to_copy"],
                                          tables[f"{name}/inverse"], name)
            remote = (tables[f"{name}/experts_to_copy"] >= 0).sum(axis=1)
            np.testing.assert_array_equal(got["replica_counts"], remote)
            assert got["plan_stats"].tolist() == [int(tpe.sum(axis=1)[0]), 0, int(remote.max()), 0]
            np.testing.assert_array_equal(got["allocation"].cumsum(axis=0).T, got["alloc_cumsum"])


def test_plan_kernel_equals_the_host_entry_point_on_random_counts():
    from mega_moe.runtime.moonep_planning import plan_moonep_b0_b3
    rng = np.random.default_rng(3)
    for world, experts, cap in ((2, 8, 31), (4, 16, 97), (8, 64, 500), (16, 64, 333),
                                (8, 384, 4096), (8, 896, 8192), (32, 128, 777)):
        for _ in range(3):
            skew = rng.dirichlet(np.full(experts, 0.3))
            tpe = np.stack([rng.multinomial(cap, skew) for _ in range(world)]).astype(np.int32)
            want = plan_moonep_b0_b3(torch.from_numpy(tpe))
            out, status = plan_on_device(dev(tpe), experts)
            assert status[0] == 0
            assert torch.equal(out["alloc_cumsum"].cpu(), want.alloc_cumsum)
            assert torch.equal(out["experts_to_copy"].cpu(), want.experts_to_copy)


def test_plan_kernel_rejects_and_keeps_every_expert_at_home():
    out, status = plan_on_device(dev([[3, 0, 0, 0], [1, 0, 0, 0]]), 4)
    assert status[:2].tolist() == [4, 2] and int(out["plan_stats"][1]) == 2
    assert out["alloc_cumsum"].tolist() == [[4, 4], [0, 0], [0, 0], [0, 0]]
    assert bool((out["experts_to_copy"] == -1).all())
    assert bool((out["inverse_experts_to_copy"] == -1).all())
    out, status = plan_on_device(dev([[4, 0, 0, 0, 4, 0], [4, 0, 0, 0, 5, 0]]), 4, total_bin=4)
    assert status[:2].tolist() == [4, 3]
    assert out["alloc_cumsum"].tolist() == [[8, 8], [0, 0], [0, 0], [0, 0]]


def route_local(sel: np.ndarray, experts: int, bins: int):
    from mega_moe import _native as N
    lib = N.lib()
    n = int(sel.size)
    sel_d = dev(sel) if n else torch.zeros(1, **I32)   # the entry point rejects a null pointer
    top_k = sel.shape[1]
    pad = max(n, 1)
    outs = dict(send_route=torch.full((pad,), -7, **I32), send_token=torch.full((pad,), -7, **I32),
                send_bucket=torch.full((pad,), -7, **I32),
                route_to_send=torch.full((pad,), -7, **I32),
                count_row=torch.full((bins,), -7, **I32), local_stats=torch.full((2,), -7, **I32))
    nbytes = lib.mm_route_scratch_bytes(n, bins)
    scratch = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=DEV)
    N.check(lib.mm_route_local(sel_d.data_ptr(), n, top_k, experts, bins,
                               outs["send_route"].data_ptr(), outs["send_token"].data_ptr(),
                               outs["send_bucket"].data_ptr(), outs["route_to_send"].data_ptr(),
                               outs["count_row"].data_ptr(), outs["local_stats"].data_ptr(),
                               scratch.data_ptr(), scratch.numel(), N.stream_ptr()),
            "mm_route_local")
    return outs


def finalize_tables(world: int, slots: int, capacity: int):
    nb = world * slots
    return dict(send_bucket_starts=torch.full((nb,), -7, **I32),
                send_bucket_dst_starts=torch.full((nb,), -7, **I32),
                recv_counts_re=torch.full((world * slots,), -7, **I32),
                recv_per_expert=torch.full((slots,), -7, **I32),
                recv_expert_offs=torch.zeros(slots + 1, **I32),
                recv_seg_starts=torch.full((slots * (world + 1),), -7, **I32),
                pull_dst_start=torch.full((slots * world,), -7, **I32),
                stats=torch.full((2 + world,), -7, **I32),
                mtile_group=torch.full((capacity // 128 + slots,), -7, **I32),
                mtile_row0=torch.full((capacity // 128 + slots,), -7, **I32),
                num_mtiles=torch.full((1,), -7, **I32),
                mtile2_group=torch.full((capacity // 256 + slots,), -7, **I32),
                mtile2_row0=torch.full((capacity // 256 + slots,), -7, **I32),
                num_mtiles2=torch.full((1,), -7, **I32),
                row_src_rank=torch.full((max(capacity, 1),), -7, **I32),
                row_src_pos=torch.full((max(capacity, 1),), -7, **I32),
                order_prefix=torch.full((nb + 1,), -7, **I32),
                bucket_done=torch.full((nb,), -7, **I32),
                row_arrival=torch.full((max(capacity, 1),), -7, **I32),
                arrival_row=torch.full((max(capacity, 1),), -7, **I32))


FINALIZE_ORDER = ["send_bucket_starts", "send_bucket_dst_starts", "recv_counts_re",
                  "recv_per_expert", "recv_expert_offs", "recv_seg_starts", "pull_dst_start",
                  "stats", "mtile_group", "mtile_row0", "num_mtiles", "mtile2_group",
                  "mtile2_row0", "num_mtiles2", "row_src_rank", "row_src_pos", "order_prefix",
                  "bucket_done", "row_arrival", "arrival_row"]


def balanced_rank_on_device(sel: np.ndarray, tpe: np.ndarray, rank: int):
    """mm_route_local -> mm_moonep_plan -> mm_moonep_count_cube -> mm_route_finalize ->
    mm_moonep_map_routes for one rank; the replicated count cube is uploaded instead of
    exchanged."""
    from mega_moe import _native as N
    from mega_moe.runtime.balanced_routing import launch_balanced_routing
    from mega_moe.runtime.workspace import next_power_of_2
    lib = N.lib()
    world, experts = tpe.shape
    epr = experts // world
    slots = 2 * epr
    bins = next_power_of_2(experts + 1)
    top_k = sel.shape[1]
    local = route_local(sel, experts, bins)
    cube = np.zeros((world, bins), np.int32)
    cube[:, :experts] = tpe
    cube_d = dev(cube)
    plan, status = plan_on_device(cube_d, experts)
    assert status[0] == 0
    capacity = int(tpe.sum(axis=1)[0]) + 7
    balanced_bins = next_power_of_2(world * slots)
    balanced_cube = torch.full((world, balanced_bins), 77, **I32)
    fin = finalize_tables(world, slots, capacity)
    fin_status = torch.zeros(8, **I32)

    def finalize(cube_t):
        N.check(lib.mm_route_finalize(cube_t.data_ptr(), rank, world, slots, balanced_bins,
                                      capacity, *[fin[k].data_ptr() for k in FINALIZE_ORDER],
                                      fin_status.data_ptr(), N.stream_ptr()), "mm_route_finalize")

    pad = max(sel.size, 1)
    out = dict(send_route=torch.full((pad,), -1, **I32), send_token=torch.full((pad,), -1, **I32),
               send_bucket=torch.full((pad,), -1, **I32))
    map_status = torch.zeros(8, **I32)
    launch_balanced_routing(
        count_cube=cube_d, rank=rank, world_size=world, num_experts=experts, top_k=top_k,
        alloc_cumsum=plan["alloc_cumsum"], experts_to_copy=plan["experts_to_copy"],
        inverse_experts_to_copy=plan["inverse_experts_to_copy"],
        expert_major_routes=local["send_route"], expert_major_experts=local["send_bucket"],
        local_stats=local["local_stats"], balanced_cube=balanced_cube,
        expert_start=torch.full((experts,), 77, **I32), below=torch.full((experts,), 77, **I32),
        finalize=finalize, send_bucket_starts=fin["send_bucket_starts"],
        route_to_send=local["route_to_send"], status=map_status, **out)
    torch.cuda.synchronize()
    assert fin_status.cpu()[0] == 0 and map_status.cpu()[0] == 0, (fin_status, map_status)
    n = int(local["local_stats"].cpu()[0])
    got = {k: v.cpu().numpy() for k, v in {**fin, **out}.items()}
    got["balanced_cube"] = balanced_cube.cpu().numpy()
    got["route_to_send"] = local["route_to_send"].cpu().numpy()
    return got, n


def test_balanced_routing_chain_matches_the_reference(tables):
    for name in names(tables, routed=True):
        tpe = np.ascontiguousarray(tables[f"{name}/tpe_all"], np.int32)
        world, experts = tpe.shape
        slots = 2 * (experts // world)
        full = bool(tables[f"{name}/full"])
        for rank in range(world):
            sel = tables[f"{name}/selected_{rank}"]
            got, n = balanced_rank_on_device(sel, tpe, rank)
            assert n == int(tables[f"{name}/r{rank}/num_valid_routes"])
            assert (got["balanced_cube"][:, world * slots:] == 0).all()
            have = {
                "final_order": got["send_route"][:n].astype(np.int64),
                "send_route_indices": got["send_route"][:n],
                "send_token_indices": got["send_token"][:n],
                "balanced_buckets": got["send_bucket"][:n],
                "balanced_counts": np.ascontiguousarray(got["balanced_cube"][:, :world * slots]),
                "send_bucket_starts": got["send_bucket_starts"],
                "send_bucket_receive_offsets": got["send_bucket_dst_starts"],
                "receive_counts_by_source_slot": got["recv_counts_re"].reshape(world, slots),
                "received_routes_per_slot": got["recv_per_expert"],
                "received_slot_offsets": got["recv_expert_offs"],
            }
            for f, v in have.items():
                want = tables[f"{name}/r{rank}/{f}"]
                if full:
                    np.testing.assert_array_equal(v, want, f"{name} r{rank} {f}")
                else:
                    assert digest(np.ascontiguousarray(v)) == str(want), (name, rank, f)
            # route_to_send: inverse of the new send order on the valid routes, -1 elsewhere
            if sel.size:
                r2s = got["route_to_send"][:sel.size]
                np.testing.assert_array_equal(r2s[got["send_route"][:n]], np.arange(n))
                assert (np.delete(r2s, got["send_route"][:n]) == -1).all()


def test_map_kernel_reports_routes_without_a_slot():
    from mega_moe import _native as N
    lib = N.lib()
    alloc = dev([[4, 8], [0, 0], [0, 0], [0, 0]])
    inverse = torch.full((2, 4), -1, **I32)
    outs = [torch.full((4,), -1, **I32) for _ in range(4)]
    status = torch.zeros(8, **I32)
    ins = [dev(np.arange(4)), dev(np.zeros(4)), dev([4, 0])]
    tables_ = [dev(np.zeros(4)), dev([4, 0, 0, 0]), alloc, inverse, dev(np.zeros(8))]
    N.check(lib.mm_moonep_map_routes(ins[0].data_ptr(), ins[1].data_ptr(), ins[2].data_ptr(), 4, 2,
                                     2, 4, *[t.data_ptr() for t in tables_],
                                     *[o.data_ptr() for o in outs], status.data_ptr(),
                                     N.stream_ptr()), "mm_moonep_map_routes")
    torch.cuda.synchronize()
    assert status.cpu()[:2].tolist() == [3, 1]
    assert all(bool((o == -1).all()) for o in outs)


def _replica_table(local: torch.Tensor, stride_bytes: int, nbytes: int, peers: torch.Tensor):
    from mega_moe import _native as N
    return N.ReplicaTable(local.data_ptr(), stride_bytes, nbytes, peers.data_ptr())


def _peer_pointers(tensors) -> torch.Tensor:
    return torch.tensor([t.data_ptr() for t in tensors], dtype=torch.int64, device=DEV)


@pytest.mark.parametrize("name", ["owners_w8_e64_k4", "owners_w4_e32_k6", "hot_w2_e4"])
@pytest.mark.parametrize("bytes0, bytes1, pad", [(40000, 16, 0), (16 * 1024, 0, 32),
                                                 (48, 33008, 16), (7168 * 512 * 2, 0, 0)])
def test_replica_push_matches_the_oracle(tables, name, bytes0, bytes1, pad):
    """All ranks of a case push in turn on one GPU (every peer pointer is local): each replica
    slot named by experts_to_copy holds its expert's home block, the rest is untouched."""
    import ctypes as C

    from mega_moe import _native as N
    from oracle import moonep_oracle as M

    etc_np = np.ascontiguousarray(tables[f"{name}/experts_to_copy"], np.int32)
    world, epr = etc_np.shape
    etc = dev(etc_np)
    sizes = [b for b in (bytes0, bytes1) if b]
    gen = torch.Generator().manual_seed(bytes0 + bytes1)
    home = [[torch.randint(0, 256, (epr, b + pad), dtype=torch.uint8, generator=gen).to(DEV)
             for _ in range(world)] for b in sizes]
    pools = [[torch.full((epr, b), 0xEE, dtype=torch.uint8, device=DEV) for _ in range(world)]
             for b in sizes]
    peers = [_peer_pointers(pools[t]) for t in range(len(sizes))]
    for rank in range(world):
        descs = [_replica_table(home[t][rank], sizes[t] + pad, sizes[t], peers[t])
                 for t in range(len(sizes))]
        N.check(N.lib().mm_moonep_push_replicas(
            etc.data_ptr(), rank, world, epr, C.byref(descs[0]),
            C.byref(descs[1]) if len(descs) > 1 else None, 0 if rank % 2 else 5, N.stream_ptr()),
            "mm_moonep_push_replicas")
    torch.cuda.synchronize()
    for t, b in enumerate(sizes):
        want = M.replica_pools(etc_np, [h[:, :b].cpu().numpy() for h in home[t]], 0xEE)
        for d in range(world):
            np.testing.assert_array_equal(pools[t][d].cpu().numpy(), want[d], f"table {t} rank {d}")


@pytest.mark.parametrize("name", ["owners_w8_e64_k4", "owners_w4_e32_k6", "one_home_w8_e64"])
def test_replica_pull_matches_the_oracle(tables, name):
    """Every home rank adds its experts' replica gradients onto its own: fp32, peers ascending,
    one rounding; bit-exact against the oracle."""
    import ctypes as C

    from mega_moe import _native as N
    from oracle import moonep_oracle as M

    inv_np = np.ascontiguousarray(tables[f"{name}/inverse"], np.int32)
    world, experts = inv_np.shape
    epr = experts // world
    inv = dev(inv_np)
    gen = torch.Generator().manual_seed(5)
    shapes = ((8 * 1031, 8 * 1031 + 8), (8 * 3, 8 * 3))        # elements per expert, expert stride
    home0, home, copies = [], [], []
    for n, stride in shapes:
        home0.append([torch.randn(epr, stride, generator=gen).to(torch.bfloat16) for _ in range(world)])
        copies.append([torch.randn(epr, n, generator=gen).to(torch.bfloat16).to(DEV)
                       for _ in range(world)])
        home.append([h.clone().to(DEV) for h in home0[-1]])
    peers = [_peer_pointers(copies[t]) for t in range(2)]
    for rank in range(world):
        descs = [_replica_table(home[t][rank], shapes[t][1] * 2, shapes[t][0] * 2, peers[t])
                 for t in range(2)]
        N.check(N.lib().mm_moonep_pull_replica_grads(
            inv.data_ptr(), rank, world, epr, C.byref(descs[0]), C.byref(descs[1]),
            0 if rank % 2 else 3, N.stream_ptr()), "mm_moonep_pull_replica_grads")
    torch.cuda.synchronize()
    for t, (n, stride) in enumerate(shapes):
        want = M.reduced_weight_grads(inv_np, [h[:, :n] for h in home0[t]],
                                      [c.cpu() for c in copies[t]])
        for rank in range(world):
            got = home[t][rank].cpu()
            assert torch.equal(got[:, :n].view(torch.int16), want[rank].view(torch.int16)), (t, rank)
            assert torch.equal(got[:, n:].view(torch.int16), home0[t][rank][:, n:].view(torch.int16))


def test_replica_buffers_on_one_rank():
    """World of one: the symmetric tables are allocated and the push has nothing to do."""
    from mega_moe.runtime.replica_transport import (allocate_replica_weight_buffers,
                                                    push_replica_weights)
    gate_up = torch.randn(4, 64, 128, device=DEV).to(torch.bfloat16)
    down = torch.randn(4, 64, 64, device=DEV).to(torch.bfloat16)
    buffers = allocate_replica_weight_buffers(gate_up, down, rank=0, world_size=1)
    try:
        assert buffers.gate_up.shape == gate_up.shape and buffers.down.shape == down.shape
        buffers.gate_up.fill_(1.0)
        etc = torch.full((1, 4), -1, **I32)
        push_replica_weights(etc, gate_up, down, buffers, rank=0, world_size=1)
        torch.cuda.synchronize()
        assert bool((buffers.gate_up == 1.0).all())
    finally:
        buffers.free()


def test_relabelled_routes_through_the_ordinary_routing_match_the_reference(tables):
    """MoonEP as a re-labelling, on the device: mm_route_local -> mm_moonep_plan ->
    mm_moonep_count_cube -> mm_moonep_relabel_routes, then the ordinary routing of a layer with
    2E experts on the relabelled ids (mm_route_local again, mm_route_finalize on the gathered
    count rows): send order, buckets, count cube and offsets are the reference's balanced
    tables."""
    from mega_moe import _native as N
    from mega_moe.runtime.balanced_routing import launch_physical_relabel
    from mega_moe.runtime.workspace import next_power_of_2
    lib = N.lib()
    for name in names(tables, routed=True):
        tpe = np.ascontiguousarray(tables[f"{name}/tpe_all"], np.int32)
        world, experts = tpe.shape
        slots = 2 * (experts // world)
        full = bool(tables[f"{name}/full"])
        if tables[f"{name}/selected_0"].size == 0:
            continue
        bins = next_power_of_2(experts + 1)
        cube = np.zeros((world, bins), np.int32)
        cube[:, :experts] = tpe
        cube_d = dev(cube)
        plan, status = plan_on_device(cube_d, experts)
        assert status[0] == 0
        phys_bins = next_power_of_2(2 * experts)
        second, rows = [], []
        for rank in range(world):
            sel = tables[f"{name}/selected_{rank}"]
            local = route_local(sel, experts, bins)
            physical = torch.full((sel.size,), 77, **I32)
            relabel_status = torch.zeros(8, **I32)
            launch_physical_relabel(
                count_cube=cube_d, rank=rank, world_size=world, num_experts=experts,
                alloc_cumsum=plan["alloc_cumsum"], experts_to_copy=plan["experts_to_copy"],
                inverse_experts_to_copy=plan["inverse_experts_to_copy"],
                expert_major_routes=local["send_route"], expert_major_experts=local["send_bucket"],
                route_to_send=local["route_to_send"], local_stats=local["local_stats"],
                balanced_cube=torch.full((world, phys_bins), 77, **I32),
                expert_start=torch.full((experts,), 77, **I32),
                below=torch.full((experts,), 77, **I32), physical=physical, status=relabel_status)
            torch.cuda.synchronize()
            assert relabel_status.cpu()[0] == 0
            want = np.full(sel.size, -1, np.int32)
            if full:
                want[tables[f"{name}/r{rank}/final_order"]] = tables[f"{name}/r{rank}/balanced_buckets"]
                np.testing.assert_array_equal(physical.cpu().numpy(), want, f"{name} r{rank}")
            # the ordinary routing of 2E experts on the relabelled ids
            again = route_local(physical.cpu().numpy().reshape(sel.shape), 2 * experts, phys_bins)
            torch.cuda.synchronize()
            second.append({k: v.cpu().numpy() for k, v in again.items()})
            rows.append(second[-1]["count_row"])
        gathered = dev(np.stack(rows))
        capacity = int(tpe.sum(axis=1)[0]) + 7
        for rank in range(world):
            fin = finalize_tables(world, slots, capacity)
            fin_status = torch.zeros(8, **I32)
            N.check(lib.mm_route_finalize(gathered.data_ptr(), rank, world, slots, phys_bins,
                                          capacity, *[fin[k].data_ptr() for k in FINALIZE_ORDER],
                                          fin_status.data_ptr(), N.stream_ptr()), "mm_route_finalize")
            torch.cuda.synchronize()
            assert fin_status.cpu()[0] == 0
            n = int(second[rank]["local_stats"][0])
            have = {
                "send_route_indices": second[rank]["send_route"][:n],
                "send_token_indices": second[rank]["send_token"][:n],
                "balanced_buckets": second[rank]["send_bucket"][:n],
                "balanced_counts": np.ascontiguousarray(np.stack(rows)[:, :world * slots]),
                "send_bucket_starts": fin["send_bucket_starts"].cpu().numpy(),
                "send_bucket_receive_offsets": fin["send_bucket_dst_starts"].cpu().numpy(),
                "received_slot_offsets": fin["recv_expert_offs"].cpu().numpy(),
            }
            for f, v in have.items():
                want = tables[f"{name}/r{rank}/{f}"]
                if full:
                    np.testing.assert_array_equal(v, want, f"{name} r{rank} {f}")
                else:
                    assert digest(np.ascontiguousarray(v)) == str(want), (name, rank, f)
