"""The text of the MoonEP device kernels (mega-moe-td_b200/csrc/moonep_kernels.cuh) executed on
the host: g++ compiles it against tests/cuda_on_threads/cuda_on_threads.h, which runs every CUDA
thread as a host thread with real block and warp barriers and warp shuffles.  The results must
equal the fixtures written by the reference's host planner and balanced routing.  This checks
the kernels' indexing, phase order, warp reductions and scans; the GPU tests check the same
entry points on the device.  With MOE_TEST_SANITIZE=1 (see cuda_on_threads/host_build.py) the
kernels run under AddressSanitizer."""

from __future__ import annotations

import ctypes as C
import hashlib
import sys
from pathlib import Path

import numpy as np
import pytest

REPO = Path(__file__).resolve().parent.parent
HERE = Path(__file__).resolve().parent
GOLDEN = HERE / "golden" / "moonep_tables.npz"
sys.path.insert(0, str(HERE))


def digest(a: np.ndarray) -> str:
    a = np.ascontiguousarray(a)
    return hashlib.sha256(str(a.dtype).encode() + str(a.shape).encode() + a.tobytes()).hexdigest()


@pytest.fixture(scope="module")
def kernels(tmp_path_factory):
    from cuda_on_threads.host_build import compile_for_host
    out = compile_for_host(HERE / "cuda_on_threads" / "moonep_kernels_on_threads.cpp",
                           tmp_path_factory.mktemp("cuda_on_threads") / "libmoonep_on_threads.so",
                           [REPO / "mega-moe-td_b200" / "csrc"])
    lib = C.CDLL(str(out))
    for name in ("cot_moonep_plan", "cot_moonep_count_cube", "cot_moonep_map_routes"):
        getattr(lib, name).restype = None
    table = [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]
    for name in ("cot_moonep_push_replicas", "cot_moonep_pull_replica_grads"):
        getattr(lib, name).restype = None
        getattr(lib, name).argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int] + table + table + [C.c_int]
    return lib


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN)


def p(a):
    return C.c_void_p(a.ctypes.data)


def run_plan(lib, counts: np.ndarray, experts: int, total_bin: int = -1):
    counts = np.ascontiguousarray(counts, np.int32)
    world, stride = counts.shape
    epr = experts // world
    out = dict(allocation=np.full((world, experts), 77, np.int32),
               alloc_cumsum=np.full((experts, world), 77, np.int32),
               experts_to_copy=np.full((world, epr), 77, np.int32),
               inverse=np.full((world, experts), 77, np.int32),
               replica_counts=np.full((world,), 77, np.int32),
               plan_stats=np.full((4,), 77, np.int32))
    status = np.zeros(8, np.int32)
    lib.cot_moonep_plan(p(counts), stride, world, experts, total_bin,
                        *[p(out[k]) for k in out], p(status))
    out["status"] = status
    return out


def names(golden, routed=None):
    all_names = sorted({k.split("/")[0] for k in golden.files})
    if routed is None:
        return all_names
    return [n for n in all_names if (f"{n}/selected_0" in golden.files) == routed]


def test_plan_kernel_matches_the_reference(kernels, golden):
    for name in names(golden):
        tpe = golden[f"{name}/tpe_all"]
        world, experts = tpe.shape
        # a wider cube with the unfiltered totals in the column after the experts, as the
        # count exchange delivers it
        cube = np.zeros((world, experts + 3), np.int32)
        cube[:, :experts] = tpe
        cube[:, experts] = tpe.sum(axis=1)
        cube[:, experts + 1:] = 12345
        for counts, total_bin in ((tpe, -1), (cube, experts)):
            out = run_plan(kernels, counts, experts, total_bin)
            assert out["status"][0] == 0, name
            np.testing.assert_array_equal(out["alloc_cumsum"], golden[f"{name}/alloc_cumsum"], name)
            np.testing.assert_array_equal(out["experts_to_copy"],
                                          golden[f"{name}/experts_to_copy"], name)
            np.testing.assert_array_equal(out["inverse"], golden[f"{name}/inverse"], name)
            remote = (golden[f"{name}/experts_to_copy"] >= 0).sum(axis=1)
            np.testing.assert_array_equal(out["replica_counts"], remote)
            assert out["plan_stats"].tolist() == [int(tpe.sum(axis=1)[0]), 0, int(remote.max()), 0]
            np.testing.assert_array_equal(out["allocation"].cumsum(axis=0).T, out["alloc_cumsum"])


def test_plan_kernel_rejects_and_keeps_every_expert_at_home(kernels):
    out = run_plan(kernels, np.array([[3, 0, 0, 0], [1, 0, 0, 0]]), 4)
    assert out["status"][:2].tolist() == [4, 2] and out["plan_stats"][1] == 2
    assert out["alloc_cumsum"].tolist() == [[4, 4], [0, 0], [0, 0], [0, 0]]
    assert (out["experts_to_copy"] == -1).all() and (out["inverse"] == -1).all()
    out = run_plan(kernels, np.array([[4, 0, 0, 0, 4, 0], [4, 0, 0, 0, 5, 0]]), 4, total_bin=4)
    assert out["status"][:2].tolist() == [4, 3]
    assert out["alloc_cumsum"].tolist() == [[8, 8], [0, 0], [0, 0], [0, 0]]
    out = run_plan(kernels, np.array([[4, -1, 0, 1], [4, 0, 0, 0]]), 4)
    assert out["status"][:2].tolist() == [4, 1]


def expert_major(selected: np.ndarray, experts: int):
    flat = selected.reshape(-1).astype(np.int64)
    ids = np.nonzero((flat >= 0) & (flat < experts))[0]
    order = np.argsort(flat[ids], kind="stable")
    return ids[order].astype(np.int32), flat[ids][order].astype(np.int32)


def test_cube_and_map_kernels_match_the_reference(kernels, golden):
    for name in names(golden, routed=True):
        tpe = np.ascontiguousarray(golden[f"{name}/tpe_all"], np.int32)
        alloc = np.ascontiguousarray(golden[f"{name}/alloc_cumsum"], np.int32)
        etc = np.ascontiguousarray(golden[f"{name}/experts_to_copy"], np.int32)
        inverse = np.ascontiguousarray(golden[f"{name}/inverse"], np.int32)
        full = bool(golden[f"{name}/full"])
        world, experts = tpe.shape
        buckets = 2 * experts
        stride = buckets + 5
        for rank in range(world):
            sel = golden[f"{name}/selected_{rank}"]
            top_k = sel.shape[1]
            cube = np.full((world, stride), 77, np.int32)
            expert_start = np.full(experts, 77, np.int32)
            below = np.full(experts, 77, np.int32)
            kernels.cot_moonep_count_cube(p(tpe), experts, rank, world, experts, p(alloc), p(etc),
                                          p(cube), stride, p(expert_start), p(below))
            assert (cube[:, buckets:] == 0).all()
            np.testing.assert_array_equal(expert_start, tpe[rank].cumsum() - tpe[rank])
            np.testing.assert_array_equal(below, tpe[:rank].sum(axis=0))
            route_in, expert_in = expert_major(sel, experts)
            n, num_routes = route_in.size, sel.size
            own = cube[rank, :buckets].astype(np.int64)
            starts = (own.cumsum() - own).astype(np.int32)
            # the device tables are sized for every route; only the valid prefix is written
            pad = max(num_routes, 1)
            route_pad = np.full(pad, -1, np.int32)
            route_pad[:n] = route_in
            expert_pad = np.full(pad, -1, np.int32)
            expert_pad[:n] = expert_in
            outs = [np.full(pad, -1, np.int32) for _ in range(4)]
            stats = np.array([n, 0], np.int32)
            status = np.zeros(8, np.int32)
            kernels.cot_moonep_map_routes(p(route_pad), p(expert_pad), p(stats), num_routes, top_k,
                                          world, experts, p(expert_start), p(below), p(alloc),
                                          p(inverse), p(starts), *[p(o) for o in outs], p(status))
            assert status[0] == 0, (name, rank, status)
            send_route, send_token, send_bucket, route_to_send = outs
            assert (send_route[n:] == -1).all()
            have = {
                "final_order": send_route[:n].astype(np.int64),
                "send_route_indices": send_route[:n],
                "send_token_indices": send_token[:n],
                "balanced_buckets": send_bucket[:n],
                "balanced_counts": np.ascontiguousarray(cube[:, :buckets]),
                "send_bucket_starts": starts,
            }
            for f, v in have.items():
                want = golden[f"{name}/r{rank}/{f}"]
                if full:
                    np.testing.assert_array_equal(v, want, f"{name} r{rank} {f}")
                else:
                    assert digest(v) == str(want), (name, rank, f)
            # route_to_send is the inverse permutation of send_route on the valid routes
            np.testing.assert_array_equal(route_to_send[send_route[:n]], np.arange(n))
            assert (np.delete(route_to_send, send_route[:n]) == -1).all()


def test_map_kernel_reports_routes_without_a_slot(kernels):
    alloc = np.array([[4, 8], [0, 0], [0, 0], [0, 0]], np.int32)
    inverse = np.full((2, 4), -1, np.int32)
    ins = [np.arange(4, dtype=np.int32), np.zeros(4, np.int32), np.array([4, 0], np.int32)]
    tables = [np.zeros(4, np.int32), np.array([4, 0, 0, 0], np.int32), alloc, inverse,
              np.zeros(8, np.int32)]
    outs = [np.full(4, -1, np.int32) for _ in range(4)]
    status = np.zeros(8, np.int32)
    kernels.cot_moonep_map_routes(p(ins[0]), p(ins[1]), p(ins[2]), 4, 2, 2, 4,
                                  *[p(t) for t in tables], *[p(o) for o in outs], p(status))
    assert status[0] == 3 and status[1] == 1
    assert all((o == -1).all() for o in outs)


def _pointer_table(arrays):
    table = (C.c_void_p * len(arrays))(*[a.ctypes.data for a in arrays])
    return table


@pytest.mark.parametrize("name", ["owners_w8_e64_k4", "owners_w4_e32_k6", "hot_w2_e4"])
@pytest.mark.parametrize("bytes0, bytes1, pad", [(40000, 16, 0), (16 * 1024, 0, 32), (48, 33008, 16)])
def test_replica_push_kernel(kernels, golden, name, bytes0, bytes1, pad):
    """Every rank pushes the experts it owns into the replica slots experts_to_copy names; empty
    slots and bytes outside the tables stay as they were."""
    from oracle import moonep_oracle as M

    etc = np.ascontiguousarray(golden[f"{name}/experts_to_copy"], np.int32)
    world, epr = etc.shape
    rng = np.random.default_rng(bytes0 + bytes1)
    sizes = [b for b in (bytes0, bytes1) if b]
    home = [[rng.integers(0, 256, size=(epr, b + pad), dtype=np.uint8) for _ in range(world)]
            for b in sizes]
    pools = [[np.full((epr, b), 0xEE, np.uint8) for _ in range(world)] for b in sizes]
    tables = [_pointer_table(pools[t]) for t in range(len(sizes))]
    for rank in range(world):
        args = []
        for t in range(2):
            if t < len(sizes):
                args += [p(home[t][rank]), sizes[t] + pad, sizes[t], tables[t]]
            else:
                args += [None, 0, 0, None]
        kernels.cot_moonep_push_replicas(p(etc), rank, world, epr, *args, 5)
    for t, b in enumerate(sizes):
        want = M.replica_pools(etc, [h[:, :b] for h in home[t]], 0xEE)
        for d in range(world):
            np.testing.assert_array_equal(pools[t][d], want[d], f"table {t} rank {d}")
    assert (etc >= 0).any()


@pytest.mark.parametrize("name", ["owners_w8_e64_k4", "owners_w4_e32_k6", "one_home_w8_e64"])
def test_replica_pull_kernel(kernels, golden, name):
    """Every home rank adds the gradients of its experts' copies onto its own, fp32, peers in
    ascending order, one rounding; experts without copies and other ranks' tables stay as they
    were."""
    import torch

    from oracle import moonep_oracle as M

    inverse = np.ascontiguousarray(golden[f"{name}/inverse"], np.int32)
    world, experts = inverse.shape
    epr = experts // world
    gen = torch.Generator().manual_seed(5)
    n0, n1 = 8 * 1031, 8 * 3                     # bf16 elements per expert (16-byte multiples)
    stride0 = n0 + 8                             # the home table may be strided
    home, copies, home_np, copies_np = [], [], [], []
    for n, stride in ((n0, stride0), (n1, n1)):
        home.append([torch.randn(epr, stride, generator=gen).to(torch.bfloat16) for _ in range(world)])
        copies.append([torch.randn(epr, n, generator=gen).to(torch.bfloat16) for _ in range(world)])
        home_np.append([h.view(torch.int16).numpy().copy() for h in home[-1]])
        copies_np.append([c.view(torch.int16).numpy().copy() for c in copies[-1]])
    tables = [_pointer_table(copies_np[t]) for t in range(2)]
    for rank in range(world):
        kernels.cot_moonep_pull_replica_grads(
            p(inverse), rank, world, epr,
            p(home_np[0][rank]), stride0 * 2, n0 * 2, tables[0],
            p(home_np[1][rank]), n1 * 2, n1 * 2, tables[1], 3)
    touched = 0
    for t, (n, stride) in enumerate(((n0, stride0), (n1, n1))):
        want = M.reduced_weight_grads(inverse, [h[:, :n] for h in home[t]], copies[t])
        for rank in range(world):
            got = torch.from_numpy(home_np[t][rank]).view(torch.bfloat16)
            assert torch.equal(got[:, :n].view(torch.int16), want[rank].view(torch.int16)), (t, rank)
            assert torch.equal(got[:, n:].view(torch.int16), home[t][rank][:, n:].view(torch.int16))
            assert np.array_equal(copies_np[t][rank], copies[t][rank].view(torch.int16).numpy())
            touched += int((got[:, :n].view(torch.int16) != home[t][rank][:, :n].view(torch.int16))
                           .any(dim=1).sum())
    assert touched > 0


def test_relabel_kernel_gives_every_route_its_bucket(kernels, golden):
    for name in names(golden, routed=True):
        if not bool(golden[f"{name}/full"]):
            continue
        tpe = np.ascontiguousarray(golden[f"{name}/tpe_all"], np.int32)
        alloc = np.ascontiguousarray(golden[f"{name}/alloc_cumsum"], np.int32)
        inverse = np.ascontiguousarray(golden[f"{name}/inverse"], np.int32)
        world, experts = tpe.shape
        for rank in range(world):
            sel = golden[f"{name}/selected_{rank}"]
            if sel.size == 0:
                continue
            route_in, expert_in = expert_major(sel, experts)
            n = route_in.size
            pad = sel.size
            route_pad = np.full(pad, -1, np.int32)
            route_pad[:n] = route_in
            expert_pad = np.full(pad, -1, np.int32)
            expert_pad[:n] = expert_in
            route_to_send = np.full(pad, -1, np.int32)
            route_to_send[route_in] = np.arange(n)
            expert_start = (tpe[rank].cumsum() - tpe[rank]).astype(np.int32)
            below = tpe[:rank].sum(axis=0).astype(np.int32)
            physical = np.full(pad, 77, np.int32)
            stats = np.array([n, 0], np.int32)
            status = np.zeros(8, np.int32)
            kernels.cot_moonep_relabel_routes(p(route_pad), p(expert_pad), p(route_to_send),
                                              p(stats), pad, world, experts, p(expert_start),
                                              p(below), p(alloc), p(inverse), p(physical), p(status))
            assert status[0] == 0
            want = np.full(pad, -1, np.int32)
            want[golden[f"{name}/r{rank}/final_order"]] = golden[f"{name}/r{rank}/balanced_buckets"]
            np.testing.assert_array_equal(physical, want, f"{name} r{rank}")
