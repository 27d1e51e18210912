"""The routing kernels of mega-moe-td_b200/csrc/routing.cu executed on the host from their own
source text: everything inside ``namespace mm`` of the file (filter + stable sort, offset
tables, row tables, router top-k) is cut out, compiled by g++ against
tests/cuda_on_threads/cuda_on_threads.h and launched with the grids and shared-memory sizes the
host entry points use.  The one textual change is the declaration form of dynamic shared memory
(``extern __shared__ T name[];`` becomes a pointer to the launch's buffer).

The GPU suite checks the same kernels bit-exactly on a B200; this file adds shapes the GPU suite
does not have (up to 4096 buckets, 64 ranks, the 2 * E/R slots per rank of MoonEP with most
groups empty, overflow far past the capacity) and, with MOE_TEST_SANITIZE=1, bounds checking of
every access (see cuda_on_threads/host_build.py)."""

from __future__ import annotations

import ctypes as C
import re
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

REPO = Path(__file__).resolve().parent.parent
HERE = Path(__file__).resolve().parent
CSRC = REPO / "mega-moe-td_b200" / "csrc"
sys.path.insert(0, str(HERE))

from oracle import moe_oracle as O  # noqa: E402

PRELUDE = r"""
#include <math.h>
#include <limits.h>
#include "cuda_on_threads.h"

namespace mm {
// what routing.cu takes from common.cuh on the device
struct StatusRecord {
  int32_t code, site, slot, want, seen, block, pad[2];
};
enum StatusCode : int32_t { kOk = 0, kWaitTimeout = 1, kCapacityOverflow = 2, kBadIndex = 3 };
inline void report_status(StatusRecord* st, int32_t code, int32_t site, int32_t slot,
                          int32_t want, int32_t seen) {
  if (st == nullptr) return;
  if (atomicCAS(&st->code, 0, code) == 0) {
    st->site = site;
    st->slot = slot;
    st->want = want;
    st->seen = seen;
    st->block = (int32_t)blockIdx.x;
    __threadfence();
  }
}
%(order_bucket)s
}  // namespace mm
"""

LAUNCHERS = r"""
using namespace mm;

extern "C" {

// launch sequence of mm_route_local
void cot_route_local(const int32_t* selected, int n, int top_k, int num_experts, int bins,
                     int32_t* send_route, int32_t* send_token, int32_t* send_bucket,
                     int32_t* route_to_send, int32_t* count_row, int32_t* local_stats,
                     int32_t* scratch) {
  const int nblk = (n + kRouteChunk - 1) / kRouteChunk;
  int32_t* block_hist = scratch;
  int32_t* bucket_start = block_hist + (size_t)nblk * bins;
  if (nblk > 0)
    cot::launch(nblk, kRouteThreads,
                [=] { route_hist_kernel(selected, n, num_experts, bins, block_hist); },
                bins * sizeof(int32_t));
  cot::launch(1, 1024,
              [=] { route_scan_kernel(block_hist, nblk, bins, bucket_start, count_row, local_stats); },
              bins * sizeof(int32_t));
  if (nblk > 0)
    cot::launch(nblk, kRouteThreads,
                [=] {
                  route_scatter_kernel(selected, n, top_k, num_experts, bins, block_hist,
                                       bucket_start, send_route, send_token, send_bucket,
                                       route_to_send);
                },
                (kRouteWarps + 1) * bins * sizeof(int32_t));
}

// launch sequence of mm_route_finalize
void cot_route_finalize(const int32_t* cube, int rank, int world, int epr, int bins, int capacity,
                        int32_t** t, void* status) {
  const int nb = world * epr;
  cot::launch(1, 1024,
              [=] {
                route_finalize_kernel(cube, rank, world, epr, bins, capacity, t[0], t[1], t[2],
                                      t[3], t[4], t[5], t[6], t[7], t[8], t[9], t[10], t[11],
                                      t[12], t[13], t[16], t[17], static_cast<StatusRecord*>(status));
              },
              (size_t)(3 * nb + epr + 1) * sizeof(int32_t));
  const int blocks = (nb + 7) / 8;
  cot::launch(blocks, 256,
              [=] {
                route_row_tables_kernel(t[4], t[5], t[6], t[2], world, epr, capacity, t[14], t[15],
                                        t[18], t[19]);
              },
              world * sizeof(int32_t));
}

void cot_router_topk(const float* logits, int64_t ld, int tokens, int experts, int top_k,
                     int32_t* selected, float* weights) {
  const int blocks = (tokens + kRouterWarps - 1) / kRouterWarps;
  cot::launch(blocks, 32 * kRouterWarps,
              [=] { router_topk_kernel(logits, ld, tokens, experts, top_k, selected, weights); });
}

}  // extern "C"
"""

FINALIZE_ORDER = ["send_bucket_starts", "send_bucket_dst_starts", "recv_counts_re",
                  "recv_per_expert", "recv_expert_offs", "recv_seg_starts", "pull_dst_start",
                  "stats", "mtile_group", "mtile_row0", "num_mtiles", "mtile2_group",
                  "mtile2_row0", "num_mtiles2", "row_src_rank", "row_src_pos", "order_prefix",
                  "bucket_done", "row_arrival", "arrival_row"]


def cut(text: str, start: str, end: str = "\n}\n") -> str:
    i = text.index(start)
    i = text.rfind("\n", 0, i) + 1
    j = text.index(end, i) + len(end)
    return text[i:j]


@pytest.fixture(scope="module")
def kernels(tmp_path_factory):
    from cuda_on_threads.host_build import compile_for_host
    routing = (CSRC / "routing.cu").read_text()
    common = (CSRC / "common.cuh").read_text()
    body = routing[routing.index("namespace mm {"):routing.index("}  // namespace mm") +
                   len("}  // namespace mm")]
    body, n = re.subn(r"extern __shared__ (\w+) (\w+)\[\];",
                      r"\1* \2 = reinterpret_cast<\1*>(::cot::dynamic_shared());", body)
    assert n >= 4
    src = (PRELUDE % dict(order_bucket=cut(common, "int32_t dispatch_order_bucket("))
           + body + "\n" + LAUNCHERS)
    d = tmp_path_factory.mktemp("routing_on_threads")
    (d / "routing_on_threads.cpp").write_text(src)
    lib = C.CDLL(str(compile_for_host(d / "routing_on_threads.cpp", d / "librouting.so")))
    for name in ("cot_route_local", "cot_route_finalize", "cot_router_topk"):
        getattr(lib, name).restype = None
    lib.cot_router_topk.argtypes = [C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_void_p,
                                    C.c_void_p]
    return lib


def p(a):
    return C.c_void_p(a.ctypes.data)


def next_pow2(n):
    return 1 if n <= 1 else 1 << (n - 1).bit_length()


def route_local(lib, sel: np.ndarray, experts: int, bins: int):
    sel = np.ascontiguousarray(sel, np.int32)
    n, top_k = sel.size, sel.shape[1]
    pad = max(n, 1)
    outs = {k: np.full(pad, -7, np.int32) for k in ("send_route", "send_token", "send_bucket",
                                                   "route_to_send")}
    outs["count_row"] = np.full(bins, -7, np.int32)
    outs["local_stats"] = np.full(2, -7, np.int32)
    nblk = (n + 2047) // 2048
    scratch = np.full((nblk + 1) * bins, -7, np.int32)        # exactly mm_route_scratch_bytes
    flat = sel.reshape(-1) if n else np.zeros(1, np.int32)
    lib.cot_route_local(p(flat), n, top_k, experts, bins, p(outs["send_route"]),
                        p(outs["send_token"]), p(outs["send_bucket"]), p(outs["route_to_send"]),
                        p(outs["count_row"]), p(outs["local_stats"]), p(scratch))
    return outs


def finalize(lib, cube: np.ndarray, rank, world, epr, bins, capacity):
    nb = world * epr
    sizes = dict(send_bucket_starts=nb, send_bucket_dst_starts=nb, recv_counts_re=world * epr,
                 recv_per_expert=epr, recv_expert_offs=epr + 1, recv_seg_starts=epr * (world + 1),
                 pull_dst_start=epr * world, stats=2 + world,
                 mtile_group=capacity // 128 + epr, mtile_row0=capacity // 128 + epr, num_mtiles=1,
                 mtile2_group=capacity // 256 + epr, mtile2_row0=capacity // 256 + epr,
                 num_mtiles2=1, row_src_rank=max(capacity, 1), row_src_pos=max(capacity, 1),
                 order_prefix=nb + 1, bucket_done=nb, row_arrival=max(capacity, 1),
                 arrival_row=max(capacity, 1))
    t = {k: np.full(sizes[k], -7, np.int32) for k in FINALIZE_ORDER}      # documented sizes, no slack
    t["recv_expert_offs"][:] = 0
    table = (C.c_void_p * 20)(*[t[k].ctypes.data for k in FINALIZE_ORDER])
    status = np.zeros(8, np.int32)
    cube = np.ascontiguousarray(cube, np.int32)
    lib.cot_route_finalize(p(cube), rank, world, epr, bins, capacity, table, p(status))
    return t, status


def check_finalize(got, status, want, cube, rank, world, epr):
    assert status[0] == 0
    for k in ("send_bucket_starts", "send_bucket_dst_starts", "recv_per_expert",
              "recv_expert_offs", "pull_dst_start", "stats"):
        np.testing.assert_array_equal(got[k], np.asarray(want[k]).reshape(-1), err_msg=k)
    np.testing.assert_array_equal(got["recv_counts_re"], np.asarray(want["recv_counts_re"]).reshape(-1))
    np.testing.assert_array_equal(got["recv_seg_starts"], np.asarray(want["recv_seg_starts"]).reshape(-1))
    m = want["num_received_routes"]
    np.testing.assert_array_equal(got["row_src_rank"][:m], want["row_src_rank"])
    np.testing.assert_array_equal(got["row_src_pos"][:m], want["row_src_pos"])
    for rows, gk, rk, nk in ((128, "mtile_group", "mtile_row0", "num_mtiles"),
                             (256, "mtile2_group", "mtile2_row0", "num_mtiles2")):
        groups, row0 = [], []
        for e in range(epr):
            for r0 in range(0, int(want["recv_per_expert"][e]), rows):
                groups.append(e)
                row0.append(int(want["recv_expert_offs"][e]) + r0)
        nt = int(got[nk][0])
        assert nt == len(groups)
        np.testing.assert_array_equal(got[gk][:nt], groups)
        np.testing.assert_array_equal(got[rk][:nt], row0)
    order = [((rank + 1 + dd) % world) * epr + le for le in range(epr) for dd in range(world)]
    np.testing.assert_array_equal(got["order_prefix"],
                                  np.r_[0, np.cumsum(np.asarray(cube)[rank, :world * epr][order])])
    assert (got["bucket_done"] == 0).all()
    # arrival permutation: source-major order of an all-to-all against the expert-major rows
    perm = O.arrival_to_slot_permutation(np.asarray(want["recv_counts_re"]),
                                         np.asarray(want["recv_expert_offs"])[:-1])
    np.testing.assert_array_equal(got["row_arrival"][:m], perm)
    np.testing.assert_array_equal(got["arrival_row"][:m][perm], np.arange(m))


ROUTE_CASES = [  # tokens, top_k, experts, world, drop share
    (64, 2, 8, 1, 0.0), (300, 3, 24, 4, 0.3), (1100, 8, 128, 2, 0.05), (700, 4, 32, 8, 1.0),
    (1, 1, 4, 2, 0.0), (520, 16, 896, 8, 0.0), (260, 8, 4096, 64, 0.1), (90, 5, 1536, 3, 0.0),
    (2049, 1, 2, 2, 0.5),
]


@pytest.mark.parametrize("tokens, top_k, experts, world, drop", ROUTE_CASES)
def test_routing_metadata_bit_exact(kernels, tokens, top_k, experts, world, drop):
    rng = np.random.default_rng(tokens + experts)
    epr = experts // world
    bins = next_pow2(experts)
    sels = []
    for _ in range(world):
        s = rng.integers(0, experts, size=(tokens, top_k)).astype(np.int32)
        if drop > 0:
            bad = rng.random((tokens, top_k)) < drop
            s[bad] = rng.choice([-1, experts, experts + 5], size=int(bad.sum()))
        sels.append(s)
    meta = O.routing_metadata(sels, experts)
    some_ranks = sorted({0, world // 2, world - 1}) if experts < 1024 else [world - 1]
    for r in some_ranks:
        got = route_local(kernels, sels[r], experts, bins)
        want = meta[r]
        n = want["num_sent_routes"]
        assert got["local_stats"].tolist() == [n, 0]
        np.testing.assert_array_equal(got["send_route"][:n], want["send_route_indices"])
        np.testing.assert_array_equal(got["send_token"][:n], want["send_token_indices"])
        np.testing.assert_array_equal(got["send_bucket"][:n], want["send_bucket"])
        np.testing.assert_array_equal(got["route_to_send"][:tokens * top_k], want["route_to_send"])
        np.testing.assert_array_equal(got["count_row"], want["count_cube"][r])
        assert (got["send_route"][n:] == -7).all()
    cube = np.ascontiguousarray(meta[0]["count_cube"], np.int32)
    capacity = int(meta[0]["stats"][1])              # exactly the largest receive total
    for r in some_ranks:
        got, status = finalize(kernels, cube, r, world, epr, bins, capacity)
        check_finalize(got, status, meta[r], cube, r, world, epr)


def test_offset_tables_over_moonep_physical_slots(kernels):
    """2 * E/R slots per rank with most replica slots empty: the balanced cubes of the MoonEP
    fixtures through the offset kernels."""
    from oracle import moonep_oracle as M

    golden = np.load(HERE / "golden" / "moonep_tables.npz")
    for name in ("owners_w8_e64_k4", "owners_w8_e384_k16_t256", "hot_w2_e4", "w1_e8_k2"):
        tpe = golden[f"{name}/tpe_all"]
        world, experts = tpe.shape
        slots = 2 * experts // world
        cube = M.balanced_count_cube(tpe, golden[f"{name}/alloc_cumsum"], golden[f"{name}/inverse"])
        bins = next_pow2(world * slots)
        wide = np.zeros((world, bins), np.int32)
        wide[:, :world * slots] = cube
        capacity = int(tpe.sum(axis=1)[0])
        for r in sorted({0, world - 1}):
            want = O.offset_tables_from_cube(cube, r, slots)
            got, status = finalize(kernels, wide, r, world, slots, bins, capacity)
            check_finalize(got, status, want, wide, r, world, slots)


def test_receive_overflow_writes_no_tile_and_nothing_past_the_tables(kernels):
    world, epr, bins = 4, 8, 32
    rng = np.random.default_rng(0)
    cube = rng.integers(200, 900, size=(world, bins)).astype(np.int32)
    cube[:, world * epr:] = 0
    capacity = 256                                    # far below any rank's receive total
    for r in range(world):
        got, status = finalize(kernels, cube, r, world, epr, bins, capacity)
        assert status[0] == 2
        assert got["num_mtiles"][0] == 0 and got["num_mtiles2"][0] == 0
        assert (got["mtile_group"] == -7).all() and (got["mtile2_row0"] == -7).all()


def test_empty_input_and_single_route(kernels):
    got = route_local(kernels, np.zeros((0, 2), np.int32), 8, 8)
    assert got["local_stats"].tolist() == [0, 0] and (got["count_row"] == 0).all()
    got = route_local(kernels, np.array([[5]], np.int32), 8, 8)
    assert got["local_stats"].tolist() == [1, 0] and got["send_bucket"][0] == 5
    assert got["route_to_send"][0] == 0


@pytest.mark.parametrize("tokens, experts, top_k", [(7, 8, 2), (33, 64, 8), (10, 384, 16),
                                                    (5, 1000, 32), (9, 33, 33 - 1)])
def test_router_topk_matches_torch(kernels, tokens, experts, top_k):
    top_k = min(top_k, 32)
    gen = torch.Generator().manual_seed(experts)
    logits = torch.randn(tokens, experts, generator=gen)
    logits[0, : experts // 2] = float("-inf")          # masked experts
    logits[1, 3] = logits[1, 4]                        # a tie
    if tokens > 2:
        logits[2, :] = float("-inf")
        logits[2, :max(1, top_k // 2)] = 0.5           # fewer finite logits than top_k
    if tokens > 3:
        logits[3, 1] = float("nan")
    ld = experts + 3
    padded = torch.zeros(tokens, ld)
    padded[:, :experts] = logits
    buf = padded.numpy().copy()
    selected = np.full((tokens, top_k), -7, np.int32)
    weights = np.full((tokens, top_k), -7, np.float32)
    kernels.cot_router_topk(p(buf), ld, tokens, experts, top_k, p(selected), p(weights))
    want_sel, want_w = O.router_topk(logits, top_k)
    np.testing.assert_array_equal(selected, want_sel.numpy())
    np.testing.assert_allclose(weights, want_w.numpy(), rtol=1e-5, atol=1e-7, equal_nan=True)
