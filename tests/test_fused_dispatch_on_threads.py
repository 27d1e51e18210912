"""The fused dispatch of mega-moe-td_b200/csrc/gemm_sm100.cuh executed on the host, all ranks at
once: ``dispatch_warp_run`` (the row push of the dispatch warps: batches of eight rows, segment
copies through two register buffers, per-bucket counting, arrival flags, self-resetting counters)
and ``wait_expert_arrival`` (the consumer side) are cut out of the source.  Their six PTX
statements are mapped one to one onto host atomics of the same ordering (``ld.global.nc.v4`` ->
a 16-byte load, ``atom.add.acq_rel`` -> fetch-add acq_rel, ``st.release`` / ``ld.acquire`` ->
release store / acquire load, ``fence.proxy.async`` -> nothing); everything else is the kernel's
own text, compiled against tests/cuda_on_threads/cuda_on_threads.h.

Every rank runs a grid of CTAs with two dispatch warps each, concurrently with the other ranks
and with one consumer per rank that waits for each local expert's flags and then reads that
expert's rows.  Checked: the receive buffers hold exactly the oracle's receive order (rows and
routing weights), a consumer never sees a row missing after the flags, every flag carries the
epoch, every delivery counter is back at zero, and a second launch with the next epoch works on
the same counters.  This is the logic of the protocol, not the GPU's memory model."""

from __future__ import annotations

import ctypes as C
import re
import sys
from pathlib import Path

import numpy as np
import pytest

REPO = Path(__file__).resolve().parent.parent
HERE = Path(__file__).resolve().parent
CSRC = REPO / "mega-moe-td_b200" / "csrc"
sys.path.insert(0, str(HERE))

from oracle import moe_oracle as O  # noqa: E402

from cuda_on_threads.host_build import cut, map_ptx  # noqa: E402


HARNESS = r"""
#include <time.h>
#include <string.h>
#include <thread>
#include <vector>
#include "cuda_on_threads.h"
struct __nv_bfloat16;

namespace mm {
struct StatusRecord {
  int32_t code, site, slot, want, seen, block, pad[2];
};
enum StatusCode : int32_t { kOk = 0, kWaitTimeout = 1, kCapacityOverflow = 2, kBadIndex = 3 };
enum WaitSite : int32_t { kSiteDispatchFlag = 7 };
static uint64_t kWaitBudgetNs = 20000000000ull;      // generous: host threads are slow
inline uint64_t globaltimer_ns() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (uint64_t)ts.tv_sec * 1000000000ull + (uint64_t)ts.tv_nsec;
}
inline void report_status(StatusRecord* st, int32_t code, int32_t site, int32_t slot,
                          int32_t want, int32_t seen) {
  if (st == nullptr) return;
  if (atomicCAS(&st->code, 0, code) == 0) {
    st->site = site; st->slot = slot; st->want = want; st->seen = seen;
    st->block = (int32_t)blockIdx.x;
  }
}
%(order_bucket)s
%(constants)s
%(params)s
%(row_struct)s
%(find_bucket)s
%(resolve)s
%(warp_run)s
%(wait_arrival)s
}  // namespace mm
using namespace mm;

struct RankIn {
  const uint8_t* src;
  const float* weights;
  const int32_t *send_token, *send_route, *bucket_starts, *dst_starts, *counts, *order_prefix,
      *num_send;
  int32_t* bucket_done;
  const int32_t* my_flags;
  const int32_t* recv_expert_offs;   // consumer: row range of each local expert
  const uint8_t* expected_rows;      // consumer: what the receive buffer must hold
  StatusRecord* status;
};

extern "C" void set_wait_budget_ns(uint64_t ns) { mm::kWaitBudgetNs = ns; }

// All ranks at once.  seen_incomplete[rank]: rows a consumer found different from the expected
// ones right after the flags of their expert; gave_up[rank]: consumers whose wait ran out.
extern "C" void run_fused_dispatch(int world, int epr, int row_bytes, int capacity, int epoch,
                                   int grid, const RankIn* in, void* const* peer_rows,
                                   float* const* peer_weights, int32_t* const* peer_flags,
                                   int32_t* seen_incomplete, int32_t* gave_up) {
  std::vector<GemmParams> params(world);
  for (int r = 0; r < world; ++r) {
    GemmParams p = {};
    p.status = in[r].status;
    p.disp_src = in[r].src;
    p.disp_row_bytes = row_bytes;
    p.disp_rank = r; p.disp_world = world; p.disp_epr = epr; p.disp_capacity = capacity;
    p.disp_epoch = epoch;
    p.disp_weights = in[r].weights;
    p.disp_send_token = in[r].send_token; p.disp_send_route = in[r].send_route;
    p.disp_bucket_starts = in[r].bucket_starts; p.disp_dst_starts = in[r].dst_starts;
    p.disp_counts = in[r].counts; p.disp_order_prefix = in[r].order_prefix;
    p.disp_num_send = in[r].num_send; p.disp_bucket_done = in[r].bucket_done;
    p.disp_peer_rows = peer_rows; p.disp_peer_weights = peer_weights;
    p.disp_peer_flags = peer_flags; p.disp_my_flags = in[r].my_flags;
    params[r] = p;
  }
  std::vector<std::thread> ranks;
  for (int r = 0; r < world; ++r) {
    ranks.emplace_back([&, r] {            // the dispatch warps of rank r's launch
      const GemmParams p = params[r];
      cot::launch(grid, 32 * kDispatchWarps, [=] {
        dispatch_warp_run(p, (int32_t)(threadIdx.x >> 5), (uint32_t)(threadIdx.x & 31));
      });
    });
    ranks.emplace_back([&, r] {            // a consumer of rank r: expert after expert
      const GemmParams p = params[r];
      const RankIn me = in[r];
      cot::launch(1, 32, [=] {
        if (threadIdx.x != 0) return;
        volatile int abort_flag = 0;
        for (int g = 0; g < epr; ++g) {
          if (!wait_expert_arrival(p, g, &abort_flag)) {
            __atomic_fetch_add(&gave_up[r], 1, __ATOMIC_SEQ_CST);
            return;
          }
          const int64_t lo = (int64_t)me.recv_expert_offs[g] * row_bytes;
          const int64_t hi = (int64_t)me.recv_expert_offs[g + 1] * row_bytes;
          const uint8_t* got = static_cast<const uint8_t*>(peer_rows[r]);
          if (hi > lo && memcmp(got + lo, me.expected_rows + lo, (size_t)(hi - lo)) != 0)
            __atomic_fetch_add(&seen_incomplete[r], 1, __ATOMIC_SEQ_CST);
        }
      });
    });
  }
  for (auto& t : ranks) t.join();
}
"""


class RankIn(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in (
        "src", "weights", "send_token", "send_route", "bucket_starts", "dst_starts", "counts",
        "order_prefix", "num_send", "bucket_done", "my_flags", "recv_expert_offs",
        "expected_rows", "status")]


@pytest.fixture(scope="module")
def fused(tmp_path_factory):
    from cuda_on_threads.host_build import compile_for_host
    gemm = (CSRC / "gemm_sm100.cuh").read_text()
    common = (CSRC / "common.cuh").read_text()
    constants = "\n".join(re.search(rf"constexpr int {n} = \d+;", gemm).group(0) for n in
                          ("kDispatchWarps", "kDispatchBatchRows", "kDispatchSegChunks"))
    src = HARNESS % dict(
        order_bucket=cut(common, "int32_t dispatch_order_bucket("),
        constants=constants,
        params=cut(gemm, "struct GemmParams {", "\n};\n"),
        row_struct=cut(gemm, "struct DispatchRow {", "\n};\n"),
        find_bucket=cut(gemm, "int32_t dispatch_find_bucket("),
        resolve=cut(gemm, "DispatchRow dispatch_resolve("),
        warp_run=map_ptx(cut(gemm, "void dispatch_warp_run(")),
        wait_arrival=map_ptx(cut(gemm, "bool wait_expert_arrival(")),
    )
    d = tmp_path_factory.mktemp("fused_dispatch")
    (d / "fused_dispatch.cpp").write_text(src)
    lib = C.CDLL(str(compile_for_host(d / "fused_dispatch.cpp", d / "libfused.so")))
    lib.run_fused_dispatch.restype = None
    lib.set_wait_budget_ns.restype = None
    lib.set_wait_budget_ns.argtypes = [C.c_uint64]
    return lib


def p(a):
    return C.c_void_p(a.ctypes.data)


CASES = [  # world, tokens, hidden, experts, top_k, drop share, grid (CTAs per rank)
    (1, 40, 64, 4, 2, 0.0, 3), (2, 33, 8, 8, 3, 0.2, 2), (4, 25, 1032, 16, 4, 0.0, 3),
    (8, 12, 520, 64, 4, 0.1, 2), (2, 20, 7168, 4, 2, 0.0, 4), (4, 30, 136, 256, 3, 0.0, 2),
]


@pytest.mark.parametrize("world, tokens, hidden, experts, top_k, drop, grid", CASES)
def test_all_ranks_dispatch_concurrently_and_consumers_see_complete_experts(
        fused, world, tokens, hidden, experts, top_k, drop, grid):
    rng = np.random.default_rng(world * 1000 + hidden)
    epr = experts // world
    nb = world * epr
    row_bytes = hidden * 2
    flags = [np.zeros(nb, np.int32) for _ in range(world)]
    done = [np.zeros(nb, np.int32) for _ in range(world)]
    for epoch in (1, 2):                          # the second launch reuses counters and flags
        sels, xs, ws = [], [], []
        for _ in range(world):
            s = rng.integers(0, experts, size=(tokens, top_k)).astype(np.int32)
            s[rng.random((tokens, top_k)) < drop] = experts + 1
            if epoch == 2:
                s[:, 0] = 0                       # a skewed second step
            sels.append(s)
            xs.append(rng.integers(0, 1 << 16, size=(tokens, hidden), dtype=np.uint16))
            ws.append(rng.random((tokens, top_k)).astype(np.float32))
        meta = O.routing_metadata(sels, experts)
        capacity = int(meta[0]["stats"][1]) + 2
        sources = O.receive_sources(meta)
        expected = []
        for d in range(world):
            src, route = sources[d]
            rows = np.full((capacity, hidden), 0xABCD, np.uint16)
            if src.size:
                rows[:src.size] = np.stack([xs[s][rt // top_k] for s, rt in zip(src, route)])
            expected.append(rows)
        recv = [np.full((capacity, hidden), 0xABCD, np.uint16) for _ in range(world)]
        recv_w = [np.full(capacity, -1.0, np.float32) for _ in range(world)]
        keep, ranks = [], (RankIn * world)()
        for r in range(world):
            m = meta[r]
            n = m["num_sent_routes"]
            pad = max(tokens * top_k, 1)
            tabs = {}
            for k in ("send_token_indices", "send_route_indices"):
                t = np.full(pad, -7, np.int32)
                t[:n] = m[k]
                tabs[k] = t
            counts = np.ascontiguousarray(m["count_cube"][r][:nb], np.int32)
            order = [((r + 1 + dd) % world) * epr + le for le in range(epr) for dd in range(world)]
            arrays = dict(
                src=xs[r], weights=ws[r], send_token=tabs["send_token_indices"],
                send_route=tabs["send_route_indices"],
                bucket_starts=np.ascontiguousarray(m["send_bucket_starts"], np.int32),
                dst_starts=np.ascontiguousarray(m["send_bucket_dst_starts"], np.int32),
                counts=counts, order_prefix=np.r_[0, counts[order].cumsum()].astype(np.int32),
                num_send=np.array([n, 0], np.int32), bucket_done=done[r], my_flags=flags[r],
                recv_expert_offs=np.ascontiguousarray(m["recv_expert_offs"], np.int32),
                expected_rows=expected[r], status=np.zeros(8, np.int32))
            keep.append(arrays)
            for k, a in arrays.items():
                setattr(ranks[r], k, a.ctypes.data)
        rows_table = (C.c_void_p * world)(*[a.ctypes.data for a in recv])
        weights_table = (C.c_void_p * world)(*[a.ctypes.data for a in recv_w])
        flags_table = (C.c_void_p * world)(*[a.ctypes.data for a in flags])
        incomplete = np.zeros(world, np.int32)
        gave_up = np.zeros(world, np.int32)
        fused.run_fused_dispatch(world, epr, row_bytes, capacity, epoch, grid, ranks, rows_table,
                                 weights_table, flags_table, p(incomplete), p(gave_up))
        assert gave_up.tolist() == [0] * world and incomplete.tolist() == [0] * world
        for r in range(world):
            assert keep[r]["status"][0] == 0
            np.testing.assert_array_equal(recv[r], expected[r])
            src, route = sources[r]
            want_w = np.array([ws[s].reshape(-1)[rt] for s, rt in zip(src, route)], np.float32)
            np.testing.assert_array_equal(recv_w[r][:src.size], want_w)
            assert (recv_w[r][src.size:] == -1.0).all()
            assert (flags[r] == epoch).all()          # every (source, expert) bucket was flagged
            assert (done[r] == 0).all()               # counters ready for the next launch


def test_a_missing_source_makes_the_consumer_give_up_with_a_status_record(fused):
    """Only rank 0's flags arrive (rank 1 sends nothing and flags nothing): rank 0's consumer
    must run out of its wait on the first expert and report where."""
    world, epr, hidden = 2, 2, 8
    nb = world * epr
    zeros = np.zeros(nb + 1, np.int32)
    flags = [np.zeros(nb, np.int32) for _ in range(world)]
    flags[0][0:epr] = 1                            # source 0 flagged both experts of rank 0
    recv = [np.zeros((4, hidden), np.uint16) for _ in range(world)]
    ranks = (RankIn * world)()
    status = [np.zeros(8, np.int32) for _ in range(world)]
    offs = np.zeros(epr + 1, np.int32)
    x = np.zeros((1, hidden), np.uint16)
    keep = []
    for r in range(world):
        arrays = dict(src=x, send_token=zeros, send_route=zeros, bucket_starts=zeros,
                      dst_starts=zeros, counts=np.ones(nb, np.int32), order_prefix=zeros,
                      num_send=zeros, bucket_done=np.zeros(nb, np.int32), my_flags=flags[r],
                      recv_expert_offs=offs, expected_rows=recv[r], status=status[r])
        keep.append(arrays)
        for k, a in arrays.items():
            setattr(ranks[r], k, a.ctypes.data)
    rows_table = (C.c_void_p * world)(*[a.ctypes.data for a in recv])
    flags_table = (C.c_void_p * world)(*[a.ctypes.data for a in flags])
    incomplete = np.zeros(world, np.int32)
    gave_up = np.zeros(world, np.int32)
    fused.set_wait_budget_ns(300_000_000)
    try:
        fused.run_fused_dispatch(world, epr, hidden * 2, 4, 1, 1, ranks, rows_table, None,
                                 flags_table, p(incomplete), p(gave_up))
    finally:
        fused.set_wait_budget_ns(20_000_000_000)
    assert gave_up.tolist() == [1, 1]
    # code 1 (wait timed out), site 7 (dispatch flag), slot = source 1, expert 0; wanted epoch 1
    assert status[0][:5].tolist() == [1, 7, 1 * epr + 0, 1, 0]
