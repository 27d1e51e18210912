"""The row lookup of the fused dispatch, executed on the host from its own source text.

``dispatch_find_bucket`` (a 32-way ballot search over the prefix of the local counts in dispatch
order), ``dispatch_resolve`` (rows of a batch -> bucket, source row, destination row) of
mega-moe-td_b200/csrc/gemm_sm100.cuh and ``dispatch_order_bucket`` of csrc/common.cuh are cut out
of the sources, compiled by g++ against tests/cuda_on_threads/cuda_on_threads.h and run with
warps of 32 host threads that walk the batches exactly as the dispatch warps do.  Every send
row must be resolved exactly once, to the source token and the destination row the routing
tables of the oracle give it.  The GPU tests reach the multi-step search (more than 32 buckets)
only through whole-layer runs; this test checks the lookup by itself, up to 4096 buckets."""

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


def cut(text: str, start: str, end: str = "\n}\n") -> str:
    """The source from the line containing ``start`` through the first ``end`` after it."""
    i = text.index(start)
    i = text.rfind("\n", 0, i) + 1
    j = text.index(end, i) + len(end)
    return text[i:j]


HARNESS = r"""
#include "cuda_on_threads.h"

// the fields of GemmParams that the lookup reads
struct GemmParams {
  const int32_t* disp_order_prefix;
  const int32_t* disp_bucket_starts;
  const int32_t* disp_dst_starts;
  const int32_t* disp_send_token;
  const int32_t* disp_send_route;
  const uint8_t* disp_src;
  const float* disp_weights;
  void* const* disp_peer_rows;
  float* const* disp_peer_weights;
  int32_t disp_rank, disp_world, disp_epr, disp_capacity, disp_row_bytes;
};

%(order_bucket)s
%(constants)s
%(row_struct)s
%(find_bucket)s
%(resolve)s

extern "C" void lookup_all(const GemmParams* p, int n_send, int warps, int32_t* out_bucket,
                           int64_t* out_src, int64_t* out_dst, int32_t* out_hits) {
  const GemmParams params = *p;
  const int nb = params.disp_world * params.disp_epr;
  cot::launch(1, warps * 32, [=] {
    const int gid = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const int stride = warps * kDispatchBatchRows;
    for (int j0 = gid * kDispatchBatchRows; j0 < n_send; j0 += stride) {
      const DispatchRow row = dispatch_resolve(params, j0, n_send, nb, lane);
      if ((int)lane < kDispatchBatchRows && row.bucket >= 0) {
        const int j = j0 + (int)lane;
        out_bucket[j] = row.bucket;
        out_src[j] = row.src ? row.src - params.disp_src : -1;
        out_dst[j] = row.dst ? row.dst - (uint8_t*)params.disp_peer_rows[row.dst_rank] : -1;
        __atomic_fetch_add(&out_hits[j], 1, __ATOMIC_SEQ_CST);
      }
    }
  });
}
"""


@pytest.fixture(scope="module")
def lookup(tmp_path_factory):
    from cuda_on_threads.host_build import compile_for_host
    gemm = (CSRC / "gemm_sm100.cuh").read_text()
    common = (CSRC / "common.cuh").read_text()
    src = HARNESS % dict(
        order_bucket=cut(common, "int32_t dispatch_order_bucket("),
        constants=re.search(r"constexpr int kDispatchBatchRows = \d+;", gemm).group(0),
        row_struct=cut(gemm, "struct DispatchRow {", "\n};\n"),
        find_bucket=cut(gemm, "int32_t dispatch_find_bucket("),
        resolve=cut(gemm, "DispatchRow dispatch_resolve("),
    )
    d = tmp_path_factory.mktemp("dispatch_lookup")
    (d / "lookup.cpp").write_text(src)
    out = compile_for_host(d / "lookup.cpp", d / "liblookup.so")
    lib = C.CDLL(str(out))
    lib.lookup_all.restype = None
    return lib


class Params(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in (
        "disp_order_prefix", "disp_bucket_starts", "disp_dst_starts", "disp_send_token",
        "disp_send_route", "disp_src", "disp_weights", "disp_peer_rows", "disp_peer_weights")] + [
        (n, C.c_int32) for n in ("disp_rank", "disp_world", "disp_epr", "disp_capacity",
                                 "disp_row_bytes")]


CASES = [  # world, experts per rank, mean rows per bucket, share of empty buckets, warps
    (1, 1, 40, 0.0, 2), (2, 1, 9, 0.0, 3), (1, 31, 5, 0.3, 4), (4, 8, 7, 0.2, 4),
    (3, 11, 3, 0.5, 5), (8, 8, 6, 0.1, 7), (8, 48, 4, 0.3, 8), (8, 96, 2, 0.6, 8),
    (8, 128, 1, 0.5, 6), (16, 64, 1, 0.8, 8), (5, 205, 2, 0.4, 8), (8, 512, 1, 0.7, 8),
]


@pytest.mark.parametrize("world, epr, mean, empty, warps", CASES)
def test_every_send_row_is_resolved_once_and_to_the_right_rows(lookup, world, epr, mean, empty,
                                                               warps):
    rng = np.random.default_rng(world * 1000 + epr)
    nb = world * epr
    row_bytes = 64
    for rank in sorted({0, world // 2, world - 1}):
        counts = rng.poisson(mean, nb) * (rng.random(nb) >= empty)
        if nb > 3:
            counts[rng.integers(nb)] += 70          # one bucket longer than several batches
        counts = counts.astype(np.int64)
        n_send = int(counts.sum())
        if n_send == 0:
            counts[0] = 1
            n_send = 1
        # send order: bucket-major; the dispatch order visits local expert slots outermost,
        # destinations rotated by the sender's rank
        starts = (counts.cumsum() - counts).astype(np.int32)
        order = [((rank + 1 + dd) % world) * epr + le for le in range(epr) for dd in range(world)]
        prefix = np.r_[0, counts[order].cumsum()].astype(np.int32)
        dst_starts = rng.integers(0, 1000, nb).astype(np.int32) * 97
        capacity = int(dst_starts.max() + counts.max() + 5)
        send_token = rng.integers(0, 500, n_send).astype(np.int32)
        send_route = np.arange(n_send, dtype=np.int32)
        src = np.zeros(500 * row_bytes, np.uint8)
        peer_rows = [np.zeros(capacity * row_bytes, np.uint8) for _ in range(world)]
        peer_table = (C.c_void_p * world)(*[a.ctypes.data for a in peer_rows])
        params = Params(prefix.ctypes.data, starts.ctypes.data, dst_starts.ctypes.data,
                        send_token.ctypes.data, send_route.ctypes.data, src.ctypes.data, None,
                        C.cast(peer_table, C.c_void_p), None, rank, world, epr, capacity, row_bytes)
        out_bucket = np.full(n_send, -1, np.int32)
        out_src = np.full(n_send, -2, np.int64)
        out_dst = np.full(n_send, -2, np.int64)
        hits = np.zeros(n_send, np.int32)
        lookup.lookup_all(C.byref(params), n_send, warps, C.c_void_p(out_bucket.ctypes.data),
                          C.c_void_p(out_src.ctypes.data), C.c_void_p(out_dst.ctypes.data),
                          C.c_void_p(hits.ctypes.data))
        assert (hits == 1).all()
        # what the tables say about dispatch-order index j
        q = np.searchsorted(prefix, np.arange(n_send), side="right") - 1
        want_bucket = np.asarray(order)[q]
        in_bucket = np.arange(n_send) - prefix[q]
        np.testing.assert_array_equal(out_bucket, want_bucket)
        np.testing.assert_array_equal(out_src, send_token[starts[want_bucket] + in_bucket].astype(
            np.int64) * row_bytes)
        np.testing.assert_array_equal(out_dst, (dst_starts[want_bucket] + in_bucket).astype(
            np.int64) * row_bytes)


def test_rows_past_the_receive_capacity_are_counted_but_not_copied(lookup):
    world, epr, rank, row_bytes = 2, 2, 0, 32
    counts = np.array([3, 0, 6, 1], np.int64)
    starts = (counts.cumsum() - counts).astype(np.int32)
    order = [((rank + 1 + dd) % world) * epr + le for le in range(epr) for dd in range(world)]
    prefix = np.r_[0, counts[order].cumsum()].astype(np.int32)
    dst_starts = np.array([0, 3, 0, 6], np.int32)
    capacity = 4                                   # rows 4 and 5 of bucket 2 do not fit
    n_send = int(counts.sum())
    send_token = np.arange(n_send, dtype=np.int32)
    src = np.zeros(64 * row_bytes, np.uint8)
    peer_rows = [np.zeros(16 * row_bytes, np.uint8) for _ in range(world)]
    peer_table = (C.c_void_p * world)(*[a.ctypes.data for a in peer_rows])
    params = Params(prefix.ctypes.data, starts.ctypes.data, dst_starts.ctypes.data,
                    send_token.ctypes.data, send_token.ctypes.data, src.ctypes.data, None,
                    C.cast(peer_table, C.c_void_p), None, rank, world, epr, capacity, row_bytes)
    out_bucket = np.full(n_send, -1, np.int32)
    out_src = np.full(n_send, -2, np.int64)
    out_dst = np.full(n_send, -2, np.int64)
    hits = np.zeros(n_send, np.int32)
    lookup.lookup_all(C.byref(params), n_send, 2, C.c_void_p(out_bucket.ctypes.data),
                      C.c_void_p(out_src.ctypes.data), C.c_void_p(out_dst.ctypes.data),
                      C.c_void_p(hits.ctypes.data))
    assert (hits == 1).all() and (out_bucket >= 0).all()
    dropped = out_dst == -1
    assert dropped.sum() == 3                       # two rows of bucket 2, the row of bucket 3
    assert (out_src[dropped] == -1).all()
    assert sorted(out_bucket[dropped].tolist()) == [2, 2, 3]
