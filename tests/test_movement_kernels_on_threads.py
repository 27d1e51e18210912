"""The two byte movers of mega-moe-td_b200/csrc/movement.cu that carry no floating-point
formula of their own, executed on the host from their source text: ``dispatch_rows_kernel`` (the
row push of the unfused dispatch) and ``topk_reduce_kernel`` (the gather-sum over a token's top-k
rows, with the routing-weight gradient gather).  The kernels are cut out of the file; their two
PTX load / store wrappers and the bf16 pack are restated in C++ in the harness.  All ranks of a
case push into per-rank receive buffers held in host memory; the result must be the receive order
of the oracle's routing tables.  Runs under AddressSanitizer with MOE_TEST_SANITIZE=1."""

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

HARNESS = r"""
#include "cuda_on_threads.h"

struct __nv_bfloat16 { uint16_t bits; };
static inline uint16_t bf16_bits(float f) {           // round to nearest even
  uint32_t u = __float_as_uint(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
  return (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
}
static inline __nv_bfloat16 __float2bfloat16(float f) { return __nv_bfloat16{bf16_bits(f)}; }
static inline float __bfloat162float(__nv_bfloat16 v) { return __uint_as_float((uint32_t)v.bits << 16); }

namespace mm {
// stand-ins for the PTX wrappers of movement.cu and for pack_bf16x2 of common.cuh
static inline uint4 ld_nc_16(const void* p) { return *static_cast<const uint4*>(p); }
static inline void st_16(void* p, const uint4& v) { *static_cast<uint4*>(p) = v; }
static inline uint32_t pack_bf16x2(float lo, float hi) {
  return (uint32_t)bf16_bits(lo) | ((uint32_t)bf16_bits(hi) << 16);
}
%(dispatch)s
%(reduce)s
}  // namespace mm
using namespace mm;

extern "C" {

// grid of mm_dispatch_rows
void cot_dispatch_rows(const uint8_t* src, int hidden, const float* weights,
                       const int32_t* send_token, const int32_t* send_route,
                       const int32_t* send_bucket, const int32_t* send_bucket_starts,
                       const int32_t* send_bucket_dst_starts, const int32_t* local_stats,
                       int max_routes, int epr, int capacity_rows, void* const* peer_rows,
                       float* const* peer_weights, int sms) {
  if (max_routes <= 0) return;
  const int warps = kDispatchThreads / 32;
  int blocks = (max_routes + warps - 1) / warps;
  if (blocks > sms * 8) blocks = sms * 8;
  cot::launch(blocks, kDispatchThreads, [=] {
    dispatch_rows_kernel(src, hidden * 2, weights, send_token, send_route, send_bucket,
                         send_bucket_starts, send_bucket_dst_starts, local_stats, epr,
                         capacity_rows, peer_rows, peer_weights);
  });
}

// grid of mm_topk_reduce
void cot_topk_reduce(const uint8_t* rows, int64_t ld_rows, const int32_t* route_to_send, int tokens,
                     int top_k, int hidden, uint8_t* out, const __nv_bfloat16* gate_in,
                     __nv_bfloat16* gate_out, float* gate_out_f32, int sms) {
  if (tokens <= 0) return;
  const int blocks = tokens < sms * 8 ? tokens : sms * 8;
  cot::launch(blocks, kReduceThreads, [=] {
    topk_reduce_kernel(rows, ld_rows * 2, route_to_send, tokens, top_k, hidden * 2, out, gate_in,
                       gate_out, gate_out_f32);
  });
}

}  // extern "C"
"""


def cut(text: str, start: str, end: str = "\n}\n") -> str:
    i = text.index(start)
    i = text.rfind("\n", 0, i) + 1
    j = text.index(end, i) + len(end)
    return text[i:j]


@pytest.fixture(scope="module")
def kernels(tmp_path_factory):
    from cuda_on_threads.host_build import compile_for_host
    movement = (CSRC / "movement.cu").read_text()
    dispatch = (re.search(r"constexpr int kDispatchThreads = \d+;", movement).group(0) + "\n"
                + cut(movement, "__global__ void __launch_bounds__(kDispatchThreads)"))
    reduce_ = (re.search(r"constexpr int kReduceThreads = \d+;", movement).group(0) + "\n"
               + re.search(r"constexpr int kMaxTopK = \d+;", movement).group(0) + "\n"
               + cut(movement, "__global__ void __launch_bounds__(kReduceThreads)"))
    d = tmp_path_factory.mktemp("movement_on_threads")
    (d / "movement.cpp").write_text(HARNESS % dict(dispatch=dispatch, reduce=reduce_))
    lib = C.CDLL(str(compile_for_host(d / "movement.cpp", d / "libmovement.so")))
    lib.cot_dispatch_rows.restype = None
    lib.cot_topk_reduce.restype = None
    lib.cot_topk_reduce.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                    C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
    return lib


def p(a):
    return C.c_void_p(a.ctypes.data)


DISPATCH_CASES = [  # world, tokens, hidden, experts, top_k, drop share, capacity slack
    (1, 20, 64, 4, 2, 0.0, 0), (2, 33, 8, 8, 3, 0.2, 0), (4, 17, 1032, 16, 4, 0.0, 3),
    (8, 9, 520, 32, 4, 0.1, 0), (2, 40, 7168, 4, 1, 0.0, 0),
]


@pytest.mark.parametrize("world, tokens, hidden, experts, top_k, drop, slack", DISPATCH_CASES)
def test_dispatch_rows_fill_the_receive_buffers_in_receive_order(kernels, world, tokens, hidden,
                                                                 experts, top_k, drop, slack):
    rng = np.random.default_rng(world * 100 + hidden)
    epr = experts // world
    sels, xs, ws = [], [], []
    for _ in range(world):
        s = rng.integers(0, experts, size=(tokens, top_k)).astype(np.int32)
        s[rng.random((tokens, top_k)) < drop] = experts + 1
        sels.append(s)
        xs.append(rng.integers(0, 1 << 16, size=(tokens, hidden), dtype=np.uint16))   # bf16 bits
        ws.append(rng.random((tokens, top_k)).astype(np.float32))
    meta = O.routing_metadata(sels, experts)
    capacity = int(meta[0]["stats"][1]) + slack
    recv = [np.full((capacity, hidden), 0xABCD, np.uint16) for _ in range(world)]
    recv_w = [np.full(capacity, -1.0, np.float32) for _ in range(world)]
    rows_table = (C.c_void_p * world)(*[a.ctypes.data for a in recv])
    weights_table = (C.c_void_p * world)(*[a.ctypes.data for a in recv_w])
    for r in range(world):
        m = meta[r]
        n = m["num_sent_routes"]
        pad = tokens * top_k
        tables = {}
        for k in ("send_token_indices", "send_route_indices", "send_bucket"):
            t = np.full(pad, -7, np.int32)
            t[:n] = m[k]
            tables[k] = t
        starts = np.ascontiguousarray(m["send_bucket_starts"], np.int32)
        dst = np.ascontiguousarray(m["send_bucket_dst_starts"], np.int32)
        stats = np.array([n, 0], np.int32)
        kernels.cot_dispatch_rows(p(xs[r]), hidden, p(ws[r]), p(tables["send_token_indices"]),
                                  p(tables["send_route_indices"]), p(tables["send_bucket"]),
                                  p(starts), p(dst), p(stats), pad, epr, capacity, rows_table,
                                  weights_table, 3)
    sources = O.receive_sources(meta)
    for d in range(world):
        src, route = sources[d]
        total = src.size
        want = np.stack([xs[s][rt // top_k] for s, rt in zip(src, route)]) if total else \
            np.zeros((0, hidden), np.uint16)
        np.testing.assert_array_equal(recv[d][:total], want)
        assert (recv[d][total:] == 0xABCD).all()
        want_w = np.array([ws[s].reshape(-1)[rt] for s, rt in zip(src, route)], np.float32)
        np.testing.assert_array_equal(recv_w[d][:total], want_w)
        assert (recv_w[d][total:] == -1.0).all()


def test_dispatch_skips_rows_past_the_capacity(kernels):
    world, tokens, hidden, experts, top_k = 2, 30, 16, 4, 2
    rng = np.random.default_rng(3)
    sels = [np.zeros((tokens, top_k), np.int32) for _ in range(world)]      # all to expert 0
    xs = [rng.integers(0, 1 << 16, size=(tokens, hidden), dtype=np.uint16) for _ in range(world)]
    meta = O.routing_metadata(sels, experts)
    capacity = 50                                        # rank 0 would receive 120 rows
    recv = [np.full((capacity, hidden), 0xABCD, np.uint16) for _ in range(world)]
    rows_table = (C.c_void_p * world)(*[a.ctypes.data for a in recv])
    for r in range(world):
        m = meta[r]
        n = m["num_sent_routes"]
        tabs = [np.ascontiguousarray(m[k], np.int32) for k in
                ("send_token_indices", "send_route_indices", "send_bucket", "send_bucket_starts",
                 "send_bucket_dst_starts")]
        stats = np.array([n, 0], np.int32)
        kernels.cot_dispatch_rows(p(xs[r]), hidden, None, *[p(t) for t in tabs], p(stats), n,
                                  experts // world, capacity, rows_table, None, 2)
    # rank 0's first 50 receive rows are rank 0's first 50 send rows; nothing else was written
    np.testing.assert_array_equal(recv[0], xs[0][meta[0]["send_token_indices"][:capacity]])
    assert (recv[1] == 0xABCD).all()


REDUCE_CASES = [(7, 2, 64), (33, 8, 1032), (5, 64, 8), (3, 1, 7168), (12, 16, 264)]


@pytest.mark.parametrize("tokens, top_k, hidden", REDUCE_CASES)
@pytest.mark.parametrize("with_gate", [False, True])
def test_topk_reduce_matches_the_oracle(kernels, tokens, top_k, hidden, with_gate):
    gen = torch.Generator().manual_seed(tokens * hidden)
    n_rows = tokens * top_k + 5
    ld = hidden + 8                                       # rows may be strided
    rows = torch.randn(n_rows, ld, generator=gen).to(torch.bfloat16)
    perm = torch.randperm(n_rows, generator=gen)[:tokens * top_k].to(torch.int32)
    route_to_send = perm.clone()
    route_to_send[torch.rand(tokens * top_k, generator=gen) < 0.2] = -1     # dropped routes
    r2s = route_to_send.numpy().copy()
    rows_np = rows.view(torch.int16).numpy().copy()
    out = np.full((tokens, hidden), 0x7777, np.int16)
    gate = torch.randn(n_rows, generator=gen).to(torch.bfloat16)
    gate_np = gate.view(torch.int16).numpy().copy()
    gate_out = np.full(tokens * top_k, 0x7777, np.int16)
    gate_f32 = np.full(tokens * top_k, -7.0, np.float32)
    kernels.cot_topk_reduce(p(rows_np), ld, p(r2s), tokens, top_k, hidden, p(out),
                            p(gate_np) if with_gate else None, p(gate_out) if with_gate else None,
                            p(gate_f32) if with_gate else None, 2)
    want = O.topk_reduce(rows[:, :hidden], r2s, tokens, top_k)
    assert torch.equal(torch.from_numpy(out).view(torch.bfloat16).view(torch.int16),
                       want.view(torch.int16))
    if with_gate:
        idx = torch.from_numpy(r2s).long()
        want_g = torch.where(idx >= 0, gate[idx.clamp(min=0)], torch.zeros((), dtype=torch.bfloat16))
        assert torch.equal(torch.from_numpy(gate_out).view(torch.bfloat16).view(torch.int16),
                           want_g.view(torch.int16))
        np.testing.assert_array_equal(gate_f32, want_g.float().numpy())
    else:
        assert (gate_out == 0x7777).all()
