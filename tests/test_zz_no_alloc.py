"""The allocation-free routing entry point must agree with the regular one.

`mm_route_local_static` serves callers that may not allocate device memory (a serving
process whose pool is frozen after start-up, a plugin without an allocator): it keeps its
scratch in a fixed array inside the library instead of taking a caller buffer.  The array is
shared by all calls and keeps whatever the previous call left behind, so the test runs two
different problems back to back and requires both to match `mm_route_local` bit for bit.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _outputs(n, bins):
    i32 = dict(dtype=torch.int32, device=DEV)
    return [torch.full((max(n, 1),), -9, **i32) for _ in range(4)] + \
           [torch.full((bins,), -9, **i32), torch.full((2,), -9, **i32)]


def _run(lib, N, sel, top_k, experts, bins, static):
    n = sel.numel()
    outs = _outputs(n, bins)
    ptrs = [t.data_ptr() for t in outs]
    if static:
        rc = lib.mm_route_local_static(sel.data_ptr(), n, top_k, experts, bins, *ptrs,
                                       N.stream_ptr())
    else:
        nbytes = lib.mm_route_scratch_bytes(n, bins)
        scratch = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=DEV)
        rc = lib.mm_route_local(sel.data_ptr(), n, top_k, experts, bins, *ptrs,
                                scratch.data_ptr(), scratch.numel(), N.stream_ptr())
    N.check(rc, "route_local")
    torch.cuda.synchronize()
    return [t.cpu() for t in outs]


def test_static_scratch_entry_point_matches_regular_entry_point():
    from mega_moe import _native as N
    from mega_moe.runtime.workspace import next_power_of_2
    lib = N.lib()
    rng = np.random.default_rng(2024)
    # two different problems in a row: the second must not see the first one's leftovers
    problems = [(8192, 16, 896, 0.0), (3000, 4, 24, 0.3)]
    for tokens, top_k, experts, drop in problems:
        sel = rng.integers(0, experts, size=(tokens, top_k)).astype(np.int32)
        if drop:
            sel[rng.random(sel.shape) < drop] = experts
        sel_t = torch.tensor(sel, device=DEV)
        bins = next_power_of_2(experts)
        got = _run(lib, N, sel_t, top_k, experts, bins, static=True)
        want = _run(lib, N, sel_t, top_k, experts, bins, static=False)
        n_valid = int(want[5][0])
        assert int(got[5][0]) == n_valid
        for g, w, name in zip(got[:3], want[:3], ("send_route", "send_token", "send_bucket")):
            assert torch.equal(g[:n_valid], w[:n_valid]), name
        assert torch.equal(got[3], want[3]), "route_to_send"
        assert torch.equal(got[4], want[4]), "count_row"


def test_static_scratch_entry_point_rejects_oversized_requests():
    from mega_moe import _native as N
    lib = N.lib()
    bins = 4096
    n = 2048 * 70          # (70 + 1) blocks x 4096 bins x 4 B > 1 MiB
    assert lib.mm_route_scratch_bytes(n, bins) > (1 << 20)
    sel = torch.zeros(n, dtype=torch.int32, device=DEV)
    outs = _outputs(n, bins)
    rc = lib.mm_route_local_static(sel.data_ptr(), n, 1, 4096, bins, *[t.data_ptr() for t in outs],
                                   N.stream_ptr())
    assert rc == -3
    assert b"1048576" in lib.mm_last_error()
    torch.cuda.synchronize()
