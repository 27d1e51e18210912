"""Every entry point of the C ABI rejects null pointers and zero sizes with MM_ERR_ARG and a
message that names it, before it touches the device: callable (and checked) without a GPU."""

from __future__ import annotations

import ctypes as C
import sys
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(REPO / "mega-moe-td_b200"))

from mega_moe import _native as N  # noqa: E402

MM_ERR_ARG = -1
INT_TYPES = (C.c_int, C.c_int32, C.c_int64, C.c_size_t)
CHECKED = sorted(n for n, (restype, _) in N.SIGNATURES.items()
                 if restype is C.c_int and n != "mm_abi_version")


def zero_arguments(argtypes):
    return [0 if t in INT_TYPES else 0.0 if t is C.c_float else None for t in argtypes]


def test_every_status_returning_entry_point_is_covered():
    assert len(CHECKED) >= 30


@pytest.mark.parametrize("name", CHECKED)
def test_null_and_zero_arguments_are_rejected(name):
    lib = N.lib()
    _, argtypes = N.SIGNATURES[name]
    assert getattr(lib, name)(*zero_arguments(argtypes)) == MM_ERR_ARG
    assert name in lib.mm_last_error().decode()


def test_size_limits_and_shapes_are_reported():
    lib = N.lib()
    buf = (C.c_int32 * 64)()
    ptr = C.cast(buf, C.c_void_p)
    # more experts than the planner's tables hold, experts not divisible by the ranks
    assert lib.mm_moonep_plan_host(ptr, 8192, 2, 8192, -1, ptr, ptr, ptr, ptr, ptr, ptr) == MM_ERR_ARG
    assert b"bad sizes" in lib.mm_last_error()
    assert lib.mm_moonep_plan_host(ptr, 3, 2, 3, -1, ptr, ptr, ptr, ptr, ptr, ptr) == MM_ERR_ARG
    # the column of unfiltered totals must lie past the experts and inside the row
    assert lib.mm_moonep_plan_host(ptr, 4, 2, 4, 4, ptr, ptr, ptr, ptr, ptr, ptr) == MM_ERR_ARG
    # the balanced cube must not be written over the counts, and must hold 2E columns
    assert lib.mm_moonep_count_cube_host(ptr, 4, 0, 2, 4, ptr, ptr, ptr, 8, ptr, ptr) == MM_ERR_ARG
    assert b"must not be written over" in lib.mm_last_error()
    other = (C.c_int32 * 64)()
    assert lib.mm_moonep_count_cube_host(ptr, 4, 0, 2, 4, ptr, ptr, C.cast(other, C.c_void_p), 7,
                                         ptr, ptr) == MM_ERR_ARG
    # replica tables: sizes in multiples of 16 bytes
    table = N.ReplicaTable(C.addressof(buf), 24, 24, C.addressof(buf))
    assert lib.mm_moonep_push_replicas(ptr, 0, 2, 2, C.byref(table), None, 0, None) == MM_ERR_ARG
    assert b"multiple of 16" in lib.mm_last_error()
    # scratch sizing of the route filter: (blocks of 2048 routes + 1) x bins x 4 bytes
    assert lib.mm_route_scratch_bytes(4096, 1024) == 3 * 1024 * 4
    assert lib.mm_route_scratch_bytes(-1, 8) == 0


def _gemm_desc(**over):
    buf = (C.c_int32 * 64)()
    base = C.addressof(buf)                      # 16-byte aligned? make it so
    base = (base + 15) & ~15
    d = N.GemmDesc()
    d.a, d.lda, d.a_rows_cap = base, 64, 128
    d.b, d.b_k_major, d.b_cols_total, d.b_ld, d.b_group_stride = base, 1, 64, 64, 64 * 64
    d.num_groups, d.N, d.K, d.grid_limit, d.pair = 1, 64, 64, 0, 0
    d.group_offs = d.mtile_group = d.mtile_row0 = d.num_mtiles = base
    for k, v in over.items():
        setattr(d, k, v)
    d._keep = buf
    return d, base


def test_grouped_gemm_descriptor_checks_precede_any_device_call():
    lib = N.lib()
    d, base = _gemm_desc(a=0)
    d.a = base + 2                                                   # not 16-byte aligned
    assert lib.mm_grouped_gemm(C.byref(d), None, base, 64, None) == MM_ERR_ARG
    assert b"16-byte aligned" in lib.mm_last_error()
    d, base = _gemm_desc(lda=68)                                     # stride not a multiple of 8
    assert lib.mm_grouped_gemm(C.byref(d), None, base, 64, None) == MM_ERR_ARG
    d, base = _gemm_desc(K=60)
    assert lib.mm_grouped_gemm(C.byref(d), None, base, 64, None) == MM_ERR_ARG
    assert b"K % 8 == 0" in lib.mm_last_error()
    d, base = _gemm_desc(N=48)
    assert lib.mm_grouped_gemm(C.byref(d), None, base, 64, None) == MM_ERR_ARG
    d, base = _gemm_desc(pair=3)
    assert lib.mm_grouped_gemm(C.byref(d), None, base, 64, None) == MM_ERR_ARG
    assert b"tile mode 3" in lib.mm_last_error()
    # a fused-dispatch descriptor with missing tables is refused before the GEMM is looked at
    d, base = _gemm_desc()
    x = N.DispatchDesc()
    x.src, x.hidden, x.world, x.epr, x.epoch = base, 64, 1, 1, 1
    assert lib.mm_grouped_gemm(C.byref(d), C.byref(x), base, 64, None) == MM_ERR_ARG
    assert b"fused dispatch descriptor" in lib.mm_last_error()


def test_weight_gradient_extent_checks():
    lib = N.lib()
    buf = (C.c_int32 * 64)()
    base = (C.addressof(buf) + 15) & ~15
    args = dict(grad_out=base, ld_go=64, Mw=64, orig_in=base, ld_in=64, Nw=64, rows_cap=128,
                group_offs=base, num_groups=1, out=base, ld_out=64, out_group_stride=64 * 64,
                status=None, grid_limit=0, pair=0, stream=None)

    def call(**over):
        a = dict(args, **over)
        return lib.mm_grouped_wgrad(*a.values())

    assert call(Mw=60) == MM_ERR_ARG and b"multiples of 8" in lib.mm_last_error()
    assert call(Nw=48) == MM_ERR_ARG
    assert call(ld_out=66) == MM_ERR_ARG
    assert call(out=base + 4) == MM_ERR_ARG and b"16-byte aligned" in lib.mm_last_error()
