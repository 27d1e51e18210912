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
