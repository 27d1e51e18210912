"""ctypes binding of ``libmegamoe_sm100.so`` (C ABI declared in ``include/mega_moe_b200.h``).

There is no CPU fallback: every operator of this package calls into the shared library,
and :func:`lib` raises ``RuntimeError`` when the library is missing.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path
from typing import Optional

import torch

_PKG_ROOT = Path(__file__).resolve().parent.parent
LIB_PATH = _PKG_ROOT / "lib" / "libmegamoe_sm100.so"
# Same sources compiled with -DMM_PROFILE: every warp role of the GEMM kernels also sums the SM
# clocks it spends in each of its waits.  Loaded instead of LIB_PATH when MOE_FWD_TIMING=1 is
# set before the first call into the library (and the file has been built).
TIMING_LIB_PATH = _PKG_ROOT / "lib" / "libmegamoe_sm100_prof.so"
# Per-CTA counters a GEMM launch of the instrumented library writes, in this order.
ROLE_COUNTER_SLOTS = (
    "prod_empty", "prod_bempty", "prod_flag", "mma_acc_empty", "mma_full", "mma_tail",
    "mma_total", "epi_acc_full", "epi_store_read", "epi_total", "tiles", "prod_issue",
    "prod_total", "mma_issue", "mma_decode")
# launch name -> int64 [160, 16] counters of the latest launch of that name (instrumented
# library only; see ops/_launch.py)
role_counters: dict = {}

MM_OK = 0
ACT_IDS = {"swiglu": 0, "situglu": 1, "clamp_swiglu": 2}

_c_i32p = C.c_void_p
_c_ptr = C.c_void_p


class StatusRecord(C.Structure):
    _fields_ = [(n, C.c_int32) for n in
                ("code", "site", "slot", "want", "seen", "block", "pad0", "pad1")]


class GemmDesc(C.Structure):
    _fields_ = [
        ("a", C.c_void_p), ("lda", C.c_int64), ("a_rows_cap", C.c_int64),
        ("b", C.c_void_p), ("b_k_major", C.c_int32), ("b_cols_total", C.c_int32),
        ("b_ld", C.c_int64), ("b_group_stride", C.c_int64),
        ("num_groups", C.c_int32), ("N", C.c_int32), ("K", C.c_int32), ("grid_limit", C.c_int32),
        ("pair", C.c_int32), ("reserved", C.c_int32),
        ("group_offs", C.c_void_p), ("mtile_group", C.c_void_p), ("mtile_row0", C.c_void_p),
        ("num_mtiles", C.c_void_p), ("status", C.c_void_p),
    ]


class ReplicaTable(C.Structure):
    _fields_ = [("local", C.c_void_p), ("local_stride", C.c_int64), ("bytes", C.c_int64),
                ("peer", C.c_void_p)]


class DispatchDesc(C.Structure):
    _fields_ = [(name, C.c_void_p) for name in (
        "src", "weights", "send_token", "send_route", "send_bucket_starts",
        "send_bucket_dst_starts", "count_row", "order_prefix", "local_stats", "bucket_done",
        "peer_rows", "peer_weights", "peer_flags", "my_flags")] + [
        (name, C.c_int32) for name in ("hidden", "rank", "world", "epr", "capacity_rows", "epoch")]


# name -> (restype, argtypes); must list every symbol of include/mega_moe_b200.h
SIGNATURES = {
    "mm_abi_version": (C.c_int, []),
    "mm_last_error": (C.c_char_p, []),
    "mm_num_sms": (C.c_int, [C.POINTER(C.c_int)]),
    "mm_status_reset": (C.c_int, [_c_ptr, _c_ptr]),
    "mm_status_read": (C.c_int, [_c_ptr, C.POINTER(StatusRecord), _c_ptr]),
    "mm_symm_alloc": (C.c_int, [C.c_size_t, C.POINTER(C.c_void_p), C.c_char_p]),
    "mm_symm_open": (C.c_int, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "mm_symm_close": (C.c_int, [_c_ptr]),
    "mm_symm_free": (C.c_int, [_c_ptr]),
    "mm_rank_barrier": (C.c_int, [_c_ptr, C.c_int, C.c_int, C.c_int, C.c_int, _c_ptr, _c_ptr]),
    "mm_route_scratch_bytes": (C.c_size_t, [C.c_int, C.c_int]),
    "mm_route_local": (C.c_int, [_c_i32p, C.c_int, C.c_int, C.c_int, C.c_int, _c_i32p, _c_i32p,
                                 _c_i32p, _c_i32p, _c_i32p, _c_i32p, _c_ptr, C.c_size_t, _c_ptr]),
    "mm_route_local_static": (C.c_int, [_c_i32p, C.c_int, C.c_int, C.c_int, C.c_int, _c_i32p,
                                        _c_i32p, _c_i32p, _c_i32p, _c_i32p, _c_i32p, _c_ptr]),
    "mm_count_exchange": (C.c_int, [_c_i32p, C.c_int, C.c_int, C.c_int, _c_ptr, C.c_int64, _c_ptr,
                                    _c_i32p, C.c_int, _c_ptr, _c_ptr]),
    "mm_route_finalize": (C.c_int, [_c_i32p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int] +
                          [_c_i32p] * 20 + [_c_ptr, _c_ptr]),
    "mm_dispatch_rows": (C.c_int, [_c_ptr, C.c_int, _c_ptr, _c_i32p, _c_i32p, _c_i32p, _c_i32p,
                                   _c_i32p, _c_i32p, C.c_int, C.c_int, C.c_int, _c_ptr, _c_ptr,
                                   _c_ptr]),
    "mm_topk_reduce": (C.c_int, [_c_ptr, C.c_int64, _c_i32p, C.c_int, C.c_int, C.c_int, _c_ptr,
                                 _c_ptr, _c_ptr, _c_ptr, _c_ptr]),
    "mm_fc1_swiglu": (C.c_int, [C.POINTER(GemmDesc), C.POINTER(DispatchDesc), _c_ptr, C.c_int64,
                                _c_ptr, C.c_int64, _c_ptr, _c_ptr, C.c_int, C.c_float, C.c_float,
                                C.c_float, _c_ptr]),
    "mm_grouped_gemm": (C.c_int, [C.POINTER(GemmDesc), C.POINTER(DispatchDesc), _c_ptr,
                                  C.c_int64, _c_ptr]),
    "mm_grouped_gemm_scatter": (C.c_int, [C.POINTER(GemmDesc), _c_i32p, _c_i32p, _c_ptr,
                                          C.c_int64, _c_ptr]),
    "mm_grouped_wgrad": (C.c_int, [_c_ptr, C.c_int64, C.c_int32, _c_ptr, C.c_int64, C.c_int32,
                                   C.c_int64, _c_i32p, C.c_int32, _c_ptr, C.c_int64, C.c_int64,
                                   _c_ptr, C.c_int32, C.c_int32, _c_ptr]),
    "mm_swiglu_bwd": (C.c_int, [_c_ptr, C.c_int64, _c_ptr, C.c_int64, _c_ptr, C.c_int, _c_i32p,
                                C.c_int, _c_ptr, C.c_int64, _c_ptr, C.c_int, C.c_float, C.c_float,
                                C.c_float, _c_i32p, _c_i32p, _c_ptr, C.c_int, _c_ptr, C.c_int,
                                _c_ptr]),
    "mm_moonep_plan": (C.c_int, [_c_i32p, C.c_int, C.c_int, C.c_int, C.c_int] + [_c_i32p] * 6 +
                       [_c_ptr, _c_ptr]),
    "mm_moonep_plan_host": (C.c_int, [_c_i32p, C.c_int, C.c_int, C.c_int, C.c_int] +
                            [_c_i32p] * 6),
    "mm_moonep_count_cube": (C.c_int, [_c_i32p, C.c_int, C.c_int, C.c_int, C.c_int, _c_i32p,
                                       _c_i32p, _c_i32p, C.c_int, _c_i32p, _c_i32p, _c_ptr]),
    "mm_moonep_count_cube_host": (C.c_int, [_c_i32p, C.c_int, C.c_int, C.c_int, C.c_int, _c_i32p,
                                            _c_i32p, _c_i32p, C.c_int, _c_i32p, _c_i32p]),
    "mm_moonep_map_routes": (C.c_int, [_c_i32p, _c_i32p, _c_i32p, C.c_int, C.c_int, C.c_int,
                                       C.c_int] + [_c_i32p] * 9 + [_c_ptr, _c_ptr]),
    "mm_moonep_map_routes_host": (C.c_int, [_c_i32p, _c_i32p, C.c_int, C.c_int, C.c_int, C.c_int,
                                            C.c_int] + [_c_i32p] * 10),
    "mm_moonep_relabel_routes": (C.c_int, [_c_i32p, _c_i32p, _c_i32p, _c_i32p, C.c_int, C.c_int,
                                           C.c_int] + [_c_i32p] * 5 + [_c_ptr, _c_ptr]),
    "mm_moonep_push_replicas": (C.c_int, [_c_i32p, C.c_int, C.c_int, C.c_int,
                                          C.POINTER(ReplicaTable), C.POINTER(ReplicaTable),
                                          C.c_int, _c_ptr]),
    "mm_moonep_pull_replica_grads": (C.c_int, [_c_i32p, C.c_int, C.c_int, C.c_int,
                                               C.POINTER(ReplicaTable), C.POINTER(ReplicaTable),
                                               C.c_int, _c_ptr]),
    "mm_router_topk": (C.c_int, [_c_ptr, C.c_int64, C.c_int, C.c_int, C.c_int, _c_i32p, _c_ptr,
                                 _c_ptr]),
    "mm_fc1_save_convert": (C.c_int, [_c_ptr, C.c_int64, C.c_int, _c_i32p, C.c_int, C.c_int,
                                      C.c_int, _c_ptr, C.c_int64, _c_ptr, _c_ptr]),
    "mm_swiglu_recompute": (C.c_int, [_c_ptr, C.c_int64, C.c_int, _c_ptr, C.c_int, _c_ptr, C.c_int,
                                      _c_i32p, C.c_int, _c_ptr, C.c_int64, C.c_int, C.c_float,
                                      C.c_float, C.c_float, _c_ptr]),
}

# saved FC1 formats (MM_FC1_* of the header) by the reference's config string / torch dtype
FC1_FORMAT_IDS = {"bf16": 0, "fp16": 1, "fp8": 2}

_lib: Optional[C.CDLL] = None

# Number of CUDA kernels this package has launched (benchmarks report it).
launch_count = 0


def count_launches(n: int) -> None:
    global launch_count
    launch_count += n


def lib() -> C.CDLL:
    """Load the shared library once; fail loudly when it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python mega-moe-td_b200/build.py` "
                "(there is no CPU or PyTorch fallback for the MoE kernels)")
        path = LIB_PATH
        if forward_timing_enabled() and TIMING_LIB_PATH.exists():
            path = TIMING_LIB_PATH
        handle = C.CDLL(str(path))
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        if path == TIMING_LIB_PATH:
            handle.mm_profile_buffer.restype = None
            handle.mm_profile_buffer.argtypes = [C.c_void_p]
        _lib = handle
    return _lib


def forward_timing_enabled() -> bool:
    """``MOE_FWD_TIMING=1``, the reference's switch for in-kernel phase timing
    (kernels/fused_forward.py:53-130)."""
    return os.environ.get("MOE_FWD_TIMING") == "1"


def role_counters_available() -> bool:
    """True when the loaded library is the instrumented one."""
    return hasattr(lib(), "mm_profile_buffer") and forward_timing_enabled()


def begin_role_counters(name: str) -> None:
    """Point the next GEMM launch's role counters at a fresh buffer filed under ``name``."""
    buf = torch.zeros(160, 16, dtype=torch.int64, device=torch.cuda.current_device())
    role_counters[name] = buf
    lib().mm_profile_buffer(buf.data_ptr())


def check(rc: int, what: str) -> None:
    if rc != MM_OK:
        msg = lib().mm_last_error()
        raise RuntimeError(f"{what} failed (code {rc}): {msg.decode() if msg else ''}")


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def stream_ptr(device=None) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def num_sms() -> int:
    out = C.c_int(0)
    check(lib().mm_num_sms(C.byref(out)), "mm_num_sms")
    return out.value


class _CudaBuffer:
    """Exposes a raw device allocation to torch through ``__cuda_array_interface__``."""

    def __init__(self, ptr_: int, nbytes: int):
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (ptr_, False), "version": 3,
            "strides": None,
        }


def tensor_from_ptr(ptr_: int, nbytes: int, dtype: torch.dtype, device) -> torch.Tensor:
    """A torch view (no ownership) of ``nbytes`` of device memory at ``ptr_``."""
    raw = torch.as_tensor(_CudaBuffer(ptr_, nbytes), device=device)
    return raw.view(dtype)
