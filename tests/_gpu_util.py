"""Helpers of the GPU tests: call single C-ABI entry points on plain tensors."""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from mega_moe import _native as N
from mega_moe.ops import _launch as L


PAIR = 1   # tile mode under test: 0 = one CTA per tile, 1 = CTA pairs (cta_group::2),
           # 2 = skinny ragged-row GEMMs / unit walk of the weight gradient


def tile_tables(counts, device, tile_rows=128):
    """group_offs / row-tile tables for per-group row counts (what mm_route_finalize builds)."""
    counts = [int(c) for c in counts]
    offs = np.r_[0, np.cumsum(counts)].astype(np.int32)
    groups, rows = [], []
    for g, c in enumerate(counts):
        for r0 in range(0, c, tile_rows):
            groups.append(g)
            rows.append(int(offs[g]) + r0)
    t = lambda a: torch.tensor(np.asarray(a, dtype=np.int32).reshape(-1), dtype=torch.int32,
                               device=device)
    return t(offs), t(groups + [0]), t(rows + [0]), t([len(groups)])


def gemm_desc(a, weight, k_dim, n_dim, n_out, k_extent, counts, status):
    dev = a.device
    offs, mg, mr, nm = tile_tables(counts, dev, 256 if PAIR else 128)
    b_k_major, ld, gs, n_total = L.weight_operand(weight, k_dim, n_dim)
    d = N.GemmDesc()
    d.a = a.data_ptr()
    d.lda = a.stride(0)
    d.a_rows_cap = a.shape[0]
    d.b = weight.data_ptr()
    d.b_k_major = b_k_major
    d.b_cols_total = n_total
    d.b_ld = ld
    d.b_group_stride = gs
    d.num_groups = weight.shape[0]
    d.N = n_out
    d.K = k_extent
    d.grid_limit = 0
    d.pair = PAIR
    d.group_offs = offs.data_ptr()
    d.mtile_group = mg.data_ptr()
    d.mtile_row0 = mr.data_ptr()
    d.num_mtiles = nm.data_ptr()
    d.status = status.data_ptr()
    keep = (offs, mg, mr, nm)
    return d, keep


def new_status(device):
    return torch.zeros(8, dtype=torch.int32, device=device)


def run_grouped_gemm(a, weight, k_dim, n_dim, counts):
    """out[rows of g] = a[rows of g] @ B_g with B_g[k, n] = weight[g] indexed by k_dim/n_dim."""
    status = new_status(a.device)
    n_out = weight.shape[n_dim]
    d, keep = gemm_desc(a, weight, k_dim, n_dim, n_out, weight.shape[k_dim], counts, status)
    out = torch.full((a.shape[0], n_out), float("nan"), dtype=torch.bfloat16, device=a.device)
    N.check(N.lib().mm_grouped_gemm(C.byref(d), None, out.data_ptr(), out.stride(0), N.stream_ptr()),
            "mm_grouped_gemm")
    torch.cuda.synchronize()
    assert int(status[0]) == 0, status.tolist()
    return out


def run_fc1_swiglu(a, gate_up, row_weight, counts, activation="swiglu", beta=1.0,
                   linear_beta=None, clamp=7.0, want_raw=True, weight_bf16=None):
    status = new_status(a.device)
    ffn = gate_up.shape[2] // 2
    d, keep = gemm_desc(a, gate_up, 1, 2, ffn, gate_up.shape[1], counts, status)
    act = torch.full((a.shape[0], ffn), float("nan"), dtype=torch.bfloat16, device=a.device)
    raw = torch.full((a.shape[0], 2 * ffn), float("nan"), dtype=torch.bfloat16,
                     device=a.device) if want_raw else None
    N.check(N.lib().mm_fc1_swiglu(
        C.byref(d), None, act.data_ptr(), act.stride(0), N.ptr(raw), raw.stride(0) if want_raw else 0,
        row_weight.data_ptr(), N.ptr(weight_bf16), N.ACT_IDS[activation], float(beta),
        float(linear_beta) if linear_beta is not None else 0.0, float(clamp), N.stream_ptr()),
        "mm_fc1_swiglu")
    torch.cuda.synchronize()
    assert int(status[0]) == 0, status.tolist()
    return act, raw


def run_wgrad(grad_out, orig_in, counts):
    dev = grad_out.device
    status = new_status(dev)
    offs = torch.tensor(np.r_[0, np.cumsum(counts)].astype(np.int32), device=dev)
    groups = len(counts)
    out = torch.full((groups, grad_out.shape[1], orig_in.shape[1]), float("nan"),
                     dtype=torch.bfloat16, device=dev)
    rows = min(grad_out.shape[0], orig_in.shape[0])
    N.check(N.lib().mm_grouped_wgrad(
        grad_out.data_ptr(), grad_out.stride(0), grad_out.shape[1], orig_in.data_ptr(),
        orig_in.stride(0), orig_in.shape[1], rows, offs.data_ptr(), groups, out.data_ptr(),
        out.stride(1), out.stride(0), status.data_ptr(), 0, PAIR, N.stream_ptr()),
        "mm_grouped_wgrad")
    torch.cuda.synchronize()
    assert int(status[0]) == 0, status.tolist()
    return out


def ref_grouped(a, weight, k_dim, n_dim, counts):
    """fp32 torch reference of run_grouped_gemm (rounded to bf16)."""
    out = torch.zeros(a.shape[0], weight.shape[n_dim], dtype=torch.float32, device=a.device)
    start = 0
    for g, c in enumerate(counts):
        if c:
            w = weight[g].float()
            b = w if (k_dim, n_dim) == (1, 2) else w.T
            out[start:start + c] = a[start:start + c].float() @ b
        start += c
    return out.to(torch.bfloat16)


def rel_err(x, ref):
    x = x.float()
    ref = ref.float()
    return float((x - ref).abs().max() / (ref.abs().max() + 1e-9))
