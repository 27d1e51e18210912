"""Thin launch helpers shared by the forward and backward operators.

Each helper turns torch tensors into the plain pointers / sizes of one C-ABI call.  Nothing
here computes on the host: a missing shared library raises from ``_native.lib()``.
"""

from __future__ import annotations

import ctypes as C

import torch

from .. import _native as N
from ..runtime.workspace import MoEForwardContext

# When set (by a benchmark) it is called as EVENT_HOOK(name) -> (start_event, end_event) and
# the pair is recorded around the grouped-GEMM launch of that name.
EVENT_HOOK = None


class _timed:
    def __init__(self, name):
        self.pair = EVENT_HOOK(name) if EVENT_HOOK is not None else None
        self.name = name

    def __enter__(self):
        if N.forward_timing_enabled() and N.role_counters_available():
            N.begin_role_counters(self.name)
        if self.pair is not None:
            self.pair[0].record()

    def __exit__(self, *exc):
        if self.pair is not None:
            self.pair[1].record()
        return False


def weight_operand(weight: torch.Tensor, k_dim: int, n_dim: int):
    """Describe a per-expert weight ``[E, *, *]`` as the B operand of ``A[rows, K] @ B[K, N]``.

    ``k_dim`` / ``n_dim`` name which of dimensions 1 and 2 is the reduction / output axis.
    Returns ``(b_k_major, ld, group_stride, n_total)``; one of the two axes must be
    contiguous, which covers both the natural layout and a transposed stride view.
    """
    if weight.dim() != 3:
        raise ValueError("expert weights must be 3-D")
    sk, sn = weight.stride(k_dim), weight.stride(n_dim)
    if sk == 1:
        b_k_major, ld = 1, sn
    elif sn == 1:
        b_k_major, ld = 0, sk
    else:
        raise ValueError("expert weight must be contiguous along its reduction or output axis")
    return b_k_major, ld, weight.stride(0), weight.shape[n_dim]


TILE_SINGLE, TILE_PAIR, TILE_SKINNY = 0, 1, 2
# Expected rows per local expert up to which the transposed ("skinny") tiles are chosen.
SKINNY_MAX_ROWS_PER_EXPERT = 256


def gemm_tile_mode(ctx=None) -> int:
    """Tile mode of the ragged-row GEMMs (``mm_gemm_desc.pair``).

    ``MOE_GEMM_MODE`` = ``single`` (one CTA per 128x256 tile, cta_group::1), ``pair`` (clusters
    of two CTAs sharing 256-row tiles, cta_group::2; also ``MOE_GEMM_PAIR=1``), ``skinny``
    (transposed product: 256 output columns x up to 256 rows, the rows as the MMA's N extent in
    steps of 16), ``auto`` (default): skinny when the expected rows per local expert
    (tokens x top_k x world / experts) fit one skinny tile, else single, or ``mixed``: auto with
    CTA pairs for the GEMMs whose weights are K-major.
    """
    import os
    mode = os.environ.get("MOE_GEMM_MODE", "auto").lower()
    if os.environ.get("MOE_GEMM_PAIR", "0") == "1" or mode == "pair":
        return TILE_PAIR
    if mode == "single":
        return TILE_SINGLE
    if mode == "skinny":
        return TILE_SKINNY
    if mode not in ("auto", "mixed"):
        raise ValueError(f"MOE_GEMM_MODE={mode!r} is not one of auto, mixed, single, pair, skinny")
    if ctx is None:
        return TILE_SINGLE
    expected = ctx.max_tokens_per_rank * ctx.top_k * ctx.world_size / max(ctx.num_experts, 1)
    return TILE_SKINNY if expected <= SKINNY_MAX_ROWS_PER_EXPERT else TILE_SINGLE


def _mixed_tile_mode() -> bool:
    """``MOE_GEMM_MODE=mixed``: like ``auto``, but CTA pairs for the GEMMs whose weights are
    K-major (FC2, FC1 input gradient).  Those two launches measured 8-10 % faster at 1170 rows
    per expert, but under the power cap the other launches of the step slowed by as much, and at
    292 / 585 rows per expert the pairs lose; so it is not the default."""
    import os
    return os.environ.get("MOE_GEMM_MODE", "auto").lower() == "mixed"


def pair_mode_enabled() -> bool:
    """MOE_GEMM_PAIR=1 / MOE_GEMM_MODE=pair: CTA pairs for every GEMM."""
    return gemm_tile_mode(None) == TILE_PAIR


WGRAD_SINGLE, WGRAD_PAIR, WGRAD_UNIT = 0, 1, 2


def wgrad_tile_mode(ctx=None) -> int:
    """Tile mode of the weight gradients (``pair`` argument of ``mm_grouped_wgrad``):
    ``MOE_WGRAD_MODE`` = ``single`` / ``pair`` / ``unit`` / ``auto`` (default).  Auto follows
    ``MOE_GEMM_MODE=pair`` when that is set, takes the unit walk (one operand resident in shared
    memory) when the expected rows per local expert fit it, and single CTAs otherwise."""
    import os
    mode = os.environ.get("MOE_WGRAD_MODE", "auto").lower()
    if mode == "single":
        return WGRAD_SINGLE
    if mode == "pair":
        return WGRAD_PAIR
    if mode == "unit":
        return WGRAD_UNIT
    if mode != "auto":
        raise ValueError(f"MOE_WGRAD_MODE={mode!r} is not one of auto, single, pair, unit")
    if pair_mode_enabled():
        return WGRAD_PAIR
    if ctx is None:
        return WGRAD_SINGLE
    expected = ctx.max_tokens_per_rank * ctx.top_k * ctx.world_size / max(ctx.num_experts, 1)
    return WGRAD_UNIT if expected <= SKINNY_MAX_ROWS_PER_EXPERT else WGRAD_SINGLE


def make_desc(ctx: MoEForwardContext, a: torch.Tensor, a_rows_cap: int, lda: int,
              weight: torch.Tensor, k_dim: int, n_dim: int, n_out: int, k_extent: int,
              *, plan=None, grid_limit: int = 0) -> N.GemmDesc:
    b_k_major, ld, gs, n_total = weight_operand(weight, k_dim, n_dim)
    d = N.GemmDesc()
    d.a = a.data_ptr()
    d.lda = lda
    d.a_rows_cap = a_rows_cap
    d.b = weight.data_ptr()
    d.b_k_major = b_k_major
    d.b_cols_total = n_total
    d.b_ld = ld
    d.b_group_stride = gs
    d.num_groups = weight.shape[0]
    d.N = n_out
    d.K = k_extent
    d.grid_limit = grid_limit
    d.pair = gemm_tile_mode(ctx)
    if (d.pair == TILE_SINGLE and b_k_major and _mixed_tile_mode()):
        # K-major weights (FC2, FC1 input gradient): a CTA pair loads half of the 256-column
        # weight tile per CTA
        d.pair = TILE_PAIR
    src = plan if plan is not None else ctx
    d.group_offs = src.metadata_recv_expert_offs.data_ptr()
    if d.pair:
        d.mtile_group = src.mtile2_group.data_ptr()
        d.mtile_row0 = src.mtile2_row0.data_ptr()
        d.num_mtiles = src.num_mtiles2.data_ptr()
    else:
        d.mtile_group = src.mtile_group.data_ptr()
        d.mtile_row0 = src.mtile_row0.data_ptr()
        d.num_mtiles = src.num_mtiles.data_ptr()
    d.status = ctx.status.data_ptr()
    return d


def fused_dispatch_enabled(ctx=None) -> bool:
    """Whether the dispatch warps ride inside the GEMM launch (FC1, FC2 input gradient) or a
    separate row-push kernel plus a rank barrier runs first.  ``MOE_FUSED_DISPATCH`` = 1 / 0
    forces one; by default the dispatch is fused when there are peers (the pushes cross NVLink
    while the GEMM works) and separate on a single rank, where there is no link latency to
    hide and the copy warps only compete with the GEMM for memory bandwidth."""
    import os
    env = os.environ.get("MOE_FUSED_DISPATCH")
    if env is not None:
        return env != "0"
    return ctx is None or ctx.world_size > 1


def make_dispatch_desc(ctx: MoEForwardContext, src: torch.Tensor, weights, plan=None,
                       region: str = "peer_mem") -> N.DispatchDesc:
    """Descriptor of the dispatch fused into the next grouped GEMM: the rows of ``src`` go to
    the owning ranks' ``region``.  The per-bucket delivery counters need no clearing: the
    metadata kernel zeroes them and every fused launch leaves them at zero again."""
    p = plan if plan is not None else ctx
    d = N.DispatchDesc()
    d.src = src.data_ptr()
    d.weights = N.ptr(weights)
    d.send_token = p.send_token_indices.data_ptr()
    d.send_route = p.send_route_indices.data_ptr()
    d.send_bucket_starts = p.metadata_send_bucket_starts.data_ptr()
    d.send_bucket_dst_starts = p.metadata_send_bucket_dst_starts.data_ptr()
    d.count_row = p.metadata_count_row.data_ptr()
    d.order_prefix = p.disp_order_prefix.data_ptr()
    d.local_stats = p.metadata_local_stats.data_ptr()
    d.bucket_done = ctx.disp_bucket_done.data_ptr()
    d.peer_rows = ctx.symm.peer_table(region).data_ptr()
    d.peer_weights = (ctx.symm.peer_table("routing_weight_mem").data_ptr()
                      if weights is not None else None)
    d.peer_flags = ctx.symm.peer_table("dispatch_flags").data_ptr()
    d.my_flags = ctx.dispatch_flags.data_ptr()
    d.hidden = ctx.hidden_size
    d.rank = ctx.rank
    d.world = ctx.world_size
    d.epr = ctx.experts_per_rank
    d.capacity_rows = ctx.max_received_routes
    d.epoch = ctx.next_dispatch_epoch()
    return d


def dispatch_rows(ctx: MoEForwardContext, src: torch.Tensor, weights, num_routes: int, plan=None,
                  region: str = "peer_mem"):
    """Push the send rows of ``src`` (and their routing weights) to the owning ranks' ``region``
    (the receive buffer, or the re-dispatch slab of the recompute backward)."""
    p = plan if plan is not None else ctx
    _t = _timed("dispatch_rows")
    _t.__enter__()
    N.check(N.lib().mm_dispatch_rows(
        src.data_ptr(), ctx.hidden_size, N.ptr(weights),
        p.send_token_indices.data_ptr(), p.send_route_indices.data_ptr(),
        p.send_bucket.data_ptr(), p.metadata_send_bucket_starts.data_ptr(),
        p.metadata_send_bucket_dst_starts.data_ptr(), p.metadata_local_stats.data_ptr(),
        num_routes, ctx.experts_per_rank, ctx.max_received_routes,
        ctx.symm.peer_table(region).data_ptr(),
        ctx.symm.peer_table("routing_weight_mem").data_ptr() if weights is not None else None,
        N.stream_ptr()), "mm_dispatch_rows")
    _t.__exit__()
    N.count_launches(1)


def fc1_swiglu(ctx, desc, act_out, raw_out, row_weight, activation, beta, linear_beta, clamp,
               dispatch=None, weight_bf16_out=None):
    with _timed("fc1_swiglu"):
        N.check(N.lib().mm_fc1_swiglu(
            C.byref(desc), C.byref(dispatch) if dispatch is not None else None,
            act_out.data_ptr(), act_out.stride(0),
            N.ptr(raw_out), raw_out.stride(0) if raw_out is not None else 0,
            row_weight.data_ptr(), N.ptr(weight_bf16_out), N.ACT_IDS[activation], float(beta),
            float(linear_beta) if linear_beta is not None else 0.0, float(clamp),
            N.stream_ptr()), "mm_fc1_swiglu")
    # skinny tiles with a raw buffer: plain GEMM + activation pass (two kernels)
    N.count_launches(2 if (desc.pair == TILE_SKINNY and raw_out is not None) else 1)


def grouped_gemm(desc, out, name="grouped_gemm", dispatch=None):
    with _timed(name):
        N.check(N.lib().mm_grouped_gemm(
            C.byref(desc), C.byref(dispatch) if dispatch is not None else None,
            out.data_ptr(), out.stride(0), N.stream_ptr()), "mm_grouped_gemm")
    N.count_launches(1)


def grouped_gemm_scatter(ctx, desc, region: str, ld_dst: int, plan=None, name="gemm_scatter"):
    p = plan if plan is not None else ctx
    with _timed(name):
        N.check(N.lib().mm_grouped_gemm_scatter(
            C.byref(desc), p.row_src_rank.data_ptr(), p.row_src_pos.data_ptr(),
            ctx.symm.peer_table(region).data_ptr(), ld_dst, N.stream_ptr()),
            "mm_grouped_gemm_scatter")
    N.count_launches(1)


def grouped_wgrad(ctx, grad_out, orig_in, rows_cap, group_offs, num_groups, out, name="wgrad"):
    """out[g] [Mw, Nw] = grad_out[rows of g]^T @ orig_in[rows of g]."""
    with _timed(name):
        N.check(N.lib().mm_grouped_wgrad(
            grad_out.data_ptr(), grad_out.stride(0), grad_out.shape[1],
            orig_in.data_ptr(), orig_in.stride(0), orig_in.shape[1], rows_cap,
            group_offs.data_ptr(), num_groups, out.data_ptr(), out.stride(1), out.stride(0),
            ctx.status.data_ptr(), 0, wgrad_tile_mode(ctx), N.stream_ptr()),
            "mm_grouped_wgrad")
    N.count_launches(1)


def topk_reduce(rows, route_to_send, tokens, top_k, hidden, out, gate_in=None, gate_out=None,
                gate_out_f32=None):
    _t = _timed("topk_reduce")
    _t.__enter__()
    N.check(N.lib().mm_topk_reduce(
        rows.data_ptr(), rows.stride(0), route_to_send.data_ptr(), tokens, top_k, hidden,
        out.data_ptr(), N.ptr(gate_in), N.ptr(gate_out), N.ptr(gate_out_f32), N.stream_ptr()),
        "mm_topk_reduce")
    _t.__exit__()
    N.count_launches(1)


def fc1_format_of(fc1_out: torch.Tensor) -> int:
    """MM_FC1_* id of a saved FC1 tensor, from its dtype (reference: ``save_fc1_dtype``)."""
    if fc1_out.dtype == torch.bfloat16:
        return N.FC1_FORMAT_IDS["bf16"]
    if fc1_out.dtype == torch.float16:
        return N.FC1_FORMAT_IDS["fp16"]
    if fc1_out.dtype == torch.float8_e4m3fn:
        return N.FC1_FORMAT_IDS["fp8"]
    raise TypeError(f"saved fc1_output must be bf16, fp16 or float8_e4m3fn, got {fc1_out.dtype}")


def _fc1_scale_args(fc1_out, fc1_scale, scale_group, ffn):
    fmt = fc1_format_of(fc1_out)
    if fmt == N.FC1_FORMAT_IDS["fp8"]:
        if fc1_scale is None or not scale_group:
            raise ValueError("fp8 fc1_output needs fc1_output_scale and fc1_scale_group_size")
        scale_group = int(scale_group)
        if (fc1_scale.dtype != torch.float32 or not fc1_scale.is_contiguous()
                or fc1_scale.shape != (fc1_out.shape[0], 2 * ffn // scale_group)):
            raise ValueError("fc1_output_scale must be FP32 [rows, 2F // fc1_scale_group_size] "
                             "matching the FP8 fc1_output")
        return fmt, fc1_scale.data_ptr(), scale_group
    return fmt, None, 0


def swiglu_bwd(ctx, grad_act, fc1_out, row_scale, ffn, num_rows_dev, max_rows, grad_fc1,
               grad_scale, activation, beta, linear_beta, clamp, plan=None, push_gate=True,
               fc1_scale=None, scale_group=0):
    p = plan if plan is not None else ctx
    fmt, scale_ptr, scale_group = _fc1_scale_args(fc1_out, fc1_scale, scale_group, ffn)
    _t = _timed("swiglu_bwd")
    _t.__enter__()
    N.check(N.lib().mm_swiglu_bwd(
        grad_act.data_ptr(), grad_act.stride(0), fc1_out.data_ptr(), fc1_out.stride(0),
        row_scale.data_ptr(), ffn, num_rows_dev.data_ptr(), max_rows,
        grad_fc1.data_ptr(), grad_fc1.stride(0), grad_scale.data_ptr(),
        N.ACT_IDS[activation], float(beta if beta is not None else 1.0),
        float(linear_beta) if linear_beta is not None else 0.0,
        float(clamp if clamp is not None else 7.0),
        p.row_src_rank.data_ptr() if push_gate else None,
        p.row_src_pos.data_ptr() if push_gate else None,
        ctx.symm.peer_table("combine_gate_mem").data_ptr() if push_gate else None,
        fmt, scale_ptr, scale_group, N.stream_ptr()), "mm_swiglu_bwd")
    _t.__exit__()
    N.count_launches(1)


def swiglu_recompute(fc1_out, row_scale, ffn, num_rows_dev, max_rows, act_out, activation, beta,
                     linear_beta, clamp, fc1_scale=None, scale_group=0):
    """Weighted activation rows from saved FC1 rows (backward-side recompute)."""
    fmt, scale_ptr, scale_group = _fc1_scale_args(fc1_out, fc1_scale, scale_group, ffn)
    with _timed("swiglu_recompute"):
        N.check(N.lib().mm_swiglu_recompute(
            fc1_out.data_ptr(), fc1_out.stride(0), fmt, scale_ptr, scale_group,
            row_scale.data_ptr(), ffn, num_rows_dev.data_ptr(), max_rows,
            act_out.data_ptr(), act_out.stride(0), N.ACT_IDS[activation],
            float(beta if beta is not None else 1.0),
            float(linear_beta) if linear_beta is not None else 0.0,
            float(clamp if clamp is not None else 7.0), N.stream_ptr()), "mm_swiglu_recompute")
    N.count_launches(1)


def fc1_save_convert(raw, num_rows_dev, max_rows, fmt_name, scale_group, out, scale=None):
    """Raw bf16 FC1 rows -> the saved format (fp16 copy, or fp8 E4M3 + scale table)."""
    with _timed("fc1_save_convert"):
        N.check(N.lib().mm_fc1_save_convert(
            raw.data_ptr(), raw.stride(0), raw.shape[1], num_rows_dev.data_ptr(), max_rows,
            N.FC1_FORMAT_IDS[fmt_name], int(scale_group), out.data_ptr(), out.stride(0),
            N.ptr(scale), N.stream_ptr()), "mm_fc1_save_convert")
    N.count_launches(1)
