"""CPU oracle of the expert-parallel MoE layer.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain torch/numpy on the CPU, what the reference computes on the
path this repository accelerates.  It is the checker of the CUDA kernels: only ``tests/``,
``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` may import it; the
``mega_moe`` package never does.

All ranks of the expert-parallel group are emulated inside one process: every function
takes lists with one entry per rank and replaces each ``all_to_all_single`` of the
reference by list shuffling (:func:`_all_to_all`).

Reference functions restated here (paths inside the reference project):

* routing metadata           runtime/routing.py:635-671 (filter + stable sort),
                             runtime/routing.py:93-140 and kernels/fused_forward.py:241-304,
                             337-358, 450-480 (offset tables); closed forms as asserted by
                             tests/function/test_single_kernel_routing_metadata.py:138-194
* forward golden             tests/_moe_baselines.py:327-471   (torch_moe_fwd_golden)
* dispatch + FC1 golden      tests/_moe_baselines.py:254-324   (torch_dispatch_fc1_golden)
* differentiable forward     src/mega_moe/ops/_torch_forward.py:212-321 (moe_forward, saved)
* gated activation           src/mega_moe/ops/_torch_forward.py:177-205
* five-stage backward        tests/_moe_baselines.py:96-226    (moe_backward_torch)
* top-k reduce with drops    tests/function/test_single_kernel_reduce.py:41-77
* tolerances                 tests/_numeric.py:24-68
* saved-contract tables      src/mega_moe/ops/_torch_forward.py:103-128 (prepare_moe_metadata),
                             src/mega_moe/ops/_moonep_torch_forward.py:192-223
                             (_arrival_to_slot_permutation),
                             src/mega_moe/ops/_single_saved_adapter.py:247-340 (enrichment)

Parity pin: ``tests/golden/`` holds outputs of the reference's own functions, produced by
``tests/golden/make_golden.py`` by importing the reference in a gloo process group;
``tests/test_oracle_golden.py`` checks this module against them.
"""

from __future__ import annotations

import numpy as np
import torch
import torch.nn.functional as F

# tests/_numeric.py:24-34 of the reference
LAYOUT_RTOL = 0
LAYOUT_ATOL = 0
APPROX_RTOL = 2e-2
APPROX_ATOL = 2e-2
OUTPUT_RTOL = 4e-2
OUTPUT_ATOL = 4e-2
GRAD_RTOL = 2e-2
GRAD_ATOL = 1e-2
MIN_COSINE = 0.9999


def next_power_of_2(n: int) -> int:
    return 1 if n <= 1 else 1 << (n - 1).bit_length()


def cmp_grad(tri: torch.Tensor, gold: torch.Tensor, rtol=GRAD_RTOL, atol=GRAD_ATOL):
    """Global-max gradient rule of tests/_numeric.py:54-68: |d| <= atol + rtol * max|gold|."""
    tri = tri.float()
    gold = gold.float()
    d = (tri - gold).abs()
    max_d = float(d.max().item()) if d.numel() else 0.0
    gmax = float(gold.abs().max().item()) if gold.numel() else 0.0
    n_bad = int((d > atol + rtol * gmax).sum().item())
    return n_bad == 0, max_d, max_d / (gmax + 1e-9), n_bad


def cosine(a: torch.Tensor, b: torch.Tensor) -> float:
    a = a.double().flatten()
    b = b.double().flatten()
    na, nb = a.norm(), b.norm()
    if na == 0 and nb == 0:
        return 1.0
    return float((a @ b) / (na * nb + 1e-300))


# ---------------------------------------------------------------------------------------
# routing metadata
# ---------------------------------------------------------------------------------------
def routing_metadata(selected: list[np.ndarray], num_experts: int):
    """Per-rank routing tables for ``selected[r]`` ([T_r, k] int32 expert ids).

    Returns a list of dicts (one per rank) of int32 numpy arrays with the reference's
    definitions; bucket id = global expert id = dst_rank * EPR + local_expert.
    """
    world = len(selected)
    epr = num_experts // world
    bins = next_power_of_2(num_experts)
    cube = np.zeros((world, bins), dtype=np.int64)
    local = []
    for r in range(world):
        sel = np.asarray(selected[r]).astype(np.int64)
        tokens, top_k = sel.shape
        flat = sel.reshape(-1)
        valid = (flat >= 0) & (flat < num_experts)
        kept_routes = np.nonzero(valid)[0]
        kept_experts = flat[kept_routes]
        order = np.argsort(kept_experts, kind="stable")
        send_route = kept_routes[order]
        send_bucket = kept_experts[order]
        route_to_send = np.full(flat.shape[0], -1, dtype=np.int64)
        route_to_send[send_route] = np.arange(send_route.shape[0])
        cube[r, :num_experts] = np.bincount(kept_experts, minlength=num_experts)
        local.append(dict(
            send_route_indices=send_route, send_token_indices=send_route // top_k,
            send_bucket=send_bucket, route_to_send=route_to_send, stable_sort_indices=order,
            valid_route_mask=valid, num_sent_routes=int(send_route.shape[0]),
        ))
    out = []
    for r in range(world):
        d = dict(local[r])
        d.update(count_cube=cube.copy())
        d.update(offset_tables_from_cube(cube[:, :num_experts], r, epr))
        out.append({k: (v.astype(np.int32) if isinstance(v, np.ndarray) and v.dtype == np.int64
                        else v) for k, v in d.items()})
    return out


def offset_tables_from_cube(cube, r: int, epr: int) -> dict:
    """Send- and receive-side offset tables of rank ``r`` from the replicated count cube
    ``cube[source, bucket]`` with ``bucket = dst_rank * epr + slot`` (int64 arrays).  With the
    logical counts and ``epr = E/R`` these are the tables of runtime/routing.py:93-140; with the
    MoonEP-balanced cube and ``epr = 2 * E/R`` physical slots they are the balanced tables of
    runtime/balanced_routing.py:760-783."""
    cube = np.asarray(cube).astype(np.int64)
    world = cube.shape[0]
    num_buckets = world * epr
    dst_totals = np.array([cube[:, d * epr:(d + 1) * epr].sum() for d in range(world)])
    row = cube[r, :num_buckets]
    send_bucket_starts = np.cumsum(row) - row
    dst_starts = np.zeros(num_buckets, dtype=np.int64)
    for d in range(world):
        block = cube[:, d * epr:(d + 1) * epr]
        sums = block.sum(0)
        dst_starts[d * epr:(d + 1) * epr] = (np.cumsum(sums) - sums) + block[:r].sum(0)
    recv_counts_re = cube[:, r * epr:(r + 1) * epr].copy()            # [W, EPR]
    recv_per_expert = recv_counts_re.sum(0)
    recv_expert_offs = np.r_[0, np.cumsum(recv_per_expert)]
    recv_seg_starts = np.column_stack(
        (np.zeros(epr, dtype=np.int64), np.cumsum(recv_counts_re.T, axis=1)))  # [EPR, W+1]
    pull = np.zeros((epr, world), dtype=np.int64)
    for s in range(world):
        excl = np.cumsum(cube[s]) - cube[s]
        pull[:, s] = excl[r * epr:(r + 1) * epr]
    stats = np.r_[recv_per_expert.sum(), dst_totals.max(), dst_totals]
    # receive order: expert-major, source-major, then the source's send order
    row_src_rank = np.zeros(int(recv_per_expert.sum()), dtype=np.int64)
    row_src_pos = np.zeros_like(row_src_rank)
    for e in range(epr):
        for s in range(world):
            c = recv_counts_re[s, e]
            start = recv_expert_offs[e] + recv_seg_starts[e, s]
            row_src_rank[start:start + c] = s
            row_src_pos[start:start + c] = pull[e, s] + np.arange(c)
    return dict(
        send_bucket_starts=send_bucket_starts, send_bucket_dst_starts=dst_starts,
        recv_counts_re=recv_counts_re, recv_per_expert=recv_per_expert,
        recv_expert_offs=recv_expert_offs, recv_seg_starts=recv_seg_starts,
        pull_dst_start=pull.reshape(-1), stats=stats, row_src_rank=row_src_rank,
        row_src_pos=row_src_pos, num_received_routes=int(recv_per_expert.sum()),
    )


SAVED_TILE_ROWS = 64   # BLOCK_SIZE_M of ops/_torch_forward.py:28


def tile_metadata(expert_counts):
    """prepare_moe_metadata (ops/_torch_forward.py:103-128): per 64-row tile of the grouped
    GEMMs its expert, the expert's first row, the tile's index inside the expert and the
    expert's first tile; plus the row prefix and the tile total.  int32 numpy arrays."""
    counts = np.asarray(expert_counts).astype(np.int64)
    tiles = (counts + SAVED_TILE_ROWS - 1) // SAVED_TILE_ROWS
    token_starts = np.cumsum(counts) - counts
    tile_starts = np.cumsum(tiles) - tiles
    i32 = lambda a: np.asarray(a).astype(np.int32)
    total = int(tiles.sum())
    return dict(
        split_size_cum_per_expert=i32(np.r_[0, np.cumsum(counts)]),
        meta_expert_ids=i32(np.repeat(np.arange(counts.shape[0]), tiles)),
        meta_split_cum=i32(np.repeat(token_starts, tiles)),
        meta_tile_num=i32(np.arange(total) - np.repeat(tile_starts, tiles)),
        meta_tile_num_cum=i32(np.repeat(tile_starts, tiles)),
        num_tiles_total=i32([total]),
    )


def arrival_to_slot_permutation(recv_counts_re, slot_starts):
    """_arrival_to_slot_permutation (ops/_moonep_torch_forward.py:192-223): entry p of the
    result is the arrival index (source-major, inside a source expert-major) of the row at
    position p of the receive order (expert-major, inside an expert source-major)."""
    counts = np.asarray(recv_counts_re).astype(np.int64)            # [W, EPR]
    source_totals = counts.sum(1)
    source_starts = np.cumsum(source_totals) - source_totals
    within_source = np.cumsum(counts, axis=1) - counts
    within_slot = np.cumsum(counts, axis=0) - counts
    arrival_start = source_starts[:, None] + within_source
    sorted_start = np.asarray(slot_starts).astype(np.int64)[None, :] + within_slot
    perm = np.zeros(int(counts.sum()), dtype=np.int64)
    for s in range(counts.shape[0]):
        for e in range(counts.shape[1]):
            c = counts[s, e]
            perm[sorted_start[s, e]:sorted_start[s, e] + c] = arrival_start[s, e] + np.arange(c)
    return perm


def saved_contract_tables(meta_r: dict, selected_r, world: int):
    """The index section the fused forward's saved dict carries after enrichment
    (ops/_single_saved_adapter.py:247-340) for one rank, from its routing tables: the
    forward's own send order as ``sort_idxs``, its inverse, the arrival permutation pair,
    the per-rank split lists and the 64-row tile tables.  Dropless routes only."""
    flat = np.asarray(selected_r).reshape(-1).astype(np.int64)
    send_route = meta_r["send_route_indices"].astype(np.int64)
    if send_route.shape[0] != flat.shape[0]:
        raise ValueError("droless routing required for the saved contract")
    counts_re = meta_r["recv_counts_re"].astype(np.int64)
    epr = counts_re.shape[1]
    local = arrival_to_slot_permutation(counts_re, meta_r["recv_expert_offs"][:-1])
    out = dict(
        sort_idxs=send_route, inv_sort=np.argsort(send_route, kind="stable"),
        forward_send_route=send_route.astype(np.int32),
        local_sort_idxs=local, inv_local=np.argsort(local, kind="stable"),
        splits_send_list=np.bincount(flat // epr, minlength=world).tolist(),
        splits_recv_list=counts_re.sum(1).tolist(),
        expert_counts=counts_re.sum(0).astype(np.int32),
    )
    out.update(tile_metadata(counts_re.sum(0)))
    return out


def receive_sources(meta: list[dict]):
    """For every rank: (source rank, flat route id on the source) of each received row."""
    out = []
    for m in meta:
        src = m["row_src_rank"].astype(np.int64)
        pos = m["row_src_pos"].astype(np.int64)
        route = np.array([meta[s]["send_route_indices"][p] for s, p in zip(src, pos)],
                         dtype=np.int64)
        out.append((src, route))
    return out


def topk_reduce(rows: torch.Tensor, route_to_send: np.ndarray, tokens: int, top_k: int):
    """out[t] = bf16(sum_j fp32(rows[route_to_send[t*k+j]])) in slot order, -1 skipped."""
    hidden = rows.shape[1]
    out = torch.zeros(tokens, hidden, dtype=torch.float32)
    idx = torch.as_tensor(np.asarray(route_to_send).astype(np.int64)).view(tokens, top_k)
    for j in range(top_k):
        col = idx[:, j]
        ok = col >= 0
        contrib = torch.zeros(tokens, hidden, dtype=torch.float32)
        contrib[ok] = rows[col[ok]].float()
        out += contrib
    return out.to(torch.bfloat16)


# ---------------------------------------------------------------------------------------
# all-to-all emulation
# ---------------------------------------------------------------------------------------
def _all_to_all(send: list[torch.Tensor], send_splits: list[list[int]]):
    """recv[d] = concat over sources s of the chunk of send[s] destined to d."""
    world = len(send)
    chunks = []
    for s in range(world):
        offs = np.r_[0, np.cumsum(send_splits[s])]
        chunks.append([send[s][offs[d]:offs[d + 1]] for d in range(world)])
    return [torch.cat([chunks[s][d] for s in range(world)], dim=0) for d in range(world)]


def gated_activation(gate, up, activation="swiglu", situ_beta=1.0, situ_linear_beta=None,
                     clamp_limit=7.0):
    """fp32 gated activation (ops/_torch_forward.py:177-205)."""
    gate = gate.float()
    up = up.float()
    if activation == "swiglu":
        return F.silu(gate) * up
    if activation == "clamp_swiglu":
        return F.silu(gate.clamp(max=clamp_limit)) * up.clamp(min=-clamp_limit, max=clamp_limit)
    if activation == "situglu":
        a = situ_beta * torch.tanh(gate / situ_beta) * torch.sigmoid(gate)
        if situ_linear_beta is not None:
            up = situ_linear_beta * torch.tanh(up / situ_linear_beta)
        return a * up
    raise ValueError(f"unknown activation {activation!r}")


# ---------------------------------------------------------------------------------------
# forward golden (fp32 routing weights, fp32 matmul, bf16 rounding points)
# ---------------------------------------------------------------------------------------
@torch.no_grad()
def forward_golden(hidden, routing_weights, selected, w_gate, w_up, w_down, num_experts,
                   activation="swiglu", situ_beta=1.0, situ_linear_beta=None, clamp_limit=7.0,
                   return_intermediates=False):
    """Independent forward (tests/_moe_baselines.py:327-471) for all ranks at once.

    Per rank r: hidden[r] [T,H] bf16, routing_weights[r] [T,k] fp32, selected[r] [T,k] int,
    w_gate[r] / w_up[r] [EPR,F,H] bf16, w_down[r] [EPR,H,F] bf16.  Returns the per-rank
    outputs [T,H] bf16 (and, on request, per-rank grouped intermediates).
    """
    world = len(hidden)
    epr = num_experts // world
    tokens_send, weights_send, experts_send, splits, rank_sorts, valid_idx = [], [], [], [], [], []
    for r in range(world):
        x = hidden[r]
        top_k = selected[r].shape[1]
        rep = x.repeat_interleave(top_k, dim=0)
        flat_w = routing_weights[r].reshape(-1)
        flat_e = selected[r].reshape(-1).long()
        valid = torch.where((flat_e >= 0) & (flat_e < num_experts))[0]
        e_valid = flat_e[valid]
        dest = (e_valid // epr)
        rank_sort = torch.argsort(dest, stable=True)
        tokens_send.append(rep[valid][rank_sort].contiguous())
        weights_send.append(flat_w[valid][rank_sort].contiguous())
        experts_send.append(e_valid[rank_sort].contiguous())
        splits.append(torch.bincount(dest, minlength=world).tolist())
        rank_sorts.append(rank_sort)
        valid_idx.append(valid)
    tokens_recv = _all_to_all(tokens_send, splits)
    weights_recv = _all_to_all(weights_send, splits)
    experts_recv = _all_to_all(experts_send, splits)

    fc2_back, inter = [], []
    for d in range(world):
        local_e = experts_recv[d] % epr
        local_sort = torch.argsort(local_e, stable=True)
        tok = tokens_recv[d][local_sort]
        wts = weights_recv[d][local_sort]
        eg = local_e[local_sort]
        total = tok.shape[0]
        ffn = w_gate[d].shape[1]
        hid = tok.shape[1] if total else hidden[d].shape[1]
        gate_out = torch.zeros(total, ffn, dtype=torch.bfloat16)
        up_out = torch.zeros(total, ffn, dtype=torch.bfloat16)
        for le in range(epr):
            mask = eg == le
            if not bool(mask.any()):
                continue
            xin = tok[mask].float()
            gate_out[mask] = (xin @ w_gate[d][le].T.float()).to(torch.bfloat16)
            up_out[mask] = (xin @ w_up[d][le].T.float()).to(torch.bfloat16)
        act = (gated_activation(gate_out, up_out, activation, situ_beta, situ_linear_beta,
                                clamp_limit) * wts.float()[:, None]).to(torch.bfloat16)
        fc2 = torch.zeros(total, hid, dtype=torch.bfloat16)
        for le in range(epr):
            mask = eg == le
            if not bool(mask.any()):
                continue
            fc2[mask] = (act[mask].float() @ w_down[d][le].T.float()).to(torch.bfloat16)
        inv = torch.argsort(local_sort)
        fc2_back.append(fc2[inv].contiguous())
        inter.append(dict(tokens_grouped=tok, weights_grouped=wts, experts_grouped=eg,
                          gate=gate_out, up=up_out, act=act, fc2=fc2))
    # reverse all-to-all: rank d returns to source s the rows it received from s
    recv_splits = [[splits[s][d] for s in range(world)] for d in range(world)]
    combined = _all_to_all(fc2_back, recv_splits)
    outs = []
    for r in range(world):
        tokens, top_k = selected[r].shape
        hid = hidden[r].shape[1]
        inv_rank_sort = torch.argsort(rank_sorts[r])
        routes = torch.zeros(tokens * top_k, hid, dtype=torch.bfloat16)
        routes[valid_idx[r]] = combined[r][inv_rank_sort]
        routes = routes.view(tokens, top_k, hid)
        acc = torch.zeros(tokens, hid, dtype=torch.float32)
        for j in range(top_k):
            acc += routes[:, j].float()
        outs.append(acc.to(torch.bfloat16))
    if return_intermediates:
        return outs, inter
    return outs


# ---------------------------------------------------------------------------------------
# differentiable-forward restatement with the saved dict of the five-stage backward
# ---------------------------------------------------------------------------------------
def _grouped_matmul(a, weight, counts, transpose=True):
    """ops/_torch_forward.py:43-67 (the 256-row zero padding there does not change values)."""
    parts = []
    start = 0
    for e in range(weight.shape[0]):
        cnt = int(counts[e])
        if cnt > 0:
            slc = a[start:start + cnt]
            w = weight[e]
            parts.append((slc @ w.T) if transpose else (slc @ w))
            start += cnt
    if not parts:
        return torch.zeros(a.shape[0], weight.shape[1] if transpose else weight.shape[2],
                           dtype=a.dtype)
    return torch.cat(parts, dim=0)


def _grouped_transposed_matmul(grad_out, orig_in, counts):
    """ops/_torch_forward.py:70-92."""
    n_exp = len(counts)
    out = torch.zeros(n_exp, grad_out.shape[1], orig_in.shape[1], dtype=grad_out.dtype)
    start = 0
    for e in range(n_exp):
        cnt = int(counts[e])
        if cnt > 0:
            out[e] = grad_out[start:start + cnt].T @ orig_in[start:start + cnt]
            start += cnt
    return out


@torch.no_grad()
def forward_saved(hidden, routing_weights, selected, fc1_1, fc1_2, fc2, top_k,
                  activation="swiglu", situ_beta=1.0, situ_linear_beta=None, clamp_limit=7.0):
    """moe_forward(return_saved=True) of ops/_torch_forward.py:212-321 for all ranks.

    No route dropping (the saved contract is dropless).  Matmuls run in the input dtype, the
    received routing weights are cast to it, exactly as in the reference.
    """
    world = len(hidden)
    epr = fc1_1[0].shape[0]
    dtype = hidden[0].dtype
    st = []
    for r in range(world):
        x = hidden[r]
        expanded = x.repeat_interleave(top_k, dim=0)
        flat_w = routing_weights[r].reshape(-1)
        flat_i = selected[r].reshape(-1).to(torch.int64)
        expert_ranks = flat_i // epr
        local_experts = flat_i % epr
        send_counts = torch.bincount(expert_ranks, minlength=world)
        sort_idxs = torch.argsort(expert_ranks, stable=True)
        st.append(dict(sort_idxs=sort_idxs, splits_send=send_counts.tolist(),
                       sorted_hidden=expanded[sort_idxs],
                       sorted_weights=flat_w[sort_idxs].to(dtype),
                       sorted_local=local_experts[sort_idxs]))
    splits = [s["splits_send"] for s in st]
    tokens_recv = _all_to_all([s["sorted_hidden"] for s in st], splits)
    weights_recv = _all_to_all([s["sorted_weights"] for s in st], splits)
    ids_recv = _all_to_all([s["sorted_local"] for s in st], splits)
    saved, fc2_unsorted = [], []
    for d in range(world):
        local_ids = ids_recv[d] % epr
        local_sort = torch.argsort(local_ids, stable=True)
        recv_hidden_sorted = tokens_recv[d][local_sort]
        recv_weights_sorted = weights_recv[d][local_sort]
        counts = torch.bincount(local_ids, minlength=epr).to(torch.int32)
        fc1_combined = torch.cat([fc1_1[d], fc1_2[d]], dim=1)
        fc1_out = _grouped_matmul(recv_hidden_sorted, fc1_combined, counts, transpose=True)
        gate, up = fc1_out.chunk(2, dim=-1)
        act = gated_activation(gate, up, activation, situ_beta, situ_linear_beta, clamp_limit)
        act_w = (act * recv_weights_sorted.float().unsqueeze(-1)).to(dtype)
        fc2_out = _grouped_matmul(act_w, fc2[d], counts, transpose=True)
        inv_local = torch.argsort(local_sort)
        fc2_unsorted.append(fc2_out[inv_local])
        offs = torch.zeros(epr + 1, dtype=torch.int32)
        offs[1:] = counts.cumsum(0)
        saved.append(dict(
            local_sort_idxs=local_sort, inv_local=inv_local,
            splits_recv_list=[splits[s][d] for s in range(world)],
            total_recv=int(counts.sum()), M=int(counts.sum()), expert_counts=counts,
            split_size_cum_per_expert=offs,
            recv_hidden_sorted=recv_hidden_sorted, fc1_output=fc1_out, gate=gate, up=up,
            swiglu_out_weighted=act_w, recv_weights_sorted=recv_weights_sorted, fc2_out=fc2_out,
            activation=activation, situ_beta=situ_beta, situ_linear_beta=situ_linear_beta,
            clamp_limit=clamp_limit,
            fc1_1=fc1_1[d], fc1_2=fc1_2[d], fc2=fc2[d], fc1_combined=fc1_combined,
        ))
    recv_splits = [[splits[s][d] for s in range(world)] for d in range(world)]
    combined = _all_to_all(fc2_unsorted, recv_splits)
    outs = []
    for r in range(world):
        tokens, hid = hidden[r].shape
        inv_sort = torch.argsort(st[r]["sort_idxs"])
        full = combined[r][inv_sort]
        out = full.view(tokens, top_k, hid).sum(dim=1)
        outs.append(out)
        saved[r].update(
            output=out, dy=None, batch_size=tokens, hidden_dim=hid,
            ffn_dim=fc1_1[r].shape[1], num_experts=epr * world, experts_per_rank=epr,
            topk=top_k, world_size=world, ep_rank=r, ep_group=None,
            sort_idxs=st[r]["sort_idxs"], inv_sort=inv_sort,
            splits_send_list=st[r]["splits_send"], total_send=int(sum(st[r]["splits_send"])),
            selected_experts=selected[r],
        )
    return outs, saved


@torch.no_grad()
def swiglu_bwd(grad_swiglu, s):
    """Stage 2 (tests/_moe_baselines.py:122-160)."""
    gate = s["gate"].float()
    up = s["up"].float()
    scale = s["recv_weights_sorted"].float().unsqueeze(-1)
    g = grad_swiglu.float()
    act = s.get("activation", "swiglu")
    if act == "situglu":
        beta = float(s.get("situ_beta") or 1.0)
        lb = s.get("situ_linear_beta")
        t = torch.tanh(gate / beta)
        sg = torch.sigmoid(gate)
        act_g = beta * t * sg
        act_p = (1 - t * t) * sg + beta * t * sg * (1 - sg)
        if lb is not None:
            tu = torch.tanh(up / float(lb))
            v, v_p = float(lb) * tu, 1 - tu * tu
        else:
            v, v_p = up, torch.ones_like(up)
    elif act == "clamp_swiglu":
        # derivative of kernels/swiglu_bwd.py:58-64 (clamp flat regions have zero slope)
        lim = float(s.get("clamp_limit") or 7.0)
        gc = gate.clamp(max=lim)
        sg = torch.sigmoid(gc)
        act_g = gc * sg
        act_p = (sg + gc * sg * (1 - sg)) * (gate <= lim).float()
        v = up.clamp(min=-lim, max=lim)
        v_p = (up.abs() <= lim).float()
    else:
        sg = torch.sigmoid(gate)
        act_g = gate * sg
        act_p = act_g * (1 - sg) + sg
        v, v_p = up, torch.ones_like(up)
    d_gate = g * act_p * v * scale
    d_up = g * act_g * v_p * scale
    grad_fc1_output = torch.cat([d_gate, d_up], dim=-1).to(grad_swiglu.dtype)
    grad_gate = (act_g * v * g).sum(dim=-1).to(grad_swiglu.dtype)
    return grad_fc1_output, grad_gate


# ---------------------------------------------------------------------------------------
# router in front of the layer
# ---------------------------------------------------------------------------------------
@torch.no_grad()
def router_topk(logits: torch.Tensor, top_k: int):
    """Post-router inputs as the reference's benchmark builds them
    (benchmark/layer/bench_moe_suite.py:487-497): top-k of the logits (descending; a stable
    sort makes ties go to the lower expert id) and the fp32 softmax over the selected logits."""
    order = torch.sort(logits.float(), dim=-1, descending=True, stable=True).indices[:, :top_k]
    picked = torch.gather(logits.float(), 1, order)
    return order.to(torch.int32), F.softmax(picked, dim=-1)


# ---------------------------------------------------------------------------------------
# saved-activation formats and the recompute backward.  The reference implements these only
# in its Triton-Ascend kernels, which cannot be launched here; their arithmetic is plain ``tl``
# tensor code, so tests/golden/make_golden_saved.py executes the reference's own source text
# (the FC1 save leg, kernels/fused_forward.py:891-949, and _recompute_act_rows,
# kernels/mega_bwd.py:1414-1465) against a torch-backed stand-in for ``tl`` and stores the
# results in tests/golden/saved_formats.npz; tests/test_oracle_formats.py requires the four
# functions below to reproduce them bit-exactly (formulas, operation order, rounding points
# and table layout are pinned; the Ascend vector unit's own sigmoid/tanh are not).
# ---------------------------------------------------------------------------------------
FP8_E4M3_MAX = 448.0


@torch.no_grad()
def quantize_fc1_fp8(raw: torch.Tensor, group_n: int):
    """fp8 E4M3 save of raw FC1 rows [rows, 2F] (kernels/fused_forward.py:905-949): one fp32
    scale per row and per ``group_n`` columns; q = e4m3(x * (448 / amax)), scale = amax / 448;
    an all-zero group keeps q = 0 and the scale 1 / 448."""
    rows, cols = raw.shape
    x = raw.float().view(rows, cols // group_n, group_n)
    amax = x.abs().amax(dim=-1)
    safe = torch.where(amax > 0, amax, torch.ones_like(amax))
    inv = torch.tensor(FP8_E4M3_MAX, dtype=torch.float32) / safe
    q = (x * inv[:, :, None]).to(torch.float8_e4m3fn).view(rows, cols)
    return q, safe / torch.tensor(FP8_E4M3_MAX, dtype=torch.float32)


@torch.no_grad()
def dequantize_fc1(fc1: torch.Tensor, scale=None, group_n: int = 0) -> torch.Tensor:
    """fp32 values of saved FC1 rows in any format, as the backward loads them
    (kernels/mega_bwd.py:1436-1443, 3187-3205)."""
    if fc1.dtype != torch.float8_e4m3fn:
        return fc1.float()
    rows, cols = fc1.shape
    return (fc1.float().view(rows, cols // group_n, group_n) * scale[:, :, None]).view(rows, cols)


@torch.no_grad()
def convert_fc1_fp16(raw: torch.Tensor) -> torch.Tensor:
    """fp16 save: a plain copy of the raw values (kernels/fused_forward.py:893-904)."""
    return raw.to(torch.float16)


@torch.no_grad()
def recompute_act(gate, up, recv_weights_bf16, activation="swiglu", situ_beta=1.0,
                  situ_linear_beta=None, clamp_limit=7.0, dtype=torch.bfloat16):
    """Backward-side recompute of the weighted activation rows from saved FC1 values and the
    saved bf16 routing weights (kernels/mega_bwd.py:1408-1465): fp32 intermediates, one
    rounding at the store."""
    act = gated_activation(gate, up, activation, situ_beta or 1.0, situ_linear_beta,
                           clamp_limit or 7.0)
    return (act * recv_weights_bf16.float().unsqueeze(-1)).to(dtype)


@torch.no_grad()
def backward(saved: list[dict], dys: list[torch.Tensor]):
    """Five-stage backward (tests/_moe_baselines.py:96-226) for all ranks."""
    world = len(saved)
    dtype = saved[0]["output"].dtype
    send_splits = [s["splits_send_list"] for s in saved]
    recv_splits = [s["splits_recv_list"] for s in saved]
    top_k = saved[0]["topk"]
    # stage 1a: un-reduce, rank sort, dispatch all-to-all, local sort
    flat = [dys[r].to(dtype).repeat_interleave(top_k, dim=0)[saved[r]["sort_idxs"]]
            for r in range(world)]
    unsorted = _all_to_all(flat, send_splits)
    res = []
    ret_rows, ret_gate = [], []
    for d in range(world):
        s = saved[d]
        g_fc2_out = unsorted[d][s["local_sort_idxs"]]
        counts = s["expert_counts"]
        grad_swiglu = _grouped_matmul(g_fc2_out, s["fc2"], counts, transpose=False)    # 1b
        grad_fc1_output, grad_gate = swiglu_bwd(grad_swiglu, s)                         # 2
        grad_fc2 = _grouped_transposed_matmul(g_fc2_out, s["swiglu_out_weighted"], counts)  # 3
        g_recv_hidden = _grouped_matmul(grad_fc1_output, s["fc1_combined"], counts,
                                        transpose=False)                                # 4a
        grad_fc1 = _grouped_transposed_matmul(grad_fc1_output, s["recv_hidden_sorted"], counts)
        g1, g2 = torch.chunk(grad_fc1, 2, dim=1)                                        # 5
        ret_rows.append(g_recv_hidden[s["inv_local"]])
        ret_gate.append(grad_gate[s["inv_local"]])
        res.append(dict(grad_fc2_out_sorted=g_fc2_out, grad_swiglu=grad_swiglu,
                        grad_fc1_output=grad_fc1_output, grad_gate=grad_gate, grad_fc2=grad_fc2,
                        grad_recv_hidden_sorted=g_recv_hidden, grad_fc1=grad_fc1,
                        grad_fc1_1=g1, grad_fc1_2=g2))
    back_rows = _all_to_all(ret_rows, recv_splits)                                      # 4b
    back_gate = _all_to_all(ret_gate, recv_splits)
    for r in range(world):
        s = saved[r]
        tokens, hid = s["batch_size"], s["hidden_dim"]
        full = back_rows[r][s["inv_sort"]]
        res[r]["grad_hidden"] = full.view(tokens, top_k, hid).sum(dim=1)
        res[r]["grad_routing_weights"] = back_gate[r][s["inv_sort"]].view(tokens, top_k)
    return res


@torch.no_grad()
def dispatch_fc1_golden(hidden, selected, w1, num_experts):
    """Dispatch + FC1 without activation (tests/_moe_baselines.py:254-324), all ranks.

    w1[r] is the logical [EPR, N, H] weight.  Returns per rank (fc1 [M,N] bf16,
    local expert per row, dispatched tokens [M,H]) in expert-grouped receive order.
    """
    world = len(hidden)
    epr = num_experts // world
    xs, es, splits = [], [], []
    for r in range(world):
        tokens, top_k = selected[r].shape
        flat_e = selected[r].reshape(-1).long()
        row_tok = torch.arange(tokens).repeat_interleave(top_k)
        keep = (flat_e >= 0) & (flat_e < num_experts)
        e_keep = flat_e[keep]
        dest = e_keep // epr
        order = torch.argsort(dest, stable=True)
        xs.append(hidden[r][row_tok[keep]][order].contiguous())
        es.append((e_keep % epr)[order].contiguous())
        splits.append(torch.bincount(dest, minlength=world).tolist())
    x_recv = _all_to_all(xs, splits)
    e_recv = _all_to_all(es, splits)
    out = []
    for d in range(world):
        order = torch.argsort(e_recv[d], stable=True)
        xg = x_recv[d][order]
        eg = e_recv[d][order]
        res = torch.zeros(xg.shape[0], w1[d].shape[1], dtype=torch.bfloat16)
        for le in range(epr):
            mask = eg == le
            if bool(mask.any()):
                res[mask] = (xg[mask].float() @ w1[d][le].T.float()).to(torch.bfloat16)
        out.append((res, eg.to(torch.int32), xg))
    return out


# ---------------------------------------------------------------------------------------
# seeded synthetic inputs
# ---------------------------------------------------------------------------------------
def make_inputs(world, tokens, hidden, ffn, num_experts, top_k, seed=0, dtype=torch.bfloat16,
                expert_bias=None, drop_frac=0.0, weight_std=0.02):
    """Per-rank synthetic inputs: x ~ N(0,1), router logits ~ N(0,1) (+ per-expert bias),
    softmax over the selected logits as fp32 routing weights, weights ~ N(0, weight_std)."""
    epr = num_experts // world
    out = dict(hidden=[], routing_weights=[], selected=[], w_gate=[], w_up=[], w_down=[], dy=[])
    for r in range(world):
        g = torch.Generator().manual_seed(1000 * seed + 17 * r + 1)
        x = torch.randn(tokens, hidden, generator=g).to(dtype)
        logits = torch.randn(tokens, num_experts, generator=g)
        if expert_bias is not None:
            logits = logits + expert_bias[None, :]
        top_v, top_i = torch.topk(logits, top_k, dim=-1)
        rw = torch.softmax(top_v, dim=-1).float().contiguous()
        sel = top_i.to(torch.int32).contiguous()
        if drop_frac > 0:
            drop = torch.rand(tokens, top_k, generator=g) < drop_frac
            sel = sel.masked_fill(drop, num_experts)
        out["hidden"].append(x)
        out["routing_weights"].append(rw)
        out["selected"].append(sel)
        out["w_gate"].append((torch.randn(epr, ffn, hidden, generator=g) * weight_std).to(dtype))
        out["w_up"].append((torch.randn(epr, ffn, hidden, generator=g) * weight_std).to(dtype))
        out["w_down"].append((torch.randn(epr, hidden, ffn, generator=g) * weight_std).to(dtype))
        out["dy"].append(torch.randn(tokens, hidden, generator=g).to(dtype))
    return out


KIMI_OWNER_LOADS = (19, 27, 11, 11, 15, 15, 15, 15)   # routes per owner rank out of every 128


def kimi_skewed_routes(tokens: int, num_experts: int, top_k: int, rank: int) -> torch.Tensor:
    """Deterministic skewed routes of the reference's benchmark
    (benchmark/layer/_kimi_routes.py:7-40): out of every 128 consecutive routes of a rank,
    owner rank o receives KIMI_OWNER_LOADS[o]; a token never repeats an expert.

    The 128 routes span ``period = 128 // top_k`` tokens.  Token phase p sends
    ``load // period`` routes to each owner, and the remainders are handed out one at a time,
    owner after owner, to phases 0, 1, 2, ... cyclically.  Within an owner the experts are taken
    round-robin from a cursor that starts at ``rank % experts_per_owner``.
    """
    world = len(KIMI_OWNER_LOADS)
    if top_k not in (8, 16) or num_experts % world:
        raise ValueError("Kimi skewed routes require W8 and top-k 8 or 16")
    period = sum(KIMI_OWNER_LOADS) // top_k
    if tokens % period:
        raise ValueError("tokens must contain whole Kimi owner periods")
    per_owner = num_experts // world
    loads = np.asarray(KIMI_OWNER_LOADS)
    quota = np.tile(loads // period, (period, 1))                  # [phase, owner]
    handed = 0
    for owner, rest in enumerate(loads % period):
        for _ in range(int(rest)):
            quota[handed % period, owner] += 1
            handed += 1
    if quota.max() > per_owner:
        raise ValueError("too few local experts for distinct per-token choices")
    per_token = quota[np.arange(tokens) % period]                  # [token, owner]
    start = rank % per_owner + np.cumsum(per_token, axis=0) - per_token   # cursor before the token
    routes = np.empty((tokens, top_k), dtype=np.int32)
    col = np.zeros(tokens, dtype=np.int64)
    rows = np.arange(tokens)
    for owner in range(world):
        for j in range(int(quota[:, owner].max())):
            take = per_token[:, owner] > j
            routes[rows[take], col[take]] = owner * per_owner + (start[take, owner] + j) % per_owner
            col[take] += 1
    return torch.from_numpy(routes)


def zipf_expert_bias(num_experts: int, s: float, seed: int = 7) -> torch.Tensor:
    """Per-expert router bias 2*log(1/rank^s) over a seeded expert permutation."""
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(num_experts, generator=g)
    rank = torch.empty(num_experts)
    rank[perm] = torch.arange(1, num_experts + 1, dtype=torch.float32)
    return 2.0 * torch.log(1.0 / rank.pow(s))
