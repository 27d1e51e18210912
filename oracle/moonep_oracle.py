"""CPU oracle of the MoonEP load-balancing tables.  TEST INFRASTRUCTURE ONLY.

MoonEP is the reference's answer to skewed routing: before the dispatch, every rank derives
from the ``[R, E]`` matrix of per-source expert counts the same plan that (a) moves surplus
rows of an overloaded home rank to under-loaded ranks, (b) names the logical experts each
rank must hold a replica of, and (c) re-buckets every route onto ``2 * E/R`` physical slots
per rank (home slots first, replica slots after them).  This module restates those integer
tables in numpy.  It is the checker of ``mega_moe.runtime.moonep_planning`` /
``mega_moe.runtime.balanced_routing`` and of the device kernels behind them; only ``tests/``
may import it.

Reference functions restated here (paths inside the reference project):

* B.0 expert counts and home loads, B.1 single-source fill, B.2 greedy cut of each home
  group, B.3 replica slot choice      src/mega_moe/runtime/moonep_planning.py:112-236
* allocation prefix ``alloc_cumsum``    src/mega_moe/runtime/moonep_planning.py:262-276
* inverse replica table                 src/mega_moe/runtime/moonep_planning.py:279-322
* balanced count cube (interval
  overlap of source and destination
  ranges of one expert)                 src/mega_moe/runtime/balanced_routing.py:274-315
* balanced route order, buckets and
  the source-major receive offsets      src/mega_moe/runtime/balanced_routing.py:620-805

Parity pin: ``tests/golden/moonep_tables.npz`` holds outputs of those reference functions,
produced by ``tests/golden/make_golden_moonep.py``; ``tests/test_oracle_moonep.py`` checks this
module against them and against the known answers written out in the reference's
tests/function/test_moonep_planning.py:57-127 and tests/function/test_balanced_routing.py:69-120.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np

INT32_MAX = (1 << 31) - 1


@dataclass
class PlanTables:
    """``alloc_cumsum[e, d]``: routes of expert ``e`` placed on ranks ``0..d`` (inclusive
    prefix); ``experts_to_copy[d, b]``: logical expert in replica slot ``b`` of rank ``d`` or
    -1; ``allocation[d, e]``, ``transfers[h, d]`` and ``expert_count[e]`` are the intermediate
    tables of the plan."""

    expert_count: np.ndarray
    transfers: np.ndarray
    allocation: np.ndarray
    alloc_cumsum: np.ndarray
    experts_to_copy: np.ndarray

    @property
    def replica_slot_high_water(self) -> int:
        used = np.nonzero((self.experts_to_copy >= 0).any(axis=0))[0]
        return int(used.max()) + 1 if used.size else 0


def _checked_counts(tpe_all) -> tuple[np.ndarray, int, int, int, int]:
    tpe = np.asarray(tpe_all)
    if tpe.dtype not in (np.int32, np.int64):
        raise TypeError("tpe_all must have dtype int32 or int64")
    if tpe.ndim != 2:
        raise ValueError("tpe_all must have shape [world_size, num_experts]")
    world, experts = tpe.shape
    if world <= 0 or experts <= 0:
        raise ValueError("world_size and num_experts must be positive")
    if experts % world:
        raise ValueError("num_experts must be divisible by world_size")
    tpe = tpe.astype(np.int64)
    if (tpe < 0).any():
        raise ValueError("tpe_all counts must be non-negative")
    if (tpe > INT32_MAX).any():
        raise ValueError("each tpe_all count must fit in int32")
    totals = tpe.sum(axis=1)
    if (totals != totals[0]).any():
        raise ValueError("MoonEP B.0-B.3 currently requires equal route counts per source rank")
    if totals[0] > INT32_MAX:
        raise ValueError("routes per source rank must fit in int32")
    return tpe, world, experts, experts // world, int(totals[0])


def plan_tables(tpe_all) -> PlanTables:
    """B.0-B.3 of moonep_planning.py:112-276 for a ``[R, E]`` count matrix with equal rows sums."""
    tpe, world, experts, epr, capacity = _checked_counts(tpe_all)

    # B.0 (:121-135): routes per logical expert and per home rank
    expert_count = tpe.sum(axis=0)
    if (expert_count > INT32_MAX).any():
        raise ValueError("global route count for each expert must fit in int32")
    home_load = expert_count.reshape(world, epr).sum(axis=1)

    # B.1 (:137-153): the rank with the largest surplus fills the whole deficit of the rank
    # with the largest deficit (it may go negative itself and be filled later); first index
    # wins ties.  A filled rank is at zero for good, so there are at most R rounds.
    balance = home_load - capacity
    transfers = np.zeros((world, world), dtype=np.int64)
    while balance.max() > 0 and balance.min() < 0:
        giver = int(np.argmax(balance))
        taker = int(np.argmin(balance))
        amount = -int(balance[taker])
        transfers[giver, taker] = amount
        balance[giver] -= amount
        balance[taker] = 0
    if balance.any():
        raise RuntimeError("MoonEP B.1 failed to balance destination capacities")

    # B.2 (:155-186): the home rank hands out its quotas largest first, each time from the
    # local expert with the most rows left; what is left stays at home
    allocation = np.zeros((world, experts), dtype=np.int64)
    for home in range(world):
        lo = home * epr
        left = expert_count[lo:lo + epr].copy()
        quota = transfers[home].copy()
        while quota.max() > 0:
            taker = int(np.argmax(quota))
            local = int(np.argmax(left))
            if left[local] <= 0:
                raise RuntimeError("MoonEP B.2 could not satisfy a transfer quota")
            amount = min(int(quota[taker]), int(left[local]))
            quota[taker] -= amount
            left[local] -= amount
            allocation[taker, lo + local] += amount
        allocation[home, lo:lo + epr] = left
    if (allocation.sum(axis=0) != expert_count).any():
        raise RuntimeError("MoonEP B.2 violated per-expert route conservation")
    if (allocation.sum(axis=1) != capacity).any():
        raise RuntimeError("MoonEP B.2 violated destination rank capacity")

    # B.3 (:196-236): replica slots of a rank hold its remote experts with rows, most rows
    # first, the larger expert id first among equals
    experts_to_copy = np.full((world, epr), -1, dtype=np.int64)
    ids = np.arange(experts)
    for taker in range(world):
        remote = allocation[taker].copy()
        remote[taker * epr:(taker + 1) * epr] = 0
        chosen = ids[remote > 0]
        if chosen.size > epr:
            raise RuntimeError("fixed replica budget cannot cover all remote allocated experts")
        order = np.lexsort((-chosen, -remote[chosen]))  # last key first: rows desc, then id desc
        experts_to_copy[taker, :chosen.size] = chosen[order]

    alloc_cumsum = allocation.cumsum(axis=0).T
    return PlanTables(
        expert_count=expert_count,
        transfers=transfers,
        allocation=allocation,
        alloc_cumsum=np.ascontiguousarray(alloc_cumsum).astype(np.int32),
        experts_to_copy=experts_to_copy.astype(np.int32),
    )


def inverse_experts_to_copy(experts_to_copy, num_experts: int) -> np.ndarray:
    """``inverse[d, e]`` = replica slot of expert ``e`` on rank ``d`` or -1
    (moonep_planning.py:279-322)."""
    etc = np.asarray(experts_to_copy)
    world, budget = etc.shape
    if num_experts <= 0 or num_experts % world:
        raise ValueError("num_experts must be divisible by world_size")
    epr = num_experts // world
    if budget != epr:
        raise ValueError("replica budget must equal experts_per_rank")
    inverse = np.full((world, num_experts), -1, dtype=np.int32)
    for rank in range(world):
        row = etc[rank]
        used = row[row != -1]
        if ((used < 0) | (used >= num_experts)).any():
            raise ValueError("experts_to_copy contains an invalid expert id")
        if (used // epr == rank).any():
            raise ValueError("experts_to_copy must contain only remote experts")
        if np.unique(used).size != used.size:
            raise ValueError("experts_to_copy contains duplicate experts in a row")
        inverse[rank, used] = np.nonzero(row != -1)[0]
    return inverse


def physical_slot_table(inverse, epr: int) -> np.ndarray:
    """``slot[d, e]``: the physical slot (0..2*epr-1) expert ``e`` executes in on rank ``d``:
    its home slot on its owner, ``epr + replica slot`` elsewhere, -1 where it has none
    (balanced_routing.py:299-303)."""
    inverse = np.asarray(inverse).astype(np.int64)
    world, experts = inverse.shape
    ids = np.arange(experts)
    at_home = (ids // epr)[None, :] == np.arange(world)[:, None]
    return np.where(at_home, (ids % epr)[None, :], np.where(inverse >= 0, epr + inverse, -1))


def balanced_count_cube(tpe_all, alloc_cumsum, inverse) -> np.ndarray:
    """``counts[s, d * 2*epr + slot]``: rows source ``s`` sends to physical slot ``slot`` of
    rank ``d`` (balanced_routing.py:274-315).  The rows of expert ``e`` are numbered globally,
    source-major; source ``s`` owns ``[lo_s, hi_s)``, rank ``d`` executes ``[alloc_lo, alloc_hi)``;
    the cell is the length of the overlap."""
    tpe = np.asarray(tpe_all).astype(np.int64)
    hi_alloc = np.asarray(alloc_cumsum).astype(np.int64)          # [E, R]
    world, experts = tpe.shape
    epr = experts // world
    lo_alloc = np.concatenate([np.zeros((experts, 1), np.int64), hi_alloc[:, :-1]], axis=1)
    hi_src = tpe.cumsum(axis=0)                                    # [R, E]
    lo_src = hi_src - tpe
    slot = physical_slot_table(inverse, epr)                      # [R(dest), E]
    counts = np.zeros((world, world * 2 * epr), dtype=np.int64)
    for dest in range(world):
        overlap = np.minimum(hi_src, hi_alloc[:, dest][None, :]) - np.maximum(
            lo_src, lo_alloc[:, dest][None, :])
        overlap = np.clip(overlap, 0, None)                        # [R(source), E]
        for expert in range(experts):
            if slot[dest, expert] >= 0:
                counts[:, dest * 2 * epr + slot[dest, expert]] += overlap[:, expert]
            elif overlap[:, expert].any():
                raise RuntimeError("a remote allocation is missing its replica slot")
    if (counts.sum(axis=1) != tpe.sum(axis=1)).any():
        raise RuntimeError("balanced count construction lost source routes")
    return counts


@dataclass
class BalancedTables:
    """Per-rank balanced routing tables, named as the reference's ``BalancedRoutingMetadata``
    (balanced_routing.py:24-55)."""

    rank: int
    world_size: int
    num_experts: int
    experts_per_rank: int
    physical_slots_per_rank: int
    num_valid_routes: int
    valid_route_mask: np.ndarray
    final_order: np.ndarray
    send_token_indices: np.ndarray
    send_route_indices: np.ndarray
    balanced_buckets: np.ndarray
    balanced_counts: np.ndarray
    send_bucket_starts: np.ndarray
    send_bucket_receive_offsets: np.ndarray
    receive_counts_by_source_slot: np.ndarray
    received_routes_per_slot: np.ndarray
    received_slot_offsets: np.ndarray


def balanced_routing_tables(selected_experts, tpe_all, alloc_cumsum, inverse, rank: int
                            ) -> BalancedTables:
    """Route order and offset tables of one source rank (balanced_routing.py:545-805).

    Invalid expert ids are left out of the communication.  Valid routes are numbered per
    expert in stable (token, top-k slot) order, shifted by the rows of lower ranks to a
    global ordinal; the rank whose allocation interval holds that ordinal executes the route,
    in the expert's physical slot there.  The send order is bucket-major
    (``bucket = rank * 2*epr + slot``), stable inside a bucket.  The receive side stores rows
    slot-major, and inside a slot in increasing source rank."""
    selected = np.asarray(selected_experts)
    tpe = np.asarray(tpe_all).astype(np.int64)
    hi_alloc = np.asarray(alloc_cumsum).astype(np.int64)
    world, experts = tpe.shape
    epr = experts // world
    slots = 2 * epr
    top_k = selected.shape[1]

    flat = selected.reshape(-1).astype(np.int64)
    valid = (flat >= 0) & (flat < experts)
    route_ids = np.nonzero(valid)[0]
    kept = flat[valid]
    if (np.bincount(kept, minlength=experts) != tpe[rank]).any():
        raise ValueError("the valid selected_experts histogram must equal tpe_all[rank]")

    by_expert = np.argsort(kept, kind="stable")
    expert_sorted = kept[by_expert]
    first_of_expert = tpe[rank].cumsum() - tpe[rank]
    ordinal = (np.arange(kept.size) - first_of_expert[expert_sorted]
               + tpe[:rank].sum(axis=0)[expert_sorted])
    # the first rank whose inclusive prefix exceeds the ordinal
    dest = (hi_alloc[expert_sorted] <= ordinal[:, None]).sum(axis=1)
    if kept.size and (dest >= world).any():
        raise RuntimeError("a route has no destination allocation")
    slot = physical_slot_table(inverse, epr)[dest, expert_sorted]
    if kept.size and (slot < 0).any():
        raise RuntimeError("a remote route has no replica slot")
    bucket = dest * slots + slot

    by_bucket = np.argsort(bucket, kind="stable")
    final_order = route_ids[by_expert[by_bucket]]
    balanced_buckets = bucket[by_bucket]

    counts = balanced_count_cube(tpe, hi_alloc, inverse)
    own = np.bincount(balanced_buckets, minlength=world * slots)
    if (own != counts[rank]).any():
        raise RuntimeError("local route buckets disagree with balanced counts")

    cube = counts.reshape(world, world, slots)                     # [source, dest, slot]
    per_dest_slot = cube.sum(axis=0)
    slot_start = per_dest_slot.cumsum(axis=1) - per_dest_slot       # [dest, slot]
    receive_offsets = slot_start.reshape(-1) + counts[:rank].sum(axis=0)
    received = cube[:, rank, :]
    per_slot = received.sum(axis=0)

    def i32(a):
        a = np.asarray(a)
        if a.size and a.max() > INT32_MAX:
            raise ValueError("metadata exceeds the int32 range")
        return np.ascontiguousarray(a).astype(np.int32)

    return BalancedTables(
        rank=rank, world_size=world, num_experts=experts, experts_per_rank=epr,
        physical_slots_per_rank=slots, num_valid_routes=int(kept.size),
        valid_route_mask=valid,
        final_order=final_order.astype(np.int64),
        send_token_indices=i32(final_order // top_k),
        send_route_indices=i32(final_order),
        balanced_buckets=i32(balanced_buckets),
        balanced_counts=i32(counts),
        send_bucket_starts=i32(own.cumsum() - own),
        send_bucket_receive_offsets=i32(receive_offsets),
        receive_counts_by_source_slot=i32(received),
        received_routes_per_slot=i32(per_slot),
        received_slot_offsets=i32(np.concatenate([[0], per_slot.cumsum()])),
    )


def logical_to_physical_rows(tables: list[BalancedTables]) -> list[np.ndarray]:
    """For every rank, the (source rank, flattened route id) of each received row in storage
    order: slot-major, source-major inside a slot, send order inside a source's share.
    Used by tests to replay a dispatch over the balanced tables."""
    world = tables[0].world_size
    slots = tables[0].physical_slots_per_rank
    out = []
    for dest in range(world):
        total = int(tables[dest].received_slot_offsets[-1])
        rows = np.full((total, 2), -1, dtype=np.int64)
        for src in range(world):
            t = tables[src]
            for slot in range(slots):
                b = dest * slots + slot
                n = int(t.balanced_counts[src, b])
                if n == 0:
                    continue
                s0 = int(t.send_bucket_starts[b])
                r0 = int(t.send_bucket_receive_offsets[b])
                if (rows[r0:r0 + n] != -1).any():
                    raise RuntimeError("receive ranges of two sources overlap")
                rows[r0:r0 + n, 0] = src
                rows[r0:r0 + n, 1] = t.final_order[s0:s0 + n]
        if (rows < 0).any():
            raise RuntimeError("a receive row was not written")
        out.append(rows)
    return out


def forward_over_physical_slots(hidden, routing_weights, selected, w_gate, w_up, w_down,
                                num_experts: int, activation: str = "swiglu"):
    """The MoE forward executed the MoonEP way, all ranks in one process: every route goes to
    the rank and physical slot the balanced tables name, replica slots compute with a copy of
    the home rank's weights, rows come back to their source and are summed over the top-k slots
    in slot order.  Must equal the forward over logical experts (the reference makes the same
    claim with tests/function/test_moonep_logical_golden.py:21-120).

    ``hidden[r]`` [T, H] bf16, ``routing_weights[r]`` [T, k] fp32, ``selected[r]`` [T, k] int32,
    ``w_gate[r]`` / ``w_up[r]`` [E/R, F, H] and ``w_down[r]`` [E/R, H, F] bf16 per home rank.
    Returns (per-rank outputs [T, H] bf16, the per-rank BalancedTables, the PlanTables)."""
    import torch

    from oracle.moe_oracle import gated_activation

    world = len(hidden)
    epr = num_experts // world
    sel_np = [np.asarray(s.cpu().numpy()) for s in selected]
    tpe = np.stack([np.bincount(s.reshape(-1)[(s.reshape(-1) >= 0) & (s.reshape(-1) < num_experts)]
                                .astype(np.int64), minlength=num_experts) for s in sel_np])
    plan = plan_tables(tpe.astype(np.int32))
    inverse = inverse_experts_to_copy(plan.experts_to_copy, num_experts)
    tables = [balanced_routing_tables(sel_np[r], tpe, plan.alloc_cumsum, inverse, r)
              for r in range(world)]
    rows = logical_to_physical_rows(tables)
    hid = hidden[0].shape[1]
    back = [torch.zeros(sel_np[r].size, hid, dtype=torch.bfloat16) for r in range(world)]
    for dest in range(world):
        offs = tables[dest].received_slot_offsets
        for slot in range(2 * epr):
            part = rows[dest][offs[slot]:offs[slot + 1]]
            if part.shape[0] == 0:
                continue
            expert = dest * epr + slot if slot < epr else int(plan.experts_to_copy[dest, slot - epr])
            owner, local = divmod(expert, epr)
            top_k = [sel_np[s].shape[1] for s in part[:, 0]]
            x = torch.stack([hidden[s][route // k] for (s, route), k in zip(part, top_k)]).float()
            wts = torch.stack([routing_weights[s].reshape(-1)[route] for s, route in part]).float()
            gate = (x @ w_gate[owner][local].T.float()).to(torch.bfloat16)
            up = (x @ w_up[owner][local].T.float()).to(torch.bfloat16)
            act = (gated_activation(gate, up, activation) * wts[:, None]).to(torch.bfloat16)
            fc2 = (act.float() @ w_down[owner][local].T.float()).to(torch.bfloat16)
            for i, (s, route) in enumerate(part):
                back[s][route] = fc2[i]
    outs = []
    for r in range(world):
        tokens, top_k = sel_np[r].shape
        routes = back[r].view(tokens, top_k, hid)
        acc = torch.zeros(tokens, hid, dtype=torch.float32)
        for j in range(top_k):
            acc += routes[:, j].float()
        outs.append(acc.to(torch.bfloat16))
    return outs, tables, plan


def replica_pools(experts_to_copy, home_tables, fill):
    """Owner-push of replica weights (kernels/replica_weight_prefetch.py:17-180):
    ``home_tables[r]`` is rank r's ``[E/R, ...]`` array; returns per rank a ``[E/R slots, ...]``
    array whose slot b holds the home rank's entry of ``experts_to_copy[r, b]`` and ``fill``
    where the slot is empty."""
    etc = np.asarray(experts_to_copy)
    world, epr = etc.shape
    pools = []
    for dest in range(world):
        pool = np.full_like(home_tables[dest], fill)
        for slot in range(epr):
            e = int(etc[dest, slot])
            if e >= 0:
                pool[slot] = home_tables[e // epr][e % epr]
        pools.append(pool)
    return pools


def reduced_weight_grads(inverse, home_grads, replica_grads):
    """Owner-pull of replica weight gradients (kernels/replica_grad_reduce.py:62-190):
    ``home_grads[r]`` [E/R, n] and ``replica_grads[d]`` [E/R slots, n] are bf16 torch tensors;
    every home expert's gradient becomes bf16(fp32(home) + sum of its copies' gradients in fp32,
    peers in ascending rank order)."""
    import torch

    inverse = np.asarray(inverse)
    world, experts = inverse.shape
    epr = experts // world
    out = []
    for rank in range(world):
        g = home_grads[rank].clone()
        for local in range(epr):
            acc = None
            for d in range(world):
                slot = int(inverse[d, rank * epr + local])
                if d == rank or slot < 0:
                    continue
                if acc is None:
                    acc = home_grads[rank][local].float()
                acc = acc + replica_grads[d][slot].float()
            if acc is not None:
                g[local] = acc.to(torch.bfloat16)
        out.append(g)
    return out
