"""Generate ``moonep_tables.npz`` from the reference itself.

    python tests/golden/make_golden_moonep.py /path/to/reference

Runs the reference's host implementations on the CPU, imported by file path (the package's
``__init__`` needs the Ascend toolchain, these two modules only need torch and an importable
``triton``):

* ``plan_moonep_b0_b3`` and ``build_inverse_experts_to_copy``
  (src/mega_moe/runtime/moonep_planning.py:239-322)
* ``build_balanced_routing_metadata`` (src/mega_moe/runtime/balanced_routing.py:545-805), in
  its stable-sort form and in its direct-scatter form; the script checks that both agree
  before it stores one of them.

Inputs are generated here from seeds and stored in the fixture next to the outputs, so the
fixture is self-contained.  Small cases store every table; the large ones (real expert counts,
thousands of routes per rank) store the planning tables in full and a SHA-256 digest of each
per-rank routing table.
"""

from __future__ import annotations

import hashlib
import importlib.util
import os
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent

FIELDS = (
    "final_order", "send_token_indices", "send_route_indices", "balanced_buckets",
    "balanced_counts", "send_bucket_starts", "send_bucket_receive_offsets",
    "receive_counts_by_source_slot", "received_routes_per_slot", "received_slot_offsets",
)


def load_reference(ref_root: Path):
    for pkg in ("mega_moe", "mega_moe.runtime"):
        if pkg not in sys.modules or not hasattr(sys.modules[pkg], "__path__"):
            m = types.ModuleType(pkg)
            m.__path__ = []
            sys.modules[pkg] = m

    def load(name, rel):
        spec = importlib.util.spec_from_file_location(name, ref_root / rel)
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod
        spec.loader.exec_module(mod)
        return mod

    planning = load("mega_moe.runtime.moonep_planning", "src/mega_moe/runtime/moonep_planning.py")
    balanced = load("mega_moe.runtime.balanced_routing", "src/mega_moe/runtime/balanced_routing.py")
    return planning, balanced


def digest(a: np.ndarray) -> str:
    a = np.ascontiguousarray(a)
    return hashlib.sha256(str(a.dtype).encode() + str(a.shape).encode() + a.tobytes()).hexdigest()


def zipf_routes(world, tokens, experts, top_k, s, seed, invalid_per_rank=0, owner_weights=None):
    """Per rank a [tokens, top_k] int32 table: every token draws ``top_k`` distinct experts
    with probability ~ 1 / (rank of the expert in a seeded permutation) ** s (uniform when
    ``s`` is None), or, with ``owner_weights``, uniformly inside an owner rank chosen with those
    weights; ``invalid_per_rank`` entries per rank are then overwritten by ids outside
    ``[0, experts)`` (the same number on every rank, so the valid totals stay equal)."""
    rng = np.random.default_rng(seed)
    perm = rng.permutation(experts)
    p = np.ones(experts) if s is None else 1.0 / (1.0 + np.arange(experts)) ** s
    prob = np.empty(experts)
    prob[perm] = p / p.sum()
    if owner_weights is not None:
        w = np.repeat(np.asarray(owner_weights, float), experts // len(owner_weights))
        prob = w / w.sum()
    out = []
    for _ in range(world):
        sel = np.stack([rng.choice(experts, size=top_k, replace=False, p=prob)
                        for _ in range(tokens)]).astype(np.int32)
        if invalid_per_rank:
            flat = sel.reshape(-1)
            where = rng.choice(flat.size, size=invalid_per_rank, replace=False)
            flat[where] = rng.choice(np.array([-1, -7, experts, experts + 5], np.int32),
                                     size=invalid_per_rank)
        out.append(sel)
    return out


def counts_of(selected, experts):
    rows = []
    for sel in selected:
        flat = sel.reshape(-1).astype(np.int64)
        rows.append(np.bincount(flat[(flat >= 0) & (flat < experts)], minlength=experts))
    return np.stack(rows).astype(np.int32)


# name -> (world, experts, how the routes are made, store full tables?)
ROUTED = {
    "hot_w2_e4": dict(world=2, experts=4,
                      routes=[np.zeros((2, 2), np.int32), np.zeros((2, 2), np.int32)], full=True),
    "uniform_w4_e16_k3": dict(world=4, experts=16, gen=dict(tokens=33, top_k=3, s=None, seed=11),
                              full=True),
    "zipf_w4_e16_k4": dict(world=4, experts=16, gen=dict(tokens=48, top_k=4, s=1.2, seed=12),
                           full=True),
    "zipf_w8_e32_k4_invalid": dict(world=8, experts=32,
                                   gen=dict(tokens=40, top_k=4, s=1.5, seed=13,
                                            invalid_per_rank=9), full=True),
    "zipf_w2_e8_k2": dict(world=2, experts=8, gen=dict(tokens=64, top_k=2, s=2.0, seed=14),
                          full=True),
    "w1_e8_k2": dict(world=1, experts=8, gen=dict(tokens=16, top_k=2, s=1.0, seed=15), full=True),
    "empty_w2_e4": dict(world=2, experts=4,
                        routes=[np.zeros((0, 2), np.int32), np.zeros((0, 2), np.int32)], full=True),
    "zipf_w8_e32_k8_t1024": dict(world=8, experts=32,
                                 gen=dict(tokens=1024, top_k=8, s=1.2, seed=16), full=False),
    "zipf_w8_e384_k16_t512": dict(world=8, experts=384,
                                  gen=dict(tokens=512, top_k=16, s=1.2, seed=17), full=False),
    "zipf_w4_e128_k8_t256": dict(world=4, experts=128,
                                 gen=dict(tokens=256, top_k=8, s=1.0, seed=18), full=False),
    "owners_w8_e64_k4": dict(world=8, experts=64,
                             gen=dict(tokens=96, top_k=4, s=None, seed=19,
                                      owner_weights=(19, 27, 11, 11, 15, 15, 15, 15)), full=True),
    "owners_w4_e32_k6": dict(world=4, experts=32,
                             gen=dict(tokens=50, top_k=6, s=None, seed=20,
                                      owner_weights=(8, 1, 1, 2)), full=True),
    "owners_w8_e384_k16_t256": dict(world=8, experts=384,
                                    gen=dict(tokens=256, top_k=16, s=None, seed=21,
                                             owner_weights=(30, 22, 6, 8, 14, 16, 12, 20)),
                                    full=False),
}

# planning only, count matrices written out directly
PLANNED = {
    "tie_w4_e16": np.array([[1, 1, 1, 1, 2, 0, 0, 0, 2, 0, 0, 0, 0, 0, 0, 0]] * 4, np.int32),
    "balanced_w2_e4": np.array([[2, 2, 0, 0], [0, 0, 2, 2]], np.int32),
    "one_home_w8_e64": np.tile(np.concatenate([np.zeros(24, np.int32), np.ones(8, np.int32),
                                               np.zeros(32, np.int32)]), (8, 1)),
    "chain_w4_e8": np.array([[5, 4, 1, 0, 0, 0, 0, 0]] * 4, np.int32),
}


def main():
    ref_root = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ["MEGA_MOE_REFERENCE"])
    planning, balanced = load_reference(ref_root)
    out = {}

    def plan(name, tpe):
        t = torch.from_numpy(np.ascontiguousarray(tpe))
        res = planning.plan_moonep_b0_b3(t)
        inv = planning.build_inverse_experts_to_copy(res.experts_to_copy, tpe.shape[1])
        out[f"{name}/tpe_all"] = tpe
        out[f"{name}/alloc_cumsum"] = res.alloc_cumsum.numpy()
        out[f"{name}/experts_to_copy"] = res.experts_to_copy.numpy()
        out[f"{name}/inverse"] = inv.numpy()
        out[f"{name}/high_water"] = np.int64(res.replica_slot_high_water)
        return t, res, inv

    for name, tpe in PLANNED.items():
        plan(name, tpe)

    for name, case in ROUTED.items():
        world, experts = case["world"], case["experts"]
        routes = case.get("routes") or zipf_routes(world, experts=experts, **case["gen"])
        tpe = counts_of(routes, experts)
        t, res, inv = plan(name, tpe)
        out[f"{name}/full"] = np.int64(case["full"])
        for r, sel in enumerate(routes):
            sel_t = torch.from_numpy(sel)
            a = balanced.build_balanced_routing_metadata(sel_t, t, res.alloc_cumsum, inv, r)
            b = balanced.build_balanced_routing_metadata(sel_t, t, res.alloc_cumsum, inv, r,
                                                         use_direct_bucket_scatter=True)
            out[f"{name}/selected_{r}"] = sel
            for f in FIELDS:
                va, vb = getattr(a, f).numpy(), getattr(b, f).numpy()
                assert va.dtype == vb.dtype and np.array_equal(va, vb), (name, r, f)
                if case["full"]:
                    out[f"{name}/r{r}/{f}"] = va
                else:
                    out[f"{name}/r{r}/{f}"] = np.array(digest(va))
            out[f"{name}/r{r}/num_valid_routes"] = np.int64(a.num_valid_routes)
        print(name, "replicas per rank:", (res.experts_to_copy >= 0).sum(dim=1).tolist())

    np.savez_compressed(HERE / "moonep_tables.npz", **out)
    print("wrote", HERE / "moonep_tables.npz", (HERE / "moonep_tables.npz").stat().st_size, "bytes")


if __name__ == "__main__":
    main()
