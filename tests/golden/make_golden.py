"""Generate the golden fixtures of ``tests/golden/*.npz`` from the reference itself.

Run where a checkout of the reference is available: ``python tests/golden/make_golden.py
/path/to/reference`` (or set ``MEGA_MOE_REFERENCE``).  The reference's Torch functional
oracle is imported by file path with a stub ``torch_npu`` module (its production package
cannot be imported without the Ascend toolchain), then executed under a gloo process group
with one CPU process per rank:

* ``torch_moe_fwd_golden`` and ``torch_dispatch_fc1_golden``  (tests/_moe_baselines.py)
* ``moe_forward(return_saved=True)``                           (ops/_torch_forward.py)
* ``moe_backward_torch``                                       (tests/_moe_baselines.py)

Inputs come from ``oracle.moe_oracle.make_inputs`` and are stored in the fixture together
with the reference's outputs (bf16 tensors as their int16 bit patterns, so the files are
exact).  The fixtures are what pins ``oracle/moe_oracle.py`` to the reference.
"""

from __future__ import annotations

import importlib.util
import os
import sys
import types
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
sys.path.insert(0, str(REPO))

from oracle import moe_oracle as O  # noqa: E402

CASES = {
    # name: world, tokens, hidden, ffn, experts, top_k, seed, zipf_s, drop_frac
    "w1_e8_k2": dict(world=1, tokens=64, hidden=128, ffn=128, experts=8, top_k=2, seed=0,
                     zipf=None, drop=0.0),
    "w2_e8_k3_drop": dict(world=2, tokens=48, hidden=128, ffn=128, experts=8, top_k=3, seed=1,
                          zipf=None, drop=0.25),
    "w4_e16_k4_zipf": dict(world=4, tokens=32, hidden=64, ffn=128, experts=16, top_k=4, seed=2,
                           zipf=1.2, drop=0.0),
    "w8_e16_k4": dict(world=8, tokens=24, hidden=64, ffn=64, experts=16, top_k=4, seed=3,
                      zipf=None, drop=0.1),
}


# Activation variants: the reference's Torch functional forward with another gated activation
# (ops/_torch_forward.py:177-205) and, where its hand-written backward covers it (situglu,
# tests/_moe_baselines.py:122-160), the backward.  Forward-saved tensors and gradients only.
ACT_CASES = {
    "act_situglu_w2": dict(world=2, tokens=40, hidden=64, ffn=128, experts=8, top_k=2, seed=5,
                           zipf=None, drop=0.0, bwd=True,
                           act=dict(activation="situglu", situ_beta=1.5, situ_linear_beta=2.0)),
    "act_situglu_plain_up_w1": dict(world=1, tokens=48, hidden=64, ffn=128, experts=4, top_k=2,
                                    seed=6, zipf=None, drop=0.0, bwd=True,
                                    act=dict(activation="situglu", situ_beta=0.75,
                                             situ_linear_beta=None)),
    "act_clamp_swiglu_w1": dict(world=1, tokens=48, hidden=64, ffn=128, experts=4, top_k=2,
                                seed=7, zipf=None, drop=0.0, bwd=False,
                                act=dict(activation="clamp_swiglu", clamp_limit=0.5)),
}


def load_reference(ref_root: Path):
    sys.modules.setdefault("torch_npu", types.ModuleType("torch_npu"))
    for pkg in ("mega_moe", "mega_moe.ops", "tests"):
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

    tf = load("mega_moe.ops._torch_forward", "src/mega_moe/ops/_torch_forward.py")
    load("tests._numeric", "tests/_numeric.py")
    bl = load("tests._moe_baselines", "tests/_moe_baselines.py")
    return tf, bl


def bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.int16).numpy()
    return t.contiguous().numpy()


def case_inputs(c):
    bias = O.zipf_expert_bias(c["experts"], c["zipf"]) if c["zipf"] else None
    dropped = O.make_inputs(c["world"], c["tokens"], c["hidden"], c["ffn"], c["experts"],
                            c["top_k"], seed=c["seed"], expert_bias=bias, drop_frac=c["drop"])
    return dropped


def worker(rank, world, port, ref_root, name, c, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    tf, bl = load_reference(Path(ref_root))
    inp = case_inputs(c)
    x = inp["hidden"][rank]
    rw = inp["routing_weights"][rank]
    sel = inp["selected"][rank]
    wg, wu, wd = inp["w_gate"][rank], inp["w_up"][rank], inp["w_down"][rank]
    dy = inp["dy"][rank]
    group = dist.group.WORLD
    res = {}
    res["fwd_golden"] = bits(bl.torch_moe_fwd_golden(x, rw, sel, wg, wu, wd, c["experts"], group))
    fc1, eg, xg = bl.torch_dispatch_fc1_golden(
        x, sel, torch.cat([wg, wu], dim=1), c["experts"], torch.bfloat16, "cpu", group)
    res["dfc1_out"] = bits(fc1)
    res["dfc1_experts"] = bits(eg)
    res["dfc1_tokens"] = bits(xg)
    # saved contract + backward need dropless routes: replace dropped ids by a valid expert
    sel_nd = torch.where(sel >= c["experts"], sel % c["experts"], sel).to(torch.int32)
    with torch.no_grad():
        out, saved = tf.moe_forward(x, rw, sel_nd, wg, wu, wd, group, c["top_k"],
                                    return_saved=True)
        grads = bl.moe_backward_torch(saved, dy)
    res["sel_dropless"] = bits(sel_nd)
    res["mf_output"] = bits(out)
    for k in ("sort_idxs", "local_sort_idxs", "inv_local", "inv_sort", "expert_counts",
              "split_size_cum_per_expert", "recv_hidden_sorted", "fc1_output",
              "swiglu_out_weighted", "recv_weights_sorted", "fc2_out"):
        res["saved_" + k] = bits(saved[k])
    res["saved_splits_send"] = np.asarray(saved["splits_send_list"])
    res["saved_splits_recv"] = np.asarray(saved["splits_recv_list"])
    for k in ("grad_hidden", "grad_routing_weights", "grad_fc1_1", "grad_fc1_2", "grad_fc2",
              "grad_fc2_out_sorted", "grad_swiglu", "grad_fc1_output", "grad_gate",
              "grad_recv_hidden_sorted"):
        res["bwd_" + k] = bits(grads[k])
    res["in_hidden"] = bits(x)
    res["in_routing_weights"] = bits(rw)
    res["in_selected"] = bits(sel)
    res["in_w_gate"] = bits(wg)
    res["in_w_up"] = bits(wu)
    res["in_w_down"] = bits(wd)
    res["in_dy"] = bits(dy)
    np.savez_compressed(Path(out_dir) / f"_{name}_rank{rank}.npz", **res)
    dist.barrier()
    dist.destroy_process_group()


def act_worker(rank, world, port, ref_root, name, c, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    tf, bl = load_reference(Path(ref_root))
    inp = case_inputs(c)
    x, rw, sel = inp["hidden"][rank], inp["routing_weights"][rank], inp["selected"][rank]
    wg, wu, wd = inp["w_gate"][rank], inp["w_up"][rank], inp["w_down"][rank]
    dy = inp["dy"][rank]
    res = {}
    with torch.no_grad():
        out, saved = tf.moe_forward(x, rw, sel, wg, wu, wd, dist.group.WORLD, c["top_k"],
                                    return_saved=True, **c["act"])
        res["mf_output"] = bits(out)
        for k in ("fc1_output", "swiglu_out_weighted", "recv_weights_sorted", "fc2_out"):
            res["saved_" + k] = bits(saved[k])
        if c["bwd"]:
            grads = bl.moe_backward_torch(saved, dy)
            for k in ("grad_hidden", "grad_routing_weights", "grad_fc1_1", "grad_fc1_2",
                      "grad_fc2", "grad_fc1_output", "grad_gate"):
                res["bwd_" + k] = bits(grads[k])
    for k, v in (("in_hidden", x), ("in_routing_weights", rw), ("in_selected", sel),
                 ("in_w_gate", wg), ("in_w_up", wu), ("in_w_down", wd), ("in_dy", dy)):
        res[k] = bits(v)
    np.savez_compressed(Path(out_dir) / f"_{name}_rank{rank}.npz", **res)
    dist.barrier()
    dist.destroy_process_group()


ROUTE_CASES = [(64, 896, 16), (8192, 896, 16), (128, 32, 8), (256, 64, 16), (4096, 128, 8)]


def route_digests(ref_root: Path):
    """SHA-256 of the reference's deterministic skewed routes
    (benchmark/layer/_kimi_routes.py) for a few shapes and ranks -> kimi_routes_digests.json."""
    import hashlib
    import json
    spec = importlib.util.spec_from_file_location(
        "_kimi_routes", ref_root / "benchmark/layer/_kimi_routes.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    out = {}
    for tokens, experts, top_k in ROUTE_CASES:
        for rank in (0, 3, 7):
            routes = mod.kimi_skewed_routes(tokens, experts, top_k, rank)
            key = f"t{tokens}_e{experts}_k{top_k}_r{rank}"
            out[key] = hashlib.sha256(routes.contiguous().numpy().tobytes()).hexdigest()
    (HERE / "kimi_routes_digests.json").write_text(json.dumps(out, indent=1, sort_keys=True))
    print("kimi_routes_digests.json", len(out), "entries")


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("MEGA_MOE_REFERENCE")
    if not ref_root:
        raise SystemExit("usage: make_golden.py /path/to/reference (or MEGA_MOE_REFERENCE)")
    port = 29610
    only = set(sys.argv[2].split(",")) if len(sys.argv) > 2 else None   # optional case filter
    todo = [(n, c, worker) for n, c in CASES.items()] + \
           [(n, c, act_worker) for n, c in ACT_CASES.items()]
    if only is None or "routes" in only:
        route_digests(Path(ref_root))
    for name, c, fn in todo:
        if only is not None and name not in only:
            continue
        port += 1
        mp.spawn(fn, args=(c["world"], port, ref_root, name, c, str(HERE)),
                 nprocs=c["world"], join=True)
        merged = {"meta": np.array([c["world"], c["tokens"], c["hidden"], c["ffn"], c["experts"],
                                    c["top_k"]], dtype=np.int64)}
        for r in range(c["world"]):
            part = HERE / f"_{name}_rank{r}.npz"
            with np.load(part) as z:
                for k in z.files:
                    merged[f"r{r}_{k}"] = z[k]
            part.unlink()
        np.savez_compressed(HERE / f"{name}.npz", **merged)
        print(name, (HERE / f"{name}.npz").stat().st_size, "bytes")


if __name__ == "__main__":
    main()
