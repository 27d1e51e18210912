"""Worker of the multi-GPU parity test: one process per GPU, launched by torch.distributed.run.

Every rank rebuilds the seeded inputs of all ranks, runs the CPU oracle for the whole group in
process, and compares its own slice of the CUDA operator's results against it.
"""
import os
import sys
import types
from pathlib import Path

import torch
import torch.distributed as dist

REPO = Path(__file__).resolve().parent.parent
for p in (REPO, REPO / "mega-moe-td_b200"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))

import mega_moe  # noqa: E402
from oracle import moe_oracle as O  # noqa: E402

CASES = [
    # tokens, hidden, ffn, experts, top_k, drop, zipf, capacity factor (None = world)
    (96, 128, 128, 8, 2, 0.0, None, None),
    (512, 256, 384, 16, 4, 0.25, None, None),
    (1024, 512, 256, 32, 8, 0.0, 1.2, None),
    (300, 256, 128, 8, 3, 1.0, None, None),      # nothing is routed anywhere
    # the real hidden / FFN size of the headline layer on a few experts (K = 7168: 112 k-blocks,
    # 28 column tiles of the FC2 output, the 4096-wide packed FC1 table)
    (64, 7168, 2048, 16, 8, 0.0, None, None),
]


def check(name, ok, detail=""):
    if not ok:
        raise AssertionError(f"{name} {detail}")


def main():
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    group = dist.group.WORLD
    for case_id, (tokens, hidden, ffn, experts, top_k, drop, zipf, cf) in enumerate(CASES):
        if experts % world:
            continue
        bias = O.zipf_expert_bias(experts, zipf) if zipf else None
        inp = O.make_inputs(world, tokens, hidden, ffn, experts, top_k, seed=50 + case_id,
                            expert_bias=bias, drop_frac=drop,
                            weight_std=0.02 if hidden > 1024 else 0.05)
        want_out = O.forward_golden(inp["hidden"], inp["routing_weights"], inp["selected"],
                                    inp["w_gate"], inp["w_up"], inp["w_down"], experts)[rank]
        meta = O.routing_metadata([s.numpy() for s in inp["selected"]], experts)[rank]
        cfg = mega_moe.MoEForwardConfig(
            receive_capacity_factor=cf,
            fc1_gemm_block_size_k=min(128, hidden), fc2_gemm_block_size_n=min(256, hidden))
        op = mega_moe.FusedMoEForward(group, max_tokens_per_rank=tokens, hidden_size=hidden,
                                      top_k=top_k, num_experts=experts, config=cfg)
        x = inp["hidden"][rank].to(dev)
        sel = inp["selected"][rank].to(dev)
        rw = inp["routing_weights"][rank].to(dev)
        gate_up = mega_moe.pack_gate_up_weights(inp["w_gate"][rank].to(dev),
                                                inp["w_up"][rank].to(dev))
        down = inp["w_down"][rank].to(dev)
        # routing metadata: bit-exact
        plan = op.build_routing_plan(sel)
        check("num_received", plan.num_received_routes == meta["num_received_routes"])
        for got, key in ((plan.send_route_indices, "send_route_indices"),
                         (plan.send_bucket_starts, "send_bucket_starts"),
                         (plan.send_bucket_receive_offsets, "send_bucket_dst_starts"),
                         (plan.received_expert_offsets, "recv_expert_offs"),
                         (plan.receive_counts_by_source_expert.reshape(-1), "recv_counts_re"),
                         (op.context.metadata_stats, "stats")):
            want = torch.as_tensor(meta[key].reshape(-1))
            check(key, torch.equal(got.cpu().to(want.dtype), want), f"case {case_id} rank {rank}")
        # forward
        out = op(x, sel, gate_up, down, rw)
        torch.testing.assert_close(out.cpu().float(), want_out.float(), rtol=O.OUTPUT_RTOL,
                                   atol=O.OUTPUT_ATOL)
        if want_out.float().abs().max() > 0:
            check("fwd cosine", O.cosine(out.cpu(), want_out) > O.MIN_COSINE)
        # epoch reuse: a second call on the same operator is bit-identical
        # (reference gate: tests/layer/test_moe_suite.py:4636-4827)
        out_again = op(x, sel, gate_up, down, rw)
        check("repeated forward is bit-identical", torch.equal(out_again, out),
              f"case {case_id} rank {rank}")
        # forward + backward through autograd (dropless routes only: the saved contract)
        if drop == 0.0:
            _, saved = O.forward_saved(inp["hidden"], inp["routing_weights"], inp["selected"],
                                       inp["w_gate"], inp["w_up"], inp["w_down"], top_k)
            want = O.backward(saved, inp["dy"])[rank]
            xg = x.clone().requires_grad_(True)
            rwg = rw.clone().requires_grad_(True)
            gu = gate_up.clone().requires_grad_(True)
            dn = down.clone().requires_grad_(True)
            o2 = mega_moe.MegaMoEFunction.apply(op, xg, rwg, sel, gu, dn, op.context.peer_mem,
                                                types.SimpleNamespace())
            o2.backward(inp["dy"][rank].to(dev))
            pairs = {
                "grad_hidden": (xg.grad, want["grad_hidden"]),
                "grad_routing_weights": (rwg.grad, want["grad_routing_weights"]),
                "grad_down": (dn.grad, want["grad_fc2"]),
                "grad_gate_up": (gu.grad, torch.cat((want["grad_fc1_1"], want["grad_fc1_2"]),
                                                    dim=1).transpose(1, 2)),
            }
            for name, (got, gold) in pairs.items():
                ok, max_d, rel, n_bad = O.cmp_grad(got.cpu(), gold)
                check(name, ok, f"case {case_id} rank {rank} max_abs={max_d:.3e} rel={rel:.3e} "
                                f"bad={n_bad}")
                if gold.float().abs().max() > 0:
                    check(name + " cosine", O.cosine(got.cpu(), gold) > O.MIN_COSINE)
            # a second forward + backward on the same operator reproduces every gradient bit
            # for bit
            first = {name: got.clone() for name, (got, _) in pairs.items()}
            for t in (xg, rwg, gu, dn):
                t.grad = None
            o3 = mega_moe.MegaMoEFunction.apply(op, xg, rwg, sel, gu, dn, op.context.peer_mem,
                                                types.SimpleNamespace())
            o3.backward(inp["dy"][rank].to(dev))
            for name, t in (("grad_hidden", xg), ("grad_routing_weights", rwg),
                            ("grad_down", dn), ("grad_gate_up", gu)):
                check("repeated " + name, torch.equal(t.grad, first[name]),
                      f"case {case_id} rank {rank}")
            # the five-stage backward also accepts the Torch functional forward's saved dict
            sd = {k: (v.to(dev) if isinstance(v, torch.Tensor) else v)
                  for k, v in saved[rank].items()}
            got = mega_moe.moe_backward_triton(sd, inp["dy"][rank].to(dev), op.context.peer_mem)
            for name in ("grad_hidden", "grad_routing_weights", "grad_fc1_1", "grad_fc1_2",
                         "grad_fc2", "grad_swiglu", "grad_gate"):
                ok, max_d, rel, n_bad = O.cmp_grad(got[name].cpu(), want[name])
                check("oracle-saved " + name, ok, f"case {case_id} rank {rank} max_abs={max_d:.3e}")
        check("status", op.context.read_status().code == 0)
        op.finalize()
        if drop == 0.0 and case_id == 2:
            # recompute backward across ranks: the input rows are dispatched again into the
            # symmetric slab and the activation is rebuilt from the saved FC1 rows
            os.environ["MOE_SAVED_RECOMPUTE"] = "1"
            try:
                op2 = mega_moe.FusedMoEForward(group, max_tokens_per_rank=tokens,
                                               hidden_size=hidden, top_k=top_k,
                                               num_experts=experts, config=cfg)
                gold = []
                for s_r in saved:
                    act = O.recompute_act(s_r["gate"], s_r["up"], s_r["recv_weights_sorted"])
                    gold.append(dict(s_r, swiglu_out_weighted=act))
                want2 = O.backward(gold, inp["dy"])[rank]
                sd = {k: (v.to(dev) if isinstance(v, torch.Tensor) else v)
                      for k, v in saved[rank].items()
                      if k not in ("recv_hidden_sorted", "swiglu_out_weighted")}
                got = mega_moe.moe_backward_triton(sd, inp["dy"][rank].to(dev),
                                                   op2.context.peer_mem, hidden_states=x)
                for name in ("grad_hidden", "grad_routing_weights", "grad_fc1_1", "grad_fc1_2",
                             "grad_fc2"):
                    ok, max_d, rel, n_bad = O.cmp_grad(got[name].cpu(), want2[name])
                    check("recompute " + name, ok,
                          f"case {case_id} rank {rank} max_abs={max_d:.3e}")
                check("recompute status", op2.context.read_status().code == 0)
                op2.finalize()
            finally:
                del os.environ["MOE_SAVED_RECOMPUTE"]
    # the reference benchmark's deterministic skewed routes (owner loads 19/27/11/11/15/15/15/15
    # of every 128): forward parity with a capacity sized for the hottest owner
    tokens, hidden, ffn, experts, top_k = 256, 256, 128, 32, 8
    if experts % world == 0:
        inp = O.make_inputs(world, tokens, hidden, ffn, experts, top_k, seed=77, weight_std=0.05)
        routes = [O.kimi_skewed_routes(tokens, experts, top_k, r) for r in range(world)]
        want_out = O.forward_golden(inp["hidden"], inp["routing_weights"], routes,
                                    inp["w_gate"], inp["w_up"], inp["w_down"], experts)[rank]
        cfg = mega_moe.MoEForwardConfig(receive_capacity_factor=min(float(world), 2.0))
        op = mega_moe.FusedMoEForward(group, max_tokens_per_rank=tokens, hidden_size=hidden,
                                      top_k=top_k, num_experts=experts, config=cfg)
        gate_up = mega_moe.pack_gate_up_weights(inp["w_gate"][rank].to(dev),
                                                inp["w_up"][rank].to(dev))
        out = op(inp["hidden"][rank].to(dev), routes[rank].to(dev), gate_up,
                 inp["w_down"][rank].to(dev), inp["routing_weights"][rank].to(dev))
        torch.testing.assert_close(out.cpu().float(), want_out.float(), rtol=O.OUTPUT_RTOL,
                                   atol=O.OUTPUT_ATOL)
        check("skewed routes status", op.context.read_status().code == 0)
        op.finalize()
    # zero-receive: every route goes to rank 0, whose buffer (capacity factor = world) holds
    # them all; the other ranks receive nothing but still dispatch, combine and reduce
    # (reference: tests/layer/test_moe_suite.py:327-357,464-500)
    tokens, hidden, ffn, experts, top_k = 96, 256, 128, 4 * world, 3
    inp = O.make_inputs(world, tokens, hidden, ffn, experts, top_k, seed=123, weight_std=0.05)
    epr = experts // world
    to_rank0 = [((torch.arange(tokens * top_k) * 7 + r) % epr).to(torch.int32).view(tokens, top_k)
                for r in range(world)]
    want_out = O.forward_golden(inp["hidden"], inp["routing_weights"], to_rank0, inp["w_gate"],
                                inp["w_up"], inp["w_down"], experts)[rank]
    _, saved = O.forward_saved(inp["hidden"], inp["routing_weights"], to_rank0, inp["w_gate"],
                               inp["w_up"], inp["w_down"], top_k)
    want = O.backward(saved, inp["dy"])[rank]
    op = mega_moe.FusedMoEForward(group, max_tokens_per_rank=tokens, hidden_size=hidden,
                                  top_k=top_k, num_experts=experts,
                                  config=mega_moe.MoEForwardConfig(receive_capacity_factor=None))
    xg = inp["hidden"][rank].to(dev).requires_grad_(True)
    rwg = inp["routing_weights"][rank].to(dev).requires_grad_(True)
    gu = mega_moe.pack_gate_up_weights(inp["w_gate"][rank].to(dev),
                                       inp["w_up"][rank].to(dev)).requires_grad_(True)
    dn = inp["w_down"][rank].to(dev).requires_grad_(True)
    out = mega_moe.MegaMoEFunction.apply(op, xg, rwg, to_rank0[rank].to(dev), gu, dn,
                                         op.context.peer_mem, types.SimpleNamespace())
    received = int(op.context.metadata_stats[0].item())
    check("zero-receive row count", received == (world * tokens * top_k if rank == 0 else 0))
    torch.testing.assert_close(out.detach().cpu().float(), want_out.float(), rtol=O.OUTPUT_RTOL,
                               atol=O.OUTPUT_ATOL)
    out.backward(inp["dy"][rank].to(dev))
    for name, got, gold in (("grad_hidden", xg.grad, want["grad_hidden"]),
                            ("grad_routing_weights", rwg.grad, want["grad_routing_weights"]),
                            ("grad_down", dn.grad, want["grad_fc2"]),
                            ("grad_gate_up", gu.grad,
                             torch.cat((want["grad_fc1_1"], want["grad_fc1_2"]),
                                       dim=1).transpose(1, 2))):
        ok, max_d, rel, n_bad = O.cmp_grad(got.cpu(), gold)
        check("zero-receive " + name, ok, f"rank {rank} max_abs={max_d:.3e} bad={n_bad}")
    check("zero-receive status", op.context.read_status().code == 0)
    op.finalize()
    # receive-capacity overflow: every rank must raise ValueError, and the device stays usable
    tokens, hidden, ffn, experts, top_k = 256, 128, 128, 2 * world, 2
    inp = O.make_inputs(world, tokens, hidden, ffn, experts, top_k, seed=99)
    sel_all = torch.zeros(tokens, top_k, dtype=torch.int32)      # everything to rank 0
    sel_all[:, 1] = 1
    cfg = mega_moe.MoEForwardConfig(receive_capacity_factor=1.0, fc2_gemm_block_size_n=128)
    op = mega_moe.FusedMoEForward(group, max_tokens_per_rank=tokens, hidden_size=hidden,
                                  top_k=top_k, num_experts=experts, config=cfg)
    gate_up = mega_moe.pack_gate_up_weights(inp["w_gate"][rank].to(dev), inp["w_up"][rank].to(dev))
    raised = False
    try:
        op(inp["hidden"][rank].to(dev), sel_all.to(dev), gate_up, inp["w_down"][rank].to(dev),
           inp["routing_weights"][rank].to(dev))
    except ValueError as exc:
        raised = "peer buffer capacity" in str(exc)
    check("capacity overflow raises", raised)
    # perfectly balanced routes fill every rank's buffer exactly to its capacity
    balanced = [((torch.arange(tokens * top_k) + r) % experts).to(torch.int32).view(tokens, top_k)
                for r in range(world)]
    out = op(inp["hidden"][rank].to(dev), balanced[rank].to(dev), gate_up,
             inp["w_down"][rank].to(dev), inp["routing_weights"][rank].to(dev))
    want_out = O.forward_golden(inp["hidden"], inp["routing_weights"], balanced,
                                inp["w_gate"], inp["w_up"], inp["w_down"], experts)[rank]
    torch.testing.assert_close(out.cpu().float(), want_out.float(), rtol=O.OUTPUT_RTOL,
                               atol=O.OUTPUT_ATOL)
    op.finalize()
    dist.barrier()
    if rank == 0:
        print(f"multirank parity ok on {world} GPUs")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
