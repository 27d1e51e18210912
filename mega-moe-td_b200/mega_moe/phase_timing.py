"""Where the time of one layer step goes: phases of the forward and the waits of the GEMM
kernels' warp roles, through the operator's own timing switch (one GPU).

    python mega-moe-td_b200/build.py --profile
    PYTHONPATH=mega-moe-td_b200 MOE_FWD_TIMING=1 python -m mega_moe.phase_timing \
        --experts 32 --rows-per-expert 146

Runs a few forward+backward steps of the layer on synthetic, balanced routes with
``MOE_FWD_TIMING=1`` and prints what ``FusedMoEForward.read_last_forward_phase_timing()``
returns for the last step: the device time of each forward phase and, per GEMM launch, the mean
over the CTAs of the SM clocks every role spent

* producer: waiting for a free A slot / B slot / the dispatch arrival flags, inside the TMA
  issue, in total;
* MMA issuer (warp 1): waiting for a free accumulator, for loads ("full"), for the tail rows,
  inside the MMA issue, in tile lookup - as fractions of its total;
* epilogue (first epilogue warp): waiting for the accumulator, for the previous TMA store's read
  of the staging buffer - as fractions of its total.

``MM_PROFILE_SKIP_MMA=1`` frees the stages without issuing MMAs: what remains is the time of the
load / epilogue pipeline alone.  ``skinny_gemm_kernel`` is not instrumented (its launches print
nothing); use ``MOE_GEMM_MODE=single`` to look at the ragged-row GEMMs.
"""
from __future__ import annotations

import argparse
import os
import types

os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
os.environ["MOE_FWD_TIMING"] = "1"

import torch  # noqa: E402

import mega_moe  # noqa: E402
from mega_moe import _native as N  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--experts", type=int, default=32)
    ap.add_argument("--rows-per-expert", type=int, default=146)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--ffn", type=int, default=2048)
    ap.add_argument("--top-k", type=int, default=16)
    args = ap.parse_args()
    if not N.TIMING_LIB_PATH.exists():
        raise SystemExit("build the instrumented library first: "
                         "python mega-moe-td_b200/build.py --profile")
    dev = torch.device("cuda", 0)
    E, k, H, F = args.experts, args.top_k, args.hidden, args.ffn
    tokens = args.rows_per_expert * E // k
    g = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn(tokens, H, generator=g, device=dev).to(torch.bfloat16).requires_grad_(True)
    dy = torch.randn(tokens, H, generator=g, device=dev).to(torch.bfloat16)
    # balanced routes: token t takes experts (t * k + j) mod E
    sel = ((torch.arange(tokens * k, device=dev) % E).view(tokens, k)).to(torch.int32)
    rw = torch.softmax(torch.randn(tokens, k, generator=g, device=dev), -1).requires_grad_(True)
    gate_up = (torch.randn(E, H, 2 * F, generator=g, device=dev) * 0.02).to(torch.bfloat16)
    down = (torch.randn(E, H, F, generator=g, device=dev) * 0.02).to(torch.bfloat16)
    gate_up.requires_grad_(True)
    down.requires_grad_(True)
    op = mega_moe.FusedMoEForward(None, max_tokens_per_rank=tokens, hidden_size=H, top_k=k,
                                  num_experts=E, config=mega_moe.MoEForwardConfig(
                                      receive_capacity_factor=1.0,
                                      enable_single_kernel_forward=True))
    op.persistent_weight_grads = op.host_sync_free = op.saved_views = True
    state = types.SimpleNamespace()

    def step():
        out = mega_moe.MegaMoEFunction.apply(op, x, rw, sel, gate_up, down, op.context.peer_mem,
                                             state)
        return torch.autograd.grad(out, [x, rw, gate_up, down], dy)

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    for _ in range(2):
        step()
    rec = op.read_last_forward_phase_timing()
    print("forward phases, ms:", {k: round(v, 3) for k, v in rec["phase_ms"].items()})
    print("mean SM clocks per CTA, last step")
    slots = rec["acc_slots"]
    for name, buf in rec["acc"].items():
        v = dict(zip(slots, buf[:148, :len(slots)].double().mean(0).tolist()))
        if v["tiles"] == 0:
            continue
        mt, et = max(v["mma_total"], 1.0), max(v["epi_total"], 1.0)
        print(f"{name:18s} tiles/CTA {v['tiles']:6.1f} | producer: empty {v['prod_empty']:9.0f} "
              f"bempty {v['prod_bempty']:8.0f} flags {v['prod_flag']:8.0f} issue "
              f"{v['prod_issue']:9.0f} of {v['prod_total']:9.0f} | MMA {mt:9.0f}: acc_empty "
              f"{v['mma_acc_empty'] / mt:4.2f} full {v['mma_full'] / mt:4.2f} tail "
              f"{v['mma_tail'] / mt:4.2f} issue {v['mma_issue'] / mt:4.2f} lookup "
              f"{v['mma_decode'] / mt:4.2f} | epilogue {et:9.0f}: acc_full "
              f"{v['epi_acc_full'] / et:4.2f} store_read {v['epi_store_read'] / et:4.2f}")
    op.finalize()


if __name__ == "__main__":
    main()
