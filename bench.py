"""Benchmark of the expert-parallel MoE layer: forward + five-stage backward, tokens/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one forward plus one backward of the layer over one batch of synthetic
tokens per rank.  The default workload is the Kimi-K3-shaped layer (896 experts, top-16,
hidden 7168, expert FFN 2048, 8192 tokens per rank) with the experts split evenly over the
N ranks.  ``value`` is measured with all inputs resident in HBM; ``e2e`` adds, inside the
timed region, the host->device copies of the step's inputs from pinned memory and the
device->host copies of its results.

``--impl reference`` times the reference's algorithm on the host CPU instead: the CPU oracle
(a restatement of the reference's Torch functional forward/backward) on a bounded sample of
the same workload, with all host threads.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time
from pathlib import Path

# The headline workload fills ~170 of the 180 GB of one B200 at N=1; expandable segments keep
# torch's caching allocator from fragmenting around the 26 GB and 52 GB gradient tensors.
os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")

REPO = Path(__file__).resolve().parent
for p in (REPO, REPO / "mega-moe-td_b200"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

WORKLOADS = {
    # the configuration the headline metric is quoted on
    "kimi_k3_e896_k16_t8192": dict(tokens=8192, hidden=7168, ffn=2048, experts=896, top_k=16,
                                   capacity=1.25),
    # the same layer at the other token counts the reference sweeps (multi-GPU runs; at one GPU
    # 16384 tokens per rank exceed the memory left beside 158 GB of weights and gradients)
    "kimi_k3_e896_k16_t4096": dict(tokens=4096, hidden=7168, ffn=2048, experts=896, top_k=16,
                                   capacity=1.25),
    "kimi_k3_e896_k16_t16384": dict(tokens=16384, hidden=7168, ffn=2048, experts=896, top_k=16,
                                    capacity=1.25),
    # Qwen3-30B-A3B-like layer, forward only
    "qwen3_30b_e128_k8_t4096": dict(tokens=4096, hidden=2048, ffn=768, experts=128, top_k=8,
                                    capacity=1.25, forward_only=True),
    # 32 experts with a Zipf(1.2) router bias: the hottest expert receives several times the
    # mean load; the receive capacity is sized from the measured hottest rank
    "e32_zipf12_k8_t8192": dict(tokens=8192, hidden=7168, ffn=2048, experts=32, top_k=8,
                                capacity="measured", zipf=1.2),
    # Qwen3-235B-A22B-like layer with a Zipf(1.0) router bias, and its small-batch case
    "qwen3_235b_e128_k8_t8192": dict(tokens=8192, hidden=4096, ffn=1536, experts=128, top_k=8,
                                     capacity="measured", zipf=1.0),
    "qwen3_235b_e128_k8_t128": dict(tokens=128, hidden=4096, ffn=1536, experts=128, top_k=8,
                                    capacity="measured", zipf=1.0),
    # ---- slices for profiler captures (ncu replays every kernel ~40 times, so a capture must
    # hold a few GB at most): the headline layer's H, F and rows per expert on fewer experts --
    # one rank's share of the headline layer at 8 GPUs (112 local experts, same rows per rank)
    "kimi_k3_rank_share_e112_k16_t8192": dict(tokens=8192, hidden=7168, ffn=2048, experts=112,
                                              top_k=16, capacity=1.25),
    # 16 experts with 1170 rows each (the per-expert load at 8 GPUs)
    "kimi_k3_rank_share_slice_e16_t1170": dict(tokens=1170, hidden=7168, ffn=2048, experts=16,
                                               top_k=16, capacity=1.25),
    # 32 experts with 146 rows each (the per-expert load on one GPU; weights 2.8 GB)
    "kimi_k3_single_gpu_slice_e32_t292": dict(tokens=292, hidden=7168, ffn=2048, experts=32,
                                              top_k=16, capacity=1.25),
    # 292 and 585 rows per expert (2 and 4 GPUs)
    "kimi_k3_two_gpu_slice_e32_t584": dict(tokens=584, hidden=7168, ffn=2048, experts=32,
                                           top_k=16, capacity=1.25),
    "kimi_k3_four_gpu_slice_e32_t1170": dict(tokens=1170, hidden=7168, ffn=2048, experts=32,
                                             top_k=16, capacity=1.25),
    "small_e32_k4_t1024": dict(tokens=1024, hidden=1024, ffn=512, experts=32, top_k=4,
                               capacity=2.0),
}
DEFAULT_WORKLOAD = "kimi_k3_e896_k16_t8192"
METRIC = "MoE fwd+bwd tokens/s (E896 top-16 H7168 F2048, 8K tok/rank), whole job"


def measured_peaks():
    path = REPO / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return dict(hbm_gbs=float(d["hbm_gbs"]), tflops=float(d["bf16_tflops_sustained"]),
                    source="measured")
    return dict(hbm_gbs=6650.0, tflops=1400.0, source="fallback")


def measured_traffic(hidden, ffn, top_k, rows, experts_per_rank):
    """DRAM bytes per step of the grouped GEMM from the committed ncu captures
    (profiles/grouped_gemm_dram_traffic.json), scaled by the number of local experts; None when
    no capture matches this shape's rows per expert within 15 %."""
    path = REPO / "profiles" / "grouped_gemm_dram_traffic.json"
    if not path.exists() or (hidden, ffn, top_k) != (7168, 2048, 16) or experts_per_rank <= 0:
        return None
    rows_per_expert = rows / experts_per_rank
    captures = json.loads(path.read_text())["captures"]
    best = min(captures, key=lambda key: abs(float(key) - rows_per_expert))
    if abs(float(best) - rows_per_expert) > 0.15 * rows_per_expert:
        return None
    return round(captures[best]["bytes_per_expert_per_step"] * experts_per_rank)


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML on a background thread while the
    timed region runs (reading only; no setting of the GPU is touched)."""

    REASONS = {
        "hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20,
        "hw_thermal_slowdown": 0x40, "hw_power_brake_slowdown": 0x80,
    }

    def __init__(self, gpu_index: int, period_s: float = 0.05):
        self.gpu_index = gpu_index
        self.period_s = period_s
        self.samples = []
        self.reason_bits = 0
        self.max_clock = None
        self.power_w_max = None
        self._stop = None
        self._thread = None
        self.error = None

    def _run(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            uuid = torch.cuda.get_device_properties(self.gpu_index).uuid
            try:
                h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + str(uuid)).encode())
            except Exception:
                h = pynvml.nvmlDeviceGetHandleByIndex(self.gpu_index)
            self.max_clock = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
            while not self._stop.is_set():
                self.samples.append(float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)))
                try:
                    self.reason_bits |= int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(h))
                except Exception:
                    self.reason_bits |= int(pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h))
                try:
                    pw = pynvml.nvmlDeviceGetPowerUsage(h) / 1000.0
                    self.power_w_max = pw if self.power_w_max is None else max(self.power_w_max, pw)
                except Exception:
                    pass
                self._stop.wait(self.period_s)
        except Exception as exc:  # NVML missing: report it instead of failing the benchmark
            self.error = repr(exc)[:200]

    def start(self):
        import threading
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def stop(self):
        if self._thread is not None:
            self._stop.set()
            self._thread.join(timeout=5)
        reasons = sorted(n for n, bit in self.REASONS.items() if self.reason_bits & bit)
        out = {"sm_mhz": statistics.median(self.samples) if self.samples else None,
               "sm_max_mhz": self.max_clock, "reasons": reasons, "samples": len(self.samples),
               "power_w_max": self.power_w_max}
        if self.error:
            out["error"] = self.error
        return out


def bind_host_threads_near_gpu(local_rank, nvml=None, uuid=None):
    """Multi-GPU runs: keep this rank's host threads on the CPU cores NVML reports as local to
    its GPU, so that the pinned staging buffers (placed by the allocating thread) and the copy
    submissions do not cross the socket interconnect when eight ranks stream their inputs at
    once.  Only this process's CPU affinity changes; nothing is written to the GPU or the driver.
    Returns the number of cores bound to, or None when nothing was changed."""
    if os.environ.get("MOE_BENCH_NO_AFFINITY"):
        return None
    try:
        if nvml is None:
            import pynvml as nvml
            nvml.nvmlInit()
        if uuid is None:
            uuid = torch.cuda.get_device_properties(local_rank).uuid
        handle = nvml.nvmlDeviceGetHandleByUUID(("GPU-" + str(uuid)).encode())
        words = ((os.cpu_count() or 64) + 63) // 64
        mask = nvml.nvmlDeviceGetCpuAffinity(handle, words)
        local = {64 * i + b for i, word in enumerate(mask) for b in range(64) if (int(word) >> b) & 1}
        cpus = local & os.sched_getaffinity(0)
        if len(cpus) < 4:      # a mask this narrow would crowd the copy and proxy threads
            return None
        os.sched_setaffinity(0, cpus)
        return len(cpus)
    except Exception:      # no NVML, no such call, not permitted: run unbound
        return None


def make_routes(w, rank, device):
    """Seeded router outputs of one rank: top-k of N(0,1) logits (plus the workload's Zipf bias)
    and the softmax over the selected logits."""
    T, E, k = w["tokens"], w["experts"], w["top_k"]
    g = torch.Generator(device=device).manual_seed(2000 + rank)
    logits = torch.randn(T, E, generator=g, device=device)
    if w.get("zipf"):
        # per-expert bias 2 * log(1 / rank_e ** s) over a seeded permutation of the experts,
        # the same on every rank
        perm = torch.randperm(E, generator=torch.Generator().manual_seed(7))
        pos = torch.empty(E, dtype=torch.float32)
        pos[perm] = torch.arange(1, E + 1, dtype=torch.float32)
        logits = logits + (2.0 * torch.log(1.0 / pos ** float(w["zipf"]))).to(device)
    top_v, top_i = torch.topk(logits, k, dim=-1)
    return top_i.to(torch.int32).contiguous(), torch.softmax(top_v, dim=-1).float().contiguous()


def make_device_inputs(w, rank, world, device):
    """Seeded synthetic inputs of one rank, created on the device (weights are tens of GB)."""
    epr = w["experts"] // world
    g = torch.Generator(device=device).manual_seed(1000 + rank)
    T, H, F = w["tokens"], w["hidden"], w["ffn"]
    x = torch.randn(T, H, generator=g, device=device).to(torch.bfloat16)
    dy = torch.randn(T, H, generator=g, device=device).to(torch.bfloat16)
    sel, rw = make_routes(w, rank, device)
    gate_up = torch.empty(epr, H, 2 * F, dtype=torch.bfloat16, device=device)
    down = torch.empty(epr, H, F, dtype=torch.bfloat16, device=device)
    for e0 in range(0, epr, 64):
        gate_up[e0:e0 + 64].normal_(0.0, 0.02, generator=g)
        down[e0:e0 + 64].normal_(0.0, 0.02, generator=g)
    return x, dy, rw, sel, gate_up, down


class GemmTimer:
    """CUDA events around every grouped-GEMM launch of the timed steps."""

    def __init__(self):
        self.pairs = []

    def __call__(self, name):
        s = torch.cuda.Event(enable_timing=True)
        e = torch.cuda.Event(enable_timing=True)
        self.pairs.append((name, s, e))
        return s, e

    def summary(self):
        per = {}
        for name, s, e in self.pairs:
            per.setdefault(name, []).append(s.elapsed_time(e))
        return per


def measured_capacity_factor(sel, experts, world, top_k, group, device):
    """Receive capacity for a skewed router: rows of the hottest rank over the rows a rank
    sends, plus 2 % head room, rounded up to 1/64 (the whole group routes first, then every
    rank sizes its buffers alike)."""
    epr = experts // world
    per_rank = torch.bincount((sel.reshape(-1).long() // epr), minlength=world).to(device)
    if world > 1:
        dist.all_reduce(per_rank, group=group)
    hottest = int(per_rank.max().item())
    factor = hottest / float(sel.numel()) * 1.02
    return min(float(world), max(1.0, -(-factor * 64 // 1) / 64)), hottest


def run_ours(args, w, name):
    import mega_moe
    from mega_moe import _native as N
    from mega_moe.ops import _launch as L

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    group = None
    host_cpus = bind_host_threads_near_gpu(local_rank) if world > 1 else None
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        group = dist.group.WORLD
    T, H, F, E, k = w["tokens"], w["hidden"], w["ffn"], w["experts"], w["top_k"]
    forward_only = bool(w.get("forward_only"))
    # the routes come first: a skewed router sizes the receive buffers from the hottest rank
    hottest_rows = None
    if w["capacity"] == "measured":
        capacity, hottest_rows = measured_capacity_factor(make_routes(w, rank, device)[0], E,
                                                          world, k, group, device)
    else:
        capacity = min(float(w["capacity"]), float(world))
    cfg = mega_moe.MoEForwardConfig(receive_capacity_factor=capacity,
                                    enable_single_kernel_forward=True)
    # symmetric buffers first: they are plain cudaMalloc blocks outside torch's allocator
    op = mega_moe.FusedMoEForward(group, max_tokens_per_rank=T, hidden_size=H, top_k=k,
                                  num_experts=E, config=cfg)

    def set_mode(fast: bool):
        # fast: expert-weight gradients land in buffers allocated once, no host synchronisation
        # inside a step, saved activations are views of fixed buffers (the work per step is the
        # same); otherwise the drop-in defaults of the reference API
        op.persistent_weight_grads = fast
        op.host_sync_free = fast
        op.saved_views = fast

    set_mode(True)
    x, dy, rw, sel, gate_up, down = make_device_inputs(w, rank, world, device)
    x.requires_grad_(True)
    rw.requires_grad_(True)
    gate_up.requires_grad_(True)
    down.requires_grad_(True)
    def pinned_copy(t):
        # straight into pinned memory, without a pageable intermediate (host memory is scarce
        # when eight ranks share one box)
        h = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
        h.copy_(t.detach())
        return h

    host = dict(x=pinned_copy(x), dy=pinned_copy(dy), rw=pinned_copy(rw), sel=pinned_copy(sel))
    host_out = torch.empty(T, H, dtype=torch.bfloat16, pin_memory=True)
    host_gh = torch.empty(T, H, dtype=torch.bfloat16, pin_memory=True)
    host_grw = torch.empty(T, k, dtype=torch.float32, pin_memory=True)
    state = __import__("types").SimpleNamespace()

    def step(xx, rr, ss, dd):
        if forward_only:
            with torch.no_grad():
                return op(xx, ss, gate_up, down, rr), None
        out = mega_moe.MegaMoEFunction.apply(op, xx, rr, ss, gate_up, down, op.context.peer_mem,
                                             state)
        grads = torch.autograd.grad(out, [xx, rr, gate_up, down], dd)
        return out, grads

    def barrier():
        if world > 1:
            dist.barrier(group=group)
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(steps):
            fn()
        t1.record()
        barrier()
        ms = torch.tensor([t0.elapsed_time(t1)], device=device)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX, group=group)
        return float(ms.item())

    def resident_step():
        step(x, rw, sel, dy)

    def forward_step():
        with torch.no_grad():
            op(x, sel, gate_up, down, rw)

    # End-to-end step: this step's inputs come from pinned host memory and its results go back
    # to pinned host memory, every step.  Two sets of device staging buffers are allocated once;
    # the upload of step i+1 (copy stream) overlaps the kernels of step i, the download of step
    # i's results (second copy stream) overlaps step i+1, as the input pipeline of a training
    # loop would.  No allocation and no allocator bookkeeping happens inside the timed region.
    copy_in = torch.cuda.Stream(device)
    copy_out = torch.cuda.Stream(device)
    stage = [dict(x=torch.empty_like(x.detach()), rw=torch.empty_like(rw.detach()),
                  sel=torch.empty_like(sel), dy=torch.empty_like(dy)) for _ in range(2)]
    in_ready = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    copy_events = []            # (kind, start, end) of the timed copies
    step_marks = []             # per timed step: before / after the wait for inputs, step end
    in_flight = []              # results whose download may still be running
    e2e_state = dict(step=0, primed=False, record=False, h2d=True, d2h=True)

    def upload(slot):
        with torch.cuda.stream(copy_in):
            copy_in.wait_event(consumed[slot])
            ev0 = torch.cuda.Event(enable_timing=True)
            ev1 = torch.cuda.Event(enable_timing=True)
            ev0.record(copy_in)
            if e2e_state["h2d"]:
                for key in ("x", "rw", "sel", "dy"):
                    stage[slot][key].copy_(host[key], non_blocking=True)
            ev1.record(copy_in)
            in_ready[slot].record(copy_in)
        if e2e_state["record"]:
            copy_events.append(("h2d", ev0, ev1))

    def e2e_step():
        main = torch.cuda.current_stream(device)
        i = e2e_state["step"]
        slot = i % 2
        if not e2e_state["primed"]:
            consumed[0].record(main)
            consumed[1].record(main)
            upload(slot)
            e2e_state["primed"] = True
        upload(1 - slot)                       # next step's inputs, behind this step's kernels
        marks = None
        if e2e_state["record"]:
            marks = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            marks[0].record(main)
        main.wait_event(in_ready[slot])
        if marks:
            marks[1].record(main)
        buf = stage[slot]
        xx = buf["x"].detach().requires_grad_(True)
        rr = buf["rw"].detach().requires_grad_(True)
        out, grads = step(xx, rr, buf["sel"], buf["dy"])
        consumed[slot].record(main)
        done = torch.cuda.Event()
        done.record(main)
        if marks:
            marks[2].record(main)
            step_marks.append(marks)
        with torch.cuda.stream(copy_out):
            copy_out.wait_event(done)
            ev0 = torch.cuda.Event(enable_timing=True)
            ev1 = torch.cuda.Event(enable_timing=True)
            ev0.record(copy_out)
            if e2e_state["d2h"]:
                host_out.copy_(out.detach(), non_blocking=True)
            if grads is not None and e2e_state["d2h"]:
                host_gh.copy_(grads[0], non_blocking=True)
                host_grw.copy_(grads[1], non_blocking=True)
            ev1.record(copy_out)
        if e2e_state["record"]:
            copy_events.append(("d2h", ev0, ev1))
        # keep the results alive until their download has finished (two steps are plenty)
        in_flight.append((out, grads, ev1))
        if len(in_flight) > 2:
            in_flight.pop(0)[2].synchronize()
        e2e_state["step"] = i + 1

    for _ in range(args.warmup):
        resident_step()
    sampler = ClockSampler(local_rank)
    if rank == 0 and not os.environ.get("MOE_BENCH_NO_CLOCKS"):
        sampler.start()
    timer = GemmTimer()
    if not os.environ.get("MOE_BENCH_NO_EVENTS"):
        L.EVENT_HOOK = timer
    total_ms = timed(resident_step, args.steps)
    L.EVENT_HOOK = None
    clocks = sampler.stop() if rank == 0 else None
    gemm_ms = timer.summary()
    before = N.launch_count
    resident_step()
    torch.cuda.synchronize()
    launches_per_step = N.launch_count - before

    # forward alone (the metric also asks for the forward's time)
    forward_step()
    fwd_ms = timed(forward_step, args.steps) / args.steps

    # MOE_BENCH_NO_E2E=1 (kernel comparisons): one end-to-end step only
    e2e_steps = 1 if os.environ.get("MOE_BENCH_NO_E2E") else args.steps
    for _ in range(max(1, min(args.warmup, 2))):
        e2e_step()
    e2e_state["record"] = True
    e2e_sampler = ClockSampler(local_rank)
    if rank == 0 and not os.environ.get("MOE_BENCH_NO_CLOCKS"):
        e2e_sampler.start()
    e2e_timer = GemmTimer()
    if not os.environ.get("MOE_BENCH_NO_EVENTS"):
        L.EVENT_HOOK = e2e_timer
    e2e_ms = timed(e2e_step, e2e_steps) * args.steps / e2e_steps
    L.EVENT_HOOK = None
    e2e_clocks = e2e_sampler.stop() if rank == 0 else None
    e2e_state["record"] = False
    while in_flight:
        in_flight.pop(0)[2].synchronize()
    copy_ms = {"h2d": 0.0, "d2h": 0.0}
    for kind, ev0, ev1 in copy_events:
        copy_ms[kind] += ev0.elapsed_time(ev1)
    # MOE_BENCH_E2E_PROBE=1: the same loop with only the uploads, and with only the downloads,
    # to see which direction of host traffic the step is sensitive to
    e2e_probe = None
    if os.environ.get("MOE_BENCH_E2E_PROBE"):
        e2e_probe = {}
        for label, h2d_on, d2h_on in (("h2d_only", True, False), ("d2h_only", False, True)):
            e2e_state.update(h2d=h2d_on, d2h=d2h_on, record=False)
            e2e_step()
            probe_timer = GemmTimer()
            L.EVENT_HOOK = probe_timer
            ms = timed(e2e_step, args.steps) / args.steps
            L.EVENT_HOOK = None
            per = probe_timer.summary()
            e2e_probe[label] = {"ms_per_step": round(ms, 3),
                                "fc1_swiglu_ms": round(sum(per["fc1_swiglu"]) / len(per["fc1_swiglu"]), 3)}
        e2e_state.update(h2d=True, d2h=True)
        while in_flight:
            in_flight.pop(0)[2].synchronize()
    input_wait_ms = sum(a.elapsed_time(b) for a, b, _ in step_marks) / max(len(step_marks), 1)
    waits = torch.tensor([input_wait_ms], device=device)
    if world > 1:
        dist.all_reduce(waits, op=dist.ReduceOp.MAX, group=group)
    input_wait_max_ms = float(waits.item())
    e2e_compute_ms = sum(b.elapsed_time(c) for _, b, c in step_marks) / max(len(step_marks), 1)
    status = op.context.read_status()
    m_rows = int(op.context.metadata_stats[0].item())

    # The same step with the reference API's defaults: host reads of the row counts, copies of
    # the saved activations, freshly allocated weight gradients.  Skipped when the allocator
    # has no room for the copies.
    default_ms = None
    if not forward_only and not os.environ.get("MOE_BENCH_NO_DEFAULT_MODE"):
        free_b, _total = torch.cuda.mem_get_info(device)
        weights_b = (gate_up.numel() + down.numel()) * 2
        need = weights_b + 4 * m_rows * (H + 3 * F) * 2
        roomy = torch.tensor([1 if free_b > need else 0], device=device)
        if world > 1:
            dist.all_reduce(roomy, op=dist.ReduceOp.MIN, group=group)
        if int(roomy.item()):
            set_mode(False)
            op._grad_ws = None
            torch.cuda.empty_cache()
            for _ in range(2):
                resident_step()
            default_ms = timed(resident_step, args.steps) / args.steps
            set_mode(True)

    ms_per_step = total_ms / args.steps
    tokens_per_s = world * T / (ms_per_step / 1e3)
    e2e_tokens_per_s = world * T / (e2e_ms / args.steps / 1e3)
    h2d = sum(t.numel() * t.element_size() for t in host.values())
    d2h = sum(t.numel() * t.element_size() for t in
              ((host_out,) if forward_only else (host_out, host_gh, host_grw)))

    # Yardstick for the write-dominated launches (the weight gradients at few rows per expert
    # write 30x what they read): the rate at which this GPU fills memory, measured here with a
    # plain fill of 2 GB outside every timed region.  A write stream does not reach the copy
    # peak the roofline fraction is quoted against.
    write_only_gbs = None
    try:
        free_b, _total = torch.cuda.mem_get_info(device)
        if free_b > (6 << 30):
            scratch = torch.empty(2 << 30, dtype=torch.uint8, device=device)
            scratch.fill_(1)
            torch.cuda.synchronize()
            w0 = torch.cuda.Event(enable_timing=True)
            w1 = torch.cuda.Event(enable_timing=True)
            w0.record()
            for _ in range(4):
                scratch.fill_(0)
            w1.record()
            torch.cuda.synchronize()
            write_only_gbs = round(4 * scratch.numel() / (w0.elapsed_time(w1) / 1e3) / 1e9, 1)
            del scratch
    except torch.OutOfMemoryError:
        write_only_gbs = None

    # roofline of the dominant kernel (the grouped GEMM, six launches per step)
    peaks = measured_peaks()
    epr = E // world
    gemm_names = ("fc1_swiglu", "fc2_combine") if forward_only else (
        "fc1_swiglu", "fc2_combine", "fc2_dgrad", "fc2_wgrad", "fc1_wgrad", "fc1_dgrad_combine")
    gemm_total_ms = max(sum(sum(gemm_ms.get(n, [])) for n in gemm_names) / args.steps, 1e-9)
    weight_bytes = epr * 3 * H * F * 2
    if forward_only:
        flops = 6.0 * m_rows * H * F
        bytes_alg = weight_bytes + m_rows * 2 * (H + F + F + H)
    else:
        flops = 18.0 * m_rows * H * F
        # weights are read twice (forward, input gradient) and their gradients written once;
        # every [M, *] operand or result of the six GEMMs is read or written once
        act_bytes = m_rows * 2 * (H + 2 * F + F + H + H + F + 2 * F + H + H + F + 2 * F + H)
        bytes_alg = 3 * weight_bytes + act_bytes
    t_tensor = flops / (peaks["tflops"] * 1e12)
    t_hbm = bytes_alg / (peaks["hbm_gbs"] * 1e9)
    if t_hbm >= t_tensor:
        achieved = bytes_alg / (gemm_total_ms / 1e3) / 1e9
        roofline = dict(bound="hbm", achieved=round(achieved, 1), peak=peaks["hbm_gbs"],
                        unit="GB/s", frac=round(achieved / peaks["hbm_gbs"], 4), traffic=None)
    else:
        achieved = flops / (gemm_total_ms / 1e3) / 1e12
        roofline = dict(bound="tensor", achieved=round(achieved, 1), peak=peaks["tflops"],
                        unit="TFLOP/s", frac=round(achieved / peaks["tflops"], 4), traffic=None)
    roofline["traffic"] = None if forward_only else measured_traffic(H, F, k, m_rows, epr)
    roofline["traffic_unit"] = "bytes per step (six launches), ncu capture of a slice scaled by local experts"
    roofline["algorithmic_bytes"] = bytes_alg
    roofline["algorithmic_flops"] = flops
    roofline["kernel"] = "grouped_gemm_kernel / skinny_gemm_kernel (the GEMM launches of a step)"
    roofline["kernel_ms_per_step"] = round(gemm_total_ms, 3)
    roofline["peak_source"] = peaks["source"]
    roofline["hbm_write_only_gbs_measured_here"] = write_only_gbs
    roofline["per_launch_ms"] = {k_: round(sum(v) / len(v), 3) for k_, v in gemm_ms.items()}
    # north_star's roofline: the slower of the step's FLOPs at the dense bf16 peak and the
    # dispatch + combine bytes that leave a rank at the NVLink rate, against the whole step
    remote = (world - 1) / world
    nvlink_bytes = (2 if forward_only else 4) * T * k * H * 2 * remote
    step_floor_ms = max(flops / (peaks["tflops"] * 1e12), nvlink_bytes / 770e9) * 1e3
    roofline["step"] = {
        "floor_ms": round(step_floor_ms, 3), "frac_of_measured": round(step_floor_ms / ms_per_step, 4),
        "frac_of_nominal_2250_tflops_900_gbs": round(
            max(flops / 2.25e15, nvlink_bytes / 900e9) * 1e3 / ms_per_step, 4),
        "nvlink_bytes_out_per_rank": int(nvlink_bytes),
        "literal_6kHF_ratio": round(6.0 * T * k * H * F / 2.25e15 * 1e3 / ms_per_step, 4)}

    line = None
    if rank == 0:
        # MOE_BENCH_NO_CPU=1 skips the CPU leg (profiler runs, where only the launches matter)
        cpu = (cpu_baseline_sample(w, seconds_hint=20.0)
               if world == 1 and not os.environ.get("MOE_BENCH_NO_CPU") else None)
        what = "fwd" if forward_only else "fwd+bwd"
        line = {
            "metric": METRIC if name == DEFAULT_WORKLOAD else f"MoE {what} tokens/s ({name})",
            "value": round(tokens_per_s, 1), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 3),
            "fwd_ms": round(fwd_ms, 3),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": name, "tokens_per_rank": T, "hidden": H, "ffn": F,
                       "experts": E, "top_k": k, "experts_per_rank": epr,
                       "router": f"zipf s={w['zipf']}" if w.get("zipf") else "balanced",
                       "receive_capacity_factor": capacity,
                       "hottest_rank_rows": hottest_rows,
                       "received_rows_rank0": m_rows, "parallelism": f"ep{world}",
                       "pass": what,
                       "gemm_tile_mode": ("single", "pair", "skinny")[L.gemm_tile_mode(op.context)],
                       "wgrad_tile_mode": ("single", "pair", "unit")[L.wgrad_tile_mode(op.context)],
                       "fused_dispatch": bool(L.fused_dispatch_enabled(op.context)),
                       "operator_mode": "persistent_weight_grads + host_sync_free + saved_views",
                       "host_threads_bound_to_gpu_local_cpus": host_cpus,
                       "l2": "inputs larger than L2 (expert weights and their gradients "
                             f"are {3 * weight_bytes / 1e9:.1f} GB per rank and step)"},
            "tokens_per_s_per_gpu": round(tokens_per_s / world, 1),
            "value_default_mode": (round(world * T / (default_ms / 1e3), 1)
                                   if default_ms else None),
            "ms_per_step_default_mode": round(default_ms, 3) if default_ms else None,
            "e2e": {"value": round(e2e_tokens_per_s, 1), "unit": "tokens/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": round(e2e_ms / args.steps, 3),
                    "h2d_gbs": round(h2d * args.steps / max(copy_ms["h2d"], 1e-6) / 1e6, 1),
                    "d2h_gbs": round(d2h * args.steps / max(copy_ms["d2h"], 1e-6) / 1e6, 1),
                    # device time of a step's kernels inside the end-to-end loop, and how long
                    # the compute stream waited for the step's inputs (rank 0)
                    "kernels_ms_per_step": round(e2e_compute_ms, 3),
                    "input_wait_ms_per_step": round(input_wait_ms, 3),
                    "input_wait_ms_per_step_max_over_ranks": round(input_wait_max_ms, 3),
                    "probe": e2e_probe,
                    "per_launch_ms": {k_: round(sum(v) / len(v), 3)
                                      for k_, v in e2e_timer.summary().items()},
                    "clocks": e2e_clocks},
            "gpu_launches": launches_per_step * args.steps,
            "gpu_launches_per_step": launches_per_step,
            "roofline": roofline,
            "clocks": clocks,
            "device_status": status.code,
            "peak_torch_mem_gb": round(torch.cuda.max_memory_allocated() / 1e9, 2),
        }
        if cpu is not None:
            line["cpu_baseline"] = cpu
    op.finalize()
    if world > 1:
        dist.destroy_process_group()
    return line


def cpu_baseline_sample(w, seconds_hint=20.0, steps=1, warmup=0):
    """Time the CPU oracle (forward_saved + backward) on a bounded sample of the workload.

    The sample keeps the per-expert problem of the workload (same hidden / FFN size, the same
    mean rows per expert) but only ``sample_experts`` experts, so that the host holds the
    weights and one pass takes seconds.  tokens/s = (sample routes / top_k) / time.
    """
    from oracle import moe_oracle as O

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    H, F, E, k, T = w["hidden"], w["ffn"], w["experts"], w["top_k"], w["tokens"]
    rows_per_expert = max(1, T * k // E)
    flop_per_expert = 18.0 * rows_per_expert * H * F
    budget = seconds_hint * 0.15e12          # assume ~0.15 TFLOP/s of bf16 matmul on the host
    sample_experts = int(max(1, min(E, 64, budget // flop_per_expert)))
    # top-k' routes per token over the sampled experts (k' = k when the sample holds at least k
    # experts), token t taking experts (t * k' + j) mod sample: every expert gets the workload's
    # rows per expert and every token's k' rows are summed back, as in the layer
    kk = min(k, sample_experts)
    tokens = max(1, rows_per_expert * sample_experts // kk)
    routes = tokens * kk
    g = torch.Generator().manual_seed(0)
    x = torch.randn(tokens, H, generator=g).to(torch.bfloat16)
    dy = torch.randn(tokens, H, generator=g).to(torch.bfloat16)
    sel = (torch.arange(tokens * kk) % sample_experts).to(torch.int32).view(tokens, kk)
    rw = torch.softmax(torch.randn(tokens, kk, generator=g), dim=-1)
    w1 = (torch.randn(sample_experts, F, H, generator=g) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(sample_experts, F, H, generator=g) * 0.02).to(torch.bfloat16)
    w3 = (torch.randn(sample_experts, H, F, generator=g) * 0.02).to(torch.bfloat16)
    forward_only = bool(w.get("forward_only"))

    def one():
        _, saved = O.forward_saved([x], [rw], [sel], [w1], [w2], [w3], kk)
        if not forward_only:
            O.backward(saved, [dy])

    for _ in range(warmup):
        one()
    t0 = time.perf_counter()
    for _ in range(steps):
        one()
    dt = (time.perf_counter() - t0) / steps
    # a token of the workload carries k routes: the sample's routes / k are its tokens
    return {"value": round(routes / k / dt, 2), "unit": "tokens/s", "cores": threads,
            "kind": "port",
            "sample": f"{sample_experts} of {E} experts with {routes // sample_experts} rows each "
                      f"(H={H}, F={F}), {tokens} tokens at top-{kk}: {routes} routes = "
                      f"{routes / k:.1f} tokens of the workload at top-{k}; "
                      f"{dt:.2f} s per {'forward' if forward_only else 'forward+backward'}",
            "seconds_per_pass": round(dt, 3)}


def run_reference(args, w, name):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return None
    cpu = cpu_baseline_sample(w, seconds_hint=10.0, steps=args.steps, warmup=min(args.warmup, 1))
    T = w["tokens"]
    return {
        "impl": "reference",
        "metric": METRIC if name == DEFAULT_WORKLOAD else f"MoE fwd+bwd tokens/s ({name})",
        "value": cpu["value"], "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(cpu["seconds_per_pass"] * 1e3, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": name, "tokens_per_rank": T, "hidden": w["hidden"],
                   "ffn": w["ffn"], "experts": w["experts"], "top_k": w["top_k"]},
        "cpu_baseline": cpu,
        "e2e": {"value": cpu["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--tokens", type=int, default=None, help="override tokens per rank")
    args = ap.parse_args()
    w = dict(WORKLOADS[args.workload])
    if args.tokens:
        w["tokens"] = args.tokens
    if args.impl == "reference":
        line = run_reference(args, w, args.workload)
    else:
        line = run_ours(args, w, args.workload)
    if line is not None:
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
