"""CPU tests of the host-side logic: config validation, the C-ABI surface, weight-operand
description, and the multi-rank plumbing (handle exchange, count cube) under gloo ranks."""
import ctypes
import os
import re
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

REPO = Path(__file__).resolve().parent.parent


def test_config_defaults_and_validation():
    from mega_moe import MoEForwardConfig
    c = MoEForwardConfig()
    assert c.num_aicore_programs >= 2 and c.num_aivector_programs >= 2
    assert c.single_kernel_group_windows == 32
    assert c.resolved_receive_capacity_factor(8) == 8.0
    assert MoEForwardConfig(receive_capacity_factor=1.25).resolved_receive_capacity_factor(8) == 1.25
    assert MoEForwardConfig(single_kernel_dispatch_block_size_m=None) \
        .single_kernel_dispatch_block_size_m == 128
    for kw, exc in [
        (dict(dispatch_fc1_block_size_m=48), ValueError),
        (dict(fc1_gemm_block_size_m=512), ValueError),
        (dict(fc1_gemm_block_size_m=256, fc1_gemm_block_size_n=512), ValueError),
        (dict(receive_capacity_factor=0.5), ValueError),
        (dict(activation="relu"), ValueError),
        (dict(situ_beta="1"), TypeError),
        (dict(situ_beta=-1.0), ValueError),
        (dict(situ_linear_beta=0.0), ValueError),
        (dict(clamp_limit=0.0), ValueError),
        (dict(enable_moonep=1), TypeError),
        (dict(enable_single_kernel_forward="yes"), TypeError),
        (dict(save_fc1_dtype="int8"), ValueError),
        (dict(single_kernel_group_windows=3), ValueError),
        (dict(enable_single_kernel_forward=True, fc1_gemm_block_size_m=128), ValueError),
        (dict(moonep_udma_chunk_bytes=3), ValueError),
        (dict(moonep_fused_balanced_count=False), ValueError),
        (dict(enable_moonep=True), NotImplementedError),
    ]:
        with pytest.raises(exc):
            MoEForwardConfig(**kw)
    for fmt in ("bf16", "fp16", "fp8"):
        assert MoEForwardConfig(save_fc1_dtype=fmt).save_fc1_dtype == fmt
    with pytest.raises(Exception):
        c.activation = "situglu"  # frozen


def test_library_exports_every_declared_symbol():
    """The shared library loads and exports each function include/mega_moe_b200.h declares,
    and the ctypes table binds exactly that set (no compute call is made)."""
    from mega_moe import _native as N
    header = (REPO / "include" / "mega_moe_b200.h").read_text()
    declared = set(re.findall(r"\b(mm_[a-z0-9_]+)\s*\(", header)) - {"mm_status_record"}
    assert declared, "no declarations found"
    lib = ctypes.CDLL(str(N.LIB_PATH))
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared but not exported"
    assert declared == set(N.SIGNATURES), declared ^ set(N.SIGNATURES)
    assert N.lib().mm_abi_version() >= 1
    assert N.lib().mm_route_scratch_bytes(131072, 1024) == (64 + 1) * 1024 * 4


def test_pack_gate_up_weights_and_operand_description():
    from mega_moe import pack_gate_up_weights
    from mega_moe.ops._launch import weight_operand
    g = torch.randn(3, 8, 16).to(torch.bfloat16)
    u = torch.randn(3, 8, 16).to(torch.bfloat16)
    packed = pack_gate_up_weights(g, u)
    assert packed.shape == (3, 16, 16) and packed.is_contiguous()
    assert torch.equal(packed[:, :, :8], g.transpose(1, 2))
    assert torch.equal(packed[:, :, 8:], u.transpose(1, 2))
    with pytest.raises(TypeError):
        pack_gate_up_weights(g.float(), u.float())
    with pytest.raises(ValueError):
        pack_gate_up_weights(g, u[:, :4])
    # [E, H, 2F] packed table as FC1 operand: n contiguous -> MN-major
    assert weight_operand(packed, 1, 2) == (0, 16, 256, 16)
    # the same table as the FC1 input-gradient operand (k = 2F): k contiguous -> K-major
    assert weight_operand(packed.transpose(1, 2), 1, 2) == (1, 16, 256, 16)
    down = torch.randn(3, 16, 8).to(torch.bfloat16)
    assert weight_operand(down, 2, 1) == (1, 8, 128, 16)
    down_view = down.transpose(1, 2).contiguous().transpose(1, 2)     # [E, H, F] view of [E, F, H]
    assert weight_operand(down_view, 2, 1) == (0, 16, 128, 16)
    with pytest.raises(ValueError):
        weight_operand(torch.randn(3, 16, 16)[:, ::2, ::2], 1, 2)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from mega_moe import _native as N
    monkeypatch.setattr(N, "_lib", None)
    monkeypatch.setattr(N, "LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        N.lib()


# ------------------------------------------------------------------------------------------
# world_size-2 gloo ranks: symmetric-handle exchange and the count-cube all-gather
# ------------------------------------------------------------------------------------------
class _FakeLib:
    """Stands in for the CUDA-IPC calls: 'allocations' are fake addresses unique per rank."""

    def __init__(self, rank):
        self.rank = rank
        self.opened = []

    def mm_symm_alloc(self, nbytes, base_ref, handle):
        base_ref._obj.value = 0x1000000 * (self.rank + 1)
        handle.raw = (b"rank%02d" % self.rank).ljust(64, b"\0")
        return 0

    def mm_symm_open(self, handle, out_ref):
        peer = int(bytes(handle)[4:6])
        self.opened.append(peer)
        out_ref._obj.value = 0x1000000 * (peer + 1) + 0x10
        return 0

    def mm_symm_close(self, p):
        return 0

    def mm_symm_free(self, p):
        return 0

    def mm_last_error(self):
        return b""


def _gloo_worker(rank, world, port, q):
    sys.path[:0] = [str(REPO), str(REPO / "mega-moe-td_b200")]
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from mega_moe import _native as N
    from mega_moe.runtime import workspace as W
    from oracle import moe_oracle as O
    fake = _FakeLib(rank)
    N.lib = lambda: fake
    blk = W.SymmetricBlock({"flags": 4096, "peer_mem": 1000, "combine_mem": 300}, rank, world,
                           dist.group.WORLD, torch.device("cpu"))
    ok = blk.offsets == {"flags": 0, "peer_mem": 4096, "combine_mem": 4096 + 1024}
    ok &= blk.peer_bases[rank] == 0x1000000 * (rank + 1)
    ok &= all(blk.peer_bases[r] == 0x1000000 * (r + 1) + 0x10 for r in range(world) if r != rank)
    ok &= sorted(fake.opened) == [r for r in range(world) if r != rank]
    table = blk.peer_table("peer_mem")
    ok &= table.tolist() == [b + 4096 for b in blk.peer_bases]
    # count rows -> replicated cube, exactly as launch_routing_metadata gathers them
    experts, k, tokens = 4 * world, 3, 50
    rng = np.random.default_rng(11)
    sels = [rng.integers(-1, experts + 1, size=(tokens, k)).astype(np.int32) for _ in range(world)]
    meta = O.routing_metadata(sels, experts)
    bins = O.next_power_of_2(experts)
    row = torch.from_numpy(meta[rank]["count_cube"][rank].astype(np.int32))
    cube = torch.zeros(world * bins, dtype=torch.int32)
    dist.all_gather_into_tensor(cube, row)
    ok &= torch.equal(cube.view(world, bins), torch.from_numpy(meta[rank]["count_cube"]))
    q.put((rank, bool(ok)))
    dist.barrier()
    dist.destroy_process_group()


def test_symmetric_exchange_and_count_cube_world2():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    world = 2
    port = 29650 + (os.getpid() % 40)
    procs = [ctx.Process(target=_gloo_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert results == {0: True, 1: True}


def test_tile_mode_and_dispatch_defaults(monkeypatch):
    """Host-side choices that need no GPU: the GEMM tile mode follows the expected rows per
    local expert, the dispatch is fused only when there are peers, and the environment
    switches override both."""
    import types
    from mega_moe.ops import _launch as L
    for var in ("MOE_GEMM_MODE", "MOE_GEMM_PAIR", "MOE_FUSED_DISPATCH"):
        monkeypatch.delenv(var, raising=False)

    def ctx(tokens, top_k, world, experts):
        return types.SimpleNamespace(max_tokens_per_rank=tokens, top_k=top_k, world_size=world,
                                     num_experts=experts)

    # the headline layer: 146 rows per expert on one GPU, 292 / 585 / 1170 on 2 / 4 / 8
    assert L.gemm_tile_mode(ctx(8192, 16, 1, 896)) == L.TILE_SKINNY
    for world in (2, 4, 8):
        assert L.gemm_tile_mode(ctx(8192, 16, world, 896)) == L.TILE_SINGLE
    assert L.gemm_tile_mode(None) == L.TILE_SINGLE and not L.pair_mode_enabled()
    assert L.fused_dispatch_enabled(ctx(8192, 16, 8, 896))
    assert not L.fused_dispatch_enabled(ctx(8192, 16, 1, 896))

    monkeypatch.setenv("MOE_GEMM_MODE", "single")
    assert L.gemm_tile_mode(ctx(8192, 16, 1, 896)) == L.TILE_SINGLE
    monkeypatch.setenv("MOE_GEMM_MODE", "skinny")
    assert L.gemm_tile_mode(ctx(8192, 16, 8, 896)) == L.TILE_SKINNY
    monkeypatch.setenv("MOE_GEMM_MODE", "pair")
    assert L.gemm_tile_mode(None) == L.TILE_PAIR and L.pair_mode_enabled()
    monkeypatch.setenv("MOE_GEMM_MODE", "wide")
    with pytest.raises(ValueError):
        L.gemm_tile_mode(None)
    monkeypatch.setenv("MOE_GEMM_MODE", "auto")
    monkeypatch.setenv("MOE_GEMM_PAIR", "1")
    assert L.gemm_tile_mode(ctx(8192, 16, 1, 896)) == L.TILE_PAIR
    monkeypatch.setenv("MOE_FUSED_DISPATCH", "1")
    assert L.fused_dispatch_enabled(ctx(8192, 16, 1, 896))
    monkeypatch.setenv("MOE_FUSED_DISPATCH", "0")
    assert not L.fused_dispatch_enabled(ctx(8192, 16, 8, 896))


def test_saved_format_helpers(monkeypatch):
    from mega_moe import _native as N
    from mega_moe.ops import _launch as L
    from mega_moe.runtime.workspace import saved_recompute_enabled
    assert N.FC1_FORMAT_IDS == {"bf16": 0, "fp16": 1, "fp8": 2}
    assert L.fc1_format_of(torch.empty(1, 2, dtype=torch.bfloat16)) == 0
    assert L.fc1_format_of(torch.empty(1, 2, dtype=torch.float16)) == 1
    assert L.fc1_format_of(torch.empty(1, 2, dtype=torch.float8_e4m3fn)) == 2
    with pytest.raises(TypeError):
        L.fc1_format_of(torch.empty(1, 2))
    q = torch.empty(4, 256, dtype=torch.float8_e4m3fn)
    with pytest.raises(ValueError):
        L._fc1_scale_args(q, None, 0, 128)
    with pytest.raises(ValueError):
        L._fc1_scale_args(q, torch.empty(4, 3), 128, 128)          # wrong table shape
    fmt, ptr, group = L._fc1_scale_args(q, torch.empty(4, 2), 128, 128)
    assert fmt == 2 and group == 128 and ptr
    assert L._fc1_scale_args(torch.empty(4, 256, dtype=torch.bfloat16), None, 0, 128) == (0, None, 0)
    monkeypatch.delenv("MOE_SAVED_RECOMPUTE", raising=False)
    assert not saved_recompute_enabled()
    monkeypatch.setenv("MOE_SAVED_RECOMPUTE", "1")
    assert saved_recompute_enabled()


class _FakeSymmetricBlock:
    """CPU stand-in for the CUDA-IPC block: same region bookkeeping, plain host tensors."""

    def __init__(self, regions, rank, world_size, group, device):
        self.regions = dict(regions)
        self.rank, self.world_size = rank, world_size
        self._mem = {name: torch.zeros(max(size, 16), dtype=torch.uint8)
                     for name, size in regions.items()}

    def local(self, name, dtype):
        return self._mem[name][:self.regions[name]].view(dtype)

    def peer_table(self, name):
        return torch.tensor([self._mem[name].data_ptr()] * self.world_size, dtype=torch.int64)

    def free(self):
        self._mem = {}


@pytest.mark.parametrize("grouped_tile,fused_tile", [(128, None), (128, 256), (256, 128), (128, 16)])
@pytest.mark.parametrize("recompute", [False, True])
def test_workspace_sizing_on_cpu(monkeypatch, grouped_tile, fused_tile, recompute):
    """Workspace sizing with host tensors in place of the symmetric block (the reference checks
    its own sizing the same way, tests/function/test_forward_workspace.py:13-44): the receive
    buffer holds int(T * k * factor) rows, the source-tile bound covers the worst case of every
    route going to one expert for both dispatch tile sizes, the count cube has
    next_pow2(world * experts_per_rank) bins per rank, and the tile tables cover every row tile
    a rank can receive."""
    from mega_moe.runtime import workspace as W
    monkeypatch.setattr(W, "SymmetricBlock", _FakeSymmetricBlock)
    if recompute:
        monkeypatch.setenv("MOE_SAVED_RECOMPUTE", "1")
    else:
        monkeypatch.delenv("MOE_SAVED_RECOMPUTE", raising=False)
    tokens, hidden, top_k, experts, world, factor = 257, 16, 3, 14, 2, 2
    ctx = W.create_moe_forward_context(
        max_tokens_per_rank=tokens, hidden_size=hidden, top_k=top_k, num_experts=experts,
        rank=0, world_size=world, receive_capacity_factor=factor,
        dispatch_fc1_block_size_m=grouped_tile, single_kernel_dispatch_block_size_m=fused_tile,
        device=torch.device("cpu"))
    try:
        routes = tokens * top_k
        cap = int(routes * factor)
        epr = experts // world
        assert ctx.experts_per_rank == ctx.physical_experts_per_rank == epr
        assert ctx.max_received_routes == cap
        for tile in (grouped_tile, fused_tile or grouped_tile):
            assert (routes + tile - 1) // tile <= ctx.max_source_tiles
        assert ctx.peer_mem.numel() == cap * hidden and ctx.peer_mem.dtype == torch.bfloat16
        assert ctx.routing_weight_mem.numel() == cap and ctx.routing_weight_mem.dtype == torch.float32
        assert tuple(ctx.combine_mem.shape) == (routes, hidden)
        assert ctx.combine_gate_mem.numel() == routes
        assert ctx.dispatch_flags.numel() == world * epr
        assert (ctx.redispatch_mem is not None) == recompute
        if recompute:
            assert ctx.redispatch_mem.numel() == cap * hidden
        bins = W.next_power_of_2(world * epr)
        assert ctx.metadata_num_bins == bins == 16
        assert ctx.metadata_counts_mem.numel() == world * bins
        assert ctx.metadata_recv_counts_re.shape == (world, epr)
        assert ctx.metadata_recv_seg_starts.shape == (epr, world + 1)
        assert ctx.metadata_recv_expert_offs.numel() == epr + 1
        assert ctx.metadata_stats.numel() == 2 + world
        # every expert can end on a partial tile: tiles <= cap // rows + experts
        assert ctx.mtile_group.numel() >= cap // 128 + epr
        assert ctx.mtile2_group.numel() >= cap // 256 + epr
        assert ctx.row_src_rank.numel() >= cap and ctx.route_to_send.numel() == routes
        assert bool((ctx.route_to_send == -1).all())
        assert ctx.disp_order_prefix.numel() == world * epr + 1
        assert W.context_of(ctx.peer_mem) is ctx
    finally:
        W.unregister_context(ctx)
    with pytest.raises(NotImplementedError):
        W.create_moe_forward_context(
            max_tokens_per_rank=8, hidden_size=16, top_k=2, num_experts=4, rank=0, world_size=1,
            receive_capacity_factor=1.0, dispatch_fc1_block_size_m=128, enable_moonep=True,
            device=torch.device("cpu"))


def test_bench_binds_host_threads_to_the_gpus_cpus(monkeypatch):
    """bench.py's NUMA binding for multi-GPU runs, against a fake NVML: the NVML core mask is
    intersected with the cores the process may use; nothing changes when NVML is missing, the
    intersection is too small, or the switch is set."""
    import types
    sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
    import bench
    calls = []
    monkeypatch.setattr(os, "sched_getaffinity", lambda pid: set(range(0, 48)), raising=False)
    monkeypatch.setattr(os, "sched_setaffinity", lambda pid, cpus: calls.append(set(cpus)),
                        raising=False)
    monkeypatch.setattr(os, "cpu_count", lambda: 96)
    monkeypatch.delenv("MOE_BENCH_NO_AFFINITY", raising=False)
    fake = types.SimpleNamespace(
        nvmlDeviceGetHandleByUUID=lambda u: u,
        nvmlDeviceGetCpuAffinity=lambda h, words: [0xFFFF0000, 0xFF][:words])   # cores 16-31, 64-71
    assert bench.bind_host_threads_near_gpu(0, nvml=fake, uuid="abc") == 16
    assert calls == [set(range(16, 32))]
    narrow = types.SimpleNamespace(nvmlDeviceGetHandleByUUID=lambda u: u,
                                   nvmlDeviceGetCpuAffinity=lambda h, words: [0, 0x1][:words])
    assert bench.bind_host_threads_near_gpu(0, nvml=narrow, uuid="abc") is None

    def broken(h, words):
        raise RuntimeError("not supported")
    bad = types.SimpleNamespace(nvmlDeviceGetHandleByUUID=lambda u: u,
                                nvmlDeviceGetCpuAffinity=broken)
    assert bench.bind_host_threads_near_gpu(0, nvml=bad, uuid="abc") is None
    monkeypatch.setenv("MOE_BENCH_NO_AFFINITY", "1")
    assert bench.bind_host_threads_near_gpu(0, nvml=fake, uuid="abc") is None
    assert len(calls) == 1


@pytest.mark.parametrize("world,experts,top_k,tokens", [(1, 8, 2, 70), (2, 8, 3, 48), (4, 16, 4, 33)])
def test_saved_index_section_from_plan_tables(world, experts, top_k, tokens):
    """The index keys the forward adds to its saved dict are pure functions of the routing
    tables; on CPU tensors they must equal the oracle's restatement of the reference's
    enrichment (ops/_single_saved_adapter.py:247-340) for every rank."""
    import types

    from mega_moe.ops.forward import FusedMoEForward
    from oracle import moe_oracle as O
    rng = np.random.default_rng(world * 100 + experts)
    sels = [rng.integers(0, experts, size=(tokens, top_k)).astype(np.int32) for _ in range(world)]
    meta = O.routing_metadata(sels, experts)
    for r in range(world):
        want = O.saved_contract_tables(meta[r], sels[r], world)
        m = meta[r]["num_received_routes"]
        sent = meta[r]["num_sent_routes"]
        t = lambda a: torch.as_tensor(np.asarray(a).astype(np.int32))
        plan = types.SimpleNamespace(
            send_route_indices=t(meta[r]["send_route_indices"]),
            route_to_send=t(meta[r]["route_to_send"]),
            row_arrival=t(want["local_sort_idxs"]), arrival_row=t(want["inv_local"]),
            metadata_recv_counts_re=t(meta[r]["recv_counts_re"]),
            metadata_count_row=t(meta[r]["count_cube"][r]))
        op = types.SimpleNamespace(num_experts=experts, world_size=world)
        got = FusedMoEForward._saved_index_section(op, plan, m, sent, True)
        for key in ("sort_idxs", "inv_sort", "forward_send_route", "local_sort_idxs", "inv_local",
                    "meta_expert_ids", "meta_split_cum", "meta_tile_num", "meta_tile_num_cum",
                    "num_tiles_total"):
            np.testing.assert_array_equal(got[key].numpy().astype(np.int64),
                                          np.asarray(want[key]).astype(np.int64), err_msg=key)
        assert got["splits_send_list"] == want["splits_send_list"]
        assert got["splits_recv_list"] == want["splits_recv_list"]
        lazy = FusedMoEForward._saved_index_section(op, plan, m, sent, False)
        assert lazy["splits_send_list"] is None and lazy["meta_expert_ids"] is None
        assert torch.equal(lazy["inv_sort"], got["inv_sort"])


def test_epochs_grow_and_exhaustion_raises_instead_of_wrapping():
    """Flags carry epochs that only grow (the reference's rule, ops/forward.py:368-385,
    tests/function/test_single_replica_epoch.py:57-62): at the end of the int32 range the
    context raises instead of wrapping to a value an old flag could satisfy."""
    from mega_moe.runtime.workspace import MoEForwardContext
    ctx = MoEForwardContext(hidden_size=64, num_experts=8, experts_per_rank=4, replica_budget=0,
                            physical_experts_per_rank=4, world_size=2, rank=0,
                            receive_capacity_factor=1.0, max_source_tiles=1)
    first = [ctx.next_dispatch_epoch() for _ in range(3)]
    assert first == sorted(first) and len(set(first)) == 3 and first[0] >= 1
    ctx.dispatch_epoch = 2**31 - 3
    assert ctx.next_dispatch_epoch() == 2**31 - 2
    with pytest.raises(RuntimeError, match="epoch exhausted"):
        ctx.next_dispatch_epoch()
    ctx.barrier_epoch = 2**31 - 2
    with pytest.raises(RuntimeError, match="epoch exhausted"):
        ctx._next_epoch()
