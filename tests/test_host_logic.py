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
