"""Generate ``saved_tables.npz`` and ``saved_formats.npz`` from the reference itself.

    python tests/golden/make_golden_saved.py /path/to/reference

Two kinds of reference code run here, on the CPU:

* plain torch helpers, imported by file path like ``make_golden.py`` does:
  ``prepare_moe_metadata`` (ops/_torch_forward.py:103-128) and
  ``_arrival_to_slot_permutation`` (ops/_moonep_torch_forward.py:192-223) -> the index
  section of the saved contract (``saved_tables.npz``);
* Triton-Ascend device code, which cannot be launched here.  Its arithmetic is plain
  ``tl`` tensor code, so the *source text* of the reference is compiled with ``ast`` and
  executed against a small torch-backed stand-in for the ``tl`` namespace (the reference's
  own host tests run production ``@triton.jit`` helpers the same way,
  tests/function/test_single_kernel_routing_metadata.py:41-135):
    - the FC1 save leg of the forward kernel, the ``if FC1_SAVE_FP16 / elif FC1_FP8 / else``
      statement at kernels/fused_forward.py:891-949, taken out of
      ``_partition_pipeline_fc1_activation_group_ub`` and run once per (row tile, column group);
    - ``_recompute_act_rows`` (kernels/mega_bwd.py:1414-1465), the activation recompute of the
      backward, for the three activations and for bf16 / fp8 saved rows.
  The stand-in computes in torch fp32 on the CPU, so the fixtures pin the reference's formulas,
  operation order, rounding points and table layouts, not the Ascend vector unit's ulp-level
  behaviour of ``sigmoid`` / ``tanh`` (``saved_formats.npz``).
"""

from __future__ import annotations

import ast
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
sys.path.insert(0, str(REPO))
sys.path.insert(0, str(HERE))

from make_golden import bits, load_reference  # noqa: E402


# ----------------------------------------------------------------------------------------
# torch-backed stand-in for the parts of ``tl`` the two code fragments use
# ----------------------------------------------------------------------------------------
class Ptr:
    """A pointer into a flat buffer: base tensor + element offsets (int or LongTensor)."""

    def __init__(self, buf: torch.Tensor, offs=0):
        self.buf = buf
        self.offs = offs

    def __add__(self, other):
        if isinstance(other, torch.Tensor):
            other = other.long()
        return Ptr(self.buf, self.offs + other)

    __radd__ = __add__

    @property
    def dtype(self):
        return types.SimpleNamespace(element_ty=self.buf.dtype)


def _raw(buf: torch.Tensor) -> torch.Tensor:
    """Byte/short view that supports indexing for every element type (fp8 included)."""
    return buf.view({1: torch.uint8, 2: torch.int16, 4: torch.int32}[buf.element_size()])


class V(torch.Tensor):
    """Tensor of the stand-in.  ``scalar / tensor`` is a true fp32 division here, as it is in
    device code (torch would compute it as ``scalar * reciprocal(tensor)``, which rounds twice)."""

    def __rtruediv__(self, other):
        return torch.full_like(self, other).as_subclass(V) / self


def as_v(t):
    return torch.as_tensor(t).as_subclass(V)


class Index(int):
    """Loop index of a ``range`` inside jitted code: an int that accepts ``.to(dtype)``."""

    def to(self, _dtype):
        return self


def jit_range(*args):
    return (Index(i) for i in range(*args))


class TL:
    constexpr = object
    float32 = torch.float32
    float16 = torch.float16
    float8e4nv = torch.float8_e4m3fn
    int64 = torch.int64
    int32 = torch.int32

    class math:
        tanh = staticmethod(torch.tanh)

    sigmoid = staticmethod(torch.sigmoid)
    abs = staticmethod(torch.abs)

    @staticmethod
    def arange(start, end):
        return as_v(torch.arange(start, end))

    @staticmethod
    def where(cond, a, b):
        return torch.where(cond, a, b)

    @staticmethod
    def max(x, axis):
        return x.max(dim=axis).values

    @staticmethod
    def minimum(a, b):
        return torch.minimum(a, torch.as_tensor(b, dtype=a.dtype))

    @staticmethod
    def maximum(a, b):
        return torch.maximum(a, torch.as_tensor(b, dtype=a.dtype))

    @staticmethod
    def load(ptr: Ptr, mask=None, other=0.0):
        offs = torch.as_tensor(ptr.offs).long()
        if mask is None:
            mask = torch.ones_like(offs, dtype=torch.bool)
        offs, mask = torch.broadcast_tensors(offs, torch.as_tensor(mask))
        safe = torch.where(mask, offs, torch.zeros_like(offs))
        assert int(safe.min()) >= 0 and int(safe.max()) < ptr.buf.numel()
        vals = _raw(ptr.buf)[safe].view(ptr.buf.dtype)
        if vals.dim() == 0:
            return as_v(vals if bool(mask) else torch.as_tensor(other, dtype=ptr.buf.dtype))
        fill = torch.full_like(vals.float(), other).to(ptr.buf.dtype)
        return as_v(torch.where(mask, _raw(vals), _raw(fill)).view(ptr.buf.dtype))

    @staticmethod
    def store(ptr: Ptr, values, mask=None):
        offs = torch.as_tensor(ptr.offs).long()
        values = torch.as_tensor(values).as_subclass(torch.Tensor)
        if mask is None:
            mask = torch.ones_like(offs, dtype=torch.bool)
        offs, values, mask = torch.broadcast_tensors(offs, values, torch.as_tensor(mask))
        values = values.to(ptr.buf.dtype)
        active = offs[mask]
        assert active.numel() == active.unique().numel(), "conflicting stores"
        assert active.numel() == 0 or (int(active.min()) >= 0 and int(active.max()) < ptr.buf.numel())
        _raw(ptr.buf)[active] = _raw(values.contiguous())[mask]


def _function_source(path: Path, name: str) -> ast.FunctionDef:
    for node in ast.parse(path.read_text()).body:
        if isinstance(node, ast.FunctionDef) and node.name == name:
            return node
    raise SystemExit(f"{name} not found in {path}")


def load_recompute_helper(ref_root: Path):
    path = ref_root / "src/mega_moe/kernels/mega_bwd.py"
    fn = _function_source(path, "_recompute_act_rows")
    fn.decorator_list = []
    scope = {"tl": TL, "range": jit_range}
    exec(compile(ast.Module(body=[fn], type_ignores=[]), str(path), "exec"), scope)
    return scope["_recompute_act_rows"]


def load_save_leg(ref_root: Path):
    """The statement that stores the raw FC1 tile in the configured saved format."""
    path = ref_root / "src/mega_moe/kernels/fused_forward.py"
    fn = _function_source(path, "_partition_pipeline_fc1_activation_group_ub")
    found = [n for n in ast.walk(fn) if isinstance(n, ast.If) and isinstance(n.test, ast.Name)
             and n.test.id == "FC1_SAVE_FP16"]
    if len(found) != 1:
        raise SystemExit("the FC1 save leg was not found exactly once")
    code = compile(ast.Module(body=[found[0]], type_ignores=[]), str(path), "exec")

    def run(scope):
        exec(code, scope)

    return run


def run_save_leg(run, raw: torch.Tensor, ffn: int, group_n: int, fmt: str, block_m: int = 16):
    """Drive the save leg over all (row tile, column group) tiles of raw [rows, 2F] bf16."""
    rows = raw.shape[0]
    dt = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp8": torch.float8_e4m3fn}[fmt]
    out = torch.zeros(rows * 2 * ffn, dtype=torch.float32).to(dt)
    scale = torch.zeros(rows * (2 * ffn // group_n), dtype=torch.float32)
    for row0 in range(0, rows, block_m):
        for col_start in range(0, ffn, group_n):
            local_rows = row0 + torch.arange(block_m)
            cols = col_start + torch.arange(group_n)
            mask_m = local_rows < rows
            mask_n = cols < ffn
            r = local_rows.clamp(max=rows - 1)
            c = cols.clamp(max=ffn - 1)
            gate_raw = as_v(raw[r][:, c])
            up_raw = as_v(raw[r][:, ffn + c])
            scope = dict(
                tl=TL, FC1_SAVE_FP16=fmt == "fp16", FC1_FP8=fmt == "fp8", FFN=ffn,
                gate_raw=gate_raw, up_raw=up_raw, mask_m=mask_m, mask_n=mask_n,
                fc1_store_mask=mask_m[:, None] & mask_n[None, :],
                fc1_row_ptr=Ptr(out) + local_rows[:, None] * (2 * ffn) + cols[None, :],
                fc1_scale_ptr=Ptr(scale), output_group_row=0, pair_block_n=group_n,
                local_row_start=0, local_rows=local_rows, col_start=col_start)
            run(scope)
    return out.view(rows, 2 * ffn), scale.view(rows, 2 * ffn // group_n)


def saved_formats(ref_root: Path):
    run_leg = load_save_leg(ref_root)
    recompute = load_recompute_helper(ref_root)
    g = torch.Generator().manual_seed(11)
    rows, ffn, group_n = 37, 256, 128
    raw = (torch.randn(rows, 2 * ffn, generator=g) * 3.0).to(torch.bfloat16)
    raw[3, :group_n] = 0                       # an all-zero scale group
    raw[5] = 0                                 # an all-zero row
    raw[7, 10] = 3.0e4                         # one large value dominates its group
    weights = torch.rand(rows, generator=g).to(torch.bfloat16)
    res = {"meta": np.array([rows, ffn, group_n], dtype=np.int64), "in_raw": bits(raw),
           "in_weights": bits(weights)}
    saved = {}
    for fmt in ("bf16", "fp16", "fp8"):
        out, scale = run_save_leg(run_leg, raw, ffn, group_n, fmt)
        saved[fmt] = (out, scale)
        res[f"save_{fmt}"] = out.view(torch.uint8).numpy() if fmt == "fp8" else (
            out.view(torch.int16).numpy())
        if fmt == "fp8":
            res["save_fp8_scale"] = scale.numpy()
    acts = {"swiglu": (0, 1.0, None, 7.0), "situglu": (1, 1.5, 2.0, 7.0),
            "situglu_plain_up": (1, 0.75, None, 7.0), "clamp_swiglu": (2, 1.0, None, 0.5)}
    for fmt in ("bf16", "fp8"):
        fc1, scale = saved[fmt]
        for name, (act_id, beta, lbeta, clamp) in acts.items():
            out = torch.zeros(rows * ffn, dtype=torch.bfloat16)
            recompute(
                0, 1, Ptr(fc1.reshape(-1)), 2 * ffn, Ptr(weights), Ptr(out), ffn, ffn, rows,
                beta, 0.0 if lbeta is None else lbeta, clamp,
                BLOCK_SIZE=ffn, ACTIVATION=act_id, HAS_LINEAR_BETA=lbeta is not None,
                fc1_scale_ptr=Ptr(scale.reshape(-1)), FC1_FP8=fmt == "fp8", FC1_GROUP_N=group_n)
            res[f"recompute_{fmt}_{name}"] = bits(out.view(rows, ffn))
    np.savez_compressed(HERE / "saved_formats.npz", **res)
    print("saved_formats.npz", (HERE / "saved_formats.npz").stat().st_size, "bytes")


def saved_tables(ref_root: Path):
    import importlib.util
    tf, _ = load_reference(ref_root)
    spec = importlib.util.spec_from_file_location(
        "mega_moe.ops._moonep_torch_forward", ref_root / "src/mega_moe/ops/_moonep_torch_forward.py")
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
    rng = np.random.default_rng(3)
    res = {}
    cases = [(1, 4), (2, 3), (4, 8), (8, 14)]
    res["cases"] = np.asarray(cases, dtype=np.int64)
    for i, (world, epr) in enumerate(cases):
        counts = rng.integers(0, 200, size=(world, epr))
        counts[rng.random((world, epr)) < 0.2] = 0
        counts_t = torch.as_tensor(counts, dtype=torch.int64)
        per_expert = counts_t.sum(0)
        slot_starts = per_expert.cumsum(0) - per_expert
        perm = mod._arrival_to_slot_permutation(counts_t, slot_starts)
        meta = tf.prepare_moe_metadata(per_expert)
        res[f"c{i}_counts"] = counts.astype(np.int64)
        res[f"c{i}_local_sort_idxs"] = perm.numpy()
        for key, val in zip(("split_size_cum_per_expert", "meta_expert_ids", "meta_split_cum",
                             "meta_tile_num", "meta_tile_num_cum", "num_tiles_total"), meta):
            res[f"c{i}_{key}"] = val.numpy()
    np.savez_compressed(HERE / "saved_tables.npz", **res)
    print("saved_tables.npz", (HERE / "saved_tables.npz").stat().st_size, "bytes")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden_saved.py /path/to/reference")
    root = Path(sys.argv[1])
    saved_tables(root)
    saved_formats(root)
