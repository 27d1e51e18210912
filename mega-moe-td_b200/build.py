"""Build libmegamoe_sm100.so in-tree with nvcc for sm_100a.

Usage: ``python mega-moe-td_b200/build.py [--force] [--verbose] [--profile]``.  The shared
library lands in ``mega-moe-td_b200/lib/`` next to the sources, so a copy of the repository
carries it.  ``--profile`` builds a second, instrumented library
(``libmegamoe_sm100_prof.so``, ``-DMM_PROFILE``) whose GEMM kernels also count the clocks each
warp role spends in its waits; the package loads it instead of the plain one when
``MOE_FWD_TIMING=1`` is set, and ``FusedMoEForward.read_last_forward_phase_timing()`` returns
the counters (``python -m mega_moe.phase_timing`` prints them).
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB_DIR = ROOT / "lib"
LIB_PATH = LIB_DIR / "libmegamoe_sm100.so"
PROFILE_LIB_PATH = LIB_DIR / "libmegamoe_sm100_prof.so"
SOURCES = ["abi.cu", "routing.cu", "movement.cu", "gemm_host.cu", "moonep.cu"]
HEADERS = (sorted(p.name for p in CSRC.glob("*.cuh")) + sorted(p.name for p in CSRC.glob("*.h"))
           + ["../../include/mega_moe_b200.h"])

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cand = Path(cuda_home) / "bin" / "nvcc"
    return str(cand) if cand.exists() else "nvcc"


def _stale(out: Path, deps: list[Path]) -> bool:
    if not out.exists():
        return True
    t = out.stat().st_mtime
    return any(d.exists() and d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False, profile: bool = False) -> Path:
    LIB_DIR.mkdir(exist_ok=True)
    obj_dir = ROOT / ("build_prof" if profile else "build")
    obj_dir.mkdir(exist_ok=True)
    lib_path = PROFILE_LIB_PATH if profile else LIB_PATH
    flags = NVCC_FLAGS + (["-DMM_PROFILE"] if profile else [])
    headers = [CSRC / h for h in HEADERS]
    sources = [s for s in SOURCES if (CSRC / s).exists()]
    objs = []
    procs = []
    for s in sources:
        src = CSRC / s
        obj = obj_dir / (src.stem + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + headers):
            cmd = [_nvcc(), *flags, "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas")
                cmd.insert(2, "-v")
            procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                                              text=True)))
    failed = False
    for name, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write(f"--- nvcc {name} ---\n{out}\n")
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed; see the compiler output above")
    if force or procs or _stale(lib_path, objs):
        cmd = [_nvcc(), "-shared", "-o", str(lib_path), *map(str, objs), "-lcudart"]
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}")
    return lib_path


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv,
                 profile="--profile" in sys.argv)
    print(path)
