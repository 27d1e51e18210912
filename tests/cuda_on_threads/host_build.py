"""Compile kernel source for the host against cuda_on_threads.h.  TEST INFRASTRUCTURE ONLY.

``MOE_TEST_SANITIZE=1`` adds ``-fsanitize=address``: run pytest with the AddressSanitizer
runtime preloaded, e.g.

    LD_PRELOAD=$(gcc -print-file-name=libasan.so) ASAN_OPTIONS=detect_leaks=0 \
        MOE_TEST_SANITIZE=1 python -m pytest tests/test_moonep_kernels_on_threads.py

and every load and store of the kernels is bounds-checked against the (heap-allocated) numpy
buffers the tests pass in.
"""
from __future__ import annotations

import os
import re
import shutil
import subprocess
from pathlib import Path

import pytest

HERE = Path(__file__).resolve().parent


def compile_for_host(source: Path, out: Path, include_dirs=()) -> Path:
    if shutil.which("g++") is None:
        pytest.skip("g++ is not installed")
    cmd = ["g++", "-O1", "-std=c++17", "-pthread", "-shared", "-fPIC", "-Wno-unknown-pragmas"]
    if os.environ.get("MOE_TEST_SANITIZE") == "1":
        cmd += ["-fsanitize=address", "-fno-omit-frame-pointer", "-g"]
    for d in (HERE, *include_dirs):
        cmd += ["-I", str(d)]
    cmd += [str(source), "-o", str(out)]
    subprocess.run(cmd, check=True)
    return out


OPERAND = r'"(=?[rl])"\(((?:[^()]|\((?:[^()]|\([^()]*\))*\))*)\)'


def map_ptx(text: str) -> str:
    """Replace each ``asm volatile(...)`` statement of a piece of kernel source by host code of the
    same meaning (loads, release stores, acquire loads, acq_rel adds); fail on any instruction
    that is not known here."""
    out, pos = [], 0
    while True:
        i = text.find("asm volatile(", pos)
        if i < 0:
            out.append(text[pos:])
            return "".join(out)
        j = text.index(");", i) + 2
        stmt = text[i:j]
        instr = re.search(r'"([^"]+)"', stmt).group(1)
        ops = re.findall(OPERAND, stmt[stmt.index(instr) + len(instr):])
        outs = [e for kind, e in ops if kind.startswith("=")]
        ins = [e for kind, e in ops if not kind.startswith("=")]
        if instr.startswith("ld.global.nc") and ".v4.u32" in instr:
            new = ("{ const uint4 t_ = *reinterpret_cast<const uint4*>(%s); %s = t_.x; %s = t_.y; "
                   "%s = t_.z; %s = t_.w; }" % (ins[0], *outs))
        elif instr.startswith("st.release.sys.global.s32"):
            new = "__atomic_store_n((int32_t*)(%s), (int32_t)(%s), __ATOMIC_RELEASE);" % tuple(ins)
        elif instr.startswith("atom.add.acq_rel.gpu.global.s32"):
            new = "%s = __atomic_fetch_add((int32_t*)(%s), 1, __ATOMIC_ACQ_REL);" % (outs[0], ins[0])
        elif instr.startswith("ld.acquire.sys.global.s32"):
            new = "%s = __atomic_load_n((const int32_t*)(%s), __ATOMIC_ACQUIRE);" % (outs[0], ins[0])
        elif instr.startswith("fence.proxy.async"):
            new = ";"
        else:
            raise AssertionError(f"unknown PTX statement: {instr}")
        out.append(text[pos:i] + new)
        pos = j


def cut(text: str, start: str, end: str = "\n}\n") -> str:
    i = text.index(start)
    i = text.rfind("\n", 0, i) + 1
    j = text.index(end, i) + len(end)
    return text[i:j]
