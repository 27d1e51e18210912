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
