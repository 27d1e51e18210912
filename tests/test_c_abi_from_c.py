"""The public header is plain C and the library links from C: gcc -std=c99 -pedantic -Werror
compiles a caller that takes the address of every function the header declares and runs the
host planner (an entry point that needs no GPU).  This is what a cgo / JNI / FFI binding of the
boundary relies on."""

from __future__ import annotations

import re
import shutil
import subprocess
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent
HEADER = REPO / "include" / "mega_moe_b200.h"
LIB_DIR = REPO / "mega-moe-td_b200" / "lib"


def declared_functions() -> list[str]:
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(mm_[a-z0-9_]+)\s*\(", text)))


def test_header_compiles_as_c99_and_links(tmp_path):
    if shutil.which("gcc") is None:
        pytest.skip("gcc is not installed")
    if not (LIB_DIR / "libmegamoe_sm100.so").exists():
        pytest.skip("the library has not been built")
    names = declared_functions()
    assert len(names) >= 30 and "mm_route_finalize" in names and "mm_moonep_plan_host" in names
    # a function pointer is not a void* in ISO C; go through an integer type
    listing = ", ".join(f"(const void*)(size_t)&{n}" for n in names)
    exe = tmp_path / "use_from_c"
    cmd = ["gcc", "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror",
           f"-DALL_ENTRY_POINTS={listing}", "-I", str(REPO / "include"),
           str(REPO / "tests" / "c_abi" / "use_from_c.c"), "-L", str(LIB_DIR), "-lmegamoe_sm100",
           f"-Wl,-rpath,{LIB_DIR}", "-o", str(exe)]
    subprocess.run(cmd, check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout
    assert out.strip() == (f"abi=3 entry_points={len(names)} rc=0 prefix=4,8 copy=0 reason=0 "
                           "record=0 table=0")
