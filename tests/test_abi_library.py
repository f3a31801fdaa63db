"""The C-ABI library loads without a GPU and exports exactly the entry points
that include/xdk_b200.h declares; no compute call is made here."""

from __future__ import annotations

import ctypes
import re

from conftest import ROOT
from cross_dsl_kernels_b200 import _native


def declared_symbols():
    text = (ROOT / "include" / "xdk_b200.h").read_text()
    return sorted(set(re.findall(r"XDK_API[^;(]*?\b(xdk_[a-z0-9_]+)\s*\(", text)))


def test_library_is_built_in_tree():
    assert _native.LIB_PATH.exists(), "run python -m cross_dsl_kernels_b200.build"
    assert _native.LIB_PATH.parent == ROOT / "cross_dsl_kernels_b200"


def test_every_declared_symbol_is_exported_and_bound():
    names = declared_symbols()
    assert len(names) >= 8
    handle = ctypes.CDLL(str(_native.LIB_PATH))
    for name in names:
        assert hasattr(handle, name), f"{name} is declared in the header but not exported"
    assert sorted(_native.SIGNATURES) == names, "ctypes table and header disagree"


def test_status_text_and_version():
    lib = _native.lib()
    assert lib.xdk_abi_version() == 2
    assert lib.xdk_strerror(0) == b"ok"
    for code in (-1, -2, -3, -4, -99):
        assert len(lib.xdk_strerror(code)) > 0


def test_header_is_plain_c_and_a_c_program_links(tmp_path):
    """The boundary is a C ABI: the header must compile as C99 and a C program must link against the library
    and call an entry point that needs no GPU."""
    import shutil
    import subprocess
    if shutil.which("gcc") is None:
        import pytest
        pytest.skip("no C compiler")
    src = tmp_path / "probe.c"
    src.write_text(
        '#include <stdio.h>\n#include <stdint.h>\n#include "xdk_b200.h"\n'
        "int main(void) {\n"
        "  int32_t plan[5];\n"
        "  if (xdk_abi_version() != 2) return 1;\n"
        "  if (xdk_gemv_tc_plan(16, 4096, 14336, 0, plan) != 1) return 2;  /* one CTA per strip at this width */\n"
        '  printf("%s %d %d\\n", xdk_strerror(XDK_OK), (int)plan[0], (int)plan[1]);\n'
        "  return 0;\n}\n")
    exe = tmp_path / "probe"
    lib_dir = _native.LIB_PATH.parent
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", str(ROOT / "include"), str(src), "-o", str(exe),
                    str(_native.LIB_PATH), f"-Wl,-rpath,{lib_dir}"], check=True, capture_output=True)
    done = subprocess.run([str(exe)], capture_output=True, text=True, timeout=60)
    assert done.returncode == 0 and done.stdout.split() == ["ok", "148", "1"], done.stdout + done.stderr
