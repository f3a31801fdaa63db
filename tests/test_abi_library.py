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
    assert lib.xdk_abi_version() == 1
    assert lib.xdk_strerror(0) == b"ok"
    for code in (-1, -2, -3, -4, -99):
        assert len(lib.xdk_strerror(code)) > 0
