"""Builds ``libxdk_b200.so`` (the C-ABI library) in-tree with nvcc for sm_100a.

    python -m cross_dsl_kernels_b200.build        # rebuild if any source is newer

No GPU is needed to build: nvcc cross-compiles.  The CUDA runtime is linked
statically, so the library loads on a machine without a GPU (calls then return
an error status) and has no dependency on any Python package.
"""

from __future__ import annotations

import os
import pathlib
import shutil
import subprocess
import sys

PKG = pathlib.Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libxdk_b200.so"
SOURCES = ("abi.cu", "rmsnorm.cu", "gemv.cu", "gemv_tc.cu", "rope_kv.cu", "w4a16.cu", "quantize.cu", "peer.cu", "swiglu.cu", "attention.cu", "unshard.cu")
ARCH_FLAGS = ("-gencode", "arch=compute_100a,code=sm_100a")


def _nvcc() -> str:
    found = shutil.which("nvcc") or os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found (set CUDA_HOME)")
    return found


def needs_build() -> bool:
    if not LIB.exists():
        return True
    stamp = LIB.stat().st_mtime
    deps = [CSRC / s for s in SOURCES] + list(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "xdk_b200.h"]
    return any(d.stat().st_mtime > stamp for d in deps)


def build(force: bool = False, verbose: bool = False) -> pathlib.Path:
    """Compile every kernel translation unit and link the shared library."""
    if not force and not needs_build():
        return LIB
    nvcc = _nvcc()
    objdir = PKG / "build"
    objdir.mkdir(exist_ok=True)
    common = [nvcc, *ARCH_FLAGS, "-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]
    if verbose:
        common += ["-Xptxas", "-v"]
    procs = []
    for src in SOURCES:
        obj = objdir / (src[:-3] + ".o")
        procs.append((src, subprocess.Popen(common + ["-c", str(CSRC / src), "-o", str(obj)],
                                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode:
            sys.stderr.write(f"--- {src}\n{out}\n")
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed; see output above")
    objs = [str(objdir / (s[:-3] + ".o")) for s in SOURCES]
    link = [nvcc, *ARCH_FLAGS, "-shared", "-cudart", "static", "-o", str(LIB), *objs]
    done = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if done.returncode:
        raise RuntimeError("link failed:\n" + done.stdout)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
