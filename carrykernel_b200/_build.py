"""Build ``libcarry_gdn.so`` in-tree with nvcc for sm_100a.

``python -m carrykernel_b200._build`` (or :func:`build`) compiles the three
translation units under ``csrc/`` into ``carrykernel_b200/libcarry_gdn.so``.
nvcc cross-compiles, so this works on a host without a GPU.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "libcarry_gdn.so")
SOURCES = ("carry_gdn_api.cu", "carry_gdn_generic.cu", "carry_gdn_tile128.cu")
HEADERS = ("carry_gdn_common.cuh", os.path.join("..", "..", "include", "carry_gdn.h"))
NVCC_FLAGS = ("-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xptxas", "-v", "-shared", "-Xcompiler", "-fPIC")


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found (set NVCC or put it on PATH)")


def is_stale() -> bool:
    if not os.path.exists(LIB):
        return True
    built = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS]
    return any(os.path.getmtime(d) > built for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if it is missing or older than its sources.
    Returns the path of the shared object; raises on compiler failure.  The
    ptxas resource report (registers, spills) goes to ``build/ptxas.log``."""
    if not force and not is_stale():
        return LIB
    cmd = [_nvcc(), *NVCC_FLAGS, "-o", LIB, *SOURCES]
    proc = subprocess.run(cmd, cwd=CSRC, capture_output=True, text=True)
    log_dir = os.path.join(os.path.dirname(PKG), "build")
    os.makedirs(log_dir, exist_ok=True)
    with open(os.path.join(log_dir, "ptxas.log"), "w") as f:
        f.write(" ".join(cmd) + "\n" + proc.stdout + proc.stderr)
    if verbose or proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed with exit code {proc.returncode}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
