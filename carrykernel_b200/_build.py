"""Build ``libcarry_gdn.so`` in-tree with nvcc for sm_100a.

``python -m carrykernel_b200._build`` (or :func:`build`) compiles the
translation units under ``csrc/`` in parallel and links them into
``carrykernel_b200/libcarry_gdn.so``.  nvcc cross-compiles, so this works on a
host without a GPU.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "libcarry_gdn.so")
SOURCES = ("carry_gdn_api.cu", "carry_gdn_generic.cu", "carry_gdn_tile128.cu",
           "carry_gdn_tile128_vk.cu", "carry_gdn_tile128_kv.cu", "carry_gdn_multi.cu",
           "carry_gdn_pool.cu", "carry_gdn_noef128.cu")
HEADERS = ("carry_gdn_common.cuh", "carry_gdn_tile128.cuh", "carry_gdn_slot_tile.inc", os.path.join("..", "..", "include", "carry_gdn.h"))
NVCC_FLAGS = ("-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xptxas", "-v", "-Xcompiler", "-fPIC")


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
    nvcc = _nvcc()
    root = os.path.dirname(PKG)
    obj_dir = os.path.join(root, "build", "obj")
    os.makedirs(obj_dir, exist_ok=True)

    def compile_one(src):
        obj = os.path.join(obj_dir, src.replace(".cu", ".o"))
        cmd = [nvcc, *NVCC_FLAGS, "-c", "-o", obj, src]
        proc = subprocess.run(cmd, cwd=CSRC, capture_output=True, text=True)
        return obj, cmd, proc

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        results = list(pool.map(compile_one, SOURCES))
    log = []
    failed = False
    for obj, cmd, proc in results:
        log.append(" ".join(cmd) + "\n" + proc.stdout + proc.stderr)
        failed = failed or proc.returncode != 0
    if not failed:
        link = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB] + [r[0] for r in results]
        proc = subprocess.run(link, cwd=CSRC, capture_output=True, text=True)
        log.append(" ".join(link) + "\n" + proc.stdout + proc.stderr)
        failed = proc.returncode != 0
    text = "\n".join(log)
    with open(os.path.join(root, "build", "ptxas.log"), "w") as f:
        f.write(text)
    if verbose or failed:
        sys.stderr.write(text)
    if failed:
        raise RuntimeError("nvcc failed; see build/ptxas.log")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
