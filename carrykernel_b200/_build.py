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
# Test-only twin of the library, built with CARRY_TEST_WAIT_EXPIRY: one tile's copies never complete and the
# wait limit is short, so that tests/test_gpu_wait_expiry.py can watch a bounded wait run out; it also
# forces, reports and (with an extra kernel that writes a buffer late) provokes the path of set-up inputs
# that changed under the streaming kernel's feet.  Nothing in the package loads it.
WAIT_TEST_LIB = os.path.join(PKG, "libcarry_gdn_waittest.so")
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
    if not os.path.exists(LIB) or not os.path.exists(WAIT_TEST_LIB):
        return True
    built = min(os.path.getmtime(LIB), os.path.getmtime(WAIT_TEST_LIB))
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

    # the sources whose code differs in the test-only twin (the streaming and multi-token kernels)
    twin_sources = ("carry_gdn_tile128_vk.cu", "carry_gdn_tile128_kv.cu", "carry_gdn_multi.cu")

    def compile_one(job):
        src, twin = job
        obj = os.path.join(obj_dir, src.replace(".cu", ".waittest.o" if twin else ".o"))
        cmd = [nvcc, *NVCC_FLAGS, *(("-DCARRY_TEST_WAIT_EXPIRY",) if twin else ()), "-c", "-o", obj, src]
        proc = subprocess.run(cmd, cwd=CSRC, capture_output=True, text=True)
        return obj, cmd, proc

    jobs = [(s, False) for s in SOURCES] + [(s, True) for s in twin_sources]
    with ThreadPoolExecutor(max_workers=len(jobs)) as pool:
        results = list(pool.map(compile_one, jobs))
    log = []
    failed = False
    for (src, twin), (obj, cmd, proc) in zip(jobs, results):
        if not twin:                                  # the resource report of the shipped library only
            log.append(" ".join(cmd) + "\n" + proc.stdout + proc.stderr)
        elif proc.returncode != 0:
            log.append(" ".join(cmd) + "\n" + proc.stdout + proc.stderr)
        failed = failed or proc.returncode != 0
    if not failed:
        objs = {job: r[0] for job, r in zip(jobs, results)}
        main_objs = [objs[(s, False)] for s in SOURCES]
        twin_objs = [objs[(s, s in twin_sources)] for s in SOURCES]
        for target, members in ((LIB, main_objs), (WAIT_TEST_LIB, twin_objs)):
            link = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", target] + members
            proc = subprocess.run(link, cwd=CSRC, capture_output=True, text=True)
            log.append(" ".join(link) + "\n" + proc.stdout + proc.stderr)
            failed = failed or proc.returncode != 0
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
