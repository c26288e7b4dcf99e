"""Stage an unmodified copy of the reference's code for this path under ``oracle/_ref/``.

TEST INFRASTRUCTURE ONLY.  ``oracle/_ref/`` is listed in ``.gitignore``: the
copy never enters this repository's history, it only travels to the GPU host
next to the built library so that

  * ``tests/test_gpu_reference_pin.py`` can run the reference's own Triton
    kernel for the slot-indexed step (vllm_integration/quantized_packed_decode.py:101-327
    of tomalmog/carrykernel) on the same seeded inputs as the CPU oracle,
  * ``tests/golden/make_slot_golden.py`` can record that kernel's outputs as
    fixtures, and
  * ``bench.py --impl reference`` can time the reference's own CPU step
    (statequant/kernel.py:149-178).

Nothing under ``carrykernel_b200/`` imports it.

    python oracle/make_ref.py [/path/to/carrykernel]

The files are copied byte for byte; ``MANIFEST.json`` records their SHA-256 so
a test can tell that the staged copy is the one the fixtures were made with.
"""

from __future__ import annotations

import hashlib
import json
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
FILES = (
    "statequant/reference.py",
    "statequant/quant.py",
    "statequant/kernel.py",
    "vllm_integration/__init__.py",
    "vllm_integration/quantized_packed_decode.py",
    "vllm_integration/test_quantized_packed_decode.py",
)


def default_source():
    for cand in (os.environ.get("CARRYKERNEL_REFERENCE"),
                 os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")):
        if cand and os.path.isfile(os.path.join(cand, "statequant", "kernel.py")):
            return cand
    return None


def stage(src_root: str | None = None, quiet: bool = False) -> str | None:
    """Copy the listed files; returns the destination, or None when no
    checkout of the reference is reachable (then an earlier copy, if any, is
    left as it is)."""
    src_root = src_root or default_source()
    if src_root is None:
        return DEST if os.path.isfile(os.path.join(DEST, "MANIFEST.json")) else None
    manifest = {}
    for rel in FILES:
        src = os.path.join(src_root, rel)
        dst = os.path.join(DEST, rel)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        shutil.copyfile(src, dst)
        manifest[rel] = hashlib.sha256(open(dst, "rb").read()).hexdigest()
    # statequant/ has no __init__.py upstream (implicit namespace package): none is added
    with open(os.path.join(DEST, "MANIFEST.json"), "w") as f:
        json.dump(manifest, f, indent=1, sort_keys=True)
    if not quiet:
        print(f"staged {len(FILES)} reference files under {DEST}")
    return DEST


def ref_path() -> str | None:
    """Directory to put on ``sys.path`` to import the staged reference, or None."""
    return DEST if os.path.isfile(os.path.join(DEST, "MANIFEST.json")) else None


if __name__ == "__main__":
    out = stage(sys.argv[1] if len(sys.argv) > 1 else None)
    if out is None:
        sys.exit("no reference checkout found (pass its path or set CARRYKERNEL_REFERENCE)")
