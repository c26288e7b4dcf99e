"""Time of the pool store / load / copy kernels.

    python -m carrykernel_b200.vllm_integration.state_pool_timing [--batches 64 256] [--layers 8]

H = HV = 32, K = V = 128, int8 state + packed int4 residual with one scale per
head.  Each call moves ``B`` requests; ``layers`` pools are cycled so that the
bytes of one pass exceed the L2, ten passes are captured into one CUDA graph
and timed with CUDA events.  Bytes per (request, head): store reads the
floating-point state and writes codes, residual and scales; load the reverse;
copy reads and writes the quantized slot.  Prints one JSON object.
"""

from __future__ import annotations

import argparse
import json

import torch

from . import quantized_packed_decode as qpd
from . import state_pool as sp

HV = 32
K = V = 128


def _time(fn, reps=10):
    for _ in range(3):
        fn()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(reps):
            fn()
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    graph.replay()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (2 * reps)


def run(batches=(64, 256), layers=8, seed=0):
    dev = torch.device("cuda")
    torch.manual_seed(seed)
    res = {"HV": HV, "K": K, "V": V, "layers": layers, "gpu": torch.cuda.get_device_name(0)}
    slot_bytes = qpd.state_bytes_per_slot(HV, V, K, True, resid_fmt=qpd.RESID_INT4, resid_scale="head")
    for B in batches:
        slots = 2 * B + 1
        pools = [qpd.init_quantized_state(slots, HV, V, K, dev, resid_fmt=qpd.RESID_INT4, resid_scale="head")
                 for _ in range(layers)]
        idx = (torch.randperm(B, device=dev) + 1).to(torch.int32)
        idx2 = idx + B
        row = {}
        for name, dtype, es in (("fp32", torch.float32, 4), ("bf16", torch.bfloat16, 2)):
            hs = [(torch.randn(B, HV, V, K, device=dev) * 0.1).to(dtype) for _ in range(layers)]

            def store(keep):
                for h, pool in zip(hs, pools):
                    sp.store_state(h, pool, idx, resid_fmt=qpd.RESID_INT4, keep_error=keep)

            def load():
                for h, pool in zip(hs, pools):
                    sp.load_state(pool, idx, out=h, resid_fmt=qpd.RESID_INT4)

            bytes_call = B * (HV * V * K * es + slot_bytes)
            for label, fn in ((f"store_{name}", lambda: store(False)),
                              (f"store_{name}_keep_error", lambda: store(True)),
                              (f"load_{name}", load)):
                us = _time(fn) / layers
                row[label] = {"us_per_call": us, "GB_per_s": bytes_call / us / 1e3}
            del hs

        def copy():
            for pool in pools:
                sp.copy_slots(pool, idx, idx2, resid_fmt=qpd.RESID_INT4)

        us = _time(copy) / layers
        row["copy"] = {"us_per_call": us, "GB_per_s": 2 * B * slot_bytes / us / 1e3}
        res[f"B{B}"] = row
    return res


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--batches", type=int, nargs="+", default=[64, 256])
    ap.add_argument("--layers", type=int, default=8)
    args = ap.parse_args()
    print(json.dumps(run(tuple(args.batches), args.layers)))


if __name__ == "__main__":
    main()
