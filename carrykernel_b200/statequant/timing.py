"""Time of one fused step through the statequant op, per residual format.

    python -m carrykernel_b200.statequant.timing [--batches 8 64 256]

``gdn_quant_step_fused`` (``[B, HV, K, V]`` layout, HV = 32, K = V = 128, fp32
q/k/v, 8-bit state) for every residual format and both residual-scale
granularities, and ``gdn_step_fused_fp32`` (the unquantised step), CUDA events around 50 calls after 3 warm-up calls.  The figure
includes the op's own work per call (five output allocations, the ctypes
call), which is what dominates at 8 requests.  Prints one JSON object.
"""

from __future__ import annotations

import argparse
import json

import torch

from . import kernel as sq

HV, K, V = 32, 128, 128
CASES = ((sq.RES_FP32, "v", "fp32"), (sq.RES_FP16, "v", "fp16"), (sq.RES_FP8, "v", "fp8_e5m2"),
         (sq.RES_INT8, "v", "int8_per_v"), (sq.RES_INT8, "head", "int8_per_head"),
         (sq.RES_INT4, "v", "int4_per_v"), (sq.RES_INT4, "head", "int4_per_head"))
RESID_BYTES = {sq.RES_FP32: 4, sq.RES_FP16: 2, sq.RES_FP8: 1, sq.RES_INT8: 1, sq.RES_INT4: 0.5}


def run(batches=(8, 64, 256), calls=50):
    dev = torch.device("cuda")
    res = {"HV": HV, "K": K, "V": V, "gpu": torch.cuda.get_device_name(0)}
    for B in batches:
        row = {}
        for res_fmt, rs, name in CASES:
            g = torch.Generator().manual_seed(0)
            h0 = (torch.randn(B, HV, K, V, generator=g) * 0.12).to(dev)
            st = sq.init_quant_state(h0, 8, res_fmt, resid_scale=rs)
            q = torch.randn(B, HV, K, generator=g).to(dev)
            k = (torch.randn(B, HV, K, generator=g) * K ** -0.5).to(dev)
            v = torch.randn(B, HV, V, generator=g).to(dev)
            alpha = torch.full((B, HV), 0.98, device=dev)
            beta = torch.rand(B, HV, generator=g).to(dev)
            call = lambda: sq.gdn_quant_step_fused(*st, q, k, v, alpha, beta, 8, res_fmt, resid_scale=rs)
            for _ in range(3):
                call()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(calls):
                call()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / calls
            state_bytes = B * HV * K * V * 2 * (1 + RESID_BYTES[res_fmt])      # codes + residual, read and written
            row[name] = {"us_per_step": us, "state_GBps": state_bytes / us / 1e3}
        # no error feedback: codes read and written once, one state scale per V column or per head
        for mode in ("v", "head"):
            g = torch.Generator().manual_seed(0)
            h0 = (torch.randn(B, HV, K, V, generator=g) * 0.12).to(dev)
            st = sq.init_quant_state(h0, 8, sq.RES_NONE, state_scale=mode)
            q = torch.randn(B, HV, K, generator=g).to(dev)
            k = (torch.randn(B, HV, K, generator=g) * K ** -0.5).to(dev)
            v = torch.randn(B, HV, V, generator=g).to(dev)
            alpha = torch.full((B, HV), 0.98, device=dev)
            beta = torch.rand(B, HV, generator=g).to(dev)
            call = lambda: sq.gdn_quant_step_fused(*st, q, k, v, alpha, beta, 8, sq.RES_NONE, state_scale=mode)
            for _ in range(3):
                call()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(calls):
                call()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / calls
            row[f"no_feedback_scale_per_{mode}"] = {"us_per_step": us, "state_GBps": B * HV * K * V * 2 / us / 1e3}
        # the unquantised arm: fp32 state read and written once
        g = torch.Generator().manual_seed(0)
        h = (torch.randn(B, HV, K, V, generator=g) * 0.12).to(dev)
        q = torch.randn(B, HV, K, generator=g).to(dev)
        k = (torch.randn(B, HV, K, generator=g) * K ** -0.5).to(dev)
        v = torch.randn(B, HV, V, generator=g).to(dev)
        alpha = torch.full((B, HV), 0.98, device=dev)
        beta = torch.rand(B, HV, generator=g).to(dev)
        call = lambda: sq.gdn_step_fused_fp32(h, q, k, v, alpha, beta)
        for _ in range(3):
            call()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(calls):
            call()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / calls
        row["fp32_state_unquantised"] = {"us_per_step": us, "state_GBps": B * HV * K * V * 8 / us / 1e3}
        res[f"B{B}"] = row
    return res


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--batches", type=int, nargs="+", default=[8, 64, 256])
    args = ap.parse_args()
    print(json.dumps(run(tuple(args.batches))))


if __name__ == "__main__":
    main()
