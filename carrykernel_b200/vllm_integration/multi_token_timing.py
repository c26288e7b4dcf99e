"""Time per token of the multi-token call against single-token calls.

    python -m carrykernel_b200.vllm_integration.multi_token_timing [--batches 64 256] [--tokens 2 4 8]

Slot-indexed path, H = HV = 32, K = V = 128, int8 state + packed int4 residual
with one scale per head, bf16 activations.  For every (batch, T): T
single-token calls (``quantized_gated_delta_rule_packed_decode``) and one
multi-token call (``quantized_gated_delta_rule_packed_decode_multi``), each
captured ten times into a CUDA graph and timed with CUDA events.  Prints one
JSON object.  The working sets fit the L2 at the smaller batch.
"""

from __future__ import annotations

import argparse
import json
import math

import torch

from . import quantized_packed_decode as qpd

H = HV = 32
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


def run(batches=(64, 256), tokens=(2, 4, 8), seed=0):
    dev = torch.device("cuda")
    res = {"H": H, "HV": HV, "K": K, "V": V, "gpu": torch.cuda.get_device_name(0)}
    for B in batches:
        for T in tokens:
            g = torch.Generator().manual_seed(seed)
            slots = B + 1
            pool = torch.randn(slots, HV, V, K, generator=g) * 0.12
            st = [x.to(dev) for x in qpd.init_quantized_state(slots, HV, V, K, "cpu", h0=pool,
                                                              resid_fmt=qpd.RESID_INT4, resid_scale="head")]
            mixed = torch.randn(B, T, 2 * H * K + HV * V, generator=g).to(torch.bfloat16).to(dev)
            a = torch.randn(B, T, HV, generator=g).to(torch.bfloat16).to(dev)
            b = torch.randn(B, T, HV, generator=g).to(torch.bfloat16).to(dev)
            A_log = torch.full((HV,), math.log(0.1), device=dev)
            dt_bias = torch.zeros(HV, device=dev)
            idx = (torch.randperm(slots - 1, generator=g)[:B] + 1).to(torch.int32).to(dev)
            out = torch.empty(B, T, HV, V, dtype=torch.bfloat16, device=dev)
            tmp = torch.empty(B, 1, HV, V, dtype=torch.bfloat16, device=dev)
            per_tok = [(mixed[:, t].contiguous(), a[:, t].contiguous(), b[:, t].contiguous()) for t in range(T)]

            def single():
                for m_, a_, b_ in per_tok:
                    qpd.quantized_gated_delta_rule_packed_decode(m_, a_, b_, A_log, dt_bias, K ** -0.5, *st, tmp, idx,
                                                                 use_qk_l2norm_in_kernel=True, resid_fmt=qpd.RESID_INT4)

            def multi():
                qpd.quantized_gated_delta_rule_packed_decode_multi(mixed, a, b, A_log, dt_bias, K ** -0.5, *st, out, idx,
                                                                   use_qk_l2norm_in_kernel=True, resid_fmt=qpd.RESID_INT4)

            res[f"B{B}_T{T}"] = {"single_token_calls_us_per_token": _time(single) / T,
                                 "multi_token_call_us_per_token": _time(multi) / T}
    return res


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--batches", type=int, nargs="+", default=[64, 256])
    ap.add_argument("--tokens", type=int, nargs="+", default=[2, 4, 8])
    args = ap.parse_args()
    print(json.dumps(run(tuple(args.batches), tuple(args.tokens))))


if __name__ == "__main__":
    main()
