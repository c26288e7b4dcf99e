"""Head-to-head timing against vLLM's own packed-decode kernel.

    python -m carrykernel_b200.vllm_integration.headtohead [--batches 1 8 16 64] [--steps 200]

Same comparison as carrykernel's ``modal_vllm_headtohead.py:105-205``: vLLM's
``fused_recurrent_gated_delta_rule_packed_decode`` with an fp32 and with a bf16
state (its serving default) against this library's int8-state step with an
int8 and with a packed int4 residual, Qwen-GDN shapes (H = 16 key heads,
HV = 32 value heads, K = V = 128), every tensor cast once outside the timed
region, CUDA events around ``steps`` calls after ``warmup``.  vLLM's kernel is
only a timing comparator here (library code); nothing of it is used by the
product.  Prints one JSON object.

The working sets of these batch sizes fit the 126 MB L2, so these are
L2-resident, launch-latency-dominated numbers, like the reference's own table.
"""

from __future__ import annotations

import argparse
import json

import torch

from . import quantized_packed_decode as qpd

H, HV, K, V = 16, 32, 128, 128


def _time(call, steps, warmup):
    for _ in range(warmup):
        call()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(steps):
        call()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / steps * 1e3          # us per call


def run(batches=(1, 8, 16, 64), steps=200, warmup=50, seed=0):
    try:
        from vllm.model_executor.layers.fla.ops.fused_recurrent import (
            fused_recurrent_gated_delta_rule_packed_decode as vllm_fn)
    except Exception as exc:                           # pragma: no cover - depends on the image
        vllm_fn, why = None, f"{type(exc).__name__}: {exc}"
    dev = torch.device("cuda")
    torch.manual_seed(seed)
    results = {"H": H, "HV": HV, "K": K, "V": V, "steps": steps, "warmup": warmup,
               "gpu": torch.cuda.get_device_name(0)}
    if vllm_fn is None:
        results["vllm"] = f"unavailable: {why}"
    for B in batches:
        mixed = torch.randn(B, 2 * H * K + HV * V, device=dev)
        a = torch.randn(B, HV, device=dev) * 0.5
        b = torch.randn(B, HV, device=dev)
        A_log = torch.randn(HV, device=dev) * 0.2
        dt_bias = torch.randn(HV, device=dev) * 0.1
        scale = K ** -0.5
        idx = torch.arange(1, B + 1, dtype=torch.int32, device=dev)
        h0 = torch.randn(B + 1, HV, V, K, device=dev) * 0.1
        row = {}
        mixed_bf, a_bf, b_bf = mixed.bfloat16(), a.bfloat16(), b.bfloat16()
        if vllm_fn is not None:
            for name, state, mx, aa, bb, out_dt in (
                    ("vllm_fp32_state", h0.clone(), mixed, a, b, torch.float32),
                    ("vllm_bf16_state", h0.bfloat16(), mixed_bf, a_bf, b_bf, torch.bfloat16)):
                out = torch.empty(B, 1, HV, V, device=dev, dtype=out_dt)
                A_, d_ = (A_log, dt_bias) if out_dt == torch.float32 else (A_log.bfloat16(), dt_bias.bfloat16())
                call = lambda state=state, mx=mx, aa=aa, bb=bb, out=out, A_=A_, d_=d_: vllm_fn(
                    mixed_qkv=mx, a=aa, b=bb, A_log=A_, dt_bias=d_, scale=scale, initial_state=state,
                    out=out, ssm_state_indices=idx, use_qk_l2norm_in_kernel=True)
                try:
                    row[name + "_us"] = _time(call, steps, warmup)
                except Exception as exc:              # pragma: no cover
                    row[name + "_us"] = None
                    row[name + "_error"] = f"{type(exc).__name__}: {exc}"[:200]
        out = torch.empty(B, 1, HV, V, device=dev, dtype=torch.bfloat16)
        for fmt, name in ((qpd.RESID_INT8, "ours_int8_resid"), (qpd.RESID_INT4, "ours_int4_resid")):
            for rscale in ("v", "head"):
                st = qpd.init_quantized_state(B + 1, HV, V, K, dev, h0=h0, resid_fmt=fmt, resid_scale=rscale)
                call = lambda st=st, fmt=fmt: qpd.quantized_gated_delta_rule_packed_decode(
                    mixed_bf, a_bf, b_bf, A_log, dt_bias, scale, *st, out, idx,
                    use_qk_l2norm_in_kernel=True, resid_fmt=fmt)
                row[f"{name}_{rscale}_us"] = _time(call, steps, warmup)
        elems = B * HV * V * K
        row["state_traffic_MB"] = {
            "vllm_fp32": 2 * elems * 4 / 1e6, "vllm_bf16": 2 * elems * 2 / 1e6,
            "ours_int8_resid": (4 * elems + 4 * B * HV * V * 4) / 1e6,
            "ours_int4_resid": (3 * elems + 4 * B * HV * V * 4) / 1e6}
        results[f"B{B}"] = row
    return results


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--batches", type=int, nargs="+", default=[1, 8, 16, 64])
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=50)
    args = ap.parse_args()
    print(json.dumps(run(tuple(args.batches), args.steps, args.warmup)))


if __name__ == "__main__":
    main()
