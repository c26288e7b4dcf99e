"""Bit-width and granularity sweep of the quantized recurrent state, on the GPU.

    python -m carrykernel_b200.statequant.granularity_sweep [--batch 256] [--steps 512] [--bits 3 4 5 6 8]

The experiment of carrykernel's ``experiments/exp2_bits_sweep.py`` and
``experiments/exp2b_granularity.py`` at serving size: B requests x 32 heads of
128 x 128 state, T chained decode steps, per-head constant decay drawn from
U[0.9, 0.999], seeded synthetic q, k (L2-normalised), v, beta = sigmoid(N(0,1)).
For every bit width two arms are run through the library's own calls and the
final dequantised state is compared with the fp32 recurrence
(``gdn_step_fused_fp32``) by relative L2 norm:

* ``uniform_no_ef``  one scale per head, no error feedback
  (``uniform_quantize`` semantics, ``statequant/quant.py:23-34``);
* ``per_v_ef``       one scale per V column with an fp32 error-feedback
  residual (``per_axis_quantize(.., -2)`` + ``ErrorFeedback``,
  ``statequant/quant.py:37-42,65-80``).

Inputs are generated on the device step by step (a fixed seed per step), so the
sweep needs no T-sized buffers.  Prints one JSON object with the errors and
the time per step of each arm.
"""

from __future__ import annotations

import argparse
import json

import torch

from . import kernel as sq

HV, K, V = 32, 128, 128


def _step_inputs(B, t, dev, seed):
    g = torch.Generator(device=dev).manual_seed(seed * 100003 + t)
    q = torch.randn(B, HV, K, generator=g, device=dev)
    k = torch.nn.functional.normalize(torch.randn(B, HV, K, generator=g, device=dev), dim=-1)
    v = torch.randn(B, HV, V, generator=g, device=dev)
    beta = torch.sigmoid(torch.randn(B, HV, generator=g, device=dev))
    return q, k, v, beta


def run(batch=256, steps=512, bits=(3, 4, 5, 6, 8), seed=0):
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(seed)
    h0 = torch.randn(batch, HV, K, V, generator=g, device=dev) * 0.1
    alpha = 0.9 + 0.099 * torch.rand(batch, HV, generator=g, device=dev)

    def timed(fn):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = fn()
        e1.record()
        torch.cuda.synchronize()
        return out, e0.elapsed_time(e1) * 1e3 / steps

    def fp32_chain():
        h = h0.clone()
        for t in range(steps):
            q, k, v, beta = _step_inputs(batch, t, dev, seed)
            h, _ = sq.gdn_step_fused_fp32(h, q, k, v, alpha, beta)
        return h

    def quant_chain(nbits, res_fmt, state_scale):
        st = sq.init_quant_state(h0, nbits, res_fmt, state_scale=state_scale)
        for t in range(steps):
            q, k, v, beta = _step_inputs(batch, t, dev, seed)
            out = sq.gdn_quant_step_fused(*st, q, k, v, alpha, beta, bits=nbits, res_fmt=res_fmt,
                                          state_scale=state_scale)
            st = out[1:]
        codes, scale = st[0], st[1]
        return codes.float() * (scale[..., None, :] if state_scale == "v" else scale[..., None, None])

    h_ref, us_ref = timed(fp32_chain)
    norm = h_ref.norm()
    res = {"batch": batch, "steps": steps, "HV": HV, "K": K, "V": V, "gpu": torch.cuda.get_device_name(0),
           "fp32_us_per_step": us_ref, "bits": {}}
    for nbits in bits:
        uni, us_u = timed(lambda: quant_chain(nbits, sq.RES_NONE, "head"))
        err_u = ((uni - h_ref).norm() / norm).item()
        del uni
        ef, us_e = timed(lambda: quant_chain(nbits, sq.RES_FP32, "v"))
        err_e = ((ef - h_ref).norm() / norm).item()
        del ef
        res["bits"][str(nbits)] = {"uniform_no_ef": err_u, "per_v_ef": err_e,
                                   "uniform_no_ef_us_per_step": us_u, "per_v_ef_us_per_step": us_e}
    return res


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--steps", type=int, default=512)
    ap.add_argument("--bits", type=int, nargs="+", default=[3, 4, 5, 6, 8])
    args = ap.parse_args()
    print(json.dumps(run(args.batch, args.steps, tuple(args.bits))))


if __name__ == "__main__":
    main()
