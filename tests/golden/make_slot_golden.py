"""Record outputs of the reference's own slot-indexed kernel as fixtures.

The slot-indexed step exists in tomalmog/carrykernel only as a Triton kernel
(vllm_integration/quantized_packed_decode.py:101-327), so it needs a GPU.  This
script runs THAT kernel -- from the unmodified copy staged by
``oracle/make_ref.py`` -- on seeded inputs and stores inputs and outputs:

    python oracle/make_ref.py /path/to/carrykernel      # where the checkout is
    python tests/golden/make_slot_golden.py OUTDIR      # on a host with a GPU

writes ``slot_step_<case>.npz`` into OUTDIR (copy them into ``tests/golden/``).
Per case: the pool after one warm-up step of the reference kernel (so the
residual is not zero), the packed activations of the recorded step, and the
pool and ``out`` the reference kernel produced from them.  One more file,
``slot_step_ties.npz``, is the reference's constructed rounding-tie case
(test_quantized_packed_decode.py:211-286).

Nothing here touches the oracle or the product: the fixtures are the
reference kernel's outputs and nothing else.
"""

from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "tests"))
sys.path.insert(0, ROOT)

# name -> (B, H, HV, K, V, resid_fmt, l2norm); slot ids include one padding request
CASES = {
    "k64_int8_l2": (3, 2, 4, 64, 64, 0, True),
    "k64_int4_l2": (3, 2, 4, 64, 64, 1, True),
    "k64_int8_raw": (3, 2, 4, 64, 64, 0, False),
    "k128_int8_l2": (3, 1, 2, 128, 128, 0, True),
    "k128_int4_l2": (3, 1, 2, 128, 128, 1, True),
    "k128_int4_raw": (3, 1, 2, 128, 128, 1, False),
}
SLOTS = (3, 0, 1)          # request 1 is padding
NUM_SLOTS = 4


def case_inputs(name, step):
    """Seeded pool seed and activations of a case (CPU tensors); step 0 warms up, step 1 is recorded."""
    from parity import make_packed_inputs
    B, H, HV, K, V, fmt, l2 = CASES[name]
    seed = 1000 + 17 * sorted(CASES).index(name)
    g = torch.Generator().manual_seed(seed)
    pool = torch.randn(NUM_SLOTS, HV, V, K, generator=g) * 0.1
    acts = make_packed_inputs(B, H, HV, K, V, seed=seed + 1 + step, qk_gain=1.0 if l2 else K ** -0.5)
    return pool, acts


def main(outdir):
    from oracle import make_ref
    ref = make_ref.ref_path()
    if ref is None:
        sys.exit("oracle/_ref is not staged: run oracle/make_ref.py first")
    sys.path.insert(0, ref)
    from vllm_integration import quantized_packed_decode as rqpd
    dev = "cuda"
    os.makedirs(outdir, exist_ok=True)
    idx = torch.tensor(SLOTS, dtype=torch.int32)
    for name, (B, H, HV, K, V, fmt, l2) in CASES.items():
        pool, _ = case_inputs(name, 0)
        st = list(rqpd.init_quantized_state(NUM_SLOTS, HV, V, K, dev, h0=pool.to(dev), resid_fmt=fmt))
        rec = {}
        for step in (0, 1):
            _, acts = case_inputs(name, step)
            mixed, a, b, A_log, dt_bias = [x.to(dev) for x in acts]
            if step == 1:
                for key, t in zip(("in_sc", "in_ss", "in_rc", "in_rs"), st):
                    rec[key] = t.cpu().numpy().copy()
            out = torch.full((B, 1, HV, V), float("nan"), device=dev)
            rqpd.quantized_gated_delta_rule_packed_decode(
                mixed, a, b, A_log, dt_bias, K ** -0.5, *st, out, idx.to(dev),
                use_qk_l2norm_in_kernel=l2, resid_fmt=fmt)
            torch.cuda.synchronize()
        for key, t in zip(("out_sc", "out_ss", "out_rc", "out_rs"), st):
            rec[key] = t.cpu().numpy()
        rec["out"] = out.cpu().numpy()
        for key, t in zip(("mixed", "a", "b", "A_log", "dt_bias"), acts):
            rec[key] = t.numpy()
        rec["slots"] = idx.numpy()
        path = os.path.join(outdir, f"slot_step_{name}.npz")
        np.savez_compressed(path, **rec)
        print(f"  {os.path.basename(path)}  {os.path.getsize(path) / 1024:.1f} KiB")

    # rounding ties: residual codes at scale 0.5 are exact half-integers, one state entry pins the row
    # maximum at 127 so that the derived scale is exactly 1 (the recurrence is switched off by the gates)
    H, HV, K, V = 1, 1, 32, 4
    odd = (torch.arange(K, dtype=torch.float32) % 8) * 2 - 7
    resid_in = odd[None, None, :].repeat(HV, V, 1).contiguous()
    resid_in[..., 0] = 0.0
    state_in = torch.zeros(HV, V, K)
    state_in[..., 0] = 1.0
    sc = torch.zeros(2, HV, V, K, dtype=torch.int8, device=dev)
    ss = torch.zeros(2, HV, V, device=dev)
    rc = torch.zeros(2, HV, V, K, dtype=torch.int8, device=dev)
    rs = torch.zeros(2, HV, V, device=dev)
    sc[1] = state_in.to(torch.int8); ss[1] = 127.0; rc[1] = resid_in.to(torch.int8); rs[1] = 0.5
    rec = {"in_sc": sc.cpu().numpy().copy(), "in_ss": ss.cpu().numpy().copy(),
           "in_rc": rc.cpu().numpy().copy(), "in_rs": rs.cpu().numpy().copy()}
    out = torch.empty(1, 1, HV, V, device=dev)
    rqpd.quantized_gated_delta_rule_packed_decode(
        torch.zeros(1, 2 * H * K + HV * V, device=dev), torch.full((1, HV), -60.0, device=dev),
        torch.full((1, HV), -60.0, device=dev), torch.zeros(HV, device=dev), torch.zeros(HV, device=dev),
        K ** -0.5, sc, ss, rc, rs, out, torch.tensor([1], dtype=torch.int32, device=dev))
    torch.cuda.synchronize()
    rec.update(out_sc=sc.cpu().numpy(), out_ss=ss.cpu().numpy(), out_rc=rc.cpu().numpy(),
               out_rs=rs.cpu().numpy(), out=out.cpu().numpy())
    np.savez_compressed(os.path.join(outdir, "slot_step_ties.npz"), **rec)
    print("  slot_step_ties.npz")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    main(sys.argv[1])
