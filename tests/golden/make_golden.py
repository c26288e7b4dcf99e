"""Generate the golden vectors in this folder by RUNNING the reference.

Usage (only where a checkout of tomalmog/carrykernel is available):

    python tests/golden/make_golden.py /path/to/carrykernel            # every fixture
    python tests/golden/make_golden.py /path/to/carrykernel config1    # only the full-size config-1 run

It imports the reference's own CPU code (statequant/reference.py,
statequant/quant.py, statequant/kernel.py, the helper oracle in
vllm_integration/test_quantized_packed_decode.py, and the quantizers at the top
of modal_residual.py), feeds it seeded inputs, and stores inputs and outputs as
small ``.npz`` files.  The committed files are what the tests read; the
reference itself is not needed to run the tests.

Nothing here touches the oracle or the product: the fixtures are the
reference's outputs and nothing else.
"""

from __future__ import annotations

import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _np(t):
    if t is None:
        return None
    if t.dtype == torch.float8_e5m2:
        return t.view(torch.uint8).numpy()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy()
    return t.numpy()


def save(name, **arrays):
    arrays = {k: (_np(v) if torch.is_tensor(v) else np.asarray(v))
              for k, v in arrays.items() if v is not None}
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **arrays)
    print(f"  {name}.npz  {os.path.getsize(path) / 1024:.1f} KiB")


def load_residual_quantizers(ref_root):
    """modal_residual.py imports `modal` further down; its quantizers sit above
    that import, so execute only that leading part of the file."""
    src = open(os.path.join(ref_root, "modal_residual.py")).read()
    head = src.split("# ---------------- hook ----------------")[0]
    mod = types.ModuleType("modal_residual_head")
    exec(compile(head, "modal_residual.py", "exec"), mod.__dict__)
    return mod


def kernel_test_inputs(T, B, HV, K, V, seed):
    """Input recipe of experiments/test_cuda_kernel.py:35-44."""
    torch.manual_seed(seed)
    q = torch.randn(T, B, HV, K)
    k = torch.randn(T, B, HV, K)
    k = k / k.norm(dim=-1, keepdim=True).clamp(min=1e-8)
    v = torch.randn(T, B, HV, V)
    alpha = torch.full((T, B, HV), 0.995)
    beta = torch.rand(T, B, HV).sigmoid()
    h0 = torch.randn(B, HV, K, V) * 0.1
    return h0, q, k, v, alpha, beta


def config1(rr, rq):
    """The CPU mechanism configuration (number 1 of the named workloads) at its stated size: batch 1, 4 heads, K = V = 128, T = 2000 sequential decode
    steps, constant decay 0.995, q and k ~ N(0,1) L2-normalised per head, v ~ N(0,1),
    beta = sigmoid(N(0,1)), seed 0, draw order of experiments/exp2b_granularity.py:49-56; int8 state
    with one scale per V column and an fp32 error-feedback residual against the unquantised fp32
    recurrence.  Stored: both final states, the relative L2 error, and sums of the inputs so that a
    test can tell its own draws are the same ones."""
    torch.manual_seed(0)
    HV, K, V, T = 4, 128, 128, 2000
    q = torch.randn(T, HV, K); q = q / q.norm(dim=-1, keepdim=True).clamp(min=1e-8)
    k = torch.randn(T, HV, K); k = k / k.norm(dim=-1, keepdim=True).clamp(min=1e-8)
    v = torch.randn(T, HV, V)
    alpha = torch.full((T, HV), 0.995)
    beta = torch.randn(T, HV).sigmoid()
    h0 = torch.randn(HV, K, V) * 0.1
    _, h_ref = rr.gdn_decode_batched(h0, q, k, v, alpha, beta)
    h = h0.clone()
    fb = rq.ErrorFeedback(h0.shape)
    for t in range(T):
        h, _ = rr.gdn_step_batched(h, q[t], k[t], v[t], alpha[t], beta[t])
        h = fb.step(h, lambda x: rq.per_axis_quantize(x, 8, -2))
    err = ((h - h_ref).norm() / h_ref.norm()).item()
    print(f"  config 1: final-state relative L2 error {err:.4e}")
    sums = torch.tensor([x.double().sum().item() for x in (q, k, v, beta, h0)], dtype=torch.float64)
    save("config1_mechanism", h_ref=h_ref, h_quant=h, err=err, input_sums=sums)


def main(ref_root, only=None):
    sys.path.insert(0, ref_root)
    from statequant import kernel as tk
    from statequant import quant as rq
    from statequant import reference as rr
    from vllm_integration import quantized_packed_decode as qpd
    from vllm_integration import test_quantized_packed_decode as tq
    mr = load_residual_quantizers(ref_root)

    torch.set_num_threads(1)   # reduction order must not depend on the host
    if only in (None, "config1"):
        config1(rr, rq)
    if only is not None:
        return

    # -- 1. quantizers ------------------------------------------------------
    torch.manual_seed(11)
    x = torch.randn(3, 32, 16) * 0.7
    x[0, :, 3] = 0.0                                   # an all-zero column (scale floor)
    out = {"x": x}
    for bits in (3, 4, 5, 6, 8):
        c, s, d = tk.per_v_channel_quantize(x, bits)
        out[f"pv_codes_{bits}"], out[f"pv_scale_{bits}"], out[f"pv_deq_{bits}"] = c, s, d
        out[f"axis_m2_{bits}"] = rq.per_axis_quantize(x, bits, -2)
        ud, us = rq.uniform_quantize(x, bits)
        out[f"uni_deq_{bits}"], out[f"uni_scale_{bits}"] = ud, us
    for prec in ("int8", "int4"):
        out[f"resid_head_{prec}"] = mr.quantize_residual(x * 1e-3, prec)
    save("quantizers", **out)

    # -- 2. exact recurrence -----------------------------------------------
    h0, q, k, v, alpha, beta = kernel_test_inputs(6, 1, 3, 32, 16, seed=3)
    o, hT = rr.gdn_decode_batched(h0[0], q[:, 0], k[:, 0], v[:, 0], alpha[:, 0], beta[:, 0])
    hb, ob = tk.gdn_step_fp32_torch(h0, q[0], k[0], v[0], alpha[0], beta[0])
    save("recurrence", h0=h0, q=q, k=k, v=v, alpha=alpha, beta=beta,
         o=o, h_final=hT, h_step_b=hb, o_step_b=ob)

    # -- 3. fused one step, every residual format, 2 shapes -----------------
    for tag, (B, HV, K, V) in {"small": (2, 3, 32, 16), "tile128": (1, 1, 128, 128)}.items():
        h0, q, k, v, alpha, beta = kernel_test_inputs(3, B, HV, K, V, seed=5)
        for res_fmt in (tk.RES_FP32, tk.RES_FP16, tk.RES_FP8, tk.RES_INT8):
            for bits in ((8, 4) if tag == "small" else (8,)):
                st = tk.init_quant_state(h0, bits, res_fmt)
                rec = {"h0": h0, "q": q, "k": k, "v": v, "alpha": alpha, "beta": beta}
                for t in range(3):          # step 2 starts from a non-zero residual
                    o, hc, sc, e, es = tk.gdn_quant_step_torch(
                        *st, q[t], k[t], v[t], alpha[t], beta[t], bits, res_fmt)
                    rec.update({f"o{t}": o, f"codes{t}": hc, f"scale{t}": sc,
                                f"e{t}": e, f"es{t}": es})
                    st = (hc, sc, e, es)
                save(f"step_{tag}_fmt{res_fmt}_b{bits}", **rec)

    # -- 4. chained decode vs the composed oracle (test_cuda_kernel.py:47-61)
    h0, q, k, v, alpha, beta = kernel_test_inputs(24, 1, 4, 64, 64, seed=0)
    _, _, deq0 = tk.per_v_channel_quantize(h0, 8)
    h = deq0[0].clone()
    fb = rq.ErrorFeedback((4, 64, 64))
    outs = []
    for t in range(24):
        h, o = rr.gdn_step_batched(h, q[t, 0], k[t, 0], v[t, 0], alpha[t, 0], beta[t, 0])
        h = fb.step(h, lambda x: rq.per_axis_quantize(x, 8, -2))
        outs.append(o)
    save("decode_oracle", h0=h0, q=q, k=k, v=v, alpha=alpha, beta=beta,
         o=torch.stack(outs), h_final=h, e_final=fb.e)

    # -- 5. mechanism experiment (exp2b_granularity.py:37-72), shortened ----
    torch.manual_seed(0)
    HV, K, V, T = 2, 32, 32, 300
    q = torch.randn(T, HV, K)
    k = torch.randn(T, HV, K); k = k / k.norm(dim=-1, keepdim=True).clamp(min=1e-8)
    v = torch.randn(T, HV, V)
    alpha = torch.full((T, HV), 0.995)
    beta = torch.rand(T, HV).sigmoid()
    h0 = torch.randn(HV, K, V) * 0.1
    _, h_ref = rr.gdn_decode_batched(h0, q, k, v, alpha, beta)
    rec = {"h0": h0, "q": q, "k": k, "v": v, "alpha": alpha, "beta": beta, "h_ref": h_ref}

    def run(qf, ef):
        h = h0.clone()
        fb = rq.ErrorFeedback(h0.shape) if ef else None
        for t in range(T):
            h, _ = rr.gdn_step_batched(h, q[t], k[t], v[t], alpha[t], beta[t])
            h = fb.step(h, qf) if ef else qf(h)
        return h

    for bits in (3, 4, 8):
        rec[f"head_noef_{bits}"] = run(lambda x, b=bits: rq.uniform_quantize(x, b)[0], False)
        rec[f"head_ef_{bits}"] = run(lambda x, b=bits: rq.uniform_quantize(x, b)[0], True)
        rec[f"col_ef_{bits}"] = run(lambda x, b=bits: rq.per_axis_quantize(x, b, -2), True)
    save("mechanism", **rec)

    # -- 6. rounding ties (test_cuda_kernel.py:64-118) ----------------------
    K, V, qmax = 32, 8, 127.0
    codes = (torch.arange(K, dtype=torch.float32) % 8) - 3.5
    target = codes[:, None].repeat(1, V).contiguous()
    target[0, :] = qmax
    scale = target.abs().amax(dim=0).clamp(min=1e-12) / qmax
    expected = torch.round(target / scale[None, :]).clamp(-qmax, qmax)
    z = lambda *s: torch.zeros(*s)
    o, hc, sc, e, es = tk.gdn_quant_step_torch(
        torch.zeros(1, 1, K, V, dtype=torch.int8), torch.ones(1, 1, V),
        target[None, None].contiguous(), None, z(1, 1, K), z(1, 1, K), z(1, 1, V),
        z(1, 1), z(1, 1), 8, tk.RES_FP32)
    assert torch.equal(hc[0, 0].float(), expected)
    save("ties_kv", target=target, expected=expected, codes=hc, scale=sc, e=e)

    # -- 7. slot path helpers ------------------------------------------------
    B, H, HV, K, V = 3, 2, 4, 32, 16
    torch.manual_seed(21)
    pool = torch.randn(5, HV, V, K) * 0.1
    sc8 = qpd.init_quantized_state(5, HV, V, K, "cpu", h0=pool)
    sc4 = qpd.init_quantized_state(5, HV, V, K, "cpu", h0=pool, resid_fmt=qpd.RESID_INT4)
    steps = [tq.make_packed_inputs(1, H, HV, K, V, "cpu", seed=100 + t) for t in range(8)]
    al, be = tq.gates_from_inputs(steps[0][1], steps[0][2], steps[0][3], steps[0][4])
    uq, uk, uv = tq.unpack_qkv(steps[0][0], 1, H, HV, K, V, K ** -0.5, True)
    c0, s0 = tq.quantize_vk(pool[1:2])
    o_ref, h_ref = tq.oracle_decode_vk((c0.float() * s0[..., None])[0], steps, H, K ** -0.5, True)
    rec = {"pool": pool, "codes8": sc8[0], "scale8": sc8[1], "rc8_shape": list(sc8[2].shape),
           "rc4_shape": list(sc4[2].shape), "alpha0": al, "beta0": be,
           "q0": uq, "k0": uk, "v0": uv, "o_ref": o_ref, "h_ref": h_ref,
           "bytes": [qpd.state_bytes_per_slot(32, 128, 128, False, 4),
                     qpd.state_bytes_per_slot(32, 128, 128, False, 2),
                     qpd.state_bytes_per_slot(32, 128, 128, True, resid_fmt=qpd.RESID_INT8),
                     qpd.state_bytes_per_slot(32, 128, 128, True, resid_fmt=qpd.RESID_INT4)]}
    for t, (m, a, b, A, d) in enumerate(steps):
        rec.update({f"mixed{t}": m, f"a{t}": a, f"b{t}": b, f"A_log{t}": A, f"dt_bias{t}": d})
    save("slot_path", **rec)


if __name__ == "__main__":
    if len(sys.argv) not in (2, 3):
        raise SystemExit(__doc__)
    main(sys.argv[1], sys.argv[2] if len(sys.argv) == 3 else None)
