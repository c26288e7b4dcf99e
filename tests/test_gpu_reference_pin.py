"""The reference's own slot-indexed kernel, run here, against the CPU oracle and
against this library.

tomalmog/carrykernel implements the slot-indexed step only as a Triton kernel
(vllm_integration/quantized_packed_decode.py:101-327).  ``oracle/make_ref.py``
stages an unmodified copy of that file; these tests run it on the GPU on the
same seeded inputs as ``oracle.gdn_oracle.packed_decode_step`` (teacher-forced:
every step starts from the reference kernel's pool) and hold the two to the
parity rule of ``tests/parity.py``.  That is the code-level anchor of the
oracle every other slot-path test leans on.  The same pools are also given to
this library's call, so the CUDA kernel is compared with the reference kernel
directly.

Skipped when the staged copy is absent (it is not part of the repository).
"""

from __future__ import annotations

import sys

import pytest
import torch

from oracle import gdn_oracle as orc
from oracle import make_ref
import parity
from parity import assert_close, make_packed_inputs

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(make_ref.ref_path() is None, reason="oracle/_ref not staged (oracle/make_ref.py)")]
DEV = "cuda"


def _ref_qpd():
    path = make_ref.ref_path()
    if path not in sys.path:
        sys.path.insert(0, path)
    from vllm_integration import quantized_packed_decode as rqpd
    return rqpd


def _ours():
    from carrykernel_b200.vllm_integration import quantized_packed_decode as qpd
    return qpd


@pytest.mark.parametrize("shape", [(4, 8, 16, 64, 64), (4, 16, 32, 128, 128)])
@pytest.mark.parametrize("resid_fmt", [orc.RESID_INT8, orc.RESID_INT4])
@pytest.mark.parametrize("l2norm", [True, False])
def test_reference_kernel_vs_oracle_and_library(shape, resid_fmt, l2norm):
    rqpd, qpd = _ref_qpd(), _ours()
    B, H, HV, K, V = shape
    num_slots = 2 * B + 1
    g = torch.Generator().manual_seed(7 * K + B + resid_fmt)
    pool = torch.randn(num_slots, HV, V, K, generator=g) * 0.1
    ref = list(rqpd.init_quantized_state(num_slots, HV, V, K, DEV, h0=pool.to(DEV), resid_fmt=resid_fmt))
    slots = (torch.randperm(num_slots - 1, generator=g)[:B] + 1).to(torch.int32)
    slots[1] = 0                                               # one padding request
    live = [s for s in slots.tolist() if s > 0]
    scale = K ** -0.5
    worst = [0.0, 0.0]
    for t in range(3):
        mixed, a, b, A_log, dt_bias = make_packed_inputs(B, H, HV, K, V, seed=300 + t,
                                                         qk_gain=1.0 if l2norm else K ** -0.5)
        cpu = [x.cpu().clone() for x in ref]                   # teacher forcing: both start from the reference's pool
        ours = [x.clone() for x in ref]
        dev_in = [x.to(DEV) for x in (mixed, a, b, A_log, dt_bias)]
        out_ref = torch.full((B, 1, HV, V), float("nan"), device=DEV)
        rqpd.quantized_gated_delta_rule_packed_decode(*dev_in, scale, *ref, out_ref, slots.to(DEV),
                                                      use_qk_l2norm_in_kernel=l2norm, resid_fmt=resid_fmt)
        out_cpu = torch.full((B, 1, HV, V), float("nan"))
        orc.packed_decode_step(mixed, a, b, A_log, dt_bias, scale, *cpu, out_cpu, slots,
                               use_qk_l2norm_in_kernel=l2norm, resid_fmt=resid_fmt)
        out_ours = torch.full((B, 1, HV, V), float("nan"), device=DEV)
        qpd.quantized_gated_delta_rule_packed_decode(*dev_in, scale, *ours, out_ours, slots.to(DEV),
                                                     use_qk_l2norm_in_kernel=l2norm, resid_fmt=resid_fmt)
        torch.cuda.synchronize()
        what = f"{shape} fmt{resid_fmt} l2={l2norm} t{t}"
        # oracle against the reference kernel
        assert_close(out_cpu, out_ref.cpu(), f"{what}: oracle out vs reference kernel")
        fs, fr = parity.check_pool(cpu, [x.cpu() for x in ref], resid_fmt == orc.RESID_INT4, live,
                                   orc.unpack_int4, f"{what}: oracle vs reference kernel")
        worst = [max(worst[0], fs), max(worst[1], fr)]
        # this library against the reference kernel
        assert_close(out_ours.cpu(), out_ref.cpu(), f"{what}: library out vs reference kernel")
        parity.check_pool(ours, [x.cpu() for x in ref], resid_fmt == orc.RESID_INT4, live,
                          orc.unpack_int4, f"{what}: library vs reference kernel")
        assert torch.all(out_ref[1] == 0) and torch.all(out_cpu[1] == 0) and torch.all(out_ours[1] == 0)
        untouched = [s for s in range(num_slots) if s not in live]
        for x, y, z in zip(cpu, ref, ours):
            assert torch.equal(x[untouched], y.cpu()[untouched]) and torch.equal(z.cpu()[untouched], y.cpu()[untouched])
    print(f"{shape} fmt{resid_fmt} l2={l2norm}: oracle-vs-reference flips state {worst[0]:.2e} residual {worst[1]:.2e}")


def test_reference_kernel_rounding_ties_equal_oracle():
    """The reference's constructed tie case (test_quantized_packed_decode.py:211-286): the reference
    kernel, the oracle and this library must produce the very same codes, 0 differences."""
    rqpd, qpd = _ref_qpd(), _ours()
    H, HV, K, V = 1, 1, 32, 4
    odd = (torch.arange(K, dtype=torch.float32) % 8) * 2 - 7
    resid_in = odd[None, None, :].repeat(HV, V, 1).contiguous()
    resid_in[..., 0] = 0.0
    state_in = torch.zeros(HV, V, K)
    state_in[..., 0] = 1.0
    sc = torch.zeros(2, HV, V, K, dtype=torch.int8); ss = torch.zeros(2, HV, V)
    rc = torch.zeros(2, HV, V, K, dtype=torch.int8); rs = torch.zeros(2, HV, V)
    sc[1] = state_in.to(torch.int8); ss[1] = 127.0; rc[1] = resid_in.to(torch.int8); rs[1] = 0.5
    mixed = torch.zeros(1, 2 * H * K + HV * V)
    a = torch.full((1, HV), -60.0); b = torch.full((1, HV), -60.0)
    A_log = torch.zeros(HV); dt_bias = torch.zeros(HV)
    idx = torch.tensor([1], dtype=torch.int32)
    cpu = [x.clone() for x in (sc, ss, rc, rs)]
    ref = [x.clone().to(DEV) for x in (sc, ss, rc, rs)]
    ours = [x.clone().to(DEV) for x in (sc, ss, rc, rs)]
    dev_in = [x.to(DEV) for x in (mixed, a, b, A_log, dt_bias)]
    rqpd.quantized_gated_delta_rule_packed_decode(*dev_in, K ** -0.5, *ref, torch.empty(1, 1, HV, V, device=DEV),
                                                  idx.to(DEV))
    qpd.quantized_gated_delta_rule_packed_decode(*dev_in, K ** -0.5, *ours, torch.empty(1, 1, HV, V, device=DEV),
                                                 idx.to(DEV))
    orc.packed_decode_step(mixed, a, b, A_log, dt_bias, K ** -0.5, *cpu, torch.empty(1, 1, HV, V), idx)
    torch.cuda.synchronize()
    expected = torch.round(state_in * 127.0 + resid_in * 0.5).clamp(-127, 127).to(torch.int8)
    assert torch.equal(ref[0][1].cpu(), expected)
    for x, y, z in zip(cpu, ref, ours):
        assert torch.equal(x, y.cpu()), "oracle differs from the reference kernel on the tie case"
        assert torch.equal(z.cpu(), y.cpu()), "library differs from the reference kernel on the tie case"


def test_reference_cpu_step_vs_library_statequant():
    """The reference's CPU step (statequant/kernel.py:149-178), imported from the staged copy, against
    this library's statequant call on fresh seeded inputs (the committed fixtures cover other seeds)."""
    path = make_ref.ref_path()
    if path not in sys.path:
        sys.path.insert(0, path)
    from statequant import kernel as tk
    from carrykernel_b200.cuda import binding
    h0, q, k, v, alpha, beta = parity.seeded_inputs(2, 4, 128, 128, seed=91, alpha_mode="gated")
    for res_fmt in (orc.RES_FP32, orc.RES_INT8):
        st = tk.init_quant_state(h0, 8, res_fmt)
        ref_step = tk.gdn_quant_step_torch(*st, q, k, v, alpha, beta, 8, res_fmt)
        got = binding.gdn_quant_step_cuda(*[None if x is None else x.to(DEV) for x in st], q.to(DEV), k.to(DEV),
                                          v.to(DEV), alpha.to(DEV), beta.to(DEV), 8, res_fmt)
        torch.cuda.synchronize()
        parity.check_quant_step(got, ref_step, res_fmt, what=f"reference CPU step fmt{res_fmt}")
