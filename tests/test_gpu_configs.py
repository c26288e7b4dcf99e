"""The named workload configurations as GPU parity cases (the benchmark line
itself only times one of them): the int8-residual single-layer step, the
slot-indexed int4 step at full size through size-independent properties, a
large batch, and the bit-width / decay sweep."""

from __future__ import annotations

import math

import pytest
import torch

from conftest import load_golden
from oracle import gdn_oracle as orc
import parity
from parity import assert_close, check_quant_step

pytestmark = pytest.mark.gpu
DEV = "cuda"
H = HV = 32
K = V = 128


def _mods():
    from carrykernel_b200.cuda import binding
    from carrykernel_b200.statequant import kernel as sq
    from carrykernel_b200.vllm_integration import quantized_packed_decode as qpd
    return sq, binding, qpd


def _gated_inputs(B, T, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.nn.functional.normalize(torch.randn(T, B, HV, K, generator=g), dim=-1)
    k = torch.nn.functional.normalize(torch.randn(T, B, HV, K, generator=g), dim=-1)
    v = torch.randn(T, B, HV, V, generator=g)
    alpha = torch.exp(-0.1 * torch.nn.functional.softplus(torch.randn(T, B, HV, generator=g)))
    beta = torch.sigmoid(torch.randn(T, B, HV, generator=g))
    return q, k, v, alpha, beta


@pytest.mark.parametrize("resid_scale", ["head", "v"])
def test_single_layer_int8_residual_after_warm_up(resid_scale):
    """8 slots x 32 heads, int8 state + int8 residual, bf16 q/k/v; the state is
    first warmed with 64 fp32 steps of the same process (on the GPU), then two
    teacher-forced quantised steps are compared with the oracle."""
    sq, binding, _ = _mods()
    B, warm = 8, 64
    q, k, v, alpha, beta = _gated_inputs(B, warm + 2, seed=0)
    h = torch.zeros(B, HV, K, V, device=DEV)
    for t in range(warm):
        h, _ = binding.gdn_fp32_step_cuda(h, q[t].to(DEV), k[t].to(DEV), v[t].to(DEV),
                                          alpha[t].to(DEV), beta[t].to(DEV))
    h0 = h.cpu()
    assert 0.5 < h0.abs().max().item() < 5.0                      # a warm, O(1) state
    qb, kb, vb = q.to(torch.bfloat16), k.to(torch.bfloat16), v.to(torch.bfloat16)
    st = orc.init_quant_state(h0, 8, orc.RES_INT8, resid_scale)
    worst = {"state_flip_frac": 0.0, "resid_flip_frac": 0.0}
    for t in (warm, warm + 1):
        ref = orc.quant_step(*st, qb[t], kb[t], vb[t], alpha[t], beta[t], 8, orc.RES_INT8, resid_scale)
        got = binding.gdn_quant_step_cuda(*[x.to(DEV) for x in st], qb[t].to(DEV), kb[t].to(DEV), vb[t].to(DEV),
                                          alpha[t].to(DEV), beta[t].to(DEV), 8, orc.RES_INT8,
                                          resid_scale=resid_scale)
        stats = check_quant_step(got, ref, orc.RES_INT8, what=f"int8 residual, {resid_scale}, t={t}")
        worst = {k_: max(worst[k_], stats[k_]) for k_ in worst}
        st = ref[1:]
    from carrykernel_b200 import _lib
    assert _lib.load_library().carry_gdn_last_kernel() == 2, "the streaming kernel should have served this shape"
    print(f"flip fractions ({resid_scale}): {worst}")


def _slot_workload(B, num_slots, resid_fmt, rscale, seed):
    g = torch.Generator().manual_seed(seed)
    pool = torch.randn(num_slots, HV, V, K, generator=g) * 0.12
    pool[0] = 0
    st = orc.init_quantized_pool(num_slots, HV, V, K, h0=pool, resid_fmt=resid_fmt, resid_scale=rscale)
    mixed = torch.randn(B, 2 * H * K + HV * V, generator=g).to(torch.bfloat16)
    a = torch.randn(B, HV, generator=g).to(torch.bfloat16)
    b = torch.randn(B, HV, generator=g).to(torch.bfloat16)
    idx = (torch.randperm(num_slots - 1, generator=g)[:B] + 1).to(torch.int32)
    return st, mixed, a, b, torch.full((HV,), math.log(0.1)), torch.zeros(HV), idx


def _run_slot(qpd, st, mixed, a, b, A_log, dt_bias, idx, resid_fmt):
    dev = [x.clone().to(DEV) for x in st]
    out = torch.full((mixed.shape[0], 1, HV, V), float("nan"), dtype=torch.bfloat16, device=DEV)
    qpd.quantized_gated_delta_rule_packed_decode(
        mixed.to(DEV), a.to(DEV), b.to(DEV), A_log.to(DEV), dt_bias.to(DEV), K ** -0.5, *dev, out, idx.to(DEV),
        use_qk_l2norm_in_kernel=True, resid_fmt=resid_fmt)
    torch.cuda.synchronize()
    return dev, out


def test_slot_step_full_size_properties():
    """64 requests on a pool of 256 slots, int4 residual, per-head scale: checked
    through properties that do not need the CPU oracle at this size, plus the
    oracle on 4 sampled requests."""
    _, _, qpd = _mods()
    B, num_slots = 64, 257
    st, mixed, a, b, A_log, dt_bias, idx = _slot_workload(B, num_slots, orc.RESID_INT4, "head", seed=3)
    dev, out = _run_slot(qpd, st, mixed, a, b, A_log, dt_bias, idx, qpd.RESID_INT4)
    got = [x.cpu() for x in dev]
    touched = torch.zeros(num_slots, dtype=torch.bool)
    touched[idx.long()] = True
    # (a) slots outside the batch are byte-identical, slots inside it moved
    for x, y in zip(got, st):
        assert torch.equal(x[~touched], y[~touched])
    assert not torch.equal(got[0][touched], st[0][touched])
    # (b) code ranges
    assert int(got[0].abs().max()) <= 127
    nib = orc.unpack_int4(got[2][touched])
    assert int(nib.abs().max()) <= 7 and int((nib != 0).sum()) > 0
    assert not torch.isnan(out.float()).any()
    # (c) batched == two half batches (paging isolation at full size), bit for bit
    half = B // 2
    dev2 = [x.clone().to(DEV) for x in st]
    out2 = torch.empty_like(out)
    for lo, hi in ((0, half), (half, B)):
        qpd.quantized_gated_delta_rule_packed_decode(
            mixed[lo:hi].to(DEV), a[lo:hi].to(DEV), b[lo:hi].to(DEV), A_log.to(DEV), dt_bias.to(DEV), K ** -0.5,
            *dev2, out2[lo:hi], idx[lo:hi].to(DEV), use_qk_l2norm_in_kernel=True, resid_fmt=qpd.RESID_INT4)
    torch.cuda.synchronize()
    assert torch.equal(out2, out)
    for x, y in zip(dev2, dev):
        assert torch.equal(x, y)
    # (d) every state scale is the row maximum of the new target: the largest code of each row is 127
    rows_max = got[0][touched].abs().amax(dim=-1)
    assert torch.all(rows_max == 127)
    # (e) the residual is at most half a state step: |code_r * es| <= 0.5 * state_scale (+ one residual step)
    es = got[3][touched][..., None, None]
    bound = 0.5 * got[1][touched][..., None] + es
    assert torch.all((nib.float() * es).abs() <= bound * 1.0001)
    # (f) oracle on a sample of the requests
    sample = [0, 17, 40, 63]
    ref = [x.clone() for x in st]
    out_r = torch.empty(len(sample), 1, HV, V, dtype=torch.bfloat16)
    orc.packed_decode_step(mixed[sample], a[sample], b[sample], A_log, dt_bias, K ** -0.5, *ref, out_r, idx[sample],
                           use_qk_l2norm_in_kernel=True, resid_fmt=orc.RESID_INT4)
    assert_close(out.cpu()[sample], out_r, "out", rtol=8e-3, atol=1e-4)
    fs, fr = parity.check_pool(got, ref, True, idx[sample].tolist(), orc.unpack_int4, "full size sample")
    print(f"flip fractions: state {fs:.2e}, residual {fr:.2e}")


@pytest.mark.parametrize("B", [128, 512, 640])
def test_large_batch_against_oracle_sample(B):
    """640 requests x 32 heads are more tiles per CTA than the streaming kernel
    caches facts and addresses for (128 per CTA on 148 SMs), so the last requests
    go through its uncached path."""
    _, _, qpd = _mods()
    num_slots = B + 1
    st, mixed, a, b, A_log, dt_bias, idx = _slot_workload(B, num_slots, orc.RESID_INT4, "head", seed=B)
    dev, out = _run_slot(qpd, st, mixed, a, b, A_log, dt_bias, idx, qpd.RESID_INT4)
    sample = [0, B // 3, B - 1]
    ref = [x.clone() for x in st]
    out_r = torch.empty(len(sample), 1, HV, V, dtype=torch.bfloat16)
    orc.packed_decode_step(mixed[sample], a[sample], b[sample], A_log, dt_bias, K ** -0.5, *ref, out_r, idx[sample],
                           use_qk_l2norm_in_kernel=True, resid_fmt=orc.RESID_INT4)
    assert_close(out.cpu()[sample], out_r, "out", rtol=8e-3, atol=1e-4)
    parity.check_pool([x.cpu() for x in dev], ref, True, idx[sample].tolist(), orc.unpack_int4, f"B={B}")


def test_bit_width_and_decay_sweep():
    """Bits in {3, 4, 5, 6, 8}; per-V-column scale + fp32 error feedback against
    the uniform per-head grid without feedback; per-head constant decay drawn
    from U[0.9, 0.999]; 96 chained steps on the GPU (reduced from 512 to keep
    the suite short).  The error of the final dequantised state is taken against
    the fp32 GPU recurrence; on a 2-request subset the GPU chain is compared
    with the CPU oracle chain."""
    sq, binding, _ = _mods()
    B, T = 4, 96
    g = torch.Generator().manual_seed(5)
    q = torch.randn(T, B, HV, K, generator=g)
    k = torch.nn.functional.normalize(torch.randn(T, B, HV, K, generator=g), dim=-1)
    v = torch.randn(T, B, HV, V, generator=g)
    alpha = (0.9 + 0.099 * torch.rand(B, HV, generator=g))[None].expand(T, B, HV).contiguous()
    beta = torch.sigmoid(torch.randn(T, B, HV, generator=g))
    h0 = torch.randn(B, HV, K, V, generator=g) * 0.1
    d = lambda x: x.to(DEV)
    h = d(h0)
    for t in range(T):
        h, _ = binding.gdn_fp32_step_cuda(h, d(q[t]), d(k[t]), d(v[t]), d(alpha[t]), d(beta[t]))
    h_ref = h.cpu()
    _, h_ref_cpu = orc.gdn_decode(h0[:2], q[:, :2], k[:, :2], v[:, :2], alpha[:, :2], beta[:, :2])
    assert ((h_ref[:2] - h_ref_cpu).norm() / h_ref_cpu.norm()).item() < 1e-4
    rel = lambda x: ((x - h_ref).norm() / h_ref.norm()).item()
    errs = {}
    for bits in (3, 4, 5, 6, 8):
        _, c, s, _, _ = binding.gdn_quant_decode_cuda(d(h0), d(q), d(k), d(v), d(alpha), d(beta), T, bits, sq.RES_FP32)
        ef = rel((c.float() * s[..., None, :]).cpu())
        _, c, s, _, _ = sq.gdn_quant_decode_fused(d(h0), d(q), d(k), d(v), d(alpha), d(beta), T, bits=bits,
                                                  res_fmt=sq.RES_NONE, state_scale="head")
        uni = rel((c.float() * s[..., None, None]).cpu())
        errs[bits] = (uni, ef)
        assert ef < uni, f"{bits} bits: error feedback ({ef:.3e}) should beat the uniform grid ({uni:.3e})"
    assert errs[8][1] < errs[4][1] < errs[3][1]
    # CPU oracle chain on the first two requests, 4 bits, both arms
    sub = (h0[:2], q[:, :2], k[:, :2], v[:, :2], alpha[:, :2], beta[:, :2])
    _, c_o, s_o, _, _ = orc.quant_decode(*sub, bits=4, res_fmt=orc.RES_FP32)
    _, c_g, s_g, _, _ = binding.gdn_quant_decode_cuda(*[d(x) for x in sub], T, 4, sq.RES_FP32)
    deq_o, deq_g = orc.dequant_state(c_o, s_o), orc.dequant_state(c_g.cpu(), s_g.cpu())
    assert ((deq_g - deq_o).norm() / deq_o.norm()).item() < 5e-2     # free-running chains drift by flips only
    print("final-state relative error (uniform no-EF, per-V + EF):", {b_: (round(u, 4), round(e, 4)) for b_, (u, e) in errs.items()})


def test_config1_mechanism_full_size_on_the_gpu():
    """The CPU mechanism configuration (number 1 of the named workloads) at its stated size through the CUDA entry point: T = 2000 chained steps of
    ``gdn_quant_decode_cuda`` (int8 state, one scale per V column, fp32 error-feedback residual) on
    batch 1 x 4 heads x 128 x 128; the final dequantised state against the reference's unquantised fp32
    recurrence (fixture) must show the error the reference's own CPU run of the mechanism shows, within
    5 % (6.9e-3; a free-running chain, so codes are not compared one by one)."""
    from carrykernel_b200.cuda import binding
    g = load_golden("config1_mechanism")
    h0, q, k, v, alpha, beta, sums = parity.config1_inputs()
    assert torch.equal(sums, g["input_sums"])
    dev = lambda x: x.to(DEV)
    o, codes, scale, e, e_scale = binding.gdn_quant_decode_cuda(
        dev(h0[None]), dev(q[:, None]), dev(k[:, None]), dev(v[:, None]), dev(alpha[:, None]), dev(beta[:, None]),
        q.shape[0], bits=8, res_fmt=orc.RES_FP32)
    torch.cuda.synchronize()
    assert e_scale is None and o.shape == (2000, 1, 4, 128)
    h_gpu = orc.dequant_state(codes.cpu(), scale.cpu())[0]
    rel = lambda x, y: ((x - y).norm() / y.norm()).item()
    err = rel(h_gpu, g["h_ref"])
    assert abs(err - float(g["err"])) < 0.05 * float(g["err"]), f"{err:.4e} vs {float(g['err']):.4e}"
