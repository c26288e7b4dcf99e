"""GPU parity of the statequant / cuda.binding surfaces against the CPU oracle
and the reference's golden vectors.  Every call goes through the C ABI."""

from __future__ import annotations

import pytest
import torch

from conftest import load_golden
from oracle import gdn_oracle as orc
from parity import assert_close, assert_codes, check_quant_step, seeded_inputs

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _mods():
    from carrykernel_b200.cuda import binding
    from carrykernel_b200.statequant import kernel as sq
    return sq, binding


def _to_dev(xs):
    return [x.to(DEV) if torch.is_tensor(x) else x for x in xs]


def test_library_is_the_in_tree_build():
    import os
    from carrykernel_b200 import _lib
    lib = _lib.load_library()
    assert lib.carry_gdn_abi_version() == _lib.ABI_VERSION
    assert os.path.dirname(_lib.LIB_PATH).endswith("carrykernel_b200")


def test_rounding_ties_exact():
    """Constructed exact .5 quotients: the codes must equal torch.round's
    (the reference's tie test, experiments/test_cuda_kernel.py:64-118)."""
    sq, binding = _mods()
    g = load_golden("ties_kv")
    K, V = g["target"].shape
    z = lambda *s: torch.zeros(*s, device=DEV)
    _, codes, scale, _, _ = binding.gdn_quant_step_cuda(
        torch.zeros(1, 1, K, V, dtype=torch.int8, device=DEV), torch.ones(1, 1, V, device=DEV),
        g["target"][None, None].contiguous().to(DEV), None, z(1, 1, K), z(1, 1, K), z(1, 1, V),
        z(1, 1), z(1, 1), 8, sq.RES_FP32)
    assert torch.equal(codes.cpu(), g["codes"])
    assert torch.equal(scale.cpu(), g["scale"])


@pytest.mark.parametrize("tag,bits", [("small", 8), ("small", 4), ("tile128", 8)])
@pytest.mark.parametrize("res_fmt", [0, 1, 2, 3])
def test_step_vs_reference_golden(tag, bits, res_fmt):
    """Teacher-forced against the reference's own recorded outputs: every step
    starts from the reference's state."""
    sq, binding = _mods()
    fp8 = ("e0", "e1", "e2") if res_fmt == 2 else ()
    g = load_golden(f"step_{tag}_fmt{res_fmt}_b{bits}", fp8_keys=fp8)
    st = orc.init_quant_state(g["h0"], bits, res_fmt)
    for t in range(3):
        got = binding.gdn_quant_step_cuda(
            *_to_dev(st), *_to_dev([g["q"][t], g["k"][t], g["v"][t], g["alpha"][t], g["beta"][t]]),
            bits, res_fmt)
        ref = (g[f"o{t}"], g[f"codes{t}"], g[f"scale{t}"], g[f"e{t}"], g.get(f"es{t}"))
        check_quant_step(got, ref, res_fmt, what=f"{tag} fmt{res_fmt} b{bits} t{t}")
        st = ref[1:]


@pytest.mark.parametrize("shape", [(2, 3, 32, 16), (1, 4, 64, 64), (2, 32, 128, 128), (3, 2, 48, 80)])
@pytest.mark.parametrize("res_fmt", [0, 1, 2, 3, 4])
@pytest.mark.parametrize("resid_scale", ["v", "head"])
def test_step_vs_oracle(shape, res_fmt, resid_scale):
    if resid_scale == "head" and res_fmt not in (3, 4):
        pytest.skip("the residual scale granularity only exists for integer residuals")
    sq, binding = _mods()
    B, HV, K, V = shape
    h0, q, k, v, alpha, beta = seeded_inputs(B, HV, K, V, seed=hash(shape) % 1000, T=3,
                                             alpha_mode="gated")
    st = orc.init_quant_state(h0, 8, res_fmt, resid_scale)
    for t in range(3):
        ref = orc.quant_step(*st, q[t], k[t], v[t], alpha[t], beta[t], 8, res_fmt, resid_scale)
        got = binding.gdn_quant_step_cuda(
            *_to_dev(st), *_to_dev([q[t], k[t], v[t], alpha[t], beta[t]]), 8, res_fmt,
            resid_scale=resid_scale)
        check_quant_step(got, ref, res_fmt, unpack_int4=orc.unpack_int4,
                         what=f"{shape} fmt{res_fmt} {resid_scale} t{t}")
        st = ref[1:]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_step_low_precision_activations(dtype):
    """bf16 / fp16 q, k, v are read as they are and widened exactly."""
    sq, binding = _mods()
    B, HV, K, V = 2, 8, 128, 128
    h0, q, k, v, alpha, beta = seeded_inputs(B, HV, K, V, seed=4, dtype=dtype, alpha_mode="gated")
    for res_fmt, rs in ((3, "head"), (4, "head"), (3, "v")):
        st = orc.init_quant_state(h0, 8, res_fmt, rs)
        ref = orc.quant_step(*st, q, k, v, alpha, beta, 8, res_fmt, rs)
        got = binding.gdn_quant_step_cuda(*_to_dev(st), *_to_dev([q, k, v, alpha, beta]), 8, res_fmt,
                                          resid_scale=rs)
        check_quant_step(got, ref, res_fmt, unpack_int4=orc.unpack_int4, what=f"{dtype} fmt{res_fmt}")


@pytest.mark.parametrize("bits", [3, 4, 5, 6, 8])
def test_bit_widths_and_uniform_grid(bits):
    """The bit-width sweep's two arms: per-V-column + error feedback (fp32
    residual) and the uniform per-head grid without error feedback."""
    sq, binding = _mods()
    B, HV, K, V = 2, 4, 128, 128
    h0, q, k, v, alpha, beta = seeded_inputs(B, HV, K, V, seed=bits)
    st = orc.init_quant_state(h0, bits, 0)
    ref = orc.quant_step(*st, q, k, v, alpha, beta, bits, 0)
    got = binding.gdn_quant_step_cuda(*_to_dev(st), *_to_dev([q, k, v, alpha, beta]), bits, 0)
    check_quant_step(got, ref, 0, what=f"bits{bits} per-V+EF")

    st = orc.init_quant_state(h0, bits, orc.RES_NONE, state_scale="head")
    ref = orc.quant_step(*st, q, k, v, alpha, beta, bits, orc.RES_NONE, state_scale="head")
    got = sq.gdn_quant_step_fused(*_to_dev(st), *_to_dev([q, k, v, alpha, beta]), bits=bits,
                                  res_fmt=sq.RES_NONE, state_scale="head")
    check_quant_step(got, ref, orc.RES_NONE, what=f"bits{bits} uniform")
    from carrykernel_b200 import _lib
    assert _lib.load_library().carry_gdn_last_kernel() == 5, "the 128x128 no-feedback kernel should have served this"

    # no feedback with one scale per V column, bf16 activations, in the same kernel
    qb, kb, vb = q.bfloat16(), k.bfloat16(), v.bfloat16()
    st = orc.init_quant_state(h0, bits, orc.RES_NONE)
    ref = orc.quant_step(*st, qb, kb, vb, alpha, beta, bits, orc.RES_NONE)
    got = sq.gdn_quant_step_fused(*_to_dev(st), *_to_dev([qb, kb, vb, alpha, beta]), bits=bits, res_fmt=sq.RES_NONE)
    check_quant_step(got, ref, orc.RES_NONE, what=f"bits{bits} per-V, no feedback")
    assert _lib.load_library().carry_gdn_last_kernel() == 5


def test_fp32_step():
    sq, binding = _mods()
    h0, q, k, v, alpha, beta = seeded_inputs(2, 8, 128, 128, seed=2)
    h_ref, o_ref = orc.gdn_step(h0, q, k, v, alpha, beta)
    h_c, o_c = binding.gdn_fp32_step_cuda(*_to_dev([h0, q, k, v, alpha, beta]))
    assert (h_c.cpu() - h_ref).abs().max().item() < 1e-5
    assert (o_c.cpu() - o_ref).abs().max().item() < 1e-4
    g = load_golden("recurrence")
    h_c, o_c = binding.gdn_fp32_step_cuda(
        *_to_dev([g["h0"], g["q"][0], g["k"][0], g["v"][0], g["alpha"][0], g["beta"][0]]))
    torch.testing.assert_close(h_c.cpu(), g["h_step_b"], rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(o_c.cpu(), g["o_step_b"], rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("res_fmt,bound", [(0, 5e-3), (1, 5e-3), (2, 1.5e-1), (3, 1.5e-1), (4, 1.5e-1)])
def test_free_running_decode_vs_oracle(res_fmt, bound):
    """T=64 chained steps, no teacher forcing, against the exact recurrence +
    fp32 error feedback (bounds: experiments/test_cuda_kernel.py:158-177)."""
    sq, binding = _mods()
    B, HV, K, V, T = 1, 32, 128, 128, 64
    h0, q, k, v, alpha, beta = seeded_inputs(B, HV, K, V, seed=0, T=T)
    _, _, deq0 = orc.quantize_per_column(h0, 8)
    h = deq0[0].clone()
    e = torch.zeros_like(h)
    outs = []
    for t in range(T):
        h, o = orc.gdn_step(h, q[t, 0], k[t, 0], v[t, 0], alpha[t, 0], beta[t, 0])
        h, e = orc.error_feedback(h, e, lambda x: orc.quantize_per_column(x, 8)[2])
        outs.append(o)
    o_ref = torch.stack(outs).unsqueeze(1)
    o_c, h_c, s_c, _, _ = binding.gdn_quant_decode_cuda(*_to_dev([h0, q, k, v, alpha, beta]), T, 8, res_fmt)
    rel = lambda x, y: ((x - y).norm() / (y.norm() + 1e-12)).item()
    assert rel(o_c.cpu(), o_ref) < bound
    assert rel((h_c.float() * s_c[..., None, :]).cpu()[0], h) < bound


def test_inputs_untouched_and_e_scale_none():
    sq, binding = _mods()
    h0, q, k, v, alpha, beta = seeded_inputs(1, 2, 128, 128, seed=9)
    st = _to_dev(orc.init_quant_state(h0, 8, 3))
    before = [x.clone() for x in st]
    out = binding.gdn_quant_step_cuda(st[0], st[1], st[2], None, *_to_dev([q, k, v, alpha, beta]), 8, 3)
    for x, y in zip(st, before):
        assert torch.equal(x, y)
    assert out[4] is not None and out[0].dtype == torch.float32 and out[0].shape == (1, 2, 128)
    out = binding.gdn_quant_step_cuda(*_to_dev(orc.init_quant_state(h0, 8, 0)),
                                      *_to_dev([q, k, v, alpha, beta]), 8, 0)
    assert out[4] is None


@pytest.mark.parametrize("shape", [(3, 4, 128, 128), (2, 3, 64, 48)])
@pytest.mark.parametrize("res_fmt,resid_scale", [(0, "v"), (1, "v"), (2, "v"), (3, "v"), (3, "head"), (4, "v"), (4, "head")])
def test_in_place_equals_out_of_place(shape, res_fmt, resid_scale):
    """The C ABI allows every output state buffer to be its input buffer (include/carry_gdn.h): the step
    run in place must leave exactly what the out-of-place call returns, for every residual format, on the
    streaming kernel (128 x 128) and on the generic one."""
    sq, binding = _mods()
    B, HV, K, V = shape
    h0, q, k, v, alpha, beta = seeded_inputs(B, HV, K, V, seed=31, alpha_mode="gated")
    st = list(_to_dev(orc.init_quant_state(h0, 8, res_fmt, resid_scale)))
    acts = _to_dev([q, k, v, alpha, beta])
    for _ in range(2):                                  # the second step starts from a non-zero residual
        ref = sq.gdn_quant_step_fused(*st, *acts, bits=8, res_fmt=res_fmt, resid_scale=resid_scale)
        inplace = [None if x is None else x.clone() for x in st]
        o = torch.full((B, HV, V), float("nan"), device=DEV)
        sq.quant_step_into(*inplace, *acts, (o, *inplace), 8, res_fmt, resid_scale)
        torch.cuda.synchronize()
        assert torch.equal(o, ref[0])
        for got, want, name in zip(inplace, ref[1:], ("codes", "scale", "residual", "residual scale")):
            if want is None:
                continue
            same = torch.equal(got.view(torch.uint8), want.view(torch.uint8)) if got.dtype == torch.float8_e5m2 \
                else torch.equal(got, want)
            assert same, f"in place: {name} differ (format {res_fmt}, {resid_scale})"
        st = list(ref[1:])


def test_zero_state_and_empty_batch():
    sq, binding = _mods()
    K = V = 128
    z8 = torch.zeros(1, 1, K, V, dtype=torch.int8, device=DEV)
    zs = torch.zeros(1, 1, V, device=DEV)
    zv = torch.zeros(1, 1, K, device=DEV)
    z1 = torch.zeros(1, 1, device=DEV)
    o, c, s, e, es = binding.gdn_quant_step_cuda(z8, zs, z8.clone(), zs.clone(), zv, zv, zv, z1, z1, 8, 3)
    assert torch.all(c == 0) and torch.all(e == 0) and torch.all(o == 0)
    assert torch.allclose(s.cpu(), torch.full((1, 1, V), 1e-12 / 127))
    empty = binding.gdn_quant_step_cuda(z8[:0], zs[:0], z8[:0].clone(), zs[:0].clone(),
                                        zv[:0], zv[:0], zv[:0], z1[:0], z1[:0], 8, 3)
    assert empty[1].shape == (0, 1, K, V)
