"""CPU-only checks of the boundary: the C-ABI library loads and exports what the
header declares, argument errors come back as codes (no kernel is launched),
and the Python surfaces keep the reference's names, defaults and exceptions."""

from __future__ import annotations

import ctypes as C
import inspect
import os
import re

import pytest
import torch

from conftest import ROOT
from oracle import gdn_oracle as orc

from carrykernel_b200 import _build, _lib
from carrykernel_b200.cuda import binding
from carrykernel_b200.statequant import kernel as sq
from carrykernel_b200.vllm_integration import quantized_packed_decode as qpd


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(_lib.LIB_PATH):
        _build.build()
    return _lib.load_library()


def test_header_symbols_are_exported(lib):
    header = open(os.path.join(ROOT, "include", "carry_gdn.h")).read()
    declared = set(re.findall(r"\b(carry_gdn_[a-z0-9_]+)\s*\(", header))
    assert {"carry_gdn_quant_step", "carry_gdn_fp32_step", "carry_gdn_packed_decode",
            "carry_gdn_strerror", "carry_gdn_abi_version"} <= declared
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert lib.carry_gdn_abi_version() == int(re.search(r"CARRY_GDN_ABI_VERSION (\d+)", header).group(1))


def test_struct_sizes_match_header_layout():
    # pointers 8, int64 8, int32/float 4, natural alignment: field counts from the header
    assert C.sizeof(_lib.StepArgs) == 14 * 8 + 11 * 4 + 4 + 8
    assert C.sizeof(_lib.Fp32Args) == 8 * 8 + 6 * 4
    assert C.sizeof(_lib.PackedArgs) % 8 == 0
    assert C.sizeof(_lib.PackedMultiArgs) == C.sizeof(_lib.PackedArgs) + 8 + 3 * 8
    assert C.sizeof(_lib.Pool) == 4 * 8 + 4 * 8 + 6 * 4
    assert C.sizeof(_lib.PoolStoreArgs) == C.sizeof(_lib.Pool) + 8 + 8 + 8 + 8 + 8 + 4 * 4 + 8
    assert C.sizeof(_lib.PoolLoadArgs) == C.sizeof(_lib.Pool) + 8 + 8 + 8 + 8 + 8 + 2 * 4 + 8
    assert C.sizeof(_lib.PoolCopyArgs) == 2 * C.sizeof(_lib.Pool) + 4 * 8 + 8 + 8


def test_argument_errors_return_codes_without_a_gpu(lib):
    assert lib.carry_gdn_quant_step(None, None) == -1
    assert lib.carry_gdn_fp32_step(None, None) == -1
    assert lib.carry_gdn_packed_decode(None, None) == -1
    assert lib.carry_gdn_packed_decode_multi(None, None) == -1
    m = _lib.PackedMultiArgs()
    m.T = 0
    assert lib.carry_gdn_packed_decode_multi(C.byref(m), None) == -2
    a = _lib.StepArgs()
    a.B, a.HV, a.K, a.V, a.qmax = 1, 1, 0, 128, 127.0
    assert lib.carry_gdn_quant_step(a, None) == -2          # K <= 0
    a.K = 128
    a.qkv_dtype = 9
    assert lib.carry_gdn_quant_step(a, None) == -3          # unknown dtype
    a.qkv_dtype = 0
    a.res_fmt = 17
    assert lib.carry_gdn_quant_step(a, None) == -4          # unknown residual format
    a.res_fmt = _lib.RES_INT4
    a.V = 127
    assert lib.carry_gdn_quant_step(a, None) == -4          # int4 needs an even contiguous length
    a.V = 128
    assert lib.carry_gdn_quant_step(a, None) == -1          # pointers missing
    a.B = 0
    assert lib.carry_gdn_quant_step(a, None) == 0           # empty batch is a no-op
    p = _lib.PackedArgs()
    p.B, p.H, p.HV, p.K, p.V, p.qmax = 1, 3, 4, 32, 16, 127.0
    assert lib.carry_gdn_packed_decode(p, None) == -2       # HV not a multiple of H
    p.H = 2
    p.res_fmt = _lib.RES_FP32
    assert lib.carry_gdn_packed_decode(p, None) == -4       # slot path is int8/int4 only
    for fn in (lib.carry_gdn_pool_store, lib.carry_gdn_pool_load, lib.carry_gdn_pool_copy):
        assert fn(None, None) == -1
    st = _lib.PoolStoreArgs()
    st.B, st.qmax = 1, 127.0
    assert lib.carry_gdn_pool_store(st, None) == -2         # empty head shape
    st.pool.HV, st.pool.V, st.pool.K = 2, 4, 7
    st.pool.res_fmt = _lib.RES_FP16
    assert lib.carry_gdn_pool_store(st, None) == -4         # the pool holds int8 / int4 residuals only
    st.pool.res_fmt = _lib.RES_INT4
    assert lib.carry_gdn_pool_store(st, None) == -4         # int4 needs an even K
    st.pool.K = 8
    st.h_dtype = 7
    assert lib.carry_gdn_pool_store(st, None) == -3
    st.h_dtype = 0
    assert lib.carry_gdn_pool_store(st, None) == -1         # pointers missing
    st.B = 0
    assert lib.carry_gdn_pool_store(st, None) == 0
    cp = _lib.PoolCopyArgs()
    cp.B = 1
    cp.src.HV, cp.src.V, cp.src.K, cp.src.res_fmt = 2, 4, 8, _lib.RES_INT8
    cp.dst.HV, cp.dst.V, cp.dst.K, cp.dst.res_fmt = 2, 4, 16, _lib.RES_INT8
    assert lib.carry_gdn_pool_copy(cp, None) == -2          # head shapes differ
    cp.dst.K, cp.dst.res_fmt = 8, _lib.RES_INT4
    assert lib.carry_gdn_pool_copy(cp, None) == -4          # residual formats differ
    assert b"NULL" in lib.carry_gdn_strerror(-1)
    assert lib.carry_gdn_strerror(-99) == b"unknown error code"


def test_reference_signatures_are_kept():
    ps = list(inspect.signature(sq.gdn_quant_step_fused).parameters)
    assert ps[:12] == ["h_int8", "scale", "e", "e_scale", "q", "k", "v", "alpha", "beta",
                       "bits", "res_fmt", "BLOCK_V"]
    d = inspect.signature(sq.gdn_quant_step_fused).parameters
    assert d["bits"].default == 8 and d["res_fmt"].default == sq.RES_FP32 and d["BLOCK_V"].default == 32
    assert inspect.signature(binding.gdn_quant_step_cuda).parameters["BLOCK_V"].default == 128
    assert list(inspect.signature(sq.gdn_step_fused_fp32).parameters) == \
        ["h", "q", "k", "v", "alpha", "beta", "BLOCK_V"]
    assert list(inspect.signature(binding.gdn_quant_decode_cuda).parameters)[:10] == \
        ["h0", "q", "k", "v", "alpha", "beta", "T", "bits", "res_fmt", "BLOCK_V"]
    ps = inspect.signature(qpd.quantized_gated_delta_rule_packed_decode).parameters
    assert list(ps)[:14] == [
        "mixed_qkv", "a", "b", "A_log", "dt_bias", "scale", "state_codes", "state_scale",
        "resid_codes", "resid_scale", "out", "ssm_state_indices", "use_qk_l2norm_in_kernel",
        "resid_fmt"]
    assert list(ps)[14:] == ["status"] and ps["status"].default is None      # additive, optional
    assert (sq.RES_FP32, sq.RES_FP16, sq.RES_FP8, sq.RES_INT8) == (0, 1, 2, 3)
    assert (qpd.RESID_INT8, qpd.RESID_INT4, qpd.NULL_BLOCK_ID) == (0, 1, 0)
    assert issubclass(binding.CudaUnavailable, RuntimeError)
    assert sq.residual_bytes(sq.RES_FP16) == 2 and sq.residual_label(sq.RES_INT8) == "int8"
    assert sq.residual_dtype(sq.RES_FP8) == torch.float8_e5m2


def test_no_cpu_path():
    h0 = torch.randn(1, 1, 16, 16)
    st = sq.init_quant_state(h0, 8, sq.RES_INT8)
    z = torch.zeros(1, 1, 16)
    with pytest.raises(sq.CudaUnavailable):
        sq.gdn_quant_step_fused(*st, z, z, z, torch.ones(1, 1), torch.ones(1, 1), res_fmt=sq.RES_INT8)
    with pytest.raises(AssertionError):
        sq.gdn_quant_step_fused(st[0].float(), *st[1:], z, z, z, torch.ones(1, 1), torch.ones(1, 1))
    with pytest.raises(AssertionError):
        sq.gdn_quant_step_fused(st[0][0], *st[1:], z, z, z, torch.ones(1, 1), torch.ones(1, 1))
    if not torch.cuda.is_available():
        with pytest.raises(binding.CudaUnavailable):
            binding.load_extension()


def test_state_pool_validation_messages():
    from carrykernel_b200.vllm_integration import state_pool as sp
    pool = qpd.init_quantized_state(3, 2, 4, 8, "cpu", resid_fmt=qpd.RESID_INT4)
    idx = torch.tensor([1], dtype=torch.int32)
    h = torch.zeros(1, 2, 4, 8)
    with pytest.raises(ValueError, match="packed two codes per byte"):
        sp.store_state(h, (pool[0], pool[1], pool[0], pool[3]), idx, resid_fmt=qpd.RESID_INT4)
    with pytest.raises(ValueError, match="same shape as the state"):
        sp.store_state(h, pool, idx, resid_fmt=qpd.RESID_INT8)
    with pytest.raises(ValueError, match="unknown residual format"):
        sp.load_state(pool, idx, resid_fmt=9)
    with pytest.raises(sp._lib.CudaUnavailable):             # no CPU path
        sp.store_state(h, pool, idx, resid_fmt=qpd.RESID_INT4)


def test_pool_oracle_round_trip():
    """store -> load on the CPU oracle: the kept error brings the state back to
    within half a residual step; copy moves all four tensors."""
    g = torch.Generator().manual_seed(2)
    h = torch.randn(2, 2, 6, 16, generator=g)
    idx = torch.tensor([2, 1], dtype=torch.int32)
    for fmt, rscale in ((orc.RESID_INT8, "v"), (orc.RESID_INT4, "head")):
        pool = list(orc.init_quantized_pool(4, 2, 6, 16, resid_fmt=fmt, resid_scale=rscale))
        orc.pool_store(h, *pool, idx, resid_fmt=fmt, keep_error=False)
        ref = orc.init_quantized_pool(4, 2, 6, 16, h0=torch.cat([h[:1] * 0, h[1:2], h[0:1], h[:1] * 0]),
                                      resid_fmt=fmt, resid_scale=rscale)
        for a, b in zip(pool, ref):
            assert torch.equal(a[1:3], b[1:3])
        orc.pool_store(h, *pool, idx, resid_fmt=fmt, keep_error=True)
        back = orc.pool_load(*pool, idx, resid_fmt=fmt)
        rs = pool[3][idx.long()]
        step = rs[..., None, None] if rscale == "head" else rs[..., None]
        assert bool(((back - h).abs() <= 0.5 * step * (1 + 1e-5) + 1e-9).all())
        spill = [torch.zeros_like(t[:2]) for t in pool]
        orc.pool_copy(pool, spill, torch.tensor([2]), torch.tensor([1]))
        for a, b in zip(pool, spill):
            assert torch.equal(a[2], b[1]) and not b[0].any()


def test_init_matches_oracle():
    torch.manual_seed(0)
    h0 = torch.randn(2, 3, 32, 16) * 0.3
    for fmt in (0, 1, 2, 3, 4):
        for rs in ("v", "head"):
            a = sq.init_quant_state(h0, 8, fmt, rs)
            b = orc.init_quant_state(h0, 8, fmt, rs)
            for x, y in zip(a, b):
                assert (x is None and y is None) or (x.dtype == y.dtype and x.shape == y.shape
                                                     and torch.equal(x.float(), y.float()))
    pool = torch.randn(4, 3, 16, 32) * 0.1
    for fmt in (qpd.RESID_INT8, qpd.RESID_INT4):
        for rs in ("v", "head"):
            a = qpd.init_quantized_state(4, 3, 16, 32, "cpu", h0=pool, resid_fmt=fmt, resid_scale=rs)
            b = orc.init_quantized_pool(4, 3, 16, 32, h0=pool, resid_fmt=fmt, resid_scale=rs)
            for x, y in zip(a, b):
                assert x.shape == y.shape and torch.equal(x, y)


def test_bytes_per_slot():
    f = qpd.state_bytes_per_slot
    assert f(32, 128, 128, False, 4) == 2097152
    assert f(32, 128, 128, False, 2) == 1048576
    assert f(32, 128, 128, True, resid_fmt=qpd.RESID_INT8) == 1081344
    assert f(32, 128, 128, True, resid_fmt=qpd.RESID_INT4) == 819200
    assert f(32, 128, 128, True, resid_fmt=qpd.RESID_INT4, resid_scale="head") == 819200 - 32 * 127 * 4


def test_packed_decode_validation_messages():
    HV, V, K, H, B = 4, 16, 32, 2, 2
    sc, ss, rc, rs = qpd.init_quantized_state(3, HV, V, K, "cpu")
    mixed = torch.zeros(B, 2 * H * K + HV * V)
    a = b = torch.zeros(B, HV)
    A = d = torch.zeros(HV)
    out = torch.zeros(B, 1, HV, V)
    idx = torch.tensor([1, 2], dtype=torch.int32)
    call = lambda **kw: qpd.quantized_gated_delta_rule_packed_decode(**{**dict(
        mixed_qkv=mixed, a=a, b=b, A_log=A, dt_bias=d, scale=1.0, state_codes=sc, state_scale=ss,
        resid_codes=rc, resid_scale=rs, out=out, ssm_state_indices=idx), **kw})
    with pytest.raises(ValueError, match="2-D"):
        call(mixed_qkv=mixed[0])
    with pytest.raises(ValueError, match="4-D"):
        call(state_codes=sc[0])
    with pytest.raises(ValueError, match="int8 storage"):
        call(state_codes=sc.float())
    with pytest.raises(ValueError, match="packed two codes per byte"):
        call(resid_fmt=qpd.RESID_INT4)
    with pytest.raises(ValueError, match="same shape"):
        call(resid_codes=rc[..., :16])
    with pytest.raises(ValueError, match="1-D"):
        call(ssm_state_indices=idx[None])
    with pytest.raises(ValueError, match="int32"):
        call(ssm_state_indices=idx.long())
    with pytest.raises(ValueError, match="out must be"):
        call(out=out[:, :, :2])
    with pytest.raises(ValueError, match="cannot infer H"):
        call(mixed_qkv=torch.zeros(B, HV * V + 3))
    # sizes the kernel would index past, and tensors that are not on the pool's device: rejected
    # before anything is launched (the kernels take raw addresses)
    with pytest.raises(ValueError, match=r"a must be \(2, 4\)"):
        call(a=torch.zeros(B, HV - 1))
    with pytest.raises(ValueError, match=r"b must be \(2, 4\)"):
        call(b=torch.zeros(B + 1, HV))
    with pytest.raises(ValueError, match="A_log must be"):
        call(A_log=torch.zeros(HV + 1))
    with pytest.raises(ValueError, match="dt_bias must be"):
        call(dt_bias=torch.zeros(1))
    with pytest.raises(ValueError, match="contiguous"):
        call(A_log=torch.zeros(2 * HV)[::2])
    with pytest.raises(ValueError, match="ssm_state_indices must be"):
        call(ssm_state_indices=idx[:1])
    with pytest.raises(ValueError, match="state_scale must be"):
        call(state_scale=ss[:2])
    with pytest.raises(ValueError, match="resid_scale must be"):
        call(resid_scale=rs[:, :2])
    rc4 = qpd.init_quantized_state(2, HV, V, K, "cpu", resid_fmt=qpd.RESID_INT4)[2]
    with pytest.raises(ValueError, match="resid_codes must be"):
        call(resid_codes=rc4, resid_fmt=qpd.RESID_INT4)        # a residual pool of fewer slots than the state's
    with pytest.raises(ValueError, match="share a dtype"):
        call(a=a.bfloat16())
    with pytest.raises(ValueError, match="ssm_state_indices is on meta"):
        call(ssm_state_indices=torch.zeros(B, dtype=torch.int32, device="meta"))
    with pytest.raises(ValueError, match="mixed_qkv is on meta"):
        call(mixed_qkv=torch.zeros(mixed.shape, device="meta"))
    with pytest.raises(ValueError, match="status must be an int32"):
        call(status=torch.zeros(1))
    with pytest.raises(qpd.CudaUnavailable):
        call()


def test_statequant_validation_messages():
    B, HV, K, V = 2, 3, 16, 8
    st = sq.init_quant_state(torch.randn(B, HV, K, V), 8, sq.RES_INT8)
    q = k = torch.zeros(B, HV, K)
    v = torch.zeros(B, HV, V)
    al = be = torch.ones(B, HV)
    base = dict(q=q, k=k, v=v, alpha=al, beta=be)
    call = lambda st_=st, **kw: sq.gdn_quant_step_fused(*st_, **{**base, **kw}, res_fmt=sq.RES_INT8)
    with pytest.raises(ValueError, match="q must be"):
        call(q=q[:, :2])
    with pytest.raises(ValueError, match="v must be"):
        call(v=q)
    with pytest.raises(ValueError, match="alpha must be"):
        call(alpha=al[0])
    with pytest.raises(ValueError, match="scale must be"):
        call((st[0], st[1][:, :, :4], st[2], st[3]))
    with pytest.raises(ValueError, match="e must be"):
        call((st[0], st[1], st[2][:, :, :8], st[3]))
    with pytest.raises(ValueError, match="k is on meta"):
        call(k=torch.zeros(B, HV, K, device="meta"))
    with pytest.raises(ValueError, match="beta must be"):
        sq.gdn_step_fused_fp32(torch.zeros(B, HV, K, V), q, k, v, al, be[:1])


@pytest.mark.parametrize("qmax", [3, 7, 15, 31, 63, 127])
def test_scale_division_shortcut_is_exact(qmax):
    """The streaming kernel computes amax / qmax as q0 = amax * (1/qmax), then
    fma(fma(-qmax, q0, amax), 1/qmax, q0) (carry_gdn_tile128.cuh, div_qmax).
    For these qmax that equals the IEEE quotient for every mantissa; float64
    emulates each float32 FMA here without a second rounding (all products of
    two float32 are exact in float64, and so are the two sums for operands this
    close)."""
    import numpy as np
    y = np.float32(1.0) / np.float32(qmax)
    for exp in (-40, 0, 60):                          # the identity does not depend on the binade
        bits = (np.uint32((exp + 127) << 23) | np.arange(1 << 23, dtype=np.uint32))
        a = bits.view(np.float32)
        a64 = a.astype(np.float64)
        want = (a64 / float(qmax)).astype(np.float32)
        q0 = (a64 * float(y)).astype(np.float32)
        r = (a64 - float(qmax) * q0.astype(np.float64)).astype(np.float32)
        got = (q0.astype(np.float64) + r.astype(np.float64) * float(y)).astype(np.float32)
        assert np.array_equal(got, want)
        # float64 division then rounding to float32 is the float32 quotient: a double rounding could
        # only bite when the float64 quotient sits exactly on a float32 tie, which a/qmax with a 24-bit
        # a and qmax < 2^7 cannot do unless it is exact
