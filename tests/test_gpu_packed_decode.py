"""GPU parity of the slot-indexed (vLLM-layout) call path against the CPU
oracle, plus the reference's own behavioural checks for that path: rounding
ties, padding slots, paging isolation, int4 nibbles
(vllm_integration/test_quantized_packed_decode.py:153-387)."""

from __future__ import annotations

import pytest
import torch

from conftest import load_golden
from oracle import gdn_oracle as orc
import parity
from parity import assert_close, make_packed_inputs

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _qpd():
    from carrykernel_b200.vllm_integration import quantized_packed_decode as qpd
    return qpd


def check_pool(got, ref, resid_fmt, slots, what):
    return parity.check_pool(got, ref, resid_fmt == orc.RESID_INT4, slots, orc.unpack_int4, what)


@pytest.mark.parametrize("shape", [(4, 8, 16, 64, 64), (3, 2, 4, 32, 16), (4, 16, 32, 128, 128)])
@pytest.mark.parametrize("resid_fmt", [orc.RESID_INT8, orc.RESID_INT4])
@pytest.mark.parametrize("rscale", ["v", "head"])
@pytest.mark.parametrize("l2norm", [True, False])
def test_step_vs_oracle_teacher_forced(shape, resid_fmt, rscale, l2norm):
    qpd = _qpd()
    B, H, HV, K, V = shape
    num_slots = 2 * B + 1
    g = torch.Generator().manual_seed(K + V + B)
    pool = torch.randn(num_slots, HV, V, K, generator=g) * 0.1
    ref = list(orc.init_quantized_pool(num_slots, HV, V, K, h0=pool, resid_fmt=resid_fmt,
                                       resid_scale=rscale))
    slots = (torch.randperm(num_slots - 1, generator=g)[:B] + 1).to(torch.int32)
    scale = K ** -0.5
    for t in range(3):
        mixed, a, b, A_log, dt_bias = make_packed_inputs(B, H, HV, K, V, seed=100 + t,
                                                         qk_gain=1.0 if l2norm else K ** -0.5)
        got = [x.clone().to(DEV) for x in ref]          # teacher forcing: start from the oracle's pool
        out_g = torch.full((B, 1, HV, V), float("nan"), device=DEV)
        qpd.quantized_gated_delta_rule_packed_decode(
            mixed.to(DEV), a.to(DEV), b.to(DEV), A_log.to(DEV), dt_bias.to(DEV), scale,
            *got, out_g, slots.to(DEV), use_qk_l2norm_in_kernel=l2norm, resid_fmt=resid_fmt)
        out_r = torch.empty(B, 1, HV, V)
        orc.packed_decode_step(mixed, a, b, A_log, dt_bias, scale, *ref, out_r, slots,
                               use_qk_l2norm_in_kernel=l2norm, resid_fmt=resid_fmt)
        assert_close(out_g.cpu(), out_r, f"t{t}: out")
        check_pool(got, ref, resid_fmt, slots.tolist(), f"{shape} fmt{resid_fmt} {rscale} t{t}")
        untouched = [s for s in range(num_slots) if s not in slots.tolist()]
        for x, y in zip(got, ref):
            assert torch.equal(x.cpu()[untouched], y[untouched]), "a slot outside the batch changed"


def test_bf16_activations_gqa_and_strided_pool():
    """bf16 mixed_qkv / a / b / out, 2 value heads per key head, and a pool whose
    slot stride is larger than one slot (a view into a wider allocation)."""
    qpd = _qpd()
    B, H, HV, K, V = 5, 16, 32, 128, 128
    num_slots = 9
    g = torch.Generator().manual_seed(5)
    pool = torch.randn(num_slots, HV, V, K, generator=g) * 0.1
    ref = list(orc.init_quantized_pool(num_slots, HV, V, K, h0=pool, resid_fmt=orc.RESID_INT4,
                                       resid_scale="head"))
    mixed, a, b, A_log, dt_bias = make_packed_inputs(B, H, HV, K, V, seed=1, dtype=torch.bfloat16)
    slots = torch.tensor([3, 8, 1, 0, 5], dtype=torch.int32)
    # wide allocations: [slots, 2, ...] and keep index 0 of the extra axis
    wide = [torch.zeros((x.shape[0], 2) + tuple(x.shape[1:]), dtype=x.dtype, device=DEV) for x in ref]
    got = [w[:, 0] for w in wide]
    for gdst, r in zip(got, ref):
        gdst.copy_(r)
    assert got[0].stride(0) == 2 * HV * V * K
    out_g = torch.full((B, 1, HV, V), float("nan"), device=DEV, dtype=torch.bfloat16)
    qpd.quantized_gated_delta_rule_packed_decode(
        mixed.to(DEV), a.to(DEV), b.to(DEV), A_log.to(DEV), dt_bias.to(DEV), K ** -0.5,
        *got, out_g, slots.to(DEV), use_qk_l2norm_in_kernel=True, resid_fmt=qpd.RESID_INT4)
    out_r = torch.empty(B, 1, HV, V, dtype=torch.bfloat16)
    orc.packed_decode_step(mixed, a, b, A_log, dt_bias, K ** -0.5, *ref, out_r, slots,
                           use_qk_l2norm_in_kernel=True, resid_fmt=orc.RESID_INT4)
    # bf16 output: one unit in the last place
    assert_close(out_g.cpu(), out_r, "out bf16", rtol=8e-3, atol=1e-4)
    assert torch.all(out_g[3] == 0)
    check_pool([x.contiguous() for x in got], ref, orc.RESID_INT4, [3, 8, 1, 5], "bf16/gqa/strided")
    for w in wide:
        assert torch.all(w[:, 1] == 0), "wrote outside the strided view"


def test_rounding_ties_through_slot_path():
    """Residual codes at scale 0.5 give exact half-integers; the state pins the
    row amax so the derived scale is exactly 1.0; 0 code differences allowed
    (test_quantized_packed_decode.py:211-286)."""
    qpd = _qpd()
    H, HV, K, V = 1, 1, 32, 4
    odd = (torch.arange(K, dtype=torch.float32) % 8) * 2 - 7
    resid_in = odd[None, None, :].repeat(HV, V, 1).contiguous()
    resid_in[..., 0] = 0.0
    state_in = torch.zeros(HV, V, K)
    state_in[..., 0] = 1.0
    target = state_in * 127.0 + resid_in * 0.5
    expected = torch.round(target).clamp(-127, 127)
    n_half = int(((target.abs() % 1.0) == 0.5).sum())
    n_diff = int((torch.floor(target + 0.5).clamp(-127, 127) != expected).sum())
    assert n_half > 0 and n_diff > 0
    sc = torch.zeros(2, HV, V, K, dtype=torch.int8, device=DEV)
    ss = torch.zeros(2, HV, V, device=DEV)
    rc = torch.zeros(2, HV, V, K, dtype=torch.int8, device=DEV)
    rs = torch.zeros(2, HV, V, device=DEV)
    sc[1] = state_in.to(torch.int8)
    ss[1] = 127.0
    rc[1] = resid_in.to(torch.int8)
    rs[1] = 0.5
    mixed = torch.zeros(1, 2 * H * K + HV * V, device=DEV)
    a = torch.full((1, HV), -60.0, device=DEV)
    b = torch.full((1, HV), -60.0, device=DEV)
    out = torch.empty(1, 1, HV, V, device=DEV)
    qpd.quantized_gated_delta_rule_packed_decode(
        mixed, a, b, torch.zeros(HV, device=DEV), torch.zeros(HV, device=DEV), K ** -0.5,
        sc, ss, rc, rs, out, torch.tensor([1], dtype=torch.int32, device=DEV))
    assert torch.equal(sc[1].float().cpu(), expected)
    assert torch.all(ss[1] == 1.0)


def test_null_block_padding():
    qpd = _qpd()
    B, H, HV, K, V = 2, 8, 16, 64, 64
    g = torch.Generator().manual_seed(3)
    pool = torch.randn(3, HV, V, K, generator=g) * 0.1
    st = [x.to(DEV) for x in qpd.init_quantized_state(3, HV, V, K, "cpu", h0=pool)]
    before = [x.clone() for x in st]
    mixed, a, b, A_log, dt_bias = [x.to(DEV) for x in make_packed_inputs(B, H, HV, K, V, seed=7)]
    out = torch.full((B, 1, HV, V), float("nan"), device=DEV)
    qpd.quantized_gated_delta_rule_packed_decode(
        mixed, a, b, A_log, dt_bias, K ** -0.5, *st, out,
        torch.tensor([2, qpd.NULL_BLOCK_ID], dtype=torch.int32, device=DEV))
    assert torch.all(out[1] == 0) and not torch.isnan(out[0]).any()
    for slot in (0, 1):
        for x, y in zip(st, before):
            assert torch.equal(x[slot], y[slot])
    assert not torch.equal(st[0][2], before[0][2])
    # a negative id is padding too
    out.fill_(float("nan"))
    qpd.quantized_gated_delta_rule_packed_decode(
        mixed, a, b, A_log, dt_bias, K ** -0.5, *st, out,
        torch.tensor([-1, -1], dtype=torch.int32, device=DEV))
    assert torch.all(out == 0)


def test_paging_isolation_batched_equals_sequential():
    qpd = _qpd()
    H, HV, K, V = 8, 16, 128, 128
    g = torch.Generator().manual_seed(4)
    pool = torch.randn(5, HV, V, K, generator=g) * 0.1
    mixed, a, b, A_log, dt_bias = [x.to(DEV) for x in make_packed_inputs(2, H, HV, K, V, seed=11)]
    for fmt in (qpd.RESID_INT8, qpd.RESID_INT4):
        st = [x.to(DEV) for x in qpd.init_quantized_state(5, HV, V, K, "cpu", h0=pool, resid_fmt=fmt)]
        out = torch.empty(2, 1, HV, V, device=DEV)
        qpd.quantized_gated_delta_rule_packed_decode(
            mixed, a, b, A_log, dt_bias, K ** -0.5, *st, out,
            torch.tensor([3, 1], dtype=torch.int32, device=DEV), resid_fmt=fmt)
        st2 = [x.to(DEV) for x in qpd.init_quantized_state(5, HV, V, K, "cpu", h0=pool, resid_fmt=fmt)]
        for r, slot in ((0, 3), (1, 1)):
            o1 = torch.empty(1, 1, HV, V, device=DEV)
            qpd.quantized_gated_delta_rule_packed_decode(
                mixed[r:r + 1], a[r:r + 1], b[r:r + 1], A_log, dt_bias, K ** -0.5, *st2, o1,
                torch.tensor([slot], dtype=torch.int32, device=DEV), resid_fmt=fmt)
            assert torch.equal(o1[0], out[r])
        for x, y in zip(st, st2):
            assert torch.equal(x, y)


def test_int4_nibbles_in_range_and_nontrivial():
    qpd = _qpd()
    H, HV, K, V = 4, 4, 32, 8
    g = torch.Generator().manual_seed(6)
    pool = torch.randn(2, HV, V, K, generator=g) * 0.1
    st = [x.to(DEV) for x in qpd.init_quantized_state(2, HV, V, K, "cpu", h0=pool, resid_fmt=qpd.RESID_INT4)]
    assert st[2].shape[-1] == K // 2
    mixed, a, b, A_log, dt_bias = [x.to(DEV) for x in make_packed_inputs(1, H, HV, K, V, seed=5)]
    out = torch.empty(1, 1, HV, V, device=DEV)
    qpd.quantized_gated_delta_rule_packed_decode(
        mixed, a, b, A_log, dt_bias, K ** -0.5, *st, out,
        torch.tensor([1], dtype=torch.int32, device=DEV), resid_fmt=qpd.RESID_INT4)
    codes = orc.unpack_int4(st[2][1].cpu())
    assert int(codes.abs().max()) <= 7 and int((codes != 0).sum()) > 0


@pytest.mark.parametrize("resid_fmt,bound", [(orc.RESID_INT8, 5e-2), (orc.RESID_INT4, 8e-2)])
def test_free_running_decode_vs_reference_vk_oracle(resid_fmt, bound):
    """8 chained steps against the outputs the reference's own [V, K] oracle
    produced (fp32 residual), recorded in the golden file."""
    qpd = _qpd()
    g = load_golden("slot_path")
    H, HV, K, V = 2, 4, 32, 16
    st = [x.to(DEV) for x in qpd.init_quantized_state(5, HV, V, K, "cpu", h0=g["pool"], resid_fmt=resid_fmt)]
    idx = torch.tensor([1], dtype=torch.int32, device=DEV)
    out = torch.empty(1, 1, HV, V, device=DEV)
    outs = []
    for t in range(8):
        qpd.quantized_gated_delta_rule_packed_decode(
            g[f"mixed{t}"].to(DEV), g[f"a{t}"].to(DEV), g[f"b{t}"].to(DEV), g[f"A_log{t}"].to(DEV),
            g[f"dt_bias{t}"].to(DEV), K ** -0.5, *st, out, idx,
            use_qk_l2norm_in_kernel=True, resid_fmt=resid_fmt)
        outs.append(out[0, 0].cpu().clone())
    rel = lambda x, y: ((x - y).norm() / (y.norm() + 1e-12)).item()
    assert rel(torch.stack(outs), g["o_ref"]) < bound
    assert rel(orc.dequant_pool_state(st[0][1].cpu(), st[1][1].cpu()), g["h_ref"]) < bound


def test_out_of_range_slot_is_flagged_not_followed():
    """A slot id beyond the pool is treated as padding and reported through the
    status word; nothing outside the pool is read or written."""
    import ctypes as C
    from carrykernel_b200 import _lib
    qpd = _qpd()
    H, HV, K, V = 2, 4, 32, 16
    st = [x.to(DEV) for x in qpd.init_quantized_state(3, HV, V, K, "cpu")]
    mixed, a, b, A_log, dt_bias = [x.to(DEV) for x in make_packed_inputs(1, H, HV, K, V, seed=5)]
    out = torch.full((1, 1, HV, V), float("nan"), device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    idx = torch.tensor([7], dtype=torch.int32, device=DEV)
    args = _lib.PackedArgs()
    args.mixed_qkv, args.stride_mixed_tok, args.qkv_dtype = mixed.data_ptr(), mixed.stride(0), _lib.F32
    args.a, args.stride_a_tok, args.b, args.stride_b_tok, args.ab_dtype = a.data_ptr(), HV, b.data_ptr(), HV, _lib.F32
    args.A_log, args.A_log_dtype, args.dt_bias, args.dt_bias_dtype = A_log.data_ptr(), _lib.F32, dt_bias.data_ptr(), _lib.F32
    args.scale = K ** -0.5
    args.state_codes, args.state_scale, args.resid_codes, args.resid_scale = [x.data_ptr() for x in st]
    args.stride_state_slot, args.stride_resid_slot = HV * V * K, HV * V * K
    args.stride_sscale_slot, args.stride_rscale_slot = HV * V, HV * V
    args.out, args.out_dtype = out.data_ptr(), _lib.F32
    args.ssm_state_indices, args.stride_indices = idx.data_ptr(), 1
    args.B, args.H, args.HV, args.K, args.V, args.num_slots = 1, H, HV, K, V, 3
    args.use_qk_l2norm, args.res_fmt, args.resid_scale_mode = 0, _lib.RES_INT8, _lib.SCALE_PER_V
    args.eps_mode, args.qmax, args.status = _lib.EPS_ON_SCALE, 127.0, status.data_ptr()
    rc = _lib.load_library().carry_gdn_packed_decode(args, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) & _lib.STATUS_BAD_SLOT
    assert torch.all(out == 0)


@pytest.mark.parametrize("K", [128, 64])
def test_status_word_through_the_public_calls(K):
    """An out-of-range slot id shows up in the optional ``status`` tensor of the Python surfaces (the
    streaming kernel at K = V = 128, the generic one otherwise), for the decode step, the multi-token
    call and the pool calls; ``raise_for_status`` turns it into an exception."""
    qpd = _qpd()
    from carrykernel_b200 import _lib
    from carrykernel_b200.vllm_integration import state_pool
    H, HV, V, num_slots = 2, 4, K, 4
    st = [x.to(DEV) for x in qpd.init_quantized_state(num_slots, HV, V, K, "cpu", resid_fmt=qpd.RESID_INT4,
                                                      resid_scale="head")]
    before = [x.clone() for x in st]
    mixed, a, b, A_log, dt_bias = [x.to(DEV) for x in make_packed_inputs(2, H, HV, K, V, seed=5)]
    idx = torch.tensor([2, num_slots + 3], dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.full((2, 1, HV, V), float("nan"), device=DEV)
    qpd.quantized_gated_delta_rule_packed_decode(mixed, a, b, A_log, dt_bias, K ** -0.5, *st, out, idx,
                                                 use_qk_l2norm_in_kernel=True, resid_fmt=qpd.RESID_INT4, status=status)
    assert int(status.item()) == _lib.STATUS_BAD_SLOT
    assert torch.all(out[1] == 0) and not torch.isnan(out[0]).any()
    for x, y in zip(st, before):
        assert torch.equal(x[[0, 1, 3]], y[[0, 1, 3]])
    with pytest.raises(RuntimeError, match="slot id beyond the pool"):
        _lib.raise_for_status(status, "decode step")
    # a clean call leaves the word alone
    status.zero_()
    qpd.quantized_gated_delta_rule_packed_decode(mixed, a, b, A_log, dt_bias, K ** -0.5, *st, out,
                                                 torch.tensor([1, 0], dtype=torch.int32, device=DEV),
                                                 use_qk_l2norm_in_kernel=True, resid_fmt=qpd.RESID_INT4, status=status)
    _lib.raise_for_status(status)
    # multi-token call
    out_m = torch.empty(2, 2, HV, V, device=DEV)
    qpd.quantized_gated_delta_rule_packed_decode_multi(
        torch.stack([mixed, mixed], 1), torch.stack([a, a], 1), torch.stack([b, b], 1), A_log, dt_bias, K ** -0.5,
        *st, out_m, idx, use_qk_l2norm_in_kernel=True, resid_fmt=qpd.RESID_INT4, status=status)
    assert int(status.item()) == _lib.STATUS_BAD_SLOT and torch.all(out_m[1] == 0)
    # pool calls
    for fn in (lambda s: state_pool.store_state(torch.zeros(2, HV, V, K, device=DEV), st, idx, qpd.RESID_INT4, status=s),
               lambda s: state_pool.load_state(st, idx, resid_fmt=qpd.RESID_INT4, status=s),
               lambda s: state_pool.copy_slots(st, torch.tensor([1, 1], dtype=torch.int32, device=DEV), idx,
                                               resid_fmt=qpd.RESID_INT4, status=s)):
        status.zero_()
        fn(status)
        assert int(status.item()) == _lib.STATUS_BAD_SLOT
