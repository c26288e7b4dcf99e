"""Pool store / load / copy kernels against the CPU oracle: integer results
(codes, packed nibbles) and fp32 results are compared bit for bit -- both sides
use true division and round each product before a sum -- and 16-bit outputs by
their round-to-nearest conversion of the same fp32 values."""

from __future__ import annotations

import pytest
import torch

from oracle import gdn_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _sp():
    from carrykernel_b200.vllm_integration import state_pool
    return state_pool


def _empty_pool(num_slots, HV, V, K, resid_fmt, rscale, fill):
    """A pool whose every byte is `fill`-derived garbage, so untouched slots show."""
    st = list(orc.init_quantized_pool(num_slots, HV, V, K, resid_fmt=resid_fmt, resid_scale=rscale))
    st[0].fill_(fill)
    st[1].fill_(float(fill))
    st[2].fill_(fill)
    st[3].fill_(float(fill))
    return st


def _state(B, HV, V, K, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    h = torch.randn(B, HV, V, K, generator=g) * 0.1
    h[0, 0, 0] = 0.0                       # an all-zero row: the scale floor
    if V > 1:
        h[0, 0, 1] *= 1e-20                # a row below the floor
    if V > 2:                              # a row of exact ties: scale 1, values k + 0.5
        h[0, 0, 2] = (torch.arange(K) % 253 - 126).float() + 0.5
        h[0, 0, 2, 0] = 127.0
    return h.to(dtype)


def _same(got, want):
    for name, g, w in zip(("state_codes", "state_scale", "resid_codes", "resid_scale"), got, want):
        assert torch.equal(g.cpu(), w), f"{name} differs: {(g.cpu() != w).sum().item()} elements"


SHAPES = [(4, 128, 128), (3, 16, 64), (2, 6, 128), (2, 5, 24), (2, 7, 30), (1, 3, 260)]   # (HV, V, K)


@pytest.mark.parametrize("HV,V,K", SHAPES)
@pytest.mark.parametrize("resid_fmt", [orc.RESID_INT8, orc.RESID_INT4])
@pytest.mark.parametrize("rscale", ["v", "head"])
@pytest.mark.parametrize("keep_error", [False, True])
def test_store_matches_oracle(HV, V, K, resid_fmt, rscale, keep_error):
    sp = _sp()
    B, num_slots = 4, 7
    h = _state(B, HV, V, K, seed=K + V, dtype=torch.float32)
    idx = torch.tensor([5, 0, 2, 6], dtype=torch.int32)
    want = _empty_pool(num_slots, HV, V, K, resid_fmt, rscale, fill=3)
    orc.pool_store(h, *want, idx, resid_fmt=resid_fmt, keep_error=keep_error)
    got = [t.to(DEV) for t in _empty_pool(num_slots, HV, V, K, resid_fmt, rscale, fill=3)]
    sp.store_state(h.to(DEV), got, idx.to(DEV), resid_fmt=resid_fmt, keep_error=keep_error)
    torch.cuda.synchronize()
    _same(got, want)
    from carrykernel_b200 import _lib
    assert _lib.load_library().carry_gdn_last_kernel() == 4


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("K", [128, 30])
def test_store_takes_16_bit_states(dtype, K):
    sp = _sp()
    B, HV, V, num_slots = 3, 2, 16, 5
    h = _state(B, HV, V, K, seed=3, dtype=dtype)
    idx = torch.tensor([1, 4, 2], dtype=torch.int32)
    want = _empty_pool(num_slots, HV, V, K, orc.RESID_INT4, "head", fill=1)
    orc.pool_store(h, *want, idx, resid_fmt=orc.RESID_INT4, keep_error=True)
    got = [t.to(DEV) for t in _empty_pool(num_slots, HV, V, K, orc.RESID_INT4, "head", fill=1)]
    sp.store_state(h.to(DEV), got, idx.to(DEV), resid_fmt=orc.RESID_INT4, keep_error=True)
    _same(got, want)


def test_store_equals_init_quantized_state():
    """The hand-off writes what seeding the pool from the same state writes."""
    from carrykernel_b200.vllm_integration import quantized_packed_decode as qpd
    sp = _sp()
    num_slots, HV, V, K = 6, 4, 128, 128
    h0 = _state(num_slots, HV, V, K, seed=9, dtype=torch.float32).to(DEV)
    want = qpd.init_quantized_state(num_slots, HV, V, K, DEV, h0=h0, resid_fmt=qpd.RESID_INT4, resid_scale="head")
    got = qpd.init_quantized_state(num_slots, HV, V, K, DEV, resid_fmt=qpd.RESID_INT4, resid_scale="head")
    idx = torch.arange(1, num_slots, dtype=torch.int32, device=DEV)
    sp.store_state(h0[1:], got, idx, resid_fmt=qpd.RESID_INT4)
    # torch's CUDA division by a constant multiplies by the reciprocal, the kernel
    # divides (like the CPU reference): scales agree to an ulp, codes up to rare ties
    torch.testing.assert_close(got[1][1:], want[1][1:], rtol=2.5e-7, atol=0)
    flips = (got[0][1:].int() - want[0][1:].int()).abs()
    assert int(flips.max()) <= 1 and float((flips > 0).float().mean()) <= 1e-4
    assert torch.equal(got[2][1:], want[2][1:]) and torch.equal(got[3][1:], want[3][1:])
    assert int(got[0][0].abs().max()) == 0          # slot 0 was not named: untouched


@pytest.mark.parametrize("HV,V,K", SHAPES)
@pytest.mark.parametrize("resid_fmt", [orc.RESID_INT8, orc.RESID_INT4])
@pytest.mark.parametrize("rscale", ["v", "head"])
@pytest.mark.parametrize("with_residual", [False, True])
def test_load_matches_oracle(HV, V, K, resid_fmt, rscale, with_residual):
    sp = _sp()
    num_slots = 6
    g = torch.Generator().manual_seed(V * K)
    rk = K // 2 if resid_fmt == orc.RESID_INT4 else K
    pool = [torch.randint(-127, 128, (num_slots, HV, V, K), generator=g, dtype=torch.int8),
            torch.rand(num_slots, HV, V, generator=g) * 1e-2,
            torch.randint(-128, 128, (num_slots, HV, V, rk), generator=g, dtype=torch.int8),
            torch.rand((num_slots, HV, V) if rscale == "v" else (num_slots, HV), generator=g) * 1e-4]
    if resid_fmt == orc.RESID_INT8:
        pool[2].clamp_(min=-127)
    idx = torch.tensor([3, 5, 0, 1], dtype=torch.int32)
    want = orc.pool_load(*pool, idx, resid_fmt=resid_fmt, with_residual=with_residual)
    dpool = [t.to(DEV) for t in pool]
    got = sp.load_state(dpool, idx.to(DEV), resid_fmt=resid_fmt, with_residual=with_residual)
    assert got.dtype == torch.float32 and torch.equal(got.cpu(), want)
    assert float(got[2].abs().max()) == 0.0          # padding request: zeros
    for dtype in (torch.bfloat16, torch.float16):
        out = torch.full((4, HV, V, K), float("nan"), dtype=dtype, device=DEV)
        ret = sp.load_state(dpool, idx.to(DEV), out=out, resid_fmt=resid_fmt, with_residual=with_residual)
        assert ret is out and torch.equal(out.cpu(), want.to(dtype))


@pytest.mark.parametrize("resid_fmt,rscale", [(orc.RESID_INT8, "v"), (orc.RESID_INT4, "head"), (orc.RESID_INT4, "v")])
def test_round_trip_error_bounds(resid_fmt, rscale):
    """store -> load returns the state to within half a state step, and to within
    half a residual step when the quantisation error is kept."""
    sp = _sp()
    B, HV, V, K, num_slots = 8, 4, 128, 128, 9
    h = _state(B, HV, V, K, seed=21, dtype=torch.float32).to(DEV)
    idx = torch.arange(1, B + 1, dtype=torch.int32, device=DEV)
    pool = [t.to(DEV) for t in orc.init_quantized_pool(num_slots, HV, V, K, resid_fmt=resid_fmt, resid_scale=rscale)]
    sp.store_state(h, pool, idx, resid_fmt=resid_fmt, keep_error=False)
    back = sp.load_state(pool, idx, resid_fmt=resid_fmt)
    step = pool[1][1:B + 1][..., None]
    assert bool(((back - h).abs() <= step * 0.5 * (1 + 1e-6) + 1e-30).all())
    plain = (back - h).norm()
    sp.store_state(h, pool, idx, resid_fmt=resid_fmt, keep_error=True)
    back = sp.load_state(pool, idx, resid_fmt=resid_fmt)
    rs = pool[3][1:B + 1]
    rstep = rs[..., None, None] if rscale == "head" else rs[..., None]
    assert bool(((back - h).abs() <= rstep * 0.5 * (1 + 1e-5) + 2e-7 * (h.abs() + 1e-2)).all())   # + fp32 rounding of the sum
    assert float((back - h).norm()) < 0.2 * float(plain)
    without = sp.load_state(pool, idx, resid_fmt=resid_fmt, with_residual=False)
    assert bool(((without - h).abs() <= step * 0.5 * (1 + 1e-6) + 1e-30).all())


@pytest.mark.parametrize("HV,V,K", [(4, 128, 128), (2, 5, 30)])
@pytest.mark.parametrize("resid_fmt,rscale", [(orc.RESID_INT8, "v"), (orc.RESID_INT4, "head")])
def test_copy_slots(HV, V, K, resid_fmt, rscale):
    sp = _sp()
    num_slots = 8
    g = torch.Generator().manual_seed(5)
    rk = K // 2 if resid_fmt == orc.RESID_INT4 else K

    def rand_pool(n):
        return [torch.randint(-127, 128, (n, HV, V, K), generator=g, dtype=torch.int8),
                torch.rand(n, HV, V, generator=g),
                torch.randint(-127, 128, (n, HV, V, rk), generator=g, dtype=torch.int8),
                torch.rand((n, HV, V) if rscale == "v" else (n, HV), generator=g)]

    # within one pool (prefix reuse / checkpoint)
    pool = rand_pool(num_slots)
    src = torch.tensor([1, 2, 0, 3, 7], dtype=torch.int32)
    dst = torch.tensor([4, 5, 6, 0, 7], dtype=torch.int32)     # two padded pairs, one slot onto itself
    want = [t.clone() for t in pool]
    orc.pool_copy(pool, want, src, dst)
    got = [t.to(DEV) for t in pool]
    sp.copy_slots(got, src.to(DEV), dst.to(DEV), resid_fmt=resid_fmt)
    _same(got, want)
    # into a second, smaller pool with its own slot stride (spill pool)
    spill_cpu = rand_pool(4)
    want2 = [t.clone() for t in spill_cpu]
    src2 = torch.tensor([6, 1], dtype=torch.int32)
    dst2 = torch.tensor([1, 3], dtype=torch.int32)
    orc.pool_copy(want, want2, src2, dst2)
    spill = [t.to(DEV) for t in spill_cpu]
    sp.copy_slots(got, src2.to(DEV), dst2.to(DEV), dst_pool=spill, resid_fmt=resid_fmt)
    _same(spill, want2)
    _same(got, want)                                            # the source is not written


def _padded(t, pad):
    """The same values in a tensor whose slot stride is `pad` elements longer."""
    n = t.shape[0]
    inner = t[0].numel()
    big = torch.zeros(n, inner + pad, dtype=t.dtype, device=t.device)
    view = big[:, :inner].view(t.shape)
    view.copy_(t)
    return view


@pytest.mark.parametrize("pad_scale", [4, 1])       # 1: scale rows off the 16-byte grid -> scalar variant
@pytest.mark.parametrize("resid_fmt,rscale", [(orc.RESID_INT4, "head"), (orc.RESID_INT8, "v")])
def test_strided_pools(pad_scale, resid_fmt, rscale):
    sp = _sp()
    B, HV, V, K, num_slots = 3, 2, 128, 128, 5
    h = _state(B, HV, V, K, seed=17, dtype=torch.float32)
    idx = torch.tensor([4, 1, 3], dtype=torch.int32)
    want = _empty_pool(num_slots, HV, V, K, resid_fmt, rscale, fill=1)
    orc.pool_store(h, *want, idx, resid_fmt=resid_fmt, keep_error=True)
    pads = (64, pad_scale, 32, pad_scale)
    got = [_padded(t.to(DEV), p) for t, p in zip(_empty_pool(num_slots, HV, V, K, resid_fmt, rscale, fill=1), pads)]
    assert not got[0].is_contiguous()
    sp.store_state(h.to(DEV), got, idx.to(DEV), resid_fmt=resid_fmt, keep_error=True)
    _same(got, want)
    back = sp.load_state(got, idx.to(DEV), resid_fmt=resid_fmt)
    assert torch.equal(back.cpu(), orc.pool_load(*want, idx, resid_fmt=resid_fmt))
    spill = [_padded(torch.zeros_like(t[:3]).to(DEV), p) for t, p in zip(want, pads)]
    sp.copy_slots(got, idx.to(DEV), torch.tensor([1, 2, 0], dtype=torch.int32, device=DEV), dst_pool=spill,
                  resid_fmt=resid_fmt)
    for g, w in zip(spill, want):
        assert torch.equal(g[1].cpu(), w[4]) and torch.equal(g[2].cpu(), w[1])

def test_hand_off_then_decode_matches_oracle():
    """prefill hand-off -> one decode step, end to end against the oracle."""
    import parity
    from carrykernel_b200.vllm_integration import quantized_packed_decode as qpd
    sp = _sp()
    B, H, HV, K, V, num_slots = 3, 2, 4, 128, 128, 5
    g = torch.Generator().manual_seed(31)
    h = torch.randn(B, HV, V, K, generator=g) * 0.1
    mixed = torch.randn(B, 2 * H * K + HV * V, generator=g).bfloat16()
    a = (torch.randn(B, HV, generator=g) * 0.5).bfloat16()
    b = torch.randn(B, HV, generator=g).bfloat16()
    A_log = torch.randn(HV, generator=g) * 0.2
    dt_bias = torch.randn(HV, generator=g) * 0.1
    idx = torch.tensor([2, 4, 1], dtype=torch.int32)
    want = list(orc.init_quantized_pool(num_slots, HV, V, K, resid_fmt=orc.RESID_INT4, resid_scale="head"))
    orc.pool_store(h, *want, idx, resid_fmt=orc.RESID_INT4, keep_error=True)
    got = [t.to(DEV) for t in orc.init_quantized_pool(num_slots, HV, V, K, resid_fmt=orc.RESID_INT4, resid_scale="head")]
    sp.store_state(h.to(DEV), got, idx.to(DEV), resid_fmt=qpd.RESID_INT4, keep_error=True)
    _same(got, want)
    out_w = torch.empty(B, 1, HV, V, dtype=torch.bfloat16)
    orc.packed_decode_step(mixed, a, b, A_log, dt_bias, K ** -0.5, *want, out_w, idx,
                           use_qk_l2norm_in_kernel=True, resid_fmt=orc.RESID_INT4)
    out_g = torch.empty(B, 1, HV, V, dtype=torch.bfloat16, device=DEV)
    qpd.quantized_gated_delta_rule_packed_decode(
        mixed.to(DEV), a.to(DEV), b.to(DEV), A_log.to(DEV), dt_bias.to(DEV), K ** -0.5, *got, out_g,
        idx.to(DEV), use_qk_l2norm_in_kernel=True, resid_fmt=qpd.RESID_INT4)
    parity.check_pool(got, want, True, idx.tolist(), orc.unpack_int4, what="hand-off + step")
    parity.assert_close(out_g.cpu().float(), out_w.float(), "hand-off + step: o", rtol=8e-3, atol=1e-4)

def test_bad_slot_is_flagged_not_written():
    """A slot id beyond the pool is skipped (C ABI status word)."""
    from carrykernel_b200 import _lib
    sp = _sp()
    HV, V, K, num_slots = 2, 8, 32, 3
    pool = [t.to(DEV) for t in _empty_pool(num_slots, HV, V, K, orc.RESID_INT8, "v", fill=2)]
    before = [t.clone() for t in pool]
    h = torch.randn(1, HV, V, K, device=DEV)
    idx = torch.tensor([9], dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    args = _lib.PoolStoreArgs()
    args.pool = sp._pool_struct(pool, orc.RESID_INT8)
    args.h, args.stride_h_req, args.h_dtype = h.data_ptr(), h.stride(0), _lib.F32
    args.slots, args.stride_slots, args.B = idx.data_ptr(), 1, 1
    args.keep_error, args.qmax, args.status = 0, 127.0, status.data_ptr()
    rc = _lib.load_library().carry_gdn_pool_store(args, _lib.current_stream_ptr(torch.device(DEV)))
    torch.cuda.synchronize()
    assert rc == 0 and int(status) == _lib.STATUS_BAD_SLOT
    for b4, now in zip(before, pool):
        assert torch.equal(b4, now)
