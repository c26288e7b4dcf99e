"""Parity protocol shared by the GPU tests, ``smoke()`` and the benchmark's
validate-before-time step.

The bar (fp32 accumulate on both sides):

* state codes equal the oracle's except for at most ``MAX_FLIP_FRAC`` of the
  elements, each of those off by exactly one code (a rounding tie that the
  reduction order of ``h^T k`` pushed to the other side);
* residual codes likewise, not counting elements whose *state* code flipped --
  there the new residual legitimately changes sign at about half a state step,
  so its code may move across the whole grid;
* ``o`` and the dequantised state within ``rtol 1e-3 / atol 1e-4``; at a flipped
  element the dequantised state may be off by one state step;
* a V channel whose whole new residual is below 0.1 % of a state step (the
  target happened to be representable almost exactly) carries nothing but fp32
  rounding noise in its residual; there the residual codes and scale are not
  compared, only the dequantised value;
* state scales within ``rtol 1e-5``; residual scales within ``rtol 5e-4``: the
  new residual is ``target - code*scale``, a difference of nearly equal numbers,
  so one unit in the last place of the state scale (3e-7 relative, from the
  reduction order of the row maximum's own target) moves the residual -- about
  1/254 of the target -- by up to 1e-4 relative; on top of that two units in the
  last place of the target itself (:func:`target_ulp_in_scale`), which is what
  counts in a channel whose residual is a small fraction of a state step.
"""

from __future__ import annotations

import torch

MAX_FLIP_FRAC = 1e-3
RTOL, ATOL = 1e-3, 1e-4
STATE_SCALE_RTOL = 1e-5
RESID_SCALE_RTOL = 5e-4


def seeded_inputs(B, HV, K, V, seed=0, T=None, dtype=torch.float32, alpha_mode="const"):
    """Input law of the reference's kernel tests (k L2-normalised, q raw,
    ``h0 = 0.1 N(0,1)``).  ``alpha_mode='gated'`` draws the per-token per-head
    decay ``exp(-0.1 softplus(N(0,1)))`` and ``beta = sigmoid(N(0,1))`` and
    also normalises q (the serving configurations)."""
    g = torch.Generator().manual_seed(seed)
    lead = (B, HV) if T is None else (T, B, HV)
    q = torch.randn(*lead, K, generator=g)
    k = torch.randn(*lead, K, generator=g)
    k = k / k.norm(dim=-1, keepdim=True).clamp(min=1e-8)
    v = torch.randn(*lead, V, generator=g)
    if alpha_mode == "const":
        alpha = torch.full(lead, 0.995)
        beta = torch.rand(*lead, generator=g).sigmoid()
    else:
        q = q / q.norm(dim=-1, keepdim=True).clamp(min=1e-8)
        alpha = torch.exp(-0.1 * torch.nn.functional.softplus(torch.randn(*lead, generator=g)))
        beta = torch.sigmoid(torch.randn(*lead, generator=g))
    h0 = torch.randn(B, HV, K, V, generator=g) * 0.1
    return h0, q.to(dtype), k.to(dtype), v.to(dtype), alpha, beta


def make_packed_inputs(B, H, HV, K, V, seed, dtype=torch.float32, qk_gain=1.0):
    """Packed activations and gates (recipe of the reference's slot-path tests).
    ``qk_gain`` scales q and k: with the in-kernel L2 norm off, raw N(0,1) keys of
    norm ~sqrt(K) make ``v - h^T k`` cancel badly and the step ill-conditioned, so
    the oracle comparisons without the norm use ``K**-0.5``."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, H, K, generator=g) * qk_gain
    k = torch.randn(B, H, K, generator=g) * qk_gain
    v = torch.randn(B, HV, V, generator=g)
    mixed = torch.cat([q.reshape(B, -1), k.reshape(B, -1), v.reshape(B, -1)], dim=1).contiguous()
    a = torch.randn(B, HV, generator=g) * 0.5
    b = torch.randn(B, HV, generator=g)
    A_log = torch.randn(HV, generator=g) * 0.2
    dt_bias = torch.randn(HV, generator=g) * 0.1
    return mixed.to(dtype), a.to(dtype), b.to(dtype), A_log, dt_bias


def config1_inputs():
    """The CPU mechanism configuration (number 1 of the named workloads): batch 1, 4 heads, K = V = 128, T = 2000, constant decay 0.995, q and k
    ~ N(0,1) L2-normalised per head, v ~ N(0,1), beta = sigmoid(N(0,1)), ``torch.manual_seed(0)``,
    drawn in the order of the reference's experiments/exp2b_granularity.py:49-56 (the same draws as
    ``tests/golden/make_golden.py:config1``).  Returns ``(h0, q, k, v, alpha, beta, input_sums)``."""
    state = torch.random.get_rng_state()
    torch.manual_seed(0)
    HV, K, V, T = 4, 128, 128, 2000
    q = torch.randn(T, HV, K); q = q / q.norm(dim=-1, keepdim=True).clamp(min=1e-8)
    k = torch.randn(T, HV, K); k = k / k.norm(dim=-1, keepdim=True).clamp(min=1e-8)
    v = torch.randn(T, HV, V)
    alpha = torch.full((T, HV), 0.995)
    beta = torch.randn(T, HV).sigmoid()
    h0 = torch.randn(HV, K, V) * 0.1
    torch.random.set_rng_state(state)
    sums = torch.tensor([x.double().sum().item() for x in (q, k, v, beta, h0)], dtype=torch.float64)
    return h0, q, k, v, alpha, beta, sums


def code_flips(got: torch.Tensor, ref: torch.Tensor):
    """Returns ``(mask_of_differing, fraction, max_abs_diff)`` for integer codes."""
    d = (got.to(torch.int32) - ref.to(torch.int32)).abs()
    mask = d > 0
    return mask, mask.float().mean().item(), int(d.max()) if d.numel() else 0


def assert_codes(got, ref, what, max_frac=MAX_FLIP_FRAC, exclude=None):
    mask, frac, dmax = code_flips(got, ref)
    if exclude is not None:
        keep = ~exclude
        d = (got.to(torch.int32) - ref.to(torch.int32)).abs()[keep]
        frac = (d > 0).float().mean().item() if d.numel() else 0.0
        dmax = int(d.max()) if d.numel() else 0
    assert dmax <= 1, f"{what}: a code differs by {dmax} (> 1 step)"
    assert frac <= max_frac, f"{what}: {frac:.2e} of codes differ (limit {max_frac:.0e})"
    return mask, frac


def assert_close(got, ref, what, rtol=RTOL, atol=ATOL, exclude=None, slack=None):
    got, ref = got.float(), ref.float()
    err = (got - ref).abs()
    tol = atol + rtol * ref.abs()
    if slack is not None:          # per-element extra allowance (e.g. one state step at flips)
        tol = tol + slack
    bad = err > tol
    if exclude is not None:
        bad = bad & ~exclude
    assert not bool(bad.any()), (
        f"{what}: {int(bad.sum())} elements out of tolerance, worst abs err "
        f"{err[bad].max().item():.3e}")


def target_ulp_in_scale(state_scale, rq):
    """What two units in the last place of the largest target of a channel (127 state steps) come to
    in its residual scale: the residual is target - code * scale, so the reduction order of the dot
    products moves it by that much whatever its own size, which shows in channels whose whole
    residual is a small fraction of a state step."""
    return 2.0 ** -22 * 127.0 / rq * state_scale


def check_quant_step(got, ref, res_fmt, unpack_int4=None, int_formats=(3, 4),
                     what="step", max_frac=MAX_FLIP_FRAC):
    """Compare one fused step ``(o, codes, scale, e, e_scale)`` in the
    statequant layout.  Returns a dict of measured flip fractions."""
    o_g, c_g, s_g, e_g, es_g = [None if x is None else x.cpu() for x in got]
    o_r, c_r, s_r, e_r, es_r = ref
    assert_close(o_g, o_r, f"{what}: o")
    torch.testing.assert_close(s_g, s_r, rtol=STATE_SCALE_RTOL, atol=1e-30, msg=f"{what}: state scale")
    flip, frac_state = assert_codes(c_g, c_r, f"{what}: state codes", max_frac)
    s_b = s_r[..., None, :] if s_r.dim() == c_r.dim() - 1 else s_r[..., None, None]
    assert_close(c_g.float() * (s_g[..., None, :] if s_g.dim() == c_g.dim() - 1 else s_g[..., None, None]),
                 c_r.float() * s_b, f"{what}: dequantised state", slack=flip.float() * s_b * 1.001)
    stats = {"state_flip_frac": frac_state, "resid_flip_frac": 0.0}
    if e_r is None:
        assert e_g is None
        return stats
    if res_fmt in int_formats:
        rq = 7.0 if res_fmt == 4 else 127.0
        per_v = es_r.dim() == s_r.dim()
        s_chan = s_r if per_v else s_r.amax(dim=-1)
        noise = (es_r * rq) < 1e-3 * s_chan                  # residual of this channel is rounding noise
        ok = ((es_g - es_r).abs() <= RESID_SCALE_RTOL * es_r + target_ulp_in_scale(s_chan, rq)) | noise
        assert bool(ok.all()), f"{what}: residual scale off in {int((~ok).sum())} channels"
        if res_fmt == 4:
            e_gc, e_rc = unpack_int4(e_g), unpack_int4(e_r)
        else:
            e_gc, e_rc = e_g, e_r
        noise_b = (noise[..., None, :] if per_v else noise[..., None, None]).expand_as(flip)
        flip = flip | noise_b
        # A flipped state code moves that element's residual across the grid, so
        # those elements are left out.  Its magnitude stays ~half a state step, so
        # the residual scale of its column (or head) moves only in the last bits.
        _, stats["resid_flip_frac"] = assert_codes(e_gc, e_rc, f"{what}: residual codes",
                                                   max_frac, exclude=flip)
    else:
        # float residual formats: one unit in the last place of the format at most
        # (the residual is a difference of nearly equal numbers: its absolute
        # error is that of the target, about 1e-7 at these magnitudes)
        rt = {0: 1e-3, 1: 2e-3, 2: 0.26}[res_fmt]
        at = 2.0 ** -16 * 1.001 if res_fmt == 2 else 1e-6      # e5m2 is subnormal below 2^-14: its steps are 2^-16
        assert_close(e_g.float(), e_r.float(), f"{what}: residual", rtol=rt, atol=at, exclude=flip)
    return stats


def check_pool(got, ref, int4: bool, slots, unpack_int4, what="pool", max_frac=MAX_FLIP_FRAC):
    """Compare slot-pool tensors ``(state_codes, state_scale, resid_codes,
    resid_scale)`` on the listed slots.  Returns ``(state, residual)`` flip
    fractions."""
    sc_g, ss_g, rc_g, rs_g = [x.cpu() for x in got]
    sc_r, ss_r, rc_r, rs_r = ref
    idx = torch.as_tensor(slots, dtype=torch.long)
    torch.testing.assert_close(ss_g[idx], ss_r[idx], rtol=STATE_SCALE_RTOL, atol=1e-30,
                               msg=f"{what}: state scale")
    rq = 7.0 if int4 else 127.0
    per_v = rs_r.dim() == 3
    s_chan = ss_r[idx] if per_v else ss_r[idx].amax(dim=-1)
    noise = (rs_r[idx] * rq) < 1e-3 * s_chan                 # residual of this channel is rounding noise
    ok = ((rs_g[idx] - rs_r[idx]).abs() <= RESID_SCALE_RTOL * rs_r[idx] + target_ulp_in_scale(s_chan, rq)) | noise
    assert bool(ok.all()), f"{what}: residual scale off in {int((~ok).sum())} channels"
    flip, f_state = assert_codes(sc_g[idx], sc_r[idx], f"{what}: state codes", max_frac)
    s_b = ss_r[idx][..., None]
    assert_close(sc_g[idx].float() * ss_g[idx][..., None], sc_r[idx].float() * s_b,
                 f"{what}: dequantised state", slack=flip.float() * s_b * 1.001)
    rg, rr = rc_g[idx], rc_r[idx]
    if int4:
        rg, rr = unpack_int4(rg), unpack_int4(rr)
    noise_b = (noise[..., None] if per_v else noise[..., None, None]).expand_as(flip)
    _, f_resid = assert_codes(rg, rr, f"{what}: residual codes", max_frac, exclude=flip | noise_b)
    # the dequantised residual itself: half a residual step at most
    rs_b = rs_r[idx][..., None] if rs_r.dim() == 3 else rs_r[idx][..., None, None]
    rs_gb = rs_g[idx][..., None] if rs_g.dim() == 3 else rs_g[idx][..., None, None]
    assert_close(rg.float() * rs_gb, rr.float() * rs_b, f"{what}: dequantised residual",
                 atol=1e-6, slack=rs_b.expand_as(rr) * 1.001, exclude=flip & ~noise_b)
    return f_state, f_resid
