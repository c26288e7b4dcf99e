"""Slot-indexed INT8 + error-feedback decode step in vLLM's GDN state layout.

Same call contract as carrykernel's
``vllm_integration/quantized_packed_decode.py:242-369`` (itself shaped on
vLLM's ``fused_recurrent_gated_delta_rule_packed_decode`` with the state tensor
replaced by four quantized tensors):

* pool ``state_codes [slots, HV, V, K]`` int8 (K contiguous),
  ``state_scale [slots, HV, V]`` fp32, ``resid_codes [slots, HV, V, K]`` int8
  (or ``[.., K // 2]`` packed int4: even K in the low nibble),
  ``resid_scale [slots, HV, V]`` fp32;
* ``mixed_qkv [B, 2*H*K + HV*V]`` = q | k | v, gates ``a, b [B, HV]``,
  ``A_log, dt_bias [HV]``, ``out [B, 1, HV, V]`` pre-allocated;
* request ``n`` updates slot ``ssm_state_indices[n]`` **in place**; a slot id
  ``<= 0`` (:data:`NULL_BLOCK_ID` padding) writes zeros to ``out[n]`` and leaves
  the pool alone.  Two requests must not name the same slot.

Additive: ``resid_scale`` may be ``[slots, HV]`` -- one residual scale per
head instead of one per V-row; the granularity is read off the shape.

The call allocates nothing, never synchronises and reads nothing back to the
host, so it can be captured in a CUDA graph.  There is no CPU path.

Deviations from the reference's contract, both stricter: ``a`` and ``b`` must
share one dtype (the reference loads each through its own pointer type), and
``A_log`` / ``dt_bias`` must be contiguous (the call does not copy them).  Every
tensor must be on the pool's device and is checked for the shape the kernel
will index; a violation raises ``ValueError`` before anything is launched.
"""

from __future__ import annotations

import torch

from .. import _lib
from .._lib import CudaUnavailable  # noqa: F401

QMAX_INT8 = 127.0
QMAX_INT4 = 7.0
EPS = 1e-12
SOFTPLUS_THRESHOLD = 20.0
NULL_BLOCK_ID = 0

RESID_INT8 = 0
RESID_INT4 = 1

_RES_ID = {RESID_INT8: _lib.RES_INT8, RESID_INT4: _lib.RES_INT4}


def _packed_args(mixed_qkv, a, b, A_log, dt_bias, scale, state_codes, state_scale, resid_codes, resid_scale,
                 out, out_shape_of, ssm_state_indices, use_qk_l2norm_in_kernel, resid_fmt, status=None):
    """Validation shared by the single- and the multi-token call (the reference's conditions,
    ``vllm_integration/quantized_packed_decode.py:268-307``) and the filled argument block.
    ``mixed_qkv``, ``a``, ``b`` are the 2-D views of one token per request."""
    if mixed_qkv.dim() != 2:
        raise ValueError(f"mixed_qkv must be 2-D, got {tuple(mixed_qkv.shape)}")
    if mixed_qkv.stride(-1) != 1:
        raise ValueError("mixed_qkv must be contiguous in its last dimension")
    if state_codes.dim() != 4:
        raise ValueError(f"state_codes must be 4-D, got {tuple(state_codes.shape)}")
    if state_codes.stride(-1) != 1:
        raise ValueError("state_codes must be contiguous in its last dimension")
    if state_codes.dtype != torch.int8 or resid_codes.dtype != torch.int8:
        raise ValueError("state_codes and resid_codes must be int8 storage")
    if resid_fmt not in _RES_ID:
        raise ValueError(f"unknown residual format {resid_fmt}")
    if resid_fmt == RESID_INT4 and resid_codes.shape[-1] * 2 != state_codes.shape[-1]:
        raise ValueError(
            "int4 residual must be packed two codes per byte: expected last dim "
            f"{state_codes.shape[-1] // 2}, got {resid_codes.shape[-1]}")
    if resid_fmt == RESID_INT8 and resid_codes.shape != state_codes.shape:
        raise ValueError("int8 residual must have the same shape as the state")
    if ssm_state_indices.dim() != 1:
        raise ValueError("ssm_state_indices must be 1-D")
    if ssm_state_indices.dtype != torch.int32:
        raise ValueError("ssm_state_indices must be int32")

    B = mixed_qkv.shape[0]
    num_slots, HV, V, K = state_codes.shape
    want_out = out_shape_of(B, HV, V)
    if tuple(out.shape) != want_out:
        raise ValueError(f"out must be {want_out}, got {tuple(out.shape)}")
    if not out.is_contiguous():
        raise ValueError("out must be contiguous")

    qkv_dim = mixed_qkv.shape[1]
    qk_dim = qkv_dim - HV * V
    if qk_dim <= 0 or qk_dim % 2 != 0:
        raise ValueError(f"cannot infer H from mixed_qkv width {qkv_dim}")
    H = (qk_dim // 2) // K
    if H <= 0 or HV % H != 0 or 2 * H * K != qk_dim:
        raise ValueError(f"cannot infer H from mixed_qkv width {qkv_dim}")
    if resid_fmt == RESID_INT4 and K % 2 != 0:
        raise ValueError(f"int4 residual packing needs an even K, got {K}")

    if resid_scale.dim() == 3:
        rmode = _lib.SCALE_PER_V
    elif resid_scale.dim() == 2:
        rmode = _lib.SCALE_PER_HEAD
    else:
        raise ValueError(f"resid_scale must be [slots, HV, V] or [slots, HV], got {tuple(resid_scale.shape)}")
    # the tile interior of the pool tensors must be dense; only the slot stride is free
    rk = resid_codes.shape[-1]
    if state_codes.stride()[1:] != (V * K, K, 1) or resid_codes.stride()[1:] != (V * rk, rk, 1):
        raise ValueError("pool tensors must be dense within a slot (only the slot stride may vary)")
    if state_scale.stride()[1:] != (V, 1) or state_scale.dtype != torch.float32:
        raise ValueError("state_scale must be fp32 [slots, HV, V], dense within a slot")
    want = (V, 1) if rmode == _lib.SCALE_PER_V else (1,)
    if resid_scale.stride()[1:] != want or resid_scale.dtype != torch.float32:
        raise ValueError("resid_scale must be fp32 and dense within a slot")
    if a.stride(-1) != 1 or b.stride(-1) != 1 or a.dtype != b.dtype:
        raise ValueError("a and b must share a dtype and be contiguous in their last dimension")
    # The kernels take raw addresses: everything has to be on the pool's device and large enough for what
    # B, HV, V, K and the slot count make the kernel index.
    dev = state_codes.device
    _lib.same_device(dev, mixed_qkv=mixed_qkv, a=a, b=b, A_log=A_log, dt_bias=dt_bias, state_scale=state_scale,
                     resid_codes=resid_codes, resid_scale=resid_scale, out=out, ssm_state_indices=ssm_state_indices)
    if a.dim() != 2 or b.dim() != 2:
        raise ValueError("a and b must be 2-D: [B, HV]")
    _lib.need_shape(a, (B, HV), "a")
    _lib.need_shape(b, (B, HV), "b")
    _lib.need_shape(A_log, (HV,), "A_log")
    _lib.need_shape(dt_bias, (HV,), "dt_bias")
    if not A_log.is_contiguous() or not dt_bias.is_contiguous():
        raise ValueError("A_log and dt_bias must be contiguous")
    _lib.need_shape(ssm_state_indices, (B,), "ssm_state_indices")
    _lib.need_shape(state_scale, (num_slots, HV, V), "state_scale")
    _lib.need_shape(resid_scale, (num_slots, HV, V) if rmode == _lib.SCALE_PER_V else (num_slots, HV), "resid_scale")
    if resid_codes.shape[:3] != (num_slots, HV, V):
        raise ValueError(f"resid_codes must be [{num_slots}, {HV}, {V}, ..], got {tuple(resid_codes.shape)}")
    status_addr = _lib.status_ptr(status, dev)
    _lib.require_cuda(state_codes, "state_codes")

    args = _lib.PackedArgs()
    args.mixed_qkv, args.stride_mixed_tok, args.qkv_dtype = mixed_qkv.data_ptr(), mixed_qkv.stride(0), _lib.dtype_id(mixed_qkv)
    args.a, args.stride_a_tok = a.data_ptr(), a.stride(0)
    args.b, args.stride_b_tok = b.data_ptr(), b.stride(0)
    args.ab_dtype = _lib.dtype_id(a)
    args.A_log, args.A_log_dtype = A_log.data_ptr(), _lib.dtype_id(A_log)
    args.dt_bias, args.dt_bias_dtype = dt_bias.data_ptr(), _lib.dtype_id(dt_bias)
    args.scale = float(scale)
    args.state_codes, args.state_scale = state_codes.data_ptr(), state_scale.data_ptr()
    args.resid_codes, args.resid_scale = resid_codes.data_ptr(), resid_scale.data_ptr()
    args.stride_state_slot, args.stride_resid_slot = state_codes.stride(0), resid_codes.stride(0)
    args.stride_sscale_slot, args.stride_rscale_slot = state_scale.stride(0), resid_scale.stride(0)
    args.out, args.out_dtype = out.data_ptr(), _lib.dtype_id(out)
    args.ssm_state_indices, args.stride_indices = ssm_state_indices.data_ptr(), ssm_state_indices.stride(0)
    args.B, args.H, args.HV, args.K, args.V = B, H, HV, K, V
    args.num_slots = num_slots
    args.use_qk_l2norm = int(bool(use_qk_l2norm_in_kernel))
    args.res_fmt = _RES_ID[resid_fmt]
    args.resid_scale_mode = rmode
    args.eps_mode = _lib.EPS_ON_SCALE
    args.qmax = QMAX_INT8
    args.status = status_addr
    return args, None


def quantized_gated_delta_rule_packed_decode(
    mixed_qkv: torch.Tensor,
    a: torch.Tensor,
    b: torch.Tensor,
    A_log: torch.Tensor,
    dt_bias: torch.Tensor,
    scale: float,
    state_codes: torch.Tensor,
    state_scale: torch.Tensor,
    resid_codes: torch.Tensor,
    resid_scale: torch.Tensor,
    out: torch.Tensor,
    ssm_state_indices: torch.Tensor,
    use_qk_l2norm_in_kernel: bool = False,
    resid_fmt: int = RESID_INT8,
    status: torch.Tensor | None = None,
):
    """Advance every request's slot by one token, in place; returns ``out``.

    ``status`` (additive, optional): an int32 tensor of one element on the pool's device that the
    kernel ORs its status bits into -- a slot id beyond the pool (that request is treated as padding:
    zeros to ``out``, pool untouched) or a wait that ran out.  Without it such a request is silently a
    padding request.  See ``_lib.raise_for_status``."""
    args, _keep = _packed_args(mixed_qkv, a, b, A_log, dt_bias, scale, state_codes, state_scale, resid_codes,
                               resid_scale, out, lambda B, HV, V: (B, 1, HV, V), ssm_state_indices,
                               use_qk_l2norm_in_kernel, resid_fmt, status)
    lib = _lib.load_library()
    dev = state_codes.device
    with torch.cuda.device(dev):
        rc = lib.carry_gdn_packed_decode(args, _lib.current_stream_ptr(dev))
    _lib.check(rc, "carry_gdn_packed_decode")
    return out


def quantized_gated_delta_rule_packed_decode_multi(
    mixed_qkv: torch.Tensor,
    a: torch.Tensor,
    b: torch.Tensor,
    A_log: torch.Tensor,
    dt_bias: torch.Tensor,
    scale: float,
    state_codes: torch.Tensor,
    state_scale: torch.Tensor,
    resid_codes: torch.Tensor,
    resid_scale: torch.Tensor,
    out: torch.Tensor,
    ssm_state_indices: torch.Tensor,
    use_qk_l2norm_in_kernel: bool = False,
    resid_fmt: int = RESID_INT8,
    status: torch.Tensor | None = None,
):
    """Advance every request's slot by T tokens in one call, in place; returns ``out``.

    ``mixed_qkv`` is ``[B, T, 2*H*K + HV*V]``, ``a`` and ``b`` ``[B, T, HV]``, ``out``
    ``[B, T, HV, V]``; everything else as in the single-token call.  The result is
    that of T single-token calls on ``mixed_qkv[:, t]`` in turn, bit for bit; the
    state tile of a request stays on chip between its tokens.  (No counterpart in
    carrykernel: this is the multi-token decode vLLM reaches through its
    speculative-decoding path.)  Shapes the streaming kernels do not take (K or V other than
    128, ...) fall back to one single-token call per token, which allocates a ``[B, 1, HV, V]``
    scratch block: that path is not CUDA-graph capturable.  ``status`` as in the single-token call."""
    if mixed_qkv.dim() != 3 or a.dim() != 3 or b.dim() != 3:
        raise ValueError("mixed_qkv, a and b must be 3-D: [B, T, ...]")
    B, T = mixed_qkv.shape[0], mixed_qkv.shape[1]
    if T < 1 or a.shape[:2] != (B, T) or b.shape[:2] != (B, T):
        raise ValueError("mixed_qkv, a and b must agree on [B, T]")
    step, _keep = _packed_args(mixed_qkv[:, 0], a[:, 0], b[:, 0], A_log, dt_bias, scale, state_codes, state_scale,
                               resid_codes, resid_scale, out, lambda B_, HV, V: (B_, T, HV, V), ssm_state_indices,
                               use_qk_l2norm_in_kernel, resid_fmt, status)
    args = _lib.PackedMultiArgs()
    args.step = step
    args.T = T
    args.stride_mixed_t, args.stride_a_t, args.stride_b_t = mixed_qkv.stride(1), a.stride(1), b.stride(1)
    lib = _lib.load_library()
    dev = state_codes.device
    with torch.cuda.device(dev):
        rc = lib.carry_gdn_packed_decode_multi(args, _lib.current_stream_ptr(dev))
    if rc == _lib.ERR_UNSUPPORTED:
        # shapes the streaming kernels do not take: one single-token call per token, each into a
        # dense [B, 1, HV, V] block that is then copied into place
        tmp = torch.empty((B, 1) + tuple(out.shape[2:]), dtype=out.dtype, device=out.device)
        for t in range(T):
            quantized_gated_delta_rule_packed_decode(
                mixed_qkv[:, t], a[:, t], b[:, t], A_log, dt_bias, scale, state_codes, state_scale, resid_codes,
                resid_scale, tmp, ssm_state_indices, use_qk_l2norm_in_kernel, resid_fmt, status)
            out[:, t:t + 1].copy_(tmp)
        return out
    _lib.check(rc, "carry_gdn_packed_decode_multi")
    return out


def init_quantized_state(num_slots: int, HV: int, V: int, K: int, device,
                         h0: torch.Tensor | None = None,
                         resid_fmt: int = RESID_INT8, resid_scale: str = "v"):
    """Allocate the quantized pool, optionally seeded from fp32
    ``h0 [num_slots, HV, V, K]``; the residual starts at zero.  Returns
    ``(state_codes, state_scale, resid_codes, resid_scale)``.
    ``resid_scale="head"`` allocates one residual scale per head."""
    if resid_scale not in ("v", "head"):
        raise ValueError(f"resid_scale must be 'v' or 'head', got {resid_scale!r}")
    resid_k = K // 2 if resid_fmt == RESID_INT4 else K
    state_codes = torch.zeros((num_slots, HV, V, K), dtype=torch.int8, device=device)
    state_scale = torch.zeros((num_slots, HV, V), dtype=torch.float32, device=device)
    resid_codes = torch.zeros((num_slots, HV, V, resid_k), dtype=torch.int8, device=device)
    rs_shape = (num_slots, HV, V) if resid_scale == "v" else (num_slots, HV)
    resid_scale_t = torch.zeros(rs_shape, dtype=torch.float32, device=device)
    if h0 is not None:
        s = h0.abs().amax(dim=-1).clamp(min=EPS) / QMAX_INT8
        codes = torch.round(h0 / s[..., None]).clamp(-QMAX_INT8, QMAX_INT8)
        state_codes.copy_(codes.to(torch.int8))
        state_scale.copy_(s)
    return state_codes, state_scale, resid_codes, resid_scale_t


def state_bytes_per_slot(HV: int, V: int, K: int, quantized: bool,
                         base_dtype_size: int = 4, resid_fmt: int = RESID_INT8,
                         resid_scale: str = "v"):
    """Bytes of recurrent state per request slot (what a cache page must hold)."""
    if not quantized:
        return HV * V * K * base_dtype_size
    codes = HV * V * K
    resid = HV * V * (K // 2 if resid_fmt == RESID_INT4 else K)
    scales = HV * V * 4 + (HV * V * 4 if resid_scale == "v" else HV * 4)
    return codes + resid + scales
