"""The statequant operator surface, backed by the sm_100a CUDA library.

Same names, argument order, defaults and return tuples as carrykernel's
``statequant/kernel.py:349-452``:

* :func:`gdn_quant_step_fused`  -- one fused INT8 + error-feedback step
* :func:`gdn_step_fused_fp32`   -- the unquantised fp32 step
* :func:`gdn_quant_decode_fused` -- T chained steps
* :func:`init_quant_state`, :func:`init_state`, :func:`per_v_channel_quantize`
* the residual-format constants and ``residual_bytes/label/dtype`` helpers

Differences, all additive: ``res_fmt`` also accepts :data:`RES_INT4` (packed
int4 residual, two codes per byte along V) and :data:`RES_NONE`; the keyword
``resid_scale`` selects one residual scale per V-column (``"v"``, upstream's
behaviour) or one per head (``"head"``); ``state_scale="head"`` selects the
uniform per-head state grid.  ``q/k/v`` may be fp32, bf16 or fp16 and are read
as they are (no cast kernel).  There is no CPU path: tensors must live on a
CUDA device, otherwise :class:`CudaUnavailable` is raised.
"""

from __future__ import annotations

import torch

from .. import _lib
from .._lib import CudaUnavailable  # noqa: F401  (re-export)

QMAX_INT8 = 127.0
EPS = 1e-12

RES_FP32 = 0
RES_FP16 = 1
RES_FP8 = 2
RES_INT8 = 3
RES_INT4 = 4   # extension: packed int4 codes + scale
RES_NONE = 5   # extension: no error feedback

_RES_BYTES = {RES_FP32: 4, RES_FP16: 2, RES_FP8: 1, RES_INT8: 1, RES_INT4: 0.5}
_RES_LABEL = {RES_FP32: "fp32", RES_FP16: "fp16", RES_FP8: "fp8", RES_INT8: "int8", RES_INT4: "int4"}
_SCALE_MODE = {"v": _lib.SCALE_PER_V, "head": _lib.SCALE_PER_HEAD}


def residual_bytes(fmt: int):
    """Bytes per residual element for a residual format."""
    return _RES_BYTES[fmt]


def residual_label(fmt: int) -> str:
    return _RES_LABEL[fmt]


def residual_dtype(fmt: int):
    if fmt == RES_FP32:
        return torch.float32
    if fmt == RES_FP16:
        return torch.float16
    if fmt == RES_FP8:
        return torch.float8_e5m2
    if fmt in (RES_INT8, RES_INT4):
        return torch.int8
    raise ValueError(f"unknown residual format {fmt}")


def _scale_mode(name: str) -> int:
    try:
        return _SCALE_MODE[name]
    except KeyError:
        raise ValueError(f"scale granularity must be 'v' or 'head', got {name!r}") from None


# ---------------------------------------------------------------------------
# state initialisation (one-off, plain torch on the tensor's own device)
# ---------------------------------------------------------------------------

def per_v_channel_quantize(x: torch.Tensor, bits: int = 8):
    """One scale per V-column of ``x [..., K, V]`` (amax over K).  Returns
    ``(codes int8, scale [..., V], dequantized)``."""
    qmax = 2 ** (bits - 1) - 1
    scale = x.abs().amax(dim=-2, keepdim=True).clamp(min=EPS) / qmax
    code = torch.round(x / scale).clamp(-qmax, qmax)
    return code.to(torch.int8), scale.squeeze(-2), code * scale


def per_head_quantize(x: torch.Tensor, bits: int = 8):
    """One scale per ``[K, V]`` matrix.  Returns ``(codes, scale [...], dequantized)``."""
    qmax = 2 ** (bits - 1) - 1
    scale = x.abs().amax(dim=(-1, -2), keepdim=True).clamp(min=EPS) / qmax
    code = torch.round(x / scale).clamp(-qmax, qmax)
    return code.to(torch.int8), scale[..., 0, 0], code * scale


def init_state(h0: torch.Tensor, bits: int = 8):
    """fp32 ``h0 [..., K, V]`` -> ``(h_int8, scale, e=0 fp32)``."""
    h_int8, scale, _ = per_v_channel_quantize(h0, bits)
    return h_int8, scale, torch.zeros_like(h0)


def init_quant_state(h0: torch.Tensor, bits: int = 8, res_fmt: int = RES_FP32,
                     resid_scale: str = "v", state_scale: str = "v"):
    """fp32 ``h0 [..., K, V]`` -> ``(h_int8, scale, e, e_scale)`` with a zero
    residual.  ``e_scale`` is a zero tensor for integer residuals, else ``None``."""
    _scale_mode(resid_scale)
    if _scale_mode(state_scale) == _lib.SCALE_PER_V:
        h_int8, scale, _ = per_v_channel_quantize(h0, bits)
    else:
        h_int8, scale, _ = per_head_quantize(h0, bits)
    if res_fmt == RES_NONE:
        return h_int8, scale, None, None
    lead, (K, V) = h0.shape[:-2], h0.shape[-2:]
    if res_fmt in (RES_INT8, RES_INT4):
        if res_fmt == RES_INT4 and V % 2:
            raise ValueError(f"int4 residual packing needs an even V, got {V}")
        e = torch.zeros((*lead, K, V // 2 if res_fmt == RES_INT4 else V),
                        dtype=torch.int8, device=h0.device)
        es_shape = (*lead, V) if resid_scale == "v" else tuple(lead)
        return h_int8, scale, e, torch.zeros(es_shape, dtype=torch.float32, device=h0.device)
    e = torch.zeros(h0.shape, dtype=residual_dtype(res_fmt), device=h0.device)
    return h_int8, scale, e, None


# ---------------------------------------------------------------------------
# the fused step
# ---------------------------------------------------------------------------

def _activation(t: torch.Tensor) -> torch.Tensor:
    t = t.contiguous()
    return t if t.dtype in (torch.float32, torch.bfloat16, torch.float16) else t.float()


def _check_step_tensors(h_int8, scale, e, e_scale, q, k, v, alpha, beta, res_fmt, resid_scale, state_scale):
    """Device and shape of everything one step reads: the kernels take raw addresses."""
    B, HV, K, V = h_int8.shape
    dev = h_int8.device
    _lib.same_device(dev, scale=scale, e=e, e_scale=e_scale, q=q, k=k, v=v, alpha=alpha, beta=beta)
    _lib.need_shape(scale, (B, HV, V) if state_scale == "v" else (B, HV), "scale")
    _lib.need_shape(q, (B, HV, K), "q")
    _lib.need_shape(k, (B, HV, K), "k")
    _lib.need_shape(v, (B, HV, V), "v")
    _lib.need_shape(alpha, (B, HV), "alpha")
    _lib.need_shape(beta, (B, HV), "beta")
    if e is not None:
        _lib.need_shape(e, (B, HV, K, V // 2 if res_fmt == RES_INT4 else V), "e")
    if e_scale is not None:
        _lib.need_shape(e_scale, (B, HV, V) if resid_scale == "v" else (B, HV), "e_scale")


def quant_step_into(h_int8, scale, e, e_scale, q, k, v, alpha, beta, outputs,
                    bits: int = 8, res_fmt: int = RES_FP32, resid_scale: str = "v",
                    state_scale: str = "v", status=None):
    """Launch one step into caller-provided ``outputs = (o, h_out, scale_out,
    e_out, e_scale_out)``; no allocation, no synchronisation.  Output state
    buffers may be the input buffers (in-place).  This is the low-level entry
    the wrappers and the benchmark share.  ``status``: optional int32 device
    word for the kernel's status bits (``_lib.status_ptr``)."""
    o, h_out, scale_out, e_out, e_scale_out = outputs
    B, HV, K, V = h_int8.shape
    _check_step_tensors(h_int8, scale, e, e_scale, q, k, v, alpha, beta, res_fmt, resid_scale, state_scale)
    _lib.same_device(h_int8.device, o=o, h_out=h_out, scale_out=scale_out, e_out=e_out, e_scale_out=e_scale_out)
    _lib.need_shape(o, (B, HV, V), "o")
    _lib.need_shape(h_out, h_int8.shape, "h_out")
    _lib.need_shape(scale_out, scale.shape, "scale_out")
    a = _lib.StepArgs()
    a.h_in, a.scale_in, a.e_in, a.e_scale_in = h_int8.data_ptr(), scale.data_ptr(), _lib.ptr(e), _lib.ptr(e_scale)
    a.q, a.k, a.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    a.alpha, a.beta = alpha.data_ptr(), beta.data_ptr()
    a.o, a.h_out, a.scale_out = o.data_ptr(), h_out.data_ptr(), scale_out.data_ptr()
    a.e_out, a.e_scale_out = _lib.ptr(e_out), _lib.ptr(e_scale_out)
    a.B, a.HV, a.K, a.V = B, HV, K, V
    a.qkv_dtype, a.o_dtype = _lib.dtype_id(q), _lib.dtype_id(o)
    a.qmax = float(2 ** (bits - 1) - 1)
    a.res_fmt = res_fmt
    a.resid_scale_mode = _scale_mode(resid_scale)
    a.state_scale_mode = _scale_mode(state_scale)
    a.eps_mode = _lib.EPS_ON_AMAX
    a.status = _lib.status_ptr(status, h_int8.device)
    lib = _lib.load_library()
    with torch.cuda.device(h_int8.device):
        rc = lib.carry_gdn_quant_step(a, _lib.current_stream_ptr(h_int8.device))
    _lib.check(rc, "carry_gdn_quant_step")


def gdn_quant_step_fused(h_int8, scale, e, e_scale, q, k, v, alpha, beta,
                         bits: int = 8, res_fmt: int = RES_FP32, BLOCK_V: int = 32,
                         resid_scale: str = "v", state_scale: str = "v"):
    """Fused GDN + INT8 quantize + error feedback, one decode step.

    Inputs are left untouched; returns fresh ``(o, h_int8_new, scale_new,
    e_new, e_scale_new)`` with ``o`` fp32 ``[B, HV, V]`` and ``e_scale_new``
    ``None`` unless the residual is int8/int4.  ``BLOCK_V`` is accepted for
    signature compatibility and ignored.
    """
    assert h_int8.dtype == torch.int8, f"h_int8 must be int8, got {h_int8.dtype}"
    assert h_int8.dim() == 4, f"expected [B, HV, K, V], got {tuple(h_int8.shape)}"
    _scale_mode(resid_scale), _scale_mode(state_scale)
    _check_step_tensors(h_int8, scale, None if res_fmt == RES_NONE else e,
                        e_scale if res_fmt in (RES_INT8, RES_INT4) else None, q, k, v, alpha, beta,
                        res_fmt, resid_scale, state_scale)
    _lib.require_cuda(h_int8, "h_int8")
    B, HV, K, V = h_int8.shape
    dev = h_int8.device
    int_resid = res_fmt in (RES_INT8, RES_INT4)
    if res_fmt not in _RES_BYTES and res_fmt != RES_NONE:
        raise ValueError(f"unknown residual format {res_fmt}")

    h_int8 = h_int8.contiguous()
    scale = scale.contiguous().float()
    q, k, v = _activation(q), _activation(k), _activation(v)
    if not (q.dtype == k.dtype == v.dtype):
        q, k, v = q.float(), k.float(), v.float()
    alpha = alpha.contiguous().float()
    beta = beta.contiguous().float()
    if res_fmt == RES_NONE:
        e = e_scale = None
    else:
        e = e.contiguous()
        if e.dtype != residual_dtype(res_fmt):
            raise TypeError(f"residual dtype {e.dtype} does not match res_fmt {res_fmt}")
    es_shape = (B, HV, V) if resid_scale == "v" else (B, HV)
    if int_resid:
        if e_scale is None:
            e_scale = torch.zeros(es_shape, device=dev, dtype=torch.float32)
        e_scale = e_scale.contiguous().float()
        if tuple(e_scale.shape) != es_shape:
            raise ValueError(f"e_scale must be {es_shape} for resid_scale={resid_scale!r}, "
                             f"got {tuple(e_scale.shape)}")
    else:
        e_scale = None

    o = torch.empty((B, HV, V), device=dev, dtype=torch.float32)
    h_out = torch.empty_like(h_int8)
    scale_out = torch.empty_like(scale)
    e_out = torch.empty_like(e) if e is not None else None
    e_scale_out = torch.empty_like(e_scale) if int_resid else None
    quant_step_into(h_int8, scale, e, e_scale, q, k, v, alpha, beta,
                    (o, h_out, scale_out, e_out, e_scale_out),
                    bits, res_fmt, resid_scale, state_scale)
    return o, h_out, scale_out, e_out, e_scale_out


def gdn_step_fused_fp32(h, q, k, v, alpha, beta, BLOCK_V: int = 32):
    """Fused fp32 GDN step (no quantisation).  Returns ``(h_out, o)``."""
    assert h.dim() == 4, f"expected [B, HV, K, V], got {tuple(h.shape)}"
    B, HV, K, V = h.shape
    dev = h.device
    _lib.same_device(dev, q=q, k=k, v=v, alpha=alpha, beta=beta)
    _lib.need_shape(q, (B, HV, K), "q")
    _lib.need_shape(k, (B, HV, K), "k")
    _lib.need_shape(v, (B, HV, V), "v")
    _lib.need_shape(alpha, (B, HV), "alpha")
    _lib.need_shape(beta, (B, HV), "beta")
    _lib.require_cuda(h, "h")
    h = h.contiguous().float()
    q, k, v = _activation(q), _activation(k), _activation(v)
    if not (q.dtype == k.dtype == v.dtype):
        q, k, v = q.float(), k.float(), v.float()
    alpha = alpha.contiguous().float()
    beta = beta.contiguous().float()
    o = torch.empty((B, HV, V), device=dev, dtype=torch.float32)
    h_out = torch.empty_like(h)
    a = _lib.Fp32Args()
    a.h_in, a.q, a.k, a.v = h.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr()
    a.alpha, a.beta, a.o, a.h_out = alpha.data_ptr(), beta.data_ptr(), o.data_ptr(), h_out.data_ptr()
    a.B, a.HV, a.K, a.V = B, HV, K, V
    a.qkv_dtype, a.o_dtype = _lib.dtype_id(q), _lib.F32
    lib = _lib.load_library()
    with torch.cuda.device(dev):
        rc = lib.carry_gdn_fp32_step(a, _lib.current_stream_ptr(dev))
    _lib.check(rc, "carry_gdn_fp32_step")
    return h_out, o


def gdn_quant_decode_fused(h0, q, k, v, alpha, beta, T, bits: int = 8,
                           res_fmt: int = RES_FP32, BLOCK_V: int = 32,
                           resid_scale: str = "v", state_scale: str = "v"):
    """T chained fused steps.  ``h0 [B, HV, K, V]`` fp32; ``q/k [T, B, HV, K]``,
    ``v [T, B, HV, V]``, ``alpha/beta [T, B, HV]``.  Returns
    ``(o [T, B, HV, V], h_int8, scale, e, e_scale)``."""
    h_int8, scale, e, e_scale = init_quant_state(h0, bits, res_fmt, resid_scale, state_scale)
    outs = []
    for t in range(T):
        o, h_int8, scale, e, e_scale = gdn_quant_step_fused(
            h_int8, scale, e, e_scale, q[t], k[t], v[t], alpha[t], beta[t],
            bits=bits, res_fmt=res_fmt, BLOCK_V=BLOCK_V,
            resid_scale=resid_scale, state_scale=state_scale)
        outs.append(o)
    return torch.stack(outs), h_int8, scale, e, e_scale
