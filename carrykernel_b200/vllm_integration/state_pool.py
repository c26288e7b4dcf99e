"""Moving a request's recurrent state in and out of the quantized slot pool.

carrykernel stops at the decode step: its pool is seeded once by eager torch ops
(``init_quantized_state``, ``vllm_integration/quantized_packed_decode.py:330-352``)
and the wiring into an engine's cache is listed as not done (same file
``:50-54``) -- with the note that the error-feedback residual is per-request
state that has to survive paging, preemption, prefix-cache reuse and
speculative-decode rollback.  These are the three device operations that wiring
needs, each one kernel launch over ``(request, head)`` tiles, no allocation, no
synchronisation, CUDA-graph capturable:

* :func:`store_state` -- prefill hand-off: quantise the floating-point final
  state of a prefill into the requests' slots (same codes and scales as
  ``init_quantized_state``; the residual is zeroed, or, with ``keep_error``,
  set to the quantisation error so that the first decode step feeds it back);
* :func:`load_state` -- the reverse: ``codes * scale (+ resid * resid_scale)``
  as fp32 / bf16 / fp16, for a kernel that wants a floating-point state;
* :func:`copy_slots` -- whole slots, residual included, bit for bit, within a
  pool or into a second pool (spill pool, checkpoint, prefix-cache entry).

Every function takes an optional ``status``: an int32 device word the kernel ORs
its status bits into (a slot id beyond the pool is skipped and flagged there;
see ``_lib.status_ptr``).

A *pool* is the 4-tuple ``(state_codes, state_scale, resid_codes, resid_scale)``
that ``init_quantized_state`` returns.  There is no CPU path.
"""

from __future__ import annotations

import torch

from .. import _lib
from .quantized_packed_decode import QMAX_INT8, RESID_INT4, RESID_INT8, _RES_ID


def _pool_struct(pool, resid_fmt):
    """Checks of the pool tensors (those of the decode call) and the filled ``CarryGdnPool``."""
    state_codes, state_scale, resid_codes, resid_scale = pool
    if state_codes.dim() != 4:
        raise ValueError(f"state_codes must be 4-D, got {tuple(state_codes.shape)}")
    if state_codes.dtype != torch.int8 or resid_codes.dtype != torch.int8:
        raise ValueError("state_codes and resid_codes must be int8 storage")
    if resid_fmt not in _RES_ID:
        raise ValueError(f"unknown residual format {resid_fmt}")
    num_slots, HV, V, K = state_codes.shape
    if resid_fmt == RESID_INT4 and (K % 2 != 0 or resid_codes.shape[-1] * 2 != K):
        raise ValueError(
            f"int4 residual must be packed two codes per byte: expected last dim {K // 2}, "
            f"got {resid_codes.shape[-1]}")
    if resid_fmt == RESID_INT8 and resid_codes.shape != state_codes.shape:
        raise ValueError("int8 residual must have the same shape as the state")
    _lib.require_cuda(state_codes, "state_codes")
    if resid_scale.dim() == 3:
        rmode = _lib.SCALE_PER_V
    elif resid_scale.dim() == 2:
        rmode = _lib.SCALE_PER_HEAD
    else:
        raise ValueError(f"resid_scale must be [slots, HV, V] or [slots, HV], got {tuple(resid_scale.shape)}")
    rk = resid_codes.shape[-1]
    if state_codes.stride()[1:] != (V * K, K, 1) or resid_codes.stride()[1:] != (V * rk, rk, 1):
        raise ValueError("pool tensors must be dense within a slot (only the slot stride may vary)")
    if state_scale.stride()[1:] != (V, 1) or state_scale.dtype != torch.float32:
        raise ValueError("state_scale must be fp32 [slots, HV, V], dense within a slot")
    want = (V, 1) if rmode == _lib.SCALE_PER_V else (1,)
    if resid_scale.stride()[1:] != want or resid_scale.dtype != torch.float32:
        raise ValueError("resid_scale must be fp32 and dense within a slot")
    if any(t.device != state_codes.device for t in (state_scale, resid_codes, resid_scale)):
        raise ValueError("the four pool tensors must live on one device")
    _lib.need_shape(state_scale, (num_slots, HV, V), "state_scale")
    _lib.need_shape(resid_scale, (num_slots, HV, V) if rmode == _lib.SCALE_PER_V else (num_slots, HV), "resid_scale")
    if resid_codes.shape[:3] != (num_slots, HV, V):
        raise ValueError(f"resid_codes must be [{num_slots}, {HV}, {V}, ..], got {tuple(resid_codes.shape)}")
    p = _lib.Pool()
    p.state_codes, p.state_scale = state_codes.data_ptr(), state_scale.data_ptr()
    p.resid_codes, p.resid_scale = resid_codes.data_ptr(), resid_scale.data_ptr()
    p.stride_state_slot, p.stride_resid_slot = state_codes.stride(0), resid_codes.stride(0)
    p.stride_sscale_slot, p.stride_rscale_slot = state_scale.stride(0), resid_scale.stride(0)
    p.num_slots, p.HV, p.V, p.K = num_slots, HV, V, K
    p.res_fmt, p.resid_scale_mode = _RES_ID[resid_fmt], rmode
    return p


def _indices(idx, name, device):
    if idx.dim() != 1:
        raise ValueError(f"{name} must be 1-D")
    if idx.dtype != torch.int32:
        raise ValueError(f"{name} must be int32")
    if idx.device != device:
        raise ValueError(f"{name} must be on the pool's device")
    return idx.data_ptr(), idx.stride(0)


def _state_tensor(h, B, HV, V, K, device, name):
    if tuple(h.shape) != (B, HV, V, K):
        raise ValueError(f"{name} must be [B, HV, V, K] = {(B, HV, V, K)}, got {tuple(h.shape)}")
    if h.stride()[1:] != (V * K, K, 1):
        raise ValueError(f"{name} must be dense within a request (only the request stride may vary)")
    if h.device != device:
        raise ValueError(f"{name} must be on the pool's device")
    return h.data_ptr(), h.stride(0), _lib.dtype_id(h)


def store_state(h, pool, ssm_state_indices, resid_fmt: int = RESID_INT8, keep_error: bool = False, status=None):
    """Quantise ``h [B, HV, V, K]`` (fp32, bf16 or fp16) into slots
    ``ssm_state_indices [B]`` of ``pool``.  Slot ids ``<= 0`` are skipped."""
    p = _pool_struct(pool, resid_fmt)
    dev = pool[0].device
    args = _lib.PoolStoreArgs()
    args.pool = p
    args.slots, args.stride_slots = _indices(ssm_state_indices, "ssm_state_indices", dev)
    args.B = ssm_state_indices.shape[0]
    args.h, args.stride_h_req, args.h_dtype = _state_tensor(h, args.B, p.HV, p.V, p.K, dev, "h")
    args.keep_error = int(bool(keep_error))
    args.qmax = QMAX_INT8
    args.status = _lib.status_ptr(status, dev)
    lib = _lib.load_library()
    with torch.cuda.device(dev):
        rc = lib.carry_gdn_pool_store(args, _lib.current_stream_ptr(dev))
    _lib.check(rc, "carry_gdn_pool_store")


def load_state(pool, ssm_state_indices, out=None, dtype=torch.float32, resid_fmt: int = RESID_INT8,
               with_residual: bool = True, status=None):
    """``out[n] = codes * scale (+ resid_codes * resid_scale)`` of slot
    ``ssm_state_indices[n]``; zeros for slot ids ``<= 0``.  ``out`` is allocated
    (``dtype``) when not given.  Returns ``out [B, HV, V, K]``."""
    p = _pool_struct(pool, resid_fmt)
    dev = pool[0].device
    B = ssm_state_indices.shape[0] if ssm_state_indices.dim() == 1 else 0
    if out is None:
        out = torch.empty((B, p.HV, p.V, p.K), dtype=dtype, device=dev)
    args = _lib.PoolLoadArgs()
    args.pool = p
    args.slots, args.stride_slots = _indices(ssm_state_indices, "ssm_state_indices", dev)
    args.B = B
    args.h, args.stride_h_req, args.h_dtype = _state_tensor(out, B, p.HV, p.V, p.K, dev, "out")
    args.with_residual = int(bool(with_residual))
    args.status = _lib.status_ptr(status, dev)
    lib = _lib.load_library()
    with torch.cuda.device(dev):
        rc = lib.carry_gdn_pool_load(args, _lib.current_stream_ptr(dev))
    _lib.check(rc, "carry_gdn_pool_load")
    return out


def copy_slots(src_pool, src_indices, dst_indices, dst_pool=None, resid_fmt: int = RESID_INT8, status=None):
    """Copy slot ``src_indices[n]`` of ``src_pool`` to slot ``dst_indices[n]`` of
    ``dst_pool`` (default: the same pool), all four tensors, bit for bit.  Pairs
    with an id ``<= 0`` are skipped; no destination may also be a source or a
    second destination in the same call."""
    dst_pool = src_pool if dst_pool is None else dst_pool
    s = _pool_struct(src_pool, resid_fmt)
    d = _pool_struct(dst_pool, resid_fmt)
    if (s.HV, s.V, s.K) != (d.HV, d.V, d.K) or s.resid_scale_mode != d.resid_scale_mode:
        raise ValueError("source and destination pools must have the same head shape and residual scale layout")
    dev = src_pool[0].device
    if dst_pool[0].device != dev:
        raise ValueError("source and destination pools must be on one device")
    if src_indices.shape != dst_indices.shape:
        raise ValueError("src_indices and dst_indices must have the same length")
    args = _lib.PoolCopyArgs()
    args.src, args.dst = s, d
    args.src_slots, args.stride_src_slots = _indices(src_indices, "src_indices", dev)
    args.dst_slots, args.stride_dst_slots = _indices(dst_indices, "dst_indices", dev)
    args.B = src_indices.shape[0]
    args.status = _lib.status_ptr(status, dev)
    lib = _lib.load_library()
    with torch.cuda.device(dev):
        rc = lib.carry_gdn_pool_copy(args, _lib.current_stream_ptr(dev))
    _lib.check(rc, "carry_gdn_pool_copy")
