"""CUDA entry point: same names and signatures as carrykernel's
``cuda/binding.py:31-156``, bound to the prebuilt C-ABI library instead of a
JIT-compiled torch extension.

``load_extension()`` loads ``libcarry_gdn.so`` once (thread-safe) and raises
:class:`CudaUnavailable` when there is no CUDA device or the library cannot be
loaded.  The step wrappers run on the tensors' device and on torch's current
stream, never synchronise, and return fresh output tensors.
"""

from __future__ import annotations

import torch

from .. import _lib
from .._lib import CudaUnavailable
from ..statequant import kernel as sq_kernel

__all__ = ["CudaUnavailable", "load_extension", "gdn_quant_step_cuda",
           "gdn_fp32_step_cuda", "gdn_quant_decode_cuda"]


def load_extension(verbose: bool = False, archs=None):
    """Return the loaded library handle.  ``archs`` is accepted for signature
    compatibility; the library is built for sm_100a only."""
    if not torch.cuda.is_available():
        raise CudaUnavailable("no CUDA device available")
    lib = _lib.load_library()
    if verbose:
        print(f"loaded {_lib.LIB_PATH} (ABI {lib.carry_gdn_abi_version()})")
    return lib


def gdn_quant_step_cuda(h_int8, scale, e, e_scale, q, k, v, alpha, beta,
                        bits: int = 8, res_fmt: int = sq_kernel.RES_FP32,
                        BLOCK_V: int = 128, resid_scale: str = "v", state_scale: str = "v"):
    """One fused GDN + INT8-quantize + error-feedback step.  Returns
    ``(o, h_int8_new, scale_new, e_new, e_scale_new)``; ``e_scale_new`` is
    ``None`` unless the residual is int8/int4.  ``e_scale=None`` is tolerated."""
    load_extension()
    return sq_kernel.gdn_quant_step_fused(
        h_int8, scale, e, e_scale, q, k, v, alpha, beta, bits=bits, res_fmt=res_fmt,
        BLOCK_V=BLOCK_V, resid_scale=resid_scale, state_scale=state_scale)


def gdn_fp32_step_cuda(h, q, k, v, alpha, beta, BLOCK_V: int = 128):
    """Fused fp32 GDN step (no quantisation).  Returns ``(h_out, o)``."""
    load_extension()
    return sq_kernel.gdn_step_fused_fp32(h, q, k, v, alpha, beta, BLOCK_V=BLOCK_V)


def gdn_quant_decode_cuda(h0, q, k, v, alpha, beta, T, bits: int = 8,
                          res_fmt: int = sq_kernel.RES_FP32, BLOCK_V: int = 128,
                          resid_scale: str = "v", state_scale: str = "v"):
    """T chained fused steps over ``[T, B, HV, *]`` inputs."""
    load_extension()
    return sq_kernel.gdn_quant_decode_fused(
        h0, q, k, v, alpha, beta, T, bits=bits, res_fmt=res_fmt, BLOCK_V=BLOCK_V,
        resid_scale=resid_scale, state_scale=state_scale)
