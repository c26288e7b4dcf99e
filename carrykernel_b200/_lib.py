"""ctypes binding of ``libcarry_gdn.so`` (the C ABI in ``include/carry_gdn.h``).

The structures below mirror the header field for field.  There is no fallback:
if the shared object is missing or a call fails, an exception is raised.
"""

from __future__ import annotations

import ctypes as C
import os
import threading

import torch

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "libcarry_gdn.so")
ABI_VERSION = 3

F32, BF16, F16 = 0, 1, 2
RES_FP32, RES_FP16, RES_FP8, RES_INT8, RES_INT4, RES_NONE = 0, 1, 2, 3, 4, 5
SCALE_PER_V, SCALE_PER_HEAD = 0, 1
EPS_ON_AMAX, EPS_ON_SCALE = 0, 1
STATUS_BAD_SLOT, STATUS_TIMEOUT = 1, 2

_DTYPE_ID = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}


class CudaUnavailable(RuntimeError):
    """The CUDA library cannot be loaded or used here."""


class StepArgs(C.Structure):
    _fields_ = [
        ("h_in", C.c_void_p), ("scale_in", C.c_void_p), ("e_in", C.c_void_p),
        ("e_scale_in", C.c_void_p), ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p),
        ("alpha", C.c_void_p), ("beta", C.c_void_p), ("o", C.c_void_p), ("h_out", C.c_void_p),
        ("scale_out", C.c_void_p), ("e_out", C.c_void_p), ("e_scale_out", C.c_void_p),
        ("B", C.c_int32), ("HV", C.c_int32), ("K", C.c_int32), ("V", C.c_int32),
        ("qkv_dtype", C.c_int32), ("o_dtype", C.c_int32), ("qmax", C.c_float),
        ("res_fmt", C.c_int32), ("resid_scale_mode", C.c_int32), ("state_scale_mode", C.c_int32),
        ("eps_mode", C.c_int32), ("status", C.c_void_p),
    ]


class Fp32Args(C.Structure):
    _fields_ = [
        ("h_in", C.c_void_p), ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p),
        ("alpha", C.c_void_p), ("beta", C.c_void_p), ("o", C.c_void_p), ("h_out", C.c_void_p),
        ("B", C.c_int32), ("HV", C.c_int32), ("K", C.c_int32), ("V", C.c_int32),
        ("qkv_dtype", C.c_int32), ("o_dtype", C.c_int32),
    ]


class PackedArgs(C.Structure):
    _fields_ = [
        ("mixed_qkv", C.c_void_p), ("stride_mixed_tok", C.c_int64), ("qkv_dtype", C.c_int32),
        ("a", C.c_void_p), ("stride_a_tok", C.c_int64), ("b", C.c_void_p),
        ("stride_b_tok", C.c_int64), ("ab_dtype", C.c_int32),
        ("A_log", C.c_void_p), ("A_log_dtype", C.c_int32),
        ("dt_bias", C.c_void_p), ("dt_bias_dtype", C.c_int32),
        ("scale", C.c_float),
        ("state_codes", C.c_void_p), ("state_scale", C.c_void_p),
        ("resid_codes", C.c_void_p), ("resid_scale", C.c_void_p),
        ("stride_state_slot", C.c_int64), ("stride_resid_slot", C.c_int64),
        ("stride_sscale_slot", C.c_int64), ("stride_rscale_slot", C.c_int64),
        ("out", C.c_void_p), ("out_dtype", C.c_int32),
        ("ssm_state_indices", C.c_void_p), ("stride_indices", C.c_int64),
        ("B", C.c_int32), ("H", C.c_int32), ("HV", C.c_int32), ("K", C.c_int32), ("V", C.c_int32),
        ("num_slots", C.c_int32), ("use_qk_l2norm", C.c_int32), ("res_fmt", C.c_int32),
        ("resid_scale_mode", C.c_int32), ("eps_mode", C.c_int32), ("qmax", C.c_float),
        ("status", C.c_void_p),
    ]


class PackedMultiArgs(C.Structure):
    _fields_ = [
        ("step", PackedArgs), ("T", C.c_int32),
        ("stride_mixed_t", C.c_int64), ("stride_a_t", C.c_int64), ("stride_b_t", C.c_int64),
    ]


class Pool(C.Structure):
    _fields_ = [
        ("state_codes", C.c_void_p), ("state_scale", C.c_void_p),
        ("resid_codes", C.c_void_p), ("resid_scale", C.c_void_p),
        ("stride_state_slot", C.c_int64), ("stride_resid_slot", C.c_int64),
        ("stride_sscale_slot", C.c_int64), ("stride_rscale_slot", C.c_int64),
        ("num_slots", C.c_int32), ("HV", C.c_int32), ("V", C.c_int32), ("K", C.c_int32),
        ("res_fmt", C.c_int32), ("resid_scale_mode", C.c_int32),
    ]


class PoolStoreArgs(C.Structure):
    _fields_ = [
        ("pool", Pool), ("h", C.c_void_p), ("stride_h_req", C.c_int64), ("h_dtype", C.c_int32),
        ("slots", C.c_void_p), ("stride_slots", C.c_int64), ("B", C.c_int32),
        ("keep_error", C.c_int32), ("qmax", C.c_float), ("status", C.c_void_p),
    ]


class PoolLoadArgs(C.Structure):
    _fields_ = [
        ("pool", Pool), ("h", C.c_void_p), ("stride_h_req", C.c_int64), ("h_dtype", C.c_int32),
        ("slots", C.c_void_p), ("stride_slots", C.c_int64), ("B", C.c_int32),
        ("with_residual", C.c_int32), ("status", C.c_void_p),
    ]


class PoolCopyArgs(C.Structure):
    _fields_ = [
        ("src", Pool), ("dst", Pool),
        ("src_slots", C.c_void_p), ("stride_src_slots", C.c_int64),
        ("dst_slots", C.c_void_p), ("stride_dst_slots", C.c_int64),
        ("B", C.c_int32), ("status", C.c_void_p),
    ]


ERR_UNSUPPORTED = -5

EXPORTS = ("carry_gdn_quant_step", "carry_gdn_fp32_step", "carry_gdn_packed_decode",
           "carry_gdn_packed_decode_multi", "carry_gdn_pool_store", "carry_gdn_pool_load",
           "carry_gdn_pool_copy", "carry_gdn_strerror", "carry_gdn_abi_version",
           "carry_gdn_last_kernel")

_lib = None
_lock = threading.Lock()


def load_library(path: str | None = None):
    """Load (once, thread-safe) and return the ctypes handle of the library."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = path or os.environ.get("CARRY_GDN_LIBRARY") or LIB_PATH
        if not os.path.exists(path):
            raise CudaUnavailable(
                f"{path} is missing: build it with `python -m carrykernel_b200._build`")
        try:
            lib = C.CDLL(path)
        except OSError as exc:
            raise CudaUnavailable(f"cannot load {path}: {exc}") from exc
        for name in EXPORTS:
            if not hasattr(lib, name):
                raise CudaUnavailable(f"{path} does not export {name}")
        lib.carry_gdn_strerror.restype = C.c_char_p
        lib.carry_gdn_strerror.argtypes = [C.c_int]
        lib.carry_gdn_abi_version.restype = C.c_int
        lib.carry_gdn_last_kernel.restype = C.c_int
        lib.carry_gdn_quant_step.argtypes = [C.POINTER(StepArgs), C.c_void_p]
        lib.carry_gdn_fp32_step.argtypes = [C.POINTER(Fp32Args), C.c_void_p]
        lib.carry_gdn_packed_decode.argtypes = [C.POINTER(PackedArgs), C.c_void_p]
        lib.carry_gdn_packed_decode_multi.argtypes = [C.POINTER(PackedMultiArgs), C.c_void_p]
        lib.carry_gdn_pool_store.argtypes = [C.POINTER(PoolStoreArgs), C.c_void_p]
        lib.carry_gdn_pool_load.argtypes = [C.POINTER(PoolLoadArgs), C.c_void_p]
        lib.carry_gdn_pool_copy.argtypes = [C.POINTER(PoolCopyArgs), C.c_void_p]
        for fn in (lib.carry_gdn_quant_step, lib.carry_gdn_fp32_step, lib.carry_gdn_packed_decode,
                   lib.carry_gdn_packed_decode_multi, lib.carry_gdn_pool_store, lib.carry_gdn_pool_load,
                   lib.carry_gdn_pool_copy):
            fn.restype = C.c_int
        if lib.carry_gdn_abi_version() != ABI_VERSION:
            raise CudaUnavailable(
                f"ABI mismatch: library {lib.carry_gdn_abi_version()}, binding {ABI_VERSION}")
        _lib = lib
        return _lib


def dtype_id(t: torch.Tensor) -> int:
    try:
        return _DTYPE_ID[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported element type {t.dtype} (need fp32, bf16 or fp16)") from None


def ptr(t):
    return None if t is None else t.data_ptr()


def check(rc: int, what: str):
    if rc != 0:
        msg = load_library().carry_gdn_strerror(rc).decode()
        raise RuntimeError(f"{what} failed: {msg} (code {rc})")


def require_cuda(t: torch.Tensor, name: str):
    if not t.is_cuda:
        raise CudaUnavailable(
            f"{name} is on {t.device}: this op has no CPU path, move the tensors to a CUDA device")


def same_device(device, **tensors):
    """Every tensor handed to a kernel must live on the state's device: the kernels take raw
    addresses, so a CPU tensor or one of another GPU would be a wild pointer on the device."""
    for name, t in tensors.items():
        if t is not None and t.device != device:
            raise ValueError(f"{name} is on {t.device} but the state is on {device}: all tensors of a call "
                             "must be on the same CUDA device")


def need_shape(t: torch.Tensor, shape, name: str):
    if tuple(t.shape) != tuple(shape):
        raise ValueError(f"{name} must be {tuple(shape)}, got {tuple(t.shape)}")


def status_ptr(status, device):
    """Address of the optional device status word: an int32 tensor of one element on the state's
    device that the kernels OR their status bits into (``STATUS_BAD_SLOT``: a slot id beyond the pool
    was treated as padding; ``STATUS_TIMEOUT``: a wait on data in flight ran out and the affected
    tiles were left untouched).  The caller zeroes it and reads it when convenient
    (:func:`raise_for_status`); the calls themselves never read it back."""
    if status is None:
        return None
    if status.dtype != torch.int32 or status.numel() != 1:
        raise ValueError("status must be an int32 tensor of one element")
    same_device(device, status=status)
    return status.data_ptr()


def raise_for_status(status: torch.Tensor, what: str = "carry_gdn"):
    """Read the status word (this synchronises with the device) and raise if a bit is set."""
    bits = int(status.item())
    if bits:
        names = [n for b, n in ((STATUS_BAD_SLOT, "slot id beyond the pool (treated as padding)"),
                                (STATUS_TIMEOUT, "a wait on data in flight ran out (tiles left untouched)"))
                 if bits & b]
        raise RuntimeError(f"{what}: device status {bits}: " + "; ".join(names))


def current_stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream
