"""CUDA entry point of the fused GDN state step (see :mod:`.binding`)."""

from .binding import (  # noqa: F401
    CudaUnavailable,
    gdn_fp32_step_cuda,
    gdn_quant_decode_cuda,
    gdn_quant_step_cuda,
    load_extension,
)
