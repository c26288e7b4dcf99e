"""carrykernel_b200 -- the fused Gated-DeltaNet decode step on an INT8 recurrent
state with an error-feedback residual, hand-written for NVIDIA B200 (sm_100a).

Three host surfaces, named after the carrykernel modules they stand in for:

* :mod:`carrykernel_b200.statequant.kernel` -- the statequant operator signature
* :mod:`carrykernel_b200.cuda.binding`      -- the CUDA entry point
* :mod:`carrykernel_b200.vllm_integration.quantized_packed_decode` -- the
  slot-indexed, in-place call path shaped like vLLM's packed decode

All three call one C-ABI library, ``libcarry_gdn.so`` (``include/carry_gdn.h``),
built from ``csrc/`` by :mod:`carrykernel_b200._build`.  There is no CPU path.
"""

from ._lib import CudaUnavailable, load_library  # noqa: F401

__all__ = ["CudaUnavailable", "load_library"]
