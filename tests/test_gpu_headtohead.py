"""The head-to-head harness (``bench.py --mode headtohead``) at a small batch: the
reference's sanity guard (modal_vllm_headtohead.py:94-103) must hold, and one
step of vLLM's own fp32-state kernel and of this library from the same
dequantised state must agree on ``out``.  Skipped where vLLM's kernel cannot be
imported."""

from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_headtohead_guard_and_numeric_agreement():
    import bench
    res = bench.headtohead(batches=(8,), steps=30, warmup=10)
    if "vllm" in res:
        pytest.skip(res["vllm"])
    row = res["B8"]
    assert row["vllm_fp32_state_us"] and row["vllm_bf16_state_us"], row
    # the guard: a bf16 state moves half the bytes of an fp32 one and must not time 1.2x slower
    assert row["bf16_comparison_valid"] and res["suspect"] == [], row
    for key in ("ours_int8_resid_v_us", "ours_int8_resid_head_us", "ours_int4_resid_v_us", "ours_int4_resid_head_us"):
        assert row[key] > 0
    # same state, same fp32 inputs: the two kernels differ only in summation order
    assert row["out_mean_abs"]["vllm"] > 1e-3 and row["out_mean_abs"]["ours"] > 1e-3, row     # not vacuous
    assert row["out_max_abs_diff_vs_vllm_fp32"] < 1e-4, row
    assert row["out_max_rel_diff_vs_vllm_fp32"] < 1e-3, row
    assert row["state_traffic_MB"]["ours_int4_resid"] < row["state_traffic_MB"]["vllm_bf16"]
