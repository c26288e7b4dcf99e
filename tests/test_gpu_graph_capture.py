"""The calls allocate nothing, never synchronise and read nothing back, so a whole
request life cycle -- hand-off, decode steps, checkpoint, multi-token step, load --
can be captured into one CUDA graph on a side stream and replayed; the replay has to
reproduce the eager run bit for bit."""

from __future__ import annotations

import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _setup(seed=3):
    from carrykernel_b200.vllm_integration import quantized_packed_decode as qpd
    B, T, H, HV, K, V, slots = 6, 3, 16, 32, 128, 128, 16
    g = torch.Generator().manual_seed(seed)
    w = 2 * H * K + HV * V
    d = dict(
        h=(torch.randn(B, HV, V, K, generator=g) * 0.1).to(DEV),
        mixed=torch.randn(B, w, generator=g).bfloat16().to(DEV),
        a=(torch.randn(B, HV, generator=g) * 0.5).bfloat16().to(DEV),
        b=torch.randn(B, HV, generator=g).bfloat16().to(DEV),
        mixed_t=torch.randn(B, T, w, generator=g).bfloat16().to(DEV),
        a_t=(torch.randn(B, T, HV, generator=g) * 0.5).bfloat16().to(DEV),
        b_t=torch.randn(B, T, HV, generator=g).bfloat16().to(DEV),
        A_log=torch.full((HV,), math.log(0.1), device=DEV),
        dt_bias=torch.zeros(HV, device=DEV),
        idx=torch.tensor([3, 7, 0, 1, 12, 5], dtype=torch.int32, device=DEV),
        spare=torch.tensor([4, 8, 0, 2, 13, 6], dtype=torch.int32, device=DEV),
        out=torch.zeros(B, 1, HV, V, dtype=torch.bfloat16, device=DEV),
        out_t=torch.zeros(B, T, HV, V, dtype=torch.bfloat16, device=DEV),
        back=torch.zeros(B, HV, V, K, device=DEV),
    )
    d["pool"] = qpd.init_quantized_state(slots, HV, V, K, DEV, resid_fmt=qpd.RESID_INT4, resid_scale="head")
    d["K"] = K
    return d


def _life_cycle(d):
    from carrykernel_b200.vllm_integration import quantized_packed_decode as qpd
    from carrykernel_b200.vllm_integration import state_pool as sp
    fmt = qpd.RESID_INT4
    scale = d["K"] ** -0.5
    sp.store_state(d["h"], d["pool"], d["idx"], resid_fmt=fmt, keep_error=True)
    for _ in range(2):
        qpd.quantized_gated_delta_rule_packed_decode(
            d["mixed"], d["a"], d["b"], d["A_log"], d["dt_bias"], scale, *d["pool"], d["out"], d["idx"],
            use_qk_l2norm_in_kernel=True, resid_fmt=fmt)
    sp.copy_slots(d["pool"], d["idx"], d["spare"], resid_fmt=fmt)            # checkpoint
    qpd.quantized_gated_delta_rule_packed_decode_multi(
        d["mixed_t"], d["a_t"], d["b_t"], d["A_log"], d["dt_bias"], scale, *d["pool"], d["out_t"], d["idx"],
        use_qk_l2norm_in_kernel=True, resid_fmt=fmt)
    sp.load_state(d["pool"], d["idx"], out=d["back"], resid_fmt=fmt)


def _results(d):
    return [t.clone() for t in (*d["pool"], d["out"], d["out_t"], d["back"])]


def test_life_cycle_in_one_graph_on_a_side_stream():
    eager = _setup()
    _life_cycle(eager)
    torch.cuda.synchronize()
    want = _results(eager)

    d = _setup()
    _life_cycle(d)                                   # loads the library outside the capture
    torch.cuda.synchronize()
    fresh = _setup()
    for k, v in fresh.items():                       # back to the initial values, same storage
        if isinstance(v, torch.Tensor):
            d[k].copy_(v)
    for t, f in zip(d["pool"], fresh["pool"]):
        t.copy_(f)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    first = torch.cuda.CUDAGraph()                   # torch sets up its capture state (a one-off allocation)
    with torch.cuda.graph(first, stream=side):
        d["out"].zero_()
    graph = torch.cuda.CUDAGraph()
    before = torch.cuda.memory_allocated()
    with torch.cuda.graph(graph, stream=side):
        _life_cycle(d)
    assert torch.cuda.memory_allocated() == before   # the calls allocated nothing while capturing
    graph.replay()
    torch.cuda.synchronize()
    for got, ref in zip(_results(d), want):
        assert torch.equal(got, ref)
    # a second replay advances the same pool again: differs from the first, equals a second eager run
    _life_cycle(eager)
    graph.replay()
    torch.cuda.synchronize()
    for got, ref in zip(_results(d), _results(eager)):
        assert torch.equal(got, ref)


def test_calls_follow_the_current_stream():
    """Work is enqueued on torch's current stream: a call made under a side stream that is
    blocked behind a long kernel does not run until that stream gets there."""
    from carrykernel_b200.vllm_integration import state_pool as sp
    from carrykernel_b200.vllm_integration import quantized_packed_decode as qpd
    d = _setup()
    side = torch.cuda.Stream()
    big = torch.empty(1 << 28, dtype=torch.float32, device=DEV)
    torch.cuda.synchronize()
    with torch.cuda.stream(side):
        for _ in range(20):
            big.add_(1.0)                            # tens of milliseconds on the side stream
        sp.store_state(d["h"], d["pool"], d["idx"], resid_fmt=qpd.RESID_INT4)
        done = torch.cuda.Event()
        done.record(side)
    torch.cuda.current_stream().synchronize()        # the default stream has nothing to wait for
    assert not done.query()                          # ... and the store has not run ahead of its stream
    side.synchronize()
    assert int(d["pool"][0][3].abs().max()) > 0
