"""A bounded wait that runs out, on the GPU, without faulting or hanging anything.

Every wait of the streaming kernels on data in flight gives up after a fixed
number of polls, sets ``STATUS_TIMEOUT`` in the status word, and the CTA stops
loading and storing.  ``libcarry_gdn_waittest.so`` is the same library built with
``CARRY_TEST_WAIT_EXPIRY``: the copies of global tile 1 (request 0, head 1)
announce 16 bytes more than they bring, so that tile's stage barrier can never
complete, and the poll limit is short.  Expected of every kernel: the launch
returns, the status bit is set, the tile's state and output are exactly as they
were, and every other tile equals what the regular library computes.

The twin also makes the streaming kernel take, for every tile whose index has
bit 1 set, the path of a launch whose set-up inputs changed between its look at
them ahead of the stream dependency and its second look after it (the whole
set-up is then done again): "every other tile equals what the regular library
computes" therefore covers that path as well, bit for bit.  For a change that
is real, the twin also exports ``carry_gdn_test_late_writer`` -- a kernel that
lets the launch behind it start, idles, and only then copies a buffer -- and
ORs bit 30 into the status word when a tile's inputs differed between the
two looks.
"""

from __future__ import annotations

import contextlib

import pytest
import torch

from oracle import gdn_oracle as orc
from parity import make_packed_inputs, seeded_inputs

pytestmark = pytest.mark.gpu
DEV = "cuda"


@contextlib.contextmanager
def wait_test_library():
    """Route the package's calls through the test-only twin for the duration of the block."""
    from carrykernel_b200 import _build, _lib
    saved = _lib._lib
    _lib._lib = None
    try:
        _lib.load_library(_build.WAIT_TEST_LIB)
        yield
    finally:
        _lib._lib = saved


def _slot_case(resid_fmt, rscale):
    from carrykernel_b200.vllm_integration import quantized_packed_decode as qpd
    B, H, HV, K, V, num_slots = 4, 32, 32, 128, 128, 6
    g = torch.Generator().manual_seed(3)
    pool = torch.randn(num_slots, HV, V, K, generator=g) * 0.1
    st = [x.to(DEV) for x in qpd.init_quantized_state(num_slots, HV, V, K, "cpu", h0=pool, resid_fmt=resid_fmt,
                                                      resid_scale=rscale)]
    idx = torch.tensor([3, 1, 5, 2], dtype=torch.int32, device=DEV)
    return qpd, (B, H, HV, K, V), st, idx


@pytest.mark.parametrize("resid_fmt,rscale", [(1, "head"), (0, "v")])
def test_single_token_kernel_wait_runs_out(resid_fmt, rscale):
    from carrykernel_b200 import _lib
    qpd, (B, H, HV, K, V), st, idx = _slot_case(resid_fmt, rscale)
    mixed, a, b, A_log, dt_bias = [x.to(DEV) for x in make_packed_inputs(B, H, HV, K, V, seed=9, dtype=torch.bfloat16)]
    A_log, dt_bias = A_log.float(), dt_bias.float()

    def run(pool, status):
        out = torch.full((B, 1, HV, V), float("nan"), dtype=torch.bfloat16, device=DEV)
        qpd.quantized_gated_delta_rule_packed_decode(mixed, a, b, A_log, dt_bias, K ** -0.5, *pool, out, idx,
                                                     use_qk_l2norm_in_kernel=True, resid_fmt=resid_fmt, status=status)
        torch.cuda.synchronize()
        return out

    good = [x.clone() for x in st]
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out_good = run(good, status)
    assert int(status.item()) == 0
    bad = [x.clone() for x in st]
    with wait_test_library():
        out_bad = run(bad, status)
    assert int(status.item()) == _lib.STATUS_TIMEOUT
    slot, head = int(idx[0]), 1                      # global tile 1 = request 0, head 1
    # that tile: nothing written
    assert torch.isnan(out_bad[0, 0, head].float()).all()
    for x_bad, x0 in zip(bad[:3], st[:3]):
        assert torch.equal(x_bad[slot, head], x0[slot, head])
    assert torch.equal(bad[3][slot, head], st[3][slot, head])
    # every other tile: what the regular library computes
    keep = torch.ones(B, HV, dtype=torch.bool, device=DEV)
    keep[0, head] = False
    assert torch.equal(out_bad[:, 0][keep], out_good[:, 0][keep])
    mask = torch.ones(st[0].shape[0], HV, dtype=torch.bool, device=DEV)
    mask[slot, head] = False
    for x_bad, x_good in zip(bad, good):
        assert torch.equal(x_bad[mask], x_good[mask])
    # the context is still usable and the regular library still clean
    status.zero_()
    run([x.clone() for x in st], status)
    assert int(status.item()) == 0


@pytest.mark.parametrize("B", [4, 160, 400])       # 1, 35 and 87 tiles per CTA: 32, 8 and 4 lanes per tile in the set-up
def test_set_up_done_again_gives_the_same_results(B):
    """Tiles whose set-up the twin does twice (index bit 1 set) against the regular library, bit for bit.

    The CTA that owns global tile 1 stops at that tile (its wait runs out), so all of that CTA's tiles
    are left out of the comparison."""
    from carrykernel_b200 import _lib
    from carrykernel_b200.vllm_integration import quantized_packed_decode as qpd
    H = HV = 32
    K = V = 128
    num_slots = B + 2
    g = torch.Generator().manual_seed(5)
    st = [x.to(DEV) for x in qpd.init_quantized_state(num_slots, HV, V, K, "cpu", resid_fmt=1, resid_scale="head")]
    st[0].copy_(torch.randint(-127, 128, st[0].shape, generator=g, dtype=torch.int8))
    st[1].copy_(torch.rand(st[1].shape, generator=g) * 1e-3 + 1e-4)
    idx = (torch.randperm(num_slots - 1, generator=g)[:B] + 1).to(torch.int32).to(DEV)
    mixed, a, b, A_log, dt_bias = [x.to(DEV) for x in make_packed_inputs(B, H, HV, K, V, seed=11, dtype=torch.bfloat16)]
    A_log, dt_bias = A_log.float(), dt_bias.float()

    def run(pool, status):
        out = torch.full((B, 1, HV, V), float("nan"), dtype=torch.bfloat16, device=DEV)
        qpd.quantized_gated_delta_rule_packed_decode(mixed, a, b, A_log, dt_bias, K ** -0.5, *pool, out, idx,
                                                     use_qk_l2norm_in_kernel=True, resid_fmt=1, status=status)
        torch.cuda.synchronize()
        return out

    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    good = [x.clone() for x in st]
    out_good = run(good, status)
    assert int(status.item()) == 0
    twin = [x.clone() for x in st]
    with wait_test_library():
        out_twin = run(twin, status)
    assert int(status.item()) == _lib.STATUS_TIMEOUT
    ctas = torch.cuda.get_device_properties(0).multi_processor_count
    tile = torch.arange(B * HV, device=DEV).view(B, HV)
    keep = (tile % ctas) != 1
    assert int((keep & ((tile & 2) != 0)).sum()) > 0
    assert torch.equal(out_twin[:, 0][keep].float(), out_good[:, 0][keep].float())
    rows = idx.long()
    for x_twin, x_good in zip(twin, good):
        assert torch.equal(x_twin[rows][keep], x_good[rows][keep])


def test_inputs_written_late_by_the_kernel_ahead():
    """A real change of the inputs between the streaming kernel's two looks at them.

    The twin library has a kernel that lets its successor start at once, idles 50 us and only then writes
    the activations.  The decode call queued right behind it takes its first look while the buffer still
    holds other values, finds them changed after its dependency wait (the twin reports that in a status bit
    of its own) and must redo its set-up: results equal the regular library's on the final inputs."""
    import ctypes as C
    from carrykernel_b200 import _lib
    from carrykernel_b200.vllm_integration import quantized_packed_decode as qpd
    B, H, HV, K, V = 16, 32, 32, 128, 128
    num_slots = B + 2
    g = torch.Generator().manual_seed(8)
    pool = torch.randn(num_slots, HV, V, K, generator=g) * 0.1
    st = [x.to(DEV) for x in qpd.init_quantized_state(num_slots, HV, V, K, "cpu", h0=pool, resid_fmt=1, resid_scale="head")]
    idx = (torch.randperm(num_slots - 1, generator=g)[:B] + 1).to(torch.int32).to(DEV)
    mixed, a, b, A_log, dt_bias = [x.to(DEV) for x in make_packed_inputs(B, H, HV, K, V, seed=12, dtype=torch.bfloat16)]
    early = make_packed_inputs(B, H, HV, K, V, seed=13, dtype=torch.bfloat16)[0].to(DEV)   # what the buffer holds first
    A_log, dt_bias = A_log.float(), dt_bias.float()

    def run(pool_, status, mixed_, out):
        qpd.quantized_gated_delta_rule_packed_decode(mixed_, a, b, A_log, dt_bias, K ** -0.5, *pool_, out, idx,
                                                     use_qk_l2norm_in_kernel=True, resid_fmt=1, status=status)

    def fresh_out():
        return torch.full((B, 1, HV, V), float("nan"), dtype=torch.bfloat16, device=DEV)

    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    good, out_good = [x.clone() for x in st], fresh_out()
    run(good, status, mixed, out_good)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    twin, out_twin, buf = [x.clone() for x in st], fresh_out(), early.clone()
    side = torch.cuda.Stream(DEV)
    with wait_test_library():
        lib = _lib.load_library()
        lib.carry_gdn_test_late_writer.argtypes = [C.c_void_p, C.c_void_p, C.c_longlong, C.c_uint, C.c_void_p]
        lib.carry_gdn_test_late_writer.restype = C.c_int
        with torch.cuda.stream(side):                 # once outside a graph: first-call set-up of the twin
            run([x.clone() for x in st], torch.zeros(1, dtype=torch.int32, device=DEV), mixed, fresh_out())
        torch.cuda.synchronize()
        # writer and decode call as neighbours in one graph: no host time between the two launches
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            rc = lib.carry_gdn_test_late_writer(buf.data_ptr(), mixed.data_ptr(), buf.numel() * buf.element_size(), 50000,
                                                torch.cuda.current_stream().cuda_stream)
            run(twin, status, buf, out_twin)
        assert rc == 0
        status.zero_()
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
    code = int(status.item())
    assert code & (1 << 30), "the decode call never saw its inputs change: the race this test is about did not happen"
    assert code & ~(1 << 30) == _lib.STATUS_TIMEOUT      # the twin's sabotaged tile 1, as in every run of it
    assert torch.equal(buf, mixed)
    ctas = torch.cuda.get_device_properties(0).multi_processor_count
    tile = torch.arange(B * HV, device=DEV).view(B, HV)
    keep = (tile % ctas) != 1
    assert torch.equal(out_twin[:, 0][keep].float(), out_good[:, 0][keep].float())
    rows = idx.long()
    for x_twin, x_good in zip(twin, good):
        assert torch.equal(x_twin[rows][keep], x_good[rows][keep])


def test_multi_token_kernel_wait_runs_out():
    from carrykernel_b200 import _lib
    qpd, (B, H, HV, K, V), st, idx = _slot_case(1, "head")
    T = 2
    toks = [make_packed_inputs(B, H, HV, K, V, seed=20 + t, dtype=torch.bfloat16) for t in range(T)]
    mixed = torch.stack([x[0] for x in toks], 1).to(DEV)
    a = torch.stack([x[1] for x in toks], 1).to(DEV)
    b = torch.stack([x[2] for x in toks], 1).to(DEV)
    A_log, dt_bias = toks[0][3].to(DEV), toks[0][4].to(DEV)

    def run(pool, status):
        out = torch.full((B, T, HV, V), float("nan"), dtype=torch.bfloat16, device=DEV)
        qpd.quantized_gated_delta_rule_packed_decode_multi(mixed, a, b, A_log, dt_bias, K ** -0.5, *pool, out, idx,
                                                           use_qk_l2norm_in_kernel=True, resid_fmt=1, status=status)
        torch.cuda.synchronize()
        return out

    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    good = [x.clone() for x in st]
    out_good = run(good, status)
    assert int(status.item()) == 0
    bad = [x.clone() for x in st]
    with wait_test_library():
        out_bad = run(bad, status)
    assert int(status.item()) == _lib.STATUS_TIMEOUT
    slot, head = int(idx[0]), 1
    assert torch.isnan(out_bad[0, :, head].float()).all()
    for x_bad, x0 in zip(bad, st):
        assert torch.equal(x_bad[slot, head], x0[slot, head])
    keep = torch.ones(B, HV, dtype=torch.bool, device=DEV)
    keep[0, head] = False
    assert torch.equal(out_bad.transpose(1, 2)[keep], out_good.transpose(1, 2)[keep])
    mask = torch.ones(st[0].shape[0], HV, dtype=torch.bool, device=DEV)
    mask[slot, head] = False
    for x_bad, x_good in zip(bad, good):
        assert torch.equal(x_bad[mask], x_good[mask])


def test_statequant_layout_kernel_wait_runs_out():
    from carrykernel_b200 import _lib
    from carrykernel_b200.statequant import kernel as sq
    B, HV, K, V = 3, 8, 128, 128
    h0, q, k, v, alpha, beta = seeded_inputs(B, HV, K, V, seed=4, alpha_mode="gated")
    st = [x.to(DEV) for x in orc.init_quant_state(h0, 8, orc.RES_INT8)]
    acts = [x.to(DEV) for x in (q, k, v, alpha, beta)]

    def run(status):
        outs = (torch.full((B, HV, V), float("nan"), device=DEV), torch.full_like(st[0], 77),
                torch.full_like(st[1], -1.0), torch.full_like(st[2], 77), torch.full_like(st[3], -1.0))
        sq.quant_step_into(*st, *acts, outs, 8, orc.RES_INT8, "v", "v", status=status)
        torch.cuda.synchronize()
        return outs

    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    good = run(status)
    assert int(status.item()) == 0
    with wait_test_library():
        bad = run(status)
    assert int(status.item()) == _lib.STATUS_TIMEOUT
    n, head = 0, 1
    assert torch.isnan(bad[0][n, head]).all()
    assert torch.all(bad[1][n, head] == 77) and torch.all(bad[2][n, head] == -1) and torch.all(bad[3][n, head] == 77)
    keep = torch.ones(B, HV, dtype=torch.bool, device=DEV)
    keep[n, head] = False
    for x_bad, x_good in zip(bad, good):
        assert torch.equal(x_bad[keep], x_good[keep])
