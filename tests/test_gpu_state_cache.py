"""Life cycle of requests in the slot cache, on the GPU: prefill hand-off,
decode, preemption to the spill pool and resumption in another slot, speculative
tokens through the multi-token call with a rollback, prefix fork.  The pools of
the interrupted requests must end bit for bit equal to those of the same token
streams applied without interruption -- state codes, state scales, residual codes
and residual scales, in every layer (the guarantee carrykernel asks of the cache
wiring, vllm_integration/quantized_packed_decode.py:50-54) -- and that
uninterrupted chain must itself track the CPU oracle."""

from __future__ import annotations

import pytest
import torch

from oracle import gdn_oracle as orc
from parity import make_packed_inputs

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("resid_fmt,rscale", [(orc.RESID_INT4, "head"), (orc.RESID_INT8, "v")])
def test_preempt_resume_speculate_rollback_fork(resid_fmt, rscale):
    from carrykernel_b200.vllm_integration import quantized_packed_decode as qpd
    from carrykernel_b200.vllm_integration import state_cache, state_pool
    L, H, HV, K, V, T = 2, 2, 4, 128, 128, 8
    scale = K ** -0.5
    g = torch.Generator().manual_seed(21)
    h0 = [torch.randn(2, HV, V, K, generator=g) * 0.1 for _ in range(L)]            # prefill states of A and B
    toks = [[make_packed_inputs(2, H, HV, K, V, seed=1000 + 10 * t + l) for l in range(L)] for t in range(T)]
    A_log, dt_bias = toks[0][0][3].to(DEV), toks[0][0][4].to(DEV)

    def step(pools, idx, rows, t):
        """one token (index t) of the requests in `rows` (0 = A, 1 = B) through every layer"""
        outs = []
        for l in range(L):
            mixed, a, b, _, _ = toks[t][l]
            out = torch.empty(len(rows), 1, HV, V, device=DEV)
            qpd.quantized_gated_delta_rule_packed_decode(mixed[rows].to(DEV), a[rows].to(DEV), b[rows].to(DEV),
                                                         A_log, dt_bias, scale, *pools[l], out, idx,
                                                         use_qk_l2norm_in_kernel=True, resid_fmt=resid_fmt)
            outs.append(out)
        return outs

    def multi(pools, idx, row, ts):
        """tokens `ts` of one request in one multi-token call per layer"""
        for l in range(L):
            mixed = torch.stack([toks[t][l][0][row] for t in ts])[None].to(DEV)
            a = torch.stack([toks[t][l][1][row] for t in ts])[None].to(DEV)
            b = torch.stack([toks[t][l][2][row] for t in ts])[None].to(DEV)
            out = torch.empty(1, len(ts), HV, V, device=DEV)
            qpd.quantized_gated_delta_rule_packed_decode_multi(mixed, a, b, A_log, dt_bias, scale, *pools[l], out, idx,
                                                               use_qk_l2norm_in_kernel=True, resid_fmt=resid_fmt)

    # ---- the uninterrupted run: a plain pool, A in slot 1, B in slot 2, eight tokens each
    plain = [qpd.init_quantized_state(3, HV, V, K, DEV, resid_fmt=resid_fmt, resid_scale=rscale) for _ in range(L)]
    both = torch.tensor([1, 2], dtype=torch.int32, device=DEV)
    for l in range(L):
        state_pool.store_state(h0[l].to(DEV), plain[l], both, resid_fmt=resid_fmt, keep_error=True)
    start = [[x.clone() for x in pool] for pool in plain]
    for t in range(T):
        step(plain, both, [0, 1], t)

    # ---- the same token streams through the cache, with interruptions
    cache = state_cache.SlotCache(L, 4, HV, V, K, DEV, resid_fmt, rscale, spill_slots=4)
    cache.allocate("A"); cache.allocate("B")
    for l in range(L):
        state_pool.store_state(h0[l].to(DEV), cache.pools[l], cache.indices(["A", "B"]), resid_fmt=resid_fmt,
                               keep_error=True)
    for t in range(3):
        step(cache.pools, cache.indices(["A", "B"]), [0, 1], t)
    old_slot = cache.slot("A")
    cache.preempt("A")                                       # A leaves after its third token
    cache.allocate("C")                                      # another request takes A's slot and scribbles on it
    assert cache.slot("C") == old_slot
    for pool in cache.pools:
        for x in pool:
            x[old_slot] = 7
    step(cache.pools, cache.indices(["B"]), [1], 3)          # B goes on alone
    token = cache.checkpoint("B")                            # four speculative tokens for B ...
    multi(cache.pools, cache.indices(["B"]), 1, [4, 5, 6, 7])
    cache.rollback(token)                                    # ... two are rejected: back to the checkpoint,
    multi(cache.pools, cache.indices(["B"]), 1, [4, 5])      # the two accepted ones are applied again
    assert cache.resume("A") != old_slot
    for t in range(3, 6):
        step(cache.pools, cache.indices(["A"]), [0], t)      # A catches up on its own
    for t in (6, 7):
        step(cache.pools, cache.indices(["A", "B"]), [0, 1], t)
    cache.free("C")
    cache.fork("A", "D")                                     # a request that starts from A's state
    torch.cuda.synchronize()

    names = ("state codes", "state scales", "residual codes", "residual scales")
    for l in range(L):
        for x_cache, x_plain, name in zip(cache.pools[l], plain[l], names):
            assert torch.equal(x_cache[cache.slot("A")], x_plain[1]), f"layer {l}: A's {name} differ"
            assert torch.equal(x_cache[cache.slot("B")], x_plain[2]), f"layer {l}: B's {name} differ"
            assert torch.equal(x_cache[cache.slot("D")], x_plain[1]), f"layer {l}: the fork's {name} differ"
    assert cache.pages_in_use() == 3 * L                     # A, B, D; every spill slot was given back

    # ---- the uninterrupted GPU chain against the CPU oracle, free running (the reference's own bound for a
    # quantized chain against its oracle is 5e-2 relative, test_quantized_packed_decode.py:149-150)
    rel = lambda x, y: ((x - y).norm() / (y.norm() + 1e-12)).item()
    for l in range(L):
        cpu = [x.cpu().clone() for x in start[l]]
        for t in range(T):
            mixed, a, b, _, _ = toks[t][l]
            orc.packed_decode_step(mixed, a, b, A_log.cpu(), dt_bias.cpu(), scale, *cpu, torch.empty(2, 1, HV, V),
                                   torch.tensor([1, 2], dtype=torch.int32), use_qk_l2norm_in_kernel=True,
                                   resid_fmt=resid_fmt)
        got = orc.dequant_pool_state(plain[l][0].cpu()[1:], plain[l][1].cpu()[1:])
        want = orc.dequant_pool_state(cpu[0][1:], cpu[1][1:])
        assert rel(got, want) < 5e-3, f"layer {l}: chained state drifted from the oracle: {rel(got, want):.2e}"
