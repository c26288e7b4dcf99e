"""The N > 1 path on CPU: two gloo ranks shard a batch by slot ownership, each
steps its own shard with the CPU oracle (standing in for the GPU kernel, which
cannot run here), and the gathered result must equal the unsharded step.  Also
checks the partition itself and the max-over-ranks timing reduction."""

from __future__ import annotations

import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT

from carrykernel_b200 import sharding


def test_shard_range_is_a_disjoint_cover():
    for n in (0, 1, 7, 64, 257):
        for world in (1, 2, 3, 8):
            spans = [sharding.shard_range(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            for (a, b), (c, d) in zip(spans, spans[1:]):
                assert b == c
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.shard_range(4, 2, 2)


def test_shard_requests_by_slot_ownership():
    num_slots = 11                                   # slot 0 is padding, 10 real slots
    ids = torch.tensor([5, 0, 10, 1, 6, -1, 3], dtype=torch.int32)
    seen = torch.zeros(len(ids), dtype=torch.int32)
    for rank in range(3):
        rows, local = sharding.shard_requests(ids, num_slots, 3, rank)
        seen[rows] += 1
        lo, hi = sharding.shard_range(num_slots - 1, 3, rank)
        for r, l in zip(rows.tolist(), local.tolist()):
            g = int(ids[r])
            if g <= 0:
                assert rank == 0 and l == 0
            else:
                assert lo + 1 <= g < hi + 1 and l == g - lo
        assert max(local.tolist(), default=0) < sharding.local_pool_slots(num_slots, 3, rank)
    assert torch.all(seen == 1)                      # every request served exactly once


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, tmpdir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from oracle import gdn_oracle as orc
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)                          # same global problem on every rank
        B, H, HV, K, V, num_slots = 6, 2, 4, 32, 16, 9
        pool = torch.randn(num_slots, HV, V, K) * 0.1
        ids = torch.tensor([4, 8, 0, 1, 5, 2], dtype=torch.int32)
        mixed = torch.randn(B, 2 * H * K + HV * V)
        a, b = torch.randn(B, HV), torch.randn(B, HV)
        A_log, dt_bias = torch.randn(HV) * 0.2, torch.randn(HV) * 0.1

        # unsharded reference
        full = list(orc.init_quantized_pool(num_slots, HV, V, K, h0=pool, resid_fmt=orc.RESID_INT4,
                                            resid_scale="head"))
        out_full = torch.empty(B, 1, HV, V)
        orc.packed_decode_step(mixed, a, b, A_log, dt_bias, K ** -0.5, *full, out_full, ids,
                               use_qk_l2norm_in_kernel=True, resid_fmt=orc.RESID_INT4)

        # this rank's shard: its block of slots (re-based, slot 0 stays padding) and its rows
        rows, local_ids = sharding.shard_requests(ids, num_slots, world, rank)
        lo, hi = sharding.shard_range(num_slots - 1, world, rank)
        keep = torch.cat([torch.zeros(1, dtype=torch.long), torch.arange(lo + 1, hi + 1)])
        local = list(orc.init_quantized_pool(num_slots, HV, V, K, h0=pool, resid_fmt=orc.RESID_INT4,
                                             resid_scale="head"))
        local = [t[keep].clone() for t in local]
        assert local[0].shape[0] == sharding.local_pool_slots(num_slots, world, rank)
        out_local = torch.empty(len(rows), 1, HV, V)
        orc.packed_decode_step(mixed[rows], a[rows], b[rows], A_log, dt_bias, K ** -0.5, *local,
                               out_local, local_ids, use_qk_l2norm_in_kernel=True,
                               resid_fmt=orc.RESID_INT4)

        gathered = sharding.gather_rows(rows, out_local, B)
        assert torch.equal(gathered, out_full), "sharded outputs differ from the unsharded step"
        for t_local, t_full in zip(local, full):
            assert torch.equal(t_local[1:], t_full[lo + 1:hi + 1]), "a shard's pool differs"

        slowest = sharding.max_over_ranks(0.25 * (rank + 1))
        assert abs(slowest - 0.25 * world) < 1e-12
        dist.barrier()
        open(os.path.join(tmpdir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_match_the_unsharded_step(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
