"""Strong scaling on real GPUs: one global batch, its slots split over the ranks
(``carrykernel_b200.sharding``), every rank stepping its shard with the CUDA
kernel on its own GPU.  The gathered outputs and every rank's block of the pool
must equal a one-GPU run of the whole batch bit for bit: a (slot, head) tile's
arithmetic does not depend on which other requests share the launch.

Needs two GPUs (skipped otherwise); one NCCL process per GPU, used only to
gather the results."""

from __future__ import annotations

import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, tmpdir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from carrykernel_b200 import sharding
    from carrykernel_b200.vllm_integration import quantized_packed_decode as qpd
    from parity import make_packed_inputs
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        B, H, HV, K, V, num_slots, steps = 24, 2, 4, 128, 128, 41, 3
        g = torch.Generator().manual_seed(0)              # the same global problem on every rank
        pool = torch.randn(num_slots, HV, V, K, generator=g) * 0.1
        ids = (torch.randperm(num_slots - 1, generator=g)[:B] + 1).to(torch.int32)
        ids[5] = 0                                        # one padding request
        acts = [make_packed_inputs(B, H, HV, K, V, seed=50 + t, dtype=torch.bfloat16) for t in range(steps)]

        def run(pool_tensors, idx, rows):
            st = [x.to(dev) for x in pool_tensors]
            outs = []
            for mixed, a, b, A_log, dt_bias in acts:
                out = torch.full((len(rows), 1, HV, V), float("nan"), dtype=torch.bfloat16, device=dev)
                qpd.quantized_gated_delta_rule_packed_decode(
                    mixed[rows].to(dev), a[rows].to(dev), b[rows].to(dev), A_log.to(dev), dt_bias.to(dev),
                    K ** -0.5, *st, out, idx.to(dev), use_qk_l2norm_in_kernel=True, resid_fmt=qpd.RESID_INT4)
                outs.append(out)
            torch.cuda.synchronize(dev)
            return st, torch.stack(outs, 1)               # [rows, steps, 1, HV, V]

        full0 = qpd.init_quantized_state(num_slots, HV, V, K, "cpu", h0=pool, resid_fmt=qpd.RESID_INT4,
                                         resid_scale="head")
        # this rank's shard: its block of slots (re-based; slot 0 stays the padding slot) and its rows
        rows, local_ids = sharding.shard_requests(ids, num_slots, world, rank)
        lo, hi = sharding.shard_range(num_slots - 1, world, rank)
        keep = torch.cat([torch.zeros(1, dtype=torch.long), torch.arange(lo + 1, hi + 1)])
        local, out_local = run([t[keep].clone() for t in full0], local_ids, rows)
        assert local[0].shape[0] == sharding.local_pool_slots(num_slots, world, rank)
        gathered = sharding.gather_rows(rows, out_local.float().cpu(), B)

        # the whole batch on one GPU (every rank does it: the comparison needs no further exchange)
        full, out_full = run([t.clone() for t in full0], ids, torch.arange(B))
        assert torch.equal(gathered, out_full.float().cpu()), "sharded outputs differ from the one-GPU step"
        assert torch.all(gathered[5] == 0)
        for t_local, t_full in zip(local, full):
            assert torch.equal(t_local[1:].cpu(), t_full[lo + 1:hi + 1].cpu()), "a shard's pool differs"
        slowest = sharding.max_over_ranks(0.25 * (rank + 1), dev)
        assert abs(slowest - 0.25 * world) < 1e-12
        dist.barrier()
        open(os.path.join(tmpdir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def test_two_gpus_sharded_equals_one_gpu(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
