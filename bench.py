"""Benchmark of the fused GDN decode step on a quantized state (B200).

Workload (one "step" = one decode step of the whole job on one GPU): 64
requests advance one token through 24 stacked GDN layers.  Each layer has its
own paged pool of 256 slots (+ padding slot 0) addressed through a random
permutation of slot ids; H = HV = 32 heads, K = V = 128; int8 state with
per-V-row scales, packed int4 error-feedback residual with one scale per head;
q | k | v, a, b and the output in bf16; q, k L2-normalised in the kernel; decay
exp(-0.1 softplus(N(0,1))), write strength sigmoid(N(0,1)); the initial state is
64 warm-up steps of the same process.  All inputs are synthetic and seeded.

With N GPUs every rank runs that same per-GPU workload on its own slots (the
pool is sharded by slot: 64 N requests in total, weak scaling) and there is no
collective on the data path; NCCL only carries the barrier and the max over
ranks of the elapsed time.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 20 --warmup 5
    python bench.py --impl reference --steps 20 --warmup 5     # CPU arm: the reference's own CPU step
    python bench.py --strong 512 --layers 4                    # one global batch split over the ranks
    python bench.py --config 5                                 # bit-width / granularity sweep (512 chained steps)
    python bench.py --mode headtohead | statequant | multi | pool   # side measurements

One JSON line goes to stdout (rank 0).  At one GPU the line also carries the
metric's other batch sizes (``sweep``: 128 / 256 / 512 requests per launch) and
the bit-width sweep (``config5``); at N GPUs it carries every rank's time and a
strong-scaling point (512 requests split over the ranks).
"""

from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

H = HV = 32
K = V = 128
LAYERS = 24
BATCH = 64
POOL_SLOTS = 256
WARM_STEPS = 64
E2E_GROUPS = 12
METRIC = "gdn_state_step_throughput"
UNIT = "slot-layer-steps/s"

# algorithmic bytes of one (slot, head) tile, each byte counted once per step:
# int8 state r+w, packed int4 residual r+w, fp32 per-V state scale r+w, per-head
# residual scale r+w, bf16 q, k, v, fp32-equivalent gate inputs (a, b as 2 x 4 B),
# bf16 output row
TILE_BYTES = 2 * K * V + 2 * (K * V // 2) + 2 * V * 4 + 2 * 4 + 2 * K * 2 + V * 2 + 2 * 4 + V * 2
SLOT_LAYER_BYTES = HV * TILE_BYTES + 4          # + the int32 slot id
assert TILE_BYTES == 51216 and SLOT_LAYER_BYTES == 1638916

# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel on this workload
# (64 requests; mean of five steady-state launches, ncu with --cache-control none so that the write-back
# of the results is inside the window), keyed by the SHA-256 of the kernel sources the profiled library
# was built from.  A library built from other sources gets null until it has been profiled again.
NCU_TRAFFIC_BY_SOURCE = {
    "a9aec0e5e4905233": 103_810_000,
}
KERNEL_SOURCES = ("carry_gdn_tile128.cuh", "carry_gdn_slot_tile.inc", "carry_gdn_common.cuh")


def kernel_source_hash():
    import hashlib
    h = hashlib.sha256()
    for name in KERNEL_SOURCES:
        with open(os.path.join(ROOT, "carrykernel_b200", "csrc", name), "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:16]


def parse_args():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["b200", "reference"], default="b200")
    ap.add_argument("--batch", type=int, default=BATCH, help="requests per GPU per step")
    ap.add_argument("--layers", type=int, default=LAYERS)
    ap.add_argument("--resid", choices=["int4", "int8"], default="int4")
    ap.add_argument("--resid-scale", choices=["head", "v"], default="head",
                    help="one residual scale per head (the named workload) or per V row")
    ap.add_argument("--warm-steps", type=int, default=WARM_STEPS,
                    help="untimed steps that build the initial state (64 = the named workload)")
    ap.add_argument("--min-sample-s", type=float, default=0.5,
                    help="keep replaying after the timed region until the clock sampler has run this long "
                         "(0 for profiler runs)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--e2e-groups", type=int, default=E2E_GROUPS,
                    help="layer groups of the host-buffer pipeline (copy in / compute / copy out overlap per group)")
    ap.add_argument("--repeats", type=int, default=5,
                    help="the timed region (--steps replays) is measured this many times; the median is reported")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the batch sweep, the strong-scaling point and the bit-width sweep (profiler runs)")
    ap.add_argument("--strong", type=int, default=0, metavar="B",
                    help="strong scaling: one global batch of B requests, its slots split evenly over the ranks")
    ap.add_argument("--config", type=int, choices=[3, 5], default=3,
                    help="3: the serving step (default); 5: bit-width / granularity sweep over 512 chained steps")
    ap.add_argument("--mode", choices=["step", "headtohead", "statequant", "multi", "pool"], default="step",
                    help="step: the benchmark (default).  Side measurements, one JSON object each: headtohead "
                         "(vLLM's and the reference's kernels beside this library's), statequant (the statequant op "
                         "per residual format), multi (multi-token call), pool (pool store / load / copy)")
    ap.add_argument("--batches", type=int, nargs="+", default=None, help="batch sizes of a side measurement")
    ap.add_argument("--pool-layers", type=int, default=8, help="pools cycled by --mode pool")
    ap.add_argument("--c5-batch", type=int, default=256)
    ap.add_argument("--c5-steps", type=int, default=512)
    return ap.parse_args()


def peak_hbm():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


# ---------------------------------------------------------------------------
# workload
# ---------------------------------------------------------------------------

class Workload:
    """Per-GPU state and inputs of the decode step, resident in HBM."""

    def __init__(self, device, batch, layers, resid, seed, resid_scale="head", shard=None):
        """``shard=(world, rank)``: ``batch`` is a global batch whose slot ids and activations every
        rank draws identically from ``seed``; this rank keeps the requests whose slots it owns
        (``sharding.shard_requests``) in a pool of its share of the slots."""
        from carrykernel_b200.vllm_integration import quantized_packed_decode as qpd
        from carrykernel_b200 import sharding
        self.qpd, self.device, self.layers = qpd, device, layers
        self.resid_fmt = qpd.RESID_INT4 if resid == "int4" else qpd.RESID_INT8
        g = torch.Generator().manual_seed(seed)
        width = 2 * H * K + HV * V
        global_batch, global_slots = batch, max(POOL_SLOTS, batch) + 1
        self.rows = []                                   # strong scaling: this rank's rows of the global batch, per layer
        if shard is not None:
            world, rank = shard
            drawn = []
            for l in range(layers):                      # same draws on every rank
                idx = (torch.randperm(global_slots - 1, generator=g)[:global_batch] + 1).to(torch.int32)
                mixed = torch.randn(global_batch, width, generator=g).to(torch.bfloat16)
                a = torch.randn(global_batch, HV, generator=g).to(torch.bfloat16)
                b = torch.randn(global_batch, HV, generator=g).to(torch.bfloat16)
                rows, local = sharding.shard_requests(idx, global_slots, world, rank)
                drawn.append((local, mixed[rows], a[rows], b[rows]))
                self.rows.append(rows)
            # every layer's shard padded to the largest one with padding requests (slot 0), so that one
            # buffer layout serves all layers
            batch = max(1, max(len(d[0]) for d in drawn))
            slots = sharding.local_pool_slots(global_slots, world, rank)
        else:
            slots = global_slots
        self.batch = batch
        self.num_slots = slots
        self.pools, self.indices, self.mixed, self.a, self.b, self.out = [], [], [], [], [], []
        # activations of all layers in one device buffer, outputs in another (per-layer views into
        # them), so that the host-buffer path can move a group of layers with one copy
        def up(x):
            return (x + 255) // 256 * 256
        seg = [("mixed", (batch, width), torch.bfloat16), ("a", (batch, HV), torch.bfloat16),
               ("b", (batch, HV), torch.bfloat16), ("idx", (batch,), torch.int32)]
        self.in_layer_bytes = sum(up(math.prod(shape) * torch.empty((), dtype=dt).element_size()) for _, shape, dt in seg)
        self.out_layer_bytes = up(batch * HV * V * 2)
        self.in_dev = torch.zeros(layers * self.in_layer_bytes, dtype=torch.uint8, device=device)
        self.out_dev = torch.zeros(layers * self.out_layer_bytes, dtype=torch.uint8, device=device)
        self.in_bytes_useful = layers * sum(math.prod(shape) * torch.empty((), dtype=dt).element_size()
                                            for _, shape, dt in seg)
        self.out_bytes_useful = layers * batch * HV * V * 2

        def view(buf, off, shape, dt):
            n = math.prod(shape) * torch.empty((), dtype=dt).element_size()
            return buf[off:off + n].view(dt).view(shape)

        for l in range(layers):
            self.pools.append(qpd.init_quantized_state(slots, HV, V, K, device,
                                                       resid_fmt=self.resid_fmt, resid_scale=resid_scale))
            off = l * self.in_layer_bytes
            views = {}
            for name, shape, dt in seg:
                views[name] = view(self.in_dev, off, shape, dt)
                off += up(math.prod(shape) * torch.empty((), dtype=dt).element_size())
            if shard is not None:
                local, mixed_l, a_l, b_l = drawn[l]
                n = len(local)
                views["idx"].zero_(); views["mixed"].zero_(); views["a"].zero_(); views["b"].zero_()
                views["idx"][:n].copy_(local); views["mixed"][:n].copy_(mixed_l)
                views["a"][:n].copy_(a_l); views["b"][:n].copy_(b_l)
            else:
                views["idx"].copy_((torch.randperm(slots - 1, generator=g)[:batch] + 1).to(torch.int32))
                views["mixed"].copy_(torch.randn(batch, width, generator=g).to(torch.bfloat16))
                views["a"].copy_(torch.randn(batch, HV, generator=g).to(torch.bfloat16))
                views["b"].copy_(torch.randn(batch, HV, generator=g).to(torch.bfloat16))
            self.indices.append(views["idx"]); self.mixed.append(views["mixed"])
            self.a.append(views["a"]); self.b.append(views["b"])
            self.out.append(view(self.out_dev, l * self.out_layer_bytes, (batch, 1, HV, V), torch.bfloat16))
        self.A_log = torch.full((HV,), math.log(0.1), device=device)
        self.dt_bias = torch.zeros(HV, device=device)
        self.scale = K ** -0.5
        # alternative activations, so the warm-up process is not one repeated token
        self.warm_mixed = [torch.randn(batch, width, generator=g).to(torch.bfloat16).to(device) for _ in range(4)]

    def layer_step(self, l, mixed=None, a=None, b=None, idx=None, out=None):
        self.qpd.quantized_gated_delta_rule_packed_decode(
            self.mixed[l] if mixed is None else mixed, self.a[l] if a is None else a,
            self.b[l] if b is None else b, self.A_log, self.dt_bias, self.scale,
            *self.pools[l], self.out[l] if out is None else out,
            self.indices[l] if idx is None else idx,
            use_qk_l2norm_in_kernel=True, resid_fmt=self.resid_fmt)

    def step(self):
        for l in range(self.layers):
            self.layer_step(l)

    def warm_state(self, steps=WARM_STEPS):
        for t in range(steps):
            for l in range(self.layers):
                self.layer_step(l, mixed=self.warm_mixed[(t + l) % 4])
        torch.cuda.synchronize(self.device)


# ---------------------------------------------------------------------------
# measurement helpers
# ---------------------------------------------------------------------------

class ClockSampler:
    """nvidia-smi clock and throttle-reason samples of one GPU during a region."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index, self.proc, self.path = gpu_index, None, None

    def start(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_index), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"], stdout=f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in open(self.path):
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def physical_gpu_index(local_rank):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        ids = [x for x in vis.split(",") if x.strip()]
        if local_rank < len(ids) and ids[local_rank].strip().isdigit():
            return int(ids[local_rank])
    return local_rank


def time_graph(graph, steps, device):
    """Device time of ``steps`` replays, CUDA events on the launching stream."""
    stream = torch.cuda.current_stream(device)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(device)
    start.record(stream)
    for _ in range(steps):
        graph.replay()
    end.record(stream)
    torch.cuda.synchronize(device)
    return start.elapsed_time(end) * 1e-3


def e2e_run(wl, steps, warmup, groups, kernels=True, repeats=1):
    """The same step through the public call with HOST buffers.  Every step copies all activations and
    slot ids from pinned host memory to the device, runs the 24 layer calls, and copies every output
    row back to pinned host memory; the step ends when the host holds all outputs (stream
    synchronise).  Layers move in `groups` groups: while one group computes, the next group's inputs
    are already on their way in and the previous group's outputs on their way out, each on its own
    stream.  The whole step -- copies, layer calls through the public function, the events that order
    them -- is captured once as one CUDA graph and replayed per step, as a serving engine would.  The
    state pools stay in HBM between steps: they are the recurrent state.  ``kernels=False`` replays the
    very same graph shape without the layer calls: the floor that the host copies alone set."""
    dev = wl.device
    L = wl.layers
    groups = max(1, min(groups, L))
    bounds = [(L * g // groups, L * (g + 1) // groups) for g in range(groups)]
    in_host = wl.in_dev.cpu().pin_memory()
    out_host = torch.empty(wl.out_dev.shape, dtype=torch.uint8).pin_memory()
    s_in, s_run, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)

    def enqueue_step():
        s_in.wait_stream(s_run)                         # fork (inside a capture: joins the other streams to it)
        s_out.wait_stream(s_run)
        for lo, hi in bounds:
            a, b = lo * wl.in_layer_bytes, hi * wl.in_layer_bytes
            with torch.cuda.stream(s_in):
                wl.in_dev[a:b].copy_(in_host[a:b], non_blocking=True)
            s_run.wait_stream(s_in)
            if kernels:
                with torch.cuda.stream(s_run):
                    for l in range(lo, hi):
                        wl.layer_step(l)
            s_out.wait_stream(s_run)
            a, b = lo * wl.out_layer_bytes, hi * wl.out_layer_bytes
            with torch.cuda.stream(s_out):
                out_host[a:b].copy_(wl.out_dev[a:b], non_blocking=True)
        s_run.wait_stream(s_in)                         # join
        s_run.wait_stream(s_out)

    torch.cuda.synchronize(dev)
    with torch.cuda.stream(s_run):
        enqueue_step()                                  # eager once: loads the library, warms the allocator
    torch.cuda.synchronize(dev)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=s_run):
        enqueue_step()

    def one_step():
        graph.replay()
        torch.cuda.synchronize(dev)

    for _ in range(warmup):
        one_step()
    walls = []
    for _ in range(max(1, repeats)):                    # the region of `steps` steps, several times: the median
        torch.cuda.synchronize(dev)                     # keeps one hiccup of a shared host out of the figure
        t0 = time.perf_counter()
        for _ in range(steps):
            one_step()
        torch.cuda.synchronize(dev)
        walls.append(time.perf_counter() - t0)
    return median(walls), wl.in_bytes_useful, wl.out_bytes_useful


# ---------------------------------------------------------------------------
# CPU arm: the oracle port, timed on the host cores; doubles as the checker
# ---------------------------------------------------------------------------

def cpu_sample_inputs(batch, layers, resid, seed=1234, resid_scale="head"):
    """CPU copy of a bounded sample of the workload (same shapes and laws)."""
    from oracle import gdn_oracle as orc
    g = torch.Generator().manual_seed(seed)
    fmt = orc.RESID_INT4 if resid == "int4" else orc.RESID_INT8
    width = 2 * H * K + HV * V
    sample = []
    for _ in range(layers):
        pool = torch.randn(batch + 1, HV, V, K, generator=g) * 0.124
        st = list(orc.init_quantized_pool(batch + 1, HV, V, K, h0=pool, resid_fmt=fmt, resid_scale=resid_scale))
        idx = (torch.randperm(batch, generator=g) + 1).to(torch.int32)
        mixed = torch.randn(batch, width, generator=g).to(torch.bfloat16)
        a = torch.randn(batch, HV, generator=g).to(torch.bfloat16)
        b = torch.randn(batch, HV, generator=g).to(torch.bfloat16)
        sample.append((st, idx, mixed, a, b))
    return sample, fmt


def cpu_oracle_pass(sample, fmt):
    from oracle import gdn_oracle as orc
    A_log = torch.full((HV,), math.log(0.1))
    dt_bias = torch.zeros(HV)
    outs = []
    for st, idx, mixed, a, b in sample:
        out = torch.empty(mixed.shape[0], 1, HV, V, dtype=torch.bfloat16)
        orc.packed_decode_step(mixed, a, b, A_log, dt_bias, K ** -0.5, *st, out, idx,
                               use_qk_l2norm_in_kernel=True, resid_fmt=fmt)
        outs.append(out)
    return outs


def time_cpu_oracle(batch, layers, resid, passes, warm=1, resid_scale="head"):
    """Seconds per pass of the oracle over the sample (all host threads)."""
    torch.set_num_threads(os.cpu_count() or 1)
    sample, fmt = cpu_sample_inputs(batch, layers, resid, resid_scale=resid_scale)
    for _ in range(warm):
        cpu_oracle_pass(sample, fmt)
    times = []
    for _ in range(passes):
        t0 = time.perf_counter()
        cpu_oracle_pass(sample, fmt)
        times.append(time.perf_counter() - t0)
    return sum(times) / len(times), batch * layers


def cpu_baseline_and_parity(wl, resid, resid_scale="head"):
    """Time the oracle on a bounded sample and, on that same sample, check the
    GPU step against it (validate before timing)."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from oracle import gdn_oracle as orc
    import parity
    s_batch, s_layers = min(wl.batch, 16), 2
    sample, fmt = cpu_sample_inputs(s_batch, s_layers, resid, resid_scale=resid_scale)
    # GPU result on the sample (teacher-forced from the same start state)
    dev = wl.device
    f_state = f_resid = 0.0
    gpu_outs, gpu_pools = [], []
    for st, idx, mixed, a, b in sample:
        pool = [x.clone().to(dev) for x in st]
        out = torch.empty(s_batch, 1, HV, V, dtype=torch.bfloat16, device=dev)
        wl.qpd.quantized_gated_delta_rule_packed_decode(
            mixed.to(dev), a.to(dev), b.to(dev), wl.A_log, wl.dt_bias, wl.scale, *pool, out, idx.to(dev),
            use_qk_l2norm_in_kernel=True, resid_fmt=wl.resid_fmt)
        gpu_outs.append(out.cpu()); gpu_pools.append([x.cpu() for x in pool])
    torch.set_num_threads(os.cpu_count() or 1)
    t0 = time.perf_counter()
    cpu_outs = cpu_oracle_pass(sample, fmt)
    first = time.perf_counter() - t0
    for (st, idx, *_), go, gp, co in zip(sample, gpu_outs, gpu_pools, cpu_outs):
        parity.assert_close(go, co, "bench: out", rtol=8e-3, atol=1e-4)
        fs, fr = parity.check_pool(gp, st, fmt == orc.RESID_INT4, idx.tolist(), orc.unpack_int4, "bench")
        f_state, f_resid = max(f_state, fs), max(f_resid, fr)
    # timing: enough passes for roughly 10-20 s of CPU work
    passes = max(2, min(20, int(12.0 / max(first, 1e-3))))
    sec, units = time_cpu_oracle(s_batch, s_layers, resid, passes, warm=0, resid_scale=resid_scale)
    return ({"value": units / sec, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
             "sample": f"{s_layers} layers x {s_batch} requests of the same workload "
                       f"({units} slot-layer-steps per pass, {passes} passes, torch CPU oracle)"},
            {"state_flip_frac": f_state, "resid_flip_frac": f_resid, "checked_slot_layer_steps": units,
             "limit": parity.MAX_FLIP_FRAC})


def run_reference_arm(args, rank):
    """--impl reference: the reference's CPU implementation of the step on the host cores.

    With the staged copy of the reference present (``oracle/make_ref.py``), its own
    ``gdn_quant_step_torch`` (statequant/kernel.py:149-178) is what runs: the fused step in its
    ``[B, HV, K, V]`` layout with the int8 residual and per-column scales, the only CPU code the
    reference has for this step (the slot-indexed int4 / per-head variant exists there as a Triton
    kernel only).  Same state size per slot-layer-step, same input laws.  Without the copy the
    oracle port of the slot-indexed step is timed instead.  One step is a bounded sample: 1 layer
    x 16 requests."""
    if rank != 0:
        return
    from oracle import make_ref
    s_batch, s_layers = 16, 1
    torch.set_num_threads(os.cpu_count() or 1)
    ref = make_ref.ref_path()
    if ref is not None:
        sys.path.insert(0, ref)
        from statequant import kernel as rk
        g = torch.Generator().manual_seed(1234)
        h0 = torch.randn(s_batch, HV, K, V, generator=g) * 0.124
        st = rk.init_quant_state(h0, 8, rk.RES_INT8)
        q = torch.nn.functional.normalize(torch.randn(s_batch, HV, K, generator=g), dim=-1)
        k = torch.nn.functional.normalize(torch.randn(s_batch, HV, K, generator=g), dim=-1)
        v = torch.randn(s_batch, HV, V, generator=g)
        alpha = torch.exp(-0.1 * torch.nn.functional.softplus(torch.randn(s_batch, HV, generator=g)))
        beta = torch.sigmoid(torch.randn(s_batch, HV, generator=g))

        def one_pass():
            nonlocal st
            st = rk.gdn_quant_step_torch(*st, q, k, v, alpha, beta, 8, rk.RES_INT8)[1:]
        kind = "reference"
        desc = (f"{s_layers} layer x {s_batch} requests per step through the reference's own CPU step "
                "gdn_quant_step_torch (statequant/kernel.py:149-178; [B,HV,K,V] layout, int8 residual, per-column "
                "scales: the reference has no CPU code for the slot-indexed int4 / per-head step), same state "
                "size and input laws")
    else:
        sample, fmt = cpu_sample_inputs(s_batch, s_layers, args.resid)

        def one_pass():
            cpu_oracle_pass(sample, fmt)
        kind = "port"
        desc = f"{s_layers} layer x {s_batch} requests per step (oracle port; same shapes and input laws)"
    for _ in range(max(args.warmup, 1)):
        one_pass()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        one_pass()
    sec = time.perf_counter() - t0
    units = s_batch * s_layers * args.steps
    value = units / sec
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": workload_config(args, args.batch, args.layers),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": torch.get_num_threads(),
                         "kind": kind, "sample": desc},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def l2_statement(args, batch, layers):
    """Whether a step's working set exceeds the 126 MB L2 (the slots a step touches are the same
    every step, so a small enough set stays cached between steps)."""
    slot = HV * (K * V + (K * V // 2 if args.resid == "int4" else K * V) + V * 4 + 4)
    per_layer, step = batch * slot / 1e6, batch * layers * slot / 1e6
    if step > 2 * 126:
        return (f"inputs larger than L2: each step touches a different {per_layer:.0f} MB of state per layer, "
                f"{step / 1e3:.2f} GB per step against 126 MB of L2")
    kind = "L2-RESIDENT" if step < 0.8 * 126 else "PARTLY L2-RESIDENT"
    return (f"{kind}: a step's state is {step:.1f} MB ({per_layer:.1f} MB per layer) against 126 MB of L2; "
            "not an HBM figure")


def workload_config(args, batch, layers, note=None):
    cfg = {"workload": "slot-indexed GDN decode step: int8 state + packed int4 residual (per-head "
                       "residual scale), 24 layers x 64 requests per GPU, pools of 256 slots"
                       if (args.resid == "int4" and args.resid_scale == "head" and batch == BATCH
                           and layers == LAYERS) else
                       f"slot-indexed GDN decode step, {args.resid} residual",
           "requests_per_gpu": batch, "layers": layers, "H": H, "HV": HV, "K": K, "V": V,
           "pool_slots": POOL_SLOTS, "resid": args.resid,
           "resid_scale": "per-head" if args.resid_scale == "head" else "per-V",
           "activations": "bf16", "parallelism": f"slot-sharded x{args.gpus}, no collective",
           "l2": l2_statement(args, batch, layers)}
    if note:
        cfg["sample"] = note
    return cfg


# ---------------------------------------------------------------------------
# the bit-width / granularity sweep (the bit-width sweep of the named workload configurations (number 5))
# ---------------------------------------------------------------------------

def config5_sweep(batch=256, steps=512, bits=(3, 4, 5, 6, 8), seed=0):
    """State bits in {3,4,5,6,8}; one scale per head without error feedback (``uniform_quantize``,
    statequant/quant.py:23-34) against one scale per V column with an fp32 error-feedback residual
    (``per_axis_quantize(.., -2)`` + ``ErrorFeedback``, statequant/quant.py:37-42,65-80); per-head
    constant decay from U[0.9, 0.999]; ``steps`` chained decode steps through the library's statequant
    calls; relative L2 error of the final dequantised state against the fp32 recurrence
    (``gdn_step_fused_fp32``).  The experiment of experiments/exp2_bits_sweep.py and exp2b_granularity.py
    at serving size; inputs are generated on the device step by step from fixed seeds."""
    from carrykernel_b200.statequant import kernel as sq
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev).manual_seed(seed)
    h0 = torch.randn(batch, HV, K, V, generator=g, device=dev) * 0.1
    alpha = 0.9 + 0.099 * torch.rand(batch, HV, generator=g, device=dev)

    def step_inputs(t):
        gt = torch.Generator(device=dev).manual_seed(seed * 100003 + t)
        q = torch.randn(batch, HV, K, generator=gt, device=dev)
        k = torch.nn.functional.normalize(torch.randn(batch, HV, K, generator=gt, device=dev), dim=-1)
        v = torch.randn(batch, HV, V, generator=gt, device=dev)
        beta = torch.sigmoid(torch.randn(batch, HV, generator=gt, device=dev))
        return q, k, v, beta

    def timed(fn):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = fn()
        e1.record()
        torch.cuda.synchronize()
        return out, e0.elapsed_time(e1) * 1e3 / steps

    def fp32_chain():
        h = h0.clone()
        for t in range(steps):
            q, k, v, beta = step_inputs(t)
            h, _ = sq.gdn_step_fused_fp32(h, q, k, v, alpha, beta)
        return h

    def quant_chain(nbits, res_fmt, state_scale):
        st = sq.init_quant_state(h0, nbits, res_fmt, state_scale=state_scale)
        for t in range(steps):
            q, k, v, beta = step_inputs(t)
            st = sq.gdn_quant_step_fused(*st, q, k, v, alpha, beta, bits=nbits, res_fmt=res_fmt,
                                         state_scale=state_scale)[1:]
        codes, scale = st[0], st[1]
        return codes.float() * (scale[..., None, :] if state_scale == "v" else scale[..., None, None])

    h_ref, us_ref = timed(fp32_chain)
    norm = h_ref.norm()
    res = {"batch": batch, "steps": steps, "fp32_us_per_step": us_ref, "rel_l2_error": {}}
    for nbits in bits:
        uni, us_u = timed(lambda: quant_chain(nbits, sq.RES_NONE, "head"))
        err_u = ((uni - h_ref).norm() / norm).item()
        del uni
        ef, us_e = timed(lambda: quant_chain(nbits, sq.RES_FP32, "v"))
        err_e = ((ef - h_ref).norm() / norm).item()
        del ef
        res["rel_l2_error"][str(nbits)] = {"per_head_no_ef": err_u, "per_v_ef": err_e,
                                           "per_head_no_ef_us_per_step": us_u, "per_v_ef_us_per_step": us_e}
    torch.cuda.empty_cache()
    return res


def run_config5(args):
    res = config5_sweep(args.c5_batch, args.c5_steps)
    launches = (1 + 2 * len(res["rel_l2_error"])) * args.c5_steps
    print(json.dumps({
        "metric": "final_state_rel_l2_error_8bit_per_v_ef", "value": res["rel_l2_error"]["8"]["per_v_ef"],
        "unit": "relative L2 error vs the fp32 recurrence", "n_gpus": 1, "steps": args.c5_steps, "warmup": 0,
        "ms_per_step": res["rel_l2_error"]["8"]["per_v_ef_us_per_step"] * 1e-3, "higher_is_better": False,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "bit-width / granularity sweep: state bits 3,4,5,6,8, per-head scale without error "
                               "feedback vs per-V scale with fp32 error feedback, per-head decay U[0.9,0.999]",
                   "requests": args.c5_batch, "chained_steps": args.c5_steps, "HV": HV, "K": K, "V": V},
        "config5": res, "gpu_launches": launches}))


# ---------------------------------------------------------------------------
# side measurements (--mode): not the headline, one JSON object each
# ---------------------------------------------------------------------------

def _events_us(call, steps, warmup):
    """us per call: CUDA events around ``steps`` calls after ``warmup``."""
    for _ in range(warmup):
        call()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(steps):
        call()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / steps * 1e3


def _graph_us(fn, reps=10):
    """us per ``fn()``: ``reps`` calls captured into one CUDA graph, two timed replays."""
    for _ in range(3):
        fn()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(reps):
            fn()
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    graph.replay()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (2 * reps)


def headtohead(batches=(1, 8, 16, 64, 256), steps=200, warmup=50, seed=0):
    """Head-to-head against vLLM's own packed-decode kernel and the reference's Triton kernel.

    The comparison of carrykernel's ``modal_vllm_headtohead.py:105-205``: vLLM's
    ``fused_recurrent_gated_delta_rule_packed_decode`` with an fp32 and with a bf16 state (its
    serving default) against this library's int8-state step, Qwen-GDN shapes (H = 16 key heads,
    HV = 32 value heads, K = V = 128), every tensor cast once outside the timed region, CUDA events
    around ``steps`` calls after ``warmup``.  Added here: the reference's own slot-indexed Triton
    kernel (from the staged copy, when present) as a third arm on the same GPU; the reference's
    ``sanity()`` guard (``:94-103``: a bf16 state slower than 1.2x the fp32 one means the harness
    is suspect and the bf16 ratio is withheld); and a numeric line per batch -- one step of vLLM's
    fp32-state kernel and of this library from the same dequantised state, fp32 activations and
    outputs, largest absolute and relative difference of ``out``.  vLLM's kernel and the reference's
    are comparators only; nothing of either is used by the product."""
    from carrykernel_b200.vllm_integration import quantized_packed_decode as qpd
    from oracle import make_ref
    HH, HHV = 16, 32
    try:
        from vllm.model_executor.layers.fla.ops.fused_recurrent import (
            fused_recurrent_gated_delta_rule_packed_decode as vllm_fn)
        why = None
    except Exception as exc:                           # depends on the image
        vllm_fn, why = None, f"{type(exc).__name__}: {exc}"
    ref_fn = None
    if make_ref.ref_path() is not None:
        sys.path.insert(0, make_ref.ref_path())
        try:
            from vllm_integration import quantized_packed_decode as rqpd
            ref_fn = rqpd.quantized_gated_delta_rule_packed_decode if rqpd.HAS_TRITON else None
        except Exception:
            ref_fn = None
    dev = torch.device("cuda")
    torch.manual_seed(seed)
    results = {"H": HH, "HV": HHV, "K": K, "V": V, "steps": steps, "warmup": warmup,
               "gpu": torch.cuda.get_device_name(0), "suspect": []}
    if vllm_fn is None:
        results["vllm"] = f"unavailable: {why}"
    if ref_fn is None:
        results["reference_triton"] = "unavailable: oracle/_ref not staged or Triton missing"
    for B in batches:
        mixed = torch.randn(B, 2 * HH * K + HHV * V, device=dev)
        a = torch.randn(B, HHV, device=dev) * 0.5
        b = torch.randn(B, HHV, device=dev)
        A_log = torch.randn(HHV, device=dev) * 0.2
        dt_bias = torch.randn(HHV, device=dev) * 0.1
        scale = K ** -0.5
        idx = torch.arange(1, B + 1, dtype=torch.int32, device=dev)
        h0 = torch.randn(B + 1, HHV, V, K, device=dev) * 0.1
        row = {}
        mixed_bf, a_bf, b_bf = mixed.bfloat16(), a.bfloat16(), b.bfloat16()
        if vllm_fn is not None:
            for name, state, mx, aa, bb, out_dt in (
                    ("vllm_fp32_state", h0.clone(), mixed, a, b, torch.float32),
                    ("vllm_bf16_state", h0.bfloat16(), mixed_bf, a_bf, b_bf, torch.bfloat16)):
                out = torch.empty(B, 1, HHV, V, device=dev, dtype=out_dt)
                A_, d_ = (A_log, dt_bias) if out_dt == torch.float32 else (A_log.bfloat16(), dt_bias.bfloat16())
                call = lambda state=state, mx=mx, aa=aa, bb=bb, out=out, A_=A_, d_=d_: vllm_fn(
                    mixed_qkv=mx, a=aa, b=bb, A_log=A_, dt_bias=d_, scale=scale, initial_state=state,
                    out=out, ssm_state_indices=idx, use_qk_l2norm_in_kernel=True)
                try:
                    row[name + "_us"] = _events_us(call, steps, warmup)
                except Exception as exc:
                    row[name + "_us"] = None
                    row[name + "_error"] = f"{type(exc).__name__}: {exc}"[:200]
            t32, tbf = row.get("vllm_fp32_state_us"), row.get("vllm_bf16_state_us")
            # the reference's guard: half the traffic must not time slower
            row["bf16_comparison_valid"] = not (t32 and tbf and tbf > 1.2 * t32)
            if not row["bf16_comparison_valid"]:
                results["suspect"].append(B)
        out = torch.empty(B, 1, HHV, V, device=dev, dtype=torch.bfloat16)
        for fmt, name in ((qpd.RESID_INT8, "ours_int8_resid"), (qpd.RESID_INT4, "ours_int4_resid")):
            for rscale in ("v", "head"):
                st = qpd.init_quantized_state(B + 1, HHV, V, K, dev, h0=h0, resid_fmt=fmt, resid_scale=rscale)
                call = lambda st=st, fmt=fmt: qpd.quantized_gated_delta_rule_packed_decode(
                    mixed_bf, a_bf, b_bf, A_log, dt_bias, scale, *st, out, idx,
                    use_qk_l2norm_in_kernel=True, resid_fmt=fmt)
                row[f"{name}_{rscale}_us"] = _events_us(call, steps, warmup)
            if ref_fn is not None:
                st = rqpd.init_quantized_state(B + 1, HHV, V, K, dev, h0=h0, resid_fmt=fmt)
                call = lambda st=st, fmt=fmt: ref_fn(mixed_bf, a_bf, b_bf, A_log, dt_bias, scale, *st, out, idx,
                                                     use_qk_l2norm_in_kernel=True, resid_fmt=fmt)
                row[f"reference_triton_{'int8' if fmt == qpd.RESID_INT8 else 'int4'}_resid_v_us"] = \
                    _events_us(call, steps, warmup)
        # numeric line: one step of both kernels from the same dequantised state, fp32 in and out
        if vllm_fn is not None:
            st = qpd.init_quantized_state(B + 1, HHV, V, K, dev, h0=h0, resid_fmt=qpd.RESID_INT4, resid_scale="head")
            h_deq = st[0].float() * st[1][..., None]
            o_v = torch.full((B, 1, HHV, V), float("nan"), device=dev)
            o_o = torch.full((B, 1, HHV, V), float("nan"), device=dev)
            vllm_fn(mixed_qkv=mixed, a=a, b=b, A_log=A_log, dt_bias=dt_bias, scale=scale, initial_state=h_deq,
                    out=o_v, ssm_state_indices=idx, use_qk_l2norm_in_kernel=True)
            qpd.quantized_gated_delta_rule_packed_decode(mixed, a, b, A_log, dt_bias, scale, *st, o_o, idx,
                                                         use_qk_l2norm_in_kernel=True, resid_fmt=qpd.RESID_INT4)
            torch.cuda.synchronize()
            row["out_max_abs_diff_vs_vllm_fp32"] = float((o_o - o_v).abs().max())
            row["out_max_rel_diff_vs_vllm_fp32"] = float(((o_o - o_v).abs() / (o_v.abs() + 1e-4)).max())
            row["out_mean_abs"] = {"vllm": float(o_v.abs().mean()), "ours": float(o_o.abs().mean())}
        elems = B * HHV * V * K
        row["state_traffic_MB"] = {
            "vllm_fp32": 2 * elems * 4 / 1e6, "vllm_bf16": 2 * elems * 2 / 1e6,
            "ours_int8_resid": (4 * elems + 4 * B * HHV * V * 4) / 1e6,
            "ours_int4_resid": (3 * elems + 4 * B * HHV * V * 4) / 1e6}
        results[f"B{B}"] = row
    return results


def statequant_timing(batches=(8, 64, 256), calls=50):
    """One fused step through the statequant op (``gdn_quant_step_fused``, [B, HV, K, V] layout, HV = 32,
    K = V = 128, fp32 q/k/v, 8-bit state) per residual format and residual-scale granularity, the step
    without error feedback, and the unquantised fp32 step; CUDA events around ``calls`` calls.  The
    figure includes the op's own work per call (five output allocations, the ctypes call)."""
    from carrykernel_b200.statequant import kernel as sq
    dev = torch.device("cuda")
    cases = ((sq.RES_FP32, "v", "fp32"), (sq.RES_FP16, "v", "fp16"), (sq.RES_FP8, "v", "fp8_e5m2"),
             (sq.RES_INT8, "v", "int8_per_v"), (sq.RES_INT8, "head", "int8_per_head"),
             (sq.RES_INT4, "v", "int4_per_v"), (sq.RES_INT4, "head", "int4_per_head"))
    resid_bytes = {sq.RES_FP32: 4, sq.RES_FP16: 2, sq.RES_FP8: 1, sq.RES_INT8: 1, sq.RES_INT4: 0.5}
    res = {"HV": HV, "K": K, "V": V, "gpu": torch.cuda.get_device_name(0)}

    def inputs(B):
        g = torch.Generator().manual_seed(0)
        h0 = (torch.randn(B, HV, K, V, generator=g) * 0.12).to(dev)
        q = torch.randn(B, HV, K, generator=g).to(dev)
        k = (torch.randn(B, HV, K, generator=g) * K ** -0.5).to(dev)
        v = torch.randn(B, HV, V, generator=g).to(dev)
        return h0, q, k, v, torch.full((B, HV), 0.98, device=dev), torch.rand(B, HV, generator=g).to(dev)

    for B in batches:
        row = {}
        for res_fmt, rs, name in cases:
            h0, q, k, v, alpha, beta = inputs(B)
            st = sq.init_quant_state(h0, 8, res_fmt, resid_scale=rs)
            us = _events_us(lambda: sq.gdn_quant_step_fused(*st, q, k, v, alpha, beta, 8, res_fmt, resid_scale=rs),
                            calls, 3)
            row[name] = {"us_per_step": us, "state_GBps": B * HV * K * V * 2 * (1 + resid_bytes[res_fmt]) / us / 1e3}
        for mode in ("v", "head"):
            h0, q, k, v, alpha, beta = inputs(B)
            st = sq.init_quant_state(h0, 8, sq.RES_NONE, state_scale=mode)
            us = _events_us(lambda: sq.gdn_quant_step_fused(*st, q, k, v, alpha, beta, 8, sq.RES_NONE,
                                                            state_scale=mode), calls, 3)
            row[f"no_feedback_scale_per_{mode}"] = {"us_per_step": us, "state_GBps": B * HV * K * V * 2 / us / 1e3}
        h, q, k, v, alpha, beta = inputs(B)
        us = _events_us(lambda: sq.gdn_step_fused_fp32(h, q, k, v, alpha, beta), calls, 3)
        row["fp32_state_unquantised"] = {"us_per_step": us, "state_GBps": B * HV * K * V * 8 / us / 1e3}
        res[f"B{B}"] = row
    return res


def multi_token_timing(batches=(64, 256), tokens=(2, 4, 8), seed=0):
    """Time per token of the multi-token call against single-token calls (slot path, int4 residual,
    per-head scale, bf16), each captured ten times into a CUDA graph."""
    from carrykernel_b200.vllm_integration import quantized_packed_decode as qpd
    dev = torch.device("cuda")
    res = {"H": H, "HV": HV, "K": K, "V": V, "gpu": torch.cuda.get_device_name(0)}
    for B in batches:
        for T in tokens:
            g = torch.Generator().manual_seed(seed)
            slots = B + 1
            pool = torch.randn(slots, HV, V, K, generator=g) * 0.12
            st = [x.to(dev) for x in qpd.init_quantized_state(slots, HV, V, K, "cpu", h0=pool,
                                                              resid_fmt=qpd.RESID_INT4, resid_scale="head")]
            mixed = torch.randn(B, T, 2 * H * K + HV * V, generator=g).to(torch.bfloat16).to(dev)
            a = torch.randn(B, T, HV, generator=g).to(torch.bfloat16).to(dev)
            b = torch.randn(B, T, HV, generator=g).to(torch.bfloat16).to(dev)
            A_log = torch.full((HV,), math.log(0.1), device=dev)
            dt_bias = torch.zeros(HV, device=dev)
            idx = (torch.randperm(slots - 1, generator=g)[:B] + 1).to(torch.int32).to(dev)
            out = torch.empty(B, T, HV, V, dtype=torch.bfloat16, device=dev)
            tmp = torch.empty(B, 1, HV, V, dtype=torch.bfloat16, device=dev)
            per_tok = [(mixed[:, t].contiguous(), a[:, t].contiguous(), b[:, t].contiguous()) for t in range(T)]

            def single():
                for m_, a_, b_ in per_tok:
                    qpd.quantized_gated_delta_rule_packed_decode(m_, a_, b_, A_log, dt_bias, K ** -0.5, *st, tmp, idx,
                                                                 use_qk_l2norm_in_kernel=True, resid_fmt=qpd.RESID_INT4)

            def multi():
                qpd.quantized_gated_delta_rule_packed_decode_multi(mixed, a, b, A_log, dt_bias, K ** -0.5, *st, out, idx,
                                                                   use_qk_l2norm_in_kernel=True, resid_fmt=qpd.RESID_INT4)

            res[f"B{B}_T{T}"] = {"single_token_calls_us_per_token": _graph_us(single) / T,
                                 "multi_token_call_us_per_token": _graph_us(multi) / T}
    return res


def state_pool_timing(batches=(64, 256), layers=8, seed=0):
    """Pool store / load / copy kernels: ``layers`` pools cycled so that one pass exceeds the L2, ten
    passes per CUDA graph.  Bytes per call: store reads the floating-point state and writes the slot,
    load the reverse, copy reads and writes the quantized slot."""
    from carrykernel_b200.vllm_integration import quantized_packed_decode as qpd
    from carrykernel_b200.vllm_integration import state_pool as sp
    dev = torch.device("cuda")
    torch.manual_seed(seed)
    res = {"HV": HV, "K": K, "V": V, "layers": layers, "gpu": torch.cuda.get_device_name(0)}
    slot_bytes = qpd.state_bytes_per_slot(HV, V, K, True, resid_fmt=qpd.RESID_INT4, resid_scale="head")
    for B in batches:
        slots = 2 * B + 1
        pools = [qpd.init_quantized_state(slots, HV, V, K, dev, resid_fmt=qpd.RESID_INT4, resid_scale="head")
                 for _ in range(layers)]
        idx = (torch.randperm(B, device=dev) + 1).to(torch.int32)
        idx2 = idx + B
        row = {}
        for name, dtype, es in (("fp32", torch.float32, 4), ("bf16", torch.bfloat16, 2)):
            hs = [(torch.randn(B, HV, V, K, device=dev) * 0.1).to(dtype) for _ in range(layers)]

            def store(keep):
                for h, pool in zip(hs, pools):
                    sp.store_state(h, pool, idx, resid_fmt=qpd.RESID_INT4, keep_error=keep)

            def load():
                for h, pool in zip(hs, pools):
                    sp.load_state(pool, idx, out=h, resid_fmt=qpd.RESID_INT4)

            bytes_call = B * (HV * V * K * es + slot_bytes)
            for label, fn in ((f"store_{name}", lambda: store(False)),
                              (f"store_{name}_keep_error", lambda: store(True)), (f"load_{name}", load)):
                us = _graph_us(fn) / layers
                row[label] = {"us_per_call": us, "GB_per_s": bytes_call / us / 1e3}
            del hs

        def copy():
            for pool in pools:
                sp.copy_slots(pool, idx, idx2, resid_fmt=qpd.RESID_INT4)

        us = _graph_us(copy) / layers
        row["copy"] = {"us_per_call": us, "GB_per_s": 2 * B * slot_bytes / us / 1e3}
        res[f"B{B}"] = row
    return res


SIDE_MODES = {"headtohead": headtohead, "statequant": statequant_timing, "multi": multi_token_timing,
              "pool": state_pool_timing}


# ---------------------------------------------------------------------------
# main
# ---------------------------------------------------------------------------

def capture_step(wl, device):
    """One decode step (all layers) of ``wl`` as a CUDA graph, warmed."""
    side = torch.cuda.Stream(device)
    with torch.cuda.stream(side):
        wl.step()
    torch.cuda.synchronize(device)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        wl.step()
    return graph


def timed_repeats(graph, steps, repeats, device, world):
    """``repeats`` measurements of ``steps`` replays each; every one is bracketed by a barrier and a
    device synchronise on both sides and reduced to the slowest rank.  Returns (per-repeat job times,
    this rank's own per-repeat times)."""
    import torch.distributed as dist
    from carrykernel_b200.sharding import max_over_ranks
    job, mine = [], []
    for _ in range(repeats):
        if world > 1:
            dist.barrier()
        t = time_graph(graph, steps, device)
        if world > 1:
            dist.barrier()
        mine.append(t)
        job.append(max_over_ranks(t, device))
    return job, mine


def median(xs):
    xs = sorted(xs)
    return xs[len(xs) // 2]


def roofline_of(args, batch, per_launch, traffic=None, kernel="gdn_tile128_kernel"):
    peak, peak_kind = peak_hbm()
    per_slot = SLOT_LAYER_BYTES if args.resid == "int4" else SLOT_LAYER_BYTES + HV * K * V
    if args.resid_scale == "v":
        per_slot += HV * (2 * V * 4 - 8)
    achieved = per_slot * batch / per_launch / 1e9
    return {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
            "peak_kind": f"of {peak_kind}", "frac_of_8000": achieved / 8000.0,
            "bytes_per_launch": per_slot * batch, "traffic": traffic, "kernel": kernel}


def batch_sweep(args, device, batches=(128, 256, 512), layers=4, steps=10, repeats=5):
    """The metric's other batch sizes on this GPU: us per launch, GB/s and fraction of the copy rate
    at 128 / 256 / 512 requests per launch (4 layers each, every step larger than the L2)."""
    out = {}
    for b in batches:
        wl = Workload(device, b, layers, args.resid, seed=77 + b, resid_scale=args.resid_scale)
        wl.warm_state(8)
        graph = capture_step(wl, device)
        for _ in range(3):
            graph.replay()
        job, _ = timed_repeats(graph, steps, repeats, device, 1)
        per_launch = median(job) / (steps * layers)
        r = roofline_of(args, b, per_launch)
        out[str(b)] = {"us_per_launch": per_launch * 1e6, "GBps": r["achieved"], "frac": r["frac"],
                       "frac_of_8000": r["frac_of_8000"], "layers": layers, "steps": steps,
                       "spread_us": [min(job) / (steps * layers) * 1e6, max(job) / (steps * layers) * 1e6]}
        del wl, graph
        torch.cuda.empty_cache()
    return out


def strong_point(args, device, world, rank, global_batch, layers=4, steps=10, repeats=5):
    """One global batch of ``global_batch`` requests, its slots split evenly over the ranks
    (``sharding.shard_requests``); every rank steps the requests it owns; time = slowest rank."""
    wl = Workload(device, global_batch, layers, args.resid, seed=4242, resid_scale=args.resid_scale,
                  shard=(world, rank))
    wl.warm_state(8)
    graph = capture_step(wl, device)
    for _ in range(3):
        graph.replay()
    job, _ = timed_repeats(graph, steps, repeats, device, world)
    t = median(job) / steps
    # reporting only: reassemble layer 0's output rows in global order and reduce them to one number
    from carrykernel_b200.sharding import gather_rows
    n0 = len(wl.rows[0])
    full = gather_rows(wl.rows[0], wl.out[0][:n0].float().cpu(), global_batch)
    res = {"global_batch": global_batch, "layers": layers, "requests_this_rank": [len(r) for r in wl.rows][:2],
           "ms_per_step": t * 1e3, "us_per_launch": t / layers * 1e6,
           "slot_layer_steps_per_s": global_batch * layers / t,
           "out_checksum": float(full.double().abs().sum())}
    del wl, graph
    torch.cuda.empty_cache()
    return res


def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference_arm(args, rank)
        return

    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if args.mode != "step":
        if rank == 0:
            kw = {} if args.batches is None else {"batches": tuple(args.batches)}
            if args.mode == "pool":
                kw["layers"] = args.pool_layers
            if args.mode == "headtohead":
                kw.update(steps=max(args.steps, 1) * 10, warmup=max(args.warmup, 3) * 10)
            print(json.dumps(SIDE_MODES[args.mode](**kw)))
        return
    if args.config == 5:
        if rank == 0:
            run_config5(args)
        return
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    n_gpus = world

    from carrykernel_b200 import _lib
    lib = _lib.load_library()

    strong = args.strong > 0
    if strong:
        wl = Workload(device, args.strong, args.layers, args.resid, seed=4242, resid_scale=args.resid_scale,
                      shard=(world, rank))
    else:
        wl = Workload(device, args.batch, args.layers, args.resid, seed=1000 + rank,
                      resid_scale=args.resid_scale)
    wl.warm_state(args.warm_steps)
    kernel_used = lib.carry_gdn_last_kernel()

    cpu_base = parity_stats = None
    if rank == 0 and n_gpus == 1 and not args.no_cpu_baseline and not strong:
        cpu_base, parity_stats = cpu_baseline_and_parity(wl, args.resid, args.resid_scale)

    graph = capture_step(wl, device)
    for _ in range(max(args.warmup, 3)):
        graph.replay()
    torch.cuda.synchronize(device)

    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    job, mine = timed_repeats(graph, args.steps, max(args.repeats, 1), device, world)
    elapsed = median(job)
    # keep the sampler alive long enough for at least a few samples under load
    if sum(mine) < args.min_sample_s:
        reps = int((args.min_sample_s - sum(mine)) / max(elapsed / args.steps, 1e-6)) + 1
        time_graph(graph, reps, device)
    clocks = sampler.stop()

    global_batch = args.strong if strong else args.batch * n_gpus
    units_per_step = global_batch * args.layers
    value = units_per_step * args.steps / elapsed
    per_launch = elapsed / (args.steps * args.layers)

    per_rank = None
    if world > 1:
        # every rank's own median and SM clock, so that a slow rank can be named
        mine_t = torch.tensor([median(mine), float(clocks["sm_mhz"] or 0)], dtype=torch.float64, device=device)
        allt = [torch.zeros_like(mine_t) for _ in range(world)]
        dist.all_gather(allt, mine_t)
        ms = [float(x[0]) / args.steps * 1e3 for x in allt]
        slow = max(range(world), key=lambda r: ms[r])
        per_rank = {"ms_per_step": ms, "min": min(ms), "median": median(ms), "max": max(ms),
                    "slowest_rank": slow, "slowest_rank_sm_mhz": float(allt[slow][1])}

    e2e = None
    if not args.no_e2e and not strong:
        from carrykernel_b200.sharding import max_over_ranks
        # the copies-only replay is taken before and after the real one and the smaller kept: the host's
        # copy rate wanders by some 20 % between one second and the next on a shared machine
        rep = max(1, args.repeats)
        t_floor0, _, _ = e2e_run(wl, args.steps, max(args.warmup, 3), groups=args.e2e_groups, kernels=False, repeats=rep)
        t_e2e, h2d, d2h = e2e_run(wl, args.steps, max(args.warmup, 3), groups=args.e2e_groups, repeats=rep)
        t_e2e = max_over_ranks(t_e2e, device)
        t_floor1, _, _ = e2e_run(wl, args.steps, max(args.warmup, 3), groups=args.e2e_groups, kernels=False, repeats=rep)
        t_floor = min(max_over_ranks(t_floor0, device), max_over_ranks(t_floor1, device))
        e2e = {"value": units_per_step * args.steps / t_e2e, "unit": UNIT,
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "ms_per_step": t_e2e / args.steps * 1e3,
               "copy_floor_ms_per_step": t_floor / args.steps * 1e3,
               "timed_regions": rep}                     # each of `steps` steps; the median region is reported

    sweep = strong_pt = c5 = None
    if not args.no_extras and not strong:
        if n_gpus == 1:
            del graph
            sweep = batch_sweep(args, device)
        else:
            strong_pt = strong_point(args, device, world, rank, 512)
        if rank == 0 and n_gpus == 1 and args.resid == "int4":
            wl = None
            torch.cuda.empty_cache()
            c5 = config5_sweep(args.c5_batch, args.c5_steps)

    if rank == 0:
        traffic = None
        if args.resid == "int4" and args.batch == BATCH and args.resid_scale == "head" and not strong:
            traffic = NCU_TRAFFIC_BY_SOURCE.get(kernel_source_hash())
        cfg = workload_config(args, args.batch if not strong else args.strong, args.layers)
        if strong:
            cfg["strong_scaling"] = (f"one global batch of {args.strong} requests; the pool's slots split evenly over "
                                     f"{n_gpus} ranks, each rank steps the requests whose slots it owns")
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": n_gpus, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": elapsed / args.steps * 1e3,
            "higher_is_better": True, "scaling": "strong" if strong else "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": cfg,
            "us_per_token": elapsed / args.steps * 1e6,
            "us_per_layer_step": per_launch * 1e6,
            "repeats": {"n": len(job), "ms_per_step_min": min(job) / args.steps * 1e3,
                        "ms_per_step_median": elapsed / args.steps * 1e3,
                        "ms_per_step_max": max(job) / args.steps * 1e3},
            "roofline": roofline_of(args, wl_batch_for_roofline(args, strong, n_gpus), per_launch, traffic,
                                    {1: "gdn_generic_kernel", 2: "gdn_tile128_kernel"}.get(kernel_used, "?")),
            "cpu_baseline": cpu_base, "parity": parity_stats, "e2e": e2e,
            "gpu_launches": args.steps * args.layers, "clocks": clocks,
            "kernel_source_hash": kernel_source_hash(),
        }
        if per_rank is not None:
            line["per_rank"] = per_rank
        if sweep is not None:
            line["sweep"] = sweep
        if strong_pt is not None:
            line["strong"] = strong_pt
        if c5 is not None:
            line["config5"] = c5
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def wl_batch_for_roofline(args, strong, n_gpus):
    """Requests one launch of one rank processes (the roofline is per GPU)."""
    return (args.strong + n_gpus - 1) // n_gpus if strong else args.batch


if __name__ == "__main__":
    main()
