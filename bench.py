#!/usr/bin/env python
"""Benchmark of the AMUSE/Muon + NVFP4 optimizer step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload gpt2-small] [--impl reference]

A step is one full optimizer step over synthetic state of the named GPT-2 configuration:
Muon (momentum, 5 Newton-Schulz iterations, schedule-free update) + NVFP4 requantisation of
every weight matrix, and schedule-free AdamW on the embeddings / LayerNorm / bias parameters
(embeddings requantised too).  Prints ONE JSON line (rank 0).

`value` is device time per step with all state resident in HBM.  `e2e` is the same step
through the C-ABI calls with HOST buffers: that step's gradients are copied from pinned host
memory and the packed NVFP4 weights are read back inside the timed region.  For N > 1 the
matrices are sharded whole across ranks and the packed weights are all-gathered (NCCL).

The headline workload is GPT-2 small (the metric's 124M).  The same line also carries the step on
GPT-2 XL (`scaling_xl`, every N) and GPT-2 medium (`scaling_medium`, N <= 4), timed with the same
event method, because the scaling claim of the path is made on those.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "ms per AMUSE/Muon+NVFP4 optimizer step (GPT-2 124M)"
MODELS = {  # name: (layers, d_model, vocab, positions)
    "gpt2-small": (12, 768, 50304, 1024),
    "gpt2-medium": (24, 1024, 50304, 1024),
    "gpt2-xl": (48, 1600, 50304, 1024),
}
HP = dict(mu=0.95, grad_scale=1.0, learning_rate=1.0e-4, weight_decay=0.025, average_coefficient=0.5,
          schedule_beta=0.2, iterations=5)
ADAM = dict(grad_scale=1.0, learning_rate=2.0e-4, weight_decay=0.005, beta1=0.9, beta2=0.95, beta1_correction=0.1,
            beta2_correction=0.05, eps=1.0e-10, average_coefficient=0.5, schedule_beta=0.2)
FIXED_TRIPLE = (3.4445, -4.7750, 2.0315)


def layer_shapes(d):
    return [(3 * d, d), (d, d), (4 * d, d), (d, 4 * d)]  # qkv, attn-proj, fc, mlp-proj as [out, in]


def model_shapes(name):
    layers, d, vocab, pos = MODELS[name]
    mats = []
    for _ in range(layers):
        mats += layer_shapes(d)
    emb = [(vocab, d), (pos, d)]
    vec = layers * (4 * d + 3 * d + d + 4 * d + d) + 2 * d  # LN weights/biases + linear biases
    vec = (vec + 15) // 16 * 16
    return mats, emb, vec


def workload_config(name, world):
    """The `config` object of the JSON line; both arms print the same one."""
    mats, emb, vec = model_shapes(name)
    d_model = MODELS[name][1]
    return {
        "workload": f"{name}: {len(mats)} weight matrices (Muon, 5 Newton-Schulz iterations, fixed triple "
                    f"3.4445/-4.7750/2.0315, BF16 operands) + AdamW on embeddings/LayerNorm/bias, NVFP4 requant of "
                    f"all matrices and embeddings",
        "matrix_elements": int(sum(r * c for r, c in mats)), "adamw_elements": int(sum(r * c for r, c in emb) + vec),
        "sharding": "whole matrices, greedy by NS FLOPs" if world > 1 else "single GPU",
        "scale_layout": "csf" if d_model % 128 == 0 else "raw",
        "l2": "per-step working set (>2 GB) exceeds the 126 MB L2; no flush needed",
    }


def ns_flops(shapes, iterations=5):
    f = 0.0
    for r, c in shapes:
        n, m = min(r, c), max(r, c)
        f += 4.0 * n * n * m + 2.0 * n ** 3
    return f * iterations


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm=d["hbm_gbs"], tf_burst=d["bf16_tflops"], tf_sustained=d["bf16_tflops_sustained"], source="measured")
    return dict(hbm=6650.0, tf_burst=1590.0, tf_sustained=1400.0, source="fallback")


def profiled_traffic(workload, world):
    """DRAM bytes per GEMM launch from the committed ncu summary of this workload, if there is one:
    the summary carries a line `dram_bytes_per_launch: <number>` (mean over the captured launches)."""
    if world != 1:
        return None
    path = os.path.join(ROOT, "profiles", f"k_ns_gemm_pair_{workload}.md")
    try:
        m = re.search(r"^dram_bytes_per_launch:\s*([0-9.eE+]+)", open(path).read(), flags=re.M)
        return float(m.group(1)) if m else None
    except OSError:
        return None


class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=self.out,
                                         stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.out.close()
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for nm, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        os.unlink(self.path)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        # Every sample of the timed region, idle gaps between the short bursts included: the plain median
        # and the minimum, so that a down-clocked or clock-locked GPU shows.
        return {"sm_mhz": float(np.median(sm)), "sm_min_mhz": float(min(sm)), "sm_max_mhz": float(max(mx)),
                "power_w_max": float(max(power)), "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------
# CPU arm: the oracle port on the host cores
# ------------------------------------------------------------------------------------------
class CpuStep:
    """The same optimizer step on the host through the CPU oracle.  One layer's matrices are held
    and stepped `layers` times (every layer has the same four shapes and the oracle works on copies), and
    the AdamW update runs over the model's full AdamW element count, so a full step costs the full
    step's arithmetic without holding the whole model on the host."""

    def __init__(self, model):
        from oracle import oracle as o

        self.o = o
        self.layers, d, vocab, pos = MODELS[model]
        rng = np.random.default_rng(0)
        self.shapes = layer_shapes(d)
        self.co = o.fixed_coefficients(5)
        self.state = []
        for r, c in self.shapes:
            n = r * c
            self.state.append(((rng.standard_normal(n) * 1e-3).astype(np.float32), np.zeros(n, np.uint16),
                               (rng.standard_normal(n) * 0.02).astype(np.float32),
                               (rng.standard_normal(n) * 0.02).astype(np.float32)))
        _, emb, vec = model_shapes(model)
        self.adam_total = int(sum(r * c for r, c in emb) + vec)
        self._adam = None

    def _adam_arrays(self, n):
        if self._adam is None or self._adam[0].size != n:
            rng = np.random.default_rng(1)
            self._adam = ((rng.standard_normal(n) * 0.02).astype(np.float32),
                          (rng.standard_normal(n) * 1e-3).astype(np.float32), np.zeros(n, np.float32), np.zeros(n, np.float32))
        return self._adam

    def run(self, layers, adam_elements):
        o = self.o
        t0 = time.perf_counter()
        for _ in range(layers):
            for (g, m, z, x), (r, c) in zip(self.state, self.shapes):
                o.muon_step(g, m, z, x, r, c, mu=HP["mu"], grad_scale=1.0, lr=HP["learning_rate"], wd=HP["weight_decay"],
                            c_avg=HP["average_coefficient"], sched_beta=HP["schedule_beta"], iterations=5, coeffs=self.co,
                            round_mode=o.ROUND_BF16)
        n = (adam_elements + 15) // 16 * 16
        az, ag, am1, am2 = self._adam_arrays(n)
        _, x2, *_ = o.adamw(az, az, ag, am1, am2, 1.0, ADAM["learning_rate"], ADAM["weight_decay"], 0.9, 0.95, 0.1,
                            0.05, 1e-10, 0.5, 0.2)
        o.nvfp4_quantize(x2)
        return (time.perf_counter() - t0) * 1e3

    def full_step_ms(self):
        return self.run(self.layers, self.adam_total)

    def layer_sample_ms(self):
        return self.run(1, self.adam_total // self.layers)


def host_threads():
    from oracle import oracle as o

    # torchrun exports OMP_NUM_THREADS=1 to its workers: ask the OpenMP runtime explicitly
    return o.set_threads(os.cpu_count() or 1)


def run_reference(args):
    """The CPU implementation of the path (the oracle port: the reference is Rust + cuda-oxide and cannot
    be built in this image) on the host cores.  A step is the full optimizer step unless W + K of those
    would take more than about four minutes, in which case a step is one transformer layer + 1/L of the
    AdamW elements and the value is that sample scaled by L, marked `extrapolated`."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = host_threads()
    job = CpuStep(args.workload)
    probe = job.layer_sample_ms()
    full = (args.warmup + args.steps) * probe * job.layers <= 240e3
    one = job.full_step_ms if full else job.layer_sample_ms
    for _ in range(args.warmup):
        one()
    t = [one() for _ in range(args.steps)]
    scale = 1 if full else job.layers
    ms = float(np.mean(t)) * scale
    sample = ("the full step: every layer's four matrices and all AdamW elements" if full else
              f"1 of {job.layers} layers (4 matrices) + 1/{job.layers} of the AdamW elements per step, scaled x{job.layers}")
    line = {
        "impl": "reference", "metric": METRIC, "value": ms, "unit": "ms", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args.workload, args.gpus),
        "note": "CPU oracle port of the reference path on the host cores (the reference itself is Rust + cuda-oxide "
                "and cannot be built in this image); rank 0 only, whatever --gpus says",
        "extrapolated": not full, "sample_scale": scale, "timed_ms_per_sample": float(np.mean(t)),
        "cpu_baseline": {"value": ms, "unit": "ms", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": ms, "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------
class GpuJob:
    """State, plan and step functions of one model configuration on this rank."""

    def __init__(self, name, args, world, rank, dev):
        import torch

        import llmini_b200 as b2
        from llmini_b200.dist import Nvfp4Arena, bucket_plan, shard_plan

        self.torch, self.b2 = torch, b2
        self.name, self.world, self.rank, self.dev = name, world, rank, dev
        self.mats, emb, vec = model_shapes(name)
        if args.shard_of > 1 and world == 1:
            # measurement aid: this GPU plays rank 0 of an N-way sharded run (its matrices and its slice of the
            # embeddings), without the collective
            own, _ = shard_plan(self.mats, args.shard_of)
            self.mats = [m for m, r in zip(self.mats, own) if r == 0]
            emb = [((rows + args.shard_of - 1) // args.shard_of // 128 * 128, cols) for rows, cols in emb]
        d_model = MODELS[name][1]
        layout = self.layout = b2.SCALES_CSF if d_model % 128 == 0 else b2.SCALES_RAW
        # Buckets: contiguous runs of matrices, each spread over all ranks.  Stages M, N and P run over all of the
        # rank's matrices at once; stage U + Q runs bucket by bucket, and the all-gather of one bucket's packed
        # weights runs while the next bucket is updated; the last bucket's gather runs beside AdamW.  A gather has a
        # fixed cost of 50-80 us, so a bucket's gather should take a quarter of a millisecond or more (estimated
        # from its bytes at 600 GB/s into a rank): one bucket per 0.25 ms of gathering, at most four.  (Measured on
        # four GPUs: GPT-2 XL 14.56 -> 14.13 ms with four buckets, GPT-2 small 0.70 -> 0.78 ms with two.)
        self.n_buckets = 1
        if world > 1:
            elems = sum(r * c for r, c in self.mats)
            gather_ms = elems * 0.5625 * (world - 1) / world / 600e9 * 1e3
            # (the library's own copy kernel has a fixed cost of a few microseconds: smaller buckets pay)
            auto = max(1, min(4, int(gather_ms / (0.06 if args.gather == "p2p" else 0.25))))
            self.n_buckets = args.gather_buckets if args.gather_buckets > 0 else auto
        self.bucket, self.owner = bucket_plan(self.mats, world, self.n_buckets)
        self.n_buckets = max(self.bucket) + 1 if self.bucket else 1
        self.mine = [i for b in range(self.n_buckets) for i, r in enumerate(self.owner)
                     if r == rank and self.bucket[i] == b]   # bucket by bucket
        self.my_shapes = [self.mats[i] for i in self.mine]

        def scales_bytes(rows, cols):
            return b2.csf_encoded_len(rows, cols) if layout == b2.SCALES_CSF else rows * cols // 16

        self.arena = Nvfp4Arena(self.mats, self.owner, world, scales_bytes, self.bucket)
        self.peers, self.gather_note = None, None
        if world > 1 and args.gather == "p2p":
            # the arena in memory that the other ranks map: a bucket is exchanged by copying this rank's slice into
            # every peer's arena (b2_peer_push) instead of an NCCL all-gather.  If a rank cannot set it up, all
            # ranks take the NCCL route.
            import torch.distributed as dist
            from llmini_b200.dist import PeerArena

            def exchange(obj):
                got = [None] * world
                dist.all_gather_object(got, obj)
                return got

            try:   # (PeerArena raises on every rank or on none)
                self.peers = PeerArena(self.arena.total_bytes, rank, world, exchange, dev)
            except RuntimeError as exc:
                self.gather_note = "peer-memory exchange unavailable, ncclAllGather instead: " + str(exc)[:200]
        if self.peers is not None:
            self.arena_t = self.arena_v = self.peers.tensor
        else:
            self.arena_t = torch.zeros(self.arena.total_bytes + 1024, dtype=torch.uint8, device=dev)
            abase = (-self.arena_t.data_ptr()) % 256
            self.arena_v = self.arena_t[abase:abase + self.arena.total_bytes]

        gen = torch.Generator(device=dev).manual_seed(1234 + rank)
        randn = lambda n, std: torch.randn(n, device=dev, generator=gen) * std
        headers = {}
        self.slots = []
        for i in self.mine:
            r, c = self.mats[i]
            co, so, go = self.arena.offsets(i)
            nb = self.arena.entries[i]
            s = b2.MuonSlot(
                grad=randn(r * c, 1e-3).view(r, c), momentum=torch.zeros(r, c, dtype=torch.bfloat16, device=dev),
                z_master=randn(r * c, 0.02).view(r, c), x_master=randn(r * c, 0.02).view(r, c),
                schedule_amax=torch.zeros(1, device=dev), bytes=self.arena_v[co:co + nb.codes_bytes],
                scales=self.arena_v[so:so + nb.scales_bytes], global_scale=self.arena_v[go:go + 4].view(torch.float32),
                rows=r, cols=c)
            if layout == b2.SCALES_CSF:
                if (r, c) not in headers:
                    headers[(r, c)] = b2.zero_scales(r, c, dev)
                s.scales.copy_(headers[(r, c)])
            self.slots.append(s)
        self.normalize = b2.NORMALIZE_TWO_PASS if args.two_pass_prepare else b2.NORMALIZE_DEFERRED
        self.schedule = {"per-phase": b2.NS_PER_PHASE, "chained": b2.NS_CHAINED,
                         "fused": b2.NS_FUSED_GRAM_POLY}[args.ns_schedule]
        self.update_input = b2.UPDATE_16BIT if args.update_16bit else b2.UPDATE_F32
        # one plan for all of this rank's matrices; its finish groups are the buckets (a rank may own nothing of one)
        self.plan = b2.MuonPlan(self.my_shapes, scale_layout=layout, device=dev, debug_flags=args.plan_flags,
                                normalize_mode=self.normalize, ns_schedule=self.schedule,
                                update_input=self.update_input) if self.my_shapes else None
        self.table = b2.slot_table(self.slots, dev) if self.slots else None
        if self.plan is not None and self.n_buckets > 1:
            first = [sum(1 for i in self.mine if self.bucket[i] < b) for b in range(self.n_buckets)]
            self.plan.set_finish_groups(first)
        self.opt = b2.OptimizerModule()
        self.margs = b2.MuonMegaUpdateArgs(coefficients=np.tile(np.asarray(FIXED_TRIPLE, np.float32), (5, 1)), **HP)

        # AdamW parameters: embeddings (requantised) split by rank on row boundaries, vectors on rank 0
        self.adam_sets = []
        for (rows, cols) in emb:
            per = (rows + world - 1) // world
            per = (per + 127) // 128 * 128
            r0, r1 = min(rank * per, rows), min((rank + 1) * per, rows)
            n = (r1 - r0) * cols
            if n == 0:
                continue
            t = dict(z_master=randn(n, 0.02), x_master=randn(n, 0.02), grad=randn(n, 1e-3),
                     first_moment=torch.zeros(n, device=dev), second_moment=torch.zeros(n, device=dev),
                     bytes=torch.zeros(n // 2, dtype=torch.uint8, device=dev),
                     scales=(b2.zero_scales(r1 - r0, cols, dev) if layout == b2.SCALES_CSF else
                             torch.zeros(n // 16, dtype=torch.uint8, device=dev)),
                     global_scale=torch.zeros(1, device=dev), amax=torch.zeros(1, device=dev),
                     chunk_amax=torch.zeros((n + 2047) // 2048, device=dev), scale_layout=layout, len=n)
            self.adam_sets.append(("quant", t))
        if rank == 0:
            t = dict(z_master=randn(vec, 0.02), x_master=randn(vec, 0.02), grad=randn(vec, 1e-3),
                     first_moment=torch.zeros(vec, device=dev), second_moment=torch.zeros(vec, device=dev), len=vec)
            self.adam_sets.append(("fp32", t))
        self.adam_table = self.adam_count = self.adam_chunks = None
        if self.adam_sets:
            # every AdamW tensor of the rank in one pointer table: three launches for all of them
            self.adam_table, self.adam_count, self.adam_chunks = self.opt.adamw_table(
                [dict(t, mode=2 if kind == "quant" else 0) for kind, t in self.adam_sets], dev)
        self.launches_per_step = 0
        if self.plan is not None:
            prepare = 3 if self.normalize == b2.NORMALIZE_TWO_PASS else 2
            gemms = {b2.NS_CHAINED: 1, b2.NS_FUSED_GRAM_POLY: 2 * HP["iterations"]}.get(self.schedule, 3 * HP["iterations"])
            finish = 2 if args.plan_flags & 16 else sum(1 for b in range(self.n_buckets)
                                                       if any(self.bucket[i] == b for i in self.mine))
            self.launches_per_step += prepare + gemms + finish
        self.launches_per_step += 3 if self.adam_sets else 0
        # (high priority, so that the few CTAs of an exchange are placed before the hundreds of the update launch beside
        # it; measured neutral on four GPUs)
        self.gather_stream = torch.cuda.Stream(device=dev, priority=-1) if world > 1 else None
        self.stage_events = []

    # -- the step ---------------------------------------------------------------------------
    def gather_bucket(self, b):
        """All-gather of bucket b's region on the side stream, ordered after what the current stream has done so
        far.  Returns nothing; `join_gathers` makes the current stream wait for all of them."""
        import torch.distributed as dist

        torch = self.torch
        fork = torch.cuda.Event()
        fork.record(torch.cuda.current_stream())
        self.gather_stream.wait_event(fork)
        base, size = self.arena.region(b)
        n = self.arena.bucket_bytes_per_rank[b]
        if self.peers is not None:
            self.peers.push(base + self.rank * n, n, self.gather_stream.cuda_stream)   # (an empty slice still counts)
            return
        if n == 0:
            return
        with torch.cuda.stream(self.gather_stream):
            region = self.arena_v[base:base + size]
            dist.all_gather_into_tensor(region, region[self.rank * n:(self.rank + 1) * n])

    def join_gathers(self):
        torch = self.torch
        if self.peers is not None:
            self.peers.wait(self.gather_stream.cuda_stream)   # every rank's copies of this step have landed here
        join = torch.cuda.Event()
        join.record(self.gather_stream)
        torch.cuda.current_stream().wait_event(join)

    def step_muon(self, marks=None, standalone=False):
        """The Muon stages.  With more than one bucket, stage U + Q runs bucket by bucket and the all-gather of a
        finished bucket runs on the side stream while the next bucket is updated; the last bucket's gather is left
        to step_adam.  `marks`, when given, receives the four events around the three stages.  `standalone`: the
        gathers started here are also waited for here (a capture of this half alone must not end with work pending
        on the side stream)."""
        torch = self.torch
        stream = torch.cuda.current_stream()
        e = [torch.cuda.Event(enable_timing=True) for _ in range(4)] if marks is not None else None
        if e: e[0].record(stream)
        if self.plan is not None:
            self.opt.muon_tma_prepare_polar(self.plan, self.table, self.margs)
        if e: e[1].record(stream)
        if self.plan is not None:
            self.opt.muon_polar(self.plan, self.margs)
        if e: e[2].record(stream)
        if self.n_buckets == 1:
            if self.plan is not None:
                self.opt.muon_tma_finish_update(self.plan, self.table, self.margs)
        else:
            for b in range(self.n_buckets):
                if self.plan is not None:
                    self.opt.muon_tma_finish_update_group(self.plan, self.table, self.margs, b)
                if self.world > 1 and b + 1 < self.n_buckets:
                    self.gather_bucket(b)
        if e: e[3].record(stream)
        if e: marks.append(e)
        if standalone and self.world > 1 and self.n_buckets > 1:
            self.join_gathers()

    def step_adam(self, marks=None):
        """AdamW on this rank's tensors; for N > 1 the all-gather of the (last) bucket of packed matrices runs
        beside it on a second stream (forked after the Muon stages, joined before the step ends)."""
        torch = self.torch
        stream = torch.cuda.current_stream()
        e0 = torch.cuda.Event(enable_timing=True) if marks is not None else None
        if e0: e0.record(stream)
        if self.world > 1:
            self.gather_bucket(self.n_buckets - 1)   # (every rank gathers every bucket, also one it owns nothing of)
        if self.adam_sets:
            self.opt.apply_adamw_update_multi(self.adam_table, self.adam_count, self.adam_chunks, **ADAM)
        if marks is not None:
            e1 = torch.cuda.Event(enable_timing=True)
            e1.record(stream)
            marks.append([e0, e1])
        if self.world > 1:
            self.join_gathers()

    def step(self, record=False):
        marks = [] if record else None
        self.step_muon(marks)
        self.step_adam(marks)
        if record:
            self.stage_events.append(marks)

    # -- timing -----------------------------------------------------------------------------
    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist

            dist.barrier()
        self.torch.cuda.synchronize()

    def timed(self, fn, steps):
        torch = self.torch
        stream = torch.cuda.current_stream()
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        self.barrier()
        ms = e0.elapsed_time(e1)
        if self.world > 1:
            import torch.distributed as dist

            t = torch.tensor([ms], device=self.dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / steps

    def check_status(self, when):
        if self.plan is not None and self.plan.status() != 0:
            raise SystemExit(f"a bounded device-side wait ran out {when}")
        if self.peers is not None and self.peers.status(self.torch.cuda.current_stream().cuda_stream) != 0:
            raise SystemExit(f"the bounded wait for the other ranks' copies ran out {when}")

    def stage_summary(self, peaks):
        """Mean device time of the four stages over the eager timed pass (this rank), and the rates."""
        self.torch.cuda.synchronize()
        # per recorded step: the four events around prepare, Newton-Schulz and finish, then the two around AdamW
        rows = []
        for m in self.stage_events:
            parts = np.zeros(4)
            for e in m[:-1]:
                parts[:3] += [e[i].elapsed_time(e[i + 1]) for i in range(3)]
            parts[3] = m[-1][0].elapsed_time(m[-1][1])
            rows.append(parts)
        st = np.array(rows) if rows else np.zeros((1, 4))
        prep_ms, ns_ms, fin_ms, adam_ms = (float(v) for v in st.mean(axis=0))
        elems = sum(r * c for r, c in self.my_shapes)
        flops = ns_flops(self.my_shapes, HP["iterations"])
        rate = lambda units, ms: units / (ms * 1e-3) if ms > 0 else 0.0
        ns_tflops = rate(flops, ns_ms) / 1e12
        # stage U+Q: reads U,z,x; writes z,x,y(schedule cache),codes,scales = 24.5625 B per element (22.5625 when the
        # Newton-Schulz result arrives in 16 bits)
        fin_bytes = 22.5625 if self.update_input else 24.5625
        fin_gbs = rate(elems * fin_bytes, fin_ms) / 1e9
        prep_gbs = rate(elems * 10.0, prep_ms) / 1e9
        adam_elems = sum(t["len"] for _, t in self.adam_sets)
        adam_gbs = rate(adam_elems * 36.0, adam_ms) / 1e9
        return {
            "prepare_ms": prep_ms, "newton_schulz_ms": ns_ms, "update_quantise_ms": fin_ms, "adamw_ms": adam_ms,
            "prepare_gbs": prep_gbs, "prepare_frac_of_hbm": prep_gbs / peaks["hbm"],
            "newton_schulz_tflops_per_gpu": ns_tflops,
            "update_quantise_gbs": fin_gbs, "update_quantise_frac_of_hbm": fin_gbs / peaks["hbm"],
            "adamw_gbs": adam_gbs, "hbm_peak_gbs": peaks["hbm"], "update_quantise_frac_of_nominal_8000": fin_gbs / 8000.0,
            "prepare": "one pass (scale folded into the first iteration)" if self.normalize else "two passes (reference rounding point)",
            "newton_schulz": {self.b2.NS_CHAINED: "one chained launch for the whole loop",
                              self.b2.NS_FUSED_GRAM_POLY: "two launches per iteration (fused Gram + polynomial tiles, apply)"
                              }.get(self.schedule, "three launches per iteration"),
            "gather_buckets": self.n_buckets,
            "gather": None if self.world == 1 else ("copies into the other ranks' arenas through peer memory"
                                                    if self.peers is not None else (self.gather_note or "ncclAllGather")),
            "update_quantise_bytes_per_element": fin_bytes,
        }

    # -- checks -----------------------------------------------------------------------------
    def gathered_arena_consistent(self):
        """After one step + all-gather every rank must hold the same arena (per-slice checksums reduced with MIN
        and MAX over the ranks must agree, slices with payload must be non-zero).  Plain NCCL collectives only."""
        from llmini_b200.dist import gathered_arena_consistent

        return gathered_arena_consistent(self.arena_v, self.arena)

    def parity_against_oracle(self, compare):
        """One matrix of the timed workload, one more step from its current state, against the CPU oracle:
        momentum bits, z', x', y, codes, scales and tensor scale bit for bit (the elementwise stages given the
        device's own Newton-Schulz result), the Newton-Schulz result within 2e-2 relative L2.  Every rank takes
        the step (it contains the collective); the rank with `compare` set checks its first matrix."""
        torch, b2 = self.torch, self.b2
        host = lambda t: t.detach().cpu().numpy()
        compare = compare and self.plan is not None
        if compare:
            i = 0
            s, (r, c) = self.slots[i], self.my_shapes[i]
            n = r * c
            g, z, x = host(s.grad).ravel().copy(), host(s.z_master).ravel().copy(), host(s.x_master).ravel().copy()
            m = host(s.momentum.view(torch.int16)).view(np.uint16).ravel().copy()
        self.step()
        self.barrier()
        if not compare:
            return None
        from oracle import oracle as o

        deferred = self.normalize == b2.NORMALIZE_DEFERRED
        ref = o.muon_step(g, m, z, x, r, c, mu=HP["mu"], grad_scale=HP["grad_scale"], lr=HP["learning_rate"],
                          wd=HP["weight_decay"], c_avg=HP["average_coefficient"], sched_beta=HP["schedule_beta"],
                          iterations=HP["iterations"], coeffs=np.tile(np.asarray(FIXED_TRIPLE, np.float32), (5, 1)),
                          round_mode=o.ROUND_BF16, deferred_normalize=deferred)
        bad = []
        if not np.array_equal(host(s.momentum.view(torch.int16)).view(np.uint16).ravel(), ref.momentum_bits):
            bad.append("momentum")
        # five iterations: the 16-bit result, when that is what stage U reads, is in the second operand buffer
        Ug = host(self.plan.scratch(i, 7).float()) if self.update_input else host(self.plan.scratch(i, 1))
        rel = float(np.linalg.norm(Ug.astype(np.float64) - ref.U) / np.linalg.norm(ref.U.astype(np.float64)))
        if not rel <= 2e-2:
            bad.append(f"Newton-Schulz rel L2 {rel:.3e}")
        z2, x2, y2, ax, ay = o.update(Ug, z, x, r, c, HP["learning_rate"], HP["weight_decay"], HP["average_coefficient"],
                                      HP["schedule_beta"])
        for name, got, want in (("z", s.z_master, z2), ("x", s.x_master, x2), ("y", s.grad, y2)):
            if not np.array_equal(host(got).ravel(), want):
                bad.append(name)
        gs = host(s.global_scale)[0]
        ins = o.rcp_inputs(gs)
        outs = host(b2.Nvfp4QuantModule().debug_rcp_approx_ftz(torch.from_numpy(ins).to(self.dev)))
        codes, raw, ogs, misses = o.nvfp4_quantize(x2, amax=ax, rcp_table=(ins.view(np.uint32), outs.view(np.uint32)))
        got_scales = host(s.scales)
        got_scales = got_scales[: n // 16] if self.layout == b2.SCALES_RAW else o.csf_decode_matrix(got_scales, r, c)
        if misses or gs != ogs:
            bad.append("tensor scale")
        if not np.array_equal(host(s.bytes)[: n // 2], codes):
            bad.append("codes")
        if not np.array_equal(got_scales, raw):
            bad.append("block scales")
        if bad:
            raise SystemExit(f"{self.name}: matrix 0 ({r}x{c}) differs from the CPU oracle in: " + ", ".join(bad))
        return {"matrix": f"{r}x{c}", "newton_schulz_rel_l2": rel, "bit_exact": ["momentum", "z", "x", "y", "codes",
                                                                                "block scales", "tensor scale"]}

    def close(self):
        if self.plan is not None:
            self.plan.close()
        if self.peers is not None:
            self.barrier()          # nobody unmaps or frees while another rank may still be copying
            self.slots, self.table, self.arena_t, self.arena_v = [], None, None, None
            self.peers.close()
            self.peers = None


def secondary_workload(name, args, world, rank, dev, peaks):
    """The step on another model configuration, timed the same way as the headline: warm-up, an eager pass
    with events between the stages, then the captured step replayed `steps` times (device time, max over ranks)."""
    import torch

    job = GpuJob(name, args, world, rank, dev)
    steps = max(3, min(args.steps, 10))
    for _ in range(3):
        job.step()
    job.barrier()
    job.check_status(f"during the {name} warm-up")
    ms_eager = job.timed(lambda: job.step(record=True), steps)
    ms_step, graphed = ms_eager, False
    if not args.no_graph:
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                job.step()
            graph.replay()
            ms_step = job.timed(graph.replay, steps)
            graphed = True
            del graph
        except Exception:
            pass
    job.check_status(f"during the {name} timed region")
    consistent = job.gathered_arena_consistent() if world > 1 else None
    if consistent is False:
        raise SystemExit(f"{name}: the ranks do not hold the same gathered arena")
    parity = job.parity_against_oracle(compare=(rank == 0))   # one matrix of this workload against the CPU oracle
    out = {"workload": workload_config(name, world)["workload"], "ms_per_step": ms_step, "eager_ms_per_step": ms_eager,
           "steps": steps, "warmup": 3, "cuda_graph": graphed, "n_gpus": world,
           "ns_tflop_per_step": ns_flops(job.mats) / 1e12, "stages_rank0": job.stage_summary(peaks),
           "gathered_arena_consistent": consistent, "parity_checked": parity is not None, "parity": parity}
    job.close()
    del job
    torch.cuda.empty_cache()
    return out


def run_gpu(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the optimizer path has no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    peaks = load_peaks()

    job = GpuJob(args.workload, args, world, rank, dev)
    slots, adam_sets, arena, arena_v, arena_t = job.slots, job.adam_sets, job.arena, job.arena_v, job.arena_t
    stream = torch.cuda.current_stream()
    step, step_muon, step_adam, barrier, timed = job.step, job.step_muon, job.step_adam, job.barrier, job.timed

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    job.check_status("during warm-up")

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms_eager = timed(lambda: step(record=True), args.steps)
    # The whole step is stream-ordered with no host synchronisation, so it is captured once in a
    # CUDA graph and replayed: the headline number is the replay, the per-stage breakdown (and
    # the roofline figure) comes from the eager pass above, whose events sit between stages.
    graph = graph_muon = graph_adam = None
    modes_match = None
    ms_step = ms_eager
    if not args.no_graph:
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step()
            graph.replay()
            ms_step = timed(graph.replay, args.steps)
            # the replayed step against the same calls launched one by one, from the same state: every
            # master, moment, cached y, code, scale byte and tensor scale bit for bit (a capture that
            # silently left work out would show here)
            state, names = [], []
            for i_, s_ in enumerate(slots):
                for k in ("grad", "momentum", "z_master", "x_master", "schedule_amax"):
                    state.append(getattr(s_, k))
                    names.append(f"matrix {i_} {k}")
            for i_, (_, t_) in enumerate(adam_sets):
                for k in ("z_master", "x_master", "grad", "first_moment", "second_moment", "amax", "bytes", "scales",
                          "global_scale"):
                    if k in t_:
                        state.append(t_[k])
                        names.append(f"adamw tensor {i_} {k}")
            state.append(arena_t)
            names.append("arena of codes, scales and tensor scales")
            if sum(t_.numel() * t_.element_size() for t_ in state) <= (8 << 30):   # three copies are held
                saved = [t_.clone() for t_ in state]

                def outcome(run):
                    for t_, s_ in zip(state, saved):
                        t_.copy_(s_)
                    barrier()   # (a rank that runs ahead may already copy into this rank's arena: restore first)
                    run()
                    barrier()
                    return [t_.clone() for t_ in state]

                first, second = outcome(step), outcome(graph.replay)
                differing = [n_ for n_, a_, b_ in zip(names, first, second) if not torch.equal(a_, b_)]
                changed = sum(int(not torch.equal(a_, s_)) for a_, s_ in zip(second, saved))
                modes_match = not differing and changed > 0
                if world > 1:
                    flag = torch.tensor([int(modes_match)], device=dev)
                    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
                    modes_match = bool(flag.item())
                del saved, first, second
                if not modes_match:
                    raise SystemExit("the replayed step and the eagerly launched step disagree in: "
                                     + "; ".join(differing[:12]) + f" ({len(differing)} tensors)")
            # the two halves on their own, for the pipelined end-to-end step below
            graph_muon, graph_adam = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph_muon):
                step_muon(None, True)
            with torch.cuda.graph(graph_adam):
                step_adam()
        except SystemExit:
            raise
        except Exception as exc:  # capture is an optimisation; report why it was skipped
            graph = graph_muon = graph_adam = None
            print(f"bench: graph capture skipped: {exc!r}"[:300], file=sys.stderr, flush=True)

    # ---- end to end: host gradients in, packed weights out, every step ----
    # What a caller with host-resident gradients does with the same public calls: the matrix
    # gradients go up first; while the Muon stages run, a second stream brings up the AdamW
    # gradients, and a third takes the packed matrices down (PCIe is full duplex); AdamW and its
    # outputs follow.  Every copy is inside the timed region; the step ends when the last byte is on
    # the host.
    n_slots = len(slots)
    grad_dev = [s.grad for s in slots] + [t["grad"] for _, t in adam_sets]
    grad_host = [torch.empty(g.shape, dtype=g.dtype, pin_memory=True).copy_(g) for g in grad_dev]
    packed_dev = [arena_v[o_:o_ + n_] for o_, n_ in arena.rank_slices(rank) if n_]   # this rank's slice of every bucket
    n_packed = len(packed_dev)
    out_dev = packed_dev + \
              [t[k] for kind, t in adam_sets if kind == "quant" for k in ("bytes", "scales", "global_scale")]
    out_host = [torch.empty(o_.shape, dtype=o_.dtype, pin_memory=True) for o_ in out_dev]
    h2d = sum(g.numel() * g.element_size() for g in grad_dev)
    d2h = sum(o_.numel() * o_.element_size() for o_ in out_dev)
    up_stream, down_stream = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    adam_done = torch.cuda.Event()
    adam_done.record(stream)

    def step_e2e():
        for gd, gh in zip(grad_dev[:n_slots], grad_host[:n_slots]):
            gd.copy_(gh, non_blocking=True)
        matrices_up = torch.cuda.Event()
        matrices_up.record(stream)
        # the AdamW gradients go second: sharing the link with the matrix gradients would only delay the
        # Muon stages, which are what hides this upload
        up_stream.wait_event(matrices_up)
        up_stream.wait_event(adam_done)          # the previous step's AdamW has consumed its gradients
        with torch.cuda.stream(up_stream):
            for gd, gh in zip(grad_dev[n_slots:], grad_host[n_slots:]):
                gd.copy_(gh, non_blocking=True)
            adam_up = torch.cuda.Event()
            adam_up.record(up_stream)
        if graph_muon is not None:
            graph_muon.replay()
        else:
            step_muon()
        muon_done = torch.cuda.Event()
        muon_done.record(stream)
        down_stream.wait_event(muon_done)
        with torch.cuda.stream(down_stream):
            for od, oh in zip(out_dev[:n_packed], out_host[:n_packed]):
                oh.copy_(od, non_blocking=True)
            down_done = torch.cuda.Event()
            down_done.record(down_stream)
        stream.wait_event(adam_up)
        if graph_adam is not None:
            graph_adam.replay()
        else:
            step_adam()
        adam_done.record(stream)
        for od, oh in zip(out_dev[n_packed:], out_host[n_packed:]):
            oh.copy_(od, non_blocking=True)
        stream.wait_event(down_done)

    step_e2e()
    ms_e2e = timed(step_e2e, args.steps)
    clocks = sampler.stop() if rank == 0 else None
    job.check_status("during the timed region")

    stages = job.stage_summary(peaks)
    # ---- checks after the timed region ----
    consistent = None
    if world > 1:
        step()
        barrier()
        consistent = job.gathered_arena_consistent()
        if not consistent:
            raise SystemExit("the ranks do not hold the same gathered arena after a step")
    parity = job.parity_against_oracle(compare=(rank == 0))
    launches_per_step = job.launches_per_step
    job.close()
    del job, slots, adam_sets, arena_v, arena_t, grad_dev, out_dev, graph_muon, graph_adam
    graph = None if graph is None else True
    torch.cuda.empty_cache()

    # ---- the scaling workloads: GPT-2 XL at every N, GPT-2 medium up to four GPUs ----
    extra = {}
    if not args.no_scaling_workloads and args.workload == "gpt2-small":
        extra["scaling_xl"] = secondary_workload("gpt2-xl", args, world, rank, dev, peaks)
        if world <= 4:
            extra["scaling_medium"] = secondary_workload("gpt2-medium", args, world, rank, dev, peaks)

    def finish():
        # A watchdog ends the process if the communicator's teardown stalls; by then the result line has been
        # printed.
        if world == 1:
            return
        import threading
        threading.Timer(30.0, lambda: os._exit(0)).start()
        torch.cuda.synchronize()
        dist.barrier()
        dist.destroy_process_group()
        os._exit(0)

    if rank != 0:
        finish()
        return
    ns_tflops = stages["newton_schulz_tflops_per_gpu"]
    # The timed region is tens of milliseconds at full clocks, not seconds under the power cap: the burst
    # figure of the measured cuBLAS peak is the denominator; the sustained one is printed beside it.
    line = {
        "metric": METRIC, "value": ms_step, "unit": "ms", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args.workload, world),
        "roofline": {
            "bound": "tensor", "kernel": "k_ns_gemm (all 15 GEMMs of the step" + {
                "chained": " as one chained launch)", "per-phase": ", one launch each)",
                "fused": ": per iteration one launch of fused Gram + polynomial tiles and one of apply tiles)"}[args.ns_schedule],
            "achieved": ns_tflops,
            "peak": peaks["tf_burst"], "unit": "TFLOP/s", "frac": ns_tflops / peaks["tf_burst"],
            "traffic": profiled_traffic(args.workload, world),
            "peak_source": f"{peaks['source']} bf16 burst (timed region well under a second at full clocks)",
            "frac_of_sustained": ns_tflops / peaks["tf_sustained"], "frac_of_nominal_2250": ns_tflops / 2250.0,
        },
        "stages": stages,
        "e2e": {"value": ms_e2e, "unit": "ms", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h)},
        "gpu_launches": int(launches_per_step * args.steps),
        "clocks": clocks,
        "eager_ms_per_step": ms_eager,
        "cuda_graph": graph is not None,
        "replayed_step_matches_eager": modes_match,
        "parity_checked": parity is not None, "parity": parity,
        "gathered_arena_consistent": consistent,
    }
    line.update(extra)
    if world == 1 and not args.no_cpu:
        cores = host_threads()
        cpu = CpuStep(args.workload)
        line["cpu_baseline"] = {"value": cpu.full_step_ms(), "unit": "ms", "cores": cores, "kind": "port",
                                "sample": "the full step once: every layer's four matrices and all AdamW elements"}
    print(json.dumps(line), flush=True)
    finish()


def run_sweep(args):
    """Bandwidth sweep of the update + quantise pass on [R, 4096] tensors (R = 256 .. 262144):
    one JSON line per shape.  Not part of the default run."""
    import torch

    import llmini_b200 as b2

    torch.cuda.set_device(0)
    peaks = load_peaks()
    opt = b2.OptimizerModule()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")   # larger than the 126 MB L2
    for R in (256, 1024, 4096, 16384, 65536, 262144):
        r, c = R, 4096
        n = r * c
        s = b2.MuonSlot.allocate(r, c)
        g = torch.Generator(device="cuda").manual_seed(R)
        s.z_master.copy_((torch.randn(n, device="cuda", generator=g) * 0.02).view(r, c))
        s.x_master.copy_(s.z_master)
        plan = b2.MuonPlan([(r, c)])
        table = b2.slot_table([s])
        margs = b2.MuonMegaUpdateArgs(**HP)
        opt.muon_tma_prepare_polar(plan, table, margs)
        plan.scratch(0, 1).copy_((torch.randn(n, device="cuda", generator=g) * 0.02).view(r, c))
        reps = max(3, min(50, int(2e9 // n)))
        for _ in range(3):
            opt.muon_tma_finish_update(plan, table, margs)
        torch.cuda.synchronize()
        # tensors that fit L2 are timed one call at a time with the L2 flushed (overwritten) in between
        small = n * 24.5625 < 400e6
        total = 0.0
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if small:
            for _ in range(reps):
                flush.fill_(1)
                e0.record()
                opt.muon_tma_finish_update(plan, table, margs)
                e1.record()
                torch.cuda.synchronize()
                total += e0.elapsed_time(e1)
        else:
            e0.record()
            for _ in range(reps):
                opt.muon_tma_finish_update(plan, table, margs)
            e1.record()
            torch.cuda.synchronize()
            total = e0.elapsed_time(e1)
        ms = total / reps
        gbs = n * 24.5625 / (ms * 1e-3) / 1e9
        print(json.dumps({"sweep": "update_quantise", "rows": r, "cols": c, "elements": n, "ms": ms,
                          "bytes_per_element": 24.5625, "gbs": gbs, "frac_of_measured_hbm": gbs / peaks["hbm"],
                          "frac_of_nominal_8000": gbs / 8000.0,
                          "l2": "flushed before every call" if small else "tensor larger than L2"}), flush=True)
        plan.close()
        del s, plan, table
        torch.cuda.empty_cache()


def run_extras(args):
    """Device time of the entry points beside the headline step (the trainer's per-step variants,
    the clip, the cached-weight materialisation, the sm_100 scale converter) on the GPT-2-small matrix
    set: one JSON line each, bytes as the algorithmic minimum the call has to move.  Not part of
    the default run."""
    import torch

    import llmini_b200 as b2

    torch.cuda.set_device(0)
    dev = "cuda"
    peaks = load_peaks()
    mats, emb, _ = model_shapes(args.workload)
    n_el = sum(r * c for r, c in mats)
    opt = b2.OptimizerModule()
    g = torch.Generator(device=dev).manual_seed(0)
    randn = lambda n, std: torch.randn(n, device=dev, generator=g) * std
    layout = b2.SCALES_CSF if MODELS[args.workload][1] % 128 == 0 else b2.SCALES_RAW
    slots = []
    for r, c in mats:
        s = b2.MuonSlot.allocate(r, c, layout)
        s.grad.copy_(randn(r * c, 1e-3).view(r, c))
        s.z_master.copy_(randn(r * c, 0.02).view(r, c))
        s.x_master.copy_(s.z_master)
        s.variance = torch.full((r, c), 1e-6, dtype=torch.bfloat16, device=dev)
        s.second_momentum = torch.full((max(r, c),), 1e-2, device=dev)
        slots.append(s)
    # fused QKV matrices (3d x d) take the per-head clip; 64-wide heads
    d_model = MODELS[args.workload][1]
    heads = d_model // 64
    for i, (s, (r, c)) in enumerate(zip(slots, mats)):
        if r == 3 * c:
            s.qk_clip_factor_offset, s.qk_clip_head_dim = (i // 4) * heads, 64
    factors = 0.5 + 0.5 * torch.rand(len(mats) // 4 * heads, device=dev, generator=g)
    plan = b2.MuonPlan(mats, scale_layout=layout, debug_flags=args.plan_flags)
    plan1 = b2.MuonPlan(mats, scale_layout=layout, normalize_mode=b2.NORMALIZE_DEFERRED)
    table = b2.slot_table(slots)
    base = dict(HP)
    for i in range(len(mats)):
        plan.scratch(i, 1).copy_(randn(mats[i][0] * mats[i][1], 0.05).view(*mats[i]))
    # the reference's trainer hands the clip 4096-value chunks (src/training/grad_clip.rs)
    cuts = [(s.grad.data_ptr() + 4 * a, min(4096, s.rows * s.cols - a)) for s in slots
            for a in range(0, s.rows * s.cols, 4096)]
    ptrs = torch.tensor([p for p, _ in cuts], dtype=torch.int64, device=dev)
    lens = torch.tensor([n for _, n in cuts], dtype=torch.int32, device=dev)
    sums, scale, norm = torch.zeros(len(cuts), device=dev), torch.zeros(1, device=dev), torch.zeros(1, device=dev)
    raw_scales = torch.randint(0, 127, (n_el // 16,), dtype=torch.uint8, device=dev, generator=g)

    A = b2.MuonMegaUpdateArgs
    cases = [
        ("prepare (plain, two passes)", 16.0, lambda: opt.muon_tma_prepare_polar(plan, table, A(**base))),
        ("prepare (plain, one pass)", 10.0, lambda: opt.muon_tma_prepare_polar(plan1, table, A(**base))),
        ("prepare (Muon-VS)", 20.0, lambda: opt.muon_tma_prepare_polar(
            plan, table, A(variance_adaptive=True, bias_correction_inv=1.5, **base))),
        ("finish, deferred quantisation (plain)", 24.0,
         lambda: opt.muon_tma_finish_update_deferred_quantization(plan, table, A(**base))),
        ("finish, deferred (NorMuon + qk-clip)", 28.0,
         lambda: opt.muon_tma_finish_update_deferred_quantization(plan, table, A(normuon=True, qk_clip_factors=factors, **base))),
        ("finish, deferred (NorMuon only)", 28.0,
         lambda: opt.muon_tma_finish_update_deferred_quantization(plan, table, A(normuon=True, **base))),
        ("finish, deferred (qk-clip only)", 24.0,
         lambda: opt.muon_tma_finish_update_deferred_quantization(plan, table, A(qk_clip_factors=factors, **base))),
        ("finish + quantise (plain)", 24.5625, lambda: opt.muon_tma_finish_update(plan, table, A(**base))),
        ("finish + quantise (NorMuon + qk-clip)", 28.5625,
         lambda: opt.muon_tma_finish_update(plan, table, A(normuon=True, qk_clip_factors=factors, **base))),
        ("finish, Hyperball", 32.0,
         lambda: opt.muon_tma_finish_hyperball_update_deferred_quantization(plan, table, A(**base))),
        ("sign-Muon update", 26.0, lambda: opt.muon_tma_sign_update_deferred_quantization(plan, table, A(**base))),
        ("materialize training weights (y -> NVFP4)", 4.5625, lambda: opt.muon_materialize_training_weights(plan, table)),
        ("clip_gradients (norm + scale, gradients left alone)", 4.0,
         lambda: opt.clip_gradients(chunk_ptrs=ptrs, chunk_lens=lens, chunk_sums=sums, extra_sums=None, scale=scale,
                                    norm=norm, chunk_count=len(cuts), extra_sum_count=0, max_norm=1.0, apply=False)),
        ("scales_to_sm100 (raw plane, all matrices as one [n/768, 768] tensor)", 2.0 / 16.0,
         lambda: b2.scales_to_sm100(raw_scales, b2.SCALES_RAW, n_el // 768, 768)),
    ]
    # the embeddings as deferred AdamW tensors (the trainer's mode): update with y cached in the gradient
    # buffer, then every tensor's y quantised by one launch (src/training/schedule_free/tensor.rs:71-89)
    emb_sets = []
    for rows, cols in emb:
        n = rows * cols
        emb_sets.append(dict(z_master=randn(n, 0.02), x_master=randn(n, 0.02), grad=randn(n, 1e-3),
                             first_moment=torch.zeros(n, device=dev), second_moment=torch.zeros(n, device=dev),
                             bytes=torch.zeros(n // 2, dtype=torch.uint8, device=dev),
                             scales=(b2.zero_scales(rows, cols, dev) if layout == b2.SCALES_CSF else
                                     torch.zeros(n // 16, dtype=torch.uint8, device=dev)),
                             global_scale=torch.zeros(1, device=dev), amax=torch.zeros(1, device=dev),
                             scale_layout=layout, len=n, mode=1))
    emb_el = sum(t["len"] for t in emb_sets)
    emb_table, emb_count, emb_chunks = opt.adamw_table(emb_sets, dev)
    adam_hp = dict(ADAM)
    cases += [
        ("AdamW, deferred quantisation, all embeddings in one table", 40.0 * emb_el / n_el,
         lambda: opt.apply_adamw_update_multi(emb_table, emb_count, emb_chunks, **adam_hp)),
        ("AdamW tensors: materialize training weights (cached y -> NVFP4), one launch", 4.5625 * emb_el / n_el,
         lambda: opt.adamw_materialize_training_weights(emb_table, emb_count, emb_chunks, ADAM["schedule_beta"])),
    ]
    co5 = np.tile(np.asarray(FIXED_TRIPLE, np.float32), (5, 1))

    def production_step():
        # the reference trainer's order for a Muon group (src/training/optimizer_muon/tma.rs:38-201): prepare,
        # five Newton-Schulz iterations, finish with NorMuon + qk-clip and deferred quantisation, then the
        # cached training weights y are materialised as NVFP4
        a = A(normuon=True, qk_clip_factors=factors, coefficients=co5, **base)
        opt.muon_tma_prepare_polar(plan, table, a)
        opt.muon_polar(plan, a)
        opt.muon_tma_finish_update_deferred_quantization(plan, table, a)
        opt.muon_materialize_training_weights(plan, table)

    cases.append(("production-order step: prepare + 5x NS + finish (NorMuon, qk-clip, deferred) + materialise y", 0.0,
                  production_step))
    for name, bpe, fn in cases:
        if args.only and args.only not in name:
            continue
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 10
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps
        gbs = n_el * bpe / (ms * 1e-3) / 1e9
        print(json.dumps({"extra": name, "workload": args.workload, "elements": n_el, "ms": ms, "bytes_per_element": bpe,
                          "gbs": gbs, "frac_of_measured_hbm": gbs / peaks["hbm"], "status": plan.status()}), flush=True)
    plan.close()
    plan1.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="gpt2-small", choices=sorted(MODELS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-graph", action="store_true", help="time eager launches instead of a CUDA graph replay")
    ap.add_argument("--no-scaling-workloads", action="store_true",
                    help="skip the GPT-2 XL / medium steps that the default run adds to the line")
    ap.add_argument("--two-pass-prepare", action="store_true",
                    help="stages M+N with the reference's rounding point (the gradients are read twice) instead of "
                         "the one-pass form")
    ap.add_argument("--ns-schedule", choices=["per-phase", "chained", "fused"], default="per-phase",
                    help="Newton-Schulz launches: three per iteration, one chained persistent launch for the whole loop, "
                         "or two per iteration with the Gram and polynomial tile of a position fused on one CTA pair")
    ap.add_argument("--update-16bit", action="store_true",
                    help="the last Newton-Schulz iteration stores BF16 and the update reads it (default: FP32, as the "
                         "reference's update input)")
    ap.add_argument("--gather", choices=["nccl", "p2p"], default="p2p",
                    help="N > 1: how the packed weights are exchanged: this library's own copy kernels into the other "
                         "ranks' arenas through peer memory (CUDA IPC; measured 2-9 %% faster steps on four GPUs), or "
                         "ncclAllGather per bucket")
    ap.add_argument("--gather-buckets", type=int, default=0,
                    help="N > 1: cut the matrices into this many buckets; the all-gather of a bucket overlaps the next "
                         "bucket's update + quantise launch (0: one per estimated 0.25 ms of gathering, at most four)")
    ap.add_argument("--shard-of", type=int, default=1,
                    help="with one GPU: run rank 0's share of an N-way sharded step (no collective), to time the "
                         "per-rank kernels of a multi-GPU run")
    ap.add_argument("--plan-flags", type=int, default=0,
                    help="kernel variants of a library built with -DB2_MEASURE (ignored otherwise)")
    ap.add_argument("--sweep", action="store_true", help="update+quantise bandwidth sweep over [R, 4096] tensors")
    ap.add_argument("--extras", action="store_true",
                    help="time the entry points beside the headline step (variants, clip, materialisation, converter)")
    ap.add_argument("--only", default="", help="with --extras: run only the cases whose name contains this text")
    args = ap.parse_args()
    if args.sweep:
        run_sweep(args)
        return
    if args.extras:
        run_extras(args)
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
