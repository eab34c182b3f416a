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
"""
from __future__ import annotations

import argparse
import json
import os
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
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for nm, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        os.unlink(self.path)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        # the load is bursty at this sampling rate: report the median of the upper half
        top = sorted(sm)[len(sm) // 2:]
        return {"sm_mhz": float(np.median(top)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------------------------------
# CPU arm: the oracle port on the host cores (bounded sample: one transformer layer)
# ------------------------------------------------------------------------------------------
def cpu_sample_ms(model, steps=1):
    from oracle import oracle as o

    layers, d, vocab, pos = MODELS[model]
    rng = np.random.default_rng(0)
    shapes = layer_shapes(d)
    co = o.fixed_coefficients(5)
    state = []
    for r, c in shapes:
        n = r * c
        state.append(((rng.standard_normal(n) * 1e-3).astype(np.float32), np.zeros(n, np.uint16),
                      (rng.standard_normal(n) * 0.02).astype(np.float32), (rng.standard_normal(n) * 0.02).astype(np.float32)))
    na = ((vocab + pos) * d // layers + 15) // 16 * 16
    az = (rng.standard_normal(na) * 0.02).astype(np.float32)
    ag = (rng.standard_normal(na) * 1e-3).astype(np.float32)
    am1, am2 = np.zeros(na, np.float32), np.zeros(na, np.float32)
    best = float("inf")
    for _ in range(max(steps, 1)):
        t0 = time.perf_counter()
        for (g, m, z, x), (r, c) in zip(state, shapes):
            o.muon_step(g, m, z, x, r, c, mu=HP["mu"], grad_scale=1.0, lr=HP["learning_rate"], wd=HP["weight_decay"],
                        c_avg=HP["average_coefficient"], sched_beta=HP["schedule_beta"], iterations=5, coeffs=co,
                        round_mode=o.ROUND_BF16)
        z2, x2, *_ = o.adamw(az, az, ag, am1, am2, 1.0, ADAM["learning_rate"], ADAM["weight_decay"], 0.9, 0.95, 0.1,
                             0.05, 1e-10, 0.5, 0.2)
        o.nvfp4_quantize(x2)
        best = min(best, (time.perf_counter() - t0) * 1e3)
    return best * layers, f"1 of {layers} layers (4 matrices) + 1/{layers} of the AdamW elements, scaled x{layers}"


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    os.environ.setdefault("OMP_NUM_THREADS", str(cores))
    for _ in range(args.warmup and 1):
        cpu_sample_ms(args.workload, 1)
    t = [cpu_sample_ms(args.workload, 1) for _ in range(min(args.steps, 3))]
    ms = float(np.mean([x[0] for x in t]))
    line = {
        "impl": "reference", "metric": METRIC, "value": ms, "unit": "ms", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args.workload, args.gpus),
        "note": "CPU oracle port of the reference path on the host cores (the reference itself is Rust + cuda-oxide "
                "and cannot be built in this image); rank 0 only, whatever --gpus says",
        "cpu_baseline": {"value": ms, "unit": "ms", "cores": cores, "kind": "port", "sample": t[0][1]},
        "e2e": {"value": ms, "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------
def run_gpu(args):
    import torch
    import torch.distributed as dist

    import llmini_b200 as b2
    from llmini_b200.dist import Nvfp4Arena, shard_plan

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the optimizer path has no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)

    mats, emb, vec = model_shapes(args.workload)
    d_model = MODELS[args.workload][1]
    layout = b2.SCALES_CSF if d_model % 128 == 0 else b2.SCALES_RAW
    owner, _ = shard_plan(mats, world)
    mine = [i for i, r in enumerate(owner) if r == rank]
    my_shapes = [mats[i] for i in mine]

    def scales_bytes(rows, cols):
        return b2.csf_encoded_len(rows, cols) if layout == b2.SCALES_CSF else rows * cols // 16

    arena = Nvfp4Arena(mats, owner, world, scales_bytes)
    arena_t = torch.zeros(arena.total_bytes + 1024, dtype=torch.uint8, device=dev)
    abase = (-arena_t.data_ptr()) % 256
    arena_v = arena_t[abase:abase + arena.total_bytes]

    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    randn = lambda n, std: torch.randn(n, device=dev, generator=gen) * std
    slots = []
    for i in mine:
        r, c = mats[i]
        co, so, go = arena.offsets(i)
        nb = arena.entries[i]
        s = b2.MuonSlot(
            grad=randn(r * c, 1e-3).view(r, c), momentum=torch.zeros(r, c, dtype=torch.bfloat16, device=dev),
            z_master=randn(r * c, 0.02).view(r, c), x_master=randn(r * c, 0.02).view(r, c),
            schedule_amax=torch.zeros(1, device=dev), bytes=arena_v[co:co + nb.codes_bytes],
            scales=arena_v[so:so + nb.scales_bytes], global_scale=arena_v[go:go + 4].view(torch.float32),
            rows=r, cols=c)
        if layout == b2.SCALES_CSF:
            s.scales.copy_(b2.zero_scales(r, c, dev))
        slots.append(s)
    plan = b2.MuonPlan(my_shapes, scale_layout=layout, device=dev, debug_flags=args.plan_flags) if my_shapes else None
    table = b2.slot_table(slots, dev) if slots else None
    opt = b2.OptimizerModule()
    margs = b2.MuonMegaUpdateArgs(coefficients=np.tile(np.asarray([3.4445, -4.7750, 2.0315], np.float32), (5, 1)), **HP)

    # AdamW parameters: embeddings (requantised) split by rank on row boundaries, vectors on rank 0
    adam_sets = []
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
        adam_sets.append(("quant", t))
    if rank == 0:
        t = dict(z_master=randn(vec, 0.02), x_master=randn(vec, 0.02), grad=randn(vec, 1e-3),
                 first_moment=torch.zeros(vec, device=dev), second_moment=torch.zeros(vec, device=dev), len=vec)
        adam_sets.append(("fp32", t))

    adam_table = adam_count = adam_chunks = None
    if adam_sets:
        # every AdamW tensor of the rank in one pointer table: three launches for all of them
        adam_table, adam_count, adam_chunks = opt.adamw_table(
            [dict(t, mode=2 if kind == "quant" else 0) for kind, t in adam_sets], dev)
    launches_per_step = 0
    if plan is not None:
        # sumsq, inv_norm, momentum_normalize; three GEMMs per iteration; update + encode in one launch
        launches_per_step += 3 + 3 * HP["iterations"] + (2 if args.plan_flags & 16 else 1)
    launches_per_step += 3 if adam_sets else 0

    stream = torch.cuda.current_stream()
    ev = lambda: torch.cuda.Event(enable_timing=True)
    stage_events = []

    def step_muon(record=False, marks=None):
        if record: marks[0].record(stream)
        if plan is not None:
            opt.muon_tma_prepare_polar(plan, table, margs)
        if record: marks[1].record(stream)
        if plan is not None:
            opt.muon_polar(plan, margs)
        if record: marks[2].record(stream)
        if plan is not None:
            opt.muon_tma_finish_update(plan, table, margs)
        if record: marks[3].record(stream)

    def step_adam(record=False, marks=None):
        if adam_sets:
            opt.apply_adamw_update_multi(adam_table, adam_count, adam_chunks, **ADAM)
        if record: marks[4].record(stream)
        if world > 1:
            n = arena.bytes_per_rank
            dist.all_gather_into_tensor(arena_v, arena_v[rank * n:(rank + 1) * n])

    def step(record=False):
        marks = [ev() for _ in range(5)] if record else None
        step_muon(record, marks)
        step_adam(record, marks)
        if record: stage_events.append(marks)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = ev(), ev()
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / steps

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    if plan is not None and plan.status() != 0:
        raise SystemExit("a bounded device-side wait ran out during warm-up")

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
                step_muon()
            with torch.cuda.graph(graph_adam):
                step_adam()
        except Exception as exc:  # capture is an optimisation; report why it was skipped
            graph = graph_muon = graph_adam = None
            graph_error = repr(exc)[:200]

    # ---- end to end: host gradients in, packed weights out, every step ----
    # What a caller with host-resident gradients does with the same public calls: the matrix
    # gradients go up first; while the Muon stages run, a second stream brings up the AdamW
    # gradients, and a third takes the packed matrices down (PCIe is full duplex); AdamW and its
    # outputs follow.  Every copy is inside the timed region; the step ends when the last byte is on
    # the host.
    n_slots = len(slots)
    grad_dev = [s.grad for s in slots] + [t["grad"] for _, t in adam_sets]
    grad_host = [torch.empty(g.shape, dtype=g.dtype, pin_memory=True).copy_(g) for g in grad_dev]
    n_mine = arena.bytes_per_rank
    out_dev = [arena_v[rank * n_mine:(rank + 1) * n_mine]] + \
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
            out_host[0].copy_(out_dev[0], non_blocking=True)
            down_done = torch.cuda.Event()
            down_done.record(down_stream)
        stream.wait_event(adam_up)
        if graph_adam is not None:
            graph_adam.replay()
        else:
            step_adam()
        adam_done.record(stream)
        for od, oh in zip(out_dev[1:], out_host[1:]):
            oh.copy_(od, non_blocking=True)
        stream.wait_event(down_done)

    step_e2e()
    ms_e2e = timed(step_e2e, args.steps)
    clocks = sampler.stop() if rank == 0 else None
    if plan is not None and plan.status() != 0:
        raise SystemExit("a bounded device-side wait ran out during the timed region")

    # ---- per-stage device times (this rank) ----
    torch.cuda.synchronize()
    st = np.array([[m[i].elapsed_time(m[i + 1]) for i in range(4)] for m in stage_events]) if stage_events else np.zeros((1, 4))
    prep_ms, ns_ms, fin_ms, adam_ms = (float(v) for v in st.mean(axis=0))
    elems = sum(r * c for r, c in my_shapes)
    flops = ns_flops(my_shapes, HP["iterations"])
    peaks = load_peaks()
    ns_tflops = flops / (ns_ms * 1e-3) / 1e12 if ns_ms > 0 else 0.0
    # stage U+Q: reads U,z,x; writes z,x,y(schedule cache),codes,scales = 24.5625 B per element
    fin_gbs = elems * 24.5625 / (fin_ms * 1e-3) / 1e9 if fin_ms > 0 else 0.0
    prep_gbs = elems * 10.0 / (prep_ms * 1e-3) / 1e9 if prep_ms > 0 else 0.0
    adam_elems = sum(t["len"] for _, t in adam_sets)
    adam_gbs = adam_elems * 36.0 / (adam_ms * 1e-3) / 1e9 if adam_ms > 0 else 0.0

    def finish():
        # Release the captured graph before the communicator: a graph that still holds NCCL
        # kernels can keep the communicator's teardown waiting.  A watchdog ends the process if
        # teardown stalls anyway; by then the result line has been printed.
        nonlocal graph, graph_muon, graph_adam
        if world == 1:
            return
        import threading
        threading.Timer(30.0, lambda: os._exit(0)).start()
        graph = graph_muon = graph_adam = None
        torch.cuda.synchronize()
        dist.barrier()
        dist.destroy_process_group()
        os._exit(0)

    if rank != 0:
        finish()
        return
    peak_tf = peaks["tf_sustained"]
    line = {
        "metric": METRIC, "value": ms_step, "unit": "ms", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args.workload, world),
        "roofline": {
            "bound": "tensor", "kernel": "k_ns_gemm (15 launches per step)", "achieved": ns_tflops, "peak": peak_tf,
            "unit": "TFLOP/s", "frac": ns_tflops / peak_tf,
            # DRAM bytes per launch, mean of the Gram / Poly / Apply launches in the committed ncu capture
            # (profiles/k_ns_gemm_pair_gpt2-small.md); known for this workload on one GPU only
            "traffic": 262.0e6 if (args.workload == "gpt2-small" and world == 1) else None,
            "peak_source": f"{peaks['source']} bf16 sustained (kernel timed inside a long step)",
            "frac_of_nominal_2250": ns_tflops / 2250.0,
        },
        "stages": {
            "prepare_ms": prep_ms, "newton_schulz_ms": ns_ms, "update_quantise_ms": fin_ms, "adamw_ms": adam_ms,
            "prepare_gbs": prep_gbs, "update_quantise_gbs": fin_gbs, "update_quantise_frac_of_hbm": fin_gbs / peaks["hbm"],
            "adamw_gbs": adam_gbs, "hbm_peak_gbs": peaks["hbm"], "update_quantise_frac_of_nominal_8000": fin_gbs / 8000.0,
        },
        "e2e": {"value": ms_e2e, "unit": "ms", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h)},
        "gpu_launches": int(launches_per_step * args.steps),
        "clocks": clocks,
        "eager_ms_per_step": ms_eager,
        "cuda_graph": graph is not None,
        "replayed_step_matches_eager": modes_match,
    }
    if world == 1 and not args.no_cpu:
        os.environ.setdefault("OMP_NUM_THREADS", str(os.cpu_count() or 1))
        cms, sample = cpu_sample_ms(args.workload, 1)
        line["cpu_baseline"] = {"value": cms, "unit": "ms", "cores": os.cpu_count() or 1, "kind": "port", "sample": sample}
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
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            opt.muon_tma_finish_update(plan, table, margs)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps
        gbs = n * 24.5625 / (ms * 1e-3) / 1e9
        print(json.dumps({"sweep": "update_quantise", "rows": r, "cols": c, "elements": n, "ms": ms,
                          "bytes_per_element": 24.5625, "gbs": gbs, "frac_of_measured_hbm": gbs / peaks["hbm"],
                          "frac_of_nominal_8000": gbs / 8000.0,
                          "note": "tensors under ~5 M elements stay in the 126 MB L2 between repetitions"}), flush=True)
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
        ("prepare (plain)", 16.0, lambda: opt.muon_tma_prepare_polar(plan, table, A(**base))),
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
    co5 = np.tile(np.asarray([3.4445, -4.7750, 2.0315], np.float32), (5, 1))

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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="gpt2-small", choices=sorted(MODELS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-graph", action="store_true", help="time eager launches instead of a CUDA graph replay")
    ap.add_argument("--plan-flags", type=int, default=0,
                    help="measurement only: kernel flags of the plan (16 = update and encode as two launches, "
                         "32 = no programmatic dependent launch between the GEMMs)")
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
