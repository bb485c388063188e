#!/usr/bin/env python
"""Benchmark of the fused INT4/INT8 dequantise + matmul operator on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one pass of the operator over every projection of the workload (default
workload: the Qwen2.5-7B decode MLP, fused gate+up GEMV then down GEMV, int4 group 128,
M=1).  Inputs are seeded synthetic tensors with the model's shapes.

  value   weight GB/s with everything resident in HBM: (packed weights + scales + zeros
          read per step) / device time per step.  The K steps are captured in one CUDA graph
          (the device, not the Python launch loop, sets the pace) whose replays are timed with
          CUDA events, enough replays for a timed region of at least 20 ms whatever K is;
          ms_per_step is the median replay divided by K.  Each step reads a different copy of
          the weights (copies x bytes > 2 x L2), so no step finds its weights in L2.
  e2e     the same metric through the public call, metal_native._C.dequant_matmul, with
          the activations in pinned host memory: every step copies them to the device,
          runs the operator and copies the result back to pinned host memory, then
          waits.  Weights stay resident (they are model state, loaded once).
  roofline  the dominant kernel (the largest projection) timed alone the same way,
          algorithmic bytes / duration against the measured HBM copy peak.
  secondary  N=1, default workload: the prefill half of the metric (M=512 tensor-core path,
          TFLOP/s) measured in the same run.
  cpu_baseline  the reference's CPU dequantise-then-matmul path on the host cores, same
          workload: the reference's own helpers compiled from its checkout (oracle/_ref) when
          that library is present, else the line-by-line port (oracle/dequant_oracle.c).

With --gpus N > 1 (launched by torch.distributed.run, one rank per GPU) the workload is
the Llama-3-70B int8 per-channel layers column-sharded over N, each step ending in an
all-gather of the output slices; the value is the whole-job aggregate.  Before the timed
region every rank checks the gathered outputs (fused gather == operator + NCCL all-gather,
bit for bit; sampled columns against the CPU oracle) and the line carries the verdict in
"parity"; config.scale_anchor holds the time of the SAME layers unsharded on one GPU,
measured in the same run, and the speed-up and efficiency against it.

--impl reference times the CPU path only (rank 0), as the reference arm.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for _p in (str(ROOT / "metal-native_b200"), str(ROOT)):
    if _p not in sys.path:
        sys.path.insert(0, _p)

FALLBACK_HBM_GBS = 6650.0   # used only if MEASURED_PEAKS.json is absent ("of fallback")
FALLBACK_TFLOPS = 1590.0
PREFILL_METRIC = "prefill TFLOP/s"
MIN_REGION_MS = 20.0
SCALING_WORKLOAD = "llama70b-int8-m1"

# dram__bytes_read.sum + dram__bytes_write.sum of one launch of a workload's dominant kernel, each
# from one ncu capture of this program on that workload (--workload NAME --steps 2 --warmup 3)
TRAFFIC = {
    "qwen7b-decode": 72_212_736 + 1_035_008,
    "qwen7b-prefill": 39_830_016 + 378_368,
}

DESCRIPTIONS = {
    "qwen7b-decode": "Qwen2.5-7B decode MLP: gate+up [1,3584]x[37888,3584]^T then down [1,18944]x[3584,18944]^T, "
                     "int4 g128 asym, fp16",
    "qwen7b-prefill": "Qwen2.5-7B prefill M=512: K=3584,N=18944 and K=18944,N=3584, int4 g128 asym, fp16",
}


def describe(name):
    if name in DESCRIPTIONS:
        return DESCRIPTIONS[name]
    M = int(name.rsplit("m", 1)[1])
    if name.startswith("llama8b-decode-m"):
        return f"Llama-3-8B batched decode M={M}: K=4096,N=14336 and K=14336,N=4096, int4 g128 sym, bf16"
    if name.startswith("llama70b-int8-m"):
        return (f"Llama-3-70B M={M}: K=8192,N=57344 and K=28672,N=8192, int8 per-channel, bf16, "
                f"column-sharded over the GPUs of the job")
    raise SystemExit(f"unknown workload {name}")


def metric_of(name):
    if name == "qwen7b-prefill":
        return PREFILL_METRIC, "TFLOP/s"
    return ("int8" if name.startswith("llama70b") else "int4") + " dequant-GEMV weight GB/s", "GB/s"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="auto",
                    help="auto | qwen7b-decode | llama8b-decode-m{4,16,32} | qwen7b-prefill | "
                         "llama70b-int8-m{1,64}")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true", help="skip the prefill and scaling-anchor measurements")
    ap.add_argument("--gather", default="auto", choices=["auto", "fused", "nccl"],
                    help="N > 1: all-gather inside the decode kernel (peer stores) or NCCL after it")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    return ap.parse_args()


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return {"hbm": float(d["hbm_gbs"]), "tensor": float(d["bf16_tflops"]),
                    "tensor_sustained": d.get("bf16_tflops_sustained"), "kind": "measured"}
        except Exception:
            pass
    return {"hbm": FALLBACK_HBM_GBS, "tensor": FALLBACK_TFLOPS, "tensor_sustained": None, "kind": "fallback"}


def workload_name(args, world):
    if args.workload != "auto":
        return args.workload
    return "qwen7b-decode" if world == 1 else SCALING_WORKLOAD


def build_layers(name, world, rank):
    """CPU tensors of this rank's share of the workload; identical on every call."""
    import mnq_workloads as workloads
    if name == "qwen7b-decode":
        return workloads.config1()
    if name.startswith("llama8b-decode-m"):
        return workloads.config2(int(name.rsplit("m", 1)[1]))
    if name == "qwen7b-prefill":
        return workloads.config3()
    if name.startswith("llama70b-int8-m"):
        return workloads.config4(int(name.rsplit("m", 1)[1]), world_size=world, rank=rank)
    raise SystemExit(f"unknown workload {name}")


# --------------------------------------------------------------------------- CPU arm

def cpu_kind():
    from oracle import ref
    return "reference" if ref.available() else "port"


def cpu_path_time(layers, seconds, max_steps=None):
    """Times the reference's CPU path on all host threads (output columns split over them): its
    own helpers when oracle/_ref is built, else the port.  Returns (times per step, threads)."""
    import numpy as np
    from oracle import check as H
    from oracle import oracle, ref
    threads = oracle.host_threads()
    use_ref = ref.available()
    prepared = []
    for L in layers:
        s = H.f32(L.scales)
        prepared.append((H.f32(L.x), L.wq.contiguous().numpy(), s,
                         H.f32(L.zeros) if L.zeros is not None else None, L.group_size, L.quant_type,
                         None if use_ref else np.empty((L.N, L.K), np.float32)))
    times = []
    t_end = time.perf_counter() + seconds
    while True:
        t0 = time.perf_counter()
        for (x, wq, s, z, g, qt, scratch) in prepared:
            if use_ref:
                ref.dequant_matmul(x, wq, s, z, g, qt, threads=threads)
            else:
                oracle.dequant_matmul(x, wq, s, z, g, qt, threads=threads, scratch=scratch)
        times.append(time.perf_counter() - t0)
        if time.perf_counter() >= t_end or (max_steps and len(times) >= max_steps):
            break
    return times, threads


def cpu_sample_layers(layers, budget_macs=4e9):
    """Bounds the CPU work of one step: if a layer needs more than `budget_macs`
    multiply-adds, keep only its first rows n (a contiguous block of output columns) and
    say so.  Throughput in weight GB/s is unaffected by the cut."""
    from mnq_workloads import Layer
    out, notes = [], []
    for L in layers:
        macs = L.M * L.N * L.K
        if macs <= budget_macs:
            out.append(L)
            continue
        n_keep = max(16, int(L.N * budget_macs / macs) // 16 * 16)
        out.append(Layer(L.name, L.quant_type, L.M, L.K, n_keep, L.group_size, L.x, L.wq[:n_keep].contiguous(),
                         L.scales[:n_keep].contiguous(), None if L.zeros is None else L.zeros[:n_keep].contiguous()))
        notes.append(f"{L.name}: first {n_keep} of {L.N} output columns")
    return out, notes


CPU_ARM = {"reference": "the reference's own CPU helpers (tests/cpp/test_dequant_matmul.mm:103-259, compiled from the "
                        "reference checkout into oracle/_ref), output columns split over host threads",
           "port": "line-by-line port of the reference's CPU helpers (tests/cpp/test_dequant_matmul.mm:119-213), "
                   "output columns split over host threads"}


def cpu_baseline(layers_cpu, unit, seconds):
    sample, notes = cpu_sample_layers(layers_cpu)
    times, threads = cpu_path_time(sample, seconds)
    best = sorted(times)[len(times) // 2]
    prefill = unit == "TFLOP/s"
    work = sum(L.flops for L in sample) / 1e3 if prefill else sum(L.weight_bytes for L in sample)
    return {"value": work / best / 1e9, "unit": unit, "cores": threads, "kind": cpu_kind(), "ms_per_step": best * 1e3,
            "sample": (f"{len(times)} whole steps" if not notes else f"{len(times)} steps of: " + "; ".join(notes))
            + f", median, {threads} threads splitting the output columns"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    name = workload_name(args, world)
    layers = build_layers(name, 1, 0)
    sample, notes = cpu_sample_layers(layers)
    metric, unit = metric_of(name)
    prefill = unit == "TFLOP/s"
    work = sum(L.flops for L in sample) / 1e3 if prefill else sum(L.weight_bytes for L in sample)
    cpu_path_time(sample, 1e9, max_steps=max(1, min(args.warmup, 3)))           # warm-up steps
    times, threads = cpu_path_time(sample, 1e9, max_steps=max(1, args.steps))   # exactly K steps
    total = sum(times)
    value = work * len(times) / total / 1e9
    kind = cpu_kind()
    sample_desc = "whole workload per step" if not notes else "; ".join(notes)
    line = {
        "impl": "reference", "metric": metric, "value": value, "unit": unit, "n_gpus": args.gpus,
        "steps": len(times), "warmup": args.warmup, "ms_per_step": total / len(times) * 1e3,
        "higher_is_better": True, "scaling": "strong" if world > 1 else "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": name, "description": describe(name), "arm": "CPU: " + CPU_ARM[kind]},
        "cpu_baseline": {"value": value, "unit": unit, "cores": threads, "kind": kind, "sample": sample_desc},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- clocks

class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(gpu_index)], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()   # the exact child started above
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        rows = [r.split(",") for r in Path(self.file.name).read_text().strip().splitlines() if r.strip()]
        os.unlink(self.file.name)
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            try:
                r = [c.strip() for c in r]
                sm.append(float(r[1])); mx.append(float(r[2])); pw.append(float(r[3]))
                for nme, val in zip(names, r[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(nme)
            except (ValueError, IndexError):
                continue
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        # samples under load: power above the midpoint between idle and peak draw
        thr = (min(pw) + max(pw)) / 2 if max(pw) - min(pw) > 50 else -1
        loaded = sorted(s for s, p in zip(sm, pw) if p >= thr) or sorted(sm)
        return {"sm_mhz": loaded[len(loaded) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm), "samples_under_load": len(loaded), "power_w_max": max(pw)}


# --------------------------------------------------------------------------- GPU arm

class Harness:
    """Device state shared by the measurements of one process."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist
        self.torch, self.dist, self.args = torch, dist, args
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != args.gpus and self.world > 1:
            raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={self.world}")
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            import datetime
            dist.init_process_group("nccl", device_id=self.dev, timeout=datetime.timedelta(seconds=300))
        from metal_native import _C
        self._C = _C
        # weights are model state, loaded once and never written while the operator runs
        _C.set_option("weights_immutable", 1)
        self.l2 = torch.cuda.get_device_properties(self.dev).L2_cache_size
        self.stream = torch.cuda.Stream()
        self.peaks = peaks()
        self.last_graph = None

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, v):
        if self.world == 1:
            return v
        t = self.torch.tensor([v], device=self.dev, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def resident_copies(self, layers_cpu):
        """copies x bytes > 2 x L2: the activations are shared, the weights cloned."""
        wbytes = sum(L.weight_bytes for L in layers_cpu)
        copies = min(16, max(2, -(-2 * self.l2 // wbytes) + 1))
        first = [L.to(self.dev) for L in layers_cpu]
        out = [first]
        for _ in range(copies - 1):
            out.append([type(L)(L.name, L.quant_type, L.M, L.K, L.N, L.group_size, L.x, L.wq.clone(), L.scales.clone(),
                                None if L.zeros is None else L.zeros.clone()) for L in first])
        return out, copies, wbytes

    def time_graph(self, step, steps, collective=False):
        """Captures `steps` calls of step(i) in one CUDA graph and times whole replays with CUDA
        events on the launching stream; returns (median ms per step, replays, region ms).  With
        collectives inside, every rank runs the same number of replays (agreed from the slowest
        rank's first replay) between two barriers, and the median is the maximum over ranks."""
        torch = self.torch
        with torch.cuda.stream(self.stream):
            step(0)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=self.stream):
                for i in range(steps):
                    step(i)
            graph.replay()          # untimed: uploads the graph
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(self.stream); graph.replay(); b.record(self.stream)
            torch.cuda.synchronize()
            first_ms = a.elapsed_time(b)
            if collective:
                first_ms = self.max_over_ranks(first_ms)
            replays = int(min(2000, max(3, -(-MIN_REGION_MS // max(first_ms, 1e-3)))))
            if collective:
                self.barrier()
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(replays + 1)]
            ev[0].record(self.stream)
            for r in range(replays):
                graph.replay()
                ev[r + 1].record(self.stream)
            if collective:
                self.barrier()
            else:
                torch.cuda.synchronize()
            per = [ev[r].elapsed_time(ev[r + 1]) for r in range(replays)]
            region = ev[0].elapsed_time(ev[replays])
        med = statistics.median(per)
        if collective:
            med = self.max_over_ranks(med)
        self.last_graph = graph
        return med / steps, replays, region


def launches_of(_C, L, fused_gather=False):
    """Kernels one projection launches: one, plus a reduce kernel when K is split on the
    tensor-core path or on the many-token (M > 8) decode path."""
    path = _C.select_path(L.M, L.N, L.K, L.group_size, L.quant_type, L.x.dtype, zeros=L.zeros is not None,
                          scale_dtype=L.scales.dtype)
    q = 0 if L.quant_type == "int4" else 1
    split = ((path == "gemm" or (path == "gemv" and L.M > 8 and not fused_gather)) and
             _C._lib.mnq_workspace_bytes(L.M, L.N, L.K, int(L.group_size), q) > 0)
    return 2 if split else 1


def measure_single_gpu(h, name, steps, want_e2e=True):
    """Device-time value, dominant-kernel roofline and e2e of a workload that runs on this
    process's GPU alone.  Returns a dict with the pieces of a JSON line."""
    torch, _C = h.torch, h._C
    layers_cpu = build_layers(name, 1, 0)
    metric, unit = metric_of(name)
    prefill = unit == "TFLOP/s"
    dev_layers, copies, wbytes = h.resident_copies(layers_cpu)
    outs = [torch.empty((L.M, L.N), dtype=L.x.dtype, device=h.dev) for L in layers_cpu]

    def step(i):
        for j, L in enumerate(dev_layers[i % copies]):
            _C.dequant_matmul(L.x, L.wq, L.scales, L.zeros, L.group_size, L.quant_type, out=outs[j])

    for i in range(max(3, h.args.warmup)):
        step(i)
    torch.cuda.synchronize()
    ms, replays, region = h.time_graph(step, steps)
    main_graph = h.last_graph
    work = sum(L.flops for L in layers_cpu) / 1e3 if prefill else wbytes   # TFLOP/s = flops / s / 1e12
    value = work / (ms * 1e-3) / 1e9

    # ---- roofline: the dominant kernel alone, same protocol
    dom = max(range(len(layers_cpu)), key=lambda j: (layers_cpu[j].flops if prefill else layers_cpu[j].weight_bytes))
    Ld = layers_cpu[dom]

    def dom_step(i):
        L = dev_layers[i % copies][dom]
        _C.dequant_matmul(L.x, L.wq, L.scales, L.zeros, L.group_size, L.quant_type, out=outs[dom])

    dom_ms, _, _ = h.time_graph(dom_step, max(50, min(steps, 400)))
    dom_us = dom_ms * 1e3
    kernel = _C.select_path(Ld.M, Ld.N, Ld.K, Ld.group_size, Ld.quant_type, Ld.x.dtype, zeros=Ld.zeros is not None,
                            scale_dtype=Ld.scales.dtype)
    pk = h.peaks
    if prefill:
        achieved = Ld.flops / (dom_us * 1e-6) / 1e12
        roofline = {"bound": "tensor", "kernel": f"{kernel} ({Ld.name})", "achieved": achieved, "peak": pk["tensor"],
                    "peak_source": f"{pk['kind']} cuBLAS bf16 burst", "unit": "TFLOP/s", "frac": achieved / pk["tensor"],
                    "frac_of_nominal_2250TF": achieved / 2250.0, "traffic": TRAFFIC.get(name),
                    "flops_per_launch": Ld.flops, "us_per_launch": dom_us}
        if pk["tensor_sustained"]:   # timed back to back for thousands of launches, i.e. under the power cap
            roofline["peak_sustained"] = float(pk["tensor_sustained"])
            roofline["frac_of_sustained"] = achieved / float(pk["tensor_sustained"])
    else:
        achieved = Ld.total_bytes / (dom_us * 1e-6) / 1e9
        roofline = {"bound": "hbm", "kernel": f"{kernel} ({Ld.name})", "achieved": achieved, "peak": pk["hbm"],
                    "peak_source": f"{pk['kind']} HBM copy bandwidth", "unit": "GB/s", "frac": achieved / pk["hbm"],
                    "frac_of_nominal_8TBs": achieved / 8000.0, "traffic": TRAFFIC.get(name),
                    "algorithmic_bytes_per_launch": Ld.total_bytes, "weight_bytes_per_launch": Ld.weight_bytes,
                    "weight_GBps": Ld.weight_bytes / (dom_us * 1e-6) / 1e9, "us_per_launch": dom_us}

    res = {"name": name, "metric": metric, "unit": unit, "value": value, "ms_per_step": ms, "replays": replays,
           "region_ms": region, "roofline": roofline, "copies": copies, "wbytes": wbytes, "work": work,
           "layers_cpu": layers_cpu, "dtype": "f16" if layers_cpu[0].x.dtype == torch.float16 else "bf16",
           "launches_per_step": sum(launches_of(_C, L) for L in layers_cpu), "graph": main_graph}

    # ---- end to end through the public call, host buffers
    if want_e2e:
        xs_host = [L.x.pin_memory() for L in layers_cpu]
        outs_host = [torch.empty((L.M, L.N), dtype=L.x.dtype).pin_memory() for L in layers_cpu]

        def host_step(c):
            def body():
                for j, L in enumerate(dev_layers[c]):
                    # host activations in, host result out: the operator enqueues the copies itself
                    _C.dequant_matmul(xs_host[j], L.wq, L.scales, L.zeros, L.group_size, L.quant_type, out=outs_host[j])
            return body

        # the public phase pipeline decides how a step is issued: a decode step is recorded once
        # and replayed with one launch (one recording per weight copy), a prefill step runs eagerly
        import metal_native
        pipe = metal_native.PhasePipeline()
        phase = pipe.auto_detect_phase(batch_size=layers_cpu[0].M, seq_len=1 if layers_cpu[0].M <= 32 else layers_cpu[0].M)
        issue = [pipe.capture_step(host_step(c)) for c in range(copies)]

        def e2e_step(i):
            issue[i % copies]()
            torch.cuda.current_stream().synchronize()

        e2e_steps = min(max(steps, 50), 400)
        for i in range(5):
            e2e_step(i)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record()
        for i in range(e2e_steps):
            e2e_step(i)
        c1.record()
        torch.cuda.synchronize()
        e2e_ms = max(c0.elapsed_time(c1), (time.perf_counter() - t0) * 1e3)
        res["e2e"] = {"value": work * e2e_steps / (e2e_ms * 1e-3) / 1e9, "unit": unit,
                      "h2d_bytes_per_step": sum(x.numel() * x.element_size() for x in xs_host),
                      "d2h_bytes_per_step": sum(o.numel() * o.element_size() for o in outs_host),
                      "ms_per_step": e2e_ms / e2e_steps, "steps": e2e_steps,
                      "call": "metal_native._C.dequant_matmul(host activations, out=host tensor) per projection (the operator "
                              "copies the activations in and writes the result to the pinned host tensor), issued through "
                              f"metal_native.PhasePipeline.capture_step ({phase.name}: "
                              + ("recorded once, replayed with one launch per step" if pipe.active_config().capture_graph
                                 else "eager") + "), stream synchronised every step; weights resident"}
    return res


def keep_load_on(h, graph, ms_per_replay, seconds=1.0, cap=3000):
    for _ in range(max(1, min(cap, int(seconds * 1e3 / max(ms_per_replay, 1e-3))))):
        graph.replay()
    h.torch.cuda.synchronize()


def run_single(h, args):
    name = workload_name(args, 1)
    sampler = ClockSampler(h.local)
    main = measure_single_gpu(h, name, args.steps, want_e2e=True)
    keep_load_on(h, main["graph"], main["ms_per_step"] * args.steps)   # for the clock sampler
    clocks = sampler.stop()
    cpu = None if args.no_cpu_baseline else cpu_baseline(main["layers_cpu"], main["unit"], args.cpu_seconds)
    pk = h.peaks
    prefill = main["unit"] == "TFLOP/s"
    config = {"workload": name, "description": describe(name), "weight_copies": main["copies"],
              "l2_policy": f"inputs larger than L2: {main['copies']} weight copies x {main['wbytes'] / 1e6:.1f} MB "
                           f"rotate, L2 = {h.l2 / 1e6:.0f} MB",
              "launch": f"{args.steps} steps captured in one CUDA graph; {main['replays']} replays timed with CUDA events "
                        f"({main['region_ms']:.1f} ms region), median replay / {args.steps}",
              "weights_immutable": True, "collective": None, "weight_bytes_per_step": main["wbytes"],
              "frac_of_measured_hbm": None if prefill else main["value"] / pk["hbm"],
              "frac_of_nominal_8TBs": None if prefill else main["value"] / 8000.0}
    line = {"metric": main["metric"], "value": main["value"], "unit": main["unit"], "n_gpus": 1, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": main["ms_per_step"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": main["dtype"], "data": "synthetic", "config": config,
            "roofline": main["roofline"], "cpu_baseline": cpu, "e2e": main["e2e"], "clocks": clocks,
            "gpu_launches": main["launches_per_step"] * args.steps * (main["replays"] + 2)}
    del main
    h.torch.cuda.empty_cache()

    if name == "qwen7b-decode" and not args.no_secondary:
        # the prefill half of the metric, same run
        pre_steps = min(args.steps, 100)
        s2 = ClockSampler(h.local)
        pre = measure_single_gpu(h, "qwen7b-prefill", pre_steps, want_e2e=False)
        keep_load_on(h, pre["graph"], pre["ms_per_step"] * pre_steps, seconds=1.5, cap=200)
        line["secondary"] = [{"metric": pre["metric"], "unit": pre["unit"], "value": pre["value"],
                              "ms_per_step": pre["ms_per_step"], "steps": pre_steps,
                              "config": {"workload": "qwen7b-prefill", "description": describe("qwen7b-prefill"),
                                         "weight_copies": pre["copies"], "replays": pre["replays"],
                                         "region_ms": pre["region_ms"]},
                              "frac_of_measured_burst": pre["value"] / pk["tensor"],
                              "frac_of_measured_sustained": (pre["value"] / float(pk["tensor_sustained"])
                                                             if pk["tensor_sustained"] else None),
                              "frac_of_nominal_2250TF": pre["value"] / 2250.0,
                              "roofline": pre["roofline"], "clocks": s2.stop(), "dtype": pre["dtype"]}]
        del pre
        h.torch.cuda.empty_cache()
        # the one-GPU anchor of the multi-GPU scaling series: the sharded workload, unsharded
        anc = measure_single_gpu(h, SCALING_WORKLOAD, min(args.steps, 100), want_e2e=False)
        line["config"]["scale_anchor"] = {"workload": SCALING_WORKLOAD, "n1_ms_per_step": anc["ms_per_step"],
                                          "n1_value": anc["value"], "unit": anc["unit"], "speedup": 1.0,
                                          "efficiency": 1.0, "frac_of_measured_hbm": anc["value"] / pk["hbm"]}
        del anc
    elif name == SCALING_WORKLOAD:
        line["config"]["scale_anchor"] = {"workload": name, "n1_ms_per_step": line["ms_per_step"],
                                          "n1_value": line["value"], "unit": line["unit"], "speedup": 1.0,
                                          "efficiency": 1.0, "frac_of_measured_hbm": line["value"] / pk["hbm"]}
    print(json.dumps(line), flush=True)


def run_sharded(h, args):
    torch, dist, _C = h.torch, h.dist, h._C
    from metal_native import sharded
    from oracle import check as H
    rank, world, dev = h.rank, h.world, h.dev
    name = workload_name(args, world)
    if not name.startswith("llama70b-int8-m"):
        raise SystemExit("--gpus N > 1 runs the column-sharded Llama-3-70B workloads only")
    layers_cpu = build_layers(name, world, rank)
    sampler = ClockSampler(h.local) if rank == 0 else None
    dev_layers, copies, wbytes_rank = h.resident_copies(layers_cpu)
    outs = [torch.empty((L.M, L.N), dtype=L.x.dtype, device=dev) for L in layers_cpu]
    gathered = [sharded.GatherBuffer(L.M, L.N, world, L.x.dtype, dev) for L in layers_cpu]
    want_fused = args.gather != "nccl" and all(
        L.M <= 32 and _C.select_path(L.M, L.N, L.K, L.group_size, L.quant_type, L.x.dtype, zeros=L.zeros is not None,
                                     scale_dtype=L.scales.dtype) == "gemv" for L in layers_cpu)
    ok = torch.tensor([1 if want_fused else 0], device=dev)
    fused = None
    if want_fused:
        try:
            fused = [sharded.PeerGather(L.M, L.N, world, L.x.dtype, dev) for L in layers_cpu]
        except Exception as e:   # no peer-mapped symmetric memory on this box
            print(f"[bench] rank {rank}: fused gather unavailable ({type(e).__name__}: {e})", file=sys.stderr)
            ok.zero_()
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)     # all ranks take the same route
    if int(ok.item()) == 0:
        if args.gather == "fused":
            raise SystemExit("--gather fused: not available for this workload / on this box")
        fused = None
    collective = ("peer stores from the decode kernel's epilogue + arrival flags (one kernel per projection)"
                  if fused else "NCCL all_gather_into_tensor after each projection")

    def nccl_layer(j, L, x):
        o = _C.dequant_matmul(x, L.wq, L.scales, L.zeros, L.group_size, L.quant_type, out=outs[j])
        return gathered[j].all_gather(o)

    def run_layer(j, L, x):
        """One projection; returns the full [M, N] result on this rank."""
        if fused is not None:
            return fused[j].matmul(x, L.wq, L.scales, L.zeros, L.group_size, L.quant_type)
        return nccl_layer(j, L, x)

    def step(i):
        for j, L in enumerate(dev_layers[i % copies]):
            run_layer(j, L, L.x)

    # ---- parity at this world size, untimed: the gathered output of every projection on every
    # rank, fused route against operator + NCCL all-gather bit for bit, and (rank 0) sampled
    # columns of every rank's slice against the CPU oracle on the unsharded seeded matrix
    full_cpu = build_layers(name, 1, 0) if rank == 0 else None
    parity = {"ranks": world, "fused_eq_nccl": None, "rel_l2": [], "max_abs": [], "columns_checked": 0,
              "device_status": 0}
    failures = []
    for j, L in enumerate(dev_layers[0]):
        via_nccl = nccl_layer(j, L, L.x).clone()
        torch.cuda.synchronize()
        if fused is not None:
            for call in range(2):   # the second call meets the flag words as the first left them
                via_fused = fused[j].matmul(L.x, L.wq, L.scales, L.zeros, L.group_size, L.quant_type).clone()
                torch.cuda.synchronize()
                same = torch.tensor([1 if torch.equal(via_fused, via_nccl) else 0], device=dev)
                dist.all_reduce(same, op=dist.ReduceOp.MIN)
                if int(same.item()) != 1:
                    failures.append(f"{L.name}: fused gather differs from operator + NCCL all-gather (call {call})")
        if rank == 0:
            F = full_cpu[j]
            cols = H.sampled_columns(F.N, 256, world, seed=j)
            ref = H.oracle_matmul(F, cols=cols)
            got = via_nccl[:, torch.as_tensor(cols, device=dev)]
            try:
                rel, mx = H.assert_close_to_oracle(got, ref, F.name)
                parity["rel_l2"].append(rel)
                parity["max_abs"].append(mx)
            except AssertionError as e:
                failures.append(str(e))
            parity["columns_checked"] += int(len(cols))
    if fused is not None:
        parity["fused_eq_nccl"] = not any("fused gather differs" in f for f in failures)
    st = torch.tensor([_C.device_status()], device=dev)
    dist.all_reduce(st, op=dist.ReduceOp.MAX)
    parity["device_status"] = int(st.item())
    if parity["device_status"]:
        failures.append(f"device status {parity['device_status']:#x} (a bounded wait gave up)")
    bad = torch.tensor([len(failures)], device=dev)
    dist.all_reduce(bad, op=dist.ReduceOp.MAX)
    parity["ok"] = int(bad.item()) == 0
    parity["oracle"] = "CPU oracle on sampled columns of every rank's slice, bf16 rounding-floor gate"

    if not parity["ok"]:
        if rank == 0:
            print(json.dumps({"error": "parity failed at world size %d" % world, "parity": parity,
                              "failures": failures}), flush=True)
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        os._exit(3)

    # ---- the one-GPU anchor: the same layers unsharded on rank 0's GPU, same protocol
    anchor = None
    if not args.no_secondary:
        if rank == 0:
            a_layers, a_copies, _ = h.resident_copies(full_cpu)
            a_outs = [torch.empty((L.M, L.N), dtype=L.x.dtype, device=dev) for L in full_cpu]

            def a_step(i):
                for j, L in enumerate(a_layers[i % a_copies]):
                    _C.dequant_matmul(L.x, L.wq, L.scales, L.zeros, L.group_size, L.quant_type, out=a_outs[j])

            for i in range(3):
                a_step(i)
            torch.cuda.synchronize()
            anchor, _, _ = h.time_graph(a_step, min(args.steps, 100))
            del a_layers, a_outs
            h.last_graph = None
            torch.cuda.empty_cache()
        t = torch.tensor([anchor or 0.0], device=dev, dtype=torch.float64)
        dist.broadcast(t, src=0)
        anchor = float(t.item())
    del full_cpu

    # ---- timed region
    for i in range(max(3, args.warmup)):
        step(i)
    torch.cuda.synchronize()
    ms, replays, region = h.time_graph(step, args.steps, collective=True)
    graph = h.last_graph
    total_wbytes = wbytes_rank * world
    metric, unit = metric_of(name)
    value = total_wbytes / (ms * 1e-3) / 1e9

    # ---- compute only: this rank's kernels without the gather (max over ranks)
    def compute_step(i):
        for j, L in enumerate(dev_layers[i % copies]):
            _C.dequant_matmul(L.x, L.wq, L.scales, L.zeros, L.group_size, L.quant_type, out=outs[j])

    comp_ms, _, _ = h.time_graph(compute_step, min(args.steps, 100))
    comp_ms = h.max_over_ranks(comp_ms)

    # ---- roofline: the dominant projection's kernel alone on this rank (no gather)
    dom = max(range(len(layers_cpu)), key=lambda j: layers_cpu[j].weight_bytes)
    Ld = layers_cpu[dom]

    def dom_step(i):
        L = dev_layers[i % copies][dom]
        _C.dequant_matmul(L.x, L.wq, L.scales, L.zeros, L.group_size, L.quant_type, out=outs[dom])

    dom_ms, _, _ = h.time_graph(dom_step, min(args.steps, 100))
    dom_us = h.max_over_ranks(dom_ms) * 1e3
    pk = h.peaks
    achieved = Ld.total_bytes / (dom_us * 1e-6) / 1e9
    roofline = {"bound": "hbm", "kernel": f"gemv ({Ld.name}, per-GPU shard, without the gather)", "achieved": achieved,
                "peak": pk["hbm"], "peak_source": f"{pk['kind']} HBM copy bandwidth", "unit": "GB/s",
                "frac": achieved / pk["hbm"], "frac_of_nominal_8TBs": achieved / 8000.0, "traffic": None,
                "algorithmic_bytes_per_launch": Ld.total_bytes, "weight_bytes_per_launch": Ld.weight_bytes,
                "us_per_launch": dom_us}

    # ---- end to end: host activations in, gathered result back to the host, every step
    xs_host = [L.x.pin_memory() for L in layers_cpu]
    outs_host = [torch.empty((L.M, L.N * world), dtype=L.x.dtype).pin_memory() for L in layers_cpu]
    xs_dev = [torch.empty_like(L.x, device=dev) for L in layers_cpu]

    def host_step(c):
        def body():
            for j, L in enumerate(dev_layers[c]):
                xs_dev[j].copy_(xs_host[j], non_blocking=True)
                outs_host[j].copy_(run_layer(j, L, xs_dev[j]), non_blocking=True)
        return body

    # a decode step is recorded once per weight copy and replayed with one launch (every rank
    # records and replays the same sequence)
    import metal_native
    pipe = metal_native.PhasePipeline()
    phase = pipe.auto_detect_phase(batch_size=layers_cpu[0].M, seq_len=1 if layers_cpu[0].M <= 32 else layers_cpu[0].M)
    issue = [pipe.capture_step(host_step(c)) for c in range(copies)]

    def e2e_step(i):
        issue[i % copies]()
        torch.cuda.current_stream().synchronize()

    e2e_steps = min(max(args.steps, 50), 400)
    for i in range(5):
        e2e_step(i)
    h.barrier()
    t0 = time.perf_counter()
    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    c0.record()
    for i in range(e2e_steps):
        e2e_step(i)
    c1.record()
    torch.cuda.synchronize()
    e2e_ms = h.max_over_ranks(max(c0.elapsed_time(c1), (time.perf_counter() - t0) * 1e3))
    e2e = {"value": total_wbytes * e2e_steps / (e2e_ms * 1e-3) / 1e9, "unit": unit,
           "h2d_bytes_per_step": sum(x.numel() * x.element_size() for x in xs_host),
           "d2h_bytes_per_step": sum(o.numel() * o.element_size() for o in outs_host),
           "ms_per_step": e2e_ms / e2e_steps, "steps": e2e_steps,
           "call": ("metal_native.sharded.PeerGather.matmul" if fused else
                    "metal_native._C.dequant_matmul + sharded.GatherBuffer.all_gather")
           + " per projection between copies from and to pinned host memory, on every rank, issued through "
             f"metal_native.PhasePipeline.capture_step ({phase.name}), stream synchronised every step; weights resident"}

    # ---- keep the load on for the clock sampler: every rank replays the same number of times
    for _ in range(max(1, min(2000, int(1000.0 / max(ms * args.steps, 1e-3))))):
        graph.replay()
    torch.cuda.synchronize()
    clocks = sampler.stop() if sampler else None

    if rank == 0:
        config = {"workload": name, "description": describe(name), "weight_copies": copies,
                  "l2_policy": f"inputs larger than L2: {copies} weight copies x {wbytes_rank / 1e6:.1f} MB per rank "
                               f"rotate, L2 = {h.l2 / 1e6:.0f} MB",
                  "launch": f"{args.steps} steps captured in one CUDA graph per rank; {replays} replays timed with CUDA "
                            f"events between barriers ({region:.1f} ms region), median replay / {args.steps}, max over ranks",
                  "weights_immutable": True, "collective": collective, "weight_bytes_per_step": total_wbytes,
                  "frac_of_measured_hbm": value / (pk["hbm"] * world),
                  "frac_of_nominal_8TBs": value / (8000.0 * world),
                  "compute_only_ms_per_step": comp_ms, "gather_ms_per_step": ms - comp_ms}
        if anchor:
            config["scale_anchor"] = {"workload": name, "n1_ms_per_step": anchor,
                                      "n1_value": total_wbytes / (anchor * 1e-3) / 1e9, "unit": unit,
                                      "speedup": anchor / ms, "efficiency": anchor / ms / world,
                                      "note": "the same layers, unsharded, on rank 0's GPU in this run; this is the "
                                              "scaling curve to read (the job's N=1 default is another workload)"}
        line = {"metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps,
                "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config, "parity": parity,
                "roofline": roofline, "cpu_baseline": None, "e2e": e2e, "clocks": clocks,
                "gpu_launches": sum(launches_of(_C, L, fused is not None) for L in layers_cpu) * args.steps * (replays + 2)}
        print(json.dumps(line), flush=True)
    # Leave together, with nothing in flight.  The process group is not torn down explicitly:
    # destroying it while captured graphs still reference its communicator was seen to block,
    # and the processes are about to exit anyway.
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
        return
    h = Harness(args)
    if h.world > 1:
        run_sharded(h, args)
    else:
        run_single(h, args)


if __name__ == "__main__":
    main()
