#!/usr/bin/env python
"""Benchmark of the fused INT4/INT8 dequantise + matmul operator on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one pass of the operator over every projection of the workload (for the
default workload: the Qwen2.5-7B decode MLP, fused gate+up GEMV then down GEMV, int4
group 128, M=1).  Inputs are seeded synthetic tensors with the model's shapes.

  value   weight GB/s with everything resident in HBM: (packed weights + scales + zeros
          read per step) x steps / device time, CUDA events around exactly K steps.  The
          K steps are replayed from one CUDA graph so that the device, not the Python
          launch loop, sets the pace; each step reads a different copy of the weights
          (copies x bytes > 2 x L2), so no step finds its weights in L2.
  e2e     the same metric through the public call, metal_native._C.dequant_matmul, with
          the activations in pinned host memory: every step copies them to the device,
          runs the operator and copies the result back to pinned host memory, then
          waits.  Weights stay resident (they are model state, loaded once).
  roofline  the dominant kernel (the largest projection's GEMV) timed alone with CUDA
          events, algorithmic bytes / duration against the measured HBM copy peak.
  cpu_baseline  the reference's CPU dequantise-then-matmul path (the oracle port of
          tests/cpp/test_dequant_matmul.mm:119-213) on the host cores, same workload.

With --gpus N > 1 (launched by torch.distributed.run, one rank per GPU) the workload is
the Llama-3-70B int8 per-channel layers column-sharded over N, each step ending in an
all-gather of the output slices; the value is the whole-job aggregate.

--impl reference times the CPU path only (rank 0), as the reference arm.
"""
from __future__ import annotations

import argparse
import json
import os
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
METRIC = "int4 dequant-GEMV weight GB/s"
UNIT = "GB/s"
PREFILL_METRIC = "prefill TFLOP/s"
FALLBACK_TFLOPS = 1590.0

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the
# ncu captures summarised under profiles/ (one capture per kernel and workload)
TRAFFIC = {
    # dram__bytes_read.sum + dram__bytes_write.sum of one launch, from the ncu captures summarised in
    # profiles/gemv_stream_qwen7b_gate_up.md and profiles/gemm_tcgen05_qwen7b_prefill_up.md
    "qwen7b-decode:qwen2.5-7b.gate_up": 72_224_256 + 705_792,
    "qwen7b-prefill:qwen2.5-7b.up.prefill": 39_830_016 + 378_368,
}


def is_prefill(name):
    return name == "qwen7b-prefill"


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
    ap.add_argument("--gather", default="auto", choices=["auto", "fused", "nccl"],
                    help="N > 1: all-gather inside the decode kernel (peer stores) or NCCL after it")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    return ap.parse_args()


def hbm_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return float(d["hbm_gbs"]), "measured", d
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback", {}


def tensor_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return float(d["bf16_tflops"]), "measured", d.get("bf16_tflops_sustained")
        except Exception:
            pass
    return FALLBACK_TFLOPS, "fallback", None


def workload_name(args, world):
    if args.workload != "auto":
        return args.workload
    return "qwen7b-decode" if world == 1 else "llama70b-int8-m1"


def build_layers(name, world, rank):
    """Returns (layers, description).  CPU tensors; identical on every call."""
    from metal_native import workloads
    if name == "qwen7b-decode":
        return workloads.config1(), "Qwen2.5-7B decode MLP: gate+up [1,3584]x[37888,3584]^T then down [1,18944]x[3584,18944]^T, int4 g128 asym, fp16"
    if name.startswith("llama8b-decode-m"):
        M = int(name.rsplit("m", 1)[1])
        return workloads.config2(M), f"Llama-3-8B batched decode M={M}: K=4096,N=14336 and K=14336,N=4096, int4 g128 sym, bf16"
    if name == "qwen7b-prefill":
        return workloads.config3(), "Qwen2.5-7B prefill M=512: K=3584,N=18944 and K=18944,N=3584, int4 g128 asym, fp16"
    if name.startswith("llama70b-int8-m"):
        M = int(name.rsplit("m", 1)[1])
        return (workloads.config4(M, world_size=world, rank=rank),
                f"Llama-3-70B M={M}: K=8192,N=57344 and K=28672,N=8192, int8 per-channel, bf16, "
                f"column-sharded over {world} GPU(s)")
    raise SystemExit(f"unknown workload {name}")


# --------------------------------------------------------------------------- CPU arm

def cpu_path_time(layers, seconds, max_steps=None):
    """Times the oracle port of the reference CPU path on all host threads.  Returns
    (seconds per step, steps run, threads)."""
    import numpy as np
    from oracle import oracle
    from tests import helpers as H
    threads = oracle.host_threads()
    prepared = []
    for L in layers:
        s = H.f32(L.scales)
        prepared.append((H.f32(L.x), L.wq.contiguous().numpy(), s,
                         H.f32(L.zeros) if L.zeros is not None else None, L.group_size, L.quant_type,
                         np.empty((L.N, L.K), np.float32)))
    times = []
    t_end = time.perf_counter() + seconds
    while True:
        t0 = time.perf_counter()
        for (x, wq, s, z, g, qt, scratch) in prepared:
            oracle.dequant_matmul(x, wq, s, z, g, qt, threads=threads, scratch=scratch)
        times.append(time.perf_counter() - t0)
        if time.perf_counter() >= t_end or (max_steps and len(times) >= max_steps):
            break
    return times, threads


def cpu_sample_layers(layers, budget_macs=4e9):
    """Bounds the CPU work of one step: if a layer needs more than `budget_macs`
    multiply-adds, keep only its first rows n (a contiguous block of output columns) and
    say so.  Throughput in weight GB/s is unaffected by the cut."""
    from metal_native.workloads import Layer
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


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    name = workload_name(args, world)
    layers, desc = build_layers(name, 1, 0)
    sample, notes = cpu_sample_layers(layers)
    prefill = is_prefill(name)
    wbytes = sum(L.weight_bytes for L in sample)
    work = sum(L.flops for L in sample) / 1e3 if prefill else wbytes     # TFLOP = flops / 1e12
    times, threads = cpu_path_time(sample, 1e9, max_steps=args.warmup)          # warm-up steps
    times, threads = cpu_path_time(sample, 1e9, max_steps=max(1, args.steps))   # exactly K steps
    total = sum(times)
    value = work * len(times) / total / 1e9
    sample_desc = "whole workload per step" if not notes else "; ".join(notes)
    line = {
        "impl": "reference", "metric": PREFILL_METRIC if prefill else METRIC, "value": value,
        "unit": "TFLOP/s" if prefill else UNIT, "n_gpus": args.gpus,
        "steps": len(times), "warmup": args.warmup, "ms_per_step": total / len(times) * 1e3,
        "higher_is_better": True, "scaling": "strong" if world > 1 else "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": name, "description": desc, "arm": "CPU oracle port of the reference's "
                   "dequantise-then-matmul helpers (tests/cpp/test_dequant_matmul.mm:119-213), "
                   "N split over host threads"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s" if prefill else UNIT, "cores": threads, "kind": "port",
                         "sample": sample_desc},
        "e2e": {"value": value, "unit": "TFLOP/s" if prefill else UNIT, "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
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

def run_ours(args):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import datetime
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))

    import metal_native
    from metal_native import _C

    name = workload_name(args, world)
    layers_cpu, desc = build_layers(name, world, rank)
    sampler = ClockSampler(local) if rank == 0 else None

    # ---- resident copies of the weights: copies x bytes > 2 x L2 -------------------
    l2 = torch.cuda.get_device_properties(dev).L2_cache_size
    wbytes_rank = sum(L.weight_bytes for L in layers_cpu)
    copies = max(2, -(-2 * l2 // wbytes_rank) + 1)
    copies = min(copies, 16)
    dev_layers = []
    for c in range(copies):
        dev_layers.append([L.to(dev) if c == 0 else
                           type(L)(L.name, L.quant_type, L.M, L.K, L.N, L.group_size, dev_layers[0][i].x,
                                   dev_layers[0][i].wq.clone(), dev_layers[0][i].scales.clone(),
                                   None if L.zeros is None else dev_layers[0][i].zeros.clone())
                           for i, L in enumerate(layers_cpu)])
    outs = [torch.empty((L.M, L.N), dtype=L.x.dtype, device=dev) for L in layers_cpu]
    gathered = None
    fused = None      # per layer: PeerGather when the all-gather runs inside the decode kernel
    collective = None
    if world > 1:
        from metal_native import sharded
        gathered = [sharded.GatherBuffer(L.M, L.N, world, L.x.dtype, dev) for L in layers_cpu]
        want_fused = args.gather != "nccl" and all(
            L.M <= 32 and _C.select_path(L.M, L.N, L.K, L.group_size, L.quant_type, L.x.dtype,
                                         zeros=L.zeros is not None) == "gemv" for L in layers_cpu)
        ok = torch.tensor([1 if want_fused else 0], device=dev)
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

    def run_layer(j, L, x):
        """One projection; returns the full [M, N] result on this rank."""
        if fused is not None:
            return fused[j].matmul(x, L.wq, L.scales, L.zeros, L.group_size, L.quant_type)
        o = _C.dequant_matmul(x, L.wq, L.scales, L.zeros, L.group_size, L.quant_type, out=outs[j])
        return gathered[j].all_gather(o) if world > 1 else o

    def step(i):
        for j, L in enumerate(dev_layers[i % copies]):
            run_layer(j, L, L.x)

    def launches(L):
        # one kernel per projection; with K split, the tensor-core path and the many-token (M > 8)
        # decode path add a reduce kernel
        path = _C.select_path(L.M, L.N, L.K, L.group_size, L.quant_type, L.x.dtype, zeros=L.zeros is not None)
        q = 0 if L.quant_type == "int4" else 1
        split = ((path == "gemm" or (path == "gemv" and L.M > 8 and fused is None)) and
                 _C._lib.mnq_workspace_bytes(L.M, L.N, L.K, int(L.group_size), q) > 0)
        return 2 if split else 1

    kernels_per_step = sum(launches(L) for L in layers_cpu)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- warm-up, graph capture ------------------------------------------------------
    for i in range(max(3, args.warmup)):
        step(i)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        step(0)
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(args.steps):
                step(i)
        graph.replay()     # untimed: uploads the graph
        torch.cuda.synchronize()

        # ---- timed region: exactly K steps ------------------------------------------
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        graph.replay()
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    total_wbytes = wbytes_rank * world
    prefill = is_prefill(name)
    total_flops = sum(L.flops for L in layers_cpu) * world
    work_per_step = total_flops / 1e3 if prefill else total_wbytes      # TFLOP/s = flops / s / 1e12
    value = work_per_step * args.steps / (ms * 1e-3) / 1e9

    # ---- roofline: the dominant kernel alone -------------------------------------------
    dom = max(range(len(layers_cpu)), key=lambda j: (layers_cpu[j].flops if prefill else layers_cpu[j].weight_bytes))
    Ld = layers_cpu[dom]
    reps = max(50, min(args.steps, 400))
    g2 = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(g2, stream=stream):
            for i in range(reps):
                L = dev_layers[i % copies][dom]
                _C.dequant_matmul(L.x, L.wq, L.scales, L.zeros, L.group_size, L.quant_type, out=outs[dom])
        g2.replay()
        torch.cuda.synchronize()
        k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        k0.record(stream)
        g2.replay()
        k1.record(stream)
        torch.cuda.synchronize()
        dom_us = k0.elapsed_time(k1) * 1e3 / reps
    peak, peak_kind, peaks = hbm_peak()
    algo_bytes = Ld.total_bytes
    traffic = TRAFFIC.get(f"{name}:{Ld.name}")
    kernel = _C.select_path(Ld.M, Ld.N, Ld.K, Ld.group_size, Ld.quant_type, Ld.x.dtype, zeros=Ld.zeros is not None)
    if prefill:
        tpeak, tkind, tsust = tensor_peak()
        achieved = Ld.flops / (dom_us * 1e-6) / 1e12
        roofline = {"bound": "tensor", "kernel": f"{kernel} ({Ld.name})", "achieved": achieved, "peak": tpeak,
                    "peak_source": f"{tkind} cuBLAS bf16 burst", "unit": "TFLOP/s", "frac": achieved / tpeak,
                    "frac_of_nominal_2250TF": achieved / 2250.0, "traffic": traffic,
                    "flops_per_launch": Ld.flops, "us_per_launch": dom_us}
        if tsust:   # the kernel is timed back to back for thousands of launches, i.e. under the power cap
            roofline["peak_sustained"] = float(tsust)
            roofline["frac_of_sustained"] = achieved / float(tsust)
    else:
        achieved = algo_bytes / (dom_us * 1e-6) / 1e9
        roofline = {"bound": "hbm", "kernel": f"{kernel} ({Ld.name})", "achieved": achieved, "peak": peak,
                    "peak_source": f"{peak_kind} HBM copy bandwidth", "unit": "GB/s", "frac": achieved / peak,
                    "frac_of_nominal_8TBs": achieved / 8000.0, "traffic": traffic,
                    "algorithmic_bytes_per_launch": algo_bytes, "weight_bytes_per_launch": Ld.weight_bytes,
                    "weight_GBps": Ld.weight_bytes / (dom_us * 1e-6) / 1e9, "us_per_launch": dom_us}

    # ---- end to end through the public call, host buffers ------------------------------
    xs_host = [L.x.pin_memory() for L in layers_cpu]
    full_N = [L.N * (world if world > 1 else 1) for L in layers_cpu]
    outs_host = [torch.empty((L.M, n), dtype=L.x.dtype).pin_memory() for L, n in zip(layers_cpu, full_N)]
    xs_dev = [torch.empty_like(L.x, device=dev) for L in layers_cpu]

    def e2e_step(i):
        for j, L in enumerate(dev_layers[i % copies]):
            if world == 1:
                # host activations in, host result out: the operator enqueues both copies itself
                _C.dequant_matmul(xs_host[j], L.wq, L.scales, L.zeros, L.group_size, L.quant_type, out=outs_host[j])
            else:
                xs_dev[j].copy_(xs_host[j], non_blocking=True)
                o = run_layer(j, L, xs_dev[j])
                outs_host[j].copy_(o, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    e2e_steps = min(args.steps, 400)
    for i in range(5):
        e2e_step(i)
    barrier()
    t0 = time.perf_counter()
    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    c0.record()
    for i in range(e2e_steps):
        e2e_step(i)
    c1.record()
    torch.cuda.synchronize()
    e2e_ms = max(c0.elapsed_time(c1), (time.perf_counter() - t0) * 1e3)
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e = {"value": work_per_step * e2e_steps / (e2e_ms * 1e-3) / 1e9, "unit": "TFLOP/s" if prefill else UNIT,
           "h2d_bytes_per_step": sum(x.numel() * x.element_size() for x in xs_host),
           "d2h_bytes_per_step": sum(o.numel() * o.element_size() for o in outs_host),
           "ms_per_step": e2e_ms / e2e_steps, "steps": e2e_steps,
           "call": ("metal_native.sharded.PeerGather.matmul per projection between torch copies, eager; weights resident"
                    if fused else
                    "metal_native._C.dequant_matmul(host activations, out=host tensor) per projection, eager: the "
                    "operator enqueues the host->device and device->host copies; weights resident" if world == 1 else
                    "metal_native._C.dequant_matmul per projection between torch copies, eager; weights resident")}

    # ---- keep the load on for the clock sampler, then read it ----------------------------
    # every rank replays the same number of times (the graph may hold collectives): about one
    # second of load, counted from the all-reduced step time, never from a local clock
    for _ in range(max(1, min(2000, int(1000.0 / max(ms, 1e-3))))):
        graph.replay()
    torch.cuda.synchronize()
    clocks = sampler.stop() if sampler else None

    # ---- CPU baseline (rank 0, N=1 only) -----------------------------------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        sample, notes = cpu_sample_layers(layers_cpu)
        times, threads = cpu_path_time(sample, args.cpu_seconds)
        best = sorted(times)[len(times) // 2]
        cpu_work = sum(L.flops for L in sample) / 1e3 if prefill else sum(L.weight_bytes for L in sample)
        cpu = {"value": cpu_work / best / 1e9, "unit": "TFLOP/s" if prefill else UNIT, "cores": threads,
               "kind": "port", "ms_per_step": best * 1e3,
               "sample": (f"{len(times)} whole steps" if not notes else f"{len(times)} steps of: " + "; ".join(notes))
               + f", median, {threads} threads splitting N"}

    if rank == 0:
        line = {
            "metric": PREFILL_METRIC if prefill else METRIC, "value": value,
            "unit": "TFLOP/s" if prefill else UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "strong" if world > 1 else "weak", "vs_baseline": None,
            "dtype": "f16" if layers_cpu[0].x.dtype == torch.float16 else "bf16", "data": "synthetic",
            "config": {"workload": name, "description": desc, "weight_copies": copies,
                       "l2_policy": f"inputs larger than L2: {copies} weight copies x {wbytes_rank / 1e6:.1f} MB "
                                    f"rotate, L2 = {l2 / 1e6:.0f} MB",
                       "launch": f"{args.steps} steps replayed from one CUDA graph",
                       "collective": collective,
                       "weight_bytes_per_step": total_wbytes,
                       "frac_of_measured_hbm": None if prefill else value / (peak * world),
                       "frac_of_nominal_8TBs": None if prefill else value / (8000.0 * world)},
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "clocks": clocks,
            "gpu_launches": kernels_per_step * args.steps,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        # Leave together, with nothing in flight.  The process group is not torn down
        # explicitly: destroying it while captured graphs still reference its communicator
        # was seen to block, and the processes are about to exit anyway.
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
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
