#!/usr/bin/env python
"""Benchmark of the dense-contraction path: bf16 GEMM TFLOP/s at M = N = K = 8192 (fused bias + ReLU).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--size S] [--layout NN|NT|TN]

One step is one pass of the hot path over one batch of synthetic input: one 8192 x 8192 x 8192 product
with N(0,1) bf16 operands, f32 accumulation, y = relu(A*B + bias) stored as bf16.  With --gpus N every rank
runs an independent replica on its own GPU (the GEMM sweep does not shard; no collective on the data
path), the timed region is bracketed by a barrier and a device synchronise, and the time is the maximum over
ranks.  Rank 0 prints ONE JSON line.

  value     whole-job TFLOP/s with operands resident in HBM (CUDA events around exactly K steps)
  e2e       the same metric through the public `Gpu.upload` / `Gpu.matmul` / `Gpu.download` calls with
            pinned HOST buffers: both operands go host->device and the result device->host every step
  roofline  tensor bound: 2*M*N*K per launch / mean launch time, against the measured cuBLAS bf16 peak
  cpu_baseline  the CPU oracle (restatement of grad's `matmulTiled`) on a bounded row slice, rank 0, N = 1
  --impl reference  times that CPU path alone (the reference is Zig and cannot be built here)
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "bf16 GEMM TFLOP/s (M=N=K=8192, fused bias+ReLU)"
UNIT = "TFLOP/s"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--size", type=int, default=8192)
    ap.add_argument("--layout", default="NN", choices=["NN", "NT", "TN"])
    ap.add_argument("--e2e-steps", type=int, default=8)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-resnet", action="store_true", help="skip the ResNet-14 inference and convolution-layer parts (small profiler captures)")
    ap.add_argument("--profile-resnet", type=int, default=0, metavar="BATCH",
                    help="run only three eager ResNet-14 inference passes at this batch and exit (launch lists under a profiler)")
    ap.add_argument("--profile-conv", default="", metavar="N,H,W,C,K,COUT,STRIDE,PAD",
                    help="run only six forward launches of this bf16 convolution layer (bias + ReLU fused) and exit")
    return ap.parse_args()


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nvml = pynvml
            self.dev = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.dev, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nvml = None

    def _run(self):
        n = self.nvml
        names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20,
                 "hw_power_brake_slowdown": 0x80}
        while not self._stop.is_set():
            try:
                self.samples.append(n.nvmlDeviceGetClockInfo(self.dev, n.NVML_CLOCK_SM))
                try:
                    mask = n.nvmlDeviceGetCurrentClocksEventReasons(self.dev)
                except Exception:
                    mask = n.nvmlDeviceGetCurrentClocksThrottleReasons(self.dev)
                for name, bit in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.005)

    def start(self):
        if self.nvml is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def cpu_sample(size: int, rows: int, reps: int):
    """Times the CPU oracle on `rows` rows of the size^3 product (same N, K, same fused epilogue); TFLOP/s."""
    import numpy as np
    from oracle import binding as orc

    rng = np.random.default_rng(1235)
    a = orc.bf16_round(rng.standard_normal((rows, size), dtype=np.float32))
    b = orc.bf16_round(rng.standard_normal((size, size), dtype=np.float32))
    bias = rng.standard_normal(size, dtype=np.float32)
    threads = orc.host_threads()
    best = float("inf")
    for _ in range(reps):
        t0 = time.perf_counter()
        out = orc.matmul_tiled(a, b, rows, size, size, threads=threads)
        out = orc.bias_act(out, bias, True)
        best = min(best, time.perf_counter() - t0)
    flops = 2.0 * rows * size * size
    return flops / best / 1e12, min(threads, 16), best


def run_reference(args):
    """The reference arm: grad's own CPU implementation of the path (its Zig cannot be built here, so the C++
    restatement in oracle/ stands in), every host thread it can use, bounded sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    size = args.size
    rows = 512 if size >= 4096 else min(size, 1024)
    steps = max(1, min(args.steps, 5))
    warmup = max(1, min(args.warmup, 1))
    cpu_sample(size, rows, warmup)
    t0 = time.perf_counter()
    value, cores, _ = cpu_sample(size, rows, steps)
    total = time.perf_counter() - t0
    sample = f"{rows} of {size} rows of A per step (N=K={size}), best of {steps} steps; oracle port of grad's matmulTiled"
    line = {"impl": "reference", "metric": METRIC, "value": round(value, 4), "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
            "warmup": warmup, "ms_per_step": round(total / steps * 1e3, 2), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32 (bf16-rounded operands)", "data": "synthetic",
            "config": {"workload": f"GEMM sweep M=N=K={size} NN + bias + ReLU, CPU tiled matmul", "sample": sample},
            "cpu_baseline": {"value": round(value, 4), "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": round(value, 4), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def resnet_inference(gpu, rank, world, dist, torch):
    """Second half of the metric: ONNX-executor inference of ResNet-14 64-192-384 (batch norm folded), bf16,
    images/s.  The batch is split across the GPUs (rank r runs images [B*r/N, B*(r+1)/N), full weight replica,
    no collective); time is the maximum over ranks.  `value` replays a captured run on device-resident
    inputs; `e2e` copies the rank's images from pinned host memory and brings its logits back every step."""
    from grad_b200.onnx_gpu import Executor, resnet14_model
    from grad_b200.replicas import shard

    model = resnet14_model(64, 192, 384)
    out = {"unit": "images/s", "model": "ResNet-14 64-192-384, 3x32x32 inputs N(0,1), He-normal weights, bf16 activations",
           "gflop_per_image": 1.482, "scaling": "strong (batch sharded)"}
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed(fn, iters):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / iters
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    for batch, iters in ((4096, 10), (100, 50)):
        lo, hi = shard(batch, world, rank)
        if hi - lo == 0:
            continue
        gen = torch.Generator(device="cuda").manual_seed(1234 + 3)
        x = torch.randn((batch, 3072), generator=gen, device="cuda")[lo:hi].contiguous()
        ex = Executor(model, gpu, "bf16")
        ex.capture({"input": x})
        ms = timed(lambda: ex.replay({"input": x}), iters)
        hx = x.cpu().pin_memory()
        hlogits = torch.empty((hi - lo, 10), dtype=torch.float32).pin_memory()

        def e2e():
            hlogits.copy_(ex.replay({"input": hx})["logits"], non_blocking=True)

        ms_e2e = timed(e2e, iters)
        out[f"batch_{batch}"] = {"value": round(batch / ms * 1e3, 1), "ms": round(ms, 4), "tflops": round(batch * 1.482e9 / ms / 1e9, 1),
                                 "e2e": round(batch / ms_e2e * 1e3, 1), "launches_per_run": 21, "per_gpu_batch": hi - lo}
    return out


def conv_layers(gpu, torch):
    """Kernel times of the ResNet-14 convolution layers at batch 128 (bf16 storage, f32 accumulation), all three
    passes, each taken from the replay of a CUDA graph of 20 launches so that host cost does not enter."""
    from grad_b200 import Epilogue, conv_geometry

    def graph_ms(fn, calls=20, reps=5):
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for _ in range(calls):
                    fn()
            graph.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                graph.replay()
            e1.record()
            torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (reps * calls)

    n = 128
    layers = (("64->64 3x3 @32", 32, 64, 3, 64, 1), ("64->192 3x3 s2 @32", 32, 64, 3, 192, 2), ("192->192 3x3 @16", 16, 192, 3, 192, 1),
              ("192->384 3x3 s2 @16", 16, 192, 3, 384, 2), ("384->384 3x3 @8", 8, 384, 3, 384, 1), ("64->192 1x1 s2 @32", 32, 64, 1, 192, 2))
    gen = torch.Generator(device="cuda").manual_seed(1234 + 2)
    rows = []
    for name, hw, c, k, co, stride in layers:
        geo = conv_geometry(n, hw, hw, c, k, co, stride, k // 2)
        x = torch.randn((n, hw, hw, c), generator=gen, device="cuda").bfloat16()
        w = (torch.randn((k * k * c, co), generator=gen, device="cuda") * (2.0 / (k * k * c)) ** 0.5).bfloat16()
        dy = torch.randn((n, geo.out_h, geo.out_w, co), generator=gen, device="cuda").bfloat16()
        y, dx = torch.empty_like(dy), torch.empty_like(x)
        dw = torch.zeros((k * k * c, co), device="cuda")
        bias = torch.randn(co, generator=gen, device="cuda")
        flop = 2.0 * geo.positions * k * k * c * co
        row = {"layer": name, "batch": n, "gflop": round(flop / 1e9, 2)}
        for key, fn in (("fprop", lambda: gpu.convForward(x, w, y, geo, epilogue=Epilogue(bias, None, True))),
                        ("dgrad", lambda: gpu.convInputGrad(dy, w, dx, geo)), ("wgrad", lambda: gpu.convWeightGrad(dy, x, dw, geo))):
            ms = graph_ms(fn)
            row[key] = {"us": round(ms * 1e3, 1), "tflops": round(flop / ms / 1e9, 1)}
        rows.append(row)
    return rows


def profile_only(args, gpu, torch):
    """Small fixed workloads for profiler captures; nothing is timed or printed as a bench line."""
    from grad_b200 import Epilogue, conv_geometry

    if args.profile_resnet:
        from grad_b200.onnx_gpu import Executor, resnet14_model

        ex = Executor(resnet14_model(64, 192, 384), gpu, "bf16")
        x = torch.randn((args.profile_resnet, 3072), device="cuda")
        for _ in range(3):
            ex.run_device({"input": x})
    else:
        n, h, w_, c, k, co, stride, pad = (int(v) for v in args.profile_conv.split(","))
        geo = conv_geometry(n, h, w_, c, k, co, stride, pad)
        x = torch.randn((n, h, w_, c), device="cuda").bfloat16()
        w = (torch.randn((k * k * c, co), device="cuda") * (2.0 / (k * k * c)) ** 0.5).bfloat16()
        y = torch.empty((n, geo.out_h, geo.out_w, co), dtype=torch.bfloat16, device="cuda")
        bias = torch.randn(co, device="cuda")
        for _ in range(6):
            gpu.convForward(x, w, y, geo, epilogue=Epilogue(bias, None, True))
    torch.cuda.synchronize()
    gpu.check_status()
    print(json.dumps({"profile_only": True, "plan": gpu.last_plan()}), flush=True)


def run_ours(args):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    import grad_b200
    from grad_b200 import Epilogue, MatmulOpts, MatmulShape

    gpu = grad_b200.Gpu(local)
    if args.profile_resnet or args.profile_conv:
        if rank == 0:
            profile_only(args, gpu, torch)
        return
    size = args.size
    m = n = k = size
    ta, tb = args.layout == "TN", args.layout == "NT"
    gen = torch.Generator(device="cuda").manual_seed(1234 + 1 + rank)   # seed = 1234 + config index (+ rank)
    a = torch.randn((k, m) if ta else (m, k), generator=gen, device="cuda").bfloat16()
    b = torch.randn((n, k) if tb else (k, n), generator=gen, device="cuda").bfloat16()
    bias = torch.randn(n, generator=gen, device="cuda")
    out = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    shape, opts, ep = MatmulShape(m, n, k), MatmulOpts(ta, tb), Epilogue(bias, None, True)

    def step():
        gpu.matmul(a, b, out, shape, opts, epilogue=ep)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    plan = gpu.last_plan()

    sampler = ClockSampler(local)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    launches0 = gpu.launches
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.start()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    if world > 1:
        dist.barrier()
    ms_total = e0.elapsed_time(e1)
    launches = gpu.launches - launches0
    gpu.check_status()
    if world > 1:
        t = torch.tensor([ms_total], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / args.steps
    flops = 2.0 * m * n * k
    value = world * flops / (ms_step * 1e-3) / 1e12

    # ---- end to end: pinned host operands in, host result out, every step ----
    # Three streams and two sets of device buffers, as a host that feeds the library from its own memory would
    # run it: step i's upload, step i-1's product and step i-2's download overlap (PCIe is full duplex), and every
    # step still copies its 268 MB of operands in and its 134 MB of result out inside the timed region.
    ha, hb = a.cpu().pin_memory(), b.cpu().pin_memory()
    hout = torch.empty((m, n), dtype=torch.bfloat16).pin_memory()
    da, db = [torch.empty_like(a) for _ in range(2)], [torch.empty_like(b) for _ in range(2)]
    dout = [torch.empty_like(out) for _ in range(2)]
    s_in, s_run, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_run = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]

    def e2e_step(i):
        s = i & 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_run[s])          # the product that last read this operand pair has finished
            gpu.upload(da[s], ha)
            gpu.upload(db[s], hb)
            ev_in[s].record(s_in)
        with torch.cuda.stream(s_run):
            s_run.wait_event(ev_in[s])
            s_run.wait_event(ev_out[s])         # the download that last read this result buffer has finished
            gpu.matmul(da[s], db[s], dout[s], shape, opts, epilogue=ep)
            ev_run[s].record(s_run)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_run[s])
            gpu.download(hout, dout[s])
            ev_out[s].record(s_out)

    def e2e_run(steps):
        for i in range(steps):
            e2e_step(i)
        for st in (s_in, s_run, s_out):
            torch.cuda.current_stream().wait_stream(st)

    e2e_run(2)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0.record()
    for st in (s_in, s_run, s_out):
        st.wait_event(e0)
    e2e_run(args.e2e_steps)
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([e2e_ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = world * flops / (e2e_ms / args.e2e_steps * 1e-3) / 1e12
    h2d = ha.numel() * 2 + hb.numel() * 2
    d2h = hout.numel() * 2

    resnet = None if args.no_resnet else resnet_inference(gpu, rank, world, dist, torch)
    convs = conv_layers(gpu, torch) if (rank == 0 and not args.no_resnet) else None

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks, peak_kind = measured_peaks()
    timed_s = ms_total * 1e-3
    sustained = timed_s > 1.0
    peak = peaks["bf16_tflops_sustained"] if sustained else peaks["bf16_tflops"]
    achieved = flops / (ms_step * 1e-3) / 1e12   # per launch on one GPU (max over ranks)
    traffic = None
    tpath = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(tpath):
        with open(tpath) as f:
            traffic = json.load(f).get(f"gemm_bf16_{size}_{args.layout}")
    line = {
        "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"GEMM sweep M=N=K={size} {args.layout}, N(0,1) bf16 operands, f32 accumulate, fused bias+ReLU, bf16 out",
                   "parallelism": f"replicas x{world} (no collective on the data path)",
                   "l2": "operands + result = %d MB per step, larger than the 126 MB L2" % ((a.numel() + b.numel() + out.numel()) * 2 // 2**20),
                   "tile": f"{plan['tile_m']}x{plan['tile_n']}", "stages": plan["stages"], "splits": plan["splits"]},
        "clocks": clocks,
        "e2e": {"value": round(e2e_value, 2), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": round(e2e_ms / args.e2e_steps, 3)},
        "gpu_launches": launches,
        "roofline": {"bound": "tensor", "achieved": round(achieved, 2), "peak": peak, "unit": UNIT, "frac": round(achieved / peak, 4),
                     "traffic": traffic, "peak_source": f"{peak_kind} cuBLAS bf16 {'sustained' if sustained else 'burst'}",
                     "frac_of_nominal_2250": round(achieved / 2250.0, 4),
                     "frac_of_measured_sustained": round(achieved / peaks["bf16_tflops_sustained"], 4)},
    }
    if resnet is not None:
        line["resnet14_inference"] = resnet
        line["conv_layers"] = convs
    if world == 1 and not args.no_cpu_baseline:
        rows = 4096 if size >= 4096 else size
        cpu_value, cores, secs = cpu_sample(size, rows, 2)
        line["cpu_baseline"] = {"value": round(cpu_value, 4), "unit": UNIT, "cores": cores, "kind": "port",
                                "sample": f"{rows} of {size} rows of A (N=K={size}), best of 2, {secs:.1f} s each; "
                                          "C++ restatement of grad's matmulTiled + bias + ReLU"}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
