#!/usr/bin/env python
"""Benchmark of the dense-contraction path: bf16 GEMM TFLOP/s at M = N = K = 8192 (fused bias + ReLU).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--size S] [--layout NN|NT|TN]
                    [--legs gemm,sustained,e2e,sweep,resnet,conv,mlp,transformer]

One step is one pass of the hot path over one batch of synthetic input: one 8192 x 8192 x 8192 product
with N(0,1) bf16 operands, f32 accumulation, y = relu(A*B + bias) stored as bf16.  With --gpus N every rank
runs an independent replica on its own GPU (the GEMM sweep does not shard; no collective on the data
path), the timed region is bracketed by a barrier and a device synchronise, and the time is the maximum over
ranks.  Rank 0 prints ONE JSON line.

  value     whole-job TFLOP/s with operands resident in HBM (CUDA events around exactly K steps)
  e2e       the same metric through the public `Gpu.upload` / `Gpu.matmul` / `Gpu.download` calls with
            pinned HOST buffers: both operands go host->device and the result device->host every step
  roofline  tensor bound: 2*M*N*K per launch / mean launch time, against the measured cuBLAS bf16 peak
  parity    rows of the timed product recomputed by the CPU oracle on the same operands
  sustained the same launch back to back for seconds: best / median TFLOP/s and the SM clocks seen
  cpu_baseline  the CPU oracle (restatement of grad's `matmulTiled`) on a bounded row slice, rank 0, N = 1
  --impl reference  times that CPU path alone (the reference is Zig and cannot be built here)

Further keys carry the other benchmark configurations, each figure beside the CPU path timed in the same run:
  gemm_sweep          M = N = K in {1024, 2048, 4096, 8192} and the skinny 128 x 4096 x 4096, NN / NT / TN, in bf16, TF32
                      and strict f32, fused bias + ReLU: microseconds and TFLOP/s per product from CUDA-graph replays
  resnet14_inference  ONNX-executor inference of ResNet-14 64-192-384, batch 4096 and 100, sharded over the ranks
  conv_layers         every convolution layer of the ResNet-14 64-128-256 stack (and the 64-192-384 widths) at batch
                      128, forward / input gradient / weight gradient, with roofline fractions and HBM GB/s
  mlp_step            the six GEMMs of one MLP 784-128-10 training step (f32, batch 64) as one captured step
  transformer_step    the contractions of one character-Transformer training step (bf16) and the gradient mean over
                      the ranks (one NCCL allreduce of the flat 3 228 737-float gradient vector)
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
NOMINAL_BF16, NOMINAL_TF32, NOMINAL_HBM = 2250.0, 1125.0, 8000.0
ALL_LEGS = ("gemm", "sustained", "e2e", "sweep", "resnet", "conv", "mlp", "transformer")


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--size", type=int, default=8192)
    ap.add_argument("--layout", default="NN", choices=["NN", "NT", "TN"])
    ap.add_argument("--e2e-steps", type=int, default=8)
    ap.add_argument("--sustained-seconds", type=float, default=3.0)
    ap.add_argument("--legs", default=",".join(ALL_LEGS), help="comma-separated subset of: " + ", ".join(ALL_LEGS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-resnet", action="store_true", help="skip every leg but the GEMM itself (small profiler captures)")
    ap.add_argument("--profile-resnet", type=int, default=0, metavar="BATCH",
                    help="run only three eager ResNet-14 inference passes at this batch and exit (launch lists under a profiler)")
    ap.add_argument("--profile-conv", default="", metavar="N,H,W,C,K,COUT,STRIDE,PAD[,PASS]",
                    help="run only six launches of this bf16 convolution layer (PASS fprop|dgrad|wgrad|stats|affine|wgrad_affine|dx_stats, default fprop) and exit")
    ap.add_argument("--profile-gemm", default="", metavar="M,N,K,LAYOUT,MATH", help="run only six launches of this product and exit")
    return ap.parse_args()


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


def nvml_handle(torch, index: int):
    """NVML handle of CUDA device `index` (matched by UUID: CUDA_VISIBLE_DEVICES may renumber the devices)."""
    import pynvml

    pynvml.nvmlInit()
    try:
        uuid = str(torch.cuda.get_device_properties(index).uuid)
        return pynvml, pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid if not uuid.startswith("GPU-") else uuid).encode())
    except Exception:
        return pynvml, pynvml.nvmlDeviceGetHandleByIndex(index)


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while a timed region runs (one sample per millisecond)."""

    def __init__(self, torch, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            self.nvml, self.dev = nvml_handle(torch, index)
            self.max_mhz = self.nvml.nvmlDeviceGetMaxClockInfo(self.dev, self.nvml.NVML_CLOCK_SM)
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
            time.sleep(0.001)

    def start(self):
        if self.nvml is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
        s = self.samples
        out = {"sm_mhz": statistics.median(s) if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(s)}
        if len(s) >= 8:
            q = sorted(s)
            out["sm_mhz_p10_p90"] = [q[len(q) // 10], q[len(q) * 9 // 10]]
        return out


def pin_to_gpu_numa_node(torch, index: int) -> str:
    """Moves this process onto the CPUs NVML names as local to the GPU before any pinned host buffer is allocated
    (pinned pages are placed on the allocating thread's node), so that with several ranks each one's host copies
    cross its own socket's PCIe root instead of all of them sharing node 0."""
    try:
        nvml, dev = nvml_handle(torch, index)
        words = (os.cpu_count() + 63) // 64
        mask = nvml.nvmlDeviceGetCpuAffinity(dev, words)
        ideal = {w * 64 + b for w, word in enumerate(mask) for b in range(64) if (int(word) >> b) & 1}
        allowed = os.sched_getaffinity(0)
        both = ideal & allowed
        if not both:
            return f"GPU-local CPUs are outside this process's cpuset ({len(allowed)} CPUs allowed): left unpinned"
        os.sched_setaffinity(0, both)
        node = "?"
        try:
            node = str(nvml.nvmlDeviceGetNumaNodeId(dev))
        except Exception:
            pass
        return f"pinned to {len(both)} GPU-local CPUs of {len(allowed)} allowed (NUMA node {node})"
    except Exception as exc:   # no NVML, or a kernel without affinity support
        return f"unpinned ({type(exc).__name__})"


def cpu_rows(a_rows, b, bias, ta, tb, reps: int):
    """The CPU oracle on the stored operands (`a_rows` = the sampled rows of A, or columns when A is stored (K, M));
    returns (result rows, TFLOP/s, threads, seconds of the best repetition)."""
    from oracle import binding as orc

    rows = a_rows.shape[1] if ta else a_rows.shape[0]
    k = a_rows.shape[0] if ta else a_rows.shape[1]
    n = b.shape[0] if tb else b.shape[1]
    threads = orc.host_threads()
    best, out = float("inf"), None
    for _ in range(reps):
        t0 = time.perf_counter()
        out = orc.matmul_tiled(a_rows, b, rows, k, n, ta, tb, threads=threads)
        out = orc.bias_act(out, bias, True)
        best = min(best, time.perf_counter() - t0)
    return out, 2.0 * rows * n * k / best / 1e12, min(threads, 16), best


def cpu_sample(size: int, rows: int, reps: int):
    """Times the CPU oracle on `rows` rows of the size^3 product (same N, K, same fused epilogue); TFLOP/s."""
    import numpy as np
    from oracle import binding as orc

    rng = np.random.default_rng(1235)
    a = orc.bf16_round(rng.standard_normal((rows, size), dtype=np.float32))
    b = orc.bf16_round(rng.standard_normal((size, size), dtype=np.float32))
    bias = rng.standard_normal(size, dtype=np.float32)
    _, value, cores, best = cpu_rows(a, b, bias, False, False, reps)
    return value, cores, best


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


# ---- shared timing helpers -------------------------------------------------------------------------------------
def graph_ms(torch, fn, calls=20, reps=5):
    """Mean device time of one `fn()` from the replay of a CUDA graph of `calls` of them (host cost does not enter)."""
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


def max_over_ranks(torch, dist, world, ms):
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


# ---- config 4: ONNX-executor inference -------------------------------------------------------------------------
def resnet_inference(gpu, rank, world, dist, torch, cpu_baseline):
    """Second half of the metric: ONNX-executor inference of ResNet-14 64-192-384 (batch norm folded), bf16,
    images/s.  The batch is split across the GPUs (rank r runs images [B*r/N, B*(r+1)/N), full weight replica,
    no collective); time is the maximum over ranks.  `value` replays a captured run on device-resident
    inputs; `e2e` copies the rank's images from pinned host memory and brings its logits back every step;
    `eager` issues every node through the C ABI call by call (host-bound at small batches)."""
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
        return max_over_ranks(torch, dist, world, e0.elapsed_time(e1) / iters)

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
        launches0 = ex.stats.launches
        ms_eager = timed(lambda: ex.run_device({"input": x}), iters)
        per_run = (ex.stats.launches - launches0) // (iters + 3)
        out[f"batch_{batch}"] = {"value": round(batch / ms * 1e3, 1), "ms": round(ms, 4), "tflops": round(batch * 1.482e9 / ms / 1e9, 1),
                                 "frac_of_nominal_2250": round(batch * 1.482e9 / ms / 1e9 / (NOMINAL_BF16 * world), 4),
                                 "e2e": round(batch / ms_e2e * 1e3, 1), "eager": round(batch / ms_eager * 1e3, 1),
                                 "launches_per_run": per_run, "per_gpu_batch": hi - lo}
    if cpu_baseline and rank == 0:
        import numpy as np
        from oracle import binding as orc
        from oracle import onnx_cpu

        images = 32
        x = np.random.default_rng(1234 + 3).standard_normal((images, 3072), dtype=np.float32)
        t0 = time.perf_counter()
        onnx_cpu.run(model, {"input": x})
        secs = time.perf_counter() - t0
        out["cpu_baseline"] = {"value": round(images / secs, 1), "unit": "images/s", "cores": min(orc.host_threads(), 16), "kind": "port",
                               "sample": f"{images} images through the CPU graph walk (convolveNhwc / matmulTiled restatements), one pass, {secs:.1f} s"}
    return out


# ---- config 3: the convolution layers --------------------------------------------------------------------------
def conv_layers(gpu, torch, cpu_baseline, peaks):
    """Kernel times of every convolution layer of ResNet-14 64-128-256 (examples/cifar/main.zig:15-34) at batch 128,
    bf16 storage and f32 accumulation, all three passes, each from the replay of a CUDA graph of 20 launches; the
    strided variants of the four transition convolutions; and the 64-192-384 widths of the inference graph.
    Per pass: TFLOP/s with its fraction of the nominal (2250) and measured tensor peak, and the HBM GB/s that the
    algorithmic bytes 2*(x + w + y elements) amount to (64-channel layers sit on the ridge: both are reported)."""
    from grad_b200 import Epilogue, conv_geometry

    n = 128
    # (name, image side, c_in, k, c_out, stride, how often the layer occurs in the network)
    stack = [("stem 3->64 3x3 @32", 32, 3, 3, 64, 1, 1), ("64->64 3x3 @32", 32, 64, 3, 64, 1, 4), ("64->128 3x3 @16", 16, 64, 3, 128, 1, 1),
             ("128->128 3x3 @16", 16, 128, 3, 128, 1, 3), ("64->128 1x1 @16", 16, 64, 1, 128, 1, 1), ("128->256 3x3 @8", 8, 128, 3, 256, 1, 1),
             ("256->256 3x3 @8", 8, 256, 3, 256, 1, 3), ("128->256 1x1 @8", 8, 128, 1, 256, 1, 1),
             ("64->128 3x3 s2 @32", 32, 64, 3, 128, 2, 0), ("64->128 1x1 s2 @32", 32, 64, 1, 128, 2, 0),
             ("128->256 3x3 s2 @16", 16, 128, 3, 256, 2, 0), ("128->256 1x1 s2 @16", 16, 128, 1, 256, 2, 0)]
    wide = [("64->192 3x3 @16", 16, 64, 3, 192, 1, 0), ("192->192 3x3 @16", 16, 192, 3, 192, 1, 0), ("192->384 3x3 @8", 8, 192, 3, 384, 1, 0),
            ("384->384 3x3 @8", 8, 384, 3, 384, 1, 0), ("64->192 3x3 s2 @32", 32, 64, 3, 192, 2, 0), ("64->192 1x1 s2 @32", 32, 64, 1, 192, 2, 0)]
    cpu_for = {"64->64 3x3 @32", "128->128 3x3 @16", "256->256 3x3 @8"}   # one layer per stage beside the CPU path
    gen = torch.Generator(device="cuda").manual_seed(1234 + 2)
    rows, totals = [], {"fprop": 0.0, "dgrad": 0.0, "wgrad": 0.0, "gflop": 0.0}
    for group, layers in (("resnet14_64_128_256", stack), ("resnet14_64_192_384", wide)):
        for name, hw, c, k, co, stride, count in layers:
            geo = conv_geometry(n, hw, hw, c, k, co, stride, k // 2)
            x = torch.randn((n, hw, hw, c), generator=gen, device="cuda").bfloat16()
            w = (torch.randn((k * k * c, co), generator=gen, device="cuda") * (2.0 / (k * k * c)) ** 0.5).bfloat16()
            dy = torch.randn((n, geo.out_h, geo.out_w, co), generator=gen, device="cuda").bfloat16()
            y, dx = torch.empty_like(dy), torch.empty_like(x)
            dw = torch.zeros((k * k * c, co), device="cuda")
            bias = torch.randn(co, generator=gen, device="cuda")
            flop = 2.0 * geo.positions * k * k * c * co
            nbytes = 2.0 * (x.numel() + w.numel() + dy.numel())
            row = {"net": group, "layer": name, "batch": n, "gflop": round(flop / 1e9, 2), "algorithmic_mb": round(nbytes / 1e6, 2)}
            for key, fn in (("fprop", lambda: gpu.convForward(x, w, y, geo, epilogue=Epilogue(bias, None, True))),
                            ("dgrad", lambda: gpu.convInputGrad(dy, w, dx, geo)), ("wgrad", lambda: gpu.convWeightGrad(dy, x, dw, geo))):
                ms = graph_ms(torch, fn)
                tf = flop / ms / 1e9
                row[key] = {"us": round(ms * 1e3, 1), "tflops": round(tf, 1), "frac_of_nominal_2250": round(tf / NOMINAL_BF16, 3),
                            "frac_of_measured": round(tf / peaks["bf16_tflops"], 3), "hbm_gbs": round(nbytes / ms / 1e6, 1),
                            "frac_of_measured_hbm": round(nbytes / ms / 1e6 / peaks["hbm_gbs"], 3)}
                if count:
                    totals[key] += count * ms
            if count:
                totals["gflop"] += count * flop / 1e9
            if name in cpu_for:
                row["batch_norm_pieces_us"] = batch_norm_pieces(gpu, torch, gen, geo, x, w, y, dy, dx, dw)
            if cpu_baseline and name in cpu_for:
                row["cpu_baseline"] = conv_cpu(n, hw, c, k, co, stride, flop)
            rows.append(row)
    summary = {"net": "resnet14_64_128_256", "batch": n, "gflop_per_pass": round(totals["gflop"], 1)}
    for key in ("fprop", "dgrad", "wgrad"):
        summary[key] = {"ms": round(totals[key], 4), "tflops": round(totals["gflop"] / totals[key], 1),
                        "frac_of_nominal_2250": round(totals["gflop"] / totals[key] / NOMINAL_BF16, 3)}
    return {"layers": rows, "network_sum": summary}


def batch_norm_pieces(gpu, torch, gen, geo, x, w, y, dy, dx, dw):
    """The fused batch-norm pieces of the bf16 training path on one layer (src/gpu/gpu.zig:915-1022), each beside the plain
    pass it extends: forward with the statistics of its result in the epilogue (atomics, and the ordered mode with its
    combine launch), forward and weight gradient over a normalised-and-rectified input that is never written out, input
    gradient with the masked batch-norm gradient sums.  Microseconds from CUDA-graph replays."""
    from grad_b200 import Epilogue

    c, co = x.shape[-1], y.shape[-1]
    mean = torch.randn(c, generator=gen, device="cuda") * 0.1
    inv_std, gamma = torch.rand(c, generator=gen, device="cuda") + 0.5, torch.rand(c, generator=gen, device="cuda") + 0.5
    beta = torch.randn(c, generator=gen, device="cuda") * 0.1
    shift, sums, dx_sums = torch.zeros(co, device="cuda"), torch.zeros(2 * co, device="cuda"), torch.zeros(2 * c, device="cuda")
    cases = (("fprop", lambda: gpu.convForward(x, w, y, geo)),
             ("fprop_stats", lambda: gpu.convForward(x, w, y, geo, epilogue=Epilogue(stats_shift=shift, stats_sums=sums))),
             ("fprop_stats_ordered", lambda: gpu.convForward(x, w, y, geo, epilogue=Epilogue(stats_shift=shift, stats_sums=sums, stats_ordered=True))),
             ("fprop_affine_input", lambda: gpu.convForwardAffine(x, w, y, geo, mean, inv_std, gamma, beta)),
             ("wgrad", lambda: gpu.convWeightGrad(dy, x, dw, geo)),
             ("wgrad_affine_input", lambda: gpu.convWeightGradAffine(dy, x, dw, geo, mean, inv_std, gamma, beta)),
             ("dgrad", lambda: gpu.convInputGrad(dy, w, dx, geo, accumulate=False)),
             ("dgrad_dx_stats", lambda: gpu.convInputGradDxStats(dy, w, dx, geo, x, mean, inv_std, gamma, beta, dx_sums)))
    return {key: round(graph_ms(torch, fn) * 1e3, 1) for key, fn in cases}


def conv_cpu(n, hw, c, k, co, stride, flop):
    """grad's CPU convolution (chunked im2col + tiled matmul, col2im, src/cpu/ops.zig:131-285) on the same layer."""
    import numpy as np
    from oracle import binding as orc

    d = orc.ConvDims(n=n, h=hw, w=hw, c=c, k=k, stride=stride, pad=k // 2, dilation=1, c_out=co)
    rng = np.random.default_rng(1234 + 2)
    x = rng.standard_normal((n, hw, hw, c), dtype=np.float32)
    w = rng.standard_normal((d.taps, co), dtype=np.float32)
    dy = rng.standard_normal((n, d.out_h, d.out_w, co), dtype=np.float32)
    threads = orc.host_threads()
    out = {"unit": "TFLOP/s", "cores": min(threads, 16), "kind": "port", "sample": "the whole layer at batch 128, best of 2"}
    for key, fn in (("fprop", lambda: orc.conv_forward(x, w, d, threads)), ("dgrad", lambda: orc.conv_input_grad(dy, w, d, threads)),
                    ("wgrad", lambda: orc.conv_weight_grad(x, dy, d, threads))):
        best = float("inf")
        for _ in range(2):
            t0 = time.perf_counter()
            fn()
            best = min(best, time.perf_counter() - t0)
        out[key] = {"ms": round(best * 1e3, 1), "tflops": round(flop / best / 1e12, 4)}
    return out


# ---- config 2: the GEMM sweep ---------------------------------------------------------------------------------
def gemm_sweep(gpu, torch, peaks):
    """The standalone GEMM sweep (src/bench.zig:177-273 runs the same shapes on the CPU): square products of 1024..8192 and
    the skinny 128 x 4096 x 4096 in the three layouts autograd uses (NN forward, NT for dX, TN for dW), with bf16 operands,
    with f32 operands under TF32 math, and in strict f32 (up to 4096: 8192^3 on the FMA path is 27 ms a launch), each
    with the fused bias + ReLU epilogue.  Device time per launch from the replay of a CUDA graph."""
    from grad_b200 import Epilogue, MatmulOpts, MatmulShape
    from grad_b200.abi import MATH_BF16, MATH_F32, MATH_TF32

    gen = torch.Generator(device="cuda").manual_seed(1234 + 1)
    rows = []
    shapes = [(1024, 1024, 1024), (2048, 2048, 2048), (4096, 4096, 4096), (8192, 8192, 8192), (128, 4096, 4096)]
    for math, name, dt, nominal in ((MATH_BF16, "bf16", torch.bfloat16, NOMINAL_BF16), (MATH_TF32, "tf32", torch.float32, NOMINAL_TF32),
                                    (MATH_F32, "f32", torch.float32, None)):
        for m, n, k in shapes:
            if math == MATH_F32 and m * n * k > 4096 ** 3:
                continue
            for layout in ("NN", "NT", "TN"):
                ta, tb = layout == "TN", layout == "NT"
                a = torch.randn((k, m) if ta else (m, k), generator=gen, device="cuda").to(dt)
                b = torch.randn((n, k) if tb else (k, n), generator=gen, device="cuda").to(dt)
                bias = torch.randn(n, generator=gen, device="cuda")
                out = torch.empty((m, n), dtype=dt, device="cuda")
                shape, opts, ep = MatmulShape(m, n, k), MatmulOpts(ta, tb), Epilogue(bias, None, True)
                flop = 2.0 * m * n * k
                calls = 3 if flop > 2e11 else (10 if flop > 1e10 else 20)
                ms = graph_ms(torch, lambda: gpu.matmul(a, b, out, shape, opts, epilogue=ep, math=math), calls=calls, reps=3)
                plan = gpu.last_plan()
                row = {"m": m, "n": n, "k": k, "layout": layout, "math": name, "us": round(ms * 1e3, 1), "tflops": round(flop / ms / 1e9, 1),
                       "tile": f"{plan['tile_m']}x{plan['tile_n']}", "splits": plan["splits"], "launches": plan["kernel_launches"]}
                if nominal:
                    row["frac_of_nominal"] = round(flop / ms / 1e9 / nominal, 3)
                if math == MATH_BF16:
                    row["frac_of_measured"] = round(flop / ms / 1e9 / peaks["bf16_tflops"], 3)
                rows.append(row)
                del a, b, out
    torch.cuda.empty_cache()
    return {"epilogue": "bias + ReLU", "nominal_tflops": {"bf16": NOMINAL_BF16, "tf32": NOMINAL_TF32}, "products": rows}


# ---- config 1: the MLP step ------------------------------------------------------------------------------------
def mlp_step(gpu, torch, cpu_baseline):
    """MLP 784-128-10, f32, batch 64: forward and backward of both Linear layers as ONE captured step of six GEMMs
    (NN 64x784x128 with bias + ReLU, NN 64x128x10 with bias; NT for dX, TN for dW, `+=` into zeroed gradients), the
    way the reference replays a captured training step (src/nn/trainer.zig:474-511); 2*64*128*(784+10)*3 = 39.0 MFLOP
    (src/bench.zig:271).  Beside it the CPU worker-pool path (`matmulTiled`) on the same six products."""
    from grad_b200 import Epilogue, MatmulOpts, MatmulShape
    from grad_b200.abi import MATH_F32

    gen = torch.Generator(device="cuda").manual_seed(1234)
    x = torch.rand((64, 784), generator=gen, device="cuda")
    w1 = torch.randn((784, 128), generator=gen, device="cuda") * (2.0 / 784) ** 0.5
    w2 = torch.randn((128, 10), generator=gen, device="cuda") * (2.0 / 128) ** 0.5
    b1, b2 = torch.zeros(128, device="cuda"), torch.zeros(10, device="cuda")
    h, y = torch.empty((64, 128), device="cuda"), torch.empty((64, 10), device="cuda")
    dy = torch.randn((64, 10), generator=gen, device="cuda")
    dh, dx = torch.empty_like(h), torch.empty_like(x)
    grads = torch.zeros(784 * 128 + 128 * 10, device="cuda")
    dw1, dw2 = grads[:784 * 128].view(784, 128), grads[784 * 128:].view(128, 10)

    def step():
        grads.zero_()
        gpu.matmul(x, w1, h, MatmulShape(64, 128, 784), MatmulOpts(), epilogue=Epilogue(b1, None, True), math=MATH_F32)
        gpu.matmul(h, w2, y, MatmulShape(64, 10, 128), MatmulOpts(), epilogue=Epilogue(b2, None, False), math=MATH_F32)
        gpu.matmul(dy, w2, dh, MatmulShape(64, 128, 10), MatmulOpts(False, True), math=MATH_F32)
        gpu.matmul(h, dy, dw2, MatmulShape(128, 10, 64), MatmulOpts(True, False, True), math=MATH_F32)
        gpu.matmul(dh, w1, dx, MatmulShape(64, 784, 128), MatmulOpts(False, True), math=MATH_F32)
        gpu.matmul(x, dh, dw1, MatmulShape(784, 128, 64), MatmulOpts(True, False, True), math=MATH_F32)

    launches0 = gpu.launches
    step()
    per_step = gpu.launches - launches0
    ms = graph_ms(torch, step, calls=10, reps=10)
    flop = 2.0 * 64 * 128 * (784 + 10) * 3
    out = {"workload": "MLP 784-128-10 f32 batch 64: six GEMMs fwd+bwd, one captured step", "steps_per_s": round(1e3 / ms, 1), "us_per_step": round(ms * 1e3, 2),
           "gflops": round(flop / ms / 1e6, 1), "launches_per_step": per_step + 1, "dtype": "f32"}
    if cpu_baseline:
        import numpy as np
        from oracle import binding as orc

        threads = orc.host_threads()
        hx, hw1, hw2, hdy = (t.cpu().numpy() for t in (x, w1, w2, dy))
        hh, hdh = h.cpu().numpy(), dh.cpu().numpy()
        g1, g2 = np.zeros((784, 128), np.float32), np.zeros((128, 10), np.float32)

        def cpu_step():
            orc.matmul_tiled(hx, hw1, 64, 784, 128, threads=threads)
            orc.matmul_tiled(hh, hw2, 64, 128, 10, threads=threads)
            orc.matmul_tiled(hdy, hw2, 64, 10, 128, False, True, threads=threads)
            orc.matmul_tiled(hh, hdy, 128, 64, 10, True, False, out=g2, threads=threads)
            orc.matmul_tiled(hdh, hw1, 64, 128, 784, False, True, threads=threads)
            orc.matmul_tiled(hx, hdh, 784, 64, 128, True, False, out=g1, threads=threads)

        best = float("inf")
        for _ in range(20):
            t0 = time.perf_counter()
            cpu_step()
            best = min(best, time.perf_counter() - t0)
        out["cpu_baseline"] = {"value": round(1.0 / best, 1), "unit": "steps/s", "cores": min(threads, 16), "kind": "port",
                               "sample": "the same six products through the matmulTiled restatement, best of 20 steps"}
    return out


# ---- config 5: the character-Transformer step ------------------------------------------------------------------
TRANSFORMER = dict(vocab=65, width=256, heads=4, layers=4, ffn=1024, seq=128, batch=64, grad_len=3228737)


def transformer_step(gpu, rank, world, dist, torch, cpu_baseline):
    """The contractions of one data-parallel training step of the character Transformer (vocab 65, width 256, 4 heads,
    4 blocks, FFN 1024, context 128, 64 sequences per replica = 8192 rows) in bf16 with f32 accumulation, through
    `Gpu.matmul`: per block the Q/K/V projections, the 256 score and 256 mixing products (batched entry), the output
    projection and the two FFN products, then the vocabulary head; every product forward, its input gradient (NT) and
    its weight gradient (TN, `+=` into a slice of ONE flat f32 gradient vector).  `per_head` issues the projections
    the way the reference composes attention (one Linear per head and per Q/K/V: 12 products of 8192x256x64 and 4 of
    8192x64x256 per block, src/nn/nn.zig:421-461); `fused_qkv` issues one 8192x256x768 and one 8192x256x256 product
    instead and each attention product of a block as ONE launch over (sequence, head) with two batch levels; `fused_qkv_two_streams` is the same list of launches captured as a graph with two branches: weight
    gradients and dV / dK go to a side stream (a second handle with its own
    workspace), so products that are one wave of tiles or less run beside each other instead of one after the other.  After the captured contraction step the flat gradient vector (3 228 737 floats, all parameters) is
    averaged over the replicas by ONE `gb_allreduce_mean`, outside the graph, where `averageGrads` sits in the
    reference (src/nn/trainer.zig:507-508).  Softmax, layer norm, embedding, loss and Adam are not contractions and
    are not part of this path."""
    from grad_b200 import Epilogue, MatmulOpts, MatmulShape
    from grad_b200.abi import MATH_BF16
    from grad_b200.replicas import Replicas

    cfg = TRANSFORMER
    d, heads, ffn, seq, vocab, layers = cfg["width"], cfg["heads"], cfg["ffn"], cfg["seq"], cfg["vocab"], cfg["layers"]
    hd = d // heads
    seqs = cfg["batch"]
    rows = seqs * seq
    gen = torch.Generator(device="cuda").manual_seed(1234 + 4)   # the same seed on every replica (src/nn/trainer.zig:411)
    bf = torch.bfloat16

    def randn(*shape, scale=1.0, dtype=bf):
        return (torch.randn(shape, generator=gen, device="cuda") * scale).to(dtype)

    flat = torch.zeros(cfg["grad_len"], device="cuda")
    cursor = [0]

    def grad_view(r, c):
        off = (cursor[0] + 3) // 4 * 4
        cursor[0] = off + r * c
        return flat[off:off + r * c].view(r, c)

    flops = [0.0]

    import grad_b200

    gpu_main = gpu
    side_stream = torch.cuda.Stream()
    gpu_side = grad_b200.Gpu(torch.cuda.current_device())   # its own workspace: its products run beside the main handle's
    two_streams = [False]
    side_used = [False]

    class on_side:
        """Runs the enclosed launches on the side stream after everything the main stream has been given so far."""

        def __enter__(self):
            self.active = two_streams[0]
            if self.active:
                side_used[0] = True
                side_stream.wait_stream(torch.cuda.current_stream())
                self.ctx = torch.cuda.stream(side_stream)
                self.ctx.__enter__()
            return gpu_side if self.active else gpu

        def __exit__(self, *exc):
            if self.active:
                self.ctx.__exit__(*exc)
            return False

    def join_side():
        if two_streams[0] and side_used[0]:   # only a stream that has joined the capture can be waited for
            torch.cuda.current_stream().wait_stream(side_stream)
            side_used[0] = False

    def mm(a, b, out, m, n, k, ta=False, tb=False, acc=False, batch=1, ep=None, strides=None, ld=(0, 0, 0), g=None):
        flops[0] += 2.0 * m * n * k * batch
        shape = MatmulShape(m, n, k, batch)
        (g or gpu).matmul(a, b, out, shape, MatmulOpts(ta, tb, acc), epilogue=ep, math=MATH_BF16, lda=ld[0], ldb=ld[1], ldc=ld[2])

    # Vocabulary 65: a bf16 row of 65 values is 130 bytes, which no TMA copy can step by (strides are multiples of 16
    # bytes), and such an operand falls to the gather warps (80-250 us per head product instead of ~10).  The head's
    # weight, logits and logit gradients therefore live in rows of 72 values (144 bytes), passed as lda / ldb / ldc: the
    # caller pads the pitch once where the reference's packMatrix pads a scratch copy on every call (gpu.zig:711-722).
    vpitch = (vocab + 7) // 8 * 8
    dy_head = randn(rows, vpitch)

    def build(fused: bool):
        cursor[0] = 0
        blocks = []
        for _ in range(layers):
            blk = {"wqkv": randn(d, 3 * d, scale=(2.0 / d) ** 0.5), "wo": randn(d, d, scale=(2.0 / d) ** 0.5),
                   "w1": randn(d, ffn, scale=(2.0 / d) ** 0.5), "w2": randn(ffn, d, scale=(2.0 / ffn) ** 0.5),
                   "b1": torch.zeros(ffn, device="cuda"), "b2": torch.zeros(d, device="cuda"),
                   "gqkv": grad_view(d, 3 * d), "go": grad_view(d, d), "g1": grad_view(d, ffn), "g2": grad_view(ffn, d),
                   # activations kept for the backward pass
                   "x": randn(rows, d), "qkv": torch.empty((3 * heads, rows, hd), dtype=bf, device="cuda"),
                   "p": torch.empty((heads * seqs, seq, seq), dtype=bf, device="cuda"), "o": torch.empty((heads, rows, hd), dtype=bf, device="cuda"),
                   "a": torch.empty((rows, d), dtype=bf, device="cuda"), "h": torch.empty((rows, ffn), dtype=bf, device="cuda"),
                   "y": torch.empty((rows, d), dtype=bf, device="cuda"),
                   "dh": torch.empty((rows, ffn), dtype=bf, device="cuda"), "da": torch.empty((rows, d), dtype=bf, device="cuda"),
                   "do": torch.empty((heads, rows, hd), dtype=bf, device="cuda"), "dp": torch.empty((heads * seqs, seq, seq), dtype=bf, device="cuda"),
                   "dqkv": torch.empty((3 * heads, rows, hd), dtype=bf, device="cuda"), "dx": torch.empty((rows, d), dtype=bf, device="cuda")}
            if fused:   # projections as single products: activations laid out (rows, 3*width) / (rows, width)
                blk["qkv2"] = torch.empty((rows, 3 * d), dtype=bf, device="cuda")
                blk["dqkv2"] = torch.empty((rows, 3 * d), dtype=bf, device="cuda")
                blk["o2"] = torch.empty((rows, d), dtype=bf, device="cuda")
                blk["do2"] = torch.empty((rows, d), dtype=bf, device="cuda")
            else:       # one weight matrix per head and per Q/K/V, as the reference holds them
                blk["wq"] = [randn(d, hd, scale=(2.0 / d) ** 0.5) for _ in range(3 * heads)]
                blk["woh"] = [randn(hd, d, scale=(2.0 / d) ** 0.5) for _ in range(heads)]
                blk["gq"] = [blk["gqkv"].view(-1)[i * d * hd:(i + 1) * d * hd].view(d, hd) for i in range(3 * heads)]
                blk["goh"] = [blk["go"].view(-1)[i * hd * d:(i + 1) * hd * d].view(hd, d) for i in range(heads)]
            blocks.append(blk)
        head = {"w": randn(d, vpitch, scale=(2.0 / d) ** 0.5), "g": grad_view(d, vocab), "logits": torch.empty((rows, vpitch), dtype=bf, device="cuda"),
                "dx": torch.empty((rows, d), dtype=bf, device="cuda")}
        return blocks, head

    def attention(blk, fused, backward):
        b = heads * seqs
        if fused:
            # (rows, 3*width) activations: head h of Q sits in columns h*hd.. of the first third, row pitch 3*width.  ONE launch
            # per product kind: the 64 sequences are the inner batch level (stride one sequence of rows), the heads the outer
            # one (stride hd columns; seqs matrices in the contiguous score tensors).  With two streams dV and dK go to the side.
            q, k_, v = (blk["qkv2"][:, part * d:] for part in range(3))
            dq, dk, dv = (blk["dqkv2"][:, part * d:] for part in range(3))
            p, dp, o, do = blk["p"], blk["dp"], blk["o2"], blk["do2"]
            st, sp = seq * 3 * d, seqs * seq * seq
            if not backward:
                batched(q, k_, p, seq, seq, hd, False, True, seqs, (st, st, seq * seq), (3 * d, 3 * d, 0), (hd, hd, sp))
                batched(p, v, o, seq, hd, seq, False, False, seqs, (seq * seq, st, seq * d), (0, 3 * d, d), (sp, hd, hd))
            else:
                with on_side() as g2:
                    batched(p, do, dv, seq, hd, seq, True, False, seqs, (seq * seq, seq * d, st), (0, d, 3 * d), (sp, hd, hd), g2)
                batched(do, v, dp, seq, seq, hd, False, True, seqs, (seq * d, st, seq * seq), (d, 3 * d, 0), (hd, hd, sp))
                with on_side() as g2:
                    batched(dp, q, dk, seq, hd, seq, True, False, seqs, (seq * seq, st, st), (0, 3 * d, 3 * d), (sp, hd, hd), g2)
                batched(dp, k_, dq, seq, hd, seq, False, False, seqs, (seq * seq, st, st), (0, 3 * d, 3 * d), (sp, hd, hd))
            join_side()
            return
        q, k_, v = blk["qkv"][0:heads].view(b, seq, hd), blk["qkv"][heads:2 * heads].view(b, seq, hd), blk["qkv"][2 * heads:].view(b, seq, hd)
        dq, dk, dv = blk["dqkv"][0:heads].view(b, seq, hd), blk["dqkv"][heads:2 * heads].view(b, seq, hd), blk["dqkv"][2 * heads:].view(b, seq, hd)
        o, do = blk["o"].view(b, seq, hd), blk["do"].view(b, seq, hd)
        if not backward:
            mm(q, k_, blk["p"], seq, seq, hd, False, True, batch=b)            # scores = Q K^T
            mm(blk["p"], v, o, seq, hd, seq, batch=b)                           # mix = P V
        else:
            mm(do, v, blk["dp"], seq, seq, hd, False, True, batch=b)           # dP = dO V^T
            mm(blk["p"], do, dv, seq, hd, seq, True, False, batch=b)           # dV = P^T dO
            mm(blk["dp"], k_, dq, seq, hd, seq, batch=b)                        # dQ = dS K
            mm(blk["dp"], q, dk, seq, hd, seq, True, False, batch=b)           # dK = dS^T Q

    def batched(a, b_, out, m, n, k, ta, tb, batch, strides, ld, outer_strides, g=None):
        flops[0] += 2.0 * m * n * k * batch * heads
        (g or gpu_main).matmulStrided(a, b_, out, m, n, k, MatmulOpts(ta, tb), batch=batch, strides=strides, ld=ld, outer=heads,
                                      outer_strides=outer_strides, math=MATH_BF16)

    def step(blocks, head, fused):
        """Weight gradients are issued before the input gradient that reads the same dy, on the side stream when there is
        one; the side stream joins before the products that read what it wrote and at the end of the step."""
        flat.zero_()                                                            # zeroGrad is part of the captured step
        for blk in blocks:                                                      # ---- forward
            if fused:
                mm(blk["x"], blk["wqkv"], blk["qkv2"], rows, 3 * d, d)
            else:
                for i in range(3 * heads):
                    mm(blk["x"], blk["wq"][i], blk["qkv"][i], rows, hd, d)
            attention(blk, fused, False)
            if fused:
                mm(blk["o2"], blk["wo"], blk["a"], rows, d, d)
            else:
                for hh in range(heads):
                    mm(blk["o"][hh], blk["woh"][hh], blk["a"], rows, d, hd, acc=hh > 0)
            mm(blk["a"], blk["w1"], blk["h"], rows, ffn, d, ep=Epilogue(blk["b1"], None, True))
            mm(blk["h"], blk["w2"], blk["y"], rows, d, ffn, ep=Epilogue(blk["b2"], None, False))
        mm(blocks[-1]["y"], head["w"], head["logits"], rows, vocab, d, ld=(0, vpitch, vpitch))
        with on_side() as g2:                                                    # ---- backward
            mm(blocks[-1]["y"], dy_head, head["g"], d, vocab, rows, True, False, acc=True, g=g2, ld=(0, vpitch, 0))
        mm(dy_head, head["w"], head["dx"], rows, d, vocab, False, True, ld=(vpitch, vpitch, 0))
        for blk in reversed(blocks):
            dy = head["dx"]
            with on_side() as g2:
                mm(blk["h"], dy, blk["g2"], ffn, d, rows, True, False, acc=True, g=g2)
            mm(dy, blk["w2"], blk["dh"], rows, ffn, d, False, True)
            with on_side() as g2:
                mm(blk["a"], blk["dh"], blk["g1"], d, ffn, rows, True, False, acc=True, g=g2)
            mm(blk["dh"], blk["w1"], blk["da"], rows, d, ffn, False, True)
            if fused:
                with on_side() as g2:
                    mm(blk["o2"], blk["da"], blk["go"], d, d, rows, True, False, acc=True, g=g2)
                mm(blk["da"], blk["wo"], blk["do2"], rows, d, d, False, True)
            else:
                for hh in range(heads):
                    mm(blk["da"], blk["woh"][hh], blk["do"][hh], rows, hd, d, False, True)
                    mm(blk["o"][hh], blk["da"], blk["goh"][hh], hd, d, rows, True, False, acc=True)
            attention(blk, fused, True)
            if fused:
                with on_side() as g2:
                    mm(blk["x"], blk["dqkv2"], blk["gqkv"], d, 3 * d, rows, True, False, acc=True, g=g2)
                mm(blk["dqkv2"], blk["wqkv"], blk["dx"], rows, d, 3 * d, False, True)
            else:
                for i in range(3 * heads):
                    mm(blk["dqkv"][i], blk["wq"][i], blk["dx"], rows, d, hd, False, True, acc=i > 0)
                    mm(blk["x"], blk["dqkv"][i], blk["gq"][i], d, hd, rows, True, False, acc=True)
        join_side()

    out = {"workload": "character Transformer: vocab 65, width 256, 4 heads, 4 blocks, FFN 1024, context 128, 64 sequences per replica; "
                       "bf16 contractions fwd + dX + dW, one captured step per replica; gradients averaged by one allreduce",
           "replicas": world, "dtype": "bf16", "grad_floats": cfg["grad_len"]}
    for label, fused, forked in (("per_head", False, False), ("fused_qkv", True, False), ("fused_qkv_two_streams", True, True)):
        blocks, head = build(fused)
        two_streams[0] = forked
        flops[0] = 0.0
        launches0 = gpu.launches + gpu_side.launches
        step(blocks, head, fused)
        torch.cuda.synchronize()
        per_step, gflop = gpu.launches + gpu_side.launches - launches0, flops[0] / 1e9
        ms = graph_ms(torch, lambda: step(blocks, head, fused), calls=2, reps=5)
        ms = max_over_ranks(torch, dist, world, ms)
        out[label] = {"ms_per_step": round(ms, 4), "gflop_per_replica_step": round(gflop, 1), "launches_per_step": per_step + 1,
                      "tflops": round(world * gflop / ms, 1), "frac_of_nominal_2250": round(gflop / ms / NOMINAL_BF16, 4),
                      "grads_finite": bool(torch.isfinite(flat).all().item())}
        if cpu_baseline and rank == 0 and label == "per_head":
            out["cpu_baseline"] = transformer_cpu(rows, d, hd, heads, ffn, vocab, seq, seqs, layers, gflop)
        del blocks, head
        torch.cuda.empty_cache()

    # ---- the gradient mean: one collective over the flat vector -------------------------------------------------
    if world > 1:
        group = Replicas(world, rank, device=torch.cuda.current_device(), timeout_s=60.0)
        gen_r = torch.Generator(device="cuda").manual_seed(5000 + rank)
        flat.copy_(torch.randn(flat.numel(), generator=gen_r, device="cuda"))
        mine = flat.clone()
        group.averageGrads(flat, finish=True)
        # identical bits on every replica (tests/replicas.zig:76) and the reference's mean (sum in replica order, times 1/N)
        gathered = [torch.empty_like(flat) for _ in range(world)]
        dist.all_gather(gathered, flat)
        identical = all(torch.equal(gathered[0], g) for g in gathered)
        inputs = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(inputs, mine)
        want = inputs[0].clone()
        for t in inputs[1:]:
            want += t
        want *= 1.0 / world
        err = float((flat - want).abs().max().item() / want.abs().max().item())
        del gathered, inputs, mine
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 50

        def timed_mean(barrier):
            for _ in range(5):
                group.averageGrads(flat, barrier=barrier)
            torch.cuda.synchronize()
            dist.barrier()
            e0.record()
            for _ in range(reps):
                group.averageGrads(flat, barrier=barrier)
            e1.record()
            torch.cuda.synchronize()
            return max_over_ranks(torch, dist, world, e0.elapsed_time(e1) / reps) * 1e3

        us = timed_mean(False)
        us_barrier = timed_mean(True)
        nbytes = flat.numel() * 4
        bus = 2.0 * (world - 1) / world * nbytes / (us * 1e-6) / 1e9
        out["allreduce"] = {"us": round(us, 1), "bytes": nbytes, "bus_gbs": round(bus, 1), "frac_of_nvlink_770": round(bus / 770.0, 3),
                            "identical_bits_on_all_replicas": bool(identical), "max_rel_err_vs_ordered_mean": err,
                            "us_with_host_barrier": round(us_barrier, 1),
                            "includes": "`us`: one ncclAllReduce(avg) over the flat vector, back to back on the device; `us_with_host_barrier` adds the "
                                        "rendezvous-store barrier in front of it (the reference's wait(), a host round trip per step)",
                            "limiter": "NCCL latency (launch + NVLink hops), not bandwidth, while bus_gbs stays far below 770"}
        for label in ("per_head", "fused_qkv", "fused_qkv_two_streams"):
            total = out[label]["ms_per_step"] + us * 1e-3
            out[label]["ms_with_allreduce"] = round(total, 4)
            out[label]["tflops_with_allreduce"] = round(world * out[label]["gflop_per_replica_step"] / total, 1)
        group.close()
    return out


def transformer_cpu(rows, d, hd, heads, ffn, vocab, seq, seqs, layers, gflop):
    """The same contraction list of ONE block (forward, dX, dW) through the CPU `matmulTiled` restatement, scaled to the
    whole step by its share of the FLOPs."""
    import numpy as np
    from oracle import binding as orc

    threads = orc.host_threads()
    rng = np.random.default_rng(1234 + 4)

    def r(*s):
        return rng.standard_normal(s, dtype=np.float32)

    x, wq, wo, w1, w2 = r(rows, d), r(d, hd), r(hd, d), r(d, ffn), r(ffn, d)
    q, p = r(seq, hd), r(seq, seq)
    dh, dd = r(rows, ffn), r(rows, d)
    done = [0.0]

    def mm(a, b, m, k, n, ta=False, tb=False, times=1):
        for _ in range(times):
            orc.matmul_tiled(a, b, m, k, n, ta, tb, threads=threads)
        done[0] += 2.0 * m * n * k * times

    t0 = time.perf_counter()
    mm(x, wq, rows, d, hd, times=3 * heads)                       # projections, forward
    mm(dd[:, :hd].copy(), wq, rows, hd, d, False, True, times=3 * heads)
    mm(x, dd[:, :hd].copy(), d, rows, hd, True, False, times=3 * heads)
    sample = 16                                                   # of the 256 attention products per kind
    mm(q, q, seq, hd, seq, False, True, times=2 * sample)         # scores and dP
    mm(p, q, seq, seq, hd, times=2 * sample)                      # mix and dQ
    mm(p, q, seq, seq, hd, True, False, times=2 * sample)         # dV and dK
    att_scale = heads * seqs / sample
    t_att0 = time.perf_counter()
    mm(x[:, :hd].copy(), wo, rows, hd, d, times=heads)
    mm(dd, wo, rows, d, hd, False, True, times=heads)
    mm(x[:, :hd].copy(), dd, hd, rows, d, True, False, times=heads)
    mm(x, w1, rows, d, ffn)
    mm(dh, w1, rows, ffn, d, False, True)
    mm(x, dh, d, rows, ffn, True, False)
    mm(dh, w2, rows, ffn, d)
    mm(dd, w2, rows, d, ffn, False, True)
    mm(dh, dd, ffn, rows, d, True, False)
    secs = time.perf_counter() - t0
    del t_att0, att_scale
    tf = done[0] / secs / 1e12
    return {"value": round(tf, 4), "unit": "TFLOP/s", "cores": min(threads, 16), "kind": "port",
            "ms_per_step_extrapolated": round(gflop / tf, 1),
            "sample": f"one block's products (16 of its 256 attention products per kind), {done[0] / 1e9:.1f} GFLOP in {secs:.2f} s, scaled by FLOPs"}


def profile_only(args, gpu, torch):
    """Small fixed workloads for profiler captures; nothing is timed or printed as a bench line."""
    from grad_b200 import Epilogue, MatmulOpts, MatmulShape, conv_geometry

    if args.profile_resnet:
        from grad_b200.onnx_gpu import Executor, resnet14_model

        ex = Executor(resnet14_model(64, 192, 384), gpu, "bf16")
        x = torch.randn((args.profile_resnet, 3072), device="cuda")
        for _ in range(3):
            ex.run_device({"input": x})
    elif args.profile_gemm:
        m, n, k, layout, math = args.profile_gemm.split(",")
        m, n, k, math = int(m), int(n), int(k), int(math)
        ta, tb = layout == "TN", layout == "NT"
        dt = torch.bfloat16 if math == 2 else torch.float32
        a = torch.randn((k, m) if ta else (m, k), device="cuda").to(dt)
        b = torch.randn((n, k) if tb else (k, n), device="cuda").to(dt)
        bias = torch.randn(n, device="cuda")
        out = torch.empty((m, n), dtype=dt, device="cuda")
        for _ in range(6):
            gpu.matmul(a, b, out, MatmulShape(m, n, k), MatmulOpts(ta, tb), epilogue=Epilogue(bias, None, True), math=math)
    else:
        parts = args.profile_conv.split(",")
        n, h, w_, c, k, co, stride, pad = (int(v) for v in parts[:8])
        which = parts[8] if len(parts) > 8 else "fprop"
        geo = conv_geometry(n, h, w_, c, k, co, stride, pad)
        x = torch.randn((n, h, w_, c), device="cuda").bfloat16()
        w = (torch.randn((k * k * c, co), device="cuda") * (2.0 / (k * k * c)) ** 0.5).bfloat16()
        y = torch.empty((n, geo.out_h, geo.out_w, co), dtype=torch.bfloat16, device="cuda")
        dx = torch.empty_like(x)
        dw = torch.zeros((k * k * c, co), device="cuda")
        bias = torch.randn(co, device="cuda")
        shift, sums, dx_sums = torch.zeros(co, device="cuda"), torch.zeros(2 * co, device="cuda"), torch.zeros(2 * c, device="cuda")
        norm = [torch.rand(c, device="cuda") + 0.5 for _ in range(4)]   # mean, inv_std, gamma, beta of a virtual normalised input
        for _ in range(6):
            if which == "fprop":
                gpu.convForward(x, w, y, geo, epilogue=Epilogue(bias, None, True))
            elif which == "dgrad":
                gpu.convInputGrad(y, w, dx, geo, accumulate=False)
            elif which == "stats":
                gpu.convForward(x, w, y, geo, epilogue=Epilogue(stats_shift=shift, stats_sums=sums))
            elif which == "affine":
                gpu.convForwardAffine(x, w, y, geo, *norm)
            elif which == "wgrad_affine":
                gpu.convWeightGradAffine(y, x, dw, geo, *norm)
            elif which == "dx_stats":
                gpu.convInputGradDxStats(y, w, dx, geo, x, *norm, dx_sums)
            else:
                gpu.convWeightGrad(y, x, dw, geo)
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
    numa = pin_to_gpu_numa_node(torch, local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    import grad_b200
    from grad_b200 import Epilogue, MatmulOpts, MatmulShape

    gpu = grad_b200.Gpu(local)
    if args.profile_resnet or args.profile_conv or args.profile_gemm:
        if rank == 0:
            profile_only(args, gpu, torch)
        return
    legs = set(args.legs.split(",")) & set(ALL_LEGS)
    legs.add("gemm")
    if args.no_resnet:
        legs -= {"resnet", "conv", "mlp", "transformer", "sustained", "sweep"}
    cpu_ok = not args.no_cpu_baseline
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

    sampler = ClockSampler(torch, local)
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
    ms_total = max_over_ranks(torch, dist, world, e0.elapsed_time(e1))
    launches = gpu.launches - launches0
    gpu.check_status()
    ms_step = ms_total / args.steps
    flops = 2.0 * m * n * k
    value = world * flops / (ms_step * 1e-3) / 1e12
    peaks, peak_kind = measured_peaks()

    # ---- parity of the timed product: sampled rows recomputed by the CPU oracle on the same operands ----
    parity, cpu_base = None, None
    if rank == 0 and world == 1 and cpu_ok:
        import numpy as np

        band = max(1, m // 64)                                   # 64 rows, one per 128-row block of an 8192-row product, varying lanes
        rows = sorted({min(m - 1, t * band + (37 * t) % band) for t in range(64)})
        idx = torch.tensor(rows, device="cuda")
        a_rows = (a[:, idx] if ta else a[idx, :]).float().cpu().numpy()
        hb, hbias = b.float().cpu().numpy(), bias.cpu().numpy()
        want, _, _, _ = cpu_rows(np.ascontiguousarray(a_rows), hb, hbias, ta, tb, 1)
        got = out[idx, :].float().cpu().numpy()
        rel = float(np.linalg.norm((got - want).ravel()) / np.linalg.norm(want.ravel()))
        parity = {"rel_fro": rel, "rows": len(rows), "tolerance": 2e-2, "ok": bool(rel <= 2e-2),
                  "against": "CPU restatement of grad's matmulTiled + bias + ReLU on the same operands"}
        # the timed CPU baseline: half of the rows of the same product
        sub = torch.arange(0, min(4096, m), device="cuda")
        a_sub = np.ascontiguousarray((a[:, sub] if ta else a[sub, :]).float().cpu().numpy())
        _, cpu_value, cores, secs = cpu_rows(a_sub, hb, hbias, ta, tb, 2)
        cpu_base = {"value": round(cpu_value, 4), "unit": UNIT, "cores": cores, "kind": "port",
                    "sample": f"{len(sub)} of {m} rows of A against the full B (N=K={size}), best of 2, {secs:.2f} s each; "
                              "C++ restatement of grad's matmulTiled + bias + ReLU"}
        del hb

    # ---- sustained: the same launch back to back for seconds, under the power cap ----
    sustained = None
    if "sustained" in legs:
        chunk = max(10, int(0.05 / (ms_step * 1e-3)))            # launches per timed chunk, about 50 ms
        chunks = max(8, int(args.sustained_seconds / (chunk * ms_step * 1e-3)))
        events = [torch.cuda.Event(enable_timing=True) for _ in range(chunks + 1)]
        s2 = ClockSampler(torch, local)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        s2.start()
        events[0].record()
        for c in range(chunks):
            for _ in range(chunk):
                step()
            events[c + 1].record()
        torch.cuda.synchronize()
        clk = s2.stop()
        per = [events[c].elapsed_time(events[c + 1]) / chunk for c in range(chunks)]
        med = max_over_ranks(torch, dist, world, statistics.median(per))
        best = min(per)
        tf_med, tf_best = flops / (med * 1e-3) / 1e12, flops / (best * 1e-3) / 1e12
        sustained = {"seconds": round(sum(per) * chunk * 1e-3, 2), "launches": chunk * chunks, "median_tflops": round(tf_med, 1), "best_tflops": round(tf_best, 1),
                     "median_ms": round(med, 4), "clocks": clk,
                     "frac_of_measured_sustained": round(tf_med / peaks["bf16_tflops_sustained"], 4), "frac_of_nominal_2250": round(tf_med / NOMINAL_BF16, 4),
                     "cycles_per_launch_at_median_clock": None if not clk.get("sm_mhz") else round(med * 1e-3 * clk["sm_mhz"] * 1e6)}

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
    e2e_ms = max_over_ranks(torch, dist, world, e0.elapsed_time(e1))
    e2e_value = world * flops / (e2e_ms / args.e2e_steps * 1e-3) / 1e12
    h2d = ha.numel() * 2 + hb.numel() * 2
    d2h = hout.numel() * 2
    del ha, hb, hout, da, db, dout
    torch.cuda.empty_cache()

    resnet = resnet_inference(gpu, rank, world, dist, torch, cpu_ok and world == 1) if "resnet" in legs else None
    transformer = transformer_step(gpu, rank, world, dist, torch, cpu_ok and world == 1) if "transformer" in legs else None
    sweep = gemm_sweep(gpu, torch, peaks) if (rank == 0 and "sweep" in legs) else None
    convs = conv_layers(gpu, torch, cpu_ok and world == 1, peaks) if (rank == 0 and "conv" in legs) else None
    mlp = mlp_step(gpu, torch, cpu_ok and world == 1) if (rank == 0 and "mlp" in legs) else None
    gpu.check_status()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    timed_s = ms_total * 1e-3
    long_run = timed_s > 1.0
    peak = peaks["bf16_tflops_sustained"] if long_run else peaks["bf16_tflops"]
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
                   "tile": f"{plan['tile_m']}x{plan['tile_n']}", "stages": plan["stages"], "splits": plan["splits"], "host_numa": numa},
        "clocks": clocks,
        "e2e": {"value": round(e2e_value, 2), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": round(e2e_ms / args.e2e_steps, 3)},
        "gpu_launches": launches,
        "roofline": {"bound": "tensor", "achieved": round(achieved, 2), "peak": peak, "unit": UNIT, "frac": round(achieved / peak, 4),
                     "traffic": traffic, "peak_source": f"{peak_kind} cuBLAS bf16 {'sustained' if long_run else 'burst'}",
                     "frac_of_nominal_2250": round(achieved / NOMINAL_BF16, 4)},
    }
    if parity is not None:
        line["parity"] = parity
    if sustained is not None:
        line["sustained"] = sustained
    if sweep is not None:
        line["gemm_sweep"] = sweep
    if resnet is not None:
        line["resnet14_inference"] = resnet
    if convs is not None:
        line["conv_layers"] = convs
    if mlp is not None:
        line["mlp_step"] = mlp
    if transformer is not None:
        line["transformer_step"] = transformer
    if cpu_base is not None:
        line["cpu_baseline"] = cpu_base
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
