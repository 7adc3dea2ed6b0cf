"""Benchmark of the TOSA data-graph hot path on B200.

    python bench.py --gpus N --steps K --warmup W          (N>1: launched under torchrun, one rank per GPU)
    python bench.py --impl reference ...                   (the CPU restatement of the reference, timed on host cores)

Workload: the ResNet-50-shaped int8 TOSA graph of BASELINE.json configs[3], N=64 images per GPU,
224x224x3, synthetic seeded data and random-init int8 weights.  One step = one dispatch of the whole
graph over one batch.  The graph is batch-sharded: each rank owns its own 64 images, pipeline,
constants and session memory; the only collective is an NCCL all-gather of the [64,1000] int8 logits.

Printed JSON (rank 0): metric images/s over all ranks, device-timed with CUDA events on the dispatch
stream (max over ranks), plus
  roofline      dominant kernel class (fused CONV2D+RESCALE): algorithmic int8 ops / measured kernel time
  cpu_baseline  the oracle (CPU restatement of the reference shaders) on a bounded sample
  e2e           the same metric through the host-buffer entry point (pinned host -> device -> host)
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

BATCH_PER_GPU = 64
IMAGE = 224
RING = 16  # input buffers rotated per step: 16 x 9.6 MB = 154 MB > 126 MB of L2


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-i", str(self.gpu_index), "-lms", "50"], stdout=self.file,
                                         stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, sm_max, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                sm_max.append(float(parts[2]))
            except ValueError:
                continue
            for name, value in zip(names, parts[5:9]):
                if value.lower() == "active":
                    reasons.add(name)
        self.file.close()
        os.unlink(self.file.name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(sm_max) if sm_max else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def graph_stats(graph):
    """Algorithmic work of the unfused operator list: MACs per class and bytes (inputs read once,
    outputs written once per operator)."""
    conv_macs = other_macs = 0
    for op in graph.ops:
        out_elems = int(np.prod(op.out.shape))
        if op.name == "CONV2D":
            _, kh, kw, ic = op.inputs[1].shape
            conv_macs += out_elems * kh * kw * ic
        elif op.name == "MATMUL":
            other_macs += out_elems * op.inputs[0].shape[2]
        elif op.name == "DEPTHWISE_CONV2D":
            kh, kw, _, _ = op.inputs[1].shape
            other_macs += out_elems * kh * kw
    return conv_macs, other_macs


class CpuReference:
    """The CPU oracle (one kernel per operator, all host threads) on a bounded sample of the benchmark
    workload: the same graph at a batch small enough that one pass takes about `target_seconds`."""

    def __init__(self, target_seconds: float):
        # torchrun gives every worker OMP_NUM_THREADS=1; the CPU arm is meant to use all host threads
        self.cores = os.cpu_count() or 1
        os.environ["OMP_NUM_THREADS"] = str(self.cores)
        from __graft_entry__ import load_package
        load_package()
        from mlel_b200.model_graphs import resnet50_graph
        from oracle import oracle
        from tests.graph_eval import evaluate
        oracle.build()
        try:  # in case the OpenMP runtime was initialised before the variable changed
            import ctypes
            ctypes.CDLL("libgomp.so.1").omp_set_num_threads(self.cores)
        except OSError:
            pass
        self.evaluate = evaluate
        g, inputs = resnet50_graph(seed=0, n=1, image=IMAGE)
        evaluate(g, inputs)  # warm-up (page-in, thread pool)
        t0 = time.perf_counter()
        evaluate(g, inputs)
        per_image = time.perf_counter() - t0
        self.n = int(max(1, min(BATCH_PER_GPU, target_seconds / max(per_image, 1e-6))))
        self.graph, self.inputs = resnet50_graph(seed=0, n=self.n, image=IMAGE)

    def step(self):
        """One pass over the sample; returns (images/s, seconds)."""
        t0 = time.perf_counter()
        self.evaluate(self.graph, self.inputs)
        dt = time.perf_counter() - t0
        return self.n / dt, dt

    def describe(self, value: float, dt: float):
        return {"value": value, "unit": "images/s", "cores": self.cores, "kind": "port",
                "sample": f"{self.n} of {BATCH_PER_GPU} images of the same graph per pass, {dt:.2f} s per pass, OpenMP "
                          f"over {self.cores} host threads"}


def cpu_reference_rate(target_seconds: float = 10.0):
    ref = CpuReference(target_seconds)
    value, dt = ref.step()
    return ref.describe(value, dt)


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, args.steps)
    # the whole run (warm-up and timed passes) is sized to about two minutes of CPU work
    ref = CpuReference(target_seconds=max(0.1, 120.0 / (steps + args.warmup)))
    for _ in range(args.warmup):
        ref.step()
    timed = [ref.step() for _ in range(steps)]
    seconds = sum(dt for _, dt in timed)
    value = ref.n * steps / seconds
    line = {
        "impl": "reference", "metric": "int8 TOSA ResNet-50 images/s", "value": value, "unit": "images/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup, "ms_per_step": 1e3 * BATCH_PER_GPU / value,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "s8 x s8 -> s32",
        "data": "synthetic",
        "config": {"workload": "BASELINE configs[3]: ResNet-50-shaped int8 TOSA graph, 224x224x3, bounded sample per step",
                   "note": "the reference has no CPU path and no Vulkan stack exists on this box; this is the CPU "
                           "restatement of its shaders (oracle/), one kernel per operator; ms_per_step is scaled to "
                           "the 64-image step of the GPU arm"},
        "cpu_baseline": ref.describe(value, seconds / steps),
        "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--batch", type=int, default=BATCH_PER_GPU, help="images per GPU (benchmark value: 64)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-int8-peak", action="store_true",
                    help="skip the 1.5 s measurement of the int8 tensor-pipe rate (the roofline denominator)")
    ap.add_argument("--no-graph", action="store_true",
                    help="enqueue every kernel of every step instead of replaying one captured CUDA graph per bound buffer")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return

    import torch
    import torch.distributed as dist

    from __graft_entry__ import load_package
    mlel = load_package()
    mlel.lib()  # fails loudly if the CUDA library is missing
    from mlel_b200.model_graphs import resnet50_graph
    from mlel_b200.runtime import GraphRunner
    from mlel_b200.sharding import all_gather_batch

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    W = max(3, args.warmup)
    K = args.steps
    n = args.batch

    # Every rank builds the same network (same seed => same weights) and owns its own batch.
    graph, _ = resnet50_graph(seed=0, n=n, image=IMAGE)
    runner = GraphRunner(graph, device=device)
    session = runner.session
    rng = np.random.Generator(np.random.PCG64(1000 + rank))
    in_bytes = n * IMAGE * IMAGE * 3
    host_ring = [torch.from_numpy(rng.integers(-128, 128, (in_bytes,), dtype=np.int8)).pin_memory() for _ in range(RING)]
    dev_ring = [h.to(device, non_blocking=True) for h in host_ring]
    out_dev = runner.outputs[0]
    out_bytes = out_dev.numel()
    host_out = torch.empty(out_bytes, dtype=torch.uint8).pin_memory()
    stream = torch.cuda.current_stream(device)

    # mlel_session_dispatch_graph keeps one captured CUDA graph per set of bound addresses, so rotating over the
    # ring (or over the two staging buffers of the end-to-end path) replays graphs after the first round.
    dispatch = session.dispatch if args.no_graph else session.dispatch_graph

    def step_resident(i):
        # inputs already in HBM: rebinding an external tensor is a descriptor update, not a copy
        session.set_external(0, 0, dev_ring[i % RING].data_ptr())
        dispatch(stream.cuda_stream)
        if world > 1:
            all_gather_batch(out_dev.view(n, -1), world * n)

    def step_run_host(i):
        # one call: host input -> device, dispatch, logits -> host, all in order on the dispatch stream
        session.set_external(0, 0, runner.inputs[0].data_ptr())
        session.run_host([(0, 0, 0, host_ring[i % RING].data_ptr(), in_bytes)],
                         [(0, 1, 0, host_out.data_ptr(), out_bytes)], stream.cuda_stream)
        if world > 1:
            all_gather_batch(out_dev.view(n, -1), world * n)

    # End to end the way a serving host drives the C ABI: the next batch's host -> device copy runs on a second
    # stream into the other of two device buffers while the current batch computes; every step still copies its
    # own 9.6 MB input from pinned host memory and reads its logits back to the host.
    copy_stream = torch.cuda.Stream(device)
    stage_in = [torch.empty(in_bytes, dtype=torch.int8, device=device) for _ in range(2)]
    ready = [torch.cuda.Event() for _ in range(2)]
    free = [torch.cuda.Event() for _ in range(2)]
    for ev in free:
        ev.record(stream)

    def step_e2e(i):
        b = i % 2
        copy_stream.wait_event(free[b])  # the dispatch that last read this buffer has finished
        with torch.cuda.stream(copy_stream):
            stage_in[b].copy_(host_ring[i % RING], non_blocking=True)
            ready[b].record(copy_stream)
        stream.wait_event(ready[b])
        session.set_external(0, 0, stage_in[b].data_ptr())
        dispatch(stream.cuda_stream)
        free[b].record(stream)
        host_out.copy_(out_dev, non_blocking=True)
        if world > 1:
            all_gather_batch(out_dev.view(n, -1), world * n)

    def barrier():
        torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    def timed(fn, warmup, steps):
        for i in range(warmup):
            fn(i)
        barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        copy_stream.wait_event(start)  # nothing of the timed steps starts before the clock does
        for i in range(steps):
            fn(warmup + i)
        stop.record(stream)
        barrier()
        ms = torch.tensor([start.elapsed_time(stop)], device=device)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    if not args.no_graph:
        for i in range(RING):  # untimed: every buffer of the ring has its graph before the clock starts
            step_resident(i)
    total_ms = timed(step_resident, W, K)
    clocks = sampler.stop() if rank == 0 else None
    e2e_steps = max(3, K // 2)
    e2e_ms = timed(step_e2e, 3, e2e_steps)
    run_host_ms = timed(step_run_host, 3, e2e_steps)

    # Per-kernel device time of the same graph (event pair per launch), for the roofline of the dominant kernel.
    names = runner.pipeline.exec_names()
    prof = np.zeros(len(names))
    reps = 3
    session.set_external(0, 0, dev_ring[0].data_ptr())
    session.dispatch_profiled(stream.cuda_stream)
    for r in range(reps):
        session.set_external(0, 0, dev_ring[(r + 1) % RING].data_ptr())
        prof += np.array(session.dispatch_profiled(stream.cuda_stream))
    prof /= reps
    conv_ms = float(sum(t for t, nm in zip(prof, names) if nm.startswith("CONV2D")))
    by_kind = {}
    for t, nm in zip(prof, names):
        by_kind[nm] = by_kind.get(nm, 0.0) + float(t)

    # one kernel per executed node, plus the im2col kernel in front of a convolution whose channel count is
    # not a multiple of 16 (the RGB stem)
    launches_per_dispatch = session.launch_count() + sum(
        1 for op in graph.ops if op.name == "CONV2D" and op.inputs[0].shape[3] % 16 != 0)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks = load_peaks()
    conv_macs, other_macs = graph_stats(graph)
    images = world * n * K
    value = images / (total_ms / 1e3)
    # Denominator of the tensor-bound fraction.  The machine's measured-peaks file has no int8 figure, so the rate
    # of back-to-back tcgen05.mma kind::i8 on shared-memory operands is measured here, after everything else:
    # a burst of about 10 ms (best of three) and a loop of about 1.5 s, which runs into the power cap as a
    # seconds-long matmul does.  The convolutions are timed inside a long step: the sustained figure applies.
    if args.no_int8_peak:
        int8_burst = int8_peak_tops = 2.0 * peaks["bf16_tflops_sustained"]
        peak_source = ("2 x %s sustained bf16 cuBLAS figure (%s); the int8 loop was skipped" %
                       (peaks["bf16_tflops_sustained"], peaks["source"]))
    else:
        int8_burst = max(mlel.measure_int8_mma_peak(2000, stream.cuda_stream) for _ in range(3))
        int8_peak_tops = mlel.measure_int8_mma_peak(300000, stream.cuda_stream)
        peak_source = ("measured in this run: tcgen05.mma kind::i8 128x256x32 back to back on every SM, sustained over "
                       "1.5 s (the burst figure over 10 ms is peak_burst); 2 x the measured sustained bf16 figure "
                       "would be %.0f" % (2.0 * peaks["bf16_tflops_sustained"]))
    conv_tops = 2.0 * conv_macs / (conv_ms / 1e3) / 1e12
    n_conv = sum(nm.startswith("CONV2D") for nm in names)
    line = {
        "metric": "int8 TOSA ResNet-50 images/s",
        "value": value,
        "unit": "images/s",
        "n_gpus": world,
        "steps": K,
        "warmup": W,
        "ms_per_step": total_ms / K,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "s8 x s8 -> s32",
        "data": "synthetic",
        "config": {
            "workload": "BASELINE configs[3]: ResNet-50-shaped int8 TOSA graph, N=%d images per GPU, 224x224x3" % n,
            "ops_per_dispatch": len(graph.ops), "kernels_per_dispatch": len(names),
            "gmac_per_image": (conv_macs + other_macs) / n / 1e9,
            "cache": "inputs rotate over a ring of %d device buffers (%.0f MB) larger than the 126 MB L2" %
                     (RING, RING * in_bytes / 1e6),
            "parallelism": "batch-sharded, one rank per GPU, NCCL all-gather of the logits" if world > 1 else "single GPU",
            "dispatch": "per-kernel launches" if args.no_graph else "CUDA-graph replay, one captured graph per bound input buffer",
        },
        "clocks": clocks,
        "gpu_launches": launches_per_dispatch * K * world,
        "e2e": {"value": world * n * e2e_steps / (e2e_ms / 1e3), "unit": "images/s",
                "h2d_bytes_per_step": in_bytes, "d2h_bytes_per_step": out_bytes,
                "path": "set_external + %s per step; host->device copy of the next batch on a second stream" %
                        ("dispatch" if args.no_graph else "dispatch_graph (one captured CUDA graph per staging buffer)"),
                "single_call_run_host": world * n * e2e_steps / (run_host_ms / 1e3)},
        "roofline": {
            "kernel": "fused CONV2D+RESCALE[+CLAMP] (%d launches per dispatch)" % n_conv,
            "bound": "tensor", "achieved": conv_tops, "peak": int8_peak_tops, "unit": "TOP/s",
            "frac": conv_tops / int8_peak_tops,
            "peak_burst": int8_burst,
            "peak_source": peak_source,
            "conv_ms_per_dispatch": conv_ms,
            # dram__bytes_read.sum + dram__bytes_write.sum per tensor-core launch, from the ncu capture summarised
            # in profiles/resnet50_n64_launch_list.md (1034 MB over the 54 launches of one 64-image dispatch);
            # scaled by the batch, which the activation bytes follow
            "traffic": 19.2e6 * n / 64.0,
            "algorithmic_bytes_per_launch": (1064e6 + 711e6) / 54.0 * n / 64.0,
        },
        "kernel_ms_per_dispatch": {k: round(v, 4) for k, v in sorted(by_kind.items(), key=lambda kv: -kv[1])},
    }
    if not args.no_cpu_baseline and world == 1:
        line["cpu_baseline"] = cpu_reference_rate(10.0)
    elif not args.no_cpu_baseline:
        line["cpu_baseline"] = None
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
