"""Benchmark of the TOSA data-graph hot path on B200.

    python bench.py --gpus N --steps K --warmup W          (N>1: launched under torchrun, one rank per GPU)
    python bench.py --impl reference ...                   (the CPU restatement of the reference, timed on host cores)

Workload: the ResNet-50-shaped int8 TOSA graph of BASELINE.json configs[3], N=64 images per GPU,
224x224x3, synthetic seeded data and random-init int8 weights.  One step = one dispatch of the whole
graph over one batch.  The graph is batch-sharded: each rank owns its own 64 images, pipeline,
constants and session memory; the only collective is an NCCL all-gather of the [64,1000] int8 logits.

Timing: a window is exactly K steps between two barriers (device synchronised on both sides), timed with
CUDA events on the dispatch stream, maximum over ranks.  Windows are repeated until about a second of
device time has been measured; the median window is reported.

Printed JSON (rank 0): metric images/s over all ranks, plus
  roofline        dominant kernel class (fused CONV2D+RESCALE): algorithmic int8 ops / measured kernel time
  cpu_baseline    the oracle (CPU restatement of the reference shaders) on a bounded sample
  e2e             the same metric with every step's input copied from pinned host memory and its logits read back
  parity_checked  the logits of the benchmarked configuration (one batch of the ring) against the oracle
  extras          (one GPU) the other BASELINE configurations and the memory-bound operators, each timed alone
  oc_sharded_matmul  (several GPUs) one MATMUL cut by output channel, joined by all-gather + interleave kernel
"""
from __future__ import annotations

import argparse
import ctypes
import json
import math
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

BATCH_PER_GPU = 64
IMAGE = 224
RING = 16  # input buffers rotated per step: 16 x 9.6 MB = 154 MB > 126 MB of L2
MIN_TIMED_SECONDS = 1.0
MAX_WINDOWS = 400


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
        sm, sm_max, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                sm_max.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for name, value in zip(names, parts[5:9]):
                if value.lower() == "active":
                    reasons.add(name)
        self.file.close()
        os.unlink(self.file.name)
        # samples "under load": the GPU idles at a few hundred watts less than it draws while the graph runs
        loaded = [s for s, w in zip(sm, power) if power and w >= 0.5 * max(power)]
        return {"sm_mhz": float(np.median(loaded)) if loaded else (float(np.median(sm)) if sm else None),
                "sm_max_mhz": max(sm_max) if sm_max else None, "reasons": sorted(reasons), "samples": len(sm),
                "samples_under_load": len(loaded), "power_w_max": max(power) if power else None}


def graph_stats(graph):
    """Algorithmic work of the unfused operator list: MACs per class (padded taps counted)."""
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
    """The CPU oracle (one kernel per operator, host threads) on a bounded sample of the benchmark workload:
    the same graph on as many images of `data` (default: the graph generator's own) as fit `target_seconds`."""

    def __init__(self, target_seconds: float, data: np.ndarray | None = None, threads: int | None = None,
                 max_images: int = BATCH_PER_GPU):
        # torchrun gives every worker OMP_NUM_THREADS=1; the CPU arm is meant to use the host threads it is given
        self.cores = threads or os.cpu_count() or 1
        os.environ["OMP_NUM_THREADS"] = str(self.cores)
        from __graft_entry__ import load_package
        load_package()
        from mlel_b200.model_graphs import resnet50_graph
        from oracle import oracle
        from tests.graph_eval import evaluate
        oracle.build()
        try:  # in case the OpenMP runtime was initialised before the variable changed
            ctypes.CDLL("libgomp.so.1").omp_set_num_threads(self.cores)
        except OSError:
            pass
        self.evaluate = evaluate
        g, inputs = resnet50_graph(seed=0, n=1, image=IMAGE)
        if data is not None:
            inputs = [data[:1]]
        evaluate(g, inputs)  # warm-up (page-in, thread pool)
        t0 = time.perf_counter()
        evaluate(g, inputs)
        per_image = time.perf_counter() - t0
        self.n = int(max(1, min(max_images, target_seconds / max(per_image, 1e-6))))
        self.graph, inputs = resnet50_graph(seed=0, n=self.n, image=IMAGE)
        self.inputs = [np.ascontiguousarray(data[:self.n])] if data is not None else inputs
        self.last_output = None

    def step(self):
        """One pass over the sample; returns (images/s, seconds)."""
        t0 = time.perf_counter()
        self.last_output = self.evaluate(self.graph, self.inputs)[0]
        dt = time.perf_counter() - t0
        return self.n / dt, dt

    def describe(self, value: float, dt: float):
        return {"value": value, "unit": "images/s", "cores": self.cores, "kind": "port",
                "sample": f"{self.n} of {BATCH_PER_GPU} images of the same graph per pass, {dt:.2f} s per pass, OpenMP "
                          f"over {self.cores} host threads"}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, args.steps)
    # the whole run (warm-up and timed passes) is sized to about a minute and a half of CPU work
    ref = CpuReference(target_seconds=max(0.1, 90.0 / (steps + args.warmup)))
    for _ in range(args.warmup):
        ref.step()
    timed = [ref.step() for _ in range(steps)]
    seconds = sum(dt for _, dt in timed)
    value = ref.n * steps / seconds
    line = {
        "impl": "reference", "metric": "int8 TOSA ResNet-50 images/s", "value": value, "unit": "images/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup, "ms_per_step": 1e3 * seconds / steps,
        "images_per_step": ref.n,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "s8 x s8 -> s32",
        "data": "synthetic",
        "config": {"workload": "BASELINE configs[3]: ResNet-50-shaped int8 TOSA graph, 224x224x3, bounded sample per step",
                   "note": "the reference has no CPU path and no Vulkan stack exists on this box; this is the CPU "
                           "restatement of its shaders (oracle/), one kernel per operator; a step is one pass over "
                           "images_per_step images (ms_per_step is the time of that pass), the value is images/s"},
        "cpu_baseline": ref.describe(value, seconds / steps),
        "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ---- the other BASELINE configurations and the memory-bound operators, each timed alone (one GPU) -----------------

SIDE_MIN_SECONDS = 0.25  # timed device time per side measurement; --only shortens it for profiler captures


def _time_dispatches(runner, stream, min_seconds=None, iters=20):
    """Median milliseconds per dispatch over windows of `iters` replays of the session's captured graph."""
    import torch
    s = stream.cuda_stream
    for _ in range(3):
        runner.session.dispatch_graph(s)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    min_seconds = SIDE_MIN_SECONDS if min_seconds is None else min_seconds
    times, total = [], 0.0
    while total < min_seconds * 1e3 and len(times) < 200:
        e0.record(stream)
        for _ in range(iters):
            runner.session.dispatch_graph(s)
        e1.record(stream)
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        times.append(ms / iters)
        total += ms
    return float(np.median(times))


def measure_extras(mlel, stream, peaks, int8_peak_tops, only=None):
    """`only` = "cfg1" | "cfg2" | "cfg4" | "ops" restricts the measurement to one part (for a profiler capture)."""
    import torch
    out = {}
    hbm = peaks["hbm_gbs"]

    want = lambda part: only is None or only == part

    # configuration 1: [16,1024,1024]^2 MATMUL + per-tensor RESCALE, two run-time inputs
    if want("cfg1"):
        out["cfg1_matmul_rescale"] = _measure_cfg1(stream, hbm, int8_peak_tops)
    if want("cfg2"):
        out["cfg2_mobilenet_v2"] = _measure_cfg2(stream)
    if want("cfg4"):
        out["cfg4_bert_base"] = _measure_cfg4(stream)
    torch.cuda.empty_cache()
    if want("ops"):
        out["memory_bound_ops"] = _measure_memory_bound_ops(stream, peaks)
    torch.cuda.empty_cache()
    return out


def _measure_cfg1(stream, hbm, int8_peak_tops):
    from mlel_b200.model_graphs import matmul_rescale_graph
    from mlel_b200.runtime import GraphRunner
    g, inputs = matmul_rescale_graph(seed=0)
    r = GraphRunner(g)
    r.set_inputs(inputs)
    ms = _time_dispatches(r, stream)
    ops = 2.0 * 16 * 1024 ** 3
    nbytes = 3 * 16 * 1024 * 1024
    # the same with twenty dispatches recorded into one CUDA graph (a host that records several dispatches into one
    # command buffer): without the per-launch cost of a graph of two kernels
    import torch
    side = torch.cuda.Stream()
    side.wait_stream(stream)
    batch = torch.cuda.CUDAGraph()
    with torch.cuda.graph(batch, stream=side):
        for _ in range(20):
            r.session.dispatch(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    batched = []
    for _ in range(7):
        e0.record(stream)
        batch.replay()
        e1.record(stream)
        torch.cuda.synchronize()
        batched.append(e0.elapsed_time(e1) / 20)
    ms20 = float(np.median(batched[2:]))
    return {
        "ms_in_one_graph_of_20": ms20, "tops_in_one_graph_of_20": ops / ms20 / 1e9,
        "frac_of_int8_peak_in_one_graph_of_20": ops / ms20 / 1e9 / int8_peak_tops,
        "workload": "BASELINE configs[1]: A,B [16,1024,1024] int8 (A_zp -7), RESCALE shift 38 -> int8; both inputs run-time",
        "ms": ms, "tops": ops / ms / 1e9, "frac_of_int8_peak": ops / ms / 1e9 / int8_peak_tops,
        "gbs": nbytes / ms / 1e6, "frac_of_hbm": nbytes / ms / 1e6 / hbm,
        "kernels": r.pipeline.exec_names(), "timing": "CUDA-graph replays back to back, inputs (32 MiB) resident"}


def _measure_cfg2(stream):
    """Configuration 2: MobileNetV2-shaped graph, 32 images."""
    from mlel_b200.model_graphs import macs_of, mobilenet_v2_graph
    from mlel_b200.runtime import GraphRunner
    g, inputs = mobilenet_v2_graph(seed=0, n=32)
    r = GraphRunner(g)
    r.set_inputs(inputs)
    ms = _time_dispatches(r, stream)
    return {"workload": "BASELINE configs[2]: MobileNetV2-shaped int8 graph, 32 images, 224x224x3",
            "ms_per_dispatch": ms, "images_per_s": 32 / ms * 1e3,
            "gmac_per_image": macs_of(g) / 32 / 1e9, "kernels_per_dispatch": len(r.pipeline.exec_names())}


def _measure_cfg4(stream):
    """Configuration 4: BERT-base-shaped encoder, 12 layers, 32 sequences of 384 tokens."""
    from mlel_b200.model_graphs import bert_graph, macs_of
    from mlel_b200.runtime import GraphRunner
    g, inputs = bert_graph(seed=0, n=32)
    r = GraphRunner(g)
    r.set_inputs(inputs)
    ms = _time_dispatches(r, stream, iters=5)
    return {"workload": "BASELINE configs[4]: BERT-base-shaped int8 encoder, 12 layers, 32 x 384 tokens",
            "ms_per_dispatch": ms, "sequences_per_s": 32 / ms * 1e3,
            "tops": 2.0 * macs_of(g) / ms / 1e9, "kernels_per_dispatch": len(r.pipeline.exec_names())}


def _measure_memory_bound_ops(stream, peaks):
    import torch
    from mlel_b200.graph_builder import GraphBuilder
    from mlel_b200.runtime import GraphRunner
    hbm = peaks["hbm_gbs"]
    # memory-bound operators: one-operator graphs on tensors larger than L2, the operator's kernel timed alone with
    # the session's per-kernel events (minimum of five); GB/s = algorithmic bytes (inputs read once, outputs
    # written once) / time
    rng = np.random.default_rng(0)
    ops_out = {}

    def run(name, g, inputs, nbytes, flags=1):
        r = GraphRunner(g, flags=flags)
        r.set_inputs(inputs)
        s = stream.cuda_stream
        for _ in range(2):
            r.session.dispatch(s)
        torch.cuda.synchronize()
        ms = min(sum(r.session.dispatch_profiled(s)) for _ in range(5))
        ops_out[name] = {"us": ms * 1e3, "gbs": nbytes / ms / 1e6, "frac_of_hbm": nbytes / ms / 1e6 / hbm}

    S = (384, 384, 384)  # the attention-score tensor of the BERT-shaped graph: 226 MB as int32
    n = int(np.prod(S))
    x32 = rng.integers(-2**20, 2**20, S, dtype=np.int32)
    row = np.ascontiguousarray(x32[:, :, :1])
    g = GraphBuilder(); x = g.input(np.int32, S)
    g.output(g.rescale(x, [1 << 30], [38], 0, 0, np.int8, True, True)); run("RESCALE i32->i8", g, [x32], n * 5)
    g = GraphBuilder(); x = g.input(np.int32, S); b = g.input(np.int32, (384, 384, 1))
    g.output(g.sub(x, b)); run("SUB i32 (one value per row)", g, [x32, row], n * 8)
    g = GraphBuilder(); x = g.input(np.int32, S)
    g.output(g.reduce("REDUCE_SUM", x, 2)); run("REDUCE_SUM i32 rows of 384", g, [x32], n * 4)
    x16 = rng.integers(-32768, 32768, S, dtype=np.int16)
    g = GraphBuilder(); x = g.input(np.int16, S)
    g.output(g.table(x, rng.integers(-32768, 32768, (513,), dtype=np.int16))); run("TABLE i16->i32", g, [x16], n * 6)
    del x32, x16

    A = (256, 112, 112, 64)  # 205 MB of int8 activations
    na = int(np.prod(A))
    x8 = rng.integers(-128, 128, A, dtype=np.int8)
    g = GraphBuilder(); x = g.input(np.int8, A)
    g.output(g.clamp(x, -20, 127)); run("CLAMP i8", g, [x8], na * 2)
    g = GraphBuilder(); x = g.input(np.int8, A)
    g.output(g.table(x, rng.integers(-128, 128, (256,), dtype=np.int8))); run("TABLE i8", g, [x8], na * 2)
    g = GraphBuilder(); x = g.input(np.int8, A)
    g.output(g.max_pool2d(x, [3, 3], [2, 2], [1, 1, 1, 1])); run("MAX_POOL2D 3x3 stride 2", g, [x8], na * 1.25)
    del x8

    T = (256, 384, 12, 64)  # 75 MB: eight BERT batches of attention heads
    xt = rng.integers(-128, 128, T, dtype=np.int8)
    g = GraphBuilder(); x = g.input(np.int8, T)
    g.output(g.transpose(x, (0, 2, 1, 3))); run("TRANSPOSE (0,2,1,3) i8", g, [xt], int(np.prod(T)) * 2)
    g = GraphBuilder(); x = g.input(np.int8, T)
    g.output(g.transpose(x, (0, 2, 3, 1))); run("TRANSPOSE (0,2,3,1) i8", g, [xt], int(np.prod(T)) * 2)

    D = (128, 112, 112, 96)  # 154 MB: a MobileNetV2 expansion layer at four times the benchmark batch
    xd = rng.integers(-128, 128, D, dtype=np.int8)
    g = GraphBuilder(); x = g.input(np.int8, D)
    w = g.constant(rng.integers(-128, 128, (3, 3, 96, 1), dtype=np.int8))
    b = g.constant(rng.integers(-1000, 1000, (96,), dtype=np.int32))
    y = g.depthwise_conv2d(x, w, b, [1] * 4, [1, 1], [1, 1], -5, 0)
    mult = rng.integers(1 << 30, 1 << 31, (96,), dtype=np.int64).astype(np.int32)
    g.output(g.rescale(y, mult, np.full(96, 36, np.int8), 0, 0, np.int8, True, True, True))
    run("DEPTHWISE_CONV2D 3x3 + RESCALE", g, [xd], int(np.prod(D)) * 2, flags=0)
    return {"peak_gbs": hbm, "peak_source": peaks["source"] + " copy bandwidth", "ops": ops_out}


def measure_oc_sharded_matmul(mlel, device, stream, rank, world):
    """One large MATMUL (constant second input, per-channel RESCALE) cut by output channel over the ranks: every
    rank multiplies all of A by its block of B's columns, the blocks are joined by one all-gather into a staging
    buffer and the library's interleave kernel, and the result is compared with the product computed whole on
    this rank."""
    import torch
    import torch.distributed as dist
    from mlel_b200.graph_builder import GraphBuilder
    from mlel_b200.runtime import GraphRunner
    from mlel_b200.sharding import all_gather_columns, shard_matmul_operands
    n, h, c, w = 4, 1024, 1024, 4096
    rng = np.random.Generator(np.random.PCG64(7))
    a = rng.integers(-128, 128, (n, h, c), dtype=np.int8)
    b = rng.integers(-128, 128, (n, c, w), dtype=np.int8)
    mult = rng.integers(1 << 30, (1 << 31) - 1, (w,), dtype=np.int64).astype(np.int32)
    shift = rng.integers(37, 40, (w,), dtype=np.int8)

    def build(bm, mu, sh):
        g = GraphBuilder()
        x = g.input(np.int8, (n, h, c))
        y = g.matmul(x, g.constant(bm), -7, 0)
        g.output(g.rescale(y, mu, sh, 0, 3, np.int8, True, True, True))
        r = GraphRunner(g, device=device)
        r.set_inputs([a])
        return r

    b_local, (mult_local, shift_local) = shard_matmul_operands(b, [mult, shift], world, rank)
    whole = build(b, mult, shift)
    part = build(b_local, mult_local, shift_local)
    s = stream.cuda_stream
    whole.session.dispatch(s)
    width_local = b_local.shape[2]

    def step():
        part.session.dispatch_graph(s)
        return all_gather_columns(part.outputs[0].view(n, h, width_local), w)

    joined = step()
    torch.cuda.synchronize(device)
    equal = bool(torch.equal(joined.view(-1), whole.outputs[0].view(joined.dtype).view(-1)))
    for _ in range(3):
        step()
    torch.cuda.synchronize(device)
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    iters = 20
    e0.record(stream)
    for _ in range(iters):
        step()
    e1.record(stream)
    torch.cuda.synchronize(device)
    ms = torch.tensor([e0.elapsed_time(e1) / iters], device=device)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    eq = torch.tensor([1 if equal else 0], device=device)
    dist.all_reduce(eq, op=dist.ReduceOp.MIN)
    ms = float(ms.item())
    return {"workload": f"A [{n},{h},{c}] x B [{n},{c},{w}] int8 (B constant) + per-channel RESCALE, B's columns cut over "
                        f"{world} ranks, all-gather + interleave kernel",
            "ms": ms, "tops": 2.0 * n * h * c * w / ms / 1e9, "equal": bool(eq.item() == 1),
            "compared_with": "the same product computed whole on each rank, byte for byte"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--batch", type=int, default=BATCH_PER_GPU, help="images per GPU (benchmark value: 64)")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU oracle (baseline and parity check)")
    ap.add_argument("--no-int8-peak", action="store_true",
                    help="skip the 1.5 s measurement of the int8 tensor-pipe rate (the roofline denominator)")
    ap.add_argument("--no-graph", action="store_true",
                    help="enqueue every kernel of every step instead of replaying one captured CUDA graph per bound buffer")
    ap.add_argument("--no-extras", action="store_true", help="skip the other configurations and the operator figures")
    ap.add_argument("--windows", type=int, default=0,
                    help="time exactly this many windows of --steps steps instead of as many as fill a second "
                         "(for a run under a profiler; the default is what a benchmark line needs)")
    ap.add_argument("--only", choices=["cfg1", "cfg2", "cfg4", "ops"],
                    help="run one of the side measurements alone and print it (a small case for a profiler capture); "
                         "not a benchmark line")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return
    if args.only:
        import torch
        from __graft_entry__ import load_package
        mlel = load_package()
        mlel.lib()
        torch.cuda.set_device(0)
        peaks = load_peaks()
        global SIDE_MIN_SECONDS
        SIDE_MIN_SECONDS = 0.01
        print(json.dumps(measure_extras(mlel, torch.cuda.current_stream(), peaks, float("nan"), only=args.only)))
        return

    import torch
    import torch.distributed as dist

    from __graft_entry__ import load_package
    mlel = load_package()
    mlel.lib()  # fails loudly if the CUDA library is missing
    from mlel_b200.model_graphs import resnet50_graph
    from mlel_b200.runtime import GraphRunner

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    torch.set_num_threads(1)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    W = max(3, args.warmup)
    K = max(1, args.steps)
    n = args.batch

    # Every rank builds the same network (same seed => same weights) and owns its own batch.
    graph, _ = resnet50_graph(seed=0, n=n, image=IMAGE)
    runner = GraphRunner(graph, device=device)
    session = runner.session
    (in_set, in_binding, _), = runner._in_keys
    (out_set, out_binding, _), = runner._out_keys
    rng = np.random.Generator(np.random.PCG64(1000 + rank))
    in_bytes = n * IMAGE * IMAGE * 3
    host_ring = [torch.from_numpy(rng.integers(-128, 128, (in_bytes,), dtype=np.int8)).pin_memory() for _ in range(RING)]
    dev_ring = [h.to(device, non_blocking=True) for h in host_ring]
    # two output buffers: the logits of step i are gathered (or copied to the host) while step i + 1 computes
    out_bufs = [runner.outputs[0], torch.zeros_like(runner.outputs[0])]
    out_bytes = out_bufs[0].numel()
    host_out = [torch.empty(out_bytes, dtype=torch.uint8).pin_memory() for _ in range(2)]
    gathered = [torch.empty(world * out_bytes, dtype=torch.uint8, device=device) for _ in range(2)]
    stream = torch.cuda.current_stream(device)
    side = torch.cuda.Stream(device)          # all-gather of the logits
    copy_stream = torch.cuda.Stream(device)   # host -> device copies of the end-to-end path
    out_done = [torch.cuda.Event() for _ in range(2)]   # dispatch that wrote out_bufs[o] has finished
    out_free = [torch.cuda.Event() for _ in range(2)]   # gather of out_bufs[o] has finished
    for ev in out_free:
        ev.record(side)

    # mlel_session_dispatch_graph keeps one captured CUDA graph per set of bound addresses, so rotating over the
    # ring (or over the staging buffers of the end-to-end path) replays graphs after the first round.
    dispatch = session.dispatch if args.no_graph else session.dispatch_graph

    def gather_logits(o):
        # on a second stream, so that a rank does not hold its next dispatch back for the slowest rank's logits
        out_done[o].record(stream)
        side.wait_event(out_done[o])
        with torch.cuda.stream(side):
            dist.all_gather_into_tensor(gathered[o], out_bufs[o])
            out_free[o].record(side)

    def run_step(i, in_ptr):
        o = i % 2
        stream.wait_event(out_free[o])  # the gather that last read this output buffer has finished
        session.set_external(in_set, in_binding, in_ptr)
        session.set_external(out_set, out_binding, out_bufs[o].data_ptr())
        dispatch(stream.cuda_stream)
        return o

    def step_resident(i):
        # inputs already in HBM: rebinding an external tensor is a descriptor update, not a copy
        o = run_step(i, dev_ring[i % RING].data_ptr())
        if world > 1:
            gather_logits(o)

    # End to end the way a serving host drives the C ABI: the next batches' host -> device copies run on a second
    # stream into three staging buffers while the current batch computes; every step still copies its own 9.6 MB
    # input from pinned host memory and reads its logits back to the host.
    STAGES = 3
    stage_in = [torch.empty(in_bytes, dtype=torch.int8, device=device) for _ in range(STAGES)]
    ready = [torch.cuda.Event() for _ in range(STAGES)]
    free = [torch.cuda.Event() for _ in range(STAGES)]
    for ev in free:
        ev.record(stream)

    def step_e2e(i):
        b = i % STAGES
        copy_stream.wait_event(free[b])  # the dispatch that last read this buffer has finished
        with torch.cuda.stream(copy_stream):
            stage_in[b].copy_(host_ring[i % RING], non_blocking=True)
            ready[b].record(copy_stream)
        stream.wait_event(ready[b])
        o = run_step(i, stage_in[b].data_ptr())
        free[b].record(stream)
        if world > 1:
            gather_logits(o)
            with torch.cuda.stream(side):
                host_out[o].copy_(out_bufs[o], non_blocking=True)
                out_free[o].record(side)
        else:
            host_out[o].copy_(out_bufs[o], non_blocking=True)

    def step_run_host(i):
        # one call: host input -> device, dispatch, logits -> host, all in order on the dispatch stream
        session.set_external(in_set, in_binding, runner.inputs[0].data_ptr())
        session.set_external(out_set, out_binding, out_bufs[0].data_ptr())
        session.run_host([(in_set, in_binding, 0, host_ring[i % RING].data_ptr(), in_bytes)],
                         [(out_set, out_binding, 0, host_out[0].data_ptr(), out_bytes)], stream.cuda_stream)

    def barrier():
        torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    def one_window(fn, first, steps):
        barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        copy_stream.wait_event(start)  # nothing of the timed steps starts before the clock does
        side.wait_event(start)
        for i in range(steps):
            fn(first + i)
        for ev in out_free:  # the last gathers and copies belong to the timed steps
            stream.wait_event(ev)
        stream.wait_stream(side)
        stop.record(stream)
        barrier()
        ms = torch.tensor([start.elapsed_time(stop)], device=device)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    def timed(fn, warmup, steps, min_seconds=MIN_TIMED_SECONDS):
        """Windows of exactly `steps` steps until `min_seconds` of device time: (median ms, all windows)."""
        for i in range(warmup):
            fn(i)
        first = one_window(fn, warmup, steps)
        count = int(min(MAX_WINDOWS, max(1, math.ceil(min_seconds * 1e3 / max(first, 1e-3)))))
        if args.windows > 0:
            count = args.windows
        ms = [first] + [one_window(fn, warmup + (k + 1) * steps, steps) for k in range(count - 1)]
        return float(np.median(ms)), ms

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    if not args.no_graph:
        for i in range(2 * RING):  # untimed: every (input, output) buffer pair has its graph before the clock starts
            step_resident(i)
    total_ms, windows = timed(step_resident, W, K)
    clocks = sampler.stop() if rank == 0 else None
    e2e_steps = max(3, K // 2)
    if not args.no_graph:
        for i in range(2 * STAGES):
            step_e2e(i)
    e2e_ms, _ = timed(step_e2e, 3, e2e_steps, min_seconds=0.5)
    run_host_ms, _ = timed(step_run_host, 3, e2e_steps, min_seconds=0.25)

    # The host -> device copy of one batch alone, all ranks at once (what the end-to-end path has to hide).
    barrier()
    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(copy_stream):
        c0.record(copy_stream)
        for i in range(10):
            stage_in[i % STAGES].copy_(host_ring[i % RING], non_blocking=True)
        c1.record(copy_stream)
    barrier()
    h2d_ms = torch.tensor([c0.elapsed_time(c1) / 10], device=device)
    if world > 1:
        dist.all_reduce(h2d_ms, op=dist.ReduceOp.MAX)
    h2d_ms = float(h2d_ms.item())

    # Per-kernel device time of the same graph (event pair per launch), for the roofline of the dominant kernel.
    names = runner.pipeline.exec_names()
    prof = np.zeros(len(names))
    reps = 3
    session.set_external(out_set, out_binding, out_bufs[0].data_ptr())
    session.set_external(in_set, in_binding, dev_ring[0].data_ptr())
    session.dispatch_profiled(stream.cuda_stream)
    for r in range(reps):
        session.set_external(in_set, in_binding, dev_ring[(r + 1) % RING].data_ptr())
        prof += np.array(session.dispatch_profiled(stream.cuda_stream))
    prof /= reps
    conv_ms = float(sum(t for t, nm in zip(prof, names) if nm.startswith("CONV2D")))
    by_kind = {}
    for t, nm in zip(prof, names):
        by_kind[nm] = by_kind.get(nm, 0.0) + float(t)

    # Parity of the benchmarked configuration: the logits of ring buffer 0 as the timed path computes them (graph
    # replay, 64 images), against the CPU oracle on the same images.  One GPU: as many of the 64 images as the oracle
    # evaluates for the CPU baseline (all of them where it takes about ten seconds); several GPUs: every rank checks
    # 64 / world images of its own batch with its share of the host threads.
    parity = None
    cpu_baseline = None
    if not args.no_cpu_baseline:
        run_step(0, dev_ring[0].data_ptr())
        torch.cuda.synchronize(device)
        gpu_logits = out_bufs[0].cpu().numpy().view(np.int8).reshape(n, -1)
        data = host_ring[0].numpy().reshape(n, IMAGE, IMAGE, 3)
        threads = max(1, (os.cpu_count() or 1) // world)
        ref = CpuReference(10.0 if world == 1 else 20.0, data=data, threads=threads,
                           max_images=n if world == 1 else max(1, n // world))
        value, dt = ref.step()
        cpu_logits = np.asarray(ref.last_output).reshape(ref.n, -1)
        equal = bool(np.array_equal(gpu_logits[:ref.n], cpu_logits))
        images = ref.n
        if world > 1:
            t = torch.tensor([1 if equal else 0, images], device=device)
            dist.all_reduce(t[0:1], op=dist.ReduceOp.MIN)
            dist.all_reduce(t[1:2], op=dist.ReduceOp.SUM)
            equal, images = bool(t[0].item() == 1), int(t[1].item())
        parity = {"images": images, "of": world * n, "equal": equal,
                  "what": "int8 logits of one timed batch per rank (CUDA-graph replay) against the CPU oracle, byte for byte"}
        if world == 1:
            cpu_baseline = ref.describe(value, dt)

    oc_sharded = None
    if world > 1:
        oc_sharded = measure_oc_sharded_matmul(mlel, device, stream, rank, world)

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
    value = world * n * K / (total_ms / 1e3)
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
    # the same operations against the share of a back-to-back step that the convolutions hold (per-kernel events
    # serialise the launches and switch off their overlap, so the sum above is larger than a step)
    conv_share = conv_ms / max(float(prof.sum()), 1e-9)
    conv_tops_b2b = 2.0 * conv_macs / (total_ms / K * conv_share / 1e3) / 1e12
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
            "parallelism": ("batch-sharded, one rank per GPU, NCCL all-gather of the logits on a second stream "
                            "(two output buffers)") if world > 1 else "single GPU",
            "dispatch": "per-kernel launches" if args.no_graph else "CUDA-graph replay, one captured graph per bound buffer pair",
            "timing": "%d windows of exactly %d steps (barrier and device synchronisation on both sides of each), "
                      "median window reported; windows span %.2f-%.2f ms" % (len(windows), K, min(windows), max(windows)),
        },
        "clocks": clocks,
        "gpu_launches": launches_per_dispatch * K * world,
        "e2e": {"value": world * n * e2e_steps / (e2e_ms / 1e3), "unit": "images/s",
                "h2d_bytes_per_step": in_bytes, "d2h_bytes_per_step": out_bytes,
                "path": "set_external + %s per step; host->device copies of the next batches on a second stream into "
                        "three staging buffers, logits read back from two alternating output buffers" %
                        ("dispatch" if args.no_graph else "dispatch_graph"),
                "h2d_ms": h2d_ms,
                "h2d_note": "one batch's pinned host->device copy timed alone, all ranks copying at once, max over ranks",
                "single_call_run_host": world * n * e2e_steps / (run_host_ms / 1e3)},
        "roofline": {
            "kernel": "fused CONV2D+RESCALE[+CLAMP] (%d launches per dispatch)" % n_conv,
            "bound": "tensor", "achieved": conv_tops, "peak": int8_peak_tops, "unit": "TOP/s",
            "frac": conv_tops / int8_peak_tops,
            "achieved_back_to_back": conv_tops_b2b, "frac_back_to_back": conv_tops_b2b / int8_peak_tops,
            "back_to_back_note": "the same operations / (ms_per_step x the convolutions' share of the per-kernel times)",
            "peak_burst": int8_burst,
            "peak_source": peak_source,
            "conv_ms_per_dispatch": conv_ms,
            # dram__bytes_read.sum + dram__bytes_write.sum per tensor-core launch: 1034 MB over the 54 launches of one
            # 64-image dispatch in an earlier ncu capture, scaled by the batch (the activation bytes follow it)
            "traffic": 19.2e6 * n / 64.0,
            "traffic_source": "ncu capture of an earlier build, not measured by this run",
            "algorithmic_bytes_per_launch": (1064e6 + 711e6) / 54.0 * n / 64.0,
        },
        "kernel_ms_per_dispatch": {k: round(v, 4) for k, v in sorted(by_kind.items(), key=lambda kv: -kv[1])},
        "parity_checked": parity,
    }
    if oc_sharded is not None:
        line["oc_sharded_matmul"] = oc_sharded
    if not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline
    if world == 1 and not args.no_extras:
        line["extras"] = measure_extras(mlel, stream, peaks, int8_peak_tops)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    if parity is not None and not parity["equal"]:
        sys.exit(3)


if __name__ == "__main__":
    main()
