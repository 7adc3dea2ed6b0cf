"""Per-operator bandwidth of the memory-bound kernels on the current GPU.

Each line is a one-operator graph dispatched through the C ABI on tensors larger than the L2 cache (where the
operator's shape allows), timed on the device with the session's per-kernel events (minimum of five runs after
two warm-up dispatches).  Bandwidth = algorithmic bytes (inputs read once, outputs written once) / time,
against the measured copy bandwidth of the machine (``MEASURED_PEAKS.json`` beside the repository root, else
6538 GB/s).

Run from the repository root:  python ai-ml-emulation-layer-for-vulkan_b200/op_bench.py
One tensor-core convolution alone:  op_bench.py --conv|--residual IMAGES SIZE IN_CHANNELS OUT_CHANNELS [KERNEL]
"""
import json
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from __graft_entry__ import load_package  # noqa: E402

mlel = load_package()
mlel.lib()
from mlel_b200.graph_builder import GraphBuilder  # noqa: E402
from mlel_b200.runtime import GraphRunner  # noqa: E402


def peak_gbs() -> float:
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"])
    except (OSError, KeyError, ValueError):
        return 6538.0


PEAK = peak_gbs()


def run(name, g, inputs, nbytes, flags=1):
    r = GraphRunner(g, flags=flags)
    r.set_inputs(inputs)
    s = torch.cuda.current_stream().cuda_stream
    for _ in range(2):
        r.session.dispatch(s)
    torch.cuda.synchronize()
    ms = min(sum(r.session.dispatch_profiled(s)) for _ in range(5))
    gbs = nbytes / ms / 1e6
    print(f"{name:36s} {ms * 1e3:9.1f} us  {gbs:8.0f} GB/s  {gbs / PEAK * 100:5.1f} % of {PEAK:.0f} GB/s  "
          f"{'+'.join(r.pipeline.exec_names())}")


def main():
    rng = np.random.default_rng(0)
    S = (384, 384, 384)  # the attention-score tensor of the BERT-shaped graph: 226 MB as int32
    n = int(np.prod(S))
    x32 = rng.integers(-2**20, 2**20, S, dtype=np.int32)
    row = np.ascontiguousarray(x32[:, :, :1])

    g = GraphBuilder(); x = g.input(np.int32, S)
    g.output(g.rescale(x, [1 << 30], [38], 0, 0, np.int8, True, True)); run("RESCALE i32->i8", g, [x32], n * 5)
    g = GraphBuilder(); x = g.input(np.int32, S)
    g.output(g.rescale(x, [1 << 30], [38], 0, 0, np.int16, True, True)); run("RESCALE i32->i16", g, [x32], n * 6)
    g = GraphBuilder(); x = g.input(np.int32, S); b = g.input(np.int32, (384, 384, 1))
    g.output(g.sub(x, b)); run("SUB i32, one value per row", g, [x32, row], n * 8)
    g = GraphBuilder(); x = g.input(np.int32, S); b = g.input(np.int32, (384, 384, 1))
    g.output(g.mul(x, b, 22)); run("MUL i32 shift 22, one value per row", g, [x32, row], n * 8)
    g = GraphBuilder(); x = g.input(np.int32, S)
    g.output(g.reduce("REDUCE_SUM", x, 2)); run("REDUCE_SUM i32, rows of 384", g, [x32], n * 4)
    g = GraphBuilder(); x = g.input(np.int32, S)
    g.output(g.reduce("REDUCE_MAX", x, 2)); run("REDUCE_MAX i32, rows of 384", g, [x32], n * 4)
    x16 = rng.integers(-32768, 32768, S, dtype=np.int16)
    g = GraphBuilder(); x = g.input(np.int16, S)
    g.output(g.table(x, rng.integers(-32768, 32768, (513,), dtype=np.int16))); run("TABLE i16->i32", g, [x16], n * 6)

    A = (256, 112, 112, 64)  # 205 MB of int8 activations
    na = int(np.prod(A))
    x8 = rng.integers(-128, 128, A, dtype=np.int8)
    g = GraphBuilder(); x = g.input(np.int8, A)
    g.output(g.clamp(x, -20, 127)); run("CLAMP i8", g, [x8], na * 2)
    g = GraphBuilder(); x = g.input(np.int8, A)
    g.output(g.table(x, rng.integers(-128, 128, (256,), dtype=np.int8))); run("TABLE i8", g, [x8], na * 2)
    g = GraphBuilder(); x = g.input(np.int8, A)
    g.output(g.max_pool2d(x, [3, 3], [2, 2], [1, 1, 1, 1])); run("MAX_POOL2D 3x3 stride 2", g, [x8], na * 1.25)

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

    B = (16, 1024, 1024)  # configuration 1's second operand
    g = GraphBuilder(); a = g.input(np.int8, B); b2 = g.input(np.int8, B)
    y = g.rescale(g.matmul(a, b2, -7, 0), [1 << 30], [38], 0, 0, np.int8, True, False)
    g.output(y)
    xa = rng.integers(-128, 128, B, dtype=np.int8)
    r = GraphRunner(g); r.set_inputs([xa, xa]); s = torch.cuda.current_stream().cuda_stream
    for _ in range(2):
        r.session.dispatch(s)
    torch.cuda.synchronize()
    ms = min(sum(r.session.dispatch_profiled(s)) for _ in range(5))
    print(f"{'MATMUL [16,1024,1024]^2 + RESCALE':36s} {ms * 1e3:9.1f} us  {2 * 16 * 1024**3 / ms / 1e9:8.0f} TOP/s "
          f"(transpose and product)  {'+'.join(r.pipeline.exec_names())}")


def one_convolution(n, hw, ic, oc, k, residual):
    """One fused int8 convolution of ``n`` images of ``hw`` x ``hw`` x ``ic`` (1x1 or 3x3, per-channel
    double-round RESCALE), optionally with the fused residual tail, timed alone: the probe behind the per-layer
    figures of the design notes and the single-layer profiles."""
    from mlel_b200.model_graphs import _Net, _rng
    rng = _rng(0)
    g = GraphBuilder("one_convolution")
    net = _Net(g, rng)
    x = g.input(np.int8, (n, hw, hw, ic))
    inputs = [rng.integers(-128, 128, (n, hw, hw, ic), dtype=np.int8)]
    if residual:
        sc = g.input(np.int8, (n, hw, hw, oc))
        t = net.conv(x, -20, oc, k, 1, k // 2, -7, None)
        g.output(net.residual_add(t, -7, sc, -20, -20, (-20, 127)))
        inputs.append(rng.integers(-128, 128, (n, hw, hw, oc), dtype=np.int8))
    else:
        g.output(net.conv(x, -20, oc, k, 1, k // 2, -20, (-20, 127)))
    r = GraphRunner(g)
    r.set_inputs(inputs)
    s = torch.cuda.current_stream().cuda_stream
    for _ in range(3):
        r.session.dispatch(s)
    torch.cuda.synchronize()
    ms = min(sum(r.session.dispatch_profiled(s)) for _ in range(5))
    ops = 2.0 * n * hw * hw * oc * k * k * ic
    print(f"{'+'.join(r.pipeline.exec_names())}: {ms * 1e3:.1f} us, {ops / ms / 1e9:.0f} TOP/s, "
          f"{n * hw * hw * oc / ms / 1e6:.0f} G outputs/s")


if __name__ == "__main__":
    if len(sys.argv) > 1 and sys.argv[1] in ("--conv", "--residual"):
        # op_bench.py --conv|--residual IMAGES SIZE IN_CHANNELS OUT_CHANNELS [KERNEL]
        a = [int(v) for v in sys.argv[2:]]
        one_convolution(a[0], a[1], a[2], a[3], a[4] if len(a) > 4 else 1, sys.argv[1] == "--residual")
    else:
        main()
