"""GPU parity on whole graphs through the C ABI: the reference's golden vectors replayed end to end,
the benchmark configurations (reduced sizes against the oracle, full sizes through size-independent
properties), fused against unfused execution, CUDA-graph replay, host-buffer dispatch and the
direct kernel entry points."""
import ctypes
import json
import os

import numpy as np
import pytest

from mlel_b200.graph_builder import GraphBuilder
from mlel_b200.model_graphs import (bert_graph, conv2d_rescale_graph, matmul_rescale_graph, mobilenet_v2_graph,
                                     resnet50_graph)
from tests.graph_eval import evaluate

pytestmark = pytest.mark.gpu

with open(os.path.join(os.path.dirname(__file__), "golden", "reference_goldens.json")) as f:
    GOLD = json.load(f)


def gold(name):
    g = GOLD[name]
    return np.array(g["values"], dtype=g["dtype"]).reshape(g["shape"])


def iota_i8(shape):
    return (np.arange(int(np.prod(shape))) & 0xFF).astype(np.uint8).view(np.int8).reshape(shape)


def run(g, inputs, flags=0, use_cuda_graph=False):
    from mlel_b200.runtime import GraphRunner
    return GraphRunner(g, flags=flags).run(inputs, use_cuda_graph=use_cuda_graph)


# ---- the reference's goldens, end to end (graphs restated from tests/shader/*.spvasm) ----

def test_golden_conv2d(mlel):
    g = GraphBuilder()
    x, w, b = g.input(np.int8, (1, 8, 8, 3)), g.input(np.int8, (3, 2, 2, 3)), g.input(np.int32, (3,))
    g.output(g.conv2d(x, w, b, [0] * 4, [2, 2], [1, 1], 0, 0))
    out = run(g, [iota_i8((1, 8, 8, 3)), np.ones((3, 2, 2, 3), np.int8), np.array([0, 1, 2], np.int32)])[0]
    np.testing.assert_array_equal(out, gold("Conv2D"))


def test_golden_conv2d_int64(mlel):
    g = GraphBuilder()
    x, w, b = g.input(np.int16, (1, 2, 2, 4)), g.input(np.int8, (4, 1, 1, 4)), g.input(np.int64, (4,))
    g.output(g.conv2d(x, w, b, [0] * 4, [1, 1], [1, 1], 0, 0, acc_type=4))
    out = run(g, [np.arange(1, 17, dtype=np.int16).reshape(1, 2, 2, 4),
                  np.array([1, 2, 3, 4, -1, 0, 1, 2, 2, -3, 4, -5, -2, -1, 0, 1], np.int8).reshape(4, 1, 1, 4),
                  np.array([10, -20, 30, -40], np.int64)])[0]
    np.testing.assert_array_equal(out, gold("Conv2DAccumulatorInt64"))


def test_golden_higher_rank_constant(mlel):
    g = GraphBuilder()
    x = g.input(np.int8, (1, 3, 3, 1))
    w = g.inline(np.arange(9, dtype=np.int8).reshape(1, 3, 3, 1))
    acc = g.conv2d(x, w, g.inline(np.zeros((1,), np.int32)), [1] * 4, [1, 1], [1, 1], 0, 0)
    g.output(g.cast(acc, np.int8))
    np.testing.assert_array_equal(run(g, [np.ones((1, 3, 3, 1), np.int8)])[0], gold("HigherRankConstant"))


@pytest.mark.parametrize("flags", [0, 1])
def test_golden_rescale_add_rescale(mlel, flags):
    g = GraphBuilder()
    a, b = g.input(np.int8, (5,)), g.input(np.int8, (5,))
    ta = g.rescale(a, [2], [0], 0, 0, np.int32)
    tb = g.rescale(b, [3], [0], 0, 0, np.int32)
    g.output(g.rescale(g.add(ta, tb), [4], [0], 0, 0, np.int8))
    out = run(g, [np.arange(5, dtype=np.int8)] * 2, flags)[0]
    np.testing.assert_array_equal(out, gold("GraphConstantARM"))


def _maxpool_input():
    x = np.zeros((1, 16, 16, 3), np.int8)
    x[0, :, :, 0] = (np.arange(256) - 128).astype(np.int8).reshape(16, 16)
    return x


def test_golden_maxpool(mlel):
    g = GraphBuilder()
    x = g.input(np.int8, (1, 16, 16, 3))
    g.output(g.max_pool2d(x, [2, 2], [2, 2], [0] * 4))
    np.testing.assert_array_equal(run(g, [_maxpool_input()])[0], gold("MaxPool2D"))


def test_golden_two_layer_maxpool_uses_session_memory(mlel):
    g = GraphBuilder()
    x = g.input(np.int8, (1, 16, 16, 3))
    g.output(g.max_pool2d(g.max_pool2d(x, [2, 2], [2, 2], [0] * 4), [2, 2], [2, 2], [0] * 4))
    np.testing.assert_array_equal(run(g, [_maxpool_input()])[0], gold("TwoLayerMaxPool2D"))


def test_golden_concat_slice_maximum(mlel):
    g = GraphBuilder()
    a, b = g.input(np.int8, (1, 2, 2, 2)), g.input(np.int8, (1, 2, 2, 2))
    g.output(g.concat([a, b], 1))
    np.testing.assert_array_equal(run(g, [iota_i8((1, 2, 2, 2))] * 2)[0], gold("Concat"))
    g = GraphBuilder()
    x = g.input(np.int8, (1, 8, 8, 3))
    g.output(g.slice(x, [0, 4, 4, 1], [1, 2, 2, 2]))
    np.testing.assert_array_equal(run(g, [iota_i8((1, 8, 8, 3))])[0], gold("Slice"))
    g = GraphBuilder()
    a, b = g.input(np.int32, (1, 2, 2, 2)), g.input(np.int32, (1, 2, 2, 2))
    g.output(g.binary("MAXIMUM", a, b))
    out = run(g, [np.arange(8, dtype=np.int32).reshape(1, 2, 2, 2),
                  (np.arange(8, dtype=np.int64) * 4 - 16).astype(np.int32).reshape(1, 2, 2, 2)])[0]
    np.testing.assert_array_equal(out, gold("Maximum"))


def test_golden_concat_interval_fp32(mlel):
    g = GraphBuilder()
    x, one, zero = g.input(np.float32, (3, 3)), g.input(np.float32, (3, 3)), g.input(np.float32, (3, 1))
    g.output(g.reshape(g.concat([g.add(x, one), zero], 1), (12,)))
    out = run(g, [np.arange(9, dtype=np.float32).reshape(3, 3), np.ones((3, 3), np.float32),
                  np.zeros((3, 1), np.float32)], flags=1)[0]
    np.testing.assert_array_equal(out, gold("ConcatMultipleDispatchesPreserveInputLiveRange"))


@pytest.mark.parametrize("axis", ["oc", "h", "w"])
def test_conv2d_large_dimension(mlel, axis):
    # tests/vulkan.cpp:1091-1156: sizes past the Vulkan grid limits, all ones -> every output is 4
    shapes = {"oc": ((1, 2, 2, 1), (262144, 2, 2, 1)), "h": ((1, 524281, 2, 1), (1, 2, 2, 1)),
              "w": ((1, 2, 524281, 1), (1, 2, 2, 1))}[axis]
    g = GraphBuilder()
    x, w = g.input(np.int8, shapes[0]), g.input(np.int8, shapes[1])
    g.output(g.conv2d(x, w, g.inline(np.zeros((shapes[1][0],), np.int32)) if shapes[1][0] == 1
             else g.constant(np.zeros((shapes[1][0],), np.int32)), [0] * 4, [1, 1], [1, 1], 0, 0))
    out = run(g, [np.ones(shapes[0], np.int8), np.ones(shapes[1], np.int8)])[0]
    assert (out == 4).all() and out.size >= 262144


# ---- benchmark configurations ----

@pytest.mark.parametrize("seed", range(4))
def test_config0_conv2d_rescale(mlel, seed):
    g, inputs = conv2d_rescale_graph(seed)
    want = evaluate(g, inputs)[0]
    for flags in (0, 1):
        np.testing.assert_array_equal(run(g, inputs, flags)[0], want)


@pytest.mark.parametrize("seed", range(2))
@pytest.mark.parametrize("double_round", [False, True])
def test_config1_matmul_rescale_reduced(mlel, seed, double_round):
    g, inputs = matmul_rescale_graph(seed, n=3, h=256, c=1024, w=384, double_round=double_round)
    want = evaluate(g, inputs)[0]
    for flags in (0, 1):
        np.testing.assert_array_equal(run(g, inputs, flags)[0], want)


def test_config1_full_size_properties(mlel):
    """[16,1024,1024]^2 at full size: the oracle would take minutes, so the kernel is checked through
    properties of the arithmetic: (1) a sampled set of rows against the oracle, (2) linearity of the
    int32 accumulator, acc(A, B1 + B2) == acc(A, B1) + acc(A, B2) with zero points 0."""
    from oracle import oracle
    g, (a, b) = matmul_rescale_graph(0)
    out = run(g, [a, b])[0]
    rows = np.array([0, 1, 511, 1023])
    for n in (0, 7, 15):
        sub = oracle.matmul(np.ascontiguousarray(a[n:n + 1, rows]), b[n:n + 1], -7, 0)
        mult = [op for op in g.ops if op.name == "RESCALE"][0].inputs[1].data
        want = oracle.rescale(sub, mult, np.array([38], np.int8), 0, 0, np.int8)
        np.testing.assert_array_equal(out[n, rows], want[0])
    r = np.random.Generator(np.random.PCG64(5))
    b1 = r.integers(-64, 64, b.shape, dtype=np.int8)
    b2 = r.integers(-64, 64, b.shape, dtype=np.int8)
    g2 = GraphBuilder()
    xa, xb = g2.input(np.int8, a.shape), g2.input(np.int8, b.shape)
    g2.output(g2.matmul(xa, xb, 0, 0))
    from mlel_b200.runtime import GraphRunner
    runner = GraphRunner(g2)
    s1 = runner.run([a, b1])[0].astype(np.int64)
    s2 = runner.run([a, b2])[0].astype(np.int64)
    s12 = runner.run([a, (b1 + b2).astype(np.int8)])[0].astype(np.int64)
    np.testing.assert_array_equal(s12, s1 + s2)


@pytest.mark.parametrize("seed", [0, 1])
def test_resnet_shaped_graph(mlel, seed):
    g, inputs = resnet50_graph(seed=seed, n=3, image=64, width=16, blocks=(2, 1, 2, 1), classes=24)
    want = evaluate(g, inputs)[0]
    assert want.std() > 2.0  # the check is only meaningful if outputs are not saturated or constant
    unfused = run(g, inputs, flags=1)[0]
    fused = run(g, inputs, flags=0)[0]
    replay = run(g, inputs, flags=0, use_cuda_graph=True)[0]
    np.testing.assert_array_equal(unfused, want)
    np.testing.assert_array_equal(fused, want)
    np.testing.assert_array_equal(replay, want)


def test_resnet_full_width_one_image(mlel):
    g, inputs = resnet50_graph(seed=2, n=1, image=224)
    np.testing.assert_array_equal(run(g, inputs)[0], evaluate(g, inputs)[0])


def test_resnet_intermediate_tensors(mlel):
    """Every activation of a small network is made a graph output so that a wrong value cannot be
    masked by later layers (this also disables most fusion, covering the stand-alone kernels)."""
    g, inputs = resnet50_graph(seed=3, n=2, image=32, width=8, blocks=(1, 1, 1, 1), classes=8)
    for op in list(g.ops):
        if op.name in ("CLAMP", "MAX_POOL2D", "AVG_POOL2D") and all(op.out is not v for v, _, _ in g.outputs):
            g.output(op.out)
    want = evaluate(g, inputs)
    got = run(g, inputs)
    assert len(got) > 10
    for a, b in zip(got, want):
        np.testing.assert_array_equal(a, b)


def test_mobilenet_shaped_graph(mlel):
    g, inputs = mobilenet_v2_graph(seed=0, n=2, image=64, width_div=2, classes=20)
    want = evaluate(g, inputs)[0]
    np.testing.assert_array_equal(run(g, inputs, flags=1)[0], want)
    np.testing.assert_array_equal(run(g, inputs, flags=0, use_cuda_graph=True)[0], want)


def test_mobilenet_full_width_one_image(mlel):
    """Configuration 2 at its real channel widths (24/144/960/1280 and so on) and image size, one image: fused with
    graph replay, and unfused (the reference's operator list), against the oracle."""
    g, inputs = mobilenet_v2_graph(seed=1, n=1, image=224, width_div=1)
    want = evaluate(g, inputs)[0]
    assert np.unique(want).size > 20
    np.testing.assert_array_equal(run(g, inputs, flags=0, use_cuda_graph=True)[0], want)
    np.testing.assert_array_equal(run(g, inputs, flags=1)[0], want)


def test_bert_full_width_one_layer(mlel):
    """One encoder layer of configuration 4 at its real sizes (hidden 768, 12 heads, FFN 3072, 384 tokens), one
    sequence: the projections with K = 768 and 3072, both attention products, fused and unfused."""
    g, inputs = bert_graph(seed=3, n=1, seq=384, hidden=768, heads=12, ffn=3072, layers=1)
    want = evaluate(g, inputs)[0]
    assert want.std() > 5.0 and np.unique(want).size > 50
    np.testing.assert_array_equal(run(g, inputs, flags=0)[0], want)
    np.testing.assert_array_equal(run(g, inputs, flags=1)[0], want)
    np.testing.assert_array_equal(run(g, inputs, flags=0, use_cuda_graph=True)[0], want)


def test_bert_shaped_graph(mlel):
    """Configuration 4 at reduced size: projections and both attention products on the tensor cores, the
    softmax / layer-norm chains (REDUCE_MAX, SUB, int16 TABLE, REDUCE_SUM, MUL), head split and merge
    (RESHAPE, TRANSPOSE), GELU as an int8 TABLE, rescaled residual ADDs."""
    g, inputs = bert_graph(seed=1, n=2, seq=48, hidden=64, heads=4, ffn=128, layers=2)
    want = evaluate(g, inputs)[0]
    assert want.std() > 5.0 and np.unique(want).size > 50
    np.testing.assert_array_equal(run(g, inputs, flags=1)[0], want)
    np.testing.assert_array_equal(run(g, inputs, flags=0)[0], want)
    np.testing.assert_array_equal(run(g, inputs, flags=0, use_cuda_graph=True)[0], want)


def test_bert_intermediate_tensors(mlel):
    """Every int8 and int16 tensor of one encoder layer is made a graph output, so that a wrong value in the
    attention or normalisation chains cannot be masked by later saturation."""
    g, inputs = bert_graph(seed=2, n=1, seq=32, hidden=32, heads=2, ffn=64, layers=1)
    outputs = [id(v) for v, _, _ in g.outputs]
    for op in list(g.ops):
        if op.name in ("RESCALE", "TABLE", "MUL", "REDUCE_SUM") and id(op.out) not in outputs:
            g.output(op.out)
    want = evaluate(g, inputs)
    got = run(g, inputs)
    assert len(got) > 20
    for a, b in zip(got, want):
        np.testing.assert_array_equal(a, b)


def test_batch_is_independent(mlel):
    """Batch sharding rests on this: sample i of a batched dispatch equals a batch-1 dispatch of it."""
    g4, inputs = resnet50_graph(seed=4, n=4, image=32, width=8, blocks=(1, 1, 1, 1), classes=8)
    full = run(g4, inputs)[0]
    for i in range(4):
        g1, _ = resnet50_graph(seed=4, n=1, image=32, width=8, blocks=(1, 1, 1, 1), classes=8)
        np.testing.assert_array_equal(run(g1, [inputs[0][i:i + 1]])[0][0, 0], full[0, i])


# ---- session behaviour ----

def test_run_host_and_rebinding(mlel):
    import torch
    from mlel_b200.runtime import GraphRunner
    g, inputs = conv2d_rescale_graph(1, hw=20, ic=16, oc=16)
    runner = GraphRunner(g)
    want = evaluate(g, inputs)[0]
    src = torch.from_numpy(inputs[0]).pin_memory()
    dst = torch.empty(want.shape, dtype=torch.int8).pin_memory()
    stream = torch.cuda.current_stream().cuda_stream
    for _ in range(2):
        dst.zero_()
        runner.session.run_host([(0, 0, 0, src.data_ptr(), src.numel())], [(0, 1, 0, dst.data_ptr(), dst.numel())],
                                stream)
        np.testing.assert_array_equal(dst.numpy(), want)
    # a second session of the same pipeline with its own memory gives the same answer
    s2 = mlel.Session(runner.pipeline)
    arena = torch.empty(max(1, s2.memory_requirements()[0]), dtype=torch.uint8, device="cuda")
    out2 = torch.zeros(want.size, dtype=torch.int8, device="cuda")
    s2.bind_memory(arena.data_ptr())
    s2.set_external(0, 0, runner.inputs[0].data_ptr())
    s2.set_external(0, 1, out2.data_ptr())
    s2.dispatch(stream)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(out2.cpu().numpy().reshape(want.shape), want)
    with pytest.raises(mlel.MlelError):
        runner.session.run_host([(0, 0, 0, src.data_ptr(), 3)], [], stream)


def test_unbound_tensor_is_an_error_not_a_fault(mlel):
    g, _ = conv2d_rescale_graph(1, hw=8, ic=4, oc=4)
    p = mlel.Pipeline()
    p.bind_external(0, 0, mlel.I8, g.inputs[0].shape)
    p.bind_external(0, 1, mlel.I8, g.outputs[0][0].shape)
    for cid, d in g.constants.items():
        p.add_constant(cid, d)
    p.lower_spvasm(g.spvasm())
    s = mlel.Session(p)
    with pytest.raises(mlel.MlelError) as e:
        s.dispatch(0)
    assert "not bound" in str(e.value)


def test_strided_external_tensors(mlel):
    import torch
    r = np.random.Generator(np.random.PCG64(9))
    big = r.integers(-128, 128, (2, 6, 6, 16), dtype=np.int8)
    view = big[:, :, :, :8]  # channel stride 1, pixel stride 16: an application tensor with explicit strides
    p = mlel.Pipeline()
    tin = p.bind_external(0, 0, mlel.I8, view.shape, strides=view.strides)
    tout = p.bind_external(0, 1, mlel.I8, view.shape)
    p.mark_input(tin)
    p.mark_output(tout)
    p.clamp(tin, tout, -50, 50)
    s = mlel.Session(p)
    d_in = torch.from_numpy(big).cuda()
    d_out = torch.zeros(view.shape, dtype=torch.int8, device="cuda")
    s.set_external(0, 0, d_in.data_ptr())
    s.set_external(0, 1, d_out.data_ptr())
    s.dispatch(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(d_out.cpu().numpy(), np.clip(view, -50, 50))


def test_direct_kernel_entry_points(mlel):
    import torch
    from oracle import oracle
    r = np.random.Generator(np.random.PCG64(3))
    a = r.integers(-128, 128, (2, 64, 128), dtype=np.int8)
    b = r.integers(-128, 128, (2, 128, 48), dtype=np.int8)
    mult = np.array([int(r.integers(1 << 30, 1 << 31))], np.int32)
    shift = np.array([37], np.int8)
    da, db, dm, ds = (torch.from_numpy(x).cuda() for x in (a, b, mult, shift))
    acc = torch.zeros((2, 64, 48), dtype=torch.int32, device="cuda")
    out = torch.zeros((2, 64, 48), dtype=torch.int8, device="cuda")
    T = mlel.device_tensor
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    ta, tb = T(da.data_ptr(), mlel.I8, a.shape), T(db.data_ptr(), mlel.I8, b.shape)
    tacc, tout = T(acc.data_ptr(), mlel.I32, acc.shape), T(out.data_ptr(), mlel.I8, out.shape)
    tm, ts = T(dm.data_ptr(), mlel.I32, (1,)), T(ds.data_ptr(), mlel.I8, (1,))
    lib = mlel.lib()
    mlel.check(lib.mlel_cuda_matmul(ctypes.byref(ta), ctypes.byref(tb), ctypes.byref(tacc), -7, 0, stream))
    mlel.check(lib.mlel_cuda_rescale(ctypes.byref(tacc), ctypes.byref(tout), ctypes.byref(tm), ctypes.byref(ts), 0, 3,
                                     1, 1, 0, stream))
    torch.cuda.synchronize()
    want_acc = oracle.matmul(a, b, -7, 0)
    want = oracle.rescale(want_acc, mult, shift, 0, 3, np.int8, True, True, False)
    np.testing.assert_array_equal(acc.cpu().numpy(), want_acc)
    np.testing.assert_array_equal(out.cpu().numpy(), want)
    out.zero_()
    mlel.check(lib.mlel_cuda_matmul_rescale(ctypes.byref(ta), ctypes.byref(tb), ctypes.byref(tout), -7, 0,
                                            ctypes.byref(tm), ctypes.byref(ts), 0, 3, 1, 0, 1, 0, stream))
    torch.cuda.synchronize()
    np.testing.assert_array_equal(out.cpu().numpy(), want)


def test_direct_convolution_entry_points(mlel):
    """mlel_cuda_conv2d, mlel_cuda_depthwise_conv2d and mlel_cuda_conv2d_rescale called directly, against the oracle."""
    import torch
    from oracle import oracle
    r = np.random.Generator(np.random.PCG64(11))
    T = mlel.device_tensor
    lib = mlel.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    pad, st, dl = (ctypes.c_int32 * 4)(1, 1, 1, 1), (ctypes.c_int32 * 2)(2, 2), (ctypes.c_int32 * 2)(1, 1)
    x = r.integers(-128, 128, (2, 13, 11, 24), dtype=np.int8)
    w = r.integers(-128, 128, (32, 3, 3, 24), dtype=np.int8)
    b = r.integers(-(1 << 14), 1 << 14, (32,), dtype=np.int32)
    dx, dw, db = (torch.from_numpy(a).cuda() for a in (x, w, b))
    want = oracle.conv2d(x, w, b, [1] * 4, [2, 2], [1, 1], -5, 0)
    out = torch.zeros(want.shape, dtype=torch.int32, device="cuda")
    tx, tw, tb = T(dx.data_ptr(), mlel.I8, x.shape), T(dw.data_ptr(), mlel.I8, w.shape), T(db.data_ptr(), mlel.I32, b.shape)
    mlel.check(lib.mlel_cuda_conv2d(ctypes.byref(tx), ctypes.byref(tw), ctypes.byref(tb),
                                    ctypes.byref(T(out.data_ptr(), mlel.I32, want.shape)), pad, st, dl, -5, 0, stream))
    torch.cuda.synchronize()
    np.testing.assert_array_equal(out.cpu().numpy(), want)
    # the fused form: CONV2D -> RESCALE (per channel, double rounding) -> CLAMP
    mult = r.integers(1 << 30, (1 << 31) - 1, (32,), dtype=np.int64).astype(np.int32)
    shift = r.integers(36, 42, (32,), dtype=np.int8)
    dm, ds = torch.from_numpy(mult).cuda(), torch.from_numpy(shift).cuda()
    want8 = oracle.clamp(oracle.rescale(want, mult, shift, 0, 4, np.int8, True, True, True), -10, 90)
    out8 = torch.zeros(want.shape, dtype=torch.int8, device="cuda")
    mlel.check(lib.mlel_cuda_conv2d_rescale(ctypes.byref(tx), ctypes.byref(tw), ctypes.byref(tb),
                                            ctypes.byref(T(out8.data_ptr(), mlel.I8, want.shape)), pad, st, dl, -5, 0,
                                            ctypes.byref(T(dm.data_ptr(), mlel.I32, (32,))),
                                            ctypes.byref(T(ds.data_ptr(), mlel.I8, (32,))), 0, 4, 1, 1, -10, 90, stream))
    torch.cuda.synchronize()
    np.testing.assert_array_equal(out8.cpu().numpy(), want8)
    # depthwise: weights [KH, KW, C, M]
    wd = r.integers(-128, 128, (3, 3, 24, 2), dtype=np.int8)
    bd = r.integers(-(1 << 14), 1 << 14, (48,), dtype=np.int32)
    dwd, dbd = torch.from_numpy(wd).cuda(), torch.from_numpy(bd).cuda()
    wantd = oracle.depthwise_conv2d(x, wd, bd, [1] * 4, [2, 2], [1, 1], 7, -2)
    outd = torch.zeros(wantd.shape, dtype=torch.int32, device="cuda")
    mlel.check(lib.mlel_cuda_depthwise_conv2d(ctypes.byref(tx), ctypes.byref(T(dwd.data_ptr(), mlel.I8, wd.shape)),
                                              ctypes.byref(T(dbd.data_ptr(), mlel.I32, bd.shape)),
                                              ctypes.byref(T(outd.data_ptr(), mlel.I32, wantd.shape)), pad, st, dl, 7, -2,
                                              stream))
    torch.cuda.synchronize()
    np.testing.assert_array_equal(outd.cpu().numpy(), wantd)


def test_direct_entry_points_of_the_other_operators(mlel):
    """Pools, TABLE, TRANSPOSE, CONCAT, CLAMP, an elementwise binary operator and a reduction called directly, each
    against the oracle."""
    import torch
    from oracle import oracle
    r = np.random.Generator(np.random.PCG64(12))
    T = mlel.device_tensor
    lib = mlel.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    keep = []

    def dev(a):
        t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
        keep.append(t)
        return ctypes.byref(T(t.data_ptr(), mlel.NP_TO_DTYPE[np.dtype(a.dtype)], a.shape)), t

    def out_like(a):
        return dev(np.zeros(a.shape, a.dtype))

    x = r.integers(-128, 128, (2, 12, 12, 32), dtype=np.int8)
    tx, _ = dev(x)
    i2, i4 = ctypes.c_int32 * 2, ctypes.c_int32 * 4
    want = oracle.avg_pool2d(x, [3, 3], [2, 2], [1, 1, 1, 1], -4, 7)
    to, o = out_like(want)
    mlel.check(lib.mlel_cuda_avg_pool2d(tx, to, i2(3, 3), i2(2, 2), i4(1, 1, 1, 1), -4, 7, stream))
    torch.cuda.synchronize()
    np.testing.assert_array_equal(o.cpu().numpy(), want)
    want = oracle.max_pool2d(x, [3, 3], [2, 2], [1, 1, 1, 1])
    to, o = out_like(want)
    mlel.check(lib.mlel_cuda_max_pool2d(tx, to, i2(3, 3), i2(2, 2), i4(1, 1, 1, 1), stream))
    torch.cuda.synchronize()
    np.testing.assert_array_equal(o.cpu().numpy(), want)
    table = r.integers(-128, 128, (256,), dtype=np.int8)
    tt, _ = dev(table)
    want = oracle.table(x, table)
    to, o = out_like(want)
    mlel.check(lib.mlel_cuda_table(tx, tt, to, stream))
    torch.cuda.synchronize()
    np.testing.assert_array_equal(o.cpu().numpy(), want)
    want = oracle.transpose(x, (0, 2, 3, 1))
    to, o = out_like(want)
    mlel.check(lib.mlel_cuda_transpose(tx, to, (ctypes.c_uint32 * 4)(0, 2, 3, 1), 4, stream))
    torch.cuda.synchronize()
    np.testing.assert_array_equal(o.cpu().numpy(), want)
    y = r.integers(-128, 128, (2, 12, 12, 16), dtype=np.int8)
    ty, _ = dev(y)
    want = oracle.concat([x, y, x], 3)
    to, o = out_like(want)
    ins = (ctypes.POINTER(mlel.Tensor) * 3)(ctypes.cast(tx, ctypes.POINTER(mlel.Tensor)),
                                            ctypes.cast(ty, ctypes.POINTER(mlel.Tensor)),
                                            ctypes.cast(tx, ctypes.POINTER(mlel.Tensor)))
    mlel.check(lib.mlel_cuda_concat(ins, 3, to, 3, stream))
    torch.cuda.synchronize()
    np.testing.assert_array_equal(o.cpu().numpy(), want)
    want = oracle.clamp(x, -20, 99)
    to, o = out_like(want)
    mlel.check(lib.mlel_cuda_clamp(tx, to, ctypes.c_double(-20), ctypes.c_double(99), stream))
    torch.cuda.synchronize()
    np.testing.assert_array_equal(o.cpu().numpy(), want)
    a32 = r.integers(-2**30, 2**30, (3, 40, 64), dtype=np.int32)
    b32 = r.integers(-2**30, 2**30, (3, 40, 64), dtype=np.int32)
    ta, _ = dev(a32)
    tb, _ = dev(b32)
    want = oracle.binary("SUB", a32, b32, np.dtype(np.int32))
    to, o = out_like(want)
    mlel.check(lib.mlel_cuda_binary(b"SUB", ta, tb, to, stream))
    torch.cuda.synchronize()
    np.testing.assert_array_equal(o.cpu().numpy(), want)
    want = oracle.reduce("REDUCE_SUM", a32, 2)
    to, o = out_like(want)
    mlel.check(lib.mlel_cuda_reduce(b"REDUCE_SUM", ta, to, 2, stream))
    torch.cuda.synchronize()
    np.testing.assert_array_equal(o.cpu().numpy(), want)
    with pytest.raises(mlel.MlelError):
        mlel.check(lib.mlel_cuda_binary(b"NO_SUCH_OPERATOR", ta, tb, to, stream))


def test_replicated_pattern_constant_values(mlel):
    """{1, 2} replicated over four elements reaches the kernels as {1, 2, 1, 2}
    (tests/graph/graph_ext_inst_context_tests.cpp:16-20), checked through x + k with x = 0."""
    import torch
    from tests.test_frontend import _replicated_pattern_module, lower
    text, shape = _replicated_pattern_module(4)
    p = lower(mlel, text, [(0, 0, 0, mlel.I32, shape), (0, 1, 0, mlel.I32, shape)])
    s = mlel.Session(p)
    x = torch.zeros(shape, dtype=torch.int32, device="cuda")
    y = torch.full(shape, -1, dtype=torch.int32, device="cuda")
    s.set_external(0, 0, x.data_ptr())
    s.set_external(0, 1, y.data_ptr())
    s.dispatch(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(y.cpu().numpy().reshape(-1), [1, 2, 1, 2])


def test_graph_replay_follows_rebinding(mlel):
    """mlel_session_dispatch_graph keeps one captured graph per set of bound addresses: a host that alternates
    between input (and output) buffers gets, from every replay, the result for the buffers bound at that moment."""
    import torch
    from mlel_b200.runtime import GraphRunner
    g, inputs = resnet50_graph(seed=4, n=2, image=32, width=16, blocks=(1, 1, 1, 1), classes=16)
    r = GraphRunner(g)
    rng = np.random.Generator(np.random.PCG64(9))
    batches = [rng.integers(-128, 128, inputs[0].shape, dtype=np.int8) for _ in range(3)]
    want = [evaluate(g, [b])[0] for b in batches]
    assert not np.array_equal(want[0], want[1])
    dev_in = [torch.from_numpy(b.reshape(-1).view(np.uint8)).cuda() for b in batches]
    dev_out = [torch.zeros_like(r.outputs[0]) for _ in range(2)]
    (s_in, b_in, _), (s_out, b_out, v_out) = r._in_keys[0], r._out_keys[0]
    stream = torch.cuda.current_stream().cuda_stream
    for step in range(9):  # every buffer pair comes round again after its graph was captured
        i, o = step % 3, step % 2
        r.session.set_external(s_in, b_in, dev_in[i].data_ptr())
        r.session.set_external(s_out, b_out, dev_out[o].data_ptr())
        dev_out[o].zero_()
        r.session.dispatch_graph(stream)
        torch.cuda.synchronize()
        got = dev_out[o].cpu().numpy().view(v_out.dtype).reshape(v_out.shape)
        np.testing.assert_array_equal(got, want[i])


def test_a_bounded_wait_that_runs_out_is_reported(mlel):
    """The give-up path of the kernels' bounded waits: a one-thread kernel waits about a millisecond on a barrier that
    nobody arrives at; the wait records its code, the kernel returns, the context stays usable."""
    import torch
    lib = mlel.lib()
    code = ctypes.c_int(-1)
    mlel.check(lib.mlel_selftest_wait_timeout(ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), ctypes.byref(code)))
    assert code.value == 99
    assert lib.mlel_device_error() == 0  # the self-test clears its own code
    x = torch.arange(8, device="cuda")
    assert int(x.sum().item()) == 28     # the context still answers


def test_int8_mma_peak_loop(mlel):
    """The measurement helper behind the roofline denominator: back-to-back tcgen05.mma kind::i8 on every SM.
    A B200's nominal dense int8 rate is 4.5 POP/s; a short burst must land within a factor of two of it."""
    tops = max(mlel.measure_int8_mma_peak(500) for _ in range(3))
    assert 2000.0 < tops < 6000.0, tops
