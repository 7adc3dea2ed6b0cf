"""Seeded synthetic int8 TOSA graphs with the shapes of the benchmark configurations.

No dataset or trained checkpoint is involved: weights, biases and RESCALE parameters are drawn
from one ``numpy.random.Generator(PCG64(seed))`` in a fixed order (weights, bias, multipliers,
shifts, layer by layer).  Graphs are expressed with ``GraphBuilder`` and enter the library as
SPIR-V assembly text.

Quantised building blocks follow the usual TOSA lowering of an int8 network:
  conv      CONV2D (int8 x int8 -> int32, input zero point = zero point of the producer)
            -> RESCALE (per-channel int32 multiplier / int8 shift, double rounding, -> int8)
            -> CLAMP (ReLU / ReLU6 in the quantised domain), when an activation follows
  residual  RESCALE(a: int8 -> int32), RESCALE(b: int8 -> int32), ADD (int32), RESCALE (-> int8), CLAMP
            (the pattern of the reference's tests/shader/graph-constant-arm.spvasm)
"""
from __future__ import annotations

import math

import numpy as np

from .graph_builder import GraphBuilder, Value


def _rng(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(seed))


def _data_rng(seed: int) -> np.random.Generator:
    """Input data come from their own stream so that the weights do not depend on the batch size."""
    return np.random.Generator(np.random.PCG64(seed + 7919))


def _calibrated_shift(k_elems: int) -> int:
    """A shift that keeps a random int8 x int8 contraction of length k inside the int8 range.

    Products of two uniform int8 values have a standard deviation of about 5460; the sum of k of
    them about 5460 * sqrt(k).  With a multiplier in [2^30, 2^31) the result is scaled to a
    standard deviation of roughly 24..48, so outputs are spread over the int8 range instead of
    being saturated."""
    sigma = 5460.0 * math.sqrt(max(k_elems, 1))
    return min(62, 30 + max(1, int(math.ceil(math.log2(sigma / 32.0)))))


class _Net:
    def __init__(self, g: GraphBuilder, rng: np.random.Generator, calibrated: bool = True):
        self.g, self.rng, self.calibrated = g, rng, calibrated

    def conv(self, x: Value, in_zp: int, oc: int, k: int, stride: int, pad: int, out_zp: int, relu=None,
             depthwise: bool = False):
        g, rng = self.g, self.rng
        ic = x.shape[3]
        if depthwise:
            w = g.constant(rng.integers(-128, 128, (k, k, ic, 1), dtype=np.int8))
            oc = ic
            klen = k * k
        else:
            w = g.constant(rng.integers(-128, 128, (oc, k, k, ic), dtype=np.int8))
            klen = k * k * ic
        bias = g.constant(rng.integers(-(1 << 14), (1 << 14) + 1, (oc,), dtype=np.int32))
        mult = rng.integers(1 << 30, (1 << 31) - 1, (oc,), dtype=np.int64).astype(np.int32)
        if self.calibrated:
            base = _calibrated_shift(klen)
            shift = rng.integers(base, base + 2, (oc,), dtype=np.int8)
        else:
            shift = rng.integers(32, 41, (oc,), dtype=np.int8)
        p, s = [pad] * 4, [stride] * 2
        if depthwise:
            y = g.depthwise_conv2d(x, w, bias, p, s, [1, 1], in_zp, 0)
        else:
            y = g.conv2d(x, w, bias, p, s, [1, 1], in_zp, 0)
        y = g.rescale(y, mult, shift, 0, out_zp, np.int8, scale32=True, double_round=True, per_channel=True)
        if relu is not None:
            y = g.clamp(y, relu[0], relu[1])
        return y

    def residual_add(self, a: Value, a_zp: int, b: Value, b_zp: int, out_zp: int, relu=None):
        g, rng = self.g, self.rng
        ma = int(rng.integers(1 << 30, (1 << 31) - 1))
        mb = int(rng.integers(1 << 30, (1 << 31) - 1))
        mo = int(rng.integers(1 << 30, (1 << 31) - 1))
        # int8 -> int32 with 8 fractional bits (x * m >> 23 ~ x * 128..256), sum, back by >> 40
        ta = g.rescale(a, [ma], [23], a_zp, 0, np.int32)
        tb = g.rescale(b, [mb], [23], b_zp, 0, np.int32)
        s = g.add(ta, tb)
        y = g.rescale(s, [mo], [40], 0, out_zp, np.int8, double_round=True)
        if relu is not None:
            y = g.clamp(y, relu[0], relu[1])
        return y


def conv2d_rescale_graph(seed: int = 0, n=1, hw=56, ic=64, oc=64, k=3, stride=1, pad=1, in_zp=-3, out_zp=5,
                         fuse_friendly=True):
    """Configuration 0: one int8 CONV2D + per-channel double-round RESCALE.

    Input NHWC [1,56,56,64] int8, weights OHWI [64,3,3,64], bias int32 in [-2^14, 2^14], multiplier
    in [2^30, 2^31-1], shift in [32, 40], output zero point 5."""
    rng = _rng(seed)
    g = GraphBuilder("conv2d_rescale")
    x = g.input(np.int8, (n, hw, hw, ic))
    data = rng.integers(-128, 128, (n, hw, hw, ic), dtype=np.int8)
    w = g.constant(rng.integers(-128, 128, (oc, k, k, ic), dtype=np.int8))
    bias = g.constant(rng.integers(-(1 << 14), (1 << 14) + 1, (oc,), dtype=np.int32))
    mult = rng.integers(1 << 30, (1 << 31) - 1, (oc,), dtype=np.int64).astype(np.int32)
    shift = rng.integers(32, 41, (oc,), dtype=np.int8)
    y = g.conv2d(x, w, bias, [pad] * 4, [stride] * 2, [1, 1], in_zp, 0)
    y = g.rescale(y, mult, shift, 0, out_zp, np.int8, scale32=True, double_round=True, per_channel=True)
    g.output(y)
    return g, [data]


def matmul_rescale_graph(seed: int = 0, n=16, h=1024, c=1024, w=1024, zp_a=-7, zp_b=0, double_round=False):
    """Configuration 1: batched int8 MATMUL + per-tensor RESCALE (shift 38)."""
    rng = _rng(seed)
    g = GraphBuilder("matmul_rescale")
    a = g.input(np.int8, (n, h, c))
    b = g.input(np.int8, (n, c, w))
    da = rng.integers(-128, 128, (n, h, c), dtype=np.int8)
    db = rng.integers(-128, 128, (n, c, w), dtype=np.int8)
    mult = int(rng.integers(1 << 30, 1 << 31))
    y = g.matmul(a, b, zp_a, zp_b)
    y = g.rescale(y, [mult], [38], 0, 0, np.int8, scale32=True, double_round=double_round)
    g.output(y)
    return g, [da, db]


def resnet50_graph(seed: int = 0, n: int = 64, image: int = 224, width: int = 64, blocks=(3, 4, 6, 3),
                   classes: int = 1000):
    """Configuration 3: ResNet-50-shaped int8 graph (7x7/2 stem, 3x3/2 max pool, bottlenecks with the
    stride on the 3x3 convolution, 7x7 average pool, MATMUL classifier).  ``width``/``image``/
    ``blocks`` shrink the network for tests; the benchmark uses the defaults."""
    rng = _rng(seed)
    g = GraphBuilder("resnet50")
    net = _Net(g, rng)
    x = g.input(np.int8, (n, image, image, 3))
    data = _data_rng(seed).integers(-128, 128, (n, image, image, 3), dtype=np.int8)
    zp = -20  # zero point of every post-ReLU activation; ReLU = CLAMP(zp, 127)
    relu = (zp, 127)
    y = net.conv(x, -3, width, 7, 2, 3, zp, relu)
    y = g.max_pool2d(y, [3, 3], [2, 2], [1, 1, 1, 1])
    in_ch = width
    for stage, count in enumerate(blocks):
        mid = width << stage
        out_ch = mid * 4
        for b in range(count):
            stride = 2 if (b == 0 and stage > 0) else 1
            if b == 0:
                shortcut = net.conv(y, zp, out_ch, 1, stride, 0, 3, None)
                sc_zp = 3
            else:
                shortcut, sc_zp = y, zp
            t = net.conv(y, zp, mid, 1, 1, 0, zp, relu)
            t = net.conv(t, zp, mid, 3, stride, 1, zp, relu)
            t = net.conv(t, zp, out_ch, 1, 1, 0, -7, None)
            y = net.residual_add(t, -7, shortcut, sc_zp, zp, relu)
            in_ch = out_ch
    hw = y.shape[1]
    y = g.avg_pool2d(y, [hw, hw], [hw, hw], [0, 0, 0, 0], zp, zp)
    y = g.reshape(y, (1, n, in_ch))
    wfc = g.constant(rng.integers(-128, 128, (1, in_ch, classes), dtype=np.int8))
    y = g.matmul(y, wfc, zp, 0)
    mult = rng.integers(1 << 30, (1 << 31) - 1, (classes,), dtype=np.int64).astype(np.int32)
    shift = np.full((classes,), _calibrated_shift(in_ch) - 3, np.int8)
    y = g.rescale(y, mult, shift, 0, 0, np.int8, scale32=True, double_round=True, per_channel=True)
    g.output(y)
    return g, [data]


def mobilenet_v2_graph(seed: int = 0, n: int = 32, image: int = 224, width_div: int = 1, classes: int = 1000):
    """Configuration 2: MobileNetV2-shaped int8 graph: 3x3/2 stem to 32 channels, 17 inverted-residual
    blocks (expansion 6: 1x1 CONV2D, 3x3 DEPTHWISE_CONV2D, 1x1 CONV2D), 1x1 to 1280, 7x7 AVG_POOL2D and a
    1x1 CONV2D classifier.  ReLU6 is CLAMP(zp, q(6)); RESCALE multipliers/shifts use the
    configuration-0 ranges."""
    rng = _rng(seed)
    g = GraphBuilder("mobilenet_v2")
    net = _Net(g, rng, calibrated=False)
    x = g.input(np.int8, (n, image, image, 3))
    data = _data_rng(seed).integers(-128, 128, (n, image, image, 3), dtype=np.int8)
    zp, q6 = -128, 64  # activation zero point and the quantised value of 6.0
    relu6 = (zp, q6)

    def ch(c):
        return max(8, c // width_div)

    y = net.conv(x, -3, ch(32), 3, 2, 1, zp, relu6)
    settings = [(1, 16, 1, 1), (6, 24, 2, 2), (6, 32, 3, 2), (6, 64, 4, 2), (6, 96, 3, 1), (6, 160, 3, 2),
                (6, 320, 1, 1)]
    y_zp = zp
    for t, c, reps, s in settings:
        for i in range(reps):
            stride = s if i == 0 else 1
            inp, inp_zp = y, y_zp
            h = y
            if t != 1:
                h = net.conv(h, y_zp, inp.shape[3] * t, 1, 1, 0, zp, relu6)
                h_zp = zp
            else:
                h_zp = y_zp
            h = net.conv(h, h_zp, 0, 3, stride, 1, zp, relu6, depthwise=True)
            h = net.conv(h, zp, ch(c), 1, 1, 0, 4, None)
            if stride == 1 and inp.shape[3] == ch(c):
                y = net.residual_add(h, 4, inp, inp_zp, 4, None)
            else:
                y = h
            y_zp = 4
    y = net.conv(y, y_zp, ch(1280), 1, 1, 0, zp, relu6)
    hw = y.shape[1]
    y = g.avg_pool2d(y, [hw, hw], [hw, hw], [0, 0, 0, 0], zp, zp)
    y = net.conv(y, zp, classes, 1, 1, 0, 0, None)
    g.output(y)
    return g, [data]


def _lut16(fn) -> np.ndarray:
    """513-entry int16 table for TABLE on int16 inputs: entry i is the function at input (i - 256) * 128."""
    x = (np.arange(513, dtype=np.float64) - 256.0) * 128.0
    return np.clip(np.round(fn(x)), -32768, 32767).astype(np.int16)


def bert_graph(seed: int = 0, n: int = 32, seq: int = 384, hidden: int = 768, heads: int = 12, ffn: int = 3072,
               layers: int = 12):
    """Configuration 4: BERT-base-shaped int8 encoder stack (random int8 weights, zero points 0).

    Per layer: Q/K/V/output/FFN projections as int8 MATMUL + per-channel RESCALE; attention scores as a batched
    int8 MATMUL of two activations, softmax as REDUCE_MAX, SUB, int16 TABLE (exp), REDUCE_SUM, int16 TABLE
    (reciprocal) and MUL; the context as a second activation MATMUL; GELU as an int8 TABLE; layer norm as
    REDUCE_SUM, MUL, SUB and an int16 TABLE (reciprocal square root); residual ADDs on int32 with RESCALE on both
    sides.  ``n``/``seq``/``hidden``/``heads``/``ffn``/``layers`` shrink the stack for tests."""
    rng = _rng(seed)
    g = GraphBuilder("bert")
    d = hidden // heads
    rows = n * seq
    x = g.input(np.int8, (1, rows, hidden))
    data = _data_rng(seed).integers(-128, 128, (1, rows, hidden), dtype=np.int8)
    exp_lut = _lut16(lambda v: 32767.0 * np.exp(np.minimum(v, 0.0) / 4096.0))
    recip_lut = _lut16(lambda v: 32767.0 * 256.0 / (v + 32768.0 + 256.0))
    rsqrt_lut = _lut16(lambda v: 32767.0 * 16.0 / np.sqrt(v + 32768.0 + 256.0))
    gelu_lut = np.clip(np.round([0.5 * v * (1.0 + math.erf(v / 32.0 / math.sqrt(2.0))) for v in range(-128, 128)]),
                       -128, 127).astype(np.int8)

    def project(t, cin, cout, out_zp=0):
        w = g.constant(rng.integers(-128, 128, (1, cin, cout), dtype=np.int8))
        mult = rng.integers(1 << 30, (1 << 31) - 1, (cout,), dtype=np.int64).astype(np.int32)
        shift = np.full((cout,), _calibrated_shift(cin), np.int8)
        y = g.matmul(t, w, 0, 0)
        return g.rescale(y, mult, shift, 0, out_zp, np.int8, scale32=True, double_round=True, per_channel=True)

    def to32(t, shift=24):
        return g.rescale(t, [1 << 30], [shift], 0, 0, np.int32)

    def layer_norm(t32):
        # t32: int32 [1, rows, hidden] with about 6 fractional bits
        total = g.reduce("REDUCE_SUM", t32, 2)
        inv = g.inline(np.asarray([(1 << 20) // hidden], np.int32).reshape(1, 1, 1))
        mean = g.mul(total, inv, 20)
        cen = g.sub(t32, mean)
        var = g.mul(g.reduce("REDUCE_SUM", g.mul(cen, cen, 8), 2), inv, 20)
        var16 = g.rescale(var, [1 << 30], [34], 0, -32768, np.int16)
        rs = g.table(var16, rsqrt_lut)
        normed = g.mul(cen, rs, 12)
        # cen / rms(cen) arrives with 20 fractional bits (13 from the look-up's scale, 7 from its interpolation)
        return g.rescale(normed, [1 << 30], [45], 0, 0, np.int8, double_round=True)

    for _ in range(layers):
        q, k, v = project(x, hidden, hidden), project(x, hidden, hidden), project(x, hidden, hidden)
        q = g.reshape(g.transpose(g.reshape(q, (n, seq, heads, d)), (0, 2, 1, 3)), (n * heads, seq, d))
        k = g.reshape(g.transpose(g.reshape(k, (n, seq, heads, d)), (0, 2, 3, 1)), (n * heads, d, seq))
        v = g.reshape(g.transpose(g.reshape(v, (n, seq, heads, d)), (0, 2, 1, 3)), (n * heads, seq, d))
        scores = g.matmul(q, k, 0, 0)                                   # int32 [n*heads, seq, seq]
        diff = g.sub(scores, g.reduce("REDUCE_MAX", scores, 2))         # <= 0
        diff16 = g.rescale(diff, [1 << 30], [30 + max(1, int(math.log2(d)) - 2)], 0, 0, np.int16)
        e = g.table(diff16, exp_lut)                                    # int32, 7 extra fractional bits
        denom = g.reduce("REDUCE_SUM", e, 2)
        denom16 = g.rescale(denom, [1 << 30], [30 + 7 + max(1, int(math.ceil(math.log2(seq))))], 0, -32768, np.int16)
        r = g.table(denom16, recip_lut)
        log_seq = max(1, int(math.ceil(math.log2(seq))))
        # e * r >> 22 is the probability with 15 + log2(seq) fractional bits; keep 8 of them
        probs = g.rescale(g.mul(e, r, 22), [1 << 30], [30 + 7 + log_seq], 0, -128, np.int8)
        ctx = g.matmul(probs, v, -128, 0)
        ctx = g.rescale(ctx, [int(rng.integers(1 << 30, 1 << 31))], [39], 0, 0, np.int8, double_round=True)
        ctx = g.reshape(g.transpose(g.reshape(ctx, (n, heads, seq, d)), (0, 2, 1, 3)), (1, rows, hidden))
        attn = project(ctx, hidden, hidden)
        x = layer_norm(g.add(to32(attn), to32(x)))
        h = g.table(project(x, hidden, ffn), gelu_lut)
        x = layer_norm(g.add(to32(project(h, ffn, hidden)), to32(x)))
    g.output(x)
    return g, [data]


def macs_of(graph: GraphBuilder) -> int:
    """Algorithmic multiply-accumulates of a graph (padded taps counted, the usual convention)."""
    total = 0
    for op in graph.ops:
        if op.name == "CONV2D":
            oc, kh, kw, ic = op.inputs[1].shape
            total += int(np.prod(op.out.shape)) * kh * kw * ic
        elif op.name == "DEPTHWISE_CONV2D":
            kh, kw, _, _ = op.inputs[1].shape
            total += int(np.prod(op.out.shape)) * kh * kw
        elif op.name == "MATMUL":
            total += int(np.prod(op.out.shape)) * op.inputs[0].shape[2]
    return total
