"""GPU parity of ARGMAX, GATHER, SCATTER, REVERSE, TILE, integer RESIZE, TRANSPOSE_CONV2D and CONV3D against
the CPU oracle, bit for bit, through the SPIR-V front end and the C ABI; CONV3D also against the reference's
own golden vector (tests/vulkan.cpp:1211-1293)."""
import json
import os

import numpy as np
import pytest

from mlel_b200.graph_builder import GraphBuilder
from tests.graph_eval import evaluate

pytestmark = pytest.mark.gpu

with open(os.path.join(os.path.dirname(__file__), "golden", "reference_goldens.json")) as f:
    GOLD = json.load(f)


def gold(name):
    g = GOLD[name]
    return np.array(g["values"], dtype=g["dtype"]).reshape(g["shape"])


def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def full_range(r, dtype, shape):
    info = np.iinfo(dtype)
    return r.integers(info.min, int(info.max) + 1, shape, dtype=np.int64).astype(dtype)


def check(g, inputs):
    from mlel_b200.runtime import GraphRunner
    want = evaluate(g, inputs)
    got = GraphRunner(g).run(inputs)
    assert len(got) == len(want)
    for k, (a, b) in enumerate(zip(got, want)):
        assert a.dtype == b.dtype and a.shape == b.shape
        if not np.array_equal(a, b):
            bad = np.argwhere(a != b)
            raise AssertionError(f"output {k}: {len(bad)} of {a.size} differ, first at {bad[0].tolist()}: "
                                 f"got {a[tuple(bad[0])]} want {b[tuple(bad[0])]}")


@pytest.mark.parametrize("dtype", [np.int8, np.int16, np.int32])
def test_argmax(mlel, dtype):
    r = rng(1)
    data = full_range(r, dtype, (4, 33, 17, 8))
    data[0, :, 0, 0] = np.iinfo(dtype).min  # nothing exceeds the start value: index 0
    data[1, :, 1, 1] = 7                    # ties: the first index
    g = GraphBuilder()
    x = g.input(dtype, data.shape)
    for axis in range(4):
        g.output(g.argmax(x, axis))
    check(g, [data])


@pytest.mark.parametrize("dtype", [np.int8, np.int16, np.int32])
def test_gather_and_scatter(mlel, dtype):
    r = rng(2)
    n, k, w, c = 3, 40, 25, 24
    values = full_range(r, dtype, (n, k, c))
    indices = np.stack([r.permutation(k)[:w] for _ in range(n)]).astype(np.int32)
    updates = full_range(r, dtype, (n, w, c))
    wild = indices.copy()
    wild[0, 3] = k        # out of range: GATHER reads zero, SCATTER matches no row
    wild[1, 5] = -1
    wild[2, 7] = wild[2, 2]  # repeated index: the first occurrence wins
    g = GraphBuilder()
    v, i1, i2, u = g.input(dtype, values.shape), g.input(np.int32, indices.shape), g.input(np.int32, wild.shape), \
        g.input(dtype, updates.shape)
    g.output(g.gather(v, i1))
    g.output(g.gather(v, i2))
    g.output(g.scatter(v, i1, u))
    g.output(g.scatter(v, i2, u))
    check(g, [values, indices, wild, updates])


@pytest.mark.parametrize("dtype", [np.int8, np.int16, np.int32, np.int64])
def test_reverse_and_tile(mlel, dtype):
    r = rng(3)
    data = full_range(r, dtype, (3, 5, 7, 16))
    g = GraphBuilder()
    x = g.input(dtype, data.shape)
    for axis in range(4):
        g.output(g.reverse(x, axis))
    g.output(g.tile(x, (2, 1, 3, 1)))
    g.output(g.tile(x, (1, 1, 1, 4)))
    g.output(g.reverse(g.tile(g.reverse(x, 3), (1, 2, 1, 1)), 1))
    check(g, [data])


RESIZE_CASES = [
    ((2, 1, 2, 1), (0, 0), (0, 0)), ((4, 2, 4, 2), (-1, -1), (1, 1)), ((3, 2, 5, 3), (1, -2), (0, 2)),
    ((1, 2, 1, 3), (0, 0), (0, 0)), ((16, 1, 16, 1), (-8, 7), (15, -7)),
]


@pytest.mark.parametrize("scale,offset,border", RESIZE_CASES)
@pytest.mark.parametrize("in_dtype,out_dtype,mode", [(np.int8, np.int8, 1), (np.int8, np.int32, 2),
                                                     (np.int16, np.int16, 1), (np.int16, np.int64, 2)])
def test_resize(mlel, scale, offset, border, in_dtype, out_dtype, mode):
    r = rng(scale[0] + mode)
    data = full_range(r, in_dtype, (2, 13, 11, 8))
    g = GraphBuilder()
    x = g.input(in_dtype, data.shape)
    g.output(g.resize(x, scale, offset, border, mode, out_dtype))
    check(g, [data])


TCONV_CASES = [
    # n, h, w, ic, oc, kh, kw, out_pad, stride, in_zp, w_zp
    (1, 9, 10, 8, 12, 3, 3, (0, 0, 0, 0), (1, 1), -3, 0),
    (2, 7, 7, 16, 8, 2, 2, (0, 0, 0, 0), (2, 2), 7, 1),
    (1, 6, 5, 3, 5, 4, 3, (-1, 0, 0, -1), (2, 3), -128, -4),
    (1, 3, 3, 1, 1, 1, 1, (1, 2, 0, 1), (3, 2), 0, 0),
]


@pytest.mark.parametrize("case", TCONV_CASES)
def test_transpose_conv2d(mlel, case):
    n, h, w, ic, oc, kh, kw, out_pad, stride, in_zp, w_zp = case
    r = rng(sum(case[:7]))
    data = full_range(r, np.int8, (n, h, w, ic))
    g = GraphBuilder()
    x = g.input(np.int8, data.shape)
    wt = g.constant(full_range(r, np.int8, (oc, kh, kw, ic)))
    bias = g.constant(r.integers(-5000, 5000, (oc,), dtype=np.int32))
    g.output(g.transpose_conv2d(x, wt, bias, out_pad, stride, in_zp, w_zp))
    check(g, [data])


def test_transpose_conv2d_int16(mlel):
    r = rng(5)
    data = full_range(r, np.int16, (1, 5, 6, 4))
    g = GraphBuilder()
    x = g.input(np.int16, data.shape)
    wt = g.constant(full_range(r, np.int8, (3, 3, 2, 4)))
    bias = g.constant(r.integers(-(1 << 40), 1 << 40, (1,), dtype=np.int64))
    g.output(g.transpose_conv2d(x, wt, bias, (0, 1, 1, 0), (2, 1), 0, 0, acc_type=4))
    check(g, [data])


CONV3D_CASES = [
    # n, d, h, w, ic, oc, kd, kh, kw, pad, stride, dil, in_zp, w_zp
    (1, 4, 9, 10, 8, 12, 2, 3, 3, (1, 0, 1, 1, 1, 1), (1, 1, 1), (1, 1, 1), -3, 0),
    (2, 5, 7, 7, 4, 6, 3, 3, 3, (1, 1, 1, 1, 1, 1), (2, 2, 2), (1, 1, 1), 9, 2),
    (1, 6, 7, 5, 3, 2, 2, 2, 2, (2, 2, 0, 3, 1, 0), (1, 2, 1), (2, 3, 2), -128, -5),
]


@pytest.mark.parametrize("case", CONV3D_CASES)
def test_conv3d(mlel, case):
    n, d, h, w, ic, oc, kd, kh, kw, pad, stride, dil, in_zp, w_zp = case
    r = rng(sum(case[:9]))
    data = full_range(r, np.int8, (n, d, h, w, ic))
    g = GraphBuilder()
    x = g.input(np.int8, data.shape)
    wt = g.constant(full_range(r, np.int8, (oc, kd, kh, kw, ic)))
    bias = g.constant(r.integers(-5000, 5000, (oc,), dtype=np.int32))
    g.output(g.conv3d(x, wt, bias, pad, stride, dil, in_zp, w_zp))
    check(g, [data])


def test_golden_conv3d_large_stride_and_pad(mlel):
    rel = gold("Conv3DLargeStridePadRegression.relevantWeights")
    w = np.zeros((3, 2, 2, 8192, 4), np.int8)
    for oc in range(3):
        for kd in range(2):
            for kh in range(2):
                base = ((oc * 2 + kd) * 2 + kh) * 8
                w[oc, kd, kh, 8190, :] = rel[base:base + 4]
                w[oc, kd, kh, 8191, :] = rel[base + 4:base + 8]
    g = GraphBuilder()
    x = g.input(np.int8, (1, 3, 2, 2, 4))
    out = g.conv3d(x, g.constant(w), g.inline(np.zeros((1,), np.int32)), [1, 0, 1, 0, 8190, 8192], [1, 1, 8192],
                   [1, 1, 1], 9, 0)
    assert out.shape == (1, 3, 2, 2, 3)
    g.output(out)
    from mlel_b200.runtime import GraphRunner
    got = GraphRunner(g).run([np.full((1, 3, 2, 2, 4), -128, np.int8)])[0]
    np.testing.assert_array_equal(got, gold("Conv3DLargeStridePadRegression"))


# ---- fp32 unary operators and POW ------------------------------------------------------------------------------
# The reference evaluates these with its Vulkan device's single-precision builtins and pins one value only (SIN,
# to 7.7e-8 absolute).  The oracle evaluates in double precision and rounds once; the CUDA single-precision
# functions are documented to stay within 2 ulp of that (4 ulp for POW), which is the tolerance used here.
# CEIL, FLOOR, ABS and RECIPROCAL are exact.

def ulp_distance(a, b):
    ia = a.view(np.int32).astype(np.int64)
    ib = b.view(np.int32).astype(np.int64)
    ia = np.where(ia < 0, -(ia & 0x7FFFFFFF), ia)  # sign-magnitude -> a monotone integer line
    ib = np.where(ib < 0, -(ib & 0x7FFFFFFF), ib)
    return np.abs(ia - ib)


def check_float(got, want, ulps, what):
    assert got.dtype == np.float32 and got.shape == want.shape
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(got), nan), what
    inf = np.isinf(want)
    assert np.array_equal(got[inf], want[inf]), what
    ok = ~(nan | inf)
    # results that round to a denormal may be flushed; compare those absolutely
    tiny = ok & (np.abs(want) < 1e-37)
    assert np.all(np.abs(got[tiny] - want[tiny]) < 1e-37), what
    rest = ok & ~tiny
    dist = ulp_distance(got[rest], want[rest])
    assert dist.size == 0 or dist.max() <= ulps, f"{what}: {dist.max()} ulp"


FLOAT_UNARY = [
    # operator, input range, ulps allowed
    ("ABS", (-100, 100), 0), ("CEIL", (-100, 100), 0), ("FLOOR", (-100, 100), 0), ("RECIPROCAL", (-100, 100), 0),
    ("COS", (-20, 20), 2), ("SIN", (-20, 20), 2), ("EXP", (-80, 80), 2), ("LOG", (-1, 1000), 2),
    ("RSQRT", (0, 1000), 2), ("SIGMOID", (-30, 30), 3), ("TANH", (-12, 12), 2), ("ERF", (-5, 5), 2),
]


@pytest.mark.parametrize("name,span,ulps", FLOAT_UNARY)
@pytest.mark.parametrize("shape", [(4, 33, 64), (3, 5, 7)])  # packed, four at a time / generic indexing
def test_float_unary(mlel, name, span, ulps, shape):
    from mlel_b200.runtime import GraphRunner
    r = rng(len(name))
    data = r.uniform(span[0], span[1], shape).astype(np.float32)
    flat = data.reshape(-1)
    special = [0.0, -0.0, np.nan, np.inf, -np.inf, 1.0, -1.0, 1e-4, -1e-4, 0.15, -0.15, 10.5, -10.5, 1e-30, 0.5, 4.5]
    flat[:len(special)] = special
    g = GraphBuilder()
    x = g.input(np.float32, shape)
    g.output(g.unary(name, x))
    want = evaluate(g, [data])[0]
    got = GraphRunner(g).run([data])[0]
    check_float(got, want, ulps, name)


def test_sin_known_answer_through_the_front_end(mlel):
    # the reference's own pin: tests/vulkan.cpp:1795-1841
    from mlel_b200.runtime import GraphRunner
    g = GraphBuilder()
    x = g.input(np.float32, (1,))
    g.output(g.unary("SIN", x))
    got = GraphRunner(g).run([np.array([0.000111731846], np.float32)])[0]
    assert abs(float(got[0]) - 0.00011173184588586903) <= 7.715463482888105e-08


def test_pow(mlel):
    from mlel_b200.runtime import GraphRunner
    r = rng(77)
    base = r.uniform(-8, 8, (6, 40, 32)).astype(np.float32)
    expo = r.uniform(-4, 4, (6, 40, 32)).astype(np.float32)
    expo[:, ::2, :] = np.round(expo[:, ::2, :])  # integral exponents: negative bases are defined
    base[0, 0, :4] = [0.0, -0.0, 2.0, -2.0]
    expo[0, 0, :4] = [0.0, 3.0, 0.5, 0.5]
    g = GraphBuilder()
    a, b = g.input(np.float32, base.shape), g.input(np.float32, expo.shape)
    g.output(g.binary("POW", a, b))
    want = evaluate(g, [base, expo])[0]
    got = GraphRunner(g).run([base, expo])[0]
    check_float(got, want, 4, "POW")


# ---- FFT2D / RFFT2D: direct sums in double on both sides; what differs is the sine/cosine (sincospi of the reduced
# fraction on the device, cos/sin of the reduced angle in the oracle), far below the float rounding of the result.
# Tolerance: 2e-6 * sqrt(H * W) absolute for unit-variance inputs (the results have standard deviation sqrt(H * W)).

@pytest.mark.parametrize("shape", [(2, 8, 16), (1, 4, 256), (3, 5, 12)])
def test_fft2d_and_rfft2d(mlel, shape):
    from mlel_b200.runtime import GraphRunner
    r = rng(shape[2])
    re = r.standard_normal(shape).astype(np.float32)
    im = r.standard_normal(shape).astype(np.float32)
    g = GraphBuilder()
    a, b = g.input(np.float32, shape), g.input(np.float32, shape)
    f_re, f_im = g.fft2d(a, b, False)
    i_re, i_im = g.fft2d(f_re, f_im, True)  # an intermediate pair: both results live in session memory
    r_re, r_im = g.rfft2d(a)
    for v in (f_re, f_im, i_re, i_im, r_re, r_im):
        g.output(v)
    want = evaluate(g, [re, im])
    got = GraphRunner(g).run([re, im])
    points = shape[1] * shape[2]
    tol = [np.sqrt(points)] * 2 + [float(points)] * 2 + [np.sqrt(points)] * 2
    for k, (x, y, t) in enumerate(zip(got, want, tol)):
        assert x.dtype == np.float32 and x.shape == y.shape
        assert np.abs(x - y).max() <= 2e-6 * t, (k, np.abs(x - y).max())
    # forward then unscaled inverse returns the input times H * W
    assert np.abs(got[2] / points - re).max() < 1e-5 and np.abs(got[3] / points - im).max() < 1e-5
    for oy in {0, shape[1] // 2}:
        for ox in {0, shape[2] // 2}:
            assert (got[5][:, oy, ox] == 0).all()
