"""Cross-checks the C++ oracle against the independent numpy restatement (oracle/np_ref.py) on
seeded random cases, including the edge cases the shaders handle specially: channel counts that
are not multiples of 4, stride 2, dilation, asymmetric padding, non-zero zero points, per-channel
and double-round RESCALE, shifts 0 / 1 / 31 / 32 / 40 / 62, and extreme accumulators."""
import numpy as np
import pytest

from oracle import np_ref, oracle


def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


CONV_CASES = [
    # n, h, w, ic, oc, kh, kw, pad, stride, dil, in_zp, w_zp
    (1, 8, 8, 3, 5, 3, 3, (1, 1, 1, 1), (1, 1), (1, 1), -3, 0),
    (2, 9, 7, 4, 8, 3, 3, (1, 1, 1, 1), (2, 2), (1, 1), 7, 0),
    (1, 12, 12, 6, 7, 3, 3, (2, 2, 2, 2), (1, 1), (2, 2), -128, 5),
    (1, 10, 11, 5, 3, 1, 1, (0, 0, 0, 0), (1, 1), (1, 1), 127, -7),
    (2, 15, 15, 3, 9, 7, 7, (3, 3, 3, 3), (2, 2), (1, 1), -3, 0),
    (1, 6, 6, 16, 16, 2, 3, (0, 1, 2, 0), (1, 2), (1, 1), 1, 1),
    (1, 5, 5, 1, 1, 5, 5, (4, 4, 4, 4), (1, 1), (1, 1), -5, 3),
]


@pytest.mark.parametrize("case", CONV_CASES)
def test_conv2d(case):
    n, h, w, ic, oc, kh, kw, pad, stride, dil, in_zp, w_zp = case
    r = rng(hash(case) & 0xFFFF)
    x = r.integers(-128, 128, (n, h, w, ic), dtype=np.int8)
    wt = r.integers(-128, 128, (oc, kh, kw, ic), dtype=np.int8)
    b = r.integers(-(1 << 14), 1 << 14, (oc,), dtype=np.int32)
    want = np_ref.conv2d(x, wt, b, pad, stride, dil, in_zp, w_zp)
    np.testing.assert_array_equal(oracle.conv2d(x, wt, b, pad, stride, dil, in_zp, w_zp), want)
    np.testing.assert_array_equal(oracle.conv2d(x, wt, b, pad, stride, dil, in_zp, w_zp, generic=True), want)
    # a one-element bias broadcasts (conv2d.comp:98-104)
    b1 = b[:1].copy()
    np.testing.assert_array_equal(oracle.conv2d(x, wt, b1, pad, stride, dil, in_zp, w_zp),
                                  np_ref.conv2d(x, wt, b1, pad, stride, dil, in_zp, w_zp))


def test_conv2d_strided_views():
    r = rng(5)
    big = r.integers(-128, 128, (2, 8, 8, 8), dtype=np.int8)
    x = big[:, :, :, ::2]  # explicit strides
    wt = r.integers(-128, 128, (3, 3, 3, 4), dtype=np.int8)
    b = r.integers(-100, 100, (3,), dtype=np.int32)
    np.testing.assert_array_equal(oracle.conv2d(x, wt, b, (1, 1, 1, 1), (1, 1), (1, 1), 2, 0),
                                  np_ref.conv2d(np.ascontiguousarray(x), wt, b, (1, 1, 1, 1), (1, 1), (1, 1), 2, 0))


def test_conv2d_extreme_accumulator_wraps():
    x = np.full((1, 1, 1, 70000), -128, np.int8)
    wt = np.full((1, 1, 1, 70000), -128, np.int8)
    b = np.array([2**31 - 1], np.int32)
    want = np_ref.conv2d(x, wt, b, (0, 0, 0, 0), (1, 1), (1, 1), 127, 127)  # (-255)^2 * 70000 wraps
    np.testing.assert_array_equal(oracle.conv2d(x, wt, b, (0, 0, 0, 0), (1, 1), (1, 1), 127, 127), want)
    np.testing.assert_array_equal(oracle.conv2d(x, wt, b, (0, 0, 0, 0), (1, 1), (1, 1), 127, 127, generic=True), want)


@pytest.mark.parametrize("case", [
    (1, 8, 8, 4, 1, 3, 3, (1, 1, 1, 1), (1, 1), (1, 1), -3, 0),
    (2, 9, 9, 5, 2, 3, 3, (1, 1, 1, 1), (2, 2), (1, 1), 4, 2),
    (1, 7, 6, 3, 3, 2, 2, (0, 1, 1, 0), (1, 1), (2, 1), -128, -1),
])
def test_depthwise(case):
    n, h, w, c, m, kh, kw, pad, stride, dil, in_zp, w_zp = case
    r = rng(11)
    x = r.integers(-128, 128, (n, h, w, c), dtype=np.int8)
    wt = r.integers(-128, 128, (kh, kw, c, m), dtype=np.int8)
    b = r.integers(-(1 << 14), 1 << 14, (c * m,), dtype=np.int32)
    np.testing.assert_array_equal(oracle.depthwise_conv2d(x, wt, b, pad, stride, dil, in_zp, w_zp),
                                  np_ref.depthwise_conv2d(x, wt, b, pad, stride, dil, in_zp, w_zp))


@pytest.mark.parametrize("shape", [(1, 4, 8, 4), (3, 5, 7, 9), (2, 16, 33, 16), (1, 1, 1, 1)])
@pytest.mark.parametrize("zps", [(0, 0), (-7, 0), (5, -3)])
def test_matmul(shape, zps):
    n, h, c, w = shape
    r = rng(3)
    a = r.integers(-128, 128, (n, h, c), dtype=np.int8)
    b = r.integers(-128, 128, (n, c, w), dtype=np.int8)
    np.testing.assert_array_equal(oracle.matmul(a, b, *zps), np_ref.matmul(a, b, *zps))


def test_matmul_int16():
    r = rng(4)
    a = r.integers(-32768, 32768, (2, 3, 5), dtype=np.int16)
    b = r.integers(-32768, 32768, (2, 5, 4), dtype=np.int16)
    np.testing.assert_array_equal(oracle.matmul(a, b, 0, 0), np_ref.matmul(a, b, 0, 0))


@pytest.mark.parametrize("shift", [0, 1, 2, 30, 31, 32, 33, 40, 62])
@pytest.mark.parametrize("double_round", [False, True])
@pytest.mark.parametrize("per_channel", [False, True])
def test_rescale_i32_to_i8(shift, double_round, per_channel):
    r = rng(shift * 4 + double_round * 2 + per_channel)
    c = 6
    x = r.integers(-(1 << 31), 1 << 31, (3, 5, c), dtype=np.int64).astype(np.int32)
    x[0, 0, :] = [0, 1, -1, 2**31 - 1, -(2**31), 12345]
    n = c if per_channel else 1
    mult = r.integers(1 << 30, (1 << 31) - 1, (n,), dtype=np.int64).astype(np.int32)
    sh = np.full((n,), shift, np.int8)
    if per_channel and shift >= 2:
        sh[1::2] -= 1
    got = oracle.rescale(x, mult, sh, 0, 5, np.int8, True, double_round, per_channel)
    want = np_ref.rescale(x, mult, sh, 0, 5, np.int8, True, double_round, per_channel)
    np.testing.assert_array_equal(got, want)


@pytest.mark.parametrize("in_dtype,out_dtype,in_zp,out_zp", [
    (np.int8, np.int32, -7, 0), (np.int8, np.int8, 3, -128), (np.int16, np.int8, 100, 7),
    (np.int32, np.int16, 0, -5), (np.int8, np.int16, -128, 32767), (np.int32, np.int32, 11, -11),
])
def test_rescale_types(in_dtype, out_dtype, in_zp, out_zp):
    r = rng(9)
    info = np.iinfo(in_dtype)
    x = r.integers(info.min, int(info.max) + 1, (4, 7), dtype=np.int64).astype(in_dtype)
    mult = np.array([int(r.integers(1 << 30, (1 << 31) - 1))], np.int32)
    for shift in (12, 23, 35):
        sh = np.array([shift], np.int8)
        np.testing.assert_array_equal(oracle.rescale(x, mult, sh, in_zp, out_zp, out_dtype, True, True, False),
                                      np_ref.rescale(x, mult, sh, in_zp, out_zp, out_dtype, True, True, False))


def test_rescale_scale16_ignores_double_round():
    r = rng(10)
    x = r.integers(-30000, 30000, (50,), dtype=np.int64).astype(np.int32)
    mult = np.array([20000], np.int16)
    sh = np.array([33], np.int8)
    a = oracle.rescale(x, mult, sh, 0, 0, np.int8, scale32=False, double_round=True)
    b = np_ref.rescale(x, mult, sh, 0, 0, np.int8, scale32=False, double_round=True)
    np.testing.assert_array_equal(a, b)
    np.testing.assert_array_equal(a, oracle.rescale(x, mult, sh, 0, 0, np.int8, scale32=False, double_round=False))


@pytest.mark.parametrize("case", [
    ((1, 7, 7, 5), (7, 7), (7, 7), (0, 0, 0, 0), -20, -20),
    ((2, 8, 9, 3), (3, 3), (2, 2), (1, 1, 1, 1), 0, 0),
    ((1, 6, 6, 4), (2, 3), (1, 2), (0, 1, 1, 1), 5, -3),
])
def test_avg_pool(case):
    shape, k, s, p, in_zp, out_zp = case
    x = rng(2).integers(-128, 128, shape, dtype=np.int8)
    np.testing.assert_array_equal(oracle.avg_pool2d(x, k, s, p, in_zp, out_zp),
                                  np_ref.avg_pool2d(x, k, s, p, in_zp, out_zp))


@pytest.mark.parametrize("case", [
    ((1, 16, 16, 3), (2, 2), (2, 2), (0, 0, 0, 0)),
    ((2, 9, 9, 5), (3, 3), (2, 2), (1, 1, 1, 1)),
    ((1, 7, 5, 2), (3, 2), (1, 1), (1, 0, 0, 1)),
])
def test_max_pool(case):
    shape, k, s, p = case
    x = rng(6).integers(-128, 128, shape, dtype=np.int8)
    np.testing.assert_array_equal(oracle.max_pool2d(x, k, s, p), np_ref.max_pool2d(x, k, s, p))


def test_table():
    r = rng(7)
    x8 = r.integers(-128, 128, (3, 50), dtype=np.int8)
    t8 = r.integers(-128, 128, (256,), dtype=np.int8)
    np.testing.assert_array_equal(oracle.table(x8, t8), np_ref.table(x8, t8))
    x16 = r.integers(-32768, 32768, (3, 50), dtype=np.int16)
    x16[0, :4] = [-32768, 32767, 0, -1]
    t16 = r.integers(-32768, 32768, (513,), dtype=np.int16)
    np.testing.assert_array_equal(oracle.table(x16, t16), np_ref.table(x16, t16))


def test_mul_and_elementwise():
    r = rng(8)
    a = r.integers(-128, 128, (2, 3, 4), dtype=np.int8)
    b = r.integers(-128, 128, (2, 1, 4), dtype=np.int8)
    for shift in (0, 1, 7):
        np.testing.assert_array_equal(oracle.mul(a, b, shift), np_ref.mul(a, np.broadcast_to(b, a.shape), shift))
    a32 = r.integers(-(1 << 31), 1 << 31, (5, 6), dtype=np.int64).astype(np.int32)
    b32 = r.integers(-(1 << 31), 1 << 31, (5, 6), dtype=np.int64).astype(np.int32)
    np.testing.assert_array_equal(oracle.binary("ADD", a32, b32), (a32.astype(np.int64) + b32).astype(np.int32))
    np.testing.assert_array_equal(oracle.binary("SUB", a32, b32), (a32.astype(np.int64) - b32).astype(np.int32))
    np.testing.assert_array_equal(oracle.binary("MAXIMUM", a32, b32), np.maximum(a32, b32))
    np.testing.assert_array_equal(oracle.binary("GREATER", a32, b32), a32 > b32)
    np.testing.assert_array_equal(oracle.binary("ADD", a, np.broadcast_to(b, a.shape).copy()),
                                  (a.astype(np.int16) + b).astype(np.int8))
    np.testing.assert_array_equal(oracle.reduce("REDUCE_SUM", a32, 1), a32.sum(axis=1, keepdims=True, dtype=np.int32))
    np.testing.assert_array_equal(oracle.reduce("REDUCE_MAX", a, 2), a.max(axis=2, keepdims=True))
    np.testing.assert_array_equal(oracle.clamp(a, -20, 64), np.clip(a, -20, 64))
    np.testing.assert_array_equal(oracle.transpose(a, [2, 0, 1]), a.transpose(2, 0, 1))
    np.testing.assert_array_equal(oracle.cast(a32, np.int8), a32.astype(np.int8))
    np.testing.assert_array_equal(oracle.pad(a, [0, 0, 1, 2, 2, 0], -5),
                                  np.pad(a, ((0, 0), (1, 2), (2, 0)), constant_values=-5))
    sh = r.integers(0, 8, a.shape, dtype=np.int8)
    np.testing.assert_array_equal(oracle.arithmetic_right_shift(a, sh, False), a >> sh)


# ---- index-driven operators, TRANSPOSE_CONV2D, CONV3D, RESIZE ------------------------------------------------

@pytest.mark.parametrize("dtype", [np.int8, np.int16, np.int32])
@pytest.mark.parametrize("axis", [0, 1, 2])
def test_argmax(dtype, axis):
    r = rng(axis)
    info = np.iinfo(dtype)
    x = r.integers(info.min, int(info.max) + 1, (5, 6, 7), dtype=np.int64).astype(dtype)
    x[0, 0, :] = info.min  # all-lowest row: index 0
    x[1, :, 1] = 5         # ties: the first one
    np.testing.assert_array_equal(oracle.argmax(x, axis), np_ref.argmax(x, axis))


@pytest.mark.parametrize("dtype", [np.int8, np.int16, np.int32, np.float32])
def test_gather_scatter_reverse_tile(dtype):
    r = rng(11)
    values = r.integers(-100, 100, (3, 9, 5)).astype(dtype)
    indices = np.stack([r.permutation(9)[:6] for _ in range(3)]).astype(np.int32)
    np.testing.assert_array_equal(oracle.gather(values, indices), np_ref.gather(values, indices))
    inp = r.integers(-100, 100, (3, 6, 5)).astype(dtype)
    np.testing.assert_array_equal(oracle.scatter(values, indices, inp), np_ref.scatter(values, indices, inp))
    dup = indices.copy()
    dup[:, 3] = dup[:, 1]  # a repeated index: the first occurrence wins (scatter.comp:26-31)
    np.testing.assert_array_equal(oracle.scatter(values, dup, inp), np_ref.scatter(values, dup, inp))
    for axis in range(3):
        np.testing.assert_array_equal(oracle.reverse(values, axis), np.flip(values, axis))
    np.testing.assert_array_equal(oracle.tile(values, (2, 1, 3)), np.tile(values, (2, 1, 3)))


def test_gather_out_of_range_index_reads_zero():
    values = np.arange(1, 1 + 2 * 4 * 3, dtype=np.int8).reshape(2, 4, 3)
    indices = np.array([[0, 4, 3], [7, 1, -1]], np.int32)  # 4, 7 and -1 (as unsigned) are out of range
    out = oracle.gather(values, indices)
    assert (out[0, 1] == 0).all() and (out[1, 0] == 0).all() and (out[1, 2] == 0).all()
    np.testing.assert_array_equal(out[0, 0], values[0, 0])
    np.testing.assert_array_equal(out[1, 1], values[1, 1])


TCONV_CASES = [
    # n, h, w, ic, oc, kh, kw, out_pad, stride, in_zp, w_zp
    (1, 4, 5, 3, 4, 3, 3, (0, 0, 0, 0), (1, 1), -3, 0),
    (2, 3, 3, 5, 2, 2, 3, (0, 0, 0, 0), (2, 2), 7, 1),
    (1, 5, 4, 2, 3, 3, 2, (-1, 0, 0, -1), (2, 3), -128, -4),
    (1, 2, 2, 1, 1, 1, 1, (1, 2, 0, 1), (3, 2), 0, 0),
]


@pytest.mark.parametrize("case", TCONV_CASES)
def test_transpose_conv2d(case):
    n, h, w, ic, oc, kh, kw, out_pad, stride, in_zp, w_zp = case
    r = rng(sum(case[:7]))
    x = r.integers(-128, 128, (n, h, w, ic), dtype=np.int8)
    wt = r.integers(-128, 128, (oc, kh, kw, ic), dtype=np.int8)
    bias = r.integers(-1000, 1000, (oc,), dtype=np.int32)
    want = np_ref.transpose_conv2d(x, wt, bias, out_pad, stride, in_zp, w_zp)
    got = oracle.transpose_conv2d(x, wt, bias, want.shape, list(out_pad), list(stride), in_zp, w_zp)
    np.testing.assert_array_equal(got, want)


CONV3D_CASES = [
    # n, d, h, w, ic, oc, kd, kh, kw, pad, stride, dil, in_zp, w_zp
    (1, 4, 5, 6, 3, 4, 2, 3, 3, (1, 0, 1, 1, 1, 1), (1, 1, 1), (1, 1, 1), -3, 0),
    (2, 5, 5, 5, 2, 3, 3, 3, 3, (1, 1, 1, 1, 1, 1), (2, 2, 2), (1, 1, 1), 9, 2),
    (1, 6, 7, 5, 4, 2, 2, 2, 2, (2, 2, 0, 3, 1, 0), (1, 2, 1), (2, 3, 2), -128, -5),
]


@pytest.mark.parametrize("case", CONV3D_CASES)
def test_conv3d(case):
    n, d, h, w, ic, oc, kd, kh, kw, pad, stride, dil, in_zp, w_zp = case
    r = rng(sum(case[:9]))
    x = r.integers(-128, 128, (n, d, h, w, ic), dtype=np.int8)
    wt = r.integers(-128, 128, (oc, kd, kh, kw, ic), dtype=np.int8)
    bias = r.integers(-1000, 1000, (oc,), dtype=np.int32)
    want = np_ref.conv3d(x, wt, bias, pad, stride, dil, in_zp, w_zp)
    got = oracle.conv3d(x, wt, bias, want.shape, list(pad), list(stride), list(dil), in_zp, w_zp)
    np.testing.assert_array_equal(got, want)


RESIZE_CASES = [
    # scale (y_n, y_d, x_n, x_d), offset, border
    ((2, 1, 2, 1), (0, 0), (0, 0)),
    ((4, 2, 4, 2), (-1, -1), (1, 1)),      # half-pixel centres, 2x up
    ((3, 2, 5, 3), (1, -2), (0, 2)),
    ((1, 2, 1, 3), (0, 0), (0, 0)),        # down-scaling
    ((16, 1, 16, 1), (-8, 7), (15, -7)),
]


@pytest.mark.parametrize("scale,offset,border", RESIZE_CASES)
@pytest.mark.parametrize("in_dtype,out_dtype,mode", [(np.int8, np.int8, 1), (np.int8, np.int32, 2),
                                                     (np.int16, np.int16, 1), (np.int16, np.int64, 2)])
def test_resize(scale, offset, border, in_dtype, out_dtype, mode):
    r = rng(scale[0] + mode)
    info = np.iinfo(in_dtype)
    x = r.integers(info.min, int(info.max) + 1, (2, 7, 9, 3), dtype=np.int64).astype(in_dtype)
    want = np_ref.resize(x, scale, offset, border, mode, out_dtype)
    got = oracle.resize(x, want.shape, out_dtype, scale, offset, border, mode)
    np.testing.assert_array_equal(got, want)


@pytest.mark.parametrize("shape", [(2, 8, 16), (1, 4, 64), (3, 1, 8), (1, 6, 10)])
def test_fft2d_and_rfft2d_against_numpy(shape):
    r = rng(shape[2])
    re = r.standard_normal(shape).astype(np.float32)
    im = r.standard_normal(shape).astype(np.float32)
    z = re.astype(np.float64) + 1j * im.astype(np.float64)
    scale = np.sqrt(shape[1] * shape[2])
    for inverse, want in ((False, np.fft.fft2(z)), (True, np.fft.ifft2(z) * shape[1] * shape[2])):
        got_re, got_im = oracle.fft2d(re, im, inverse)
        assert np.abs(got_re - want.real).max() < 1e-6 * scale and np.abs(got_im - want.imag).max() < 1e-6 * scale
    want = np.fft.rfft2(re.astype(np.float64))
    got_re, got_im = oracle.rfft2d(re)
    assert got_re.shape == want.shape
    assert np.abs(got_re - want.real).max() < 1e-6 * scale and np.abs(got_im - want.imag).max() < 1e-6 * scale
    for oy in {0, shape[1] // 2}:       # the self-conjugate bins are written as exact zeros (rfft2d.comp:33-38)
        for ox in {0, shape[2] // 2}:
            assert (got_im[:, oy, ox] == 0).all()
