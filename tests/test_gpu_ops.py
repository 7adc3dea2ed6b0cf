"""GPU parity, operator by operator: every CUDA kernel behind the C ABI against the CPU oracle on
seeded inputs, bit-exact.  Each case is a one- or two-operator graph that enters through the
SPIR-V text front end, is dispatched by a session, and is run twice: with the fusion pass on
(default) and off (one kernel per TOSA operator, the reference's op list)."""
import numpy as np
import pytest

from mlel_b200.graph_builder import GraphBuilder
from tests.graph_eval import evaluate

pytestmark = pytest.mark.gpu


def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def check(mlel, g, inputs, modes=(0, 1)):
    from mlel_b200.runtime import GraphRunner
    want = evaluate(g, inputs)
    for flags in modes:
        runner = GraphRunner(g, flags=flags)
        got = runner.run(inputs)
        for k, (a, b) in enumerate(zip(got, want)):
            assert a.dtype == b.dtype and a.shape == b.shape
            if not np.array_equal(a, b):
                bad = np.argwhere(a != b)
                raise AssertionError(f"flags={flags} output {k}: {len(bad)} of {a.size} differ, first at "
                                     f"{bad[0].tolist()}: got {a[tuple(bad[0])]} want {b[tuple(bad[0])]}; "
                                     f"kernels={runner.pipeline.exec_names()}")


CONV_CASES = [
    # n, h, w, ic, oc, k, pad, stride, dil, in_zp, w_zp
    (1, 8, 8, 3, 5, 3, 1, 1, 1, -3, 0),
    (2, 9, 7, 4, 8, 3, 1, 2, 1, 7, 0),
    (1, 12, 12, 6, 7, 3, 2, 1, 2, -128, 5),
    (1, 10, 11, 5, 3, 1, 0, 1, 1, 127, -7),
    (2, 15, 15, 3, 9, 7, 3, 2, 1, -3, 0),
    # an RGB stem over several tiles and images, odd sizes (windows start every 8 bytes of the padded copy:
    # even and odd pixels take turns); one and two channels the same way
    (3, 33, 37, 3, 64, 7, 3, 2, 1, 5, 0),
    (2, 21, 18, 1, 16, 5, 2, 2, 1, -9, 0),
    # rows of whole 32-bit words in the source image: three, two and one channel
    (2, 20, 16, 3, 16, 7, 3, 2, 1, -7, 0),
    (1, 12, 12, 2, 8, 3, 1, 1, 1, 4, 0),
    (3, 9, 16, 1, 8, 3, 1, 2, 1, -1, 0),
    (1, 14, 14, 16, 32, 3, 1, 1, 1, -20, 0),
    (2, 7, 7, 64, 64, 1, 0, 1, 1, -20, 0),
    (1, 56, 56, 64, 64, 3, 1, 1, 1, -3, 0),   # configuration 0
    (3, 28, 28, 32, 48, 3, 1, 2, 1, 11, 0),
    (1, 5, 5, 128, 256, 1, 0, 2, 1, -7, 0),
    # more than 64 output channels: channel count not a multiple of the 128-channel tile, pixel counts that
    # end inside a tile, border classes, and layers large enough for the 256-pixel tiles
    (1, 20, 20, 32, 200, 3, 1, 1, 1, -5, 0),
    (2, 30, 30, 64, 136, 3, 1, 1, 1, 9, 0),
    (4, 17, 17, 128, 130, 1, 0, 1, 1, -11, 0),
    (8, 56, 56, 32, 128, 1, 0, 1, 1, 6, 0),
    (8, 40, 40, 16, 192, 3, 1, 1, 1, 3, 0),
    # gather variants: channel counts whose taps do not split a 128-byte K block evenly (48), dilation, a
    # 5x5 window with stride 2, and a 7x7 window (49 taps) over 16 channels
    (1, 9, 9, 48, 32, 3, 1, 1, 1, 4, 0),
    (1, 9, 9, 48, 144, 3, 1, 1, 1, 4, 0),
    (1, 13, 13, 32, 80, 3, 2, 1, 2, -9, 0),
    (2, 15, 15, 16, 16, 5, 2, 2, 1, 1, 0),
    (1, 20, 20, 16, 96, 7, 3, 2, 1, -2, 0),
    (2, 11, 11, 256, 128, 3, 1, 1, 1, 12, 0),
    # channel counts that are multiples of 128 with more than 64 output channels (hardware im2col loads):
    # dilation, stride 2 over an odd size, a 5x5 window, and a tile that spans several images
    (1, 12, 12, 128, 96, 3, 2, 1, 2, 5, 0),
    (2, 15, 15, 128, 80, 3, 1, 2, 1, -4, 0),
    (1, 9, 9, 128, 96, 5, 2, 1, 1, 3, 0),
    (40, 7, 7, 128, 144, 3, 1, 1, 1, -8, 0),
    # output channel counts that are not multiples of 16 (MobileNet's 24-channel projections, a single channel)
    (2, 14, 14, 96, 24, 1, 0, 1, 1, -5, 0),
    (1, 10, 10, 32, 40, 3, 1, 1, 1, 4, 0),
    (1, 6, 6, 16, 1, 1, 0, 1, 1, 0, 0),
    (2, 9, 9, 128, 72, 3, 1, 1, 1, 7, 0),
    # 1x1 convolutions whose input channel count is not a multiple of 16 (MobileNet's 24 -> 144 expansions): the
    # input goes through a copy with padded channels, which the TMA kernels then read as a plain matrix
    (3, 14, 14, 24, 144, 1, 0, 1, 1, -6, 0),
    (2, 9, 9, 40, 80, 1, 0, 1, 1, 11, 0),
    (1, 7, 7, 24, 32, 1, 0, 1, 1, 2, 0),
    (2, 8, 8, 20, 96, 1, 0, 2, 1, -3, 0),   # stride 2: stays on the table gather
]


@pytest.mark.parametrize("case", CONV_CASES)
@pytest.mark.parametrize("with_rescale", [False, True])
def test_conv2d(mlel, case, with_rescale):
    n, h, w, ic, oc, k, pad, stride, dil, in_zp, w_zp = case
    r = rng(hash(case) & 0xFFFF)
    g = GraphBuilder()
    x = g.input(np.int8, (n, h, w, ic))
    wt = g.constant(r.integers(-128, 128, (oc, k, k, ic), dtype=np.int8))
    b = g.constant(r.integers(-(1 << 14), 1 << 14, (oc,), dtype=np.int32))
    y = g.conv2d(x, wt, b, [pad] * 4, [stride] * 2, [dil] * 2, in_zp, w_zp)
    if with_rescale:
        mult = r.integers(1 << 30, (1 << 31) - 1, (oc,), dtype=np.int64).astype(np.int32)
        shift = r.integers(36, 46, (oc,), dtype=np.int8)
        y = g.rescale(y, mult, shift, 0, 5, np.int8, True, True, True)
        y = g.clamp(y, -20, 100)
    g.output(y)
    check(mlel, g, [r.integers(-128, 128, (n, h, w, ic), dtype=np.int8)])


def test_conv2d_asymmetric_padding_and_stride(mlel):
    r = rng(1)
    g = GraphBuilder()
    x = g.input(np.int8, (1, 9, 10, 8))
    wt = g.constant(r.integers(-128, 128, (16, 2, 3, 8), dtype=np.int8))
    b = g.constant(r.integers(-100, 100, (1,), dtype=np.int32))  # one-element bias broadcasts
    y = g.conv2d(x, wt, b, [0, 1, 2, 0], [1, 2], [1, 1], 9, 0)
    y = g.rescale(y, [1 << 30], [38], 0, -1, np.int8, True, False, False)
    g.output(y)
    check(mlel, g, [r.integers(-128, 128, (1, 9, 10, 8), dtype=np.int8)])


def test_conv2d_asymmetric_padding_many_channels(mlel):
    """The same geometry on the 128-channel path (hardware im2col loads): uneven padding, a 2x3 window,
    different strides per axis, more than 64 output channels, residual-free RESCALE with small shifts."""
    r = rng(5)
    g = GraphBuilder()
    x = g.input(np.int8, (3, 9, 10, 128))
    wt = g.constant(r.integers(-128, 128, (80, 2, 3, 128), dtype=np.int8))
    b = g.constant(r.integers(-(1 << 14), 1 << 14, (80,), dtype=np.int32))
    y = g.conv2d(x, wt, b, [0, 1, 2, 0], [1, 2], [1, 1], 9, 0)
    mult = r.integers(1 << 30, (1 << 31) - 1, (80,), dtype=np.int64).astype(np.int32)
    y = g.rescale(y, mult, r.integers(28, 44, (80,), dtype=np.int8), 0, -1, np.int8, True, True, True)
    g.output(y)
    check(mlel, g, [r.integers(-128, 128, (3, 9, 10, 128), dtype=np.int8)])


@pytest.mark.parametrize("double_round", [False, True])
@pytest.mark.parametrize("bias_bits", [12, 29, 31])
def test_conv2d_channel_major_bias_range_and_rounding(mlel, bias_bits, double_round):
    """The channel-major kernel's short RESCALE form applies when accumulator + correction cannot leave int32;
    biases of 2^31 make the convolution's int32 output wrap (conv2d.comp adds the bias in 32 bits) and take the
    general form.  Both rounding modes, shifts from 32 up, a negative zero point, with and without a border."""
    r = rng(bias_bits + double_round)
    lim = (1 << bias_bits) - 1
    for k, pad in ((1, 0), (3, 1)):
        g = GraphBuilder()
        x = g.input(np.int8, (2, 14, 14, 128))
        wt = g.constant(r.integers(-128, 128, (160, k, k, 128), dtype=np.int8))
        bias = r.integers(-lim - 1, lim + 1, (160,), dtype=np.int64).astype(np.int32)
        bias[:4] = [lim, -lim - 1, 0, -1]
        y = g.conv2d(x, wt, g.constant(bias), [pad] * 4, [1, 1], [1, 1], -128, 0)
        mult = r.integers(1 << 30, (1 << 31) - 1, (160,), dtype=np.int64).astype(np.int32)
        mult[5:8] = -mult[5:8]
        shift = r.integers(32, 48, (160,), dtype=np.int8)
        shift[:3] = [32, 33, 62]
        g.output(g.rescale(y, mult, shift, 0, -9, np.int8, True, double_round, True))
        data = r.integers(-128, 128, (2, 14, 14, 128), dtype=np.int8)
        data[0, :2] = -128
        data[1, :2] = 127
        check(mlel, g, [data])


@pytest.mark.parametrize("clamp", [None, (-9, 127), (-3, 100), (-20, 127)])
@pytest.mark.parametrize("double_round", [False, True])
def test_conv2d_rescale_from_32_bit_words(mlel, double_round, clamp):
    """Small corrections and shifts of 32 to 60 in all 32 channels of an epilogue warp take the RESCALE form that
    only uses the high word of (4x) * multiplier; with a lower clamp bound at or above the output zero point it also
    drops the sign of x from the double rounding.  Groups of 32 channels: shifts at both ends of the range, shifts
    outside it (those warps take the 64-bit form), negative, tiny and zero multipliers; accumulators of both signs
    and of zero (bias 0, zero weights)."""
    r = rng(40 + double_round + (0 if clamp is None else clamp[0] + clamp[1]))
    oc = 288
    for k, pad in ((1, 0), (3, 1)):
        g = GraphBuilder()
        x = g.input(np.int8, (3, 12, 12, 64))
        w = r.integers(-128, 128, (oc, k, k, 64), dtype=np.int8)
        w[40:44] = 0
        bias = r.integers(-(1 << 16), 1 << 16, (oc,), dtype=np.int32)
        bias[40:42] = 0
        y = g.conv2d(x, g.constant(w), g.constant(bias), [pad] * 4, [1, 1], [1, 1], -5, 0)
        mult = r.integers(1 << 30, (1 << 31) - 1, (oc,), dtype=np.int64).astype(np.int32)
        shift = r.integers(32, 47, (oc,), dtype=np.int8)
        shift[32:64] = 32
        shift[64:96] = r.integers(55, 61, (32,))
        shift[64:66] = 60
        shift[96:128] = r.integers(30, 64, (32,))    # a warp with shifts outside 32..60
        mult[128:160] = -mult[128:160]               # negative multipliers: the sign of x stays
        mult[160:192] = r.integers(0, 1 << 20, (32,))
        mult[160:163] = [0, 1, 2]
        shift[160:192] = r.integers(32, 40, (32,))
        shift[192:224] = 33
        mult[192:224] = (1 << 31) - 1
        shift[224:256] = 61                          # just past the range
        y = g.rescale(y, mult, shift, 0, -9, np.int8, True, double_round, True)
        if clamp is not None:
            y = g.clamp(y, clamp[0], clamp[1])
        g.output(y)
        data = r.integers(-128, 128, (3, 12, 12, 64), dtype=np.int8)
        data[0, :3] = -5  # x - zero point = 0: accumulators of exactly the bias
        check(mlel, g, [data])


@pytest.mark.parametrize("clamp", [None, (-9, 127), (-20, 100)])
@pytest.mark.parametrize("double_round", [False, True])
@pytest.mark.parametrize("odd_one", [None, "shift 61", "shift 31", "negative multiplier"])
def test_conv2d_64_channels_rescale_from_32_bit_words(mlel, odd_one, double_round, clamp):
    """The same form in the pixel-major kernel (at most 64 output channels), where all columns of a tile share one
    form of the constants table: every shift in 32..60, or one column just outside the range, or one negative
    multiplier (which keeps the sign of x in the double rounding)."""
    r = rng(70 + double_round + (0 if clamp is None else clamp[0]) + (0 if odd_one is None else len(odd_one)))
    for oc, k, pad in ((64, 1, 0), (48, 3, 1)):
        g = GraphBuilder()
        x = g.input(np.int8, (2, 13, 13, 32))
        w = r.integers(-128, 128, (oc, k, k, 32), dtype=np.int8)
        w[7] = 0
        bias = r.integers(-(1 << 16), 1 << 16, (oc,), dtype=np.int32)
        bias[7] = 0
        y = g.conv2d(x, g.constant(w), g.constant(bias), [pad] * 4, [1, 1], [1, 1], -5, 0)
        mult = r.integers(1 << 30, (1 << 31) - 1, (oc,), dtype=np.int64).astype(np.int32)
        mult[:3] = [0, 1, (1 << 31) - 1]
        shift = r.integers(32, 61, (oc,), dtype=np.int8)
        shift[3:6] = [32, 33, 60]
        if odd_one == "shift 61":
            shift[20] = 61
        elif odd_one == "shift 31":
            shift[20] = 31
        elif odd_one == "negative multiplier":
            mult[20] = -mult[20]
        y = g.rescale(y, mult, shift, 0, -9, np.int8, True, double_round, True)
        if clamp is not None:
            y = g.clamp(y, clamp[0], clamp[1])
        g.output(y)
        data = r.integers(-128, 128, (2, 13, 13, 32), dtype=np.int8)
        data[0, :3] = -5
        check(mlel, g, [data])


def test_conv2d_int16_int64(mlel):
    r = rng(2)
    g = GraphBuilder()
    x = g.input(np.int16, (1, 5, 5, 4))
    wt = g.constant(r.integers(-128, 128, (6, 3, 3, 4), dtype=np.int8))
    b = g.constant(r.integers(-1000, 1000, (6,), dtype=np.int64))
    g.output(g.conv2d(x, wt, b, [1] * 4, [1, 1], [1, 1], 0, 0, acc_type=4))
    check(mlel, g, [r.integers(-32768, 32768, (1, 5, 5, 4), dtype=np.int16)])


@pytest.mark.parametrize("case", [
    (1, 8, 8, 4, 1, 3, 1, 1, 1, -3, 0), (2, 9, 9, 5, 2, 3, 1, 2, 1, 4, 2), (1, 16, 16, 32, 1, 3, 1, 1, 1, -128, 0),
    (1, 7, 6, 3, 3, 2, 0, 1, 2, -128, -1), (2, 14, 14, 96, 1, 3, 1, 2, 1, -128, 0),
    # the vectorised 3x3 kernel: weight zero point, widths that end inside a 4-pixel group, no padding
    (1, 10, 10, 8, 1, 3, 1, 1, 1, 5, -3), (1, 11, 13, 12, 1, 3, 1, 2, 1, -7, 2), (2, 9, 9, 16, 1, 3, 0, 1, 1, 3, 0),
    (3, 28, 28, 144, 1, 3, 1, 1, 1, -128, 0),
])
@pytest.mark.parametrize("with_rescale", [False, True])
def test_depthwise_conv2d(mlel, case, with_rescale):
    n, h, w, c, m, k, pad, stride, dil, in_zp, w_zp = case
    r = rng(hash(case) & 0xFFFF)
    g = GraphBuilder()
    x = g.input(np.int8, (n, h, w, c))
    wt = g.constant(r.integers(-128, 128, (k, k, c, m), dtype=np.int8))
    b = g.constant(r.integers(-(1 << 14), 1 << 14, (c * m,), dtype=np.int32))
    y = g.depthwise_conv2d(x, wt, b, [pad] * 4, [stride] * 2, [dil] * 2, in_zp, w_zp)
    if with_rescale:
        mult = r.integers(1 << 30, (1 << 31) - 1, (c * m,), dtype=np.int64).astype(np.int32)
        shift = r.integers(34, 40, (c * m,), dtype=np.int8)
        y = g.clamp(g.rescale(y, mult, shift, 0, -128, np.int8, True, True, True), -128, 64)
    g.output(y)
    check(mlel, g, [r.integers(-128, 128, (n, h, w, c), dtype=np.int8)])


@pytest.mark.parametrize("shape", [(1, 4, 8, 4), (3, 5, 7, 9), (2, 16, 33, 16), (1, 1, 1, 1), (2, 128, 64, 128),
                                   (1, 130, 200, 72), (4, 64, 1024, 64), (3, 100, 48, 80), (2, 70, 32, 272),
                                   (5, 384, 64, 384)])
@pytest.mark.parametrize("zps", [(0, 0), (-7, 0), (5, -3)])
@pytest.mark.parametrize("with_rescale", [False, True])
def test_matmul(mlel, shape, zps, with_rescale):
    n, h, c, w = shape
    r = rng(3)
    g = GraphBuilder()
    a = g.input(np.int8, (n, h, c))
    b = g.input(np.int8, (n, c, w))
    y = g.matmul(a, b, *zps)
    if with_rescale:
        y = g.rescale(y, [int(r.integers(1 << 30, 1 << 31))], [38], 0, 0, np.int8, True, False, False)
    g.output(y)
    check(mlel, g, [r.integers(-128, 128, (n, h, c), dtype=np.int8), r.integers(-128, 128, (n, c, w), dtype=np.int8)])


def test_matmul_constant_weights_per_channel(mlel):
    r = rng(4)
    g = GraphBuilder()
    a = g.input(np.int8, (1, 6, 96))
    b = g.constant(r.integers(-128, 128, (1, 96, 40), dtype=np.int8))
    y = g.matmul(a, b, -20, 0)
    mult = r.integers(1 << 30, (1 << 31) - 1, (40,), dtype=np.int64).astype(np.int32)
    y = g.rescale(y, mult, np.full(40, 39, np.int8), 0, 3, np.int8, True, True, True)
    g.output(y)
    check(mlel, g, [r.integers(-128, 128, (1, 6, 96), dtype=np.int8)])


@pytest.mark.parametrize("shift", [0, 1, 2, 30, 31, 32, 33, 40, 62])
@pytest.mark.parametrize("double_round", [False, True])
@pytest.mark.parametrize("per_channel", [False, True])
def test_rescale_i32_to_i8(mlel, shift, double_round, per_channel):
    r = rng(shift * 4 + double_round * 2 + per_channel)
    c = 6
    data = r.integers(-(1 << 31), 1 << 31, (3, 5, c), dtype=np.int64).astype(np.int32)
    data[0, 0, :] = [0, 1, -1, 2**31 - 1, -(2**31), 12345]
    n = c if per_channel else 1
    mult = r.integers(1 << 30, (1 << 31) - 1, (n,), dtype=np.int64).astype(np.int32)
    sh = np.full((n,), shift, np.int8)
    if per_channel and shift >= 2:
        sh[1::2] -= 1
    g = GraphBuilder()
    x = g.input(np.int32, data.shape)
    g.output(g.rescale(x, mult, sh, 0, 5, np.int8, True, double_round, per_channel))
    check(mlel, g, [data], modes=(0,))


@pytest.mark.parametrize("in_dtype,out_dtype,in_zp,out_zp", [
    (np.int8, np.int32, -7, 0), (np.int8, np.int8, 3, -128), (np.int16, np.int8, 100, 7),
    (np.int32, np.int16, 0, -5), (np.int8, np.int16, -128, 32767), (np.int32, np.int32, 11, -11),
])
def test_rescale_types(mlel, in_dtype, out_dtype, in_zp, out_zp):
    r = rng(9)
    info = np.iinfo(in_dtype)
    data = r.integers(info.min, int(info.max) + 1, (4, 7), dtype=np.int64).astype(in_dtype)
    g = GraphBuilder()
    x = g.input(in_dtype, data.shape)
    g.output(g.rescale(x, [int(r.integers(1 << 30, (1 << 31) - 1))], [23], in_zp, out_zp, out_dtype, True, True))
    check(mlel, g, [data], modes=(0,))


def test_residual_add_pattern(mlel):
    r = rng(10)
    for shape in [(2, 7, 7, 24), (1, 3, 5, 7), (1, 1, 1, 1), (4, 14, 14, 256)]:
        g = GraphBuilder()
        a = g.input(np.int8, shape)
        b = g.input(np.int8, shape)
        ta = g.rescale(a, [int(r.integers(1 << 30, 1 << 31))], [23], -7, 0, np.int32)
        tb = g.rescale(b, [int(r.integers(1 << 30, 1 << 31))], [23], 3, 0, np.int32)
        y = g.rescale(g.add(ta, tb), [int(r.integers(1 << 30, 1 << 31))], [40], 0, -20, np.int8, True, True)
        g.output(g.clamp(y, -20, 127))
        check(mlel, g, [r.integers(-128, 128, shape, dtype=np.int8), r.integers(-128, 128, shape, dtype=np.int8)])


@pytest.mark.parametrize("oc", [32, 160])            # pixel-major kernel / channel-major kernel with the residual table
@pytest.mark.parametrize("main_first", [True, False])  # ADD(main, shortcut) and ADD(shortcut, main)
@pytest.mark.parametrize("main_clamp", [False, True])  # a CLAMP between the convolution's RESCALE and the add
def test_conv_with_fused_residual_tail(mlel, oc, main_first, main_clamp):
    """CONV2D -> RESCALE [-> CLAMP] -> RESCALE, RESCALE(shortcut) -> ADD -> RESCALE -> CLAMP is one kernel; all
    three tail RESCALEs with their own zero points, multipliers and rounding modes, shortcut bytes over the whole
    int8 range, against the one-kernel-per-operator oracle."""
    from mlel_b200.runtime import GraphRunner
    r = rng(oc + 2 * main_first + main_clamp)
    g = GraphBuilder()
    x = g.input(np.int8, (3, 14, 14, 64))
    sc = g.input(np.int8, (3, 14, 14, oc))
    wt = g.constant(r.integers(-128, 128, (oc, 1, 1, 64), dtype=np.int8))
    b = g.constant(r.integers(-(1 << 14), 1 << 14, (oc,), dtype=np.int32))
    y = g.conv2d(x, wt, b, [0] * 4, [1, 1], [1, 1], -20, 0)
    mult = r.integers(1 << 30, (1 << 31) - 1, (oc,), dtype=np.int64).astype(np.int32)
    y = g.rescale(y, mult, r.integers(34, 40, (oc,), dtype=np.int8), 0, -7, np.int8, True, True, True)
    if main_clamp:
        y = g.clamp(y, -100, 90)
    ta = g.rescale(y, [int(r.integers(1 << 30, 1 << 31))], [22], -7, 11, np.int32, True, False)
    tb = g.rescale(sc, [int(r.integers(1 << 30, 1 << 31))], [24], 3, -5, np.int32, True, True)
    s = g.add(ta, tb) if main_first else g.add(tb, ta)
    out = g.rescale(s, [int(r.integers(1 << 30, 1 << 31))], [39], 2, -20, np.int8, True, True)
    g.output(g.clamp(out, -20, 127))
    assert GraphRunner(g).pipeline.exec_names() == ["CONV2D+RESCALE" + ("+CLAMP" if main_clamp else "") +
                                                     "+ADD+RESCALE+CLAMP"]
    shortcut = r.integers(-128, 128, (3, 14, 14, oc), dtype=np.int8)
    shortcut[0, 0, :, :] = -20  # many equal shortcut bytes in one warp (what a ReLU leaves behind)
    check(mlel, g, [r.integers(-128, 128, (3, 14, 14, 64), dtype=np.int8), shortcut])


@pytest.mark.parametrize("case", [
    ((1, 7, 7, 5), (7, 7), (7, 7), (0, 0, 0, 0), -20, -20), ((2, 8, 9, 3), (3, 3), (2, 2), (1, 1, 1, 1), 0, 0),
    ((1, 6, 6, 4), (2, 3), (1, 2), (0, 1, 1, 1), 5, -3), ((4, 7, 7, 2048), (7, 7), (7, 7), (0, 0, 0, 0), -20, -20),
    # large windows on 16-channel multiples (block-per-pixel kernel): padded borders with fewer in-range taps,
    # overlapping windows, a channel count that ends inside a 128-channel chunk, saturating zero points
    ((2, 11, 13, 16), (5, 5), (2, 2), (2, 2, 2, 2), 7, -5), ((1, 14, 14, 144), (4, 4), (3, 3), (1, 0, 0, 1), -128, 127),
    ((3, 7, 7, 1280), (7, 7), (7, 7), (0, 0, 0, 0), 0, 0),
])
def test_avg_pool2d(mlel, case):
    shape, k, s, p, in_zp, out_zp = case
    g = GraphBuilder()
    x = g.input(np.int8, shape)
    g.output(g.avg_pool2d(x, k, s, p, in_zp, out_zp))
    check(mlel, g, [rng(2).integers(-128, 128, shape, dtype=np.int8)], modes=(0,))


@pytest.mark.parametrize("case", [
    ((1, 16, 16, 3), (2, 2), (2, 2), (0, 0, 0, 0)), ((2, 9, 9, 5), (3, 3), (2, 2), (1, 1, 1, 1)),
    ((1, 7, 5, 2), (3, 2), (1, 1), (1, 0, 0, 1)), ((2, 56, 56, 64), (3, 3), (2, 2), (1, 1, 1, 1)),
    # the 16-channel-group kernel: its 2x2 variant, and the any-window variant with an even and an odd tap count
    ((2, 12, 12, 16), (2, 2), (2, 2), (0, 0, 0, 0)), ((1, 9, 10, 32), (3, 2), (1, 2), (1, 0, 0, 1)),
    ((1, 8, 8, 48), (5, 5), (1, 1), (2, 2, 2, 2)),
    # 3x3: stride 1, stride 2 with an odd output width (one output per thread), stride 2 without padding (two)
    ((1, 10, 10, 16), (3, 3), (1, 1), (1, 1, 1, 1)), ((1, 9, 9, 16), (3, 3), (2, 2), (1, 1, 1, 1)),
    ((2, 9, 13, 32), (3, 3), (2, 2), (0, 0, 0, 0)),
    # stride 2, even output width and odd output height (two outputs per thread); even both ways with padding (four)
    ((1, 11, 13, 16), (3, 3), (2, 2), (0, 0, 0, 0)), ((3, 12, 20, 48), (3, 3), (2, 2), (1, 1, 1, 1)),
])
def test_max_pool2d(mlel, case):
    shape, k, s, p = case
    g = GraphBuilder()
    x = g.input(np.int8, shape)
    g.output(g.max_pool2d(x, k, s, p))
    check(mlel, g, [rng(6).integers(-128, 128, shape, dtype=np.int8)], modes=(0,))


def test_table(mlel):
    r = rng(7)
    g = GraphBuilder()
    x = g.input(np.int8, (3, 50, 16))
    g.output(g.table(x, r.integers(-128, 128, (256,), dtype=np.int8)))
    check(mlel, g, [r.integers(-128, 128, (3, 50, 16), dtype=np.int8)], modes=(0,))
    g = GraphBuilder()
    x = g.input(np.int16, (3, 50))
    g.output(g.table(x, r.integers(-32768, 32768, (513,), dtype=np.int16)))
    data = r.integers(-32768, 32768, (3, 50), dtype=np.int16)
    data[0, :4] = [-32768, 32767, 0, -1]
    check(mlel, g, [data], modes=(0,))


@pytest.mark.parametrize("shape,perms", [((2, 3, 4), (2, 0, 1)), ((4, 12, 6, 8), (0, 2, 1, 3)), ((5, 7), (1, 0)),
                                         ((2, 3, 4, 5, 6, 2), (5, 3, 1, 0, 2, 4)), ((2, 384, 12, 64), (0, 2, 1, 3))])
@pytest.mark.parametrize("dtype", [np.int8, np.int32])
def test_transpose(mlel, shape, perms, dtype):
    g = GraphBuilder()
    x = g.input(dtype, shape)
    g.output(g.transpose(x, perms))
    check(mlel, g, [rng(8).integers(-128, 128, shape).astype(dtype)], modes=(0,))


def test_data_movement(mlel):
    r = rng(11)
    g = GraphBuilder()
    a = g.input(np.int8, (2, 3, 4, 5))
    b = g.input(np.int8, (2, 2, 4, 5))
    c = g.concat([a, b, a], 1)
    d = g.reshape(c, (2, 8, 20))
    e = g.slice(d, (0, 1, 3), (2, 5, 9))
    f = g.pad(e, [0, 1, 2, 0, 1, 1], -9)
    g.output(f)
    g.output(g.cast(f, np.int32))
    check(mlel, g, [r.integers(-128, 128, (2, 3, 4, 5), dtype=np.int8), r.integers(-128, 128, (2, 2, 4, 5), dtype=np.int8)],
          modes=(0,))


def test_elementwise_integer(mlel):
    r = rng(12)
    g = GraphBuilder()
    a = g.input(np.int32, (3, 4, 5))
    b = g.input(np.int32, (3, 1, 5))   # broadcast along axis 1
    for name in ("ADD", "SUB", "BITWISE_AND", "BITWISE_OR", "BITWISE_XOR", "MAXIMUM", "MINIMUM", "EQUAL", "GREATER",
                 "GREATER_EQUAL", "LOGICAL_LEFT_SHIFT", "LOGICAL_RIGHT_SHIFT", "INTDIV"):
        g.output(g.binary(name, a, b))
    g.output(g.mul(a, b, 0))
    g.output(g.mul(a, b, 5))
    g.output(g.clamp(a, -1000, 5000))
    g.output(g.negate(a, 3, -4))
    for name in ("ABS", "BITWISE_NOT", "CLZ"):
        g.output(g.unary(name, a))
    g.output(g.reduce("REDUCE_SUM", a, 1))
    g.output(g.reduce("REDUCE_MAX", a, 2))
    g.output(g.reduce("REDUCE_MIN", a, 0))
    da = r.integers(-(1 << 31), 1 << 31, (3, 4, 5), dtype=np.int64).astype(np.int32)
    db = r.integers(-40, 40, (3, 1, 5), dtype=np.int64).astype(np.int32)
    db[0, 0, 0] = 0
    check(mlel, g, [da, db], modes=(0,))


def test_elementwise_int8_and_shifts(mlel):
    r = rng(13)
    g = GraphBuilder()
    a = g.input(np.int8, (4, 33))
    s = g.input(np.int8, (4, 33))
    g.output(g.add(a, s))
    g.output(g.arithmetic_right_shift(a, s, True))
    g.output(g.arithmetic_right_shift(a, s, False))
    g.output(g.reduce("REDUCE_SUM", a, 1))
    c = g.binary("GREATER", a, s)
    g.output(g.select(c, a, s))
    g.output(g.unary("LOGICAL_NOT", c))
    check(mlel, g, [r.integers(-128, 128, (4, 33), dtype=np.int8), r.integers(0, 8, (4, 33), dtype=np.int8)], modes=(0,))
