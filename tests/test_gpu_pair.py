"""GPU parity of the paired tensor-core kernel (two CTAs of a cluster on one 256-channel tile,
``tcgen05.mma.cta_group::2``) against the CPU oracle, bit-exact, through the C ABI.

Every case checks that the paired kernel is the one that ran (the library counts the launches of its three
tensor-core kernels).  Shapes cover: channel counts that end inside the pair's second CTA or leave it empty,
pixel counts that end inside either half of a tile, tiles that span images, border classes of padded windows,
strides and dilation through the im2col loads, channel counts that are not multiples of 128, the fused
residual tail, and batched matrix products with a run-time second input."""
import numpy as np
import pytest

from mlel_b200.graph_builder import GraphBuilder
from tests.graph_eval import evaluate

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _pair_kernel_for_convolutions(mlel):
    """Convolutions take the paired kernel only on request; these tests request it."""
    lib = mlel.lib()
    assert lib.mlel_set_tuning(b"pair_kernel", 2) == 0
    yield
    assert lib.mlel_set_tuning(b"pair_kernel", 1) == 0


def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def run_and_compare(mlel, g, inputs, expect_pair=True):
    from mlel_b200.runtime import GraphRunner
    lib = mlel.lib()
    lib.mlel_tensor_core_launches.restype = __import__("ctypes").c_longlong
    want = evaluate(g, inputs)
    before = lib.mlel_tensor_core_launches(2)
    runner = GraphRunner(g, flags=0)
    got = runner.run(inputs)
    assert lib.mlel_device_error() == 0
    if expect_pair:
        assert lib.mlel_tensor_core_launches(2) > before, "the paired kernel did not take this case"
    for k, (a, b) in enumerate(zip(got, want)):
        assert a.dtype == b.dtype and a.shape == b.shape
        if not np.array_equal(a, b):
            bad = np.argwhere(a != b)
            raise AssertionError(f"output {k}: {len(bad)} of {a.size} differ, first at {bad[0].tolist()}: "
                                 f"got {a[tuple(bad[0])]} want {b[tuple(bad[0])]}; last at {bad[-1].tolist()}")
    # the same bytes when the captured CUDA graph is replayed
    again = runner.run(inputs, use_cuda_graph=True)
    for a, b in zip(again, want):
        assert np.array_equal(a, b)


def conv_graph(r, n, h, w, ic, oc, k, pad, stride, dil, in_zp, relu=True):
    g = GraphBuilder()
    x = g.input(np.int8, (n, h, w, ic))
    wt = g.constant(r.integers(-128, 128, (oc, k, k, ic), dtype=np.int8))
    b = g.constant(r.integers(-(1 << 14), 1 << 14, (oc,), dtype=np.int32))
    y = g.conv2d(x, wt, b, [pad] * 4, [stride] * 2, [dil] * 2, in_zp, 0)
    mult = r.integers(1 << 30, (1 << 31) - 1, (oc,), dtype=np.int64).astype(np.int32)
    shift = r.integers(36, 46, (oc,), dtype=np.int8)
    y = g.rescale(y, mult, shift, 0, 5, np.int8, True, True, True)
    if relu:
        y = g.clamp(y, -20, 100)
    g.output(y)
    return g


PAIR_CONV_CASES = [
    # n, h, w, ic, oc, k, pad, stride, dil, in_zp
    (2, 14, 14, 128, 256, 1, 0, 1, 1, -7),     # plain matrix, one pair tile of channels
    (1, 7, 7, 256, 512, 1, 0, 1, 1, 3),        # 49 pixels: the second CTA's half of the pixels is empty
    (3, 9, 9, 64, 384, 1, 0, 1, 1, -11),       # 384 channels: the last pair's second CTA has no channels
    (2, 13, 13, 128, 272, 1, 0, 1, 1, 9),      # 272 channels: 16 in the last pair's second CTA
    (5, 14, 14, 256, 256, 3, 1, 1, 1, -5),     # 3x3 window, border classes, tiles spanning images
    (4, 15, 15, 128, 320, 3, 1, 2, 1, 4),      # stride 2 over an odd size
    (2, 12, 12, 128, 256, 3, 2, 1, 2, -9),     # dilation 2
    (3, 10, 10, 48, 288, 3, 1, 1, 1, 6),       # 48 channels: one zero-filled K block per tap
    (2, 11, 11, 160, 256, 3, 1, 1, 1, -3),     # 160 channels: two K blocks per tap, the second partly filled
    (9, 8, 8, 512, 1024, 1, 0, 1, 1, -128),    # four channel pairs, K = 512, extreme zero point
    (16, 14, 14, 256, 256, 1, 0, 2, 1, 7),     # 1x1 with stride 2 (a projection shortcut)
    (1, 40, 40, 32, 256, 3, 1, 1, 1, 2),       # many pixel tiles of one image
]


@pytest.mark.parametrize("case", PAIR_CONV_CASES)
def test_pair_conv2d(mlel, case):
    n, h, w, ic, oc, k, pad, stride, dil, in_zp = case
    r = rng(hash(case) & 0xFFFF)
    g = conv_graph(r, n, h, w, ic, oc, k, pad, stride, dil, in_zp)
    run_and_compare(mlel, g, [r.integers(-128, 128, (n, h, w, ic), dtype=np.int8)])


@pytest.mark.parametrize("width", [128, 192, 256])
@pytest.mark.parametrize("case", [(5, 14, 14, 256, 256, 3, 1, 1, 1, -5), (3, 17, 17, 64, 512, 1, 0, 1, 1, 8)])
def test_pair_conv2d_every_tile_width(mlel, width, case):
    """The three tile widths (normally chosen per problem) on problems whose pixel count ends inside a tile."""
    n, h, w, ic, oc, k, pad, stride, dil, in_zp = case
    r = rng(width + oc)
    g = conv_graph(r, n, h, w, ic, oc, k, pad, stride, dil, in_zp)
    lib = mlel.lib()
    assert lib.mlel_set_tuning(b"pair_tile_pixels", width) == 0
    try:
        run_and_compare(mlel, g, [r.integers(-128, 128, (n, h, w, ic), dtype=np.int8)])
    finally:
        assert lib.mlel_set_tuning(b"pair_tile_pixels", 0) == 0


def test_pair_kernel_can_be_switched_off(mlel):
    """With "pair_kernel" 0 the same graph runs on the single-CTA kernels and gives the same bytes."""
    case = (2, 14, 14, 128, 256, 1, 0, 1, 1, -7)
    n, h, w, ic, oc, k, pad, stride, dil, in_zp = case
    r = rng(77)
    g = conv_graph(r, n, h, w, ic, oc, k, pad, stride, dil, in_zp)
    lib = mlel.lib()
    lib.mlel_tensor_core_launches.restype = __import__("ctypes").c_longlong
    assert lib.mlel_set_tuning(b"pair_kernel", 0) == 0
    try:
        before = lib.mlel_tensor_core_launches(2)
        run_and_compare(mlel, g, [r.integers(-128, 128, (n, h, w, ic), dtype=np.int8)], expect_pair=False)
        assert lib.mlel_tensor_core_launches(2) == before
    finally:
        assert lib.mlel_set_tuning(b"pair_kernel", 2) == 0
    assert lib.mlel_set_tuning(b"pair_tile_pixels", 100) != 0 and lib.mlel_set_tuning(b"no_such_key", 1) != 0
    assert lib.mlel_set_tuning(b"pair_kernel", 3) != 0


def residual_block_graph(r, n, hw, cin, cout, double_round=True):
    """1x1 convolution with the fused residual tail: RESCALE(main), RESCALE(shortcut), ADD, RESCALE, CLAMP."""
    g = GraphBuilder()
    x = g.input(np.int8, (n, hw, hw, cin))
    sc = g.input(np.int8, (n, hw, hw, cout))
    wt = g.constant(r.integers(-128, 128, (cout, 1, 1, cin), dtype=np.int8))
    b = g.constant(r.integers(-(1 << 14), 1 << 14, (cout,), dtype=np.int32))
    y = g.conv2d(x, wt, b, [0] * 4, [1, 1], [1, 1], -4, 0)
    mult = r.integers(1 << 30, (1 << 31) - 1, (cout,), dtype=np.int64).astype(np.int32)
    y = g.rescale(y, mult, r.integers(38, 44, (cout,), dtype=np.int8), 0, 3, np.int8, True, double_round, True)
    ta = g.rescale(y, [int(r.integers(1 << 30, 1 << 31))], [23], 3, 0, np.int32)
    tb = g.rescale(sc, [int(r.integers(1 << 30, 1 << 31))], [23], -9, 0, np.int32)
    z = g.rescale(g.add(ta, tb), [int(r.integers(1 << 30, 1 << 31))], [39], 0, -11, np.int8, True, True)
    g.output(g.clamp(z, -11, 127))
    return g


@pytest.mark.parametrize("shape", [(2, 14, 64, 256), (6, 14, 256, 1024), (33, 7, 512, 2048), (1, 9, 128, 384)])
def test_pair_conv2d_residual_tail(mlel, shape):
    n, hw, cin, cout = shape
    r = rng(n * 1000 + cout)
    g = residual_block_graph(r, n, hw, cin, cout)
    run_and_compare(mlel, g, [r.integers(-128, 128, (n, hw, hw, cin), dtype=np.int8),
                              r.integers(-128, 128, (n, hw, hw, cout), dtype=np.int8)])


@pytest.mark.parametrize("shape", [(2, 70, 32, 272), (5, 384, 64, 384), (3, 200, 128, 256), (1, 1024, 256, 512),
                                   (4, 130, 1024, 640)])
@pytest.mark.parametrize("zps", [(0, 0), (-7, 0)])
def test_pair_matmul_two_runtime_inputs(mlel, shape, zps):
    n, h, c, w = shape
    r = rng(3 + n)
    g = GraphBuilder()
    a = g.input(np.int8, (n, h, c))
    b = g.input(np.int8, (n, c, w))
    y = g.matmul(a, b, *zps)
    y = g.rescale(y, [int(r.integers(1 << 30, 1 << 31))], [38], 0, 0, np.int8, True, False, False)
    g.output(y)
    run_and_compare(mlel, g, [r.integers(-128, 128, (n, h, c), dtype=np.int8),
                              r.integers(-128, 128, (n, c, w), dtype=np.int8)])


def test_pair_matmul_constant_weights_per_channel(mlel):
    r = rng(4)
    g = GraphBuilder()
    a = g.input(np.int8, (1, 300, 768))
    b = g.constant(r.integers(-128, 128, (1, 768, 3072), dtype=np.int8))
    y = g.matmul(a, b, -20, 0)
    mult = r.integers(1 << 30, (1 << 31) - 1, (3072,), dtype=np.int64).astype(np.int32)
    y = g.rescale(y, mult, r.integers(38, 42, (3072,), dtype=np.int8), 0, 3, np.int8, True, True, True)
    g.output(y)
    run_and_compare(mlel, g, [r.integers(-128, 128, (1, 300, 768), dtype=np.int8)])
