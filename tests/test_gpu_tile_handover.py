"""Tile-level hand-over between consecutive tensor-core convolutions, against the CPU oracle, bit-exact.

A channel-major convolution whose pixel operand is the output of the convolution launched just before it does not
wait for that whole launch: the producer counts every finished (pixel tile, channel tile) in a table, and the
consumer starts a tile as soon as the pixel tiles under its windows are complete (and stores nothing before the
producer has ended).  These graphs are chains of exactly such convolutions, sized so that a launch has several
rounds of tiles per SM (the hand-over then overlaps the producer's last round) or fewer tiles than SMs (it then
starts on the idle SMs): 1x1, 3x3 with padding, stride 2, residual tails whose shortcut comes from three launches
back, pixel counts that end inside a tile.  Every graph is run with the hand-over on and off, plain and as a
replayed CUDA graph (where the counters must be cleared by every replay), several times in a row.
"""
import numpy as np
import pytest

from mlel_b200.graph_builder import GraphBuilder
from tests.graph_eval import evaluate

pytestmark = pytest.mark.gpu


def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def _conv(g, r, x, oc, k, pad, stride, in_zp, out_zp, relu=True):
    ic = x.shape[3]
    wt = g.constant(r.integers(-128, 128, (oc, k, k, ic), dtype=np.int8))
    b = g.constant(r.integers(-(1 << 12), 1 << 12, (oc,), dtype=np.int32))
    y = g.conv2d(x, wt, b, [pad] * 4, [stride] * 2, [1, 1], in_zp, 0)
    mult = r.integers(1 << 30, (1 << 31) - 1, (oc,), dtype=np.int64).astype(np.int32)
    shift = r.integers(38, 43, (oc,), dtype=np.int8)
    y = g.rescale(y, mult, shift, 0, out_zp, np.int8, True, True, True)
    return g.clamp(y, out_zp, 127) if relu else y


def _residual(g, r, main, shortcut, zp_main, zp_short, out_zp):
    a = g.rescale(main, [int(r.integers(1 << 30, 1 << 31))], [23], zp_main, 0, np.int32)
    b = g.rescale(shortcut, [int(r.integers(1 << 30, 1 << 31))], [23], zp_short, 0, np.int32)
    y = g.rescale(g.add(a, b), [int(r.integers(1 << 30, 1 << 31))], [39], 0, out_zp, np.int8, True, True)
    return g.clamp(y, out_zp, 127)


def bottleneck_chain(seed, n, hw, width, blocks, stride_first=1):
    """`blocks` bottleneck blocks (1x1 reduce, 3x3, 1x1 expand + residual tail) behind a 1x1 convolution that makes the
    first block's input; 4 * width channels between the blocks."""
    r = rng(seed)
    g = GraphBuilder()
    x = g.input(np.int8, (n, hw, hw, 64))
    y = _conv(g, r, x, 4 * width, 1, 0, 1, 3, -7)
    for b in range(blocks):
        stride = stride_first if b == 0 else 1
        a = _conv(g, r, y, width, 1, 0, 1, -7, 5)
        c = _conv(g, r, a, width, 3, 1, stride, 5, -3)
        d = _conv(g, r, c, 4 * width, 1, 0, 1, -3, 9, relu=False)
        if stride != 1:
            short = _conv(g, r, y, 4 * width, 1, 0, stride, -7, -7, relu=False)
            y = _residual(g, r, d, short, 9, -7, -7)
        else:
            y = _residual(g, r, d, y, 9, -7, -7)
    g.output(y)
    return g, [r.integers(-128, 128, (n, hw, hw, 64), dtype=np.int8)]


CASES = [
    # seed, images, height = width, bottleneck width, blocks, stride of the first block
    (1, 8, 28, 128, 2, 1),    # 6272 pixels: 33 tiles of 192 x 1 and 4 channel tiles; fewer tiles than SMs, then more
    (2, 20, 28, 128, 1, 1),   # 15680 pixels: 82 pixel tiles, up to 328 tiles per launch (several rounds per SM)
    (3, 3, 30, 128, 1, 2),    # stride 2 in the 3x3 and in the projection; 2700 pixels end inside a tile
    (4, 5, 14, 256, 2, 1),    # 980 pixels: six pixel tiles, 2 and 8 channel tiles
    (5, 33, 7, 256, 1, 1),    # 1617 pixels of 7x7 images: windows of a tile span many images
    # 50176 pixels: the layers with 512 output channels have more than three rounds of tiles per SM and take 256-pixel
    # tiles, the others 192-pixel ones -- producer and consumer of a hand-over count in different tile widths
    (7, 16, 56, 128, 2, 1),
]


def _run(mlel, g, inputs, want, use_cuda_graph, times):
    from mlel_b200.runtime import GraphRunner
    runner = GraphRunner(g)
    for _ in range(times):
        got = runner.run(inputs, use_cuda_graph=use_cuda_graph)
        assert mlel.lib().mlel_device_error() == 0
        for k, (a, b) in enumerate(zip(got, want)):
            if not np.array_equal(a, b):
                bad = np.argwhere(a != b)
                raise AssertionError(f"output {k}: {len(bad)} of {a.size} differ, first at {bad[0].tolist()}, "
                                     f"last at {bad[-1].tolist()}")


@pytest.mark.parametrize("case", CASES)
def test_chain_of_convolutions_with_and_without_the_hand_over(mlel, case):
    g, inputs = bottleneck_chain(*case)
    want = evaluate(g, inputs)
    lib = mlel.lib()
    try:
        for mode in (7, 0, 3):  # on; off; on with the pixel-tile-first order
            assert lib.mlel_set_tuning(b"tile_progress", mode) == 0
            _run(mlel, g, inputs, want, use_cuda_graph=False, times=2)
            _run(mlel, g, inputs, want, use_cuda_graph=True, times=3)
    finally:
        assert lib.mlel_set_tuning(b"tile_progress", 7) == 0


def test_hand_over_is_refused_without_dependent_launch(mlel):
    """Without programmatic dependent launch a kernel only starts when the one before it has ended: the table is not
    used, the results are the same."""
    g, inputs = bottleneck_chain(6, 4, 14, 128, 1, 1)
    want = evaluate(g, inputs)
    lib = mlel.lib()
    try:
        assert lib.mlel_set_tuning(b"dependent_launch", 0) == 0
        _run(mlel, g, inputs, want, use_cuda_graph=False, times=2)
    finally:
        assert lib.mlel_set_tuning(b"dependent_launch", 1) == 0
