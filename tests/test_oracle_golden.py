"""Pins the CPU oracle to the golden vectors of the reference's own tests.

The expected arrays in ``tests/golden/reference_goldens.json`` were extracted from the reference's
``tests/vulkan.cpp`` by ``tests/golden/extract_reference_goldens.py``.  Inputs and operator
attributes are restated here from the named test and its SPIR-V fixture (path:line in the
reference project).
"""
import json
import os

import numpy as np
import pytest

from oracle import oracle

with open(os.path.join(os.path.dirname(__file__), "golden", "reference_goldens.json")) as f:
    GOLD = json.load(f)


def gold(name):
    g = GOLD[name]
    return np.array(g["values"], dtype=g["dtype"]).reshape(g["shape"])


def iota_i8(shape):
    # std::iota over the bytes of an int8 tensor, wrapping at 256 (tests/vulkan.cpp:1002)
    return (np.arange(int(np.prod(shape))) & 0xFF).astype(np.uint8).view(np.int8).reshape(shape)


def test_conv2d():
    # tests/vulkan.cpp:998-1089 + tests/shader/conv2d.spvasm: pad 0, stride 2, dilation 1, zero points 0
    x = iota_i8((1, 8, 8, 3))
    w = np.ones((3, 2, 2, 3), np.int8)
    bias = np.array([0, 1, 2], np.int32)
    out = oracle.conv2d(x, w, bias, [0, 0, 0, 0], [2, 2], [1, 1], 0, 0)
    np.testing.assert_array_equal(out, gold("Conv2D"))
    np.testing.assert_array_equal(oracle.conv2d(x, w, bias, [0, 0, 0, 0], [2, 2], [1, 1], 0, 0, generic=True),
                                  gold("Conv2D"))


def test_conv2d_int64_accumulator():
    # tests/vulkan.cpp:1158-1209 + tests/shader/conv2_acc_int64.spvasm: int16 x int8 -> int64, 1x1
    x = np.arange(1, 17, dtype=np.int16).reshape(1, 2, 2, 4)
    w = np.array([1, 2, 3, 4, -1, 0, 1, 2, 2, -3, 4, -5, -2, -1, 0, 1], np.int8).reshape(4, 1, 1, 4)
    bias = np.array([10, -20, 30, -40], np.int64)
    out = oracle.conv2d(x, w, bias, [0, 0, 0, 0], [1, 1], [1, 1], 0, 0)
    np.testing.assert_array_equal(out, gold("Conv2DAccumulatorInt64"))


@pytest.mark.parametrize("axis", ["oc", "h", "w"])
def test_conv2d_large_dimension(axis):
    # tests/vulkan.cpp:1091-1156 (conv2d_large_*.spvasm): all-ones 2x2x1 kernel over all-ones input -> 4.
    # The reference uses 262144 channels / 524281 rows to cross Vulkan's grid limits; grid splitting
    # does not exist here, so a reduced size of the same structure pins the arithmetic.
    if axis == "oc":
        x = np.ones((1, 2, 2, 1), np.int8)
        w = np.ones((4099, 2, 2, 1), np.int8)
    elif axis == "h":
        x = np.ones((1, 4099, 2, 1), np.int8)
        w = np.ones((1, 2, 2, 1), np.int8)
    else:
        x = np.ones((1, 2, 4099, 1), np.int8)
        w = np.ones((1, 2, 2, 1), np.int8)
    bias = np.zeros((w.shape[0],), np.int32)
    out = oracle.conv2d(x, w, bias, [0, 0, 0, 0], [1, 1], [1, 1], 0, 0)
    assert (out == 4).all()


def test_higher_rank_constant():
    # tests/vulkan.cpp:1636-1678 + inlined-higher-rank-constant.spvasm: 3x3 weights 0..8, pad 1, then CAST
    x = np.ones((1, 3, 3, 1), np.int8)
    w = np.arange(9, dtype=np.int8).reshape(1, 3, 3, 1)
    bias = np.zeros((1,), np.int32)
    acc = oracle.conv2d(x, w, bias, [1, 1, 1, 1], [1, 1], [1, 1], 0, 0)
    out = oracle.cast(acc, np.int8)
    np.testing.assert_array_equal(out, gold("HigherRankConstant"))


def test_rescale_add_rescale():
    # tests/vulkan.cpp:1579-1634 + graph-constant-arm.spvasm: scale32, SINGLE_ROUND, per-tensor, shift 0
    x0 = np.arange(5, dtype=np.int8)
    x1 = np.arange(5, dtype=np.int8)
    a = oracle.rescale(x0, np.array([2], np.int32), np.array([0], np.int8), 0, 0, np.int32)
    b = oracle.rescale(x1, np.array([3], np.int32), np.array([0], np.int8), 0, 0, np.int32)
    s = oracle.binary("ADD", a, b)
    out = oracle.rescale(s, np.array([4], np.int32), np.array([0], np.int8), 0, 0, np.int8)
    np.testing.assert_array_equal(out, gold("GraphConstantARM"))


def _maxpool_input():
    # tests/vulkan.cpp:632-634: channel 0 of pixel p holds -128 + p, other channels 0
    x = np.zeros((1, 16, 16, 3), np.int8)
    x[0, :, :, 0] = (np.arange(256) - 128).astype(np.int8).reshape(16, 16)
    return x


def test_max_pool2d():
    out = oracle.max_pool2d(_maxpool_input(), [2, 2], [2, 2], [0, 0, 0, 0])
    np.testing.assert_array_equal(out, gold("MaxPool2D"))


def test_two_layer_max_pool2d():
    mid = oracle.max_pool2d(_maxpool_input(), [2, 2], [2, 2], [0, 0, 0, 0])
    out = oracle.max_pool2d(mid, [2, 2], [2, 2], [0, 0, 0, 0])
    np.testing.assert_array_equal(out, gold("TwoLayerMaxPool2D"))


def test_concat():
    # tests/vulkan.cpp:1333-1404 + concat.spvasm: axis 1
    x = iota_i8((1, 2, 2, 2))
    np.testing.assert_array_equal(oracle.concat([x, x], 1), gold("Concat"))


def test_concat_interval():
    # tests/vulkan.cpp:1406-1439 + concat_interval.spvasm: ADD fp32, CONCAT axis 1, RESHAPE to [12]
    x = np.arange(9, dtype=np.float32).reshape(3, 3)
    one = np.ones((3, 3), np.float32)
    zero = np.zeros((3, 1), np.float32)
    s = oracle.binary("ADD", x, one)
    c = oracle.concat([s, zero], 1)
    np.testing.assert_array_equal(oracle.reshape(c, (12,)), gold("ConcatMultipleDispatchesPreserveInputLiveRange"))


def test_slice():
    # tests/vulkan.cpp:1441-1492 + slice.spvasm: start (0,4,4,1), size (1,2,2,2)
    x = iota_i8((1, 8, 8, 3))
    np.testing.assert_array_equal(oracle.slice_(x, [0, 4, 4, 1], [1, 2, 2, 2]), gold("Slice"))
    np.testing.assert_array_equal(oracle.slice_(x, [0, 4, 4, 1], [1, 2, 2, 2]), gold("NOPOutputs"))


def test_maximum():
    # tests/vulkan.cpp:1680-1744 + maximum.spvasm (int32)
    a = np.arange(8, dtype=np.int32).reshape(1, 2, 2, 2)
    b = (np.arange(8, dtype=np.int64) * 4 - 16).astype(np.int32).reshape(1, 2, 2, 2)
    np.testing.assert_array_equal(oracle.binary("MAXIMUM", a, b), gold("Maximum"))


def test_conv3d_large_stride_and_pad():
    # tests/vulkan.cpp:1211-1293 + tests/shader/conv3d_large_stride.spvasm: input [1,3,2,2,4] all -128 with zero
    # point 9; weights [3,2,2,8192,4] zero except the last two taps of the 8192-wide kernel, which hold
    # `relevantWeights` in blocks of 8 per (oc, kd, kh); pad (1,0, 1,0, 8190,8192), stride (1,1,8192).
    rel = gold("Conv3DLargeStridePadRegression.relevantWeights")
    w = np.zeros((3, 2, 2, 8192, 4), np.int8)
    for oc in range(3):
        for kd in range(2):
            for kh in range(2):
                base = ((oc * 2 + kd) * 2 + kh) * 8
                w[oc, kd, kh, 8190, :] = rel[base:base + 4]
                w[oc, kd, kh, 8191, :] = rel[base + 4:base + 8]
    x = np.full((1, 3, 2, 2, 4), -128, np.int8)
    bias = np.zeros((1,), np.int32)
    out = oracle.conv3d(x, w, bias, (1, 3, 2, 2, 3), [1, 0, 1, 0, 8190, 8192], [1, 1, 8192], [1, 1, 1], 9, 0)
    np.testing.assert_array_equal(out, gold("Conv3DLargeStridePadRegression"))


def test_sin_known_answer():
    # tests/vulkan.cpp:1795-1841: sin(0.000111731846f) must lie within 7.715463482888105e-08 of 0.00011173184588586903
    out = oracle.unary("SIN", np.array([0.000111731846], np.float32))
    assert out.dtype == np.float32
    assert abs(float(out[0]) - 0.00011173184588586903) <= 7.715463482888105e-08
