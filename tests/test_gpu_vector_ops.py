"""GPU parity of the vectorised element-wise, table, reduction and row-transpose kernels.

The generic kernels take every rank, stride and type; the vectorised ones take packed tensors whose sizes
allow 4-, 8- or 16-byte accesses.  The shapes here are chosen to land on the vectorised kernels (the
operator-by-operator tests in test_gpu_ops.py mostly use small odd shapes that do not); values include the
extremes of each type.  All comparisons are bit-exact against the CPU oracle.
"""
import numpy as np
import pytest

from mlel_b200.graph_builder import GraphBuilder
from tests.graph_eval import evaluate

pytestmark = pytest.mark.gpu


def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def full_range(r, dtype, shape):
    info = np.iinfo(dtype)
    data = r.integers(info.min, int(info.max) + 1, shape, dtype=np.int64).astype(dtype)
    flat = data.reshape(-1)
    extremes = [info.min, info.max, 0, -1]
    flat[:min(4, flat.size)] = extremes[:min(4, flat.size)]
    return data


def check(g, inputs):
    from mlel_b200.runtime import GraphRunner
    want = evaluate(g, inputs)
    got = GraphRunner(g, flags=1).run(inputs)  # no fusion: every operator runs as its own kernel
    assert len(got) == len(want)
    for k, (a, b) in enumerate(zip(got, want)):
        assert a.dtype == b.dtype and a.shape == b.shape
        if not np.array_equal(a, b):
            bad = np.argwhere(a != b)
            raise AssertionError(f"output {k}: {len(bad)} of {a.size} differ, first at {bad[0].tolist()}: "
                                 f"got {a[tuple(bad[0])]} want {b[tuple(bad[0])]}")


@pytest.mark.parametrize("in_dtype,out_dtype", [
    (np.int32, np.int8), (np.int32, np.int16), (np.int32, np.int32), (np.int8, np.int32), (np.int8, np.int8),
    (np.int16, np.int32), (np.int16, np.int16), (np.int16, np.int8), (np.int8, np.int16),
])
@pytest.mark.parametrize("shift,double_round", [(0, False), (23, True), (31, True), (32, True), (45, True), (62, False)])
@pytest.mark.parametrize("per_channel", [False, True])
def test_rescale(mlel, in_dtype, out_dtype, shift, double_round, per_channel):
    r = rng(shift + 7 * per_channel)
    shape = (3, 40, 64)
    data = full_range(r, in_dtype, shape)
    n = shape[-1] if per_channel else 1
    mult = r.integers(1 << 30, (1 << 31) - 1, (n,), dtype=np.int64).astype(np.int32)
    sh = np.full((n,), shift, np.int8)
    if per_channel and shift >= 2:
        sh[1::2] -= 1
        mult[::3] = -mult[::3]  # negative multipliers are legal in the shader arithmetic
    in_zp = int(np.iinfo(in_dtype).max) if in_dtype != np.int32 else -123456789
    g = GraphBuilder()
    x = g.input(in_dtype, shape)
    g.output(g.rescale(x, mult, sh, in_zp, -3, out_dtype, True, double_round, per_channel))
    check(g, [data])


def test_table_int8_and_int16(mlel):
    r = rng(1)
    g = GraphBuilder()
    a = g.input(np.int8, (5, 48, 64))
    b = g.input(np.int16, (5, 48, 64))
    g.output(g.table(a, r.integers(-128, 128, (256,), dtype=np.int8)))
    g.output(g.table(b, r.integers(-32768, 32768, (513,), dtype=np.int16)))
    check(g, [full_range(r, np.int8, (5, 48, 64)), full_range(r, np.int16, (5, 48, 64))])


@pytest.mark.parametrize("b_shape", [(6, 24, 128), (6, 24, 1), (1, 1, 1)])
def test_add_sub_mul_int32(mlel, b_shape):
    r = rng(2)
    shape = (6, 24, 128)
    g = GraphBuilder()
    a = g.input(np.int32, shape)
    b = g.input(np.int32, b_shape)
    g.output(g.add(a, b))
    g.output(g.sub(a, b))
    g.output(g.mul(a, b, 0))
    g.output(g.mul(a, b, 17))
    g.output(g.mul(a, b, 62))
    check(g, [full_range(r, np.int32, shape), full_range(r, np.int32, b_shape)])


def test_clamp_int8(mlel):
    r = rng(3)
    g = GraphBuilder()
    x = g.input(np.int8, (4, 28, 28, 32))
    g.output(g.clamp(x, -20, 127))
    g.output(g.clamp(x, -128, 6))
    check(g, [full_range(r, np.int8, (4, 28, 28, 32))])


@pytest.mark.parametrize("dtype,length", [(np.int32, 384), (np.int32, 4), (np.int32, 768), (np.int16, 136), (np.int8, 400)])
def test_reduce_along_the_last_axis(mlel, dtype, length):
    r = rng(4)
    shape = (3, 37, length)
    g = GraphBuilder()
    x = g.input(dtype, shape)
    if dtype == np.int32:
        g.output(g.reduce("REDUCE_SUM", x, 2))  # wraps modulo 2^32 in any order
    g.output(g.reduce("REDUCE_MAX", x, 2))
    g.output(g.reduce("REDUCE_MIN", x, 2))
    check(g, [full_range(r, dtype, shape)])


@pytest.mark.parametrize("dtype,shape,perms", [
    (np.int8, (2, 48, 4, 64), (0, 2, 1, 3)), (np.int32, (3, 5, 7, 8), (2, 0, 1, 3)), (np.int16, (6, 10, 24), (1, 0, 2)),
    (np.int8, (2, 3, 4, 5, 32), (3, 1, 0, 2, 4)),
])
def test_transpose_that_keeps_the_last_axis(mlel, dtype, shape, perms):
    r = rng(5)
    g = GraphBuilder()
    x = g.input(dtype, shape)
    g.output(g.transpose(x, perms))
    check(g, [full_range(r, dtype, shape)])


@pytest.mark.parametrize("shape,perms", [
    ((2, 48, 4, 64), (0, 2, 3, 1)),   # attention keys: [batch, seq, heads, d] -> [batch, heads, d, seq]
    ((3, 32, 80), (0, 2, 1)), ((80, 144), (1, 0)), ((2, 16, 3, 5, 32), (3, 0, 2, 4, 1)),
])
def test_transpose_that_swaps_the_last_axis_of_bytes(mlel, shape, perms):
    r = rng(6)
    g = GraphBuilder()
    x = g.input(np.int8, shape)
    g.output(g.transpose(x, perms))
    check(g, [full_range(r, np.int8, shape)])


def check_fused(mlel, g, inputs, expect_names):
    """Runs with the fusion pass on; checks that the expected fused nodes were made and compares with the oracle."""
    from mlel_b200.runtime import GraphRunner
    want = evaluate(g, inputs)
    runner = GraphRunner(g)
    names = runner.pipeline.exec_names()
    for name in expect_names:  # as a node of its own or as part of a longer row-wise run
        assert any(name in n for n in names), (name, names)
    for use_cuda_graph in (False, True):
        got = runner.run(inputs, use_cuda_graph=use_cuda_graph)
        for k, (a, b) in enumerate(zip(got, want)):
            assert a.dtype == b.dtype and a.shape == b.shape
            if not np.array_equal(a, b):
                bad = np.argwhere(a != b)
                raise AssertionError(f"output {k}: {len(bad)} of {a.size} differ, first at {bad[0].tolist()}: "
                                     f"got {a[tuple(bad[0])]} want {b[tuple(bad[0])]}")


def _lut16(r):
    return r.integers(-32768, 32768, (513,), dtype=np.int64).astype(np.int16)


@pytest.mark.parametrize("shape", [(5, 7, 384), (3, 1, 4), (2, 9, 36), (1, 33, 388), (4, 16, 128)])
@pytest.mark.parametrize("shift,double_round", [(31, False), (38, True), (30, False)])
def test_fused_softmax_rows(mlel, shape, shift, double_round):
    """REDUCE_MAX -> SUB -> RESCALE -> TABLE with the REDUCE_SUM of the TABLE's output as one node: row lengths that are
    and are not multiples of a warp's 128 elements, differences that overflow int16 (they clamp), a row sum that
    wraps, and a second reader of the TABLE's output after the sum."""
    r = rng(shape[-1] + shift)
    g = GraphBuilder()
    x = g.input(np.int32, shape)
    diff = g.sub(x, g.reduce("REDUCE_MAX", x, 2))
    d16 = g.rescale(diff, [int(r.integers(1 << 30, (1 << 31) - 1))], [shift], 0, 11, np.int16, True, double_round)
    e = g.table(d16, _lut16(r))
    total = g.reduce("REDUCE_SUM", e, 2)
    g.output(g.mul(e, total, 9))      # reads both results of the fused node
    g.output(total)
    data = r.integers(-(1 << 22), 1 << 22, shape, dtype=np.int64).astype(np.int32)
    data.reshape(-1)[:3] = [np.iinfo(np.int32).max, np.iinfo(np.int32).min, 0]
    check_fused(mlel, g, [data], ["REDUCE_MAX+SUB+RESCALE+TABLE+REDUCE_SUM"])


def test_softmax_rows_are_not_fused_when_the_sum_comes_after_another_reader(mlel):
    r = rng(3)
    g = GraphBuilder()
    x = g.input(np.int32, (2, 6, 32))
    diff = g.sub(x, g.reduce("REDUCE_MAX", x, 2))
    e = g.table(g.rescale(diff, [1 << 30], [33], 0, 0, np.int16), _lut16(r))
    first = g.clamp(g.rescale(e, [1 << 30], [40], 0, 0, np.int8), -100, 100)   # reads e before the sum is taken
    total = g.reduce("REDUCE_SUM", e, 2)
    g.output(first)
    g.output(total)
    from mlel_b200.runtime import GraphRunner
    data = r.integers(-(1 << 20), 1 << 20, (2, 6, 32), dtype=np.int64).astype(np.int32)
    runner = GraphRunner(g)
    assert "REDUCE_MAX+SUB+RESCALE+TABLE+REDUCE_SUM" not in runner.pipeline.exec_names()
    for a, b in zip(runner.run([data]), evaluate(g, [data])):
        assert np.array_equal(a, b)


@pytest.mark.parametrize("b_shape", ["same", "row", "one"])
@pytest.mark.parametrize("out_dtype,shift,rshift,clamp", [(np.int8, 22, 37, None), (np.int8, 0, 33, (-20, 90)),
                                                         (np.int16, 12, 45, None), (np.int8, 31, 30, None)])
def test_fused_mul_rescale(mlel, b_shape, out_dtype, shift, rshift, clamp):
    """MUL(a, b, shift) -> RESCALE [-> CLAMP] as one node: second operand of the same shape, one value per row, one
    value; products that need all 64 bits before the shift; int8 and int16 results."""
    r = rng(shift + rshift)
    shape = (3, 50, 36)
    g = GraphBuilder()
    a = g.input(np.int32, shape)
    bs = {"same": shape, "row": shape[:-1] + (1,), "one": (1, 1, 1)}[b_shape]
    b = g.input(np.int32, bs)
    y = g.rescale(g.mul(a, b, shift), [int(r.integers(1 << 30, (1 << 31) - 1))], [rshift], -5, 3, out_dtype, True,
                  rshift > 31)
    if clamp is not None:
        y = g.clamp(y, *clamp)
    g.output(y)
    lim = 1 << 30 if shift >= 22 else 1 << 15
    da = r.integers(-lim, lim, shape, dtype=np.int64).astype(np.int32)
    db = r.integers(-lim, lim, bs, dtype=np.int64).astype(np.int32)
    da.reshape(-1)[:2] = [lim - 1, -lim]
    check_fused(mlel, g, [da, db], ["MUL+RESCALE+CLAMP" if clamp is not None else "MUL+RESCALE"])


def _norm_chain(g, r, t32, hidden, out_dtype=np.int8, lut=None):
    """The layer-norm chain of the BERT-shaped graph on an int32 tensor with the rows along the last axis."""
    total = g.reduce("REDUCE_SUM", t32, 2)
    inv = g.inline(np.asarray([(1 << 20) // hidden], np.int32).reshape(1, 1, 1))
    cen = g.sub(t32, g.mul(total, inv, 20))
    var = g.mul(g.reduce("REDUCE_SUM", g.mul(cen, cen, 8), 2), inv, 20)
    rs = g.table(g.rescale(var, [1 << 30], [34], 0, -32768, np.int16), lut if lut is not None else _lut16(r))
    return g.rescale(g.mul(cen, rs, 12), [1 << 30], [45], 0, 3, out_dtype, True, True), cen, total


@pytest.mark.parametrize("shape", [(3, 17, 768), (1, 5, 4), (2, 33, 132), (1, 3, 2048), (4, 8, 64)])
def test_fused_row_run_layer_norm(mlel, shape):
    """A residual add with its layer norm as one row-wise node: two int8 inputs, rows of 4 to 2048 elements (a multiple
    of a warp's 128 or not), the int8 result and, as further outputs, a full-shaped intermediate and the row sums."""
    r = rng(shape[-1])
    g = GraphBuilder()
    a = g.input(np.int8, shape)
    b = g.input(np.int8, shape)
    t32 = g.add(g.rescale(a, [1 << 30], [24], -3, 0, np.int32), g.rescale(b, [1 << 30], [24], 5, 0, np.int32))
    y, cen, total = _norm_chain(g, r, t32, shape[-1])
    g.output(y)
    g.output(cen)
    g.output(total)
    check_fused(mlel, g, [full_range(r, np.int8, shape), full_range(r, np.int8, shape)], ["ROWS(RESCALE+RESCALE+ADD+REDUCE_SUM"])


def test_fused_row_run_with_int8_table_clamp_and_int16(mlel):
    """TABLE on int8, CLAMP, MIN and MAX reductions, an int16 result, a constant operand of one element and a
    row-shaped input from outside the run."""
    r = rng(77)
    shape = (2, 21, 96)
    g = GraphBuilder()
    x = g.input(np.int8, shape)
    bias = g.input(np.int32, shape[:-1] + (1,))
    t = g.clamp(g.table(x, r.integers(-128, 128, (256,), dtype=np.int64).astype(np.int8)), -100, 90)
    v = g.rescale(t, [1 << 30], [20], 0, 0, np.int32)
    lo, hi = g.reduce("REDUCE_MIN", v, 2), g.reduce("REDUCE_MAX", v, 2)
    span = g.add(g.sub(hi, lo), g.inline(np.asarray([1], np.int32).reshape(1, 1, 1)))
    w = g.add(g.sub(v, lo), bias)
    g.output(g.rescale(g.mul(w, span, 3), [int(r.integers(1 << 30, (1 << 31) - 1))], [33], 0, -7, np.int16, True, True))
    g.output(span)
    data = [full_range(r, np.int8, shape), r.integers(-5000, 5000, shape[:-1] + (1,), dtype=np.int64).astype(np.int32)]
    check_fused(mlel, g, data, ["ROWS(TABLE+CLAMP+RESCALE+REDUCE_MIN+REDUCE_MAX"])


def test_row_run_is_left_alone_when_it_does_not_pay(mlel):
    """A softmax's nine operators: the row kernel would cost more than the two smaller fused nodes."""
    r = rng(5)
    shape = (6, 12, 64)
    g = GraphBuilder()
    x = g.input(np.int32, shape)
    d16 = g.rescale(g.sub(x, g.reduce("REDUCE_MAX", x, 2)), [1 << 30], [33], 0, 0, np.int16)
    e = g.table(d16, _lut16(r))
    den = g.table(g.rescale(g.reduce("REDUCE_SUM", e, 2), [1 << 30], [40], 0, -32768, np.int16), _lut16(r))
    g.output(g.rescale(g.mul(e, den, 22), [1 << 30], [37], 0, -128, np.int8))
    from mlel_b200.runtime import GraphRunner
    runner = GraphRunner(g)
    names = runner.pipeline.exec_names()
    assert not any(n.startswith("ROWS") for n in names), names
    assert "REDUCE_MAX+SUB+RESCALE+TABLE+REDUCE_SUM" in names and "MUL+RESCALE" in names
    data = [r.integers(-(1 << 20), 1 << 20, shape, dtype=np.int64).astype(np.int32)]
    for a, b in zip(runner.run(data), evaluate(g, data)):
        assert np.array_equal(a, b)
