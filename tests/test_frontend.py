"""SPIR-V text front end and TOSA registry (host logic, no GPU).

Where the reference checkout is present its own fixtures (tests/shader/*.spvasm) are lowered
unmodified and the resulting operator lists are checked; the same structures are also covered by
graphs emitted by GraphBuilder, which travel with the repository."""
import os

import numpy as np
import pytest

from mlel_b200.graph_builder import GraphBuilder
from mlel_b200.model_graphs import mobilenet_v2_graph, resnet50_graph


def lower(mlel, text, externals, constants=(), flags=0):
    p = mlel.Pipeline(flags)
    for (s, b, idx, dtype, dims) in externals:
        p.bind_external(s, b, dtype, dims, array_index=idx)
    for cid, arr in constants:
        p.add_constant(cid, arr)
    p.lower_spvasm(text)
    return p


def fixture(reference_root, name):
    return open(os.path.join(reference_root, "tests", "shader", name)).read()


def test_reference_conv2d_fixture(mlel, reference_root):
    p = lower(mlel, fixture(reference_root, "conv2d.spvasm"),
              [(0, 0, 0, mlel.I8, (1, 8, 8, 3)), (0, 1, 0, mlel.I8, (3, 2, 2, 3)), (0, 2, 0, mlel.I32, (3,)),
               (0, 3, 0, mlel.I32, (1, 4, 4, 3))])
    assert p.op_names() == ["CONV2D"]
    s = mlel.Session(p)
    assert s.memory_requirements()[0] == 0  # no intermediate tensors


def test_reference_maxpool_fixture_uses_array_element(mlel, reference_root):
    # graph input 0 is element 1 of a tensor array bound at (0, 0) (tests/shader/maxpool.spvasm:33-41)
    p = lower(mlel, fixture(reference_root, "maxpool.spvasm"),
              [(0, 0, 0, mlel.I8, (1, 16, 16, 3)), (0, 0, 1, mlel.I8, (1, 16, 16, 3)),
               (0, 1, 0, mlel.I8, (1, 8, 8, 3))])
    assert p.op_names() == ["MAX_POOL2D"]


def test_reference_two_layer_maxpool_plans_one_intermediate(mlel, reference_root):
    p = lower(mlel, fixture(reference_root, "twolayer-maxpool.spvasm"),
              [(0, 0, 0, mlel.I8, (1, 16, 16, 3)), (0, 1, 0, mlel.I8, (1, 4, 4, 3))])
    assert p.op_names() == ["MAX_POOL2D", "MAX_POOL2D"]
    size, align = mlel.Session(p).memory_requirements()
    assert align == 256 and size == 256  # [1,8,8,3] int8 = 192 bytes, rounded up to the alignment


def test_reference_graph_constant_fixture(mlel, reference_root):
    consts = [(0, np.array([2], np.int32)), (1, np.array([0], np.int8)), (2, np.array([3], np.int32)),
              (3, np.array([0], np.int8)), (4, np.array([4], np.int32)), (5, np.array([0], np.int8))]
    ext = [(0, 0, 0, mlel.I8, (5,)), (0, 1, 0, mlel.I8, (5,)), (0, 2, 0, mlel.I8, (5,))]
    p = lower(mlel, fixture(reference_root, "graph-constant-arm.spvasm"), ext, consts, mlel.PIPELINE_NO_FUSION)
    assert p.op_names() == ["RESCALE", "RESCALE", "ADD", "RESCALE"]
    assert p.exec_names() == ["RESCALE", "RESCALE", "ADD", "RESCALE"]
    fused = lower(mlel, fixture(reference_root, "graph-constant-arm.spvasm"), ext, consts)
    assert fused.exec_names() == ["RESCALE+RESCALE+ADD+RESCALE"]


def test_reference_misc_fixtures(mlel, reference_root):
    p = lower(mlel, fixture(reference_root, "inlined-higher-rank-constant.spvasm"),
              [(0, 0, 0, mlel.I8, (1, 3, 3, 1)), (0, 1, 0, mlel.I8, (1, 3, 3, 1))])
    assert p.op_names() == ["CONV2D", "CAST"]
    p = lower(mlel, fixture(reference_root, "concat_interval.spvasm"),
              [(0, 0, 0, mlel.F32, (3, 3)), (0, 1, 0, mlel.F32, (3, 3)), (0, 2, 0, mlel.F32, (3, 1)),
               (0, 3, 0, mlel.F32, (12,))])
    assert p.op_names() == ["ADD", "CONCAT", "CONCAT", "RESHAPE"]  # one CONCAT pass per input
    p = lower(mlel, fixture(reference_root, "nop-outputs.spvasm"),
              [(0, 0, 0, mlel.I8, (1, 8, 8, 3)), (0, 1, 0, mlel.I8, (1, 2, 2, 2)), (0, 2, 0, mlel.I8, (1, 8, 8, 3)),
               (0, 3, 0, mlel.I8, (1, 8, 8, 3))], [(0, np.arange(192, dtype=np.int8).reshape(1, 8, 8, 3))])
    assert sorted(p.op_names()) == ["CAST", "CAST", "SLICE"]  # pass-through outputs become CAST
    p = lower(mlel, fixture(reference_root, "arshift_specbool.spvasm"),
              [(0, 0, 0, mlel.I8, (4,)), (0, 1, 0, mlel.I8, (4,)), (0, 2, 0, mlel.I8, (4,))])
    assert p.op_names() == ["ARITHMETIC_RIGHT_SHIFT"]
    p = lower(mlel, fixture(reference_root, "conv2_acc_int64.spvasm"),
              [(0, 0, 0, mlel.I16, (1, 2, 2, 4)), (0, 1, 0, mlel.I8, (4, 1, 1, 4)), (0, 2, 0, mlel.I64, (4,)),
               (0, 3, 0, mlel.I64, (1, 2, 2, 4))])
    assert p.op_names() == ["CONV2D"]


def test_reference_conv3d_fixture(mlel, reference_root):
    # tests/shader/conv3d_large_stride.spvasm: rank-5 tensors, six pads, OpConstantNull bias and zero point
    w = np.zeros((3, 2, 2, 8192, 4), np.int8)
    p = lower(mlel, fixture(reference_root, "conv3d_large_stride.spvasm"),
              [(0, 0, 0, mlel.I8, (1, 3, 2, 2, 4)), (0, 1, 0, mlel.I32, (1, 3, 2, 2, 3))], [(0, w)])
    assert p.op_names() == ["CONV3D"]


def test_reference_sin_fixture(mlel, reference_root):
    p = lower(mlel, fixture(reference_root, "sin.spvasm"), [(0, 0, 0, mlel.F32, (1,)), (0, 1, 0, mlel.F32, (1,))])
    assert p.op_names() == ["SIN"]


def test_reference_fft2d_fixture(mlel, reference_root):
    # tests/shader/fft2d.spvasm: a two-result instruction (OpTypeStruct result, OpCompositeExtract per output)
    p = lower(mlel, fixture(reference_root, "fft2d.spvasm"), [(0, b, 0, mlel.F32, (1, 4, 4096)) for b in range(4)])
    assert p.op_names() == ["FFT2D"]


def test_every_tosa_operator_is_registered_and_built(mlel):
    names = mlel.tosa_op_names()
    assert len(names) == 66  # graph/graph_tosa_1_0_ext_inst.cpp:41-108
    assert all(mlel.tosa_op_supported(n) for n in names)


def test_unbuilt_variant_is_feature_not_present(mlel):
    # every operator is lowered, but not for every element type: a transcendental of an integer tensor is refused
    g = GraphBuilder()
    x = g.input(np.int8, (4,))
    g.output(g.unary("SIN", x))
    with pytest.raises(mlel.MlelError) as e:
        lower(mlel, g.spvasm(), [(0, 0, 0, mlel.I8, (4,)), (0, 1, 0, mlel.I8, (4,))])
    assert e.value.status == -8
    assert "SIN" in str(e.value)


def test_unregistered_instruction_set_is_rejected(mlel):
    g = GraphBuilder()
    x = g.input(np.int8, (4,))
    g.output(g.unary("ABS", x))
    text = g.spvasm().replace("TOSA.001000.1", "TOSA.000080.2")
    with pytest.raises(mlel.MlelError) as e:
        lower(mlel, text, [(0, 0, 0, mlel.I8, (4,)), (0, 1, 0, mlel.I8, (4,))])
    assert "Unsupported extension" in str(e.value)


def test_emitted_resnet_lowers_and_fuses(mlel):
    g, _ = resnet50_graph(seed=0, n=2, image=64, width=16, blocks=(2, 1, 1, 1), classes=10)
    ext = [(v.binding[0], v.binding[1], 0, mlel.NP_TO_DTYPE[v.dtype], v.shape) for v in g.inputs]
    ext += [(s, b, 0, mlel.NP_TO_DTYPE[v.dtype], v.shape) for v, s, b in g.outputs]
    consts = list(g.constants.items())
    p = lower(mlel, g.spvasm(), ext, consts, mlel.PIPELINE_NO_FUSION)
    assert p.op_names() == [op.name for op in g.ops]
    assert p.exec_names() == p.op_names()
    unfused_mem = mlel.Session(p).memory_requirements()[0]
    pf = lower(mlel, g.spvasm(), ext, consts)
    names = pf.exec_names()
    assert sum(n.startswith("CONV2D+RESCALE") for n in names) == sum(o.name == "CONV2D" for o in g.ops)
    # every residual add runs in the epilogue of the convolution that produces its main operand
    assert sum("+ADD+RESCALE" in n for n in names) == sum(o.name == "ADD" for o in g.ops)
    assert "RESCALE" not in names and "ADD" not in names and "CLAMP" not in names
    assert names[-1] == "MATMUL+RESCALE"
    assert 0 < mlel.Session(pf).memory_requirements()[0] < unfused_mem


def test_emitted_bert_lowers_and_fuses(mlel):
    from mlel_b200.model_graphs import bert_graph
    g, _ = bert_graph(seed=0, n=2, seq=16, hidden=32, heads=2, ffn=64, layers=2)
    ext = [(v.binding[0], v.binding[1], 0, mlel.NP_TO_DTYPE[v.dtype], v.shape) for v in g.inputs]
    ext += [(s, b, 0, mlel.NP_TO_DTYPE[v.dtype], v.shape) for v, s, b in g.outputs]
    consts = list(g.constants.items())
    p = lower(mlel, g.spvasm(), ext, consts, mlel.PIPELINE_NO_FUSION)
    assert p.op_names() == [op.name for op in g.ops]
    names = lower(mlel, g.spvasm(), ext, consts).exec_names()
    # every projection and the context product carry their RESCALE; the score product feeds REDUCE_MAX and SUB
    # as int32 and stays a plain MATMUL
    assert names.count("MATMUL+RESCALE") == 2 * 7 and names.count("MATMUL") == 2
    assert names.count("TRANSPOSE") == 2 * 4
    # The thirteen operators of each residual add with its layer norm are one row-wise node.  The softmax's are not
    # (its RESCALEs, exponential TABLE and MUL cost more in the row kernel than the passes it would save): its row
    # maximum, subtraction, RESCALE, TABLE and row sum are one node and its final MUL + RESCALE another, with the
    # reciprocal's RESCALE and TABLE on the row sums between them.  The other TABLE is the GELU.
    norm = "ROWS(RESCALE+RESCALE+ADD+REDUCE_SUM+MUL+SUB+MUL+REDUCE_SUM+MUL+RESCALE+TABLE+MUL+RESCALE)"
    assert names.count(norm) == 2 * 2
    assert names.count("REDUCE_MAX+SUB+RESCALE+TABLE+REDUCE_SUM") == 2 and names.count("MUL+RESCALE") == 2
    assert names.count("TABLE") == 2 * 2 and names.count("RESCALE") == 2
    assert "REDUCE_MAX" not in names and "MUL" not in names and len(names) == 2 * 27


def test_graph_outputs_are_never_elided(mlel):
    g = GraphBuilder()
    a = g.input(np.int8, (1, 4, 4, 8))
    w = g.constant(np.ones((8, 1, 1, 8), np.int8))
    b = g.constant(np.zeros((8,), np.int32))
    acc = g.conv2d(a, w, b, [0] * 4, [1, 1], [1, 1], 0, 0)
    y = g.rescale(acc, [1 << 30], [35], 0, 0, np.int8)
    g.output(y)
    g.output(acc)  # the int32 accumulator is itself an output: the pair must not be fused
    ext = [(0, 0, 0, mlel.I8, a.shape), (0, 1, 0, mlel.I8, y.shape), (0, 2, 0, mlel.I32, acc.shape)]
    p = lower(mlel, g.spvasm(), ext, list(g.constants.items()))
    assert p.exec_names() == ["CONV2D", "RESCALE"]


def test_mobilenet_lowers(mlel):
    g, _ = mobilenet_v2_graph(seed=0, n=1, image=32, width_div=4, classes=10)
    ext = [(v.binding[0], v.binding[1], 0, mlel.NP_TO_DTYPE[v.dtype], v.shape) for v in g.inputs]
    ext += [(s, b, 0, mlel.NP_TO_DTYPE[v.dtype], v.shape) for v, s, b in g.outputs]
    p = lower(mlel, g.spvasm(), ext, list(g.constants.items()))
    names = p.exec_names()
    assert sum(n.startswith("DEPTHWISE_CONV2D+RESCALE") for n in names) == 17


def _replicated_pattern_module(count):
    """``x + k`` on int32 tensors of ``count`` elements where ``k`` is OpConstantCompositeReplicateEXT of the
    two-element composite {1, 2}: the flattened constant holds a pattern of two values for ``count`` elements."""
    shape = (count // 2, 2) if count % 2 == 0 else (count,)
    g = GraphBuilder()
    row = g._tensor_type(np.dtype(np.int32), (2,))
    x = g.input(np.int32, shape)
    k = g.inline(np.arange(1, count + 1, dtype=np.int32).reshape(shape))
    g.output(g.add(x, k))
    lines = []
    for line in g.spvasm().splitlines():
        if line.startswith(f"%{k.name} = OpConstantComposite "):
            tensor_type = line.split()[3]
            lines.append(f"%pattern_row = OpConstantComposite {row} %i32_1 %i32_2")
            lines.append(f"%{k.name} = OpConstantCompositeReplicateEXT {tensor_type} %pattern_row")
        else:
            lines.append(line)
    return "\n".join(lines) + "\n", shape


def test_replicated_pattern_two_to_four_is_expanded(mlel):
    # tests/graph/graph_ext_inst_context_tests.cpp:16-20: {1, 2} for four elements becomes {1, 2, 1, 2}
    text, shape = _replicated_pattern_module(4)
    p = lower(mlel, text, [(0, 0, 0, mlel.I32, shape), (0, 1, 0, mlel.I32, shape)])
    assert p.op_names() == ["ADD"]


def test_replicated_pattern_rejects_non_divisible_counts(mlel):
    # tests/graph/graph_ext_inst_context_tests.cpp:22-26: {1, 2} cannot fill three elements
    text, shape = _replicated_pattern_module(3)
    with pytest.raises(mlel.MlelError) as e:
        lower(mlel, text, [(0, 0, 0, mlel.I32, shape), (0, 1, 0, mlel.I32, shape)])
    assert "replicated constant element count" in str(e.value)
