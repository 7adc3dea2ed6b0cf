"""GPU: the graph's results do not depend on which planner placed its intermediate tensors."""
import numpy as np
import pytest

from mlel_b200 import PIPELINE_NO_FUSION
from mlel_b200.model_graphs import mobilenet_v2_graph, resnet50_graph
from tests.graph_eval import evaluate

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("planner", ["Linear", "BestFit", "Interval"])
@pytest.mark.parametrize("flags", [0, PIPELINE_NO_FUSION])
def test_results_are_the_same_under_every_planner(mlel, monkeypatch, planner, flags):
    from mlel_b200.runtime import GraphRunner
    monkeypatch.setenv("VMEL_MEMORY_PLANNER", planner)
    for g, inputs in (resnet50_graph(seed=9, n=2, image=32, width=8, blocks=(2, 1, 1, 1), classes=8),
                      mobilenet_v2_graph(seed=9, n=1, image=32, classes=8)):
        r = GraphRunner(g, flags=flags)
        assert r.session.planner_name() == planner
        want = evaluate(g, inputs)
        for got, ref in zip(r.run(inputs), want):
            np.testing.assert_array_equal(got, ref)


@pytest.mark.parametrize("planner", ["Linear", "BestFit", "Interval"])
def test_reshape_between_session_tensors_shares_storage(mlel, monkeypatch, planner):
    """With fusion on, a RESHAPE of one intermediate tensor into another moves no bytes: both get one offset, the
    storage outlives both, and later tensors may not land on it while the reshaped view is still read.  Without
    fusion the copy is kept.  Results equal the oracle's either way."""
    from mlel_b200.graph_builder import GraphBuilder
    from mlel_b200.runtime import GraphRunner
    monkeypatch.setenv("VMEL_MEMORY_PLANNER", planner)
    r = np.random.Generator(np.random.PCG64(3))
    g = GraphBuilder()
    x = g.input(np.int8, (4, 6, 8, 16))
    a = g.max_pool2d(x, [2, 2], [2, 2], [0] * 4)            # (4, 3, 4, 16)
    b = g.reshape(g.reshape(a, (4, 12, 16)), (48, 16))      # two views of the same bytes
    c = g.table(b, r.integers(-128, 128, (256,), dtype=np.int8))
    d = g.table(c, r.integers(-128, 128, (256,), dtype=np.int8))
    g.output(g.binary("MAXIMUM", d, b))                     # the view is read again after two other tensors were made
    inputs = [r.integers(-128, 128, (4, 6, 8, 16), dtype=np.int8)]
    want = evaluate(g, inputs)
    fused, plain = GraphRunner(g), GraphRunner(g, flags=PIPELINE_NO_FUSION)
    for runner in (fused, plain):
        for got, ref in zip(runner.run(inputs), want):
            np.testing.assert_array_equal(got, ref)
    assert len(fused.session.plan()) == len(plain.session.plan()) - 2
