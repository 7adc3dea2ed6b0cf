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
