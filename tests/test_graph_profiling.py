"""Per-operator profiling behind VMEL_GRAPH_PROFILING and the pipeline-property queries that return it, after
the reference's own tests (tests/vulkan.cpp:660-745, 2560-2640): the property is offered only when the
variable is truthy, text is returned through the two-call pattern with INCOMPLETE on a short buffer, one
sample per operator and dispatch with the document layout of graph/graph_profiler.cpp:563-620."""
import ctypes
import json

import numpy as np
import pytest

from mlel_b200 import INCOMPLETE, PROPERTY_CREATION_LOG, PROPERTY_PROFILING, MlelError, lib
from mlel_b200.graph_builder import GraphBuilder
from mlel_b200.runtime import make_pipeline
from tests.graph_eval import evaluate


def max_pool_graph():
    """The reference's profiling graph (tests/vulkan.cpp:327-345): int8 [1,16,16,3] -> MAX_POOL2D 2x2/2."""
    g = GraphBuilder("maxpool")
    x = g.input(np.int8, (1, 16, 16, 3))
    g.output(g.max_pool2d(x, [2, 2], [2, 2], [0, 0, 0, 0]))
    return g


@pytest.mark.parametrize("value,enabled", [("1", True), ("true", True), ("yes", True), ("0", False), ("", False),
                                           ("OFF", False), ("No", False), ("False", False), (None, False)])
def test_profiling_property_is_offered_only_when_enabled(mlel, monkeypatch, value, enabled):
    if value is None:
        monkeypatch.delenv("VMEL_GRAPH_PROFILING", raising=False)
    else:
        monkeypatch.setenv("VMEL_GRAPH_PROFILING", value)
    pipeline, _, _ = make_pipeline(max_pool_graph())
    props = pipeline.available_properties()
    assert PROPERTY_CREATION_LOG in props
    assert (PROPERTY_PROFILING in props) == enabled
    assert pipeline.text_property(PROPERTY_CREATION_LOG) == "Graph pipeline created"
    if not enabled:
        with pytest.raises(MlelError):
            pipeline.text_property(PROPERTY_PROFILING)
    with pytest.raises(MlelError):
        pipeline.text_property(12345)


def test_available_properties_two_call_pattern(mlel, monkeypatch):
    monkeypatch.setenv("VMEL_GRAPH_PROFILING", "1")
    pipeline, _, _ = make_pipeline(max_pool_graph())
    n = ctypes.c_uint32()
    assert lib().mlel_pipeline_available_properties(pipeline._h, ctypes.byref(n), None) == 0 and n.value == 2
    ids = (ctypes.c_uint32 * 2)()
    n = ctypes.c_uint32(1)
    assert lib().mlel_pipeline_available_properties(pipeline._h, ctypes.byref(n), ids) == INCOMPLETE
    assert n.value == 1 and ids[0] == PROPERTY_CREATION_LOG


def test_empty_profile_document_and_short_buffer(mlel, monkeypatch):
    monkeypatch.setenv("VMEL_GRAPH_PROFILING", "1")
    pipeline, _, _ = make_pipeline(max_pool_graph())
    text = pipeline.text_property(PROPERTY_PROFILING)
    assert text == '{\n  "timestamp_period_ns": 1.0,\n  "samples": [],\n  "by_operator": []\n}'
    assert json.loads(text) == {"timestamp_period_ns": 1.0, "samples": [], "by_operator": []}
    # a 4-byte buffer: INCOMPLETE, 4 bytes written, still flagged as text (tests/vulkan.cpp:2615-2640)
    buf = ctypes.create_string_buffer(4)
    size, is_text = ctypes.c_size_t(4), ctypes.c_int(0)
    rc = lib().mlel_pipeline_get_property(pipeline._h, ctypes.c_uint32(PROPERTY_PROFILING), buf, ctypes.byref(size),
                                          ctypes.byref(is_text))
    assert rc == INCOMPLETE and size.value == 4 and is_text.value == 1 and buf.raw == text[:4].encode()
    # exact size: success, zero-terminated
    size = ctypes.c_size_t(len(text) + 1)
    buf = ctypes.create_string_buffer(len(text) + 1)
    assert lib().mlel_pipeline_get_property(pipeline._h, ctypes.c_uint32(PROPERTY_PROFILING), buf,
                                            ctypes.byref(size), ctypes.byref(is_text)) == 0
    assert size.value == len(text) + 1 and buf.raw[-1] == 0


# ---- on the device ----

def profiled_runner(monkeypatch, graph, flags=0):
    from mlel_b200.runtime import GraphRunner
    monkeypatch.setenv("VMEL_GRAPH_PROFILING", "1")
    return GraphRunner(graph, flags=flags)


@pytest.mark.gpu
def test_max_pool_profile_document(mlel, monkeypatch):
    g = max_pool_graph()
    data = np.random.Generator(np.random.PCG64(1)).integers(-128, 128, (1, 16, 16, 3), dtype=np.int8)
    r = profiled_runner(monkeypatch, g)
    np.testing.assert_array_equal(r.run([data])[0], evaluate(g, [data])[0])
    text = r.pipeline.text_property(PROPERTY_PROFILING)
    for needle in ('"samples"', '"by_operator"', '"pipeline_kind": "tosa"', '"operator_name": "MAX_POOL2D"',
                   '"cycle_count_before"', '"cycle_count_after"', '"time_ms"'):
        assert needle in text, needle
    doc = json.loads(text)
    assert list(doc) == ["timestamp_period_ns", "samples", "by_operator"]
    assert list(doc["samples"][0]) == ["submission", "graph_dispatch", "pipeline_index", "pipeline_kind",
                                       "operator_name", "cycle_count_before", "cycle_count_after",
                                       "cycle_count_delta", "time_ms"]
    assert list(doc["by_operator"][0]) == ["pipeline_kind", "operator_name", "dispatch_count", "total_time_ms",
                                           "average_time_ms", "min_time_ms", "max_time_ms"]


@pytest.mark.gpu
@pytest.mark.parametrize("use_cuda_graph", [False, True])
def test_two_dispatches_give_two_samples(mlel, monkeypatch, use_cuda_graph):
    """tests/vulkan.cpp:704-723: two submissions without a wait in between."""
    g = max_pool_graph()
    data = np.zeros((1, 16, 16, 3), np.int8)
    r = profiled_runner(monkeypatch, g)
    r.set_inputs([data])
    r.dispatch(use_cuda_graph)
    r.dispatch(use_cuda_graph)
    doc = r.pipeline.profile()
    s = doc["samples"]
    assert len(s) == 2
    assert s[1]["submission"] == s[0]["submission"] + 1
    assert s[1]["graph_dispatch"] == s[0]["graph_dispatch"] + 1
    assert s[0]["cycle_count_before"] != s[1]["cycle_count_before"]
    assert s[0]["cycle_count_after"] != s[1]["cycle_count_after"]
    for x in s:
        assert x["cycle_count_delta"] == x["cycle_count_after"] - x["cycle_count_before"] > 0
        assert x["time_ms"] == pytest.approx(x["cycle_count_delta"] * doc["timestamp_period_ns"] / 1e6)
    assert len(doc["by_operator"]) == 1
    agg = doc["by_operator"][0]
    assert agg["dispatch_count"] == 2
    assert agg["total_time_ms"] == pytest.approx(s[0]["time_ms"] + s[1]["time_ms"])
    assert agg["min_time_ms"] == min(x["time_ms"] for x in s) and agg["max_time_ms"] == max(x["time_ms"] for x in s)
    assert agg["average_time_ms"] == pytest.approx(agg["total_time_ms"] / 2)
    r.pipeline.clear_profile()
    assert r.pipeline.profile()["samples"] == []


@pytest.mark.gpu
def test_profile_is_scoped_to_its_pipeline_and_names_fused_kernels(mlel, monkeypatch):
    """tests/vulkan.cpp:738-760: the samples of one pipeline do not show up in another's document."""
    from mlel_b200.model_graphs import resnet50_graph
    g, inputs = resnet50_graph(seed=5, n=2, image=32, width=8, blocks=(1, 1, 1, 1), classes=8)
    net = profiled_runner(monkeypatch, g)
    idle = profiled_runner(monkeypatch, max_pool_graph())
    got = net.run(inputs)
    np.testing.assert_array_equal(got[0], evaluate(g, inputs)[0])
    assert idle.pipeline.profile()["samples"] == []
    doc = net.pipeline.profile()
    launches = net.session.launch_count()
    assert len(doc["samples"]) == launches
    assert [x["pipeline_index"] for x in doc["samples"]] == list(range(launches))
    names = [x["operator_name"] for x in doc["samples"]]
    assert names == net.pipeline.exec_names()
    assert any(n.startswith("CONV2D+RESCALE") for n in names) and "MAX_POOL2D" in names
    keys = [(a["pipeline_kind"], a["operator_name"]) for a in doc["by_operator"]]
    assert keys == sorted(set(("tosa", n) for n in names))
    assert sum(a["dispatch_count"] for a in doc["by_operator"]) == launches
    # consecutive operators share a timestamp: one event closes an operator and opens the next
    for a, b in zip(doc["samples"], doc["samples"][1:]):
        assert b["cycle_count_before"] == a["cycle_count_after"]
