"""The three session memory planners (VMEL_MEMORY_PLANNER = Interval | Linear | BestFit, read when a session
is created: graph/graph_layer.cpp:282-297) on whole graphs, without a device: the plan of every planner must
keep tensors that are alive at the same time apart, Linear must give every tensor its own storage
(graph/memory_planner.cpp:52-98), and BestFit must reuse the best-fitting slot (memory_planner.cpp:239-381)."""
import numpy as np
import pytest

from mlel_b200 import PIPELINE_NO_FUSION, Session
from mlel_b200.graph_builder import GraphBuilder
from mlel_b200.model_graphs import mobilenet_v2_graph, resnet50_graph
from mlel_b200.runtime import make_pipeline

SMALL_RESNET = dict(n=2, image=32, width=8, blocks=(2, 1, 1, 1), classes=8)


def plan_of(graph, flags, planner, monkeypatch):
    if planner is None:
        monkeypatch.delenv("VMEL_MEMORY_PLANNER", raising=False)
    else:
        monkeypatch.setenv("VMEL_MEMORY_PLANNER", planner)
    pipeline, _, _ = make_pipeline(graph, flags)
    session = Session(pipeline)
    size, align = session.memory_requirements()
    return session, session.plan(), size, align


def check_plan(plan, size, align):
    for p in plan:
        assert p.offset % align == 0 and p.size % align == 0
        assert p.offset + p.size <= size
    for i, a in enumerate(plan):
        for b in plan[i + 1:]:
            alive_together = not (a.seen and b.seen) or not (a.last < b.first or b.last < a.first)
            if alive_together:
                assert a.offset + a.size <= b.offset or b.offset + b.size <= a.offset, (a.tensor, b.tensor)


@pytest.mark.parametrize("flags", [0, PIPELINE_NO_FUSION])
@pytest.mark.parametrize("planner,name", [(None, "Interval"), ("Interval", "Interval"), ("Linear", "Linear"),
                                          ("BestFit", "BestFit"), ("linear", "Interval"), ("", "Interval")])
def test_every_planner_keeps_live_tensors_apart(mlel, monkeypatch, flags, planner, name):
    g, _ = resnet50_graph(seed=3, **SMALL_RESNET)
    session, plan, size, align = plan_of(g, flags, planner, monkeypatch)
    assert session.planner_name() == name
    assert len(plan) > 10
    check_plan(plan, size, align)
    for p in plan:
        assert session.tensor_offset(p.tensor) == p.offset


@pytest.mark.parametrize("flags", [0, PIPELINE_NO_FUSION])
@pytest.mark.parametrize("graph", ["resnet", "mobilenet"])
def test_linear_is_the_sum_and_the_others_reuse(mlel, monkeypatch, flags, graph):
    if graph == "resnet":
        g, _ = resnet50_graph(seed=3, **SMALL_RESNET)
    else:
        g, _ = mobilenet_v2_graph(seed=3, n=1, image=32, classes=8)
    _, linear, linear_size, align = plan_of(g, flags, "Linear", monkeypatch)
    assert linear_size == sum(p.size for p in linear)
    offset = 0
    for p in linear:  # one after the other, in session-tensor order
        assert p.offset == offset
        offset += p.size
    for planner in ("Interval", "BestFit"):
        _, plan, size, _ = plan_of(g, flags, planner, monkeypatch)
        assert [p.tensor for p in plan] == [p.tensor for p in linear]
        check_plan(plan, size, align)
        assert size < linear_size
        assert size >= max(p.size for p in plan)


def chain(sizes):
    """x -> CLAMP -> CLAMP ... with a RESHAPE-free way to vary sizes: SLICE shrinks the row count."""
    g = GraphBuilder("chain")
    x = g.input(np.int8, (sizes[0], 256))
    y = x
    for rows in sizes[1:]:
        y = g.slice(y, [0, 0], [rows, 256]) if rows != y.shape[0] else g.clamp(y, -100, 100)
    g.output(g.clamp(y, -50, 50))
    return g


def test_best_fit_on_a_chain(mlel, monkeypatch):
    """Four equal intermediates t1..t4 alive over launches (1,2) (2,3) (3,4) (4,5): neighbours overlap, so two
    slots suffice; t3 moves in with t1 and t4 with t2."""
    g = chain([4, 4, 4, 4, 4])
    _, plan, size, _ = plan_of(g, PIPELINE_NO_FUSION, "BestFit", monkeypatch)
    assert [(p.first, p.last) for p in plan] == [(1, 2), (2, 3), (3, 4), (4, 5)]
    assert [p.offset for p in plan] == [0, 1024, 0, 1024] and size == 2048


def test_best_fit_takes_the_tightest_slot_and_largest_first(mlel, monkeypatch):
    """Intermediates of 8, 4, 2 and 2 rows of 256 bytes, alive over (1,2) (2,3) (3,4) (4,5).  Largest first:
    the 8-row tensor opens slot A at 0, the 4-row one overlaps it and opens slot B at 2048; the first 2-row
    tensor (3,4) may share with the 8-row tensor only (the 4-row one is still alive) and moves into A; the
    last one (4,5) may share with both earlier slots' first tenants but A now also holds (3,4), which it
    overlaps, so it takes B."""
    g = chain([8, 8, 4, 2, 2])
    _, plan, size, _ = plan_of(g, PIPELINE_NO_FUSION, "BestFit", monkeypatch)
    assert [p.size for p in plan] == [2048, 1024, 512, 512]
    assert [p.offset for p in plan] == [0, 2048, 0, 2048] and size == 3072
    _, interval, interval_size, _ = plan_of(g, PIPELINE_NO_FUSION, "Interval", monkeypatch)
    check_plan(interval, interval_size, 256)


def test_plan_enumeration_reports_short_arrays(mlel, monkeypatch):
    import ctypes
    from mlel_b200 import INCOMPLETE, PlannedTensor, lib
    g = chain([4, 4, 4, 4])
    session, plan, _, _ = plan_of(g, PIPELINE_NO_FUSION, None, monkeypatch)
    n = ctypes.c_uint32(1)
    out = (PlannedTensor * 1)()
    assert lib().mlel_session_plan(session._h, ctypes.byref(n), out) == INCOMPLETE
    assert n.value == 1 and out[0].tensor == plan[0].tensor
