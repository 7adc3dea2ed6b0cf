"""Interval memory planner: the C++ implementation behind the C ABI against the reference's own
unit-test cases (tests/graph/interval_memory_planner_tests.cpp:17-106, values restated here) and
against a plain-Python restatement on random live ranges."""
import numpy as np
import pytest

from oracle import planner_ref


def test_non_overlapping_tensors_reuse_memory(mlel):
    off, size = mlel.allocate_intervals([(0, 0, 0, 64, 0), (1, 1, 1, 64, 1)], [], 16)
    assert off[0] == 0 and off[1] == off[0] and size == 64


def test_overlapping_tensors_do_not_alias(mlel):
    off, size = mlel.allocate_intervals([(0, 0, 2, 64, 0), (1, 1, 3, 64, 1)], [], 16)
    assert off[0] != off[1] and size == 128


def test_splits_oversized_free_blocks(mlel):
    off, size = mlel.allocate_intervals([(0, 0, 0, 128, 0), (1, 1, 2, 64, 1), (2, 1, 2, 64, 2)], [], 16)
    assert (off[0], off[1], off[2], size) == (0, 0, 64, 128)


def test_does_not_coalesce_adjacent_free_blocks(mlel):
    off, size = mlel.allocate_intervals([(0, 0, 0, 64, 0), (1, 0, 0, 64, 1), (2, 1, 1, 128, 2)], [], 16)
    assert (off[0], off[1], off[2], size) == (0, 64, 128, 256)


def test_unseen_tensors_receive_unique_storage(mlel):
    off, size = mlel.allocate_intervals([(0, 0, 0, 64, 0)], [(1, 32), (2, 32)], 16)
    assert (off[0], off[1], off[2], size) == (0, 64, 96, 128)


def test_external_tensors_are_not_included(mlel):
    off, size = mlel.allocate_intervals([(0, 0, 0, 64, 0)], [(1, 64)], 16)
    assert 0 in off and 1 in off and 2 not in off and size == 128


@pytest.mark.parametrize("seed", range(20))
def test_matches_python_restatement_on_random_ranges(mlel, seed):
    rng = np.random.Generator(np.random.PCG64(seed))
    n = int(rng.integers(1, 60))
    intervals = []
    for i in range(n):
        first = int(rng.integers(0, 40))
        last = first + int(rng.integers(0, 6))
        intervals.append((i, first, last, int(rng.integers(1, 9)) * 256, i))
    unseen = [(n + k, int(rng.integers(1, 4)) * 256) for k in range(int(rng.integers(0, 3)))]
    got = mlel.allocate_intervals(intervals, unseen, 256)
    want = planner_ref.allocate_intervals(intervals, unseen, 256)
    assert got == want
    # no two tensors alive at the same time overlap in memory
    off = got[0]
    for a in intervals:
        for b in intervals:
            if a[0] < b[0] and not (a[2] < b[1] or b[2] < a[1]):
                assert off[a[0]] + a[3] <= off[b[0]] or off[b[0]] + b[3] <= off[a[0]]
