"""Batch sharding over ranks, exercised with two gloo ranks on CPU.

Each rank builds the same network (same seed, same weights) for its own shard of the batch, evaluates the
shard (here with the CPU oracle standing in for the device, which these tests do not have), and the ranks
all-gather their logits.  The result on every rank must equal the single-process evaluation of the whole
batch.  On GPUs ``bench.py`` runs the same host logic over NCCL with the library dispatching each shard.
"""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
NET = dict(image=32, width=8, blocks=(1, 1, 1, 1), classes=8)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, total: int, seed: int, result_dir: str) -> None:
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from __graft_entry__ import load_package
    load_package()
    from mlel_b200.model_graphs import resnet50_graph
    from mlel_b200.sharding import all_gather_batch, shard_arrays, shard_range
    from tests.graph_eval import evaluate

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        _, full_inputs = resnet50_graph(seed=seed, n=total, **NET)
        first, count = shard_range(total, world, rank)
        mine = shard_arrays(full_inputs, world, rank)
        assert mine[0].shape[0] == count
        if count > 0:
            g, _ = resnet50_graph(seed=seed, n=count, **NET)
            logits = evaluate(g, mine)[0].reshape(count, -1)
        else:
            logits = np.zeros((0, NET["classes"]), dtype=np.int8)
        gathered = all_gather_batch(torch.from_numpy(np.ascontiguousarray(logits)), total)
        np.save(os.path.join(result_dir, f"rank{rank}.npy"), gathered.numpy())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("total", [4, 5, 1])
def test_two_ranks_reproduce_the_whole_batch(tmp_path, total):
    import torch.multiprocessing as mp
    sys.path.insert(0, ROOT)
    from __graft_entry__ import load_package
    load_package()
    from mlel_b200.model_graphs import resnet50_graph
    from tests.graph_eval import evaluate

    world, seed = 2, 11
    g, inputs = resnet50_graph(seed=seed, n=total, **NET)
    want = evaluate(g, inputs)[0].reshape(total, -1)
    assert want.std() > 1.0
    mp.spawn(_rank_main, args=(world, _free_port(), total, seed, str(tmp_path)), nprocs=world, join=True)
    for rank in range(world):
        got = np.load(tmp_path / f"rank{rank}.npy")
        np.testing.assert_array_equal(got, want)


def _matmul_graph(a_shape, b, mult, shift, per_channel):
    from mlel_b200.graph_builder import GraphBuilder
    g = GraphBuilder("matmul_shard")
    a = g.input(np.int8, a_shape)
    bv = g.input(np.int8, b.shape)
    y = g.matmul(a, bv, -7, 0)
    g.output(g.rescale(y, mult, shift, 0, 3, np.int8, scale32=True, double_round=True, per_channel=per_channel))
    return g


def _column_rank_main(rank: int, world: int, port: int, width: int, per_channel: bool, result_dir: str) -> None:
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from __graft_entry__ import load_package
    load_package()
    from mlel_b200.sharding import all_gather_columns, shard_columns, shard_matmul_operands
    from tests.graph_eval import evaluate

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        a, b, mult, shift = _matmul_case(width, per_channel)
        b_r, (mult_r, shift_r) = shard_matmul_operands(b, [mult, shift], world, rank)
        count = shard_columns(width, world, rank)[1]
        assert b_r.shape[2] == count
        if count > 0:
            out = evaluate(_matmul_graph(a.shape, b_r, mult_r, shift_r, per_channel), [a, b_r])[0]
        else:
            out = np.zeros(a.shape[:2] + (0,), dtype=np.int8)
        joined = all_gather_columns(torch.from_numpy(np.ascontiguousarray(out)), width)
        np.save(os.path.join(result_dir, f"rank{rank}.npy"), joined.numpy())
    finally:
        dist.destroy_process_group()


def _matmul_case(width: int, per_channel: bool):
    r = np.random.Generator(np.random.PCG64(width + per_channel))
    a = r.integers(-128, 128, (2, 24, 32), dtype=np.int8)
    b = r.integers(-128, 128, (2, 32, width), dtype=np.int8)
    n = width if per_channel else 1
    mult = r.integers(1 << 30, (1 << 31) - 1, (n,), dtype=np.int64).astype(np.int32)
    shift = r.integers(36, 40, (n,), dtype=np.int8)
    return a, b, mult, shift


@pytest.mark.parametrize("width,per_channel", [(80, True), (64, False), (8, True)])
def test_two_ranks_reproduce_a_matmul_sharded_by_output_channel(tmp_path, width, per_channel):
    """Each rank computes its block of output columns (all of A, its columns of B, its slice of the per-channel
    RESCALE parameters); the joined blocks equal the unsharded product bit for bit.  80 columns split 48 + 32,
    8 columns leave the second rank empty."""
    import torch.multiprocessing as mp
    sys.path.insert(0, ROOT)
    from __graft_entry__ import load_package
    load_package()
    from tests.graph_eval import evaluate

    a, b, mult, shift = _matmul_case(width, per_channel)
    want = evaluate(_matmul_graph(a.shape, b, mult, shift, per_channel), [a, b])[0]
    assert want.std() > 1.0
    mp.spawn(_column_rank_main, args=(2, _free_port(), width, per_channel, str(tmp_path)), nprocs=2, join=True)
    for rank in range(2):
        np.testing.assert_array_equal(np.load(tmp_path / f"rank{rank}.npy"), want)


def test_shard_columns_are_aligned_and_cover_the_width():
    sys.path.insert(0, ROOT)
    from __graft_entry__ import load_package
    load_package()
    from mlel_b200.sharding import shard_columns
    for total in (0, 8, 16, 1000, 1024, 3072):
        for world in (1, 2, 4, 8):
            spans = [shard_columns(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and sum(c for _, c in spans) == total
            for (f0, c0), (f1, _) in zip(spans, spans[1:]):
                assert f1 == f0 + c0
            assert all(f % 16 == 0 for f, c in spans if c > 0)


def test_shard_range_covers_the_batch_exactly():
    sys.path.insert(0, ROOT)
    from __graft_entry__ import load_package
    load_package()
    from mlel_b200.sharding import shard_range
    for total in (0, 1, 7, 64, 65):
        for world in (1, 2, 3, 8):
            spans = [shard_range(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and sum(c for _, c in spans) == total
            for (f0, c0), (f1, _) in zip(spans, spans[1:]):
                assert f1 == f0 + c0
            assert max(c for _, c in spans) - min(c for _, c in spans) <= 1
    with pytest.raises(ValueError):
        shard_range(4, 2, 2)
