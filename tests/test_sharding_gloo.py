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
