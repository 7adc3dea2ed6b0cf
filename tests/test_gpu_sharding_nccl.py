"""Two GPUs, one process each, NCCL: batch sharding of a whole graph and output-channel sharding of one MATMUL
give, after the all-gather, the bits the CPU oracle gives for the unsharded problem.  Skipped on machines with
fewer than two GPUs (the single-GPU logic of the same functions is covered with gloo ranks on CPU in
test_sharding_gloo.py)."""
import os
import socket
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
NET = dict(image=32, width=16, blocks=(1, 1, 1, 1), classes=16)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _matmul_case(width: int):
    r = np.random.Generator(np.random.PCG64(width))
    a = r.integers(-128, 128, (2, 256, 128), dtype=np.int8)
    b = r.integers(-128, 128, (2, 128, width), dtype=np.int8)
    mult = r.integers(1 << 30, (1 << 31) - 1, (width,), dtype=np.int64).astype(np.int32)
    shift = r.integers(36, 40, (width,), dtype=np.int8)
    return a, b, mult, shift


def _matmul_graph(a_shape, b, mult, shift):
    from mlel_b200.graph_builder import GraphBuilder
    g = GraphBuilder("matmul_shard")
    a = g.input(np.int8, a_shape)
    bv = g.constant(b)
    y = g.matmul(a, bv, -7, 0)
    g.output(g.rescale(y, mult, shift, 0, 3, np.int8, scale32=True, double_round=True, per_channel=True))
    return g


def _rank_main(rank: int, world: int, port: int, total: int, width: int, result_dir: str) -> None:
    sys.path.insert(0, ROOT)
    # NVLS off: a rank that dies while bound to a multicast object disturbs the other rank's GPU
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import torch
    import torch.distributed as dist
    from __graft_entry__ import load_package
    load_package()
    from mlel_b200.model_graphs import resnet50_graph
    from mlel_b200.runtime import GraphRunner
    from mlel_b200.sharding import (all_gather_batch, all_gather_columns, shard_arrays, shard_columns,
                                    shard_matmul_operands, shard_range)

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        device = torch.device("cuda", rank)
        # batch sharding of a whole graph
        _, full_inputs = resnet50_graph(seed=21, n=total, **NET)
        count = shard_range(total, world, rank)[1]
        g, _ = resnet50_graph(seed=21, n=count, **NET)
        logits = GraphRunner(g, device=device).run(shard_arrays(full_inputs, world, rank))[0].reshape(count, -1)
        gathered = all_gather_batch(torch.from_numpy(np.ascontiguousarray(logits)).to(device), total)
        np.save(os.path.join(result_dir, f"batch{rank}.npy"), gathered.cpu().numpy())
        # output-channel sharding of one MATMUL + per-channel RESCALE
        a, b, mult, shift = _matmul_case(width)
        b_r, (mult_r, shift_r) = shard_matmul_operands(b, [mult, shift], world, rank)
        assert b_r.shape[2] == shard_columns(width, world, rank)[1] > 0
        out = GraphRunner(_matmul_graph(a.shape, b_r, mult_r, shift_r), device=device).run([a])[0]
        joined = all_gather_columns(torch.from_numpy(np.ascontiguousarray(out)).to(device), width)
        np.save(os.path.join(result_dir, f"cols{rank}.npy"), joined.cpu().numpy())
    finally:
        dist.destroy_process_group()


def test_two_gpus_reproduce_the_unsharded_results(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from mlel_b200.model_graphs import resnet50_graph
    from tests.graph_eval import evaluate

    total, width = 5, 208  # uneven shards: 3 + 2 images, 112 + 96 columns
    g, inputs = resnet50_graph(seed=21, n=total, **NET)
    want_batch = evaluate(g, inputs)[0].reshape(total, -1)
    a, b, mult, shift = _matmul_case(width)
    want_cols = evaluate(_matmul_graph(a.shape, b, mult, shift), [a])[0]
    assert want_batch.std() > 1.0 and want_cols.std() > 1.0
    mp.spawn(_rank_main, args=(2, _free_port(), total, width, str(tmp_path)), nprocs=2, join=True)
    for rank in range(2):
        np.testing.assert_array_equal(np.load(tmp_path / f"batch{rank}.npy"), want_batch)
        np.testing.assert_array_equal(np.load(tmp_path / f"cols{rank}.npy"), want_cols)
