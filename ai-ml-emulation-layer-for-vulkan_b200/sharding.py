"""Sharding of a data-graph dispatch over ranks (one process per GPU): by batch, and by output channel.

A TOSA data graph of the kind this library runs treats the images of a batch independently: every
operator on the path is per-pixel, per-window or per-row of one image, so a batch of B images can be
cut into contiguous shards, each rank dispatches its own shard through its own pipeline and session,
and no tensor crosses ranks while the graph runs.  The only exchange is the all-gather of the graph's
outputs (the logits) at the end, and only when the caller wants the whole batch on every rank.

The reference has no multi-device path (one VkDevice per graph pipeline, graph/graph_layer.cpp:853-1003);
this module is the host-side logic a data-parallel host needs on top of the C ABI.  It uses
``torch.distributed`` with whatever backend the process group was created with (NCCL on GPUs, gloo in the
CPU tests).
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import numpy as np
import torch
import torch.distributed as dist


def shard_range(total: int, world: int, rank: int) -> Tuple[int, int]:
    """``(first, count)`` of the contiguous shard of ``total`` items owned by ``rank``.

    Shards differ by at most one item; the first ``total % world`` ranks hold the larger ones.  Ranks past
    the end of a batch smaller than the world get an empty shard.
    """
    if world <= 0 or not 0 <= rank < world or total < 0:
        raise ValueError(f"bad shard request: total={total} world={world} rank={rank}")
    base, extra = divmod(total, world)
    first = rank * base + min(rank, extra)
    return first, base + (1 if rank < extra else 0)


def shard_arrays(arrays: Sequence[np.ndarray], world: int, rank: int) -> List[np.ndarray]:
    """The rank's slice along axis 0 (the batch axis) of every graph input."""
    out = []
    for a in arrays:
        first, count = shard_range(a.shape[0], world, rank)
        out.append(np.ascontiguousarray(a[first:first + count]))
    return out


def all_gather_batch(local: torch.Tensor, total: int, group=None) -> torch.Tensor:
    """Concatenates every rank's output shard along axis 0 and returns the whole batch on every rank.

    ``local`` is this rank's ``[count, ...]`` output, ``total`` the batch size that ``shard_range`` cut.
    Shards of equal size go through one ``all_gather_into_tensor``; uneven shards are padded to the largest
    one for the exchange and trimmed afterwards.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    first, count = shard_range(total, world, rank)
    if local.shape[0] != count:
        raise ValueError(f"rank {rank} holds {local.shape[0]} items, its shard of {total} has {count}")
    biggest = shard_range(total, world, 0)[1]
    tail = tuple(local.shape[1:])
    if total % world == 0:
        out = torch.empty((total,) + tail, dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(out, local.contiguous(), group=group)
        return out
    padded = torch.zeros((biggest,) + tail, dtype=local.dtype, device=local.device)
    padded[:count] = local
    pieces = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(pieces, padded, group=group)
    return torch.cat([pieces[r][:shard_range(total, world, r)[1]] for r in range(world)], dim=0)


# ---- output-channel sharding of one large MATMUL ---------------------------------------------------------------
#
# A single-batch (or few-batch) MATMUL  out[n, h, w] = sum_c A[n, h, c] * B[n, c, w]  with its RESCALE can be cut
# along w: every rank keeps all of A, takes a block of B's columns and the matching slice of the per-channel
# RESCALE parameters, and computes  out[:, :, w0:w1]  with the fused epilogue.  The contraction axis is never
# split, so no reduction crosses ranks and the integer results are the same bits as on one GPU; the only exchange
# is the all-gather of the column blocks.

def shard_columns(total: int, world: int, rank: int, align: int = 16) -> Tuple[int, int]:
    """``(first, count)`` of the block of ``total`` output columns owned by ``rank``.

    Blocks are multiples of ``align`` columns (the tensor-core path moves 16-byte pieces of a row) except that
    the last non-empty block takes the remainder; ranks past the end get an empty block."""
    if world <= 0 or not 0 <= rank < world or total < 0 or align <= 0:
        raise ValueError(f"bad shard request: total={total} world={world} rank={rank} align={align}")
    units = -(-total // align)  # blocks of `align` columns, the last one possibly short
    first_unit, count_units = shard_range(units, world, rank)
    first = min(first_unit * align, total)
    last = min((first_unit + count_units) * align, total)
    return first, last - first


def shard_matmul_operands(b: np.ndarray, per_channel: Sequence[np.ndarray], world: int, rank: int,
                          align: int = 16) -> Tuple[np.ndarray, List[np.ndarray]]:
    """The rank's column block of ``b`` ``[N, C, W]`` and the same slice of every per-channel parameter vector
    (RESCALE multipliers and shifts of length ``W``; vectors of length 1 are per-tensor and pass unchanged)."""
    first, count = shard_columns(b.shape[2], world, rank, align)
    params = [np.ascontiguousarray(p if p.shape[0] == 1 else p[first:first + count]) for p in per_channel]
    return np.ascontiguousarray(b[:, :, first:first + count]), params


def all_gather_columns(local: torch.Tensor, total: int, align: int = 16, group=None) -> torch.Tensor:
    """Joins every rank's ``[N, H, count]`` block along the last axis into ``[N, H, total]`` on every rank.

    The column axis is the contiguous one, so the blocks cannot be gathered in place: one
    ``all_gather_into_tensor`` brings them, each padded to the widest block, into a ``[world, N, H, widest]``
    staging buffer, and one local pass interleaves them.  On CUDA tensors that pass is the library's own kernel
    (``mlel_cuda_interleave_columns``, on the current stream); CPU ranks (the gloo tests of this logic) do the
    same join on the host."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    first, count = shard_columns(total, world, rank, align)
    if local.shape[-1] != count:
        raise ValueError(f"rank {rank} holds {local.shape[-1]} columns, its block of {total} has {count}")
    blocks = [shard_columns(total, world, r, align) for r in range(world)]
    widest = max(c for _, c in blocks)
    if count == widest and local.is_contiguous():
        padded = local
    else:
        padded = torch.zeros(tuple(local.shape[:-1]) + (widest,), dtype=local.dtype, device=local.device)
        padded[..., :count] = local
    if padded.dim() == 0:
        padded = padded.reshape(1)
    # the gathered tensor is the ranks' blocks concatenated along axis 0 (the form every backend accepts)
    flat = torch.empty((world * padded.shape[0],) + tuple(padded.shape[1:]), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(flat, padded, group=group)
    staging = flat.view((world,) + tuple(padded.shape))
    if local.is_cuda:
        import ctypes

        from . import check, lib
        item = local.element_size()
        rows = int(np.prod(local.shape[:-1])) if local.dim() > 1 else 1
        out = torch.empty(tuple(local.shape[:-1]) + (total,), dtype=local.dtype, device=local.device)
        firsts = (ctypes.c_int32 * world)(*[f * item for f, _ in blocks])
        counts = (ctypes.c_int32 * world)(*[c * item for _, c in blocks])
        stream = torch.cuda.current_stream(local.device).cuda_stream
        check(lib().mlel_cuda_interleave_columns(ctypes.c_void_p(staging.data_ptr()), ctypes.c_void_p(out.data_ptr()),
                                                 ctypes.c_uint64(rows), ctypes.c_uint32(world),
                                                 ctypes.c_uint32(widest * item), firsts, counts,
                                                 ctypes.c_void_p(stream)))
        return out
    return torch.cat([staging[r][..., :blocks[r][1]] for r in range(world)], dim=-1)
