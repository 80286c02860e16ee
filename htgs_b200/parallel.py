"""Multi-GPU use of the rasterizer: one process per GPU, views partitioned across ranks.

Rendering a view needs nothing from any other view, so forward workloads shard by view with
no data-path collective (the scene is replicated on every GPU).  Only the training step has
an exchange: the per-Gaussian gradients of the ranks' views are summed with an all-reduce
(NCCL over NVLink on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

import os
from typing import Iterable, List, Sequence


def rank_world():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))


def shard_views(n_views: int, rank: int, world: int) -> List[int]:
    """Round-robin partition of view indices: rank r renders views r, r + world, ..."""
    if not (0 <= rank < world):
        raise ValueError("rank must be in [0, world)")
    return list(range(rank, n_views, world))


def step_view_indices(step: int, views_per_step: int, rank: int, world: int, n_views: int) -> List[int]:
    """Views rank `rank` renders in step `step` when every rank renders `views_per_step` frames per step
    (weak scaling: the per-GPU work is fixed, the job covers world * views_per_step views per step)."""
    base = step * views_per_step * world
    return [(base + i * world + rank) % n_views for i in range(views_per_step)]


def init_process_group(backend: str):
    import torch.distributed as dist
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        dist.init_process_group(backend=backend)
    return dist


def allreduce_gradients(grads: Sequence, group=None, async_op: bool = False):
    """Sums per-Gaussian gradient tensors over the ranks, in place.  Returns the work handles when async."""
    import torch.distributed as dist
    handles = []
    for g in grads:
        if g is None:
            continue
        h = dist.all_reduce(g, op=dist.ReduceOp.SUM, group=group, async_op=async_op)
        if async_op:
            handles.append(h)
    return handles


def allreduce_gradients_rows(grads: Sequence, rows, group=None) -> int:
    """Sums per-Gaussian gradient tensors over the ranks, in place, exchanging only the rows some rank can have touched.

    `rows` is a bool tensor [N]: the rows of this rank's tensors that may be non-zero (the Gaussians its view kept,
    `torch_bindings.rasterization.last_training_visibility`); all other rows MUST be zero on this rank.  The union of the
    ranks' row sets is formed with one small all-reduce, the union's rows are gathered into dense buffers, summed, and
    written back; rows outside the union are zero on every rank and stay untouched.  A view keeps a sixth of a scene's
    Gaussians, so the exchange moves the union's share of the 236 bytes per Gaussian instead of all of them.
    One host synchronisation (the size of the union).  Returns the number of rows exchanged."""
    import torch
    import torch.distributed as dist
    tensors = [g for g in grads if g is not None]
    if not tensors:
        return 0
    n = rows.shape[0]
    union = rows.to(torch.int32)
    dist.all_reduce(union, op=dist.ReduceOp.MAX, group=group)
    index = torch.nonzero(union, as_tuple=False).squeeze(1)
    count = int(index.numel())
    if count == 0:
        return 0
    for g in tensors:
        if g.shape[0] != n:
            raise ValueError("every gradient tensor needs one leading row per Gaussian")
        flat = g.view(n, -1)
        packed = flat.index_select(0, index)
        dist.all_reduce(packed, op=dist.ReduceOp.SUM, group=group)
        flat.index_copy_(0, index, packed)
    return count


def max_over_ranks(value: float, device=None) -> float:
    """Maximum of a host scalar over all ranks (timings are reported as the slowest rank's)."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(value: float, device=None) -> float:
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())
