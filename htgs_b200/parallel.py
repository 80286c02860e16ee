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


# Packing and unpacking read and write the exchanged rows once more each; measured on B200s the row exchange stops paying
# when the union holds more than about 0.65 of the rows, so above this share the dense tensors are all-reduced instead.
kDenseAbove = 0.6


class RowExchange:
    """The rows (`index`, ascending, int64) the ranks are going to exchange and the stream the list was made on."""
    def __init__(self, index, side_stream=None):
        self.index = index
        self.count = int(index.numel())
        self.side_stream = side_stream


_side_streams: dict = {}


def begin_row_exchange(rows, group=None, ready=None) -> "RowExchange":
    """First half of the row exchange; call it right after the training forward, while its kernels still run.

    `rows` is a bool tensor [N]: the rows of this rank's gradient tensors that can become non-zero (the Gaussians its view
    kept, `torch_bindings.rasterization.last_training_visibility`).  One small MAX all-reduce forms the union over the
    ranks and its row indices are listed.  On CUDA this happens on a side stream, so the one host synchronisation it needs
    (the size of the union) does not wait for the work queued on the current stream: pass `ready`, the CUDA event after
    which `rows` is valid (`last_training_visibility(device, with_event=True)`), and the side stream waits for that event
    alone, i.e. for the preprocess pass, while the GPU keeps blending."""
    import torch
    import torch.distributed as dist
    if rows.is_cuda:
        device = rows.device
        side = _side_streams.get(device)
        if side is None:
            side = _side_streams[device] = torch.cuda.Stream(device=device)
        if ready is not None:
            side.wait_event(ready)
        else:
            side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            union = rows.to(torch.int32)
            dist.all_reduce(union, op=dist.ReduceOp.MAX, group=group)
            index = torch.nonzero(union, as_tuple=False).squeeze(1)
        rows.record_stream(side)
        return RowExchange(index, side)
    union = rows.to(torch.int32)
    dist.all_reduce(union, op=dist.ReduceOp.MAX, group=group)
    return RowExchange(torch.nonzero(union, as_tuple=False).squeeze(1))


def finish_row_exchange(grads: Sequence, exchange: "RowExchange", group=None) -> int:
    """Second half: sums rows `exchange.index` of the per-Gaussian gradient tensors over the ranks, in place; every other row
    must be zero on every rank and stays untouched.  On CUDA the rows of all tensors are packed into one buffer by one kernel
    (`htgs_gather_rows`), summed by one all-reduce and written back by one kernel; no host synchronisation.
    When the union holds more than `kDenseAbove` of the rows the dense tensors are all-reduced instead.
    Returns the number of rows exchanged."""
    import torch
    import torch.distributed as dist
    tensors = [g for g in grads if g is not None]
    if not tensors or exchange.count == 0:
        return 0
    n = tensors[0].shape[0]
    for g in tensors:
        if g.shape[0] != n:
            raise ValueError("every gradient tensor needs one leading row per Gaussian")
    index = exchange.index
    if exchange.count > kDenseAbove * n:     # the same decision on every rank: the union and n are the same everywhere
        allreduce_gradients(tensors, group=group)
        return n
    if tensors[0].is_cuda:
        import ctypes
        from . import _native
        if len(tensors) > 8 or any(g.dtype != torch.float32 or not g.is_contiguous() for g in tensors):
            raise ValueError("the row exchange takes up to 8 contiguous float32 tensors")
        device = tensors[0].device
        current = torch.cuda.current_stream(device)
        if exchange.side_stream is not None:
            current.wait_stream(exchange.side_stream)
            index.record_stream(current)
        table = _native.HtgsRowTensors()
        table.n_tensors = len(tensors)
        width = 0
        for k, g in enumerate(tensors):
            table.data[k] = g.data_ptr()
            table.width[k] = g[0].numel()
            width += g[0].numel()
        packed = torch.empty((exchange.count, width), dtype=torch.float32, device=device)
        lib = _native.lib()
        with torch.cuda.device(device):
            _native.check(lib.htgs_gather_rows(ctypes.byref(table), index.data_ptr(), exchange.count, packed.data_ptr(), current.cuda_stream))
            dist.all_reduce(packed, op=dist.ReduceOp.SUM, group=group)
            _native.check(lib.htgs_scatter_rows(ctypes.byref(table), index.data_ptr(), exchange.count, packed.data_ptr(), current.cuda_stream))
        return exchange.count
    for g in tensors:          # host tensors (the gloo tests of this logic)
        flat = g.view(n, -1)
        packed = flat.index_select(0, index)
        dist.all_reduce(packed, op=dist.ReduceOp.SUM, group=group)
        flat.index_copy_(0, index, packed)
    return exchange.count


def allreduce_gradients_rows(grads: Sequence, rows, group=None) -> int:
    """Sums per-Gaussian gradient tensors over the ranks, in place, exchanging only the rows some rank can have touched:
    `begin_row_exchange` and `finish_row_exchange` in one call (the host then waits for the backward pass before it can
    size the exchange; call the two halves separately to avoid that).

    A view keeps a sixth of a scene's Gaussians, so the exchange moves the union's share of the 236 bytes per Gaussian
    instead of all of them.  The result equals the dense all-reduce's exactly: rows outside the union are zero on every rank."""
    return finish_row_exchange(grads, begin_row_exchange(rows, group), group)


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
