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


def rows_outside_are_zero(grads: Sequence, exchange: "RowExchange") -> bool:
    """Debug check for the row exchange's one assumption: on this rank, every gradient row outside `exchange.index` is exactly
    zero.  It fails when something other than the rasterizer's backward reaches the parameters - a regulariser on opacities
    or scales, weight decay - or when a step ran several forwards without accumulating their visibility
    (`track_training_visibility(True, accumulate=True)`): such rows would stay un-summed and the replicas would drift apart.
    One masked abs-max per tensor and a host read: for tests and debugging, not for the training loop."""
    import torch
    tensors = [g for g in grads if g is not None and g.numel() > 0]
    if not tensors:
        return True
    n = tensors[0].shape[0]
    outside = torch.ones(n, dtype=torch.bool, device=tensors[0].device)
    outside[exchange.index] = False
    return all(float(g.reshape(n, -1)[outside].abs().max().item() if bool(outside.any()) else 0.0) == 0.0 for g in tensors)


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


def _sum_rows(tensors, index, lo: int, hi: int, stream, group) -> None:
    """Sums rows index[lo:hi] of the tensors over the ranks (gather -> one all-reduce -> scatter), queued on `stream`."""
    import ctypes
    import torch
    import torch.distributed as dist
    if hi <= lo:
        return
    if tensors[0].is_cuda:
        from . import _native
        table = _native.HtgsRowTensors()
        table.n_tensors = len(tensors)
        width = 0
        for k, g in enumerate(tensors):
            table.data[k] = g.data_ptr()
            table.width[k] = g[0].numel()
            width += g[0].numel()
        packed = torch.empty((hi - lo, width), dtype=torch.float32, device=tensors[0].device)
        lib = _native.lib()
        first = index.data_ptr() + 8 * lo
        _native.check(lib.htgs_gather_rows(ctypes.byref(table), first, hi - lo, packed.data_ptr(), stream.cuda_stream))
        dist.all_reduce(packed, op=dist.ReduceOp.SUM, group=group)
        _native.check(lib.htgs_scatter_rows(ctypes.byref(table), first, hi - lo, packed.data_ptr(), stream.cuda_stream))
        return
    n = tensors[0].shape[0]
    rows = index[lo:hi]
    for g in tensors:          # host tensors (the gloo tests of this logic)
        flat = g.view(n, -1)
        packed = flat.index_select(0, rows)
        dist.all_reduce(packed, op=dist.ReduceOp.SUM, group=group)
        flat.index_copy_(0, rows, packed)


class BackwardExchange:
    """Sums the rasterizer's six gradient tensors over the ranks WHILE the backward pass still runs.

    The six tensors become final in the last kernel of the backward pass, so an exchange that starts after `loss.backward()`
    has nothing to hide behind.  Here the pass runs over `n_chunks` ranges of Gaussian indices, one after the other
    (`htgs_backward_range`: a tile's list is ascending in Gaussian index, so a range costs its share of the pass), and as
    soon as a range has been queued its rows are summed on a second stream: gather of the rows some rank's view kept ->
    one NCCL all-reduce -> scatter, all while the next range is computed.  Only the last range's exchange is exposed.
    Every rank uses the same ranges (they depend on the scene size alone), so the collectives match.

    Use per training step:
        xchg.begin(visible, ready)     # right after the forward: union of the ranks' visible sets (overlaps the blend)
        loss.backward()                # with rasterization.set_backward_hook(xchg) installed
    after which the gradients autograd received from `diff_rasterize` are sums over the ranks.  What the rasterizer's
    gradients are chained through on the way to the leaves (the activation functions of the parameters) is the same linear
    map on every rank, so summing before it equals summing after it; loss terms that reach the parameters by other paths
    (regularisers, weight decay) are NOT summed by this and stay the caller's to handle.
    ALPHA_BLEND_GLOBAL_ORDERING cannot run over a part of the Gaussians: it gets one range (no overlap)."""

    def __init__(self, n_chunks: int = 4, group=None, measure: bool = False, split_pass: bool = False):
        self.n_chunks = max(1, int(n_chunks))
        self.group = group
        # split_pass = True: the per-tile pass of the backward runs range by range too (`htgs_backward_range`), so a range's
        # exchange overlaps the next range's share of the whole pass - but every extra pass over the tiles has a fixed cost
        # (measured: about a third of the whole pass per extra range at 3 M Gaussians), which only a slow interconnect repays.
        # split_pass = False (default): the per-tile pass runs once and only the per-Gaussian chain rule runs range by range;
        # packing, all-reduce and unpacking of successive ranges then overlap each other on three streams.
        self.split_pass = bool(split_pass)
        self._pack = self._unpack = None
        self.measure = measure          # record CUDA events around the wait for the last range's exchange (exposed_ms)
        self._marks = []
        self.exchange = None
        self.bounds = None
        self.dense = False
        self.rows_exchanged = 0
        self._chunk_ranges = None
        self._comm = None

    def chunk_ranges(self, n: int, mode: int = 0):
        chunks = 1 if (mode == 2 and self.split_pass) else self.n_chunks
        edges = [(n * k) // chunks for k in range(chunks + 1)]
        return [(edges[k], edges[k + 1] - edges[k]) for k in range(chunks)]

    ranges = chunk_ranges       # the name the autograd hook calls

    def begin(self, rows, ready=None, mode: int = 0) -> None:
        """`rows`: bool tensor [N] of the Gaussians this rank's view kept (`last_training_visibility`); `ready`: the event
        after which it is valid.  Forms the union over the ranks and finds where each range of Gaussians starts in its
        (ascending) index list.  One host synchronisation, on the side stream."""
        import torch
        n = rows.shape[0]
        self.exchange = begin_row_exchange(rows, self.group, ready)
        self._chunk_ranges = self.chunk_ranges(n, mode)
        index = self.exchange.index
        self.dense = self.exchange.count > kDenseAbove * n
        edges = [first for first, _ in self._chunk_ranges] + [n]
        if self.dense or self.exchange.count == 0:
            self.bounds = None
        elif index.is_cuda:
            with torch.cuda.stream(self.exchange.side_stream):
                self.bounds = torch.searchsorted(index, torch.tensor(edges, dtype=index.dtype, device=index.device)).tolist()
        else:
            self.bounds = torch.searchsorted(index, torch.tensor(edges, dtype=index.dtype)).tolist()
        self.rows_exchanged = n if self.dense else self.exchange.count

    def after_range(self, k: int, first: int, count: int, grads) -> None:
        import torch
        import torch.distributed as dist
        tensors = [g for g in grads if g is not None and g.numel() > 0]
        if not tensors or count == 0 or self.exchange is None:
            return
        cuda = tensors[0].is_cuda
        if cuda:
            device = tensors[0].device
            comm = self.exchange.side_stream
            if comm is None:
                comm = _side_streams.get(device) or _side_streams.setdefault(device, torch.cuda.Stream(device=device))
            self._comm = comm
            done = torch.cuda.Event()
            done.record(torch.cuda.current_stream(device))
            if not self.dense and self.bounds is not None:
                self._sum_rows_pipelined(tensors, self.bounds[k], self.bounds[k + 1], done)
                return
            comm.wait_event(done)
            context = torch.cuda.stream(comm)
        else:
            import contextlib
            comm, context = None, contextlib.nullcontext()
        with context:
            if self.dense:
                for g in tensors:
                    dist.all_reduce(g[first:first + count], op=dist.ReduceOp.SUM, group=self.group)
            elif self.bounds is not None:
                _sum_rows(tensors, self.exchange.index, self.bounds[k], self.bounds[k + 1], comm, self.group)

    def _sum_rows_pipelined(self, tensors, lo: int, hi: int, done) -> None:
        """Packing, all-reduce and unpacking of one range on three streams, so that the packing of range k + 1 and the unpacking
        of range k - 1 run while range k is on the wire."""
        import ctypes
        import torch
        import torch.distributed as dist
        from . import _native
        if hi <= lo:
            return
        device = tensors[0].device
        comm = self._comm
        if self._pack is None:
            self._pack, self._unpack = torch.cuda.Stream(device=device), torch.cuda.Stream(device=device)
        table = _native.HtgsRowTensors()
        table.n_tensors = len(tensors)
        width = 0
        for t, g in enumerate(tensors):
            table.data[t] = g.data_ptr()
            table.width[t] = g[0].numel()
            width += g[0].numel()
        lib = _native.lib()
        first = self.exchange.index.data_ptr() + 8 * lo
        self._pack.wait_event(done)
        self._pack.wait_stream(comm)         # the index list was made on the communication stream
        with torch.cuda.stream(self._pack):
            packed = torch.empty((hi - lo, width), dtype=torch.float32, device=device)
            _native.check(lib.htgs_gather_rows(ctypes.byref(table), first, hi - lo, packed.data_ptr(), self._pack.cuda_stream))
        comm.wait_stream(self._pack)
        with torch.cuda.stream(comm):
            dist.all_reduce(packed, op=dist.ReduceOp.SUM, group=self.group)
        packed.record_stream(comm)
        self._unpack.wait_stream(comm)
        with torch.cuda.stream(self._unpack):
            _native.check(lib.htgs_scatter_rows(ctypes.byref(table), first, hi - lo, packed.data_ptr(), self._unpack.cuda_stream))
        packed.record_stream(self._unpack)

    def finish(self, grads) -> None:
        import torch
        if self._comm is not None:
            current = torch.cuda.current_stream(self._comm.device)
            if self.measure:
                before, after = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                before.record(current)
            current.wait_stream(self._comm)
            if self._unpack is not None:
                current.wait_stream(self._unpack)
            if self.measure:
                after.record(current)
                self._marks.append((before, after))
            for g in grads:
                if g is not None and g.is_cuda:
                    g.record_stream(self._comm)
            self.exchange.index.record_stream(self._comm)


    def exposed_ms(self, last: int = 0):
        """With `measure`: per step, the time the compute stream waited for the exchange after its own last kernel of the
        backward pass (call after a device synchronisation).  `last` > 0 keeps the most recent steps only."""
        marks = self._marks[-last:] if last else self._marks
        return [a.elapsed_time(b) for a, b in marks]


kCompactRowBytes = 64      # one header and one row of a compact gradient buffer (include/htgs_b200.h: htgs_backward_compact)


class _DeviceSpan:
    """A piece of device memory that is not a torch tensor (what `CompactExchange.buffer` hands out for the peer transport)."""
    def __init__(self, address: int, nbytes: int):
        self._address, self._nbytes = int(address), int(nbytes)

    def data_ptr(self) -> int:
        return self._address

    def numel(self) -> int:
        return self._nbytes


class _PeerBuffers:
    """Two compact-row buffers per rank (used in turn), each mapped into every other rank's process (`htgs_peer_buffer_*`)."""
    def __init__(self, device_index: int, nbytes: int, group):
        """Collective.  Does not raise when a CUDA call fails: `problem` holds the first failure of this rank (or tells that
        another rank failed), so that all ranks can decide together what to do."""
        import ctypes
        import torch.distributed as dist
        from . import _native
        self.lib, self.device_index, self.nbytes, self.group = _native.lib(), int(device_index), int(nbytes), group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.local, self.opened, self.problem, self.turn = [], [], None, 0
        self.maps = [[0] * self.world for _ in range(2)]
        handles = []
        try:
            for _ in range(2):
                ptr, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
                _native.check(self.lib.htgs_peer_buffer_create(self.device_index, self.nbytes, ctypes.byref(ptr), handle))
                self.local.append(int(ptr.value))
                handles.append(bytes(handle.raw))
        except Exception as exc:
            self.problem, handles = exc, None
        everyone = [None] * self.world
        dist.all_gather_object(everyone, (self.nbytes, handles), group=group)
        if self.problem is not None:
            return
        if any(theirs is None for _, theirs in everyone):
            self.problem = RuntimeError("another rank could not create its compact-row buffers")
            return
        if any(size != self.nbytes for size, _ in everyone):
            self.problem = RuntimeError("the ranks disagree on the size of the compact-row buffers (different scenes?)")
            return
        try:
            for r, (_, theirs) in enumerate(everyone):
                for b in range(2):
                    if r == self.rank:
                        self.maps[b][r] = self.local[b]
                    else:
                        ptr = ctypes.c_void_p()
                        _native.check(self.lib.htgs_peer_buffer_open(self.device_index, theirs[b], ctypes.byref(ptr)))
                        self.maps[b][r] = int(ptr.value)
                        self.opened.append(int(ptr.value))
        except Exception as exc:
            self.problem = exc

    def close(self) -> None:
        """Collective: every rank closes its mappings, then the owners free the buffers."""
        import torch
        import torch.distributed as dist
        from . import _native
        if self.lib is None:
            return
        torch.cuda.synchronize(self.device_index)
        for ptr in self.opened:
            _native.check(self.lib.htgs_peer_buffer_close(self.device_index, ptr))
        self.opened = []
        dist.barrier(group=self.group)
        for ptr in self.local:
            _native.check(self.lib.htgs_peer_buffer_destroy(self.device_index, ptr))
        self.local, self.lib = [], None


class CompactExchange:
    """Sums the rasterizer's six gradient tensors over the ranks by exchanging COMPACT rows.

    A rank's backward pass makes non-zero gradient rows only for the Gaussians its view kept (about a sixth of the scene), and
    48 of a row's 59 floats (SH degree 3) are the 3-vector dL/drgb times functions of the view direction.  So instead of
    all-reducing dense rows (236 bytes per Gaussian of the union of all ranks' views) every rank publishes 64 bytes per
    Gaussian ITS view kept (`htgs_backward_compact`) and every rank forms the dense sums itself from all ranks' buffers, in
    rank order (`htgs_expand_add_rows` / `htgs_expand_sum_rows`).  Same order on every rank: the sums are bit-identical
    everywhere, like an all-reduce's.  At 8 ranks and configuration 2 a rank reads 7 x 33 MB instead of taking part in the
    reduction of 383 MB.

    transport = "peer" (default on CUDA with more than one rank): every rank's buffer is plain device memory that the other
        ranks' GPUs read over NVLink with ordinary loads (CUDA IPC mappings made once; `htgs_peer_buffer_*`).  Per step the
        ranks pass one tiny all-reduce on their streams - the barrier between writing and reading - and nothing else: no
        sizes to agree on, no host synchronisation.  Two ranks: the expanding kernel reads the peer's rows in place.  More:
        each rank first pulls the peers' buffers into local memory, starting with a different peer each, and sums all buffers
        in one pass (see `exchange`).  Two buffers per rank are used in turn, so the next step's barrier also orders a buffer's
        readers before its next writer.  Costs 2 x 64 bytes x N of device memory, plus (ranks - 1) x 64 x N for the copies.
    transport = "nccl": buffers padded to the largest kept count of any rank, one all-gather, expansion from the gathered
        copy.  `begin` agrees on that count (one tiny all-gather and a host synchronisation on a side stream).

    Use per training step, with `rasterization.set_backward_hook(xchg)` installed once:
        xchg.begin(visible, ready)     # right after the forward; needed by the "nccl" transport only
        loss.backward()                # the gradients autograd receives from diff_rasterize are sums over the ranks
    The caveats of BackwardExchange apply: loss terms that reach the parameters past the rasterizer are not summed, and a
    step with several forwards per rank needs one backward per forward.  Call `close()` (collective) before the process
    group is destroyed."""

    compact = True      # what the autograd hook of torch_bindings.rasterization looks for

    def __init__(self, group=None, transport: str = "auto"):
        if transport not in ("auto", "peer", "nccl"):
            raise ValueError("transport must be 'auto', 'peer' or 'nccl'")
        self.group = group
        self.transport = transport
        self._capacity = None
        self._peers = None
        self._token = None
        self._staging = None
        self.always_stage = False     # tests and profiles: take the route of more than two ranks (copy, then one-pass sums) with fewer
        self.rows_published = 0       # "nccl": rows of this rank in the last step
        self.bytes_gathered = 0       # "nccl": bytes the last all-gather delivered to this rank (all ranks' buffers)

    @staticmethod
    def _world(group) -> int:
        import torch.distributed as dist
        return dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1

    def _use_peers(self, is_cuda: bool) -> bool:
        if self._world(self.group) == 1:      # a single rank expands its own buffer: nothing to map
            self.transport = "nccl"
        if self.transport == "auto":
            self.transport = "peer" if (is_cuda and self._world(self.group) > 1) else "nccl"
        if self.transport == "peer" and not is_cuda:
            raise ValueError("the peer transport needs CUDA tensors")
        return self.transport == "peer"

    def begin(self, rows, ready=None) -> None:
        """`rows`: bool tensor [N] of the Gaussians this rank's view kept; `ready`: the event after which it is valid.
        Does nothing for the peer transport."""
        import torch
        import torch.distributed as dist
        if self._use_peers(rows.is_cuda):
            return
        world = self._world(self.group)
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
                count = rows.sum(dtype=torch.int64).reshape(1)
                counts = torch.empty(world, dtype=torch.int64, device=device)
                if world > 1:
                    dist.all_gather_into_tensor(counts, count, group=self.group)
                else:
                    counts.copy_(count)
                mine, largest = int(count.item()), int(counts.max().item())
            rows.record_stream(side)
        else:
            count = rows.sum(dtype=torch.int64).reshape(1)
            gathered = [torch.empty_like(count) for _ in range(world)]
            if world > 1:
                dist.all_gather(gathered, count, group=self.group)
            else:
                gathered[0].copy_(count)
            mine, largest = int(count.item()), max(int(c.item()) for c in gathered)
        self.rows_published = mine
        self._capacity = max(1024, -(-largest // 1024) * 1024)      # whole kilorows: few distinct buffer sizes over a run

    def expansion(self) -> str:
        """How the autograd hook turns the buffers into dense sums: "sum" = one pass that writes every dense row once
        (`htgs_expand_sum_rows`; needs all buffers in local memory), "add" = buffer after buffer (`htgs_expand_add_rows`; reads
        the one peer's buffer of a two-rank job in place)."""
        world = self._world(self.group)
        if self.transport == "auto":
            self._use_peers(True)
        if world > 2:
            return "sum"
        return "sum" if (self.always_stage or (world == 2 and self.transport == "nccl")) else "add"

    def capacity(self, n: int) -> int:
        if self.transport == "auto":
            self._use_peers(True)
        if self.transport == "peer":      # the buffer holds a row for every Gaussian of the scene; readers go by the header's count
            return max(int(n), 1)
        if self._capacity is None:
            raise RuntimeError("CompactExchange.begin was not called after the forward of this step")
        return min(self._capacity, max(int(n), 1))

    def prepare(self, n: int, device) -> str:
        """Collective, optional: sets the peer transport up for a scene of `n` Gaussians before the first step (otherwise the
        first backward pass does it).  If any rank cannot create or map the buffers (no peer access between the GPUs, CUDA
        IPC not permitted in this environment) all ranks fall back to the "nccl" transport together.  Returns the transport."""
        import torch
        import torch.distributed as dist
        device = torch.device(device)
        if not self._use_peers(device.type == "cuda") or self._peers is not None:
            return self.transport
        index = torch.cuda.current_device() if device.index is None else device.index
        nbytes = (max(int(n), 1) + 1) * kCompactRowBytes
        peers = _PeerBuffers(index, nbytes, self.group)      # records a failure instead of raising: decided together below
        ok = torch.tensor([0 if peers.problem is not None else 1], dtype=torch.int32, device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)
        if int(ok.item()) == 0:
            problem = peers.problem
            peers.close()
            import warnings
            warnings.warn(f"htgs_b200: compact exchange falls back to the all-gather transport ({problem if problem is not None else 'another rank could not map the buffers'})")
            self.transport = "nccl"
            return self.transport
        self._peers = peers
        self._token = torch.zeros(1, dtype=torch.int32, device=device)
        return self.transport

    def buffer(self, nbytes: int, device):
        import torch
        if self.transport == "peer" and self._peers is None:
            self.prepare(int(nbytes) // kCompactRowBytes - 1, device)
        if self.transport == "peer":
            if int(nbytes) != self._peers.nbytes:
                raise RuntimeError("the scene's size changed: make a new CompactExchange (the peer buffers are sized once)")
            return _DeviceSpan(self._peers.local[self._peers.turn], nbytes)
        return torch.empty(int(nbytes), dtype=torch.uint8, device=device)

    def exchange(self, rows, capacity: int):
        """`rows`: this rank's buffer (header + capacity rows), written by the work queued on the current stream.  Returns
        (address, capacity, owner) per rank, in rank order; `owner` keeps the memory alive."""
        import torch
        import torch.distributed as dist
        world = self._world(self.group)
        self._capacity = None
        if self.transport == "peer":
            dist.all_reduce(self._token, group=self.group)      # every rank's rows are written before any rank reads them
            turn = self._peers.turn
            self._peers.turn = 1 - turn
            if world == 2 and not self.always_stage:      # one peer: the expanding kernel reads its buffer directly
                return [(self._peers.maps[turn][r], capacity, self._peers) for r in range(world)]
            # More peers: pull their buffers into local memory first, this rank starting with its right-hand neighbour, so that
            # at any time every GPU is read by ONE other GPU.  (Expanding straight from the mappings would have all ranks read
            # rank 0's buffer at once, then rank 1's, ...: the order of the sums has to be the same everywhere.)
            import ctypes
            from . import _native
            lib, rank, nbytes = _native.lib(), self._peers.rank, self._peers.nbytes
            if self._staging is None or self._staging.numel() != (world - 1) * nbytes:
                self._staging = torch.empty((world - 1) * nbytes, dtype=torch.uint8, device=self._token.device)
            stream = torch.cuda.current_stream(self._token.device).cuda_stream
            local = {rank: self._peers.maps[turn][rank]}
            for k in range(1, world):
                src = (rank + k) % world
                local[src] = self._staging.data_ptr() + (k - 1) * nbytes
                _native.check(lib.htgs_copy_rows(local[src], self._peers.maps[turn][src], int(capacity), stream))
            return [(local[r], capacity, self._staging) for r in range(world)]
        if world == 1:
            self.bytes_gathered = rows.numel()
            return [(rows.data_ptr(), capacity, rows)]
        gathered = torch.empty(world * rows.numel(), dtype=torch.uint8, device=rows.device)
        if rows.is_cuda:
            dist.all_gather_into_tensor(gathered, rows, group=self.group)
        else:          # host tensors (the gloo tests of this logic)
            dist.all_gather(list(gathered.view(world, -1).unbind(0)), rows, group=self.group)
        self.bytes_gathered = gathered.numel()
        return [(gathered.data_ptr() + r * rows.numel(), capacity, gathered) for r in range(world)]

    def published_rows(self):
        """Peer transport: the row counts in the headers of the buffers the last step used, per rank (host synchronisation;
        for reporting, not for the training loop)."""
        import ctypes
        import torch
        from . import _native
        if self._peers is None:
            return None
        torch.cuda.synchronize(self._peers.device_index)
        turn = 1 - self._peers.turn
        counts = []
        for r in range(self._peers.world):
            word = ctypes.c_uint32()
            _native.lib().htgs_memcpy_d2h(ctypes.byref(word), self._peers.maps[turn][r], 4)
            counts.append(int(word.value))
        return counts

    def close(self) -> None:
        if self._peers is not None:
            self._peers.close()
            self._peers = None
        self._staging = None


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
