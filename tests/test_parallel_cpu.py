"""CPU: the multi-rank host logic (view partitioning, gradient all-reduce, max-over-ranks timing) with two
gloo ranks; plus a host-side failure case (a rank that never joins makes the collective time out with an error)."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from htgs_b200 import parallel


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def test_view_partition_is_disjoint_and_complete():
    for world in (1, 2, 4, 8):
        seen = []
        for rank in range(world):
            seen += parallel.shard_views(200, rank, world)
        assert sorted(seen) == list(range(200))
        step = [v for r in range(world) for v in parallel.step_view_indices(3, 8, r, world, 200)]
        assert len(set(step)) == 8 * world, "ranks must render different views inside a step"
    with pytest.raises(ValueError):
        parallel.shard_views(10, 2, 2)


def _worker(rank, world, port, out):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist = parallel.init_process_group("gloo")
    n = 1000
    grads = [torch.full((n, 3), float(rank + 1)), torch.full((n, 15, 3), float(10 * (rank + 1))), None]
    parallel.allreduce_gradients(grads)
    ok = bool((grads[0] == 3.0).all() and (grads[1] == 30.0).all())
    slowest = parallel.max_over_ranks(5.0 + rank)
    total = parallel.sum_over_ranks(float(len(parallel.step_view_indices(0, 8, rank, world, 200))))
    out.put((rank, ok, slowest, total))
    dist.barrier()
    dist.destroy_process_group()


def _rows_worker(rank, world, port, out):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist = parallel.init_process_group("gloo")
    n = 500
    gen = torch.Generator().manual_seed(77)             # the same draws on both ranks: every rank can rebuild the other's data
    keep = [torch.rand(n, generator=gen) < 0.2 for _ in range(world)]
    data = [[torch.randn((n, 3), generator=gen), torch.randn((n, 5, 3), generator=gen), torch.randn((n, 1), generator=gen)] for _ in range(world)]
    for r in range(world):
        for t in data[r]:
            t[~keep[r]] = 0.0                            # rows a rank's view did not keep are zero on that rank
    mine = [t.clone() for t in data[rank]] + [None]
    count = parallel.allreduce_gradients_rows(mine, keep[rank])
    expected = [sum(data[r][i] for r in range(world)) for i in range(3)]
    union = torch.stack(keep).any(0)
    ok = count == int(union.sum()) and all(torch.equal(a, b) for a, b in zip(mine[:3], expected))
    # the debug check of the exchange's assumption: true for conforming gradients, false once a row outside the union is touched
    exchange = parallel.begin_row_exchange(keep[rank])
    probe = [t.clone() for t in data[rank]]
    ok = ok and parallel.rows_outside_are_zero(probe, exchange)
    outside = torch.nonzero(~union).squeeze(1)
    if outside.numel():
        probe[0][outside[0]] = 1e-3         # what an opacity regulariser or weight decay would do
        ok = ok and not parallel.rows_outside_are_zero(probe, exchange)
    empty = parallel.allreduce_gradients_rows([torch.zeros((n, 3))], torch.zeros(n, dtype=torch.bool))
    # a union above parallel.kDenseAbove of the rows switches to the dense all-reduce: same result
    wide = torch.rand(n, generator=gen) < 0.9
    full = [torch.full((n, 2), float(r + 1)) * wide[:, None] for r in range(world)]
    mine = full[rank].clone()
    moved = parallel.allreduce_gradients_rows([mine], wide)
    ok = ok and moved == n and torch.equal(mine, sum(full))
    out.put((rank, ok, empty))
    dist.barrier()
    dist.destroy_process_group()


def _chunked_worker(rank, world, port, out):
    """BackwardExchange on host tensors: a stand-in backward pass fills the gradient rows range by range and calls
    `after_range` as the rasterizer's binding does; the result must equal the dense sum, for a sparse and a dense union."""
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist = parallel.init_process_group("gloo")
    n = 1003                                            # not a multiple of the chunk count
    gen = torch.Generator().manual_seed(5)
    ok = True
    for share in (0.2, 0.9):
        keep = [torch.rand(n, generator=gen) < share for _ in range(world)]
        data = [[torch.randn((n, 3), generator=gen), torch.randn((n, 4), generator=gen), torch.randn((n, 15, 3), generator=gen)] for _ in range(world)]
        for r in range(world):
            for t in data[r]:
                t[~keep[r]] = 0.0
        expected = [sum(data[r][k] for r in range(world)) for k in range(3)]
        xchg = parallel.BackwardExchange(n_chunks=4)
        xchg.begin(keep[rank])
        grads = [torch.zeros_like(t) for t in data[rank]]
        ranges = xchg.ranges(n, 0)
        ok = ok and len(ranges) == 4 and sum(c for _, c in ranges) == n and ranges[0][0] == 0
        for k, (first, count) in enumerate(ranges):
            for g, t in zip(grads, data[rank]):
                g[first:first + count] = t[first:first + count]         # what htgs_backward_range leaves: rows of the range are final
            xchg.after_range(k, first, count, grads)
        xchg.finish(grads)
        ok = ok and all(torch.allclose(a, b, atol=1e-6) for a, b in zip(grads, expected))
        ok = ok and xchg.dense == (share > 0.6) and xchg.rows_exchanged == (n if share > 0.6 else int(torch.stack(keep).any(0).sum()))
    one = parallel.BackwardExchange(n_chunks=4, split_pass=True).ranges(n, 2)          # GLOBAL_ORDERING: the per-pixel pass cannot be split
    ok = ok and one == [(0, n)] and len(parallel.BackwardExchange(n_chunks=4).ranges(n, 2)) == 4
    out.put((rank, ok, 0))
    dist.barrier()
    dist.destroy_process_group()


def _compact_worker(rank, world, port, out):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist = parallel.init_process_group("gloo")
    n = 5000
    gen = torch.Generator().manual_seed(91)
    keep = [torch.rand(n, generator=gen) < (0.2 + 0.3 * r) for r in range(world)]      # rank 1 keeps more than rank 0
    xchg = parallel.CompactExchange()
    xchg.begin(keep[rank])
    capacity = xchg.capacity(n)
    largest = max(int(k.sum()) for k in keep)
    ok = capacity >= largest and capacity % 1024 == 0 and capacity - largest < 1024 and xchg.rows_published == int(keep[rank].sum())
    rows = torch.full(((capacity + 1) * parallel.kCompactRowBytes,), rank + 1, dtype=torch.uint8)     # stands in for header + rows
    parts = xchg.exchange(rows, capacity)
    ok = ok and len(parts) == world and xchg.bytes_gathered == world * rows.numel()
    owner = parts[0][2]
    for r, (address, cap, keep_alive) in enumerate(parts):
        ok = ok and cap == capacity and address == owner.data_ptr() + r * rows.numel()
        ok = ok and bool((owner.view(world, -1)[r] == r + 1).all())                                 # buffers come back in rank order
    try:
        xchg.capacity(n)            # a second backward without begin() must not reuse a stale capacity
        ok = False
    except RuntimeError:
        pass
    out.put((rank, ok))
    dist.barrier()
    dist.destroy_process_group()


def test_compact_exchange_agrees_on_capacity_and_gathers_in_rank_order_two_gloo_ranks():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_compact_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(out.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert results == [(0, True), (1, True)]


def test_chunked_backward_exchange_equals_dense_sum_two_gloo_ranks():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_chunked_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = [out.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok, _ in results:
        assert ok


def test_row_exchange_equals_dense_sum_two_gloo_ranks():
    """Summing only the rows of the union of the ranks' kept Gaussians gives exactly the dense all-reduce's result."""
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rows_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = [out.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok, empty in results:
        assert ok and empty == 0


def test_allreduce_and_timing_reduction_two_gloo_ranks():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = [out.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok, slowest, total in results:
        assert ok and slowest == 6.0 and total == 16.0


def _lonely_worker(port, out):
    import datetime
    import torch.distributed as dist
    os.environ.update(RANK="0", WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    try:
        dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=3))
        out.put("joined")
    except Exception as e:   # the peer never joins: rendezvous times out on the host, nothing hangs
        out.put("error:" + type(e).__name__)


def test_missing_rank_is_reported_not_hung():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    p = ctx.Process(target=_lonely_worker, args=(_free_port(), out))
    p.start()
    msg = out.get(timeout=120)
    p.join(timeout=60)
    assert msg.startswith("error:")
