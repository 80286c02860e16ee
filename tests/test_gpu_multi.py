"""GPU, two or more devices: the compact gradient exchange (htgs_b200.parallel.CompactExchange) over NCCL ranks, one process per GPU.
Skipped on a single-GPU box; the host-side logic is covered with gloo ranks in test_parallel_cpu.py."""
import os
import socket

import pytest

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, transport, out):
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, here)
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch
    import torch.distributed as dist
    import harness
    from htgs_b200 import parallel, scenes
    import htgs_b200.torch_bindings as tb
    from htgs_b200.torch_bindings import rasterization
    from golden.make_golden import target_image
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    parallel.init_process_group("nccl")
    scene = scenes.outdoor_scene(n=80_000, n_views=8, seed=57, width=480, height=270, focal=360.0)
    tensors = harness.scene_tensors(scene, device=device)
    empty = torch.empty(0, device=device)

    def step(view_index, hook):
        leaves = [t.clone().requires_grad_(True) for t in tensors]
        view = scene.views[view_index]
        st = harness.settings_for(tb, scene, view, 0, 8, device=device)
        rasterization.set_backward_hook(hook)
        image = tb.diff_rasterize(*leaves, empty, st, False)
        if hook is not None:
            visible, ready = rasterization.last_training_visibility(device, with_event=True)
            hook.begin(visible, ready)
        target = torch.from_numpy(target_image(view.height, view.width, 300 + view_index)).to(device)
        (image - target).abs().mean().backward()
        rasterization.set_backward_hook(None)
        return [l.grad for l in leaves]

    rasterization.track_training_visibility(True)
    xchg = parallel.CompactExchange(transport="peer" if transport == "peer-staged" else transport)
    xchg.always_stage = transport == "peer-staged"      # the path more than two ranks take: peers' buffers copied to local memory, then expanded
    ok, worst = True, 0.0
    for s in range(3):                                      # three steps: both buffers of the peer transport get reused
        vi = (2 * s + (8 // world) * rank) % 8
        dense = step(vi, None)
        parallel.allreduce_gradients(dense)
        compact = step(vi, xchg)
        for a, b in zip(compact, dense):                    # two passes of float atomics: equal to rounding
            err = (a - b).abs().max().item() / max(b.abs().max().item(), 1e-30)
            worst = max(worst, err)
        # every rank must hold the same bits: compare with rank 0's
        for g in compact:
            mine = g.clone()
            dist.broadcast(mine, src=0)
            ok = ok and torch.equal(mine, g)
    rasterization.track_training_visibility(False)
    counts = xchg.published_rows()
    xchg.close()
    torch.cuda.synchronize()
    out.put((rank, ok, worst, counts))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("transport", ["peer", "peer-staged", "nccl"])
def test_compact_exchange_sums_like_a_dense_allreduce_and_is_identical_on_all_ranks(transport):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    # two ranks read the one peer's buffer in place; with four, every rank pulls three peers' buffers in its own order and sums in one pass
    world = 4 if (torch.cuda.device_count() >= 4 and transport != "peer") else 2
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, transport, out)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(out.get(timeout=600) for _ in procs)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, ok, worst, counts in results:
        assert ok, f"rank {rank}: the summed gradients differ from rank 0's"
        assert worst <= 1e-5, f"rank {rank}: compact sums differ from the dense all-reduce by {worst:.2e} of a tensor's scale"
        if transport.startswith("peer"):
            assert counts is not None and len(counts) == world and all(0 < c < 80_000 for c in counts)
