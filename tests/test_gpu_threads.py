"""GPU: the Python surface is safe to call from several host threads at once (one library context per thread, each thread on
its own CUDA stream) and concurrent frames do not disturb each other: every image equals the one rendered alone."""
import threading

import numpy as np
import pytest

import harness
from htgs_b200 import scenes

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode,K", [(0, 16), (2, 1)])
def test_concurrent_renders_match_serial(mode, K):
    import torch
    ours = harness.ours()
    scene = scenes.outdoor_scene(n=200_000, n_views=12, width=640, height=400, focal=560.0)
    tensors = harness.scene_tensors(scene)
    settings = [harness.settings_for(ours, scene, v, mode, K) for v in scene.views]
    serial = []
    for st in settings:
        img, depth = ours.rasterize(*tensors, st, True, False)
        serial.append((img.cpu().numpy(), depth.cpu().numpy()))
    results = [None] * len(settings)
    errors = []
    n_threads = 3

    def worker(k):
        try:
            torch.cuda.set_device(0)
            stream = torch.cuda.Stream()
            with torch.cuda.stream(stream):
                for rep in range(3):
                    for i in range(k, len(settings), n_threads):
                        img, depth = ours.rasterize(*tensors, settings[i], True, False)
                        stream.synchronize()
                        results[i] = (img.cpu().numpy(), depth.cpu().numpy())
        except Exception as exc:  # noqa: BLE001
            errors.append(exc)

    threads = [threading.Thread(target=worker, args=(k,)) for k in range(n_threads)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    for i, (a, b) in enumerate(zip(results, serial)):
        assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1]), f"view {i}"


def test_contexts_are_per_thread():
    from htgs_b200 import _native
    seen = {}
    together = threading.Barrier(2)   # both threads alive at once (the ident of a finished thread may be reused)

    def worker(name):
        seen[name] = _native.context(0)
        together.wait()

    threads = [threading.Thread(target=worker, args=(n,)) for n in ("a", "b")]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert seen["a"] != seen["b"] != _native.context(0)
    assert _native.context(0) == _native.context(0)


def test_front_priority_switch_leaves_results_unchanged():
    """htgs_set_front_priority only moves the front of a frame to another stream: same image and depth, bit for bit, also
    when the caller's stream has unfinished work queued ahead of the frame (the scene upload here)."""
    import torch
    from htgs_b200 import _native
    scene = scenes.tiny_scene(n=20_000, size=160, seed=12, sh_degree=2)
    view = scene.views[0]
    results = []
    ctx = _native.context(0)
    try:
        for enable in (1, 0, 1):
            _native.check(_native.lib().htgs_set_front_priority(ctx, enable))
            side = torch.cuda.Stream()
            with torch.cuda.stream(side):
                tensors = [torch.from_numpy(np.ascontiguousarray(a)).pin_memory().to("cuda", non_blocking=True) for a in scene.arrays()]
                img, depth = harness.ours().rasterize(*tensors, harness.settings_for(harness.ours(), scene, view, 0, 16), True, False)
            side.synchronize()
            results.append((img.clone(), depth.clone()))
    finally:
        _native.check(_native.lib().htgs_set_front_priority(ctx, 1))
    for img, depth in results[1:]:
        assert torch.equal(img, results[0][0]) and torch.equal(depth, results[0][1])
