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


def test_deferred_checks_two_streams_one_thread_match_blocking_calls():
    """The non-blocking path (`set_deferred_checks`: htgs_render_async, status checked when the stream is used again): one
    host thread alternates between two CUDA streams, every image and depth equals the blocking call's bit for bit, and
    `frame_results` reports every queued frame as rendered once."""
    import torch
    from htgs_b200.torch_bindings import rasterization
    ours = harness.ours()
    scene = scenes.outdoor_scene(n=200_000, n_views=10, width=640, height=400, focal=560.0)
    tensors = harness.scene_tensors(scene)
    settings = [harness.settings_for(ours, scene, v, 0, 16) for v in scene.views]
    serial = [ours.rasterize(*tensors, st, True, False) for st in settings]
    fast_serial = [ours.fast_rasterize(*tensors, st, True) for st in settings[:4]]
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    for s in streams:                       # blocking calls first: each stream's workspace grows to what these views need
        with torch.cuda.stream(s):
            for st in settings:
                ours.rasterize(*tensors, st, True, False)
    rasterization.set_deferred_checks(True)
    try:
        out = []
        for rep in range(2):
            for i, st in enumerate(settings):
                with torch.cuda.stream(streams[i % 2]):
                    out.append((i, ours.rasterize(*tensors, st, True, False)))
        infos = rasterization.frame_results()
        assert len(infos) == 2 and all(fi.reruns == 0 and fi.device_error == 0 and fi.n_instances > 0 for fi in infos)
        fast_out = []
        for i, st in enumerate(settings[:4]):
            with torch.cuda.stream(streams[i % 2]):
                fast_out.append(ours.fast_rasterize(*tensors, st, True))
        rasterization.frame_results()
    finally:
        rasterization.set_deferred_checks(False)
    torch.cuda.synchronize()
    for i, (img, depth) in out:
        assert torch.equal(img, serial[i][0]) and torch.equal(depth, serial[i][1]), f"view {i}"
    for a, b in zip(fast_out, fast_serial):
        assert (a - b).abs().max().item() < 1e-2 and (a - b).abs().mean().item() < 1e-5      # the fast path's lists are unordered: sums may differ in the last bits


def test_deferred_check_renders_an_overflowing_frame_again():
    """C-ABI: a frame queued with htgs_render_async on a fresh context whose first guess of the instance capacity is too
    small is rendered again by htgs_frame_result (info.reruns > 0) and ends up equal to the blocking render; a later call on
    the context finds nothing pending."""
    import ctypes
    import torch
    from htgs_b200 import _native
    from htgs_b200.torch_bindings import _C
    scene = scenes.tiny_scene(n=3000, size=512, seed=19)
    scene.scales *= 8.0                     # every Gaussian covers hundreds of the 4096 tiles: far more than 4 instances per Gaussian
    view = scene.views[0]
    t = [x.contiguous() for x in harness.scene_tensors(scene)]
    M, VPM, cam = (torch.from_numpy(a).cuda() for a in (view.M, view.VPM, view.cam_position))
    sc, vw = _C._scene_view(t, M, VPM, cam, 0, 16, 1, view.width, view.height, view.near_plane, view.far_plane, 1.0)
    lib = _native.lib()
    want_img = torch.empty((3, view.height, view.width), device="cuda")
    want_depth = torch.empty((view.height, view.width), device="cuda")
    fi = _native.HtgsFrameInfo()
    _native.check(lib.htgs_render(_native.context(0), ctypes.byref(sc), ctypes.byref(vw), want_img.data_ptr(), want_depth.data_ptr(), None, 1, 0, None, 0,
                                  None, ctypes.byref(fi)))
    assert fi.n_instances > (1 << 20), "the scene must need more instances than a fresh context guesses"
    ctx = lib.htgs_create(0)
    assert ctx
    try:
        img = torch.zeros_like(want_img)
        depth = torch.zeros_like(want_depth)
        stream = torch.cuda.Stream()
        _native.check(lib.htgs_render_async(ctx, ctypes.byref(sc), ctypes.byref(vw), img.data_ptr(), depth.data_ptr(), None, 1, 0, stream.cuda_stream))
        info = _native.HtgsFrameInfo()
        _native.check(lib.htgs_frame_result(ctx, ctypes.byref(info)))
        stream.synchronize()
        assert info.reruns >= 1 and info.n_instances == fi.n_instances and info.device_error == 0
        assert torch.equal(img, want_img) and torch.equal(depth, want_depth)
        again = _native.HtgsFrameInfo()
        _native.check(lib.htgs_frame_result(ctx, ctypes.byref(again)))      # nothing pending: reports the same frame
        assert again.n_instances == info.n_instances
        # the next frame on the context fits at once
        _native.check(lib.htgs_render_async(ctx, ctypes.byref(sc), ctypes.byref(vw), img.data_ptr(), depth.data_ptr(), None, 1, 0, stream.cuda_stream))
        _native.check(lib.htgs_frame_result(ctx, ctypes.byref(info)))
        assert info.reruns == 0 and torch.equal(img, want_img)
    finally:
        lib.htgs_destroy(ctypes.c_void_p(ctx))
