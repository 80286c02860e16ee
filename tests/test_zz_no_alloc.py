"""GPU: the allocation-free backward entry point (htgs_backward_static) against the regular one.

Some hosts cannot give the backward pass a scratch buffer because they must not allocate device memory where
the call happens (a plug-in whose host application owns all allocations, a process whose free memory belongs to
another allocator).  For them the library keeps the per-Gaussian accumulation records in a built-in array.  This
test calls both entry points through the C-ABI on the same forward state and checks that the six gradient
tensors agree, twice in a row (the built-in array keeps the previous call's contents, so the second call proves
that it is cleared), and that a scene above the built-in capacity is refused with a clear error.  The file name
sorts last so that a run stopping at the first failure has already run every other test.
"""
import ctypes

import numpy as np
import pytest

import harness
from htgs_b200 import scenes

pytestmark = pytest.mark.gpu


def _forward_state(scene, view, mode, K):
    """Runs the training forward through the C-ABI and returns everything a backward call needs."""
    import torch
    from htgs_b200 import _native
    from htgs_b200.torch_bindings import _C
    tensors = [t.contiguous() for t in harness.scene_tensors(scene)]
    M, VPM, cam = (torch.from_numpy(a).cuda() for a in (view.M, view.VPM, view.cam_position))
    image, pp, pt, pi, px, n_inst, _ = _C.forward(*tensors, M, VPM, cam, mode, K, scene.active_sh_bases, view.width, view.height,
                                                  view.near_plane, view.far_plane, 1.0)
    sc, vw = _C._scene_view(tensors, M, VPM, cam, mode, K, scene.active_sh_bases, view.width, view.height, view.near_plane, view.far_plane, 1.0)
    blobs = _native.HtgsTrainBlobs(pp.data_ptr(), pp.numel(), pt.data_ptr(), pt.numel(), pi.data_ptr(), pi.numel(), px.data_ptr(), px.numel())
    keep = (tensors, M, VPM, cam, image, pp, pt, pi, px)
    return sc, vw, blobs, n_inst, image, keep


def _run_backward(entry, sc, vw, blobs, n_inst, image, grad_image, n, total_sh, with_scratch):
    import torch
    from htgs_b200 import _native
    lib, ctx = _native.lib(), _native.context(0)
    outs = [torch.full(shape, float("nan"), device="cuda") for shape in ((n, 3), (n, 3), (n, 4), (n, 1), (n, 1, 3), (n, max(total_sh, 1), 3))]
    scratch = torch.empty(lib.htgs_backward_scratch_bytes(ctypes.byref(sc)), dtype=torch.uint8, device="cuda") if with_scratch else None
    grads = _native.HtgsGradients(*(o.data_ptr() for o in outs[:5]), outs[5].data_ptr() if total_sh else None,
                                  scratch.data_ptr() if with_scratch else None, scratch.numel() if with_scratch else 0, None, 0, 0)
    rc = getattr(lib, entry)(ctx, ctypes.byref(sc), ctypes.byref(vw), ctypes.byref(blobs), n_inst, grad_image.data_ptr(), image.data_ptr(),
                             ctypes.byref(grads), None)
    torch.cuda.synchronize()
    return rc, [o.cpu().numpy() for o in (outs if total_sh else outs[:5])]


@pytest.mark.parametrize("mode,K", [(0, 8), (2, 1)])
def test_static_scratch_backward_matches_regular_backward(mode, K):
    import torch
    from htgs_b200 import _native
    scene = scenes.tiny_scene(n=6000, size=128, seed=41, sh_degree=2)
    view = scene.views[0]
    sc, vw, blobs, n_inst, image, keep = _forward_state(scene, view, mode, K)
    total_sh = scene.sh_rest.shape[1]
    for call in range(2):   # two calls in a row: the second sees the first call's leftovers in the built-in array
        grad_image = torch.from_numpy(np.random.default_rng(100 + call).standard_normal((3, view.height, view.width)).astype(np.float32)).cuda()
        rc_ref, want = _run_backward("htgs_backward", sc, vw, blobs, n_inst, image, grad_image, scene.n, total_sh, True)
        rc_new, got = _run_backward("htgs_backward_static", sc, vw, blobs, n_inst, image, grad_image, scene.n, total_sh, False)
        assert rc_ref == _native.HTGS_OK and rc_new == _native.HTGS_OK, _native.last_error()
        for a, b in zip(got, want):
            assert np.isfinite(a).all()
            scale = max(np.abs(b).max(), 1e-20)
            assert np.abs(a - b).max() <= 1e-3 * scale     # same tolerance as the other gradient tests (float atomics reorder sums)
    del keep


def test_static_scratch_backward_rejects_scenes_above_its_capacity():
    from htgs_b200 import _native
    lib = _native.lib()
    cap = lib.htgs_backward_static_max_gaussians()
    assert cap == 131072
    sc = _native.HtgsScene(1, 1, 1, 1, 1, None, cap + 1, 0)   # never dereferenced: the size check comes first
    rc = lib.htgs_backward_static(_native.context(0), ctypes.byref(sc), None, None, 0, None, None, None, None)
    assert rc == _native.HTGS_ERR_INVALID_ARGUMENT and "131072" in _native.last_error()


def test_static_scratch_backward_leaves_free_device_memory_unchanged():
    """After one warm-up call (first launches load kernels and look up the built-in array), a call of
    htgs_backward_static must not change the amount of free device memory the driver reports: nothing is allocated or freed."""
    import torch
    from htgs_b200 import _native
    scene = scenes.tiny_scene(n=6000, size=128, seed=43, sh_degree=1)
    view = scene.views[0]
    sc, vw, blobs, n_inst, image, keep = _forward_state(scene, view, 0, 8)
    n, total_sh = scene.n, scene.sh_rest.shape[1]
    lib, ctx = _native.lib(), _native.context(0)
    grad_image = torch.ones((3, view.height, view.width), device="cuda")
    outs = [torch.empty(shape, device="cuda") for shape in ((n, 3), (n, 3), (n, 4), (n, 1), (n, 1, 3), (n, total_sh, 3))]
    grads = _native.HtgsGradients(*(o.data_ptr() for o in outs), None, 0, None, 0, 0)
    args = (ctx, ctypes.byref(sc), ctypes.byref(vw), ctypes.byref(blobs), n_inst, grad_image.data_ptr(), image.data_ptr(), ctypes.byref(grads), None)
    assert lib.htgs_backward_static(*args) == _native.HTGS_OK, _native.last_error()
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    assert lib.htgs_backward_static(*args) == _native.HTGS_OK, _native.last_error()
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    del keep
