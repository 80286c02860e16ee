"""GPU: parity with the live reference extension at the benchmark configurations' stated sizes.

  configuration 2: 3,000,000 Gaussians, 1297x840, HYBRID_BLEND K=16, training forward + backward (one view)
  configuration 3: 1,500,000 Gaussians, 980x545, five mode / K variants, `rasterize` and `diff_rasterize` (two views each)
  configuration 4: 8,000,000 Gaussians, 3840x2160, HYBRID_BLEND K=32, `rasterize` (one view) - the runnable stand-in with
                   log-scale mean -5.5: with the specified -3.5 a view has about 6e9 (tile, Gaussian) instances, more than
                   the 32-bit instance counters of the reference (and of this library) hold.

Bars: images and depth of `rasterize` bit-identical; training image within 1e-5; each gradient tensor within 1e-3 of
its largest magnitude.  Gaussians the reference's HYBRID backward gives a gradient that depends on uninitialised memory
are excluded from the gradient comparison and counted: a pixel whose K-buffer entries already exhaust the transmittance
while it has no tail mass makes the reference read a tail record its forward never wrote
(hybrid_blend/kernels/forward.cuh:193, 211-212; backward.cuh:230-236).  The tests need the reference built under
baseline/_ref and are skipped without it.
"""
import numpy as np
import pytest

import harness
from htgs_b200 import scenes

pytestmark = pytest.mark.gpu

GRAD_NAMES = ("positions", "scales", "rotations", "opacities", "sh_0", "sh_rest")
GRAD_RTOL = 1e-3
IMAGE_ATOL = 1e-5

_scene_cache = {}


def cached_scene(kind):
    """One scene per configuration for the whole module (generating 3 M to 8 M Gaussians takes tens of seconds)."""
    if kind not in _scene_cache:
        _scene_cache.clear()      # keep one at a time: the 8 M scene alone holds 1.9 GB of host memory
        if kind == "config2":
            _scene_cache[kind] = scenes.outdoor_scene(n=3_000_000, n_views=200)
        elif kind == "config3":
            _scene_cache[kind] = scenes.compact_scene()
        else:
            _scene_cache[kind] = scenes.stress_scene(log_scale_mean=-5.5)
    return _scene_cache[kind]


def need_reference():
    ref = harness.reference()
    if ref is None:
        pytest.skip("reference extension not built under baseline/_ref")
    return ref


def _align256(x):
    return (x + 255) & ~255


def uninitialised_tail_readers(per_pixel, per_tile, per_instance, view, n_instances, K, n_primitives):
    """Gaussians whose HYBRID gradient in the reference depends on uninitialised memory, from this library's forward blobs
    (layout: htgs_b200/csrc/api.cu, carve_pixel_blob / carve_instance_blob): every Gaussian in the list of a tile that has
    a pixel whose stored core entries leave less than the transmittance threshold and whose tail record is empty."""
    import torch
    grid_w, grid_h = (view.width + 7) // 8, (view.height + 7) // 8
    n_tiles = grid_w * grid_h
    PP = n_tiles * 64
    off_info = _align256(4 * K * PP)
    off_tail = _align256(off_info + 16 * K * PP)
    idx_core = per_pixel[: 4 * K * PP].view(torch.int32).view(K, PP)
    info_core = per_pixel[off_info: off_info + 16 * K * PP].view(torch.float32).view(K, PP, 4)
    tail = per_pixel[off_tail: off_tail + 24 * PP].view(torch.float32).view(6, PP)
    weights = torch.where(idx_core != -1, info_core[:, :, 3], torch.zeros_like(info_core[:, :, 3])).sum(dim=0)
    exhausted = (1.0 - weights) < 1.2e-4
    no_tail = tail[3] == 0
    # pixel slots are tile-major; slots of pixels beyond the image border are never written
    slot = torch.arange(PP, device=per_pixel.device)
    tile, p = slot // 64, slot % 64
    inside = ((tile % grid_w) * 8 + p % 8 < view.width) & ((tile // grid_w) * 8 + p // 8 < view.height)
    bad = exhausted & no_tail & inside
    bad_tiles = bad.view(n_tiles, 64).any(dim=1)
    n_bad_pixels = int(bad.sum().item())
    excluded = torch.zeros(n_primitives, dtype=torch.bool, device=per_pixel.device)
    if n_bad_pixels:
        ranges = per_tile[: 8 * n_tiles].view(torch.int32).view(n_tiles, 2).long()
        key_bytes = 2 if max(n_tiles - 1, 0).bit_length() <= 16 else 4
        n_passes = (max(n_tiles - 1, 0).bit_length() + 8) // 9
        off_p0 = _align256(_align256(n_instances * key_bytes) + n_instances * key_bytes)
        off_p1 = _align256(off_p0 + 4 * n_instances)
        off = off_p1 if (n_passes & 1) else off_p0
        prims = per_instance[off: off + 4 * n_instances].view(torch.int32).long()
        for t in torch.nonzero(bad_tiles).squeeze(1).tolist():
            excluded[prims[ranges[t, 0]: ranges[t, 1]]] = True
    return excluded, n_bad_pixels


def training_step(mod, scene, tensors, view, mode, K, target, keep_blobs=False):
    import torch
    leaves = [t.detach().clone().requires_grad_(True) for t in tensors]
    st = harness.settings_for(mod, scene, view, mode, K)
    blobs = None
    if keep_blobs:
        from htgs_b200.torch_bindings import _C
        fwd = _C.forward(*tensors, *st.as_tuple())
        blobs = fwd[1:6]
    image = mod.diff_rasterize(*leaves, torch.empty(0, device="cuda"), st, False)
    loss = (image - target).abs().mean()
    loss.backward()
    torch.cuda.synchronize()
    return image.detach(), [l.grad for l in leaves], blobs


def compare_gradients(ours, ref, excluded, what):
    import torch
    keep = ~excluded if excluded is not None else None
    if keep is not None and excluded.any():       # reported, not asserted: how the excluded rows compare
        worst = max(((a[excluded] - b[excluded]).abs().max().item() / max(b.abs().max().item(), 1e-30)) for a, b in zip(ours, ref) if b.numel())
        print(f"{what}: largest error among the excluded rows {worst:.2e} of the tensor's scale")
    for name, a, b in zip(GRAD_NAMES, ours, ref):
        assert a.shape == b.shape, f"{what} grad_{name}: shape {tuple(a.shape)} vs {tuple(b.shape)}"
        if b.numel() == 0:
            continue
        if keep is not None:
            a, b = a[keep], b[keep]
        assert torch.isfinite(a).all(), f"{what} grad_{name}: non-finite values"
        scale = b.abs().max().item()
        err = (a - b).abs().max().item()
        assert scale > 0 and err <= GRAD_RTOL * scale, f"{what} grad_{name}: max error {err / max(scale, 1e-30):.2e} of the tensor's scale"


def test_config2_training_step_at_full_size():
    import torch
    ref = need_reference()
    scene = cached_scene("config2")
    tensors = harness.scene_tensors(scene)
    view = scene.views[0]
    target = torch.rand((3, view.height, view.width), generator=torch.Generator().manual_seed(1234)).cuda()
    img_o, g_o, blobs = training_step(harness.ours(), scene, tensors, view, 0, 16, target, keep_blobs=True)
    img_r, g_r, _ = training_step(ref, scene, tensors, view, 0, 16, target)
    assert (img_o - img_r).abs().max().item() <= IMAGE_ATOL
    per_primitive, per_tile, per_instance, per_pixel, n_instances = blobs
    excluded, n_bad_pixels = uninitialised_tail_readers(per_pixel, per_tile, per_instance, view, n_instances, 16, scene.n)
    print(f"config 2: {n_bad_pixels} pixels without tail mass and with an exhausted core; {int(excluded.sum().item())} of {scene.n} "
          f"Gaussians excluded from the gradient comparison; {n_instances} instances")
    assert excluded.sum().item() < 0.1 * scene.n
    compare_gradients(g_o, g_r, excluded, "config 2")
    visible = sum(int((g.reshape(scene.n, -1) != 0).any(dim=1).sum().item()) for g in g_o[:1])
    assert visible > 100_000, "the view should keep a good share of the scene"


CONFIG3_VARIANTS = [(0, 8), (0, 16), (1, 16), (2, 1), (3, 1)]


@pytest.mark.parametrize("mode,K", CONFIG3_VARIANTS)
def test_config3_rasterize_bit_exact_at_full_size(mode, K):
    import torch
    ref = need_reference()
    scene = cached_scene("config3")
    tensors = harness.scene_tensors(scene)
    for vi in (0, 57):
        view = scene.views[vi]
        median = vi != 0
        img, depth = harness.ours().rasterize(*tensors, harness.settings_for(harness.ours(), scene, view, mode, K), True, median)
        rimg, rdepth = ref.rasterize(*tensors, harness.settings_for(ref, scene, view, mode, K), True, median)
        assert torch.equal(img, rimg), f"mode {mode} K {K} view {vi}: {(img != rimg).sum().item()} image values differ"
        assert torch.equal(depth, rdepth), f"mode {mode} K {K} view {vi}: {(depth != rdepth).sum().item()} depth values differ"
        assert img.max().item() > 0.1


@pytest.mark.parametrize("mode,K", CONFIG3_VARIANTS)
def test_config3_gradients_at_full_size(mode, K):
    import torch
    ref = need_reference()
    scene = cached_scene("config3")
    tensors = harness.scene_tensors(scene)
    for vi in (0, 57):
        view = scene.views[vi]
        target = torch.rand((3, view.height, view.width), generator=torch.Generator().manual_seed(77 + vi)).cuda()
        hybrid = mode == scenes.HYBRID_BLEND
        img_o, g_o, blobs = training_step(harness.ours(), scene, tensors, view, mode, K, target, keep_blobs=hybrid)
        img_r, g_r, _ = training_step(ref, scene, tensors, view, mode, K, target)
        assert (img_o - img_r).abs().max().item() <= IMAGE_ATOL, f"mode {mode} K {K} view {vi}"
        excluded = None
        if hybrid:
            per_primitive, per_tile, per_instance, per_pixel, n_instances = blobs
            excluded, n_bad = uninitialised_tail_readers(per_pixel, per_tile, per_instance, view, n_instances, K, scene.n)
            print(f"config 3 HYBRID K={K} view {vi}: {n_bad} pixels, {int(excluded.sum().item())} Gaussians excluded")
            assert excluded.sum().item() < 0.1 * scene.n
        compare_gradients(g_o, g_r, excluded, f"config 3 mode {mode} K {K} view {vi}")


def test_config4_stand_in_bit_exact_at_full_size():
    import torch
    from htgs_b200.torch_bindings import _C
    ref = need_reference()
    scene = cached_scene("config4")
    tensors = harness.scene_tensors(scene)
    view = scene.views[5]
    img, depth = harness.ours().rasterize(*tensors, harness.settings_for(harness.ours(), scene, view, 0, 32), True, False)
    info = _C.last_frame_info
    assert info.key_bytes == 4 and info.end_bit == 17 and info.n_instances > 50_000_000
    rimg, rdepth = ref.rasterize(*tensors, harness.settings_for(ref, scene, view, 0, 32), True, False)
    assert torch.equal(img, rimg), f"{(img != rimg).sum().item()} image values differ"
    assert torch.equal(depth, rdepth), f"{(depth != rdepth).sum().item()} depth values differ"
    print(f"config 4 stand-in: {info.n_instances} instances, {info.n_visible} visible Gaussians")


def test_config4_as_specified_is_refused_not_mis_rendered():
    """With the specified log-scale mean (-3.5) a 4K view needs more (tile, Gaussian) instances than 32 bits count; the call
    must fail with a clear error instead of rendering from wrapped counters.  The stand-in scene with its scales multiplied
    by e^5 shows it cheaply (every stage after the prefix sum skips such a frame); the count of the configuration as
    specified was measured with the CPU oracle."""
    import torch
    from htgs_b200 import _native
    scene = cached_scene("config4")
    tensors = harness.scene_tensors(scene)
    big = [t.clone() for t in tensors]
    big[1] = big[1] * float(np.exp(5.0))      # log-scale mean -5.5 -> -0.5: every Gaussian that survives culling covers a large part of the 4K image
    view = scene.views[5]
    with pytest.raises(RuntimeError) as err:      # _native.HtgsError through the ctypes binding, torch's RuntimeError through the extension module
        harness.ours().rasterize(*big, harness.settings_for(harness.ours(), scene, view, 0, 32), True, False)
    assert "32 bits" in str(err.value)
    torch.cuda.synchronize()
