"""GPU: parity of the CUDA path (called through the Python surface -> C-ABI) against
  * the golden vectors produced by the reference extension (bit-exact integers; images <= 1e-5),
  * the CPU oracle on the same seeded inputs,
  * the reference extension itself when it was built beside the repo (bit-exact everything),
plus edge cases and size-independent properties at the full benchmark size."""
import os

import numpy as np
import pytest

import harness
from htgs_b200 import scenes
from golden.make_golden import CASES

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
IMAGE_TOL = 1e-5   # max-abs tolerance for rendered RGB / depth in float32


def render_ours(scene, view, mode, K, to_chw=True, median=False, scale_modifier=1.0):
    import torch
    tb = harness.ours()
    from htgs_b200.torch_bindings import _C
    tensors = harness.scene_tensors(scene)
    st = harness.settings_for(tb, scene, view, mode, K, scale_modifier)
    img, depth = tb.rasterize(*tensors, st, to_chw, median)
    torch.cuda.synchronize()
    info = _C.last_frame_info
    assert info.device_error == 0
    return img.cpu().numpy(), depth.cpu().numpy(), info


def golden_cases():
    for name, case in CASES.items():
        for mode, K in case["modes"]:
            yield name, mode, K


@pytest.mark.parametrize("name,mode,K", list(golden_cases()))
def test_against_reference_golden(name, mode, K):
    scene = scenes.tiny_scene(**CASES[name]["kwargs"])
    view = scene.views[0]
    gold = np.load(os.path.join(GOLDEN, f"{name}.npz"))
    tag = f"m{mode}_k{K}"
    for median in (False, True):
        img, depth, info = render_ours(scene, view, mode, K, True, median)
        suffix = "_median" if median else ""
        assert np.abs(img - gold[f"{tag}_image{suffix}"]).max() <= IMAGE_TOL
        assert np.abs(depth - gold[f"{tag}_depth{suffix}"]).max() <= IMAGE_TOL
    inter = harness.our_intermediates(0, scene.n, info.n_instances)
    assert info.n_instances == gold[f"{tag}_sorted_prims"].shape[0]
    assert np.array_equal(inter["n_touched"], gold[f"{tag}_n_touched"].astype(np.uint32))
    vis = inter["n_touched"] > 0
    assert np.array_equal(inter["bounds"][vis], gold[f"{tag}_bounds"][vis])
    assert np.array_equal(inter["keys_sorted"].astype(np.uint64), gold[f"{tag}_sorted_keys"])
    assert np.array_equal(inter["prims_sorted"], gold[f"{tag}_sorted_prims"])
    assert np.array_equal(inter["ranges"], gold[f"{tag}_ranges"])


@pytest.mark.parametrize("mode,K", [(0, 16), (0, 1), (0, 2), (0, 8), (0, 32), (1, 16), (1, 2), (2, 1), (3, 1)])
def test_against_oracle(oracle_lib, mode, K):
    scene = scenes.tiny_scene(n=6000, size=160, seed=5, sh_degree=2)
    view = scene.views[0]
    img, depth, info = render_ours(scene, view, mode, K)
    inter = harness.our_intermediates(0, scene.n, info.n_instances)
    # integer stages: the oracle's binning on OUR tile boxes must give identical keys, order and ranges
    zdepth = inter["eval"][:, 3, 3] if mode == scenes.ALPHA_BLEND_GLOBAL_ORDERING else None
    ob = oracle_lib.bin_instances(inter["n_touched"], inter["bounds"].astype(np.uint32), inter["grid_w"], inter["n_tiles"], zdepth)
    assert np.array_equal(ob["sorted_keys"], inter["keys_sorted"].astype(np.uint64))
    assert np.array_equal(ob["sorted_prims"], inter["prims_sorted"])
    assert np.array_equal(ob["ranges"], inter["ranges"])
    # tile boxes vs the float32 oracle: libm logf vs CUDA logf may move an edge of very few Gaussians
    op = oracle_lib.preprocess(scene, view, mode, dtype=np.float32)
    assert np.count_nonzero(op["n_touched"] != inter["n_touched"]) <= 3
    # blend: oracle (float64 arithmetic) fed with OUR float32 records and OUR instance list
    pre = {k: inter["eval"][:, i].astype(np.float64) for i, k in enumerate(("vpmt1", "vpmt2", "vpmt4", "mt3", "rgba"))}
    o_img, o_depth, o_alpha = oracle_lib.blend(mode, inter["ranges"], inter["prims_sorted"], pre, view, K)
    d = np.abs(img - o_img)
    assert np.mean(d > IMAGE_TOL) < 1e-3 and d.max() < 2e-2      # threshold flips between float32 and float64 are rare and bounded
    dd = np.abs(depth[0] - o_depth)
    assert np.mean(dd > 1e-3) < 2e-3


def test_output_layouts_and_scale_modifier(oracle_lib):
    scene = scenes.tiny_scene(n=3000, size=100, seed=7, sh_degree=1)   # 100 is not a multiple of the tile size
    view = scene.views[0]
    chw, d_chw, _ = render_ours(scene, view, 0, 8, True)
    hwc, d_hwc, _ = render_ours(scene, view, 0, 8, False)
    assert chw.shape == (3, 100, 100) and hwc.shape == (100, 100, 3) and d_chw.shape == (1, 100, 100) and d_hwc.shape == (100, 100, 1)
    assert np.array_equal(np.transpose(chw, (1, 2, 0)), hwc) and np.array_equal(d_chw[0], d_hwc[..., 0])
    big, _, info_big = render_ours(scene, view, 0, 8, True, False, 1.7)
    o_img, _, _, o_inst = oracle_lib.render(scene, view, mode=0, K=8, scale_modifier=1.7)
    assert abs(info_big.n_instances - o_inst) <= 4
    assert np.mean(np.abs(big - o_img) > IMAGE_TOL) < 1e-3


def test_empty_and_degenerate_inputs():
    import torch
    tb = harness.ours()
    scene = scenes.tiny_scene(n=64, size=40, seed=3)
    view = scene.views[0]
    # no Gaussians at all
    empty = scenes.Scene(*(a[:0] for a in scene.arrays()), active_sh_bases=1, views=scene.views)
    img, depth, info = render_ours(empty, view, 0, 16)
    assert info.n_instances == 0 and not img.any() and not depth.any()
    # everything behind the camera -> culled
    behind = scenes.Scene(scene.positions * np.float32(-1), *scene.arrays()[1:], active_sh_bases=1, views=scene.views)
    img, depth, info = render_ours(behind, view, 2, 1)
    assert info.n_instances == 0 and info.n_visible == 0 and not img.any()
    # a single Gaussian, 1x1 tile image
    one = scenes.Scene(*(a[:1] for a in scene.arrays()), active_sh_bases=1, views=scene.views)
    one.positions[:] = (0.0, 0.0, 3.0)
    tiny_view = scenes.make_view(np.eye(4), 8, 8, 8.0, 8.0, 4.0, 4.0, 0.2, 100.0)
    for mode in (0, 1, 2, 3):
        img, depth, info = render_ours(one, tiny_view, mode, 4)
        assert info.n_instances == 1 and np.isfinite(img).all()
    # unsupported mode -> RuntimeError like the reference
    t = harness.scene_tensors(scene)
    st = harness.settings_for(tb, scene, view, 0, 16)
    from htgs_b200.torch_bindings import _C
    args = list(st.as_tuple())
    args[3] = 7
    with pytest.raises(RuntimeError):
        _C.render(*t, *args, True, False)


def test_caller_workspace_and_overflow_report():
    """C-ABI with a caller-provided workspace: too small -> error code + needed size; big enough -> same image."""
    import ctypes
    import torch
    from htgs_b200 import _native
    from htgs_b200.torch_bindings import _C
    scene = scenes.tiny_scene(n=5000, size=128, seed=9)
    view = scene.views[0]
    ref_img, _, info = render_ours(scene, view, 0, 16)
    t = [x.contiguous() for x in harness.scene_tensors(scene)]
    M, VPM, cam = (torch.from_numpy(a).cuda() for a in (view.M, view.VPM, view.cam_position))
    sc, vw = _C._scene_view(t, M, VPM, cam, 0, 16, 1, view.width, view.height, view.near_plane, view.far_plane, 1.0)
    img = torch.empty((3, view.height, view.width), device="cuda")
    depth = torch.empty((view.height, view.width), device="cuda")
    lib, ctx = _native.lib(), _native.context(0)
    fi = _native.HtgsFrameInfo()
    small = torch.empty(lib.htgs_render_workspace_bytes(ctypes.byref(sc), ctypes.byref(vw), 1000), dtype=torch.uint8, device="cuda")
    rc = lib.htgs_render(ctx, ctypes.byref(sc), ctypes.byref(vw), img.data_ptr(), depth.data_ptr(), None, 1, 0, small.data_ptr(), small.numel(), None, ctypes.byref(fi))
    assert rc == _native.HTGS_ERR_WORKSPACE_TOO_SMALL and fi.n_instances == info.n_instances and fi.workspace_bytes > small.numel()
    big = torch.empty(int(fi.workspace_bytes), dtype=torch.uint8, device="cuda")
    rc = lib.htgs_render(ctx, ctypes.byref(sc), ctypes.byref(vw), img.data_ptr(), depth.data_ptr(), None, 1, 0, big.data_ptr(), big.numel(), None, ctypes.byref(fi))
    assert rc == _native.HTGS_OK
    torch.cuda.synchronize()
    assert np.array_equal(img.cpu().numpy(), ref_img)


def test_host_buffer_entry_point():
    import ctypes
    from htgs_b200 import _native
    scene = scenes.tiny_scene(n=4000, size=96, seed=13)
    view = scene.views[0]
    ref_img, ref_depth, _ = render_ours(scene, view, 0, 16)
    arrs = [np.ascontiguousarray(a) for a in scene.arrays()]
    sc = _native.HtgsScene(*(a.ctypes.data for a in arrs[:5]), None, scene.n, 0)
    M, VPM, cam = (np.ascontiguousarray(a) for a in (view.M, view.VPM, view.cam_position))
    vw = _native.HtgsView(M.ctypes.data, VPM.ctypes.data, cam.ctypes.data, 0, 16, 1, view.width, view.height, view.near_plane, view.far_plane, 1.0)
    img = np.empty((3, view.height, view.width), np.float32)
    depth = np.empty((view.height, view.width), np.float32)
    fi = _native.HtgsFrameInfo()
    rc = _native.lib().htgs_render_host(_native.context(0), ctypes.byref(sc), ctypes.byref(vw), img.ctypes.data, depth.ctypes.data, 1, 0, ctypes.byref(fi))
    _native.check(rc)
    assert np.array_equal(img, ref_img) and np.array_equal(depth, ref_depth[0])


@pytest.mark.parametrize("mode,K", [(0, 16), (2, 1)])
def test_full_size_properties(mode, K):
    """Configuration 1 at full size (3 M Gaussians, 1297x840): properties that need no oracle."""
    scene = scenes.outdoor_scene(n=3_000_000, n_views=4)
    view = scene.views[1]
    img, depth, info = render_ours(scene, view, mode, K)
    inter = harness.our_intermediates(0, scene.n, info.n_instances)
    assert int(inter["n_touched"].astype(np.int64).sum()) == info.n_instances      # checksum of counts
    assert np.all(np.diff(inter["keys_sorted"].astype(np.int64)) >= 0)               # sortedness
    r = inter["ranges"].astype(np.int64)
    lens = r[:, 1] - r[:, 0]
    assert lens.min() >= 0 and int(lens.sum()) == info.n_instances                   # ranges partition the list
    nonempty = r[lens > 0]
    assert np.array_equal(nonempty[1:, 0], nonempty[:-1, 1]) and nonempty[0, 0] == 0
    if mode != scenes.ALPHA_BLEND_GLOBAL_ORDERING:
        # stable sort by tile only: inside a tile the Gaussian indices ascend
        same_tile = np.diff(inter["keys_sorted"].astype(np.int64)) == 0
        assert np.all(np.diff(inter["prims_sorted"].astype(np.int64))[same_tile] > 0)
    tile_of = inter["keys_sorted"].astype(np.uint64) >> np.uint64(32) if mode == scenes.ALPHA_BLEND_GLOBAL_ORDERING else inter["keys_sorted"].astype(np.uint64)
    assert np.array_equal(np.bincount(tile_of.astype(np.int64), minlength=inter["n_tiles"]), lens)
    img2, depth2, _ = render_ours(scene, view, mode, K)                             # idempotence: same bits twice
    assert np.array_equal(img, img2) and np.array_equal(depth, depth2)
    assert np.isfinite(img).all() and img.min() >= 0.0 and img.max() <= 1.0


@pytest.mark.parametrize("mode,K", [(0, 16), (1, 8), (2, 1), (3, 1)])
def test_bit_exact_against_reference_extension(mode, K):
    import torch
    ref = harness.reference()
    if ref is None:
        pytest.skip("reference extension not built under baseline/_ref")
    scene = scenes.outdoor_scene(n=400_000, n_views=3, seed=21)
    tensors = harness.scene_tensors(scene)
    for view in scene.views[:2]:
        for median in (False, True):
            img, depth = harness.ours().rasterize(*tensors, harness.settings_for(harness.ours(), scene, view, mode, K), True, median)
            rimg, rdepth = ref.rasterize(*tensors, harness.settings_for(ref, scene, view, mode, K), True, median)
            assert torch.equal(img, rimg), f"max diff {(img - rimg).abs().max().item():.3e}"
            assert torch.equal(depth, rdepth), f"max depth diff {(depth - rdepth).abs().max().item():.3e}"


@pytest.mark.parametrize("mode,K", [(0, 16), (2, 1)])
def test_benchmark_scene_bit_exact_against_reference_extension(mode, K):
    """The benchmark's own scene and orbit at full size (3 M Gaussians, 1297x840): image and depth of views spread over the
    orbit equal the reference's bit for bit, mean and median depth."""
    import torch
    ref = harness.reference()
    if ref is None:
        pytest.skip("reference extension not built under baseline/_ref")
    scene = scenes.outdoor_scene(n=3_000_000, n_views=200)
    tensors = harness.scene_tensors(scene)
    for vi in (0, 37, 74, 111, 148, 199):
        view = scene.views[vi]
        median = vi % 2 == 1
        img, depth = harness.ours().rasterize(*tensors, harness.settings_for(harness.ours(), scene, view, mode, K), True, median)
        rimg, rdepth = ref.rasterize(*tensors, harness.settings_for(ref, scene, view, mode, K), True, median)
        assert torch.equal(img, rimg) and torch.equal(depth, rdepth), f"view {vi}"


@pytest.mark.parametrize("mode,K,width,height", [(0, 32, 3840, 2160), (3, 1, 3840, 2160), (2, 1, 3000, 2400)])
def test_large_images_use_wider_sort_keys(mode, K, width, height):
    """More than 65 536 tiles (4K images with 8x8 tiles): 32-bit tile keys, 17 bits in two radix passes; GLOBAL_ORDERING with
    16x16 tiles sorts 47-bit (tile, depth) keys in six.  Lists, images and depth must still equal the reference's bit for bit."""
    import torch
    from htgs_b200.torch_bindings import _C
    ref = harness.reference()
    if ref is None:
        pytest.skip("reference extension not built under baseline/_ref")
    scene = scenes.outdoor_scene(n=150_000, n_views=2, seed=33, width=width, height=height, focal=0.9 * width)
    view = scene.views[1]
    tensors = harness.scene_tensors(scene)
    img, depth = harness.ours().rasterize(*tensors, harness.settings_for(harness.ours(), scene, view, mode, K), True, False)
    info = _C.last_frame_info
    n_tiles_8 = ((width + 7) // 8) * ((height + 7) // 8)
    assert info.key_bytes == (8 if mode == 2 else (4 if n_tiles_8 > 65536 else 2))
    rimg, rdepth = ref.rasterize(*tensors, harness.settings_for(ref, scene, view, mode, K), True, False)
    assert torch.equal(img, rimg) and torch.equal(depth, rdepth)
    # the sorted lists against the reference's scratch blobs
    from HTGSCudaBackend import _C as RC
    fwd = RC.forward(*tensors, *harness.settings_for(ref, scene, view, mode, K).as_tuple())
    torch.cuda.synchronize()
    _, pp, pt, pi, _, n_inst, sel = fwd
    assert n_inst == info.n_instances
    tw = 16 if mode == 2 else 8
    n_tiles = ((width + tw - 1) // tw) * ((height + tw - 1) // tw)
    rinst = harness.parse_ref_per_instance(pi.cpu().numpy(), n_inst, harness.sort_key_bytes(mode, n_tiles), sel)
    inter = harness.our_intermediates(0, scene.n, n_inst)
    assert np.array_equal(inter["prims_sorted"], rinst["prims_sorted"])
    assert np.array_equal(inter["keys_sorted"].astype(np.uint64), rinst["keys_sorted"].astype(np.uint64))
    assert np.array_equal(inter["ranges"], harness.parse_ref_per_tile(pt.cpu().numpy(), n_tiles))
