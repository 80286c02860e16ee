"""GPU: the compiled torch extension modules (htgs_b200/pybind: `_C`, `_C_benchmarking`).

1. Drop-in: an UNMODIFIED copy of the reference's Python surface (torch_bindings/__init__.py, rasterization.py, filter3d.py,
   taken at test time from the reference checkout under baseline/_ref) is placed in a scratch package named
   `HTGSCudaBackend` whose `_C` / `_C_benchmarking` are this library's modules, and driven in a child process
   (the real reference, imported in this process for comparison, owns the package name here).  `rasterize` must equal the
   reference bit for bit, `diff_rasterize` gradients to 1e-3, `update_max_weights` and `update_3d_filter` bit for bit,
   `fast_rasterize` within the relaxed-precision budget.
2. Both bindings of this package (extension modules, ctypes) give identical results, and their per-call host time is reported.
"""
import os
import shutil
import subprocess
import sys
import textwrap
import time

import numpy as np
import pytest

import harness
from htgs_b200 import scenes

pytestmark = pytest.mark.gpu

REF_BINDINGS = os.path.join(harness.REF_ROOT, "HTGSCudaBackend", "torch_bindings")


def extension_modules():
    try:
        from htgs_b200 import pybind
        return pybind.load()
    except ImportError:
        pytest.skip("htgs_b200/pybind modules not built (python -m htgs_b200.build)")


DRIVER = textwrap.dedent('''
    import sys
    import numpy as np, torch
    sys.path.insert(0, sys.argv[1]); sys.path.insert(0, sys.argv[2]); sys.path.insert(0, sys.argv[2] + "/tests")
    import HTGSCudaBackend
    from HTGSCudaBackend.torch_bindings import (diff_rasterize, rasterize, fast_rasterize, update_max_weights, update_3d_filter,
                                                RasterizerSettings, RasterizerMode)
    from HTGSCudaBackend import _C
    assert "htgs_b200" not in (_C.__file__ or "") and HTGSCudaBackend.__file__.startswith(sys.argv[1])
    import harness
    from htgs_b200 import scenes
    import HTGSCudaBackend.torch_bindings as tb
    scene = scenes.outdoor_scene(n=120_000, n_views=3, seed=71, width=500, height=300, focal=420.0)
    tensors = harness.scene_tensors(scene)
    out = {}
    for mode, K in ((0, 16), (1, 8), (2, 1), (3, 1)):
        view = scene.views[mode % 3]
        st = harness.settings_for(tb, scene, view, mode, K)
        img, depth = rasterize(*tensors, st, True, mode == 1)
        out[f"img{mode}"], out[f"depth{mode}"] = img.cpu().numpy(), depth.cpu().numpy()
        leaves = [t.clone().requires_grad_(True) for t in tensors]
        image = diff_rasterize(*leaves, torch.empty(0, device="cuda"), st, False)
        target = torch.rand(image.shape, generator=torch.Generator().manual_seed(5 + mode)).cuda()
        (image - target).abs().mean().backward()
        out[f"train{mode}"] = image.detach().cpu().numpy()
        for k, l in enumerate(leaves):
            out[f"grad{mode}_{k}"] = l.grad.cpu().numpy()
        w = torch.zeros((scene.n, 1), device="cuda")
        update_max_weights(w, *tensors[:4], st, 0.01)
        out[f"weights{mode}"] = w.cpu().numpy()
        if mode != 2:
            out[f"fast{mode}"] = fast_rasterize(*tensors, st, False).cpu().numpy()
    view = scene.views[0]
    f3 = torch.full((scene.n, 1), 1e6, device="cuda")
    mask = torch.zeros(scene.n, dtype=torch.bool, device="cuda")
    update_3d_filter(tensors[0], torch.from_numpy(view.M).cuda(), f3, mask, view.width, view.height, 420.0, 420.0, 250.0, 150.0, 0.2, 0.15, 0.2)
    out["filter"], out["mask"] = f3.cpu().numpy(), mask.cpu().numpy()
    bad = list(st.as_tuple())
    bad[3] = 7                       # not a RasterizerMode: the reference throws "unsupported rasterizer mode"
    try:
        _C.render(*tensors, *bad, True, False)
        out["error"] = np.array(0)
    except RuntimeError as exc:
        out["error"] = np.array(1 if "unsupported rasterizer mode" in str(exc) else 2)
    np.savez(sys.argv[3], **out)
''')


def test_unmodified_reference_surface_runs_on_the_extension_modules(tmp_path):
    import torch
    ref = harness.reference()
    if ref is None or not os.path.isdir(REF_BINDINGS):
        pytest.skip("reference checkout not present under baseline/_ref")
    mod_c, mod_b = extension_modules()
    pkg = tmp_path / "site" / "HTGSCudaBackend"
    (pkg / "torch_bindings").mkdir(parents=True)
    (pkg / "__init__.py").write_text("")
    for name in ("__init__.py", "rasterization.py", "filter3d.py"):
        shutil.copyfile(os.path.join(REF_BINDINGS, name), pkg / "torch_bindings" / name)      # byte for byte the reference's files
    shutil.copyfile(mod_c.__file__, pkg / os.path.basename(mod_c.__file__))
    shutil.copyfile(mod_b.__file__, pkg / os.path.basename(mod_b.__file__))
    driver = tmp_path / "driver.py"
    driver.write_text(DRIVER)
    result = tmp_path / "out.npz"
    env = dict(os.environ)
    env["LD_LIBRARY_PATH"] = os.path.join(harness.REPO, "htgs_b200") + os.pathsep + env.get("LD_LIBRARY_PATH", "")
    env["HTGS_B200_BINDING"] = "ctypes"      # the child uses htgs_b200 only for scenes / harness helpers
    proc = subprocess.run([sys.executable, str(driver), str(tmp_path / "site"), harness.REPO, str(result)], env=env, stdout=subprocess.PIPE,
                          stderr=subprocess.STDOUT, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-3000:]
    got = np.load(result)
    assert int(got["error"]) == 1, "an invalid mode must raise the reference's RuntimeError through the extension module"

    scene = scenes.outdoor_scene(n=120_000, n_views=3, seed=71, width=500, height=300, focal=420.0)
    tensors = harness.scene_tensors(scene)
    for mode, K in ((0, 16), (1, 8), (2, 1), (3, 1)):
        view = scene.views[mode % 3]
        st = harness.settings_for(ref, scene, view, mode, K)
        img, depth = ref.rasterize(*tensors, st, True, mode == 1)
        assert np.array_equal(got[f"img{mode}"], img.cpu().numpy()) and np.array_equal(got[f"depth{mode}"], depth.cpu().numpy()), f"mode {mode}"
        leaves = [t.clone().requires_grad_(True) for t in tensors]
        image = ref.diff_rasterize(*leaves, torch.empty(0, device="cuda"), st, False)
        target = torch.rand(image.shape, generator=torch.Generator().manual_seed(5 + mode)).cuda()
        (image - target).abs().mean().backward()
        assert np.abs(got[f"train{mode}"] - image.detach().cpu().numpy()).max() <= 1e-5
        for k, l in enumerate(leaves):
            want = l.grad.cpu().numpy()
            assert np.abs(got[f"grad{mode}_{k}"] - want).max() <= 1e-3 * max(np.abs(want).max(), 1e-30), f"mode {mode} gradient {k}"
        w = torch.zeros((scene.n, 1), device="cuda")
        ref.update_max_weights(w, *tensors[:4], st, 0.01)
        assert np.array_equal(got[f"weights{mode}"], w.cpu().numpy()), f"mode {mode} max weights"
        if mode != 2:
            fast = ref.fast_rasterize(*tensors, st, False).cpu().numpy()
            d = np.abs(got[f"fast{mode}"] - fast)
            assert d.mean() < 1e-5 and np.mean(d > 1e-3) < 2e-4 and d.max() < 0.1
    view = scene.views[0]
    f3 = torch.full((scene.n, 1), 1e6, device="cuda")
    mask = torch.zeros(scene.n, dtype=torch.bool, device="cuda")
    from HTGSCudaBackend.torch_bindings import update_3d_filter as ref_filter
    ref_filter(tensors[0], torch.from_numpy(view.M).cuda(), f3, mask, view.width, view.height, 420.0, 420.0, 250.0, 150.0, 0.2, 0.15, 0.2)
    assert np.array_equal(got["filter"], f3.cpu().numpy()) and np.array_equal(got["mask"], mask.cpu().numpy())


def test_both_bindings_agree_and_host_time_per_call():
    """Configuration 0 (16,384 Gaussians, 256x256): the frame is tens of microseconds of GPU work, so the binding's host
    time is what a caller sees.  Both bindings must return identical tensors; their host time per call is printed."""
    import torch
    mod_c, _ = extension_modules()
    from htgs_b200.torch_bindings import _C as ctypes_c
    import htgs_b200.torch_bindings as tb
    scene = scenes.tiny_scene()
    tensors = harness.scene_tensors(scene)
    st = harness.settings_for(tb, scene, scene.views[0], 0, 16)
    args = (*tensors, *st.as_tuple(), True, False)
    a_img, a_depth = mod_c.render(*args)
    b_img, b_depth = ctypes_c.render(*args)
    assert torch.equal(a_img, b_img) and torch.equal(a_depth, b_depth)
    fa = mod_c.forward(*tensors, *st.as_tuple())
    fb = ctypes_c.forward(*tensors, *st.as_tuple())
    assert torch.equal(fa[0], fb[0]) and fa[5] == fb[5]
    grad = torch.ones_like(fa[0])
    empty = torch.empty(0, device="cuda")
    ga = mod_c.backward(empty, grad, empty, *tensors[:3], empty, tensors[5], *fa[1:5], *st.as_tuple(), fa[5], fa[6], False)
    gb = ctypes_c.backward(empty, grad, empty, *tensors[:3], empty, tensors[5], *fb[1:5], *st.as_tuple(), fb[5], fb[6], False)
    for x, y in zip(ga, gb):
        assert x.shape == y.shape
        if y.numel():
            assert (x - y).abs().max().item() <= 1e-5 * max(y.abs().max().item(), 1e-30)
    times = {}
    for name, fn in (("extension module", mod_c.render), ("ctypes", ctypes_c.render)):
        for _ in range(20):
            fn(*args)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(300):
            fn(*args)
        torch.cuda.synchronize()
        times[name] = (time.perf_counter() - t0) / 300 * 1e6
    print(f"configuration 0, `_C.render` wall time per call: " + ", ".join(f"{k} {v:.0f} us" for k, v in times.items()))
    assert times["extension module"] < 5000 and times["ctypes"] < 5000


def test_surface_reports_its_binding():
    from htgs_b200 import _native
    from htgs_b200.torch_bindings import rasterization
    assert rasterization.binding() == _native.active_binding()
    assert rasterization.binding() in ("pybind", "ctypes")
