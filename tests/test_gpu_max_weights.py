"""GPU: update_max_weights against the golden vectors of the reference, the live reference and the CPU oracle.

The result is a maximum over pixels, independent of evaluation order, so every mode must match the reference extension bit
for bit.  HYBRID_BLEND has two behaviours.  The reference's kernel SOURCE credits `alpha * tail_weight` to every fragment in
a second walk over the tile list (hybrid_blend/kernels/update_max_weights.cuh:170-210); the EXTENSION built from it never
does (a Gaussian that only ever lands in the tail keeps weight 0): the template that picks the kernel for K is defined with
the same name and signature for HYBRID and for FIRST_K (hybrid_blend/update_max_weights.cu:15-28,
alpha_blend_first_k/update_max_weights.cu:15-28), the link keeps one definition, and HYBRID launches FIRST_K's kernel
(`oracle/umw_probe.cu` links the reference's host function alone and beside FIRST_K's, in both orders; run below).  The default of
this library reproduces the extension (bit-exact, tested against golden vectors and the live reference); with
`set_max_weights_tail_credit(True)` it does what the source describes, which is what the CPU oracle restates: then the
result is >= the extension's, equal to the oracle's, and bounded from above by the largest alpha of each Gaussian."""
import os

import numpy as np
import pytest

import harness
from htgs_b200 import scenes
from golden.make_golden import CASES, MAX_WEIGHT_THRESHOLD

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def run(mod, scene, view, mode, K, threshold, start=None, tail_credit=False):
    import torch
    from htgs_b200.torch_bindings import rasterization
    rasterization.set_max_weights_tail_credit(tail_credit)      # read by this library's binding only
    tensors = harness.scene_tensors(scene)
    st = harness.settings_for(mod, scene, view, mode, K)
    w = torch.zeros((scene.n, 1), device="cuda") if start is None else start.clone()
    try:
        mod.update_max_weights(w, *tensors[:4], st, threshold)
        torch.cuda.synchronize()
    finally:
        rasterization.set_max_weights_tail_credit(False)
    return w


def golden_cases():
    for name, case in CASES.items():
        for mode, K in case["modes"]:
            yield name, mode, K


@pytest.mark.parametrize("name,mode,K", list(golden_cases()))
def test_against_reference_golden(name, mode, K):
    gold = np.load(os.path.join(GOLDEN, f"{name}.npz"))
    key = f"m{mode}_k{K}_max_weights"
    if key not in gold.files:
        pytest.skip("golden file predates the max-weight vectors")
    scene = scenes.tiny_scene(**CASES[name]["kwargs"])
    got = run(harness.ours(), scene, scene.views[0], mode, K, MAX_WEIGHT_THRESHOLD).cpu().numpy()
    assert np.array_equal(got, gold[key])
    assert got.max() <= 1.0 and (got > 0).any()
    if mode == scenes.HYBRID_BLEND:       # what the source describes: never less, and never more than a fragment's alpha can be
        with_tail = run(harness.ours(), scene, scene.views[0], mode, K, MAX_WEIGHT_THRESHOLD, tail_credit=True).cpu().numpy()
        assert (with_tail >= got).all() and (with_tail <= np.minimum(scene.opacities.reshape(with_tail.shape), 1.0) * (1 + 1e-6)).all()


@pytest.mark.parametrize("mode,K", [(0, 4), (0, 16), (1, 4), (2, 1), (3, 1)])
def test_against_oracle(oracle_lib, mode, K):
    from htgs_b200.torch_bindings import _C
    scene = scenes.tiny_scene(n=3000, size=112, seed=61, sh_degree=0)
    view = scene.views[0]
    got = run(harness.ours(), scene, view, mode, K, 0.01, tail_credit=True).cpu().numpy().reshape(-1)      # the oracle restates the source
    info = _C.last_frame_info
    inter = harness.our_intermediates(0, scene.n, info.n_instances)
    pre = {k: inter["eval"][:, i].astype(np.float64) for i, k in enumerate(("vpmt1", "vpmt2", "vpmt4", "mt3", "rgba"))}
    pre["rgba"][:, 3] = scene.opacities.reshape(-1)      # the colour-less preprocess still stores the opacity
    want = oracle_lib.max_weights(mode, inter["ranges"], inter["prims_sorted"], pre, view, K, 0.01)
    d = np.abs(got - want)
    assert np.mean(d > 1e-5) < 2e-3 and d.max() < 0.05    # a fragment on a threshold may flip between float32 and float64


@pytest.mark.parametrize("mode,K", [(0, 16), (1, 8), (2, 1), (3, 1)])
def test_bit_exact_against_reference_extension(mode, K):
    import torch
    ref = harness.reference()
    if ref is None:
        pytest.skip("reference extension not built under baseline/_ref")
    scene = scenes.outdoor_scene(n=300_000, n_views=3, seed=51, width=800, height=450, focal=600.0)
    start = torch.rand((scene.n, 1), device="cuda") * 0.05      # in-place maximum with existing content
    for view in scene.views[:2]:
        a = run(harness.ours(), scene, view, mode, K, 0.01, start)
        b = run(ref, scene, view, mode, K, 0.01, start)
        assert torch.equal(a, b), f"{(a != b).sum().item()} of {scene.n} weights differ"
        if mode == scenes.HYBRID_BLEND:
            c = run(harness.ours(), scene, view, mode, K, 0.01, start, tail_credit=True)
            assert bool((c >= b).all()) and bool((c > b).any()), "the second walk can only raise weights, and raises some"
            ceiling = torch.maximum(start, torch.from_numpy(scene.opacities).cuda().reshape(start.shape) * (1 + 1e-6))
            assert bool((c <= ceiling).all()), "a credited weight is alpha * (a factor <= 1): never above the Gaussian's opacity"
        start = a


@pytest.mark.parametrize("K", [1, 16])
def test_hybrid_at_full_size_bit_exact_against_reference_extension(K):
    """Configuration 1's scene (3 M Gaussians, 1297x840), two views, weights accumulated over both."""
    import torch
    ref = harness.reference()
    if ref is None:
        pytest.skip("reference extension not built under baseline/_ref")
    scene = scenes.outdoor_scene(n=3_000_000, n_views=200)
    a = b = torch.zeros((scene.n, 1), device="cuda")
    for vi in (0, 100):
        a = run(harness.ours(), scene, scene.views[vi], 0, K, 0.01, a)
        b = run(ref, scene, scene.views[vi], 0, K, 0.01, b)
    assert torch.equal(a, b) and int((a > 0).sum().item()) > 1_000


def _probe(name, threshold, K):
    import subprocess
    path = os.path.join(harness.REPO, "oracle", "_ref", name)
    if not os.path.exists(path):
        pytest.skip(f"{path} not built (make -C oracle umw_probe, needs the reference's sources)")
    out = subprocess.run([path, str(threshold), str(K)], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=120)
    assert out.returncode == 0, out.stderr
    words = out.stdout.split()
    return float(words[1]), float(words[3])


@pytest.mark.parametrize("K", [1, 16])
def test_reference_host_function_linked_alone_and_beside_first_k(K):
    """Pins WHERE the reference's two behaviours come from.  `oracle/umw_probe.cu` runs the reference's own HYBRID
    `update_max_weights` host function, compiled from its sources, on a faint Gaussian (opacity 0.03: tail only) and an
    opaque one (opacity 0.9: enters the K-buffer).  Linked with HYBRID's translation unit alone the faint one gets
    alpha * tail weight, as the kernel source says.  Linked the way the extension is - FIRST_K's translation unit first - it
    keeps weight 0: both units define `update_max_weights_k_templated` (rasterization/src/hybrid_blend/update_max_weights.cu:15-28,
    rasterization/src/alpha_blend_first_k/update_max_weights.cu:15-28) with identical instantiations, the linker keeps the
    first, and HYBRID launches FIRST_K's tail-less kernel.  With the two units swapped the tail credit is back.  This library
    gives the extension's answer by default and the source's with the tail credit on, bit for bit."""
    import torch
    from htgs_b200.torch_bindings import RasterizerMode, RasterizerSettings, rasterization
    tail_alone, core_alone = _probe("umw_probe_hybrid_only", 0.01, K)
    tail_ext, core_ext = _probe("umw_probe_first_k_then_hybrid", 0.01, K)
    tail_swapped, core_swapped = _probe("umw_probe_hybrid_then_first_k", 0.01, K)
    # the same two Gaussians and camera through this library
    dev = "cuda"
    pos = torch.tensor([[-0.25, 0.0, 3.0], [0.25, 0.0, 3.0]], device=dev)
    scl = torch.full((2, 3), 0.05, device=dev)
    rot = torch.tensor([[1.0, 0.0, 0.0, 0.0]] * 2, device=dev)
    opa = torch.tensor([[0.03], [0.9]], device=dev)
    near, far, focal, centre = 0.2, 100.0, 64.0, 32.0
    zs, zo = np.float32((far + near) / (far - near)), np.float32(-2.0 * far * near / (far - near))
    VPM = torch.tensor([[focal, 0, centre - 0.5, 0], [0, focal, centre - 0.5, 0], [0, 0, zs, zo], [0, 0, 1, 0]], dtype=torch.float32, device=dev)
    st = RasterizerSettings(torch.eye(4, device=dev), VPM, torch.zeros(3, device=dev), RasterizerMode.HYBRID_BLEND, K, 1, 64, 64, near, far, 1.0)
    got = {}
    for credit in (False, True):
        w = torch.zeros((2, 1), device=dev)
        rasterization.set_max_weights_tail_credit(credit)
        try:
            harness.ours().update_max_weights(w, pos, scl, rot, opa, st, 0.01)
        finally:
            rasterization.set_max_weights_tail_credit(False)
        got[credit] = w.cpu().numpy().reshape(-1)
    print(f"K={K}: HYBRID unit alone -> tail-only {tail_alone}, core {core_alone}; FIRST_K unit linked first (as in the extension) -> "
          f"{tail_ext}, {core_ext}; HYBRID unit first -> {tail_swapped}, {core_swapped}; this library -> {got[False].tolist()} (default), "
          f"{got[True].tolist()} (tail credit)")
    assert core_alone == core_ext == core_swapped and core_alone > 0.5
    assert np.float32(core_alone) == got[False][1] == got[True][1]
    assert tail_ext == 0.0 and got[False][0] == 0.0, "linked like the extension, the tail-only Gaussian stays at 0"
    assert 0.02 < tail_alone < 0.03 and tail_alone == tail_swapped, "HYBRID's own dispatcher credits alpha * tail weight"
    assert np.float32(tail_alone) == got[True][0]
