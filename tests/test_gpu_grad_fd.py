"""GPU: gradients of `diff_rasterize` against central finite differences of the float64 CPU oracle's forward.

An independent check of the backward pass (the other gradient tests compare with the reference's gradients): for a tiny
scene the loss L = mean |image - target| is evaluated with the oracle at theta +- h for a sample of parameter entries, and
(L+ - L-) / 2h must agree with the CUDA gradient.  The forward has thresholds (alpha cutoffs, K-buffer membership and
order), so an entry whose two one-sided differences disagree (a discontinuity inside the step) is skipped; at least
two thirds of the sampled entries must remain and agree to 2 % (plus a small absolute floor)."""
import copy

import numpy as np
import pytest

import harness
from htgs_b200 import scenes
from golden.make_golden import target_image

pytestmark = pytest.mark.gpu

PARAMS = ("positions", "scales", "rotations", "opacities", "sh_0", "sh_rest")


def oracle_loss(oracle_lib, scene, view, mode, K, target):
    img, _, _, _ = oracle_lib.render(scene, view, mode=mode, K=K, dtype=np.float64)
    return float(np.abs(img - target).mean())


@pytest.mark.parametrize("mode,K", [(0, 4), (1, 4), (2, 1), (3, 1)])
def test_gradients_against_finite_differences(oracle_lib, mode, K):
    import torch
    scene = scenes.tiny_scene(n=48, size=32, seed=77 + mode, sh_degree=1)
    scene.scales *= 2.5                       # larger footprints: every Gaussian covers many pixels
    scene.opacities[:] = np.clip(scene.opacities, 0.15, 0.85)
    view = scene.views[0]
    target = target_image(view.height, view.width, 1000 + mode).astype(np.float64) * 0.2   # keep |image - target| away from its kink
    ours = harness.ours()
    leaves = [t.clone().requires_grad_(True) for t in harness.scene_tensors(scene)]
    st = harness.settings_for(ours, scene, view, mode, K)
    image = ours.diff_rasterize(*leaves, torch.empty(0, device="cuda"), st, False)
    assert image.max().item() < 1.0           # the oracle's inference image is clamped to [0, 1]; stay below the clamp
    loss = (image - torch.from_numpy(target).float().cuda()).abs().mean()
    loss.backward()
    grads = {name: leaf.grad.cpu().numpy().astype(np.float64) for name, leaf in zip(PARAMS, leaves)}
    base = oracle_loss(oracle_lib, scene, view, mode, K, target)
    assert abs(base - loss.item()) <= 1e-5 * max(1.0, abs(base))

    rng = np.random.default_rng(5 + mode)
    checked = agreed = skipped = 0
    for name in PARAMS:
        arr = getattr(scene, name)
        if arr.size == 0:
            continue
        g = grads[name].reshape(arr.shape)
        # sample among the entries with a noticeable gradient
        flat = np.argsort(-np.abs(g).reshape(-1))[: max(8, arr.size // 8)]
        for idx in rng.choice(flat, size=min(6, flat.size), replace=False):
            ix = np.unravel_index(int(idx), arr.shape)
            h = 1e-4 * max(1.0, abs(float(arr[ix])))
            losses = []
            for sign in (+1.0, -1.0):
                s2 = copy.deepcopy(scene)
                a2 = getattr(s2, name).astype(np.float64)
                a2[ix] += sign * h
                setattr(s2, name, a2.astype(np.float32))
                step = float(getattr(s2, name)[ix]) - float(arr[ix])   # the step actually taken in float32
                losses.append((oracle_loss(oracle_lib, s2, view, mode, K, target), step))
            (lp, hp), (lm, hm) = losses
            if hp == 0.0 or hm == 0.0:
                continue
            d_plus, d_minus = (lp - base) / hp, (lm - base) / hm
            checked += 1
            if abs(d_plus - d_minus) > 0.05 * max(abs(d_plus), abs(d_minus)) + 1e-9:
                skipped += 1                  # a threshold or a change of order inside the step
                continue
            fd = (lp - lm) / (hp - hm)
            if name == "rotations":
                # the rasterizer treats the quaternion as given (no normalisation inside), so does the oracle: comparable as is
                pass
            assert abs(fd - g[ix]) <= 0.02 * abs(fd) + 2e-7, f"{name}{ix}: finite difference {fd:.6e} vs gradient {g[ix]:.6e}"
            agreed += 1
    assert checked >= 20 and agreed >= (2 * checked) // 3, (checked, agreed, skipped)
