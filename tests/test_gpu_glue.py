"""GPU: fused parameter activations (`htgs_activate`, `htgs_activate_backward`) against the element-wise PyTorch
formulation of the reference's model (Model.py:45-49, 82-100), values and gradients; tolerance 2e-6 relative to each
tensor's scale (libdevice expf vs the ATen kernels)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def raw_parameters(n, seed, with_filter):
    import torch
    g = torch.Generator(device="cpu").manual_seed(seed)
    raw_scales = (torch.randn((n, 3), generator=g) - 4.0).cuda()
    raw_rotations = torch.randn((n, 4), generator=g).cuda()
    raw_opacities = (torch.randn((n, 1), generator=g) * 1.5).cuda()
    filter_3d = (torch.rand((n, 1), generator=g) * 0.02 + 1e-3).cuda() if with_filter else None
    return raw_scales, raw_rotations, raw_opacities, filter_3d


@pytest.mark.parametrize("n", [1, 255, 100_000])
@pytest.mark.parametrize("with_filter", [False, True])
def test_activation_values_and_gradients(n, with_filter):
    import torch
    from htgs_b200 import glue
    rs, rr, ro, f = raw_parameters(n, 7 + n, with_filter)
    a = [t.clone().requires_grad_(True) for t in (rs, rr, ro)]
    b = [t.clone().requires_grad_(True) for t in (rs, rr, ro)]
    out_a = glue.activate(*a, f)
    out_b = glue.reference_activate(*b, f)
    g = torch.Generator(device="cpu").manual_seed(99)
    weights = [torch.randn(o.shape, generator=g).cuda() for o in out_b]
    sum((o * w).sum() for o, w in zip(out_a, weights)).backward()
    sum((o * w).sum() for o, w in zip(out_b, weights)).backward()
    for name, x, y in zip(("scales", "rotations", "opacities"), out_a, out_b):
        scale = y.abs().max().item()
        assert (x - y).abs().max().item() <= 2e-6 * scale, name
    for name, x, y in zip(("raw_scales", "raw_rotations", "raw_opacities"), a, b):
        scale = y.grad.abs().max().item()
        assert (x.grad - y.grad).abs().max().item() <= 4e-6 * scale, f"gradient of {name}"
    assert torch.allclose(out_a[1].norm(dim=1), torch.ones(n, device="cuda"), atol=1e-6)


def test_activation_feeds_the_rasterizer():
    """raw parameters -> activate -> diff_rasterize -> loss.backward(): gradients reach the raw parameters."""
    import torch
    import harness
    from htgs_b200 import glue, scenes
    scene = scenes.tiny_scene(n=4000, size=96, seed=21, sh_degree=1)
    ours = harness.ours()
    t = harness.scene_tensors(scene)
    raw_scales = t[1].log().requires_grad_(True)
    raw_rot = (t[2] * 1.7).requires_grad_(True)
    raw_op = torch.special.logit(t[3].clamp(1e-4, 1 - 1e-4)).requires_grad_(True)
    st = harness.settings_for(ours, scene, scene.views[0], 0, 8)

    def loss_with(act):
        for p in (raw_scales, raw_rot, raw_op):
            p.grad = None
        s, r, o = act(raw_scales, raw_rot, raw_op)
        img = ours.diff_rasterize(t[0], s, r, o, t[4], t[5], torch.empty(0, device="cuda"), st, False)
        loss = img.square().mean()
        loss.backward()
        return loss.item(), [p.grad.clone() for p in (raw_scales, raw_rot, raw_op)]

    la, ga = loss_with(glue.activate)
    lb, gb = loss_with(glue.reference_activate)
    assert abs(la - lb) <= 1e-5 * abs(lb)
    for x, y in zip(ga, gb):
        assert (x - y).abs().max().item() <= 1e-3 * y.abs().max().item()
        assert y.abs().max().item() > 0


def test_activation_rejects_bad_input():
    import torch
    from htgs_b200 import glue
    rs, rr, ro, _ = raw_parameters(8, 1, False)
    with pytest.raises(ValueError):
        glue.activate(rs.double(), rr, ro)
    with pytest.raises(ValueError):
        glue.activate(rs, rr[:, :3], ro)
    with pytest.raises(ValueError):
        glue.activate(rs.cpu(), rr, ro)
