"""GPU: update_3d_filter against the numpy restatement and, when built, the reference extension."""
import numpy as np
import pytest

import harness
from htgs_b200 import scenes

pytestmark = pytest.mark.gpu


def _inputs(n=200_000, seed=5):
    rng = np.random.default_rng(seed)
    positions = (rng.standard_normal((n, 3)) * 3.0).astype(np.float32)
    w2c = scenes.look_at((3.0, 1.0, 2.0)).astype(np.float32)
    filter_3d = np.full((n, 1), 1e5, np.float32)
    filter_3d[::3] = 0.0        # already smaller than anything a view can give: must stay untouched
    return positions, w2c, filter_3d, np.zeros(n, bool)


ARGS = dict(width=1297, height=840, focal_x=1150.0, focal_y=1100.0, center_x=640.0, center_y=425.0, near_plane=0.2, clipping_tolerance=0.15,
            distance2filter=0.0007)


def test_against_numpy_restatement(oracle_lib):
    import torch
    tb = harness.ours()
    positions, w2c, filter_3d, mask = _inputs()
    t = [torch.from_numpy(a).cuda() for a in (positions, w2c, filter_3d, mask)]
    tb.update_3d_filter(*t, *ARGS.values())
    torch.cuda.synchronize()
    want_f, want_m = oracle_lib.update_3d_filter(positions, w2c, filter_3d, mask, **ARGS)
    got_f, got_m = t[2].cpu().numpy(), t[3].cpu().numpy()
    differ = got_m != want_m          # a point exactly on a frustum plane may round differently (fused multiply-add on the GPU)
    assert differ.mean() < 1e-4
    assert np.allclose(got_f[~differ], want_f[~differ], rtol=1e-4, atol=1e-7)   # fused multiply-adds on the GPU, cancellation in the depth
    assert got_m.any() and not got_m[::3].any()


def test_bit_exact_against_reference_extension():
    import torch
    ref = harness.reference()
    if ref is None:
        pytest.skip("reference extension not built under baseline/_ref")
    positions, w2c, filter_3d, mask = _inputs(seed=6)
    ours = [torch.from_numpy(a).cuda() for a in (positions, w2c, filter_3d, mask)]
    theirs = [torch.from_numpy(a).cuda() for a in (positions, w2c, filter_3d, mask)]
    harness.ours().update_3d_filter(*ours, *ARGS.values())
    ref.update_3d_filter(*theirs, *ARGS.values())
    assert torch.equal(ours[2], theirs[2]) and torch.equal(ours[3], theirs[3])
