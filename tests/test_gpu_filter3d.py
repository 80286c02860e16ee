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


@pytest.mark.parametrize("n_views", [1, 7, 48, 113])
def test_all_views_in_one_pass_equals_the_loop(n_views):
    """`update_3d_filter_views` must equal, bit for bit, one `update_3d_filter` call per view in order (and, when the reference is
    built, the reference's loop)."""
    import torch
    tb = harness.ours()
    rng = np.random.default_rng(40 + n_views)
    n = 150_000
    positions = (rng.standard_normal((n, 3)) * 3.0).astype(np.float32)
    w2cs = np.stack([scenes.look_at(p).astype(np.float32) for p in scenes.orbit_positions(n_views, 4.0, 1.5)]) if hasattr(scenes, "orbit_positions") else \
        np.stack([scenes.look_at((4.0 * np.cos(a), 1.5 + 0.3 * np.sin(3 * a), 4.0 * np.sin(a))).astype(np.float32) for a in np.linspace(0, 2 * np.pi, n_views, endpoint=False)])
    widths = [1297 - 8 * (v % 5) for v in range(n_views)]
    heights = [840 + 4 * (v % 3) for v in range(n_views)]
    fxs = [1150.0 + v for v in range(n_views)]
    fys = [1100.0 - v for v in range(n_views)]
    cxs = [640.0 + 0.5 * v for v in range(n_views)]
    cys = [425.0 - 0.25 * v for v in range(n_views)]
    nears = [0.2 + 0.01 * (v % 4) for v in range(n_views)]
    start_f = np.full((n, 1), np.finfo(np.float32).max, np.float32)
    start_f[::5] = 0.002       # a few points start below what some views would give
    pos_t = torch.from_numpy(positions).cuda()
    loop_f, loop_m = torch.from_numpy(start_f).cuda(), torch.zeros(n, dtype=torch.bool, device="cuda")
    for v in range(n_views):
        tb.update_3d_filter(pos_t, torch.from_numpy(w2cs[v]).cuda(), loop_f, loop_m, widths[v], heights[v], fxs[v], fys[v], cxs[v], cys[v], nears[v], 0.15, 0.0007)
    one_f, one_m = torch.from_numpy(start_f).cuda(), torch.zeros(n, dtype=torch.bool, device="cuda")
    tb.update_3d_filter_views(pos_t, torch.from_numpy(w2cs), one_f, one_m, widths, heights, fxs, fys, cxs, cys, nears, 0.15, 0.0007)
    torch.cuda.synchronize()
    assert torch.equal(one_f, loop_f) and torch.equal(one_m, loop_m)
    assert one_m.any() and not one_m.all()
    ref = harness.reference()
    if ref is not None:
        ref_f, ref_m = torch.from_numpy(start_f).cuda(), torch.zeros(n, dtype=torch.bool, device="cuda")
        for v in range(n_views):
            ref.update_3d_filter(pos_t, torch.from_numpy(w2cs[v]).cuda(), ref_f, ref_m, widths[v], heights[v], fxs[v], fys[v], cxs[v], cys[v], nears[v], 0.15, 0.0007)
        assert torch.equal(one_f, ref_f) and torch.equal(one_m, ref_m.reshape(-1))
