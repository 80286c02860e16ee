"""CPU: the callers' glue around the hot path (ply files in the reference's layout, camera -> settings)."""
import os

import numpy as np
import pytest

from htgs_b200 import ply, scenes


def random_model(n, n_rest, seed=0):
    rng = np.random.default_rng(seed)
    f = np.float32
    return dict(positions=rng.standard_normal((n, 3)).astype(f), sh_0=rng.standard_normal((n, 1, 3)).astype(f),
                sh_rest=rng.standard_normal((n, n_rest, 3)).astype(f), raw_opacities=rng.standard_normal((n, 1)).astype(f),
                raw_scales=rng.standard_normal((n, 3)).astype(f), rotations=rng.standard_normal((n, 4)).astype(f))


@pytest.mark.parametrize("n,n_rest", [(0, 15), (1, 0), (257, 3), (1000, 15)])
def test_ply_round_trip(tmp_path, n, n_rest):
    m = random_model(n, n_rest, seed=n)
    path = os.path.join(tmp_path, "model.ply")
    ply.write_ply(path, **m)
    back = ply.read_ply(path)
    for k, v in m.items():
        assert back[k].shape == v.shape, k
        assert np.array_equal(back[k], v), k


def test_ply_layout_is_the_reference_layout(tmp_path):
    """Header and byte layout as Model.py:404-435 writes them: property order, SH coefficients channel-major."""
    m = random_model(3, 2, seed=5)
    path = os.path.join(tmp_path, "model.ply")
    ply.write_ply(path, **m)
    raw = open(path, "rb").read()
    header, body = raw.split(b"end_header\n")
    lines = header.decode().strip().split("\n")
    assert lines[:3] == ["ply", "format binary_little_endian 1.0", "element vertex 3"]
    assert [l.split()[2] for l in lines[3:]] == ply.property_names(2)
    rows = np.frombuffer(body, "<f4").reshape(3, -1)
    assert rows.shape[1] == 3 + 3 + 6 + 1 + 3 + 4
    assert np.array_equal(rows[:, 6:12], m["sh_rest"].transpose(0, 2, 1).reshape(3, 6))   # R of all bases, then G, then B
    assert np.array_equal(rows[:, 12], m["raw_opacities"][:, 0])


def test_ply_ascii_and_extra_properties(tmp_path):
    path = os.path.join(tmp_path, "a.ply")
    names = ["x", "y", "z", "nx", "ny", "nz"] + ply.property_names(0)[3:]
    vals = np.arange(2 * len(names), dtype=np.float64).reshape(2, len(names)) / 7.0
    with open(path, "w") as f:
        f.write("ply\nformat ascii 1.0\ncomment made by hand\nelement vertex 2\n" + "".join(f"property float {n}\n" for n in names) + "end_header\n")
        for r in vals:
            f.write(" ".join(repr(float(v)) for v in r) + "\n")
    back = ply.read_ply(path)
    assert back["sh_rest"].shape == (2, 0, 3)
    assert np.allclose(back["positions"], vals[:, :3].astype(np.float32))
    assert np.allclose(back["rotations"], vals[:, -4:].astype(np.float32))


def test_ply_errors(tmp_path):
    path = os.path.join(tmp_path, "bad.ply")
    open(path, "wb").write(b"plx\n")
    with pytest.raises(ValueError):
        ply.read_ply(path)
    m = random_model(4, 1)
    ply.write_ply(path, **m)
    raw = open(path, "rb").read()
    open(path, "wb").write(raw[:-5])
    with pytest.raises(ValueError, match="truncated"):
        ply.read_ply(path)


def test_extract_settings_matches_the_scene_generator():
    """`glue.extract_settings` and `scenes.make_view` restate the same camera contract (Renderer.py:34-57)."""
    from htgs_b200 import glue
    for k, (pos, w, h, f) in enumerate([((4.0, 1.5, 0.0), 1297, 840, 1150.0), ((0.3, -2.0, 5.0), 980, 545, 580.0), ((0.0, 0.0, -3.0), 64, 48, 60.0)]):
        w2c = scenes.look_at(pos)
        cx, cy = 0.5 * w + 0.25 * k, 0.5 * h - 0.125 * k
        v = scenes.make_view(w2c, w, h, f, f * 1.01, cx, cy, 0.2, 1000.0)
        st = glue.extract_settings(w2c, f, f * 1.01, cx, cy, w, h, 0.2, 1000.0, v.cam_position, mode=k, K=16, active_sh_bases=4, device="cpu")
        assert np.array_equal(st.M.numpy(), v.M)
        assert np.array_equal(st.VPM.numpy(), v.VPM)
        assert np.array_equal(st.cam_position.numpy(), v.cam_position)
        assert st.width == w and st.height == h and st.mode.value == k and st.K == 16 and st.active_sh_bases == 4
        assert len(st.as_tuple()) == 11
    with pytest.warns(UserWarning):
        st = glue.extract_settings(np.eye(4), 10, 10, 5, 5, 10, 10, 0.1, 10.0, [0, 0, 0], mode=7, K=4, active_sh_bases=1, device="cpu")
    assert st.mode.value == 0
