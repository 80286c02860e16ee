"""Seeded synthetic scenes and the camera contract of the rasterizer.

The public datasets the reference is normally evaluated on are not available
offline, so every workload is a seeded synthetic stand-in with the shapes,
sizes and value distributions of the benchmark configurations.  Everything is
generated on the host with numpy (PCG64) so that the CUDA path, the CPU oracle
and the reference extension all receive identical bits.

The camera matrices follow the reference renderer's `extract_settings`
(Renderer.py:34-57): pixel centres sit at integer coordinates, the camera
looks along +z, and `VPM = VP @ w2c`.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List

import numpy as np

# RasterizerMode values (torch_bindings/rasterization.py:9-13)
HYBRID_BLEND, ALPHA_BLEND_FIRST_K, ALPHA_BLEND_GLOBAL_ORDERING, OIT_BLEND = 0, 1, 2, 3


@dataclass
class View:
    """One camera: float32 matrices exactly as the rasterizer receives them."""
    M: np.ndarray             # [4,4] world -> view
    VPM: np.ndarray           # [4,4] world -> screen (homogeneous)
    cam_position: np.ndarray  # [3]
    width: int
    height: int
    near_plane: float
    far_plane: float


@dataclass
class Scene:
    positions: np.ndarray   # [N,3]
    scales: np.ndarray      # [N,3] activated (exp of the log-scales)
    rotations: np.ndarray   # [N,4] (r,x,y,z), unit length
    opacities: np.ndarray   # [N,1] activated (sigmoid of the logits)
    sh_0: np.ndarray        # [N,1,3]
    sh_rest: np.ndarray     # [N,B,3]
    active_sh_bases: int
    views: List[View] = field(default_factory=list)
    name: str = ""
    mode: int = HYBRID_BLEND
    K: int = 16

    @property
    def n(self) -> int:
        return int(self.positions.shape[0])

    def arrays(self):
        return (self.positions, self.scales, self.rotations, self.opacities, self.sh_0, self.sh_rest)


def make_view(w2c: np.ndarray, width: int, height: int, fx: float, fy: float, cx: float, cy: float,
              near_plane: float, far_plane: float) -> View:
    """Camera matrices as in Renderer.py:34-57 (evaluated in float64, then cast)."""
    w2c = np.asarray(w2c, dtype=np.float64)
    z_range = far_plane - near_plane
    VP = np.array([
        [fx, 0.0, cx - 0.5, 0.0],
        [0.0, fy, cy - 0.5, 0.0],
        [0.0, 0.0, (far_plane + near_plane) / z_range, -2.0 * far_plane * near_plane / z_range],
        [0.0, 0.0, 1.0, 0.0],
    ], dtype=np.float64)
    VPM = VP @ w2c
    cam_position = -w2c[:3, :3].T @ w2c[:3, 3]
    return View(M=np.ascontiguousarray(w2c, dtype=np.float32), VPM=np.ascontiguousarray(VPM, dtype=np.float32),
                cam_position=np.ascontiguousarray(cam_position, dtype=np.float32), width=int(width), height=int(height),
                near_plane=float(near_plane), far_plane=float(far_plane))


def look_at(position, target=(0.0, 0.0, 0.0), up=(0.0, 1.0, 0.0)) -> np.ndarray:
    """World -> view matrix of a camera at `position` looking at `target` (+z forward, +x right, +y down)."""
    position = np.asarray(position, dtype=np.float64)
    forward = np.asarray(target, dtype=np.float64) - position
    forward /= np.linalg.norm(forward)
    right = np.cross(forward, np.asarray(up, dtype=np.float64))
    right /= np.linalg.norm(right)
    down = np.cross(forward, right)
    rot = np.stack([right, down, forward])
    w2c = np.eye(4)
    w2c[:3, :3] = rot
    w2c[:3, 3] = -rot @ position
    return w2c


def orbit_views(n_views: int, radius: float, height: float, width: int, img_height: int, focal: float,
                near_plane: float = 0.2, far_plane: float = 1000.0) -> List[View]:
    views = []
    for i in range(n_views):
        phi = 2.0 * np.pi * i / n_views
        pos = (radius * np.cos(phi), height, radius * np.sin(phi))
        views.append(make_view(look_at(pos), width, img_height, focal, focal, width / 2.0, img_height / 2.0, near_plane, far_plane))
    return views


def _unit_quaternions(rng, n):
    q = rng.standard_normal((n, 4))
    q /= np.linalg.norm(q, axis=1, keepdims=True)
    return q.astype(np.float32)


def _sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def _mixture_positions(rng, n, n_components, ball_radius, sigma_lo=0.3, sigma_hi=2.0):
    direction = rng.standard_normal((n_components, 3))
    direction /= np.linalg.norm(direction, axis=1, keepdims=True)
    centres = direction * (ball_radius * rng.random((n_components, 1)) ** (1.0 / 3.0))
    sigma = rng.uniform(sigma_lo, sigma_hi, size=(n_components, 1))
    comp = rng.integers(0, n_components, size=n)
    return centres[comp] + sigma[comp] * rng.standard_normal((n, 3))


def _sh(rng, n, degree):
    sh_0 = (0.3 * rng.standard_normal((n, 1, 3))).astype(np.float32)
    n_rest = (degree + 1) ** 2 - 1
    sh_rest = (0.05 * rng.standard_normal((n, n_rest, 3))).astype(np.float32)
    return sh_0, sh_rest


def tiny_scene(n: int = 16384, size: int = 256, seed: int = 0, mode: int = HYBRID_BLEND, K: int = 16, sh_degree: int = 0) -> Scene:
    """Configuration 0: camera-space cloud in front of one pinhole camera (M = identity)."""
    rng = np.random.default_rng(seed)
    pos = np.empty((n, 3))
    pos[:, :2] = rng.uniform(-1.0, 1.0, size=(n, 2))
    pos[:, 2] = rng.uniform(2.0, 6.0, size=n)
    scales = np.exp(-3.0 + 0.5 * rng.standard_normal((n, 3)))
    rot = _unit_quaternions(rng, n)
    opac = _sigmoid(rng.standard_normal((n, 1)))
    sh_0, sh_rest = _sh(rng, n, sh_degree)
    view = make_view(np.eye(4), size, size, float(size), float(size), size / 2.0, size / 2.0, 0.2, 100.0)
    return Scene(pos.astype(np.float32), scales.astype(np.float32), rot, opac.astype(np.float32), sh_0, sh_rest,
                 active_sh_bases=(sh_degree + 1) ** 2, views=[view], name=f"tiny_n{n}_{size}px", mode=mode, K=K)


def outdoor_scene(n: int = 3_000_000, n_views: int = 200, seed: int = 1, width: int = 1297, height: int = 840,
                  focal: float = 1150.0, n_components: int = 64, ball_radius: float = 10.0, log_scale_mean: float = -4.5,
                  mode: int = HYBRID_BLEND, K: int = 16, name: str = "outdoor") -> Scene:
    """Configuration 1 (and 2): Gaussian-mixture scene seen from an orbit of radius 4 at height 1.5."""
    rng = np.random.default_rng(seed)
    pos = _mixture_positions(rng, n, n_components, ball_radius)
    scales = np.exp(log_scale_mean + rng.standard_normal((n, 3)))
    rot = _unit_quaternions(rng, n)
    opac = _sigmoid(1.5 * rng.standard_normal((n, 1)))
    sh_0, sh_rest = _sh(rng, n, 3)
    views = orbit_views(n_views, 4.0, 1.5, width, height, focal)
    return Scene(pos.astype(np.float32), scales.astype(np.float32), rot, opac.astype(np.float32), sh_0, sh_rest,
                 active_sh_bases=16, views=views, name=f"{name}_n{n}_{width}x{height}", mode=mode, K=K)


def compact_scene(n: int = 1_500_000, n_views: int = 100, seed: int = 3, mode: int = HYBRID_BLEND, K: int = 16) -> Scene:
    """Configuration 3: 32 mixture components in a radius-6 ball, 980x545, focal 580."""
    return outdoor_scene(n=n, n_views=n_views, seed=seed, width=980, height=545, focal=580.0, n_components=32,
                         ball_radius=6.0, mode=mode, K=K, name="compact")


def stress_scene(n: int = 8_000_000, n_views: int = 64, seed: int = 4, width: int = 3840, height: int = 2160,
                 focal: float = 3000.0, K: int = 32, log_scale_mean: float = -3.5) -> Scene:
    """Configuration 4: half of the Gaussians as in configuration 1, half in dense clusters (sigma 0.5).

    "A cluster 1.5 units in front of every camera" is realised as a ring of clusters: camera i of the orbit gets
    its own cluster centred 1.5 units along its viewing direction, and the dense half is split evenly over them.

    With the specified log-scales ~N(-3.5, 1) one 4K view has about 6e9 (tile, Gaussian) instances (measured with the
    CPU oracle), which exceeds the 32-bit instance counters of the reference (and of this library, which reports it as
    an error); `log_scale_mean=-5.5` is the variant that both implementations can run (about 1e8 instances per view).
    """
    rng = np.random.default_rng(seed)
    n_dense = n // 2
    pos_bg = _mixture_positions(rng, n - n_dense, 64, 10.0)
    views = orbit_views(n_views, 4.0, 1.5, width, height, focal)
    centres = np.stack([v.cam_position.astype(np.float64) + 1.5 * v.M[2, :3].astype(np.float64) for v in views])
    which = rng.integers(0, n_views, size=n_dense)
    pos_dense = centres[which] + 0.5 * rng.standard_normal((n_dense, 3))
    pos = np.concatenate([pos_dense, pos_bg])
    pos = pos[rng.permutation(n)]
    scales = np.exp(log_scale_mean + rng.standard_normal((n, 3)))
    rot = _unit_quaternions(rng, n)
    opac = _sigmoid(1.5 * rng.standard_normal((n, 1)))
    sh_0, sh_rest = _sh(rng, n, 3)
    return Scene(pos.astype(np.float32), scales.astype(np.float32), rot, opac.astype(np.float32), sh_0, sh_rest,
                 active_sh_bases=16, views=views, name=f"stress_n{n}_{width}x{height}", mode=HYBRID_BLEND, K=K)
