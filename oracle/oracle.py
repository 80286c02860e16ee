"""ctypes wrapper around the CPU oracle (libhtgs_oracle.so).  TEST INFRASTRUCTURE ONLY.

Only tests/, the smoke entry and the CPU-baseline legs of bench.py may import this
module.  The product path (htgs_b200) never does.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Optional

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libhtgs_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside this file."""
    src = os.path.join(_HERE, "htgs_oracle.cpp")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libhtgs_oracle.so"])
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.htgs_oracle_bin.restype = ctypes.c_int64
        _lib.htgs_oracle_render_f32.restype = ctypes.c_int64
        _lib.htgs_oracle_render_f64.restype = ctypes.c_int64
    return _lib


def hardware_threads() -> int:
    return int(lib().htgs_oracle_hardware_threads())


def tile_size(mode: int):
    w, h = ctypes.c_int(), ctypes.c_int()
    lib().htgs_oracle_tile_size(int(mode), ctypes.byref(w), ctypes.byref(h))
    return w.value, h.value


def _p(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _scene_ptrs(scene, view):
    arrs = [_f32(a) for a in scene.arrays()] + [_f32(view.M), _f32(view.VPM), _f32(view.cam_position)]
    return arrs, [_p(a) for a in arrs]


def grid_of(view, mode):
    tw, th = tile_size(mode)
    return (view.width + tw - 1) // tw, (view.height + th - 1) // th


def preprocess(scene, view, mode: int, scale_modifier: float = 1.0, dtype=np.float64, with_clamp: bool = False, n_threads: int = 0):
    """Per-Gaussian stage.  Returns a dict of arrays (rows of culled Gaussians are zero)."""
    n = scene.n
    keep, ptrs = _scene_ptrs(scene, view)
    out = {
        "n_touched": np.zeros(n, np.uint32), "bounds": np.zeros((n, 4), np.uint32),
        "vpmt1": np.zeros((n, 4), dtype), "vpmt2": np.zeros((n, 4), dtype), "vpmt4": np.zeros((n, 4), dtype),
        "mt3": np.zeros((n, 4), dtype), "rgba": np.zeros((n, 4), dtype),
        "clamp": np.zeros((3, n), np.uint8) if with_clamp else None,
    }
    fn = lib().htgs_oracle_preprocess_f64 if dtype == np.float64 else lib().htgs_oracle_preprocess_f32
    fn(*ptrs, ctypes.c_int64(n), int(mode), int(scene.active_sh_bases), int(scene.sh_rest.shape[1]), int(view.width), int(view.height),
       ctypes.c_float(view.near_plane), ctypes.c_float(view.far_plane), ctypes.c_float(scale_modifier),
       _p(out["n_touched"]), _p(out["bounds"]), _p(out["vpmt1"]), _p(out["vpmt2"]), _p(out["vpmt4"]), _p(out["mt3"]), _p(out["rgba"]),
       _p(out["clamp"]), int(n_threads or hardware_threads()))
    del keep
    return out


def bin_instances(n_touched, bounds, grid_w: int, n_tiles: int, depth: Optional[np.ndarray] = None):
    """Instance emission, stable sort and per-tile ranges from per-Gaussian tile boxes.

    `depth` (float32 view depth per Gaussian) switches to the 64-bit (tile, depth) keys of
    ALPHA_BLEND_GLOBAL_ORDERING.  Returns keys/prims in emission order, sorted keys/prims and ranges.
    """
    n_touched = np.ascontiguousarray(n_touched, np.uint32)
    bounds = np.ascontiguousarray(bounds, np.uint32)
    depth = None if depth is None else _f32(depth)
    n = n_touched.shape[0]
    total = int(lib().htgs_oracle_bin(_p(n_touched), _p(bounds), _p(depth), ctypes.c_int64(n), int(grid_w), int(n_tiles), None, None, None, None, None))
    out = {"keys": np.zeros(total, np.uint64), "prims": np.zeros(total, np.uint32), "sorted_keys": np.zeros(total, np.uint64),
           "sorted_prims": np.zeros(total, np.uint32), "ranges": np.zeros((n_tiles, 2), np.uint32)}
    # zero-length arrays still need a valid pointer for the "not a size query" test
    sp = out["sorted_prims"] if total > 0 else np.zeros(1, np.uint32)
    lib().htgs_oracle_bin(_p(n_touched), _p(bounds), _p(depth), ctypes.c_int64(n), int(grid_w), int(n_tiles), _p(out["keys"]), _p(out["prims"]),
                          _p(out["sorted_keys"]), _p(sp), _p(out["ranges"]))
    return out


def blend(mode: int, ranges, prim_idx, pre: dict, view, K: int, use_median_depth: bool = False, to_chw: bool = True, n_threads: int = 0):
    """Per-tile blend from preprocess outputs and a sorted instance list."""
    dtype = pre["vpmt1"].dtype
    h, w = view.height, view.width
    image = np.zeros((3, h, w) if to_chw else (h, w, 3), dtype)
    depth = np.zeros((h, w), dtype)
    alpha = np.zeros((h, w), dtype)
    ranges = np.ascontiguousarray(ranges, np.uint32)
    prim_idx = np.ascontiguousarray(prim_idx, np.uint32)
    fn = lib().htgs_oracle_blend_f64 if dtype == np.float64 else lib().htgs_oracle_blend_f32
    fn(int(mode), _p(ranges), _p(prim_idx), _p(pre["vpmt1"]), _p(pre["vpmt2"]), _p(pre["vpmt4"]), _p(pre["mt3"]), _p(pre["rgba"]),
       int(w), int(h), int(K), int(use_median_depth), int(to_chw), _p(image), _p(depth), _p(alpha), int(n_threads or hardware_threads()))
    return image, depth, alpha


def max_weights(mode: int, ranges, prim_idx, pre: dict, view, K: int, weight_threshold: float, start=None, hybrid_tail_credit: bool = True):
    """update_max_weights from preprocess outputs and a sorted instance list (sequential; small cases only).
    `hybrid_tail_credit`: HYBRID_BLEND as the reference's kernel source describes it (True) or as the reference extension
    computes it (False: core weights only, see htgs_oracle.cpp)."""
    dtype = pre["vpmt1"].dtype
    n = pre["vpmt1"].shape[0]
    out = np.zeros(n, dtype) if start is None else np.ascontiguousarray(start, dtype).reshape(-1).copy()
    ranges = np.ascontiguousarray(ranges, np.uint32)
    prim_idx = np.ascontiguousarray(prim_idx, np.uint32)
    thr = ctypes.c_double(weight_threshold) if dtype == np.float64 else ctypes.c_float(weight_threshold)
    fn = lib().htgs_oracle_max_weights_f64 if dtype == np.float64 else lib().htgs_oracle_max_weights_f32
    fn(int(mode), _p(ranges), _p(prim_idx), _p(pre["vpmt1"]), _p(pre["vpmt2"]), _p(pre["vpmt4"]), _p(pre["mt3"]), _p(pre["rgba"]),
       int(view.width), int(view.height), int(K), thr, _p(out), int(bool(hybrid_tail_credit)))
    return out


def render(scene, view, mode: Optional[int] = None, K: Optional[int] = None, scale_modifier: float = 1.0, to_chw: bool = True,
           use_median_depth: bool = False, dtype=np.float64, n_threads: int = 0):
    """Whole forward (the `rasterize` path).  Returns image, depth, alpha, n_instances."""
    mode = scene.mode if mode is None else mode
    K = scene.K if K is None else K
    keep, ptrs = _scene_ptrs(scene, view)
    h, w = view.height, view.width
    image = np.zeros((3, h, w) if to_chw else (h, w, 3), dtype)
    depth = np.zeros((h, w), dtype)
    alpha = np.zeros((h, w), dtype)
    fn = lib().htgs_oracle_render_f64 if dtype == np.float64 else lib().htgs_oracle_render_f32
    n_inst = fn(*ptrs, ctypes.c_int64(scene.n), int(mode), int(K), int(scene.active_sh_bases), int(scene.sh_rest.shape[1]), int(w), int(h),
                ctypes.c_float(view.near_plane), ctypes.c_float(view.far_plane), ctypes.c_float(scale_modifier), int(to_chw),
                int(use_median_depth), _p(image), _p(depth), _p(alpha), int(n_threads or hardware_threads()))
    del keep
    return image, depth, alpha, int(n_inst)


def update_3d_filter(positions, w2c, filter_3d, visibility_mask, width, height, focal_x, focal_y, center_x, center_y, near_plane,
                     clipping_tolerance, distance2filter):
    """numpy restatement of the 3D-filter update (filter3d/src/filter3d_kernels.cu:6-35, filter3d/src/filter3d_api.cu:23-33).
    Returns new (filter_3d, visibility_mask); float32 arithmetic in the reference's order."""
    f32 = np.float32
    p = np.asarray(positions, f32)
    w = np.asarray(w2c, f32).reshape(4, 4)
    bounds = f32(clipping_tolerance) + f32(0.5)
    mx, my = bounds * f32(width), bounds * f32(height)
    ox, oy = f32(center_x) - f32(0.5) * f32(width), f32(center_y) - f32(0.5) * f32(height)
    left, right = (-mx - ox) / f32(focal_x), (mx - ox) / f32(focal_x)
    top, bottom = (-my - oy) / f32(focal_y), (my - oy) / f32(focal_y)

    def row(r):
        return (w[r, 0] * p[:, 0] + w[r, 1] * p[:, 1] + w[r, 2] * p[:, 2] + w[r, 3]).astype(f32)
    z, x, y = row(2), row(0), row(1)
    inside = (z >= f32(near_plane)) & ~((x < left * z) | (x > right * z)) & ~((y < top * z) | (y > bottom * z))
    new = (f32(distance2filter) * z).astype(f32)
    old = np.asarray(filter_3d, f32).reshape(-1)
    update = inside & ~(old < new)
    out = np.where(update, new, old).astype(f32)
    return out.reshape(np.asarray(filter_3d).shape), np.asarray(visibility_mask, bool).reshape(-1) | update
