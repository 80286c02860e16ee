"""Shared helpers of the parity tests: scene upload, calls into the CUDA path through the
C-ABI / Python surface, access to intermediates, and (when it was built beside the repo)
the reference extension with parsers for its scratch blobs."""
from __future__ import annotations

import ctypes
import os
import sys
from typing import Optional

import numpy as np

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if REPO not in sys.path:
    sys.path.insert(0, REPO)

from htgs_b200 import scenes  # noqa: E402

REF_ROOT = os.path.join(REPO, "baseline", "_ref", "HTGSCudaBackend")


def scene_tensors(scene, device="cuda"):
    import torch
    return [torch.from_numpy(np.ascontiguousarray(a)).to(device) for a in scene.arrays()]


def settings_for(mod, scene, view, mode=None, K=None, scale_modifier=1.0, device="cuda"):
    """RasterizerSettings of `mod` (our torch_bindings or the reference's) for one view."""
    import torch
    mode = scene.mode if mode is None else mode
    K = scene.K if K is None else K
    return mod.RasterizerSettings(
        M=torch.from_numpy(view.M).to(device), VPM=torch.from_numpy(view.VPM).to(device),
        cam_position=torch.from_numpy(view.cam_position).to(device), mode=mod.RasterizerMode(mode), K=K,
        active_sh_bases=scene.active_sh_bases, width=view.width, height=view.height, near_plane=view.near_plane,
        far_plane=view.far_plane, scale_modifier=scale_modifier)


def ours():
    import htgs_b200.torch_bindings as tb
    return tb


_ref_mod = None


def reference():
    """The reference's torch_bindings module, or None when it has not been built under baseline/_ref."""
    global _ref_mod
    if _ref_mod is None:
        so = [f for f in os.listdir(os.path.join(REF_ROOT, "HTGSCudaBackend"))] if os.path.isdir(os.path.join(REF_ROOT, "HTGSCudaBackend")) else []
        if not any(f.startswith("_C.") and f.endswith(".so") for f in so):
            _ref_mod = False
        else:
            if REF_ROOT not in sys.path:
                sys.path.insert(0, REF_ROOT)
            try:
                import HTGSCudaBackend.torch_bindings as rtb
                _ref_mod = rtb
            except Exception:
                _ref_mod = False
    return _ref_mod or None


def d2h(ptr: int, count: int, dtype) -> np.ndarray:
    from htgs_b200 import _native
    out = np.empty(count, dtype=dtype)
    if count:
        _native.check(_native.lib().htgs_memcpy_d2h(out.ctypes.data_as(ctypes.c_void_p), ctypes.c_void_p(ptr), out.nbytes))
    return out


def our_intermediates(device_index: int, n_primitives: int, n_instances: int):
    """Copies of the binning/preprocess intermediates of the last frame rendered on the device."""
    from htgs_b200 import _native
    inter = _native.HtgsIntermediates()
    _native.check(_native.lib().htgs_get_intermediates(_native.context(device_index), ctypes.byref(inter)))
    key_dtype = {2: np.uint16, 4: np.uint32, 8: np.uint64}[inter.key_bytes]
    n = n_primitives
    out = {
        "n_touched": d2h(inter.n_touched, n, np.uint32),
        "bounds": d2h(inter.bounds, 4 * n, np.uint16).reshape(n, 4),
        "eval": d2h(inter.eval_records, 20 * n, np.float32).reshape(n, 5, 4),
        "cull": d2h(inter.cull_records, 8 * n, np.float32).reshape(n, 8),
        "keys_sorted": d2h(inter.keys_sorted, n_instances, key_dtype),
        "prims_sorted": d2h(inter.prims_sorted, n_instances, np.uint32),
        "ranges": d2h(inter.tile_ranges, 2 * inter.n_tiles, np.uint32).reshape(inter.n_tiles, 2),
        "grid_w": inter.grid_width, "grid_h": inter.grid_height, "n_tiles": inter.n_tiles, "key_bytes": inter.key_bytes,
    }
    if inter.keys_unsorted:
        out["keys_unsorted"] = d2h(inter.keys_unsorted, n_instances, key_dtype)
        out["prims_unsorted"] = d2h(inter.prims_unsorted, n_instances, np.uint32)
    return out


# ----------------------------------------------------------------------------------------------
# parsers for the reference's scratch blobs (layouts: rasterization/include/*/buffer_utils.h;
# every section starts on a 128-byte boundary of the absolute address, torch allocations are
# at least 512-byte aligned, so offsets relative to the blob follow the same rule)
# ----------------------------------------------------------------------------------------------
def _align128(x: int) -> int:
    return (x + 127) & ~127


def parse_ref_per_primitive(blob: np.ndarray, n: int, mode: int, store_rgba=True, store_clamp=True):
    off = 0
    out = {}

    def take(name, count, dtype, shape=None):
        nonlocal off
        off = _align128(off)
        nbytes = count * np.dtype(dtype).itemsize
        arr = blob[off:off + nbytes].view(dtype)
        out[name] = arr.reshape(shape) if shape else arr
        off += nbytes

    take("n_touched", n, np.uint32)
    take("offset", n, np.uint32)
    take("bounds", 4 * n, np.uint32, (n, 4))
    take("vpmt1", 4 * n, np.float32, (n, 4))
    take("vpmt2", 4 * n, np.float32, (n, 4))
    take("vpmt4", 4 * n, np.float32, (n, 4))
    if mode == scenes.ALPHA_BLEND_GLOBAL_ORDERING:
        take("depth", n, np.float32)
    elif mode != scenes.OIT_BLEND:          # the OIT training forward does not store MT3 (oit_blend/forward.cu:48)
        take("mt3", 4 * n, np.float32, (n, 4))
    if mode == scenes.ALPHA_BLEND_FIRST_K:
        if store_rgba:
            take("rgb", 3 * n, np.float32, (n, 3))
    elif store_rgba:
        take("rgba", 4 * n, np.float32, (n, 4))
    if store_clamp:
        take("clamp", 3 * n, np.uint8, (3, n))
    return out


def parse_ref_per_instance(blob: np.ndarray, n_instances: int, key_bytes: int, selector: int):
    key_dtype = {2: np.uint16, 4: np.uint32, 8: np.uint64}[key_bytes]
    off = 0
    secs = []
    for count, dtype in ((n_instances, key_dtype), (n_instances, key_dtype), (n_instances, np.uint32), (n_instances, np.uint32)):
        off = _align128(off)
        nbytes = count * np.dtype(dtype).itemsize
        secs.append(blob[off:off + nbytes].view(dtype))
        off += nbytes
    return {"keys_sorted": secs[selector], "prims_sorted": secs[2 + selector]}


def parse_ref_per_tile(blob: np.ndarray, n_tiles: int):
    return blob[: 8 * n_tiles].view(np.uint32).reshape(n_tiles, 2)


def sort_key_bytes(mode: int, n_tiles: int) -> int:
    if mode == scenes.ALPHA_BLEND_GLOBAL_ORDERING:
        return 8
    return 2 if max(n_tiles - 1, 0).bit_length() <= 16 else 4
