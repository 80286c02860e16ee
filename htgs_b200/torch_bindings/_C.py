"""Stand-in for the reference's pybind module `HTGSCudaBackend._C` (torch_bindings/bindings.cpp:8-16).

Same function names, argument order and return values; the work is done by the C-ABI
library (include/htgs_b200.h).  PyTorch is used only to allocate outputs and to hand over
device pointers and the current stream.  Inputs are validated up front (dtype, device,
shape) and a Python exception is raised before anything is launched on bad input.
"""
from __future__ import annotations

import ctypes
from typing import Tuple

import torch

from .. import _native
from .._native import HtgsFrameInfo, HtgsScene, HtgsView

last_frame_info = None  # HtgsFrameInfo of the most recent call (diagnostics)


def _check_inputs(positions, scales, rotations, opacities, sh_0, sh_rest, M, VPM, cam_position):
    n = positions.shape[0] if positions.dim() >= 1 else -1
    named = (("positions", positions, (n, 3)), ("scales", scales, (n, 3)), ("rotations", rotations, (n, 4)), ("opacities", opacities, None),
             ("sh_0", sh_0, None), ("sh_rest", sh_rest, None), ("M", M, (4, 4)), ("VPM", VPM, (4, 4)), ("cam_position", cam_position, (3,)))
    device = positions.device
    if device.type != "cuda":
        raise ValueError("htgs_b200 rasterizer: tensors must live on a CUDA device")
    for name, t, shape in named:
        if not isinstance(t, torch.Tensor):
            raise TypeError(f"{name} must be a torch.Tensor")
        if t.dtype != torch.float32:
            raise TypeError(f"{name} must be float32, got {t.dtype}")
        if t.device != device:
            raise ValueError(f"{name} is on {t.device}, expected {device}")
        if shape is not None and tuple(t.shape) != shape:
            raise ValueError(f"{name} must have shape {shape}, got {tuple(t.shape)}")
    if opacities.numel() != n:
        raise ValueError(f"opacities must hold {n} values, got shape {tuple(opacities.shape)}")
    if sh_0.numel() != 3 * n:
        raise ValueError(f"sh_0 must have shape ({n}, 1, 3), got {tuple(sh_0.shape)}")
    if sh_rest.dim() != 3 or sh_rest.shape[0] != n or sh_rest.shape[2] != 3:
        raise ValueError(f"sh_rest must have shape ({n}, B, 3), got {tuple(sh_rest.shape)}")
    return n, device


def _scene_view(tensors, M, VPM, cam_position, mode, K, active_sh_bases, width, height, near_plane, far_plane, scale_modifier):
    positions, scales, rotations, opacities, sh_0, sh_rest = tensors
    scene = HtgsScene(positions.data_ptr(), scales.data_ptr(), rotations.data_ptr(), opacities.data_ptr(), sh_0.data_ptr(),
                      sh_rest.data_ptr() if sh_rest.numel() else None, positions.shape[0], sh_rest.shape[1])
    view = HtgsView(M.data_ptr(), VPM.data_ptr(), cam_position.data_ptr(), int(mode), int(K), int(active_sh_bases), int(width), int(height),
                    float(near_plane), float(far_plane), float(scale_modifier))
    return scene, view


def render(positions, scales, rotations, opacities, sh_0, sh_rest, M, VPM, cam_position, rasterizer_mode, K, active_sh_bases,
           width, height, near_plane, far_plane, scale_modifier, to_chw, use_median_depth) -> Tuple[torch.Tensor, torch.Tensor]:
    """`_C.render` (rasterization/include/rasterization_api.h:57-77): returns (image, depth)."""
    global last_frame_info
    n, device = _check_inputs(positions, scales, rotations, opacities, sh_0, sh_rest, M, VPM, cam_position)
    tensors = [t.contiguous() for t in (positions, scales, rotations, opacities, sh_0, sh_rest)]
    M, VPM, cam_position = M.contiguous(), VPM.contiguous(), cam_position.contiguous()
    with torch.cuda.device(device):
        image = torch.empty((3, height, width) if to_chw else (height, width, 3), dtype=torch.float32, device=device)
        depth = torch.empty((height, width), dtype=torch.float32, device=device)
        scene, view = _scene_view(tensors, M, VPM, cam_position, rasterizer_mode, K, active_sh_bases, width, height, near_plane, far_plane, scale_modifier)
        info = HtgsFrameInfo()
        stream = torch.cuda.current_stream(device).cuda_stream
        rc = _native.lib().htgs_render(_native.context(device.index if device.index is not None else torch.cuda.current_device()),
                                       ctypes.byref(scene), ctypes.byref(view), image.data_ptr(), depth.data_ptr(), None, int(bool(to_chw)),
                                       int(bool(use_median_depth)), None, 0, stream, ctypes.byref(info))
    _native.check(rc)
    last_frame_info = info
    return image, depth


def forward(*args):
    raise NotImplementedError("htgs_b200: the training forward is provided by htgs_b200.torch_bindings._train once built")


def backward(*args):
    raise NotImplementedError("htgs_b200: the backward pass is provided by htgs_b200.torch_bindings._train once built")


def update_max_weights(*args):
    raise NotImplementedError("htgs_b200: update_max_weights is outside the rasterizer hot path of this build")


def update_3d_filter_cuda(*args):
    raise NotImplementedError("htgs_b200: update_3d_filter is outside the rasterizer hot path of this build")
