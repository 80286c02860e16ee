"""Counterpart of the reference's second extension module `HTGSCudaBackend._C_benchmarking`
(rasterization/src/fast_inference_api.cu:21-162, bound in torch_bindings/bindings.cpp): one function, `benchmark`,
the relaxed-precision RGB-only forward behind `fast_rasterize`.  Calls `htgs_render_fast` of the C-ABI library.
"""
from __future__ import annotations

import ctypes

import torch

from .. import _native
from .._native import HtgsFrameInfo
from . import _C


def benchmark(positions, scales, rotations, opacities, sh_0, sh_rest, M, VPM, cam_position, rasterizer_mode, K, active_sh_bases,
              width, height, near_plane, far_plane, scale_modifier, to_chw) -> torch.Tensor:
    """Same 18 positional arguments as the reference (rasterization/include/fast_inference_api.h:7-25); returns the image,
    [3,H,W] if `to_chw` else [H,W,3], clamped to [0,1]."""
    n, device = _C._check_inputs(positions, scales, rotations, opacities, sh_0, sh_rest, M, VPM, cam_position)
    tensors = [t.contiguous() for t in (positions, scales, rotations, opacities, sh_0, sh_rest)]
    M, VPM, cam_position = M.contiguous(), VPM.contiguous(), cam_position.contiguous()
    with torch.cuda.device(device):
        image = torch.empty((3, height, width) if to_chw else (height, width, 3), dtype=torch.float32, device=device)
        scene, view = _C._scene_view(tensors, M, VPM, cam_position, rasterizer_mode, K, active_sh_bases, width, height, near_plane, far_plane,
                                     scale_modifier)
        info = HtgsFrameInfo()
        stream = torch.cuda.current_stream(device).cuda_stream
        if _C.deferred_checks:     # see _C.deferred_checks: queued without a host wait, checked by the next call on this stream
            ctx = _native.context(_C._device_index(device), stream)
            rc = _native.lib().htgs_render_fast_async(ctx, ctypes.byref(scene), ctypes.byref(view), image.data_ptr(), int(bool(to_chw)), stream)
            _C._queued[ctx] = (tensors, M, VPM, cam_position, image)
            _native.check(rc)
            return image
        rc = _native.lib().htgs_render_fast(_native.context(_C._device_index(device)), ctypes.byref(scene), ctypes.byref(view), image.data_ptr(),
                                            int(bool(to_chw)), None, 0, stream, ctypes.byref(info))
    _native.check(rc)
    _C._set_info(info)
    return image
