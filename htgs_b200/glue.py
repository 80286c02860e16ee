"""What the callers of the rasterizer do on either side of it, restated so that the hot path can be used without
the NeRFICG framework the reference lives in:

* `extract_settings`  - camera -> `RasterizerSettings` (Renderer.py:18-57 of the reference);
* `activate`          - raw model parameters -> rasterizer inputs in one fused CUDA pass, differentiable
                        (Model.py:45-49 and 82-100: exp / normalize / expit and the 3D-filter adjustment);
* `reference_activate`- the same with the element-wise PyTorch operations the reference uses (for comparison).
"""
from __future__ import annotations

import ctypes
import warnings

import numpy as np
import torch

from . import _native
from .torch_bindings import RasterizerMode, RasterizerSettings


def extract_settings(w2c, focal_x: float, focal_y: float, center_x: float, center_y: float, width: int, height: int, near_plane: float,
                     far_plane: float, cam_position, mode: int, K: int, active_sh_bases: int, scale_modifier: float = 1.0,
                     device="cuda") -> RasterizerSettings:
    """Camera -> settings, as Renderer.py:18-57: `VP` maps view space to pixel coordinates with pixel centres at integer
    positions (hence the -0.5) and depth to [-1, 1]; `VPM = VP @ w2c` is evaluated in the dtype of `w2c` and cast to
    float32.  An invalid mode falls back to HYBRID_BLEND with a warning, as the reference does."""
    try:
        rasterizer_mode = RasterizerMode(mode)
    except ValueError:
        warnings.warn(f"Invalid rasterizer mode: {mode}. Defaulting to HYBRID_BLEND.")
        rasterizer_mode = RasterizerMode.HYBRID_BLEND
    M = w2c.detach().cpu().numpy() if isinstance(w2c, torch.Tensor) else np.asarray(w2c)
    if M.shape != (4, 4):
        raise ValueError("w2c must be a 4x4 matrix")
    z_range = far_plane - near_plane
    VP = np.array([
        [focal_x, 0.0, center_x - 0.5, 0.0],
        [0.0, focal_y, center_y - 0.5, 0.0],
        [0.0, 0.0, (far_plane + near_plane) / z_range, -2.0 * far_plane * near_plane / z_range],
        [0.0, 0.0, 1.0, 0.0]], dtype=M.dtype)
    VPM = VP @ M
    return RasterizerSettings(
        M=torch.as_tensor(M, dtype=torch.float32, device=device),
        VPM=torch.as_tensor(VPM, dtype=torch.float32, device=device),
        cam_position=torch.as_tensor(cam_position, dtype=torch.float32, device=device),
        mode=rasterizer_mode, K=K, active_sh_bases=active_sh_bases, width=int(width), height=int(height),
        near_plane=float(near_plane), far_plane=float(far_plane), scale_modifier=float(scale_modifier))


def _check(t: torch.Tensor, name: str, cols: int, n: int):
    if t.dtype != torch.float32 or t.device.type != "cuda":
        raise ValueError(f"{name} must be a float32 CUDA tensor")
    if t.numel() != n * cols:
        raise ValueError(f"{name} must hold {cols} values per Gaussian")
    return t.contiguous()


class _Activate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, raw_scales, raw_rotations, raw_opacities, filter_3d):
        n = raw_scales.shape[0]
        rs, rr, ro = _check(raw_scales, "raw_scales", 3, n), _check(raw_rotations, "raw_rotations", 4, n), _check(raw_opacities, "raw_opacities", 1, n)
        f = None if filter_3d is None else _check(filter_3d, "filter_3d", 1, n)
        scales, rotations, opacities = torch.empty_like(rs), torch.empty_like(rr), torch.empty_like(ro)
        with torch.cuda.device(rs.device):
            stream = torch.cuda.current_stream(rs.device).cuda_stream
            _native.check(_native.lib().htgs_activate(rs.data_ptr(), rr.data_ptr(), ro.data_ptr(), None if f is None else f.data_ptr(),
                                                      scales.data_ptr(), rotations.data_ptr(), opacities.data_ptr(), n, stream))
        ctx.save_for_backward(rs, rr, ro, *(() if f is None else (f,)))
        ctx.has_filter = f is not None
        return scales, rotations, opacities

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad_scales, grad_rotations, grad_opacities):
        saved = ctx.saved_tensors
        rs, rr, ro = saved[:3]
        f = saved[3] if ctx.has_filter else None
        n = rs.shape[0]
        gs, gr, go = grad_scales.contiguous(), grad_rotations.contiguous(), grad_opacities.contiguous()
        d_rs, d_rr, d_ro = torch.empty_like(rs), torch.empty_like(rr), torch.empty_like(ro)
        with torch.cuda.device(rs.device):
            stream = torch.cuda.current_stream(rs.device).cuda_stream
            _native.check(_native.lib().htgs_activate_backward(rs.data_ptr(), rr.data_ptr(), ro.data_ptr(), None if f is None else f.data_ptr(),
                                                               gs.data_ptr(), gr.data_ptr(), go.data_ptr(), d_rs.data_ptr(), d_rr.data_ptr(),
                                                               d_ro.data_ptr(), n, stream))
        return d_rs, d_rr, d_ro, None


def activate(raw_scales: torch.Tensor, raw_rotations: torch.Tensor, raw_opacities: torch.Tensor, filter_3d: torch.Tensor | None = None):
    """(log-scales [N,3], unnormalised quaternions [N,4], opacity logits [N,1], optional 3D filter [N,1]) ->
    (scales, rotations, opacities) as the rasterizer expects them.  One kernel forward, one backward."""
    return _Activate.apply(raw_scales, raw_rotations, raw_opacities, filter_3d)


def reference_activate(raw_scales: torch.Tensor, raw_rotations: torch.Tensor, raw_opacities: torch.Tensor, filter_3d: torch.Tensor | None = None):
    """The element-wise PyTorch formulation of Model.py:45-49 / 82-100."""
    scales = torch.exp(raw_scales)
    rotations = torch.nn.functional.normalize(raw_rotations)
    opacities = torch.special.expit(raw_opacities)
    if filter_3d is not None:
        scales_square = torch.square(scales)
        det1 = scales_square.prod(dim=1)
        scales_after_square = scales_square + torch.square(filter_3d)
        det2 = scales_after_square.prod(dim=1)
        opacities = opacities * torch.sqrt(det1 / det2)[..., None]
        scales = torch.sqrt(scales_after_square)
    return scales, rotations, opacities
