"""Python surface of the rasterizer, name for name the reference's
`HTGSCudaBackend.torch_bindings.rasterization` (torch_bindings/rasterization.py:9-206):
`RasterizerMode`, `RasterizerSettings`, `diff_rasterize`, `rasterize`, `fast_rasterize`,
`update_max_weights`.  Code written against the reference runs unchanged after
`from htgs_b200.torch_bindings import ...`.
"""
from __future__ import annotations

from enum import Enum
from typing import Any, NamedTuple

import torch
from torch.autograd.function import once_differentiable

from .. import _native
from . import _C, _C_benchmarking

# The binding behind this surface: the compiled torch extension module `htgs_b200.pybind._C` when it has been built (same
# entry points as the reference's `_C`, plus this library's extras), else the ctypes binding `_C` of this package.  Both call
# the same C-ABI library and share one set of library contexts.
_mods = _native.pybind_modules()
_impl = _mods[0] if _mods else _C
_via_pybind = _mods is not None


def binding() -> str:
    """"pybind" or "ctypes": which binding serves this surface (environment variable HTGS_B200_BINDING)."""
    return "pybind" if _via_pybind else "ctypes"


def _mark():
    if _via_pybind:
        _C._last_source = "pybind"     # `_C.last_frame_info` then reports the extension module's frame


class RasterizerMode(Enum):
    HYBRID_BLEND = 0
    ALPHA_BLEND_FIRST_K = 1
    ALPHA_BLEND_GLOBAL_ORDERING = 2
    OIT_BLEND = 3


class RasterizerSettings(NamedTuple):
    M: torch.Tensor  # affine transformation from model/world space to camera/view space
    VPM: torch.Tensor  # homogeneous transformation from model/world space to screen space
    cam_position: torch.Tensor  # camera position in world space
    mode: RasterizerMode
    K: int  # only used for HYBRID_BLEND and ALPHA_BLEND_FIRST_K
    active_sh_bases: int  # number of spherical harmonics bases used for the colour
    width: int
    height: int
    near_plane: float
    far_plane: float
    scale_modifier: float  # scaling factor applied to every Gaussian

    def as_tuple(self) -> tuple:
        return (self.M, self.VPM, self.cam_position, self.mode.value, self.K, self.active_sh_bases, self.width, self.height,
                self.near_plane, self.far_plane, self.scale_modifier)


# Multi-GPU training exchanges only the gradient rows some rank can have touched (htgs_b200.parallel): when tracking is on,
# every training forward leaves the visibility of its Gaussians, per device.  No counterpart in the reference.
def track_training_visibility(enable: bool, accumulate: bool = False) -> None:
    """`accumulate`: a training step with SEVERAL `diff_rasterize` forwards per rank needs the union of what they kept;
    with it the masks of successive forwards are OR-ed until `reset_training_visibility()` (call that once per step)."""
    _impl.set_track_visibility(bool(enable))
    if _via_pybind:
        _impl.set_accumulate_visibility(bool(enable and accumulate))
    else:
        _C.accumulate_visibility = bool(enable and accumulate)


def reset_training_visibility(device=None) -> None:
    index = None if device is None else (torch.cuda.current_device() if torch.device(device).index is None else torch.device(device).index)
    if _via_pybind:
        _impl.reset_visibility(-1 if index is None else index)
    else:
        _C.reset_visibility(index)


def last_training_visibility(device, with_event: bool = False):
    """Bool tensor [N] of the Gaussians the last `diff_rasterize` forward on `device` kept (needs
    track_training_visibility(True)); with `with_event` also the CUDA event recorded once the tensor was written, which is
    early in the forward (after the preprocess pass), so that a side stream can use it while the forward still runs."""
    key = torch.device(device)
    index = torch.cuda.current_device() if key.index is None else key.index
    record = _impl.last_visibility(index) if _via_pybind else _C.get_last_visibility(index)
    if record is None:
        raise RuntimeError("no training forward was tracked on this device: call track_training_visibility(True) first")
    visible, ready = record
    return (visible, ready) if with_event else visible


# Forward renders without a host wait.  No counterpart in the reference (its `rasterize` blocks in mid-frame).
def set_deferred_checks(enable: bool) -> None:
    """With deferred checks `rasterize` and `fast_rasterize` queue the frame on the current CUDA stream and return at once;
    the frame's status (device error flags, instance buffers that were too small) is checked by the next call on that
    stream or by `frame_results()`.  Each CUDA stream renders with a workspace of its own, so one host thread keeps two
    frames in flight by alternating between two streams.  Render every kind of view once with the checks on (the default)
    first: a frame whose instance buffers turn out too small is rendered again when it is checked, i.e. after work queued
    behind it has already read its image (`HtgsFrameInfo.reruns` of `frame_results()` tells)."""
    _impl.set_deferred_checks(bool(enable))


def deferred_checks() -> bool:
    return bool(_impl.deferred_checks()) if _via_pybind else bool(_C.deferred_checks)


def frame_results(device=None):
    """Waits for and checks the frames queued with deferred checks by this host thread; see `set_deferred_checks`.
    Returns one frame-statistics object per CUDA stream that had a frame queued."""
    _mark()
    if _via_pybind:
        index = -1 if device is None else (torch.cuda.current_device() if torch.device(device).index is None else torch.device(device).index)
        return _impl.frame_results(index)
    return _C.frame_results(device)


# Multi-GPU training (htgs_b200.parallel.BackwardExchange): when set, the backward pass of `diff_rasterize` runs in ranges of
# Gaussians and hands every finished range to the hook, which sums it over the ranks while the next range is computed; the
# gradients autograd receives are then already the sums.  No counterpart in the reference (it is single-GPU).
_backward_hook = None


def set_backward_hook(hook) -> None:
    """`hook` needs ranges(n_primitives, mode) -> [(first, count), ...], after_range(k, first, count, grads) and finish(grads);
    an attribute `split_pass` (default True) says whether the per-tile pass is split along the ranges too or runs once."""
    global _backward_hook
    _backward_hook = hook


class _Rasterize(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, positions, scales, rotations, opacities, sh_0, sh_rest, densification_info,
                rasterizer_settings: RasterizerSettings, use_distance_scaling: bool) -> torch.Tensor:
        _mark()
        image, per_primitive_buffers, per_tile_buffers, per_instance_buffers, per_pixel_buffers, n_instances, selector = _impl.forward(
            positions, scales, rotations, opacities, sh_0, sh_rest, *rasterizer_settings.as_tuple())
        ctx.rasterizer_settings = rasterizer_settings
        ctx.n_instances = n_instances
        ctx.instance_primitive_indices_selector = selector
        ctx.save_for_backward(
            image if rasterizer_settings.mode == RasterizerMode.ALPHA_BLEND_GLOBAL_ORDERING else torch.empty(0),
            positions, scales, rotations,
            opacities if rasterizer_settings.mode == RasterizerMode.ALPHA_BLEND_FIRST_K else torch.empty(0),
            sh_rest, per_primitive_buffers, per_tile_buffers, per_instance_buffers, per_pixel_buffers)
        ctx.densification_info = densification_info
        ctx.mark_non_differentiable(densification_info)
        ctx.use_distance_scaling = use_distance_scaling
        return image

    @staticmethod
    @once_differentiable
    def backward(ctx: Any, grad_image: torch.Tensor):
        hook = _backward_hook
        if hook is None:
            grads = _impl.backward(ctx.densification_info, grad_image, *ctx.saved_tensors, *ctx.rasterizer_settings.as_tuple(),
                                   ctx.n_instances, ctx.instance_primitive_indices_selector, ctx.use_distance_scaling)
        elif getattr(hook, "compact", False):      # compact rows, exchanged by the hook, expanded into sums (htgs_b200.parallel.CompactExchange)
            grads = _C.backward(ctx.densification_info, grad_image, *ctx.saved_tensors, *ctx.rasterizer_settings.as_tuple(),
                                ctx.n_instances, ctx.instance_primitive_indices_selector, ctx.use_distance_scaling, compact=hook)
        else:      # range by range over the C-ABI (the ctypes binding drives the loop; both bindings share the library contexts)
            n = ctx.saved_tensors[1].shape[0]
            grads = _C.backward(ctx.densification_info, grad_image, *ctx.saved_tensors, *ctx.rasterizer_settings.as_tuple(),
                                ctx.n_instances, ctx.instance_primitive_indices_selector, ctx.use_distance_scaling,
                                ranges=hook.ranges(n, ctx.rasterizer_settings.mode.value), after_range=hook.after_range,
                                split_pass=bool(getattr(hook, "split_pass", True)))
            hook.finish(grads)
        grad_positions, grad_scales, grad_rotations, grad_opacities, grad_sh_0, grad_sh_rest = grads
        return (grad_positions, grad_scales, grad_rotations, grad_opacities, grad_sh_0, grad_sh_rest, None, None, None)


def diff_rasterize(positions, scales, rotations, opacities, sh_0, sh_rest, densification_info, settings: RasterizerSettings,
                   use_distance_scaling: bool) -> torch.Tensor:
    return _Rasterize.apply(positions, scales, rotations, opacities, sh_0, sh_rest, densification_info, settings, use_distance_scaling)


def rasterize(positions, scales, rotations, opacities, sh_0, sh_rest, settings: RasterizerSettings, to_chw: bool,
              use_median_depth: bool) -> tuple[torch.Tensor, torch.Tensor]:
    _mark()
    image, depth = _impl.render(positions, scales, rotations, opacities, sh_0, sh_rest, *settings.as_tuple(), to_chw, use_median_depth)
    depth = depth.unsqueeze(0) if to_chw else depth.unsqueeze(-1)
    return image, depth


def fast_rasterize(positions, scales, rotations, opacities, sh_0, sh_rest, settings: RasterizerSettings, to_chw: bool) -> torch.Tensor:
    """The reference's relaxed-precision benchmark path (torch_bindings/rasterization.py:166-186): RGB only."""
    _mark()
    return _impl.benchmark(positions, scales, rotations, opacities, sh_0, sh_rest, *settings.as_tuple(), to_chw)


def set_max_weights_tail_credit(enable: bool) -> None:
    """HYBRID_BLEND `update_max_weights` only.  The reference's kernel source walks every tile's list a second time and
    credits `alpha * tail weight` to each fragment (hybrid_blend/kernels/update_max_weights.cuh:170-210), but the extension
    built from it never runs that kernel: the function template that picks the kernel for K has the same name and signature in
    hybrid_blend/update_max_weights.cu:15-28 and alpha_blend_first_k/update_max_weights.cu:15-28, the linker keeps one of the
    two definitions, and HYBRID_BLEND ends up launching FIRST_K's kernel, which credits K-buffer weights only (a Gaussian that
    only lands in the tail keeps weight 0).  The default (False) reproduces the extension's output bit for bit; True gives what
    the source describes.  No counterpart in the reference."""
    _impl.set_max_weights_tail_credit(bool(enable))


def update_max_weights(max_weights, positions, scales, rotations, opacities, settings: RasterizerSettings, weight_threshold: float) -> None:
    _mark()
    return _impl.update_max_weights(max_weights, positions, scales, rotations, opacities, *settings.as_tuple(), weight_threshold)
