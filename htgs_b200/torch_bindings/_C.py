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

_last_frame_info = None     # HtgsFrameInfo of the most recent call through this (ctypes) binding
_last_source = "ctypes"     # which binding made the most recent call (torch_bindings.rasterization sets "pybind")


def __getattr__(name):
    # `_C.last_frame_info`: statistics of the most recent frame, whichever binding rendered it (diagnostics)
    if name == "last_frame_info":
        mods = _native.pybind_modules()
        return mods[0].frame_info() if (mods and _last_source == "pybind") else _last_frame_info
    raise AttributeError(name)


def _set_info(info):
    global _last_frame_info, _last_source
    _last_frame_info = info
    _last_source = "ctypes"

# Deferred checks (torch_bindings.rasterization.set_deferred_checks): `render` and `_C_benchmarking.benchmark` queue the frame
# with htgs_render_async and return without waiting for the GPU; the frame's status is checked by the next call on the same
# CUDA stream, or by `frame_results`.  Each CUDA stream gets a context (workspace) of its own, so one host thread can keep
# frames in flight on several streams.  The tensors of a queued frame are kept alive here until its check.
deferred_checks = False
_queued: dict = {}


def frame_results(device=None):
    """Waits for and checks every frame this host thread queued with deferred checks (on `device`, or on all devices);
    raises what the blocking call would have raised.  Returns the HtgsFrameInfo of each context that was checked."""
    index = None if device is None else _device_index(torch.device(device))
    infos = []
    for ctx in _native.contexts_of_thread(index):
        if ctx not in _queued:
            continue
        info = HtgsFrameInfo()
        rc = _native.lib().htgs_frame_result(ctx, ctypes.byref(info))
        _queued.pop(ctx, None)
        _native.check(rc)
        infos.append(info)
        _set_info(info)
    return infos


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
    n, device = _check_inputs(positions, scales, rotations, opacities, sh_0, sh_rest, M, VPM, cam_position)
    tensors = [t.contiguous() for t in (positions, scales, rotations, opacities, sh_0, sh_rest)]
    M, VPM, cam_position = M.contiguous(), VPM.contiguous(), cam_position.contiguous()
    with torch.cuda.device(device):
        image = torch.empty((3, height, width) if to_chw else (height, width, 3), dtype=torch.float32, device=device)
        depth = torch.empty((height, width), dtype=torch.float32, device=device)
        scene, view = _scene_view(tensors, M, VPM, cam_position, rasterizer_mode, K, active_sh_bases, width, height, near_plane, far_plane, scale_modifier)
        info = HtgsFrameInfo()
        stream = torch.cuda.current_stream(device).cuda_stream
        if deferred_checks:
            ctx = _native.context(_device_index(device), stream)
            rc = _native.lib().htgs_render_async(ctx, ctypes.byref(scene), ctypes.byref(view), image.data_ptr(), depth.data_ptr(), None,
                                                 int(bool(to_chw)), int(bool(use_median_depth)), stream)
            _queued[ctx] = (tensors, M, VPM, cam_position, image, depth)
            _native.check(rc)
            return image, depth
        rc = _native.lib().htgs_render(_native.context(_device_index(device)),
                                       ctypes.byref(scene), ctypes.byref(view), image.data_ptr(), depth.data_ptr(), None, int(bool(to_chw)),
                                       int(bool(use_median_depth)), None, 0, stream, ctypes.byref(info))
    _native.check(rc)
    _set_info(info)
    return image, depth


def _device_index(device):
    return device.index if device.index is not None else torch.cuda.current_device()


def forward(positions, scales, rotations, opacities, sh_0, sh_rest, M, VPM, cam_position, rasterizer_mode, K, active_sh_bases,
            width, height, near_plane, far_plane, scale_modifier):
    """`_C.forward` (rasterization/include/rasterization_api.h:8-26): returns
    (image, per_primitive_buffers, per_tile_buffers, per_instance_buffers, per_pixel_buffers, n_instances, selector).
    The four byte tensors are opaque to the caller and only meaningful to `backward` of this module."""
    n, device = _check_inputs(positions, scales, rotations, opacities, sh_0, sh_rest, M, VPM, cam_position)
    tensors = [t.contiguous() for t in (positions, scales, rotations, opacities, sh_0, sh_rest)]
    M, VPM, cam_position = M.contiguous(), VPM.contiguous(), cam_position.contiguous()
    lib = _native.lib()
    with torch.cuda.device(device):
        ctx = _native.context(_device_index(device))
        scene, view = _scene_view(tensors, M, VPM, cam_position, rasterizer_mode, K, active_sh_bases, width, height, near_plane, far_plane, 1.0)
        sz = [ctypes.c_size_t() for _ in range(3)]
        _native.check(lib.htgs_forward_blob_sizes(ctypes.byref(scene), ctypes.byref(view), *(ctypes.byref(x) for x in sz)))
        byte = dict(dtype=torch.uint8, device=device)
        per_primitive = torch.empty(sz[0].value, **byte)
        per_tile = torch.empty(sz[1].value, **byte)
        per_pixel = torch.empty(sz[2].value, **byte)
        image = torch.empty((3, height, width), dtype=torch.float32, device=device)
        stream = torch.cuda.current_stream(device).cuda_stream
        n_inst = ctypes.c_uint32()
        _native.check(lib.htgs_forward_begin(ctx, ctypes.byref(scene), ctypes.byref(view), per_primitive.data_ptr(), per_primitive.numel(), stream,
                                             ctypes.byref(n_inst)))
        if track_visibility:     # before the rest of the forward is enqueued: the list is final and the stream is idle here
            visible = torch.empty(n, dtype=torch.uint8, device=device)
            head = _native.HtgsTrainBlobs(per_primitive.data_ptr(), per_primitive.numel(), None, 0, None, 0, None, 0)
            _native.check(lib.htgs_forward_visibility(ctypes.byref(scene), ctypes.byref(head), visible.data_ptr(), stream))
            ready = torch.cuda.Event()
            key = torch.device(device)
            mask = visible.view(torch.bool)
            earlier = last_visibility.get(key)
            if earlier is not None and accumulate_visibility and earlier[0].shape == mask.shape:
                mask |= earlier[0]          # several forwards per step: a row any of them kept can be non-zero
            ready.record(torch.cuda.current_stream(device))
            last_visibility[key] = (mask, ready)
        # The instance count changes from view to view; exact sizes would miss torch's block cache on every heavier view.  Two
        # sizes per power of two, and never smaller than the largest this device has needed (unless that is over four times too
        # much: another scene): the same request step after step.
        capacity = int(lib.htgs_forward_instance_capacity(n_inst.value))
        largest = max(capacity, _largest_instance_capacity.get(_device_index(device), 0))
        _largest_instance_capacity[_device_index(device)] = largest
        if largest <= 4 * capacity:
            capacity = largest
        per_instance = torch.empty(lib.htgs_forward_instance_bytes(ctypes.byref(view), capacity), **byte)
        blobs = _native.HtgsTrainBlobs(per_primitive.data_ptr(), per_primitive.numel(), per_tile.data_ptr(), per_tile.numel(),
                                       per_instance.data_ptr(), per_instance.numel(), per_pixel.data_ptr(), per_pixel.numel())
        info = HtgsFrameInfo()
        _native.check(lib.htgs_forward_finish(ctx, ctypes.byref(scene), ctypes.byref(view), ctypes.byref(blobs), n_inst.value, image.data_ptr(), stream,
                                              ctypes.byref(info)))
    _set_info(info)
    return image, per_primitive, per_tile, per_instance, per_pixel, int(n_inst.value), 0


# When set, every training forward leaves (bool tensor [N] of the Gaussians it kept, event recorded after the tensor was
# written) here, per device; see torch_bindings.rasterization.track_training_visibility.
track_visibility = False
last_visibility: dict = {}
_largest_instance_capacity: dict = {}      # device index -> largest per-instance capacity a training forward has allocated
accumulate_visibility = False     # OR the masks of successive forwards until the mask is reset (several forwards per training step)


# The extras of the compiled module `htgs_b200.pybind._C` under the same names, so that the surface can use either binding.
def frame_info():
    return _last_frame_info


def set_deferred_checks(enable: bool) -> None:
    global deferred_checks
    if not enable:
        frame_results()
    deferred_checks = bool(enable)


def set_max_weights_tail_credit(enable: bool) -> None:
    global max_weights_tail_credit
    max_weights_tail_credit = bool(enable)


def set_track_visibility(enable: bool) -> None:
    global track_visibility
    track_visibility = bool(enable)
    if not enable:
        last_visibility.clear()


def get_last_visibility(device_index: int):
    return last_visibility.get(torch.device("cuda", int(device_index)))


def reset_visibility(device_index=None) -> None:
    if device_index is None:
        last_visibility.clear()
    else:
        last_visibility.pop(torch.device("cuda", int(device_index)), None)


def benchmark(*args):
    from . import _C_benchmarking
    return _C_benchmarking.benchmark(*args)


def forward_visibility(per_primitive_buffers, n_primitives: int):
    """Bool tensor [N]: the Gaussians the training forward that filled `per_primitive_buffers` kept (the only rows of the
    gradient tensors its backward pass can make non-zero).  No counterpart in the reference."""
    device = per_primitive_buffers.device
    visible = torch.empty(n_primitives, dtype=torch.uint8, device=device)
    scene = _native.HtgsScene()
    scene.n_primitives = n_primitives
    blobs = _native.HtgsTrainBlobs(per_primitive_buffers.data_ptr(), per_primitive_buffers.numel(), None, 0, None, 0, None, 0)
    with torch.cuda.device(device):
        stream = torch.cuda.current_stream(device).cuda_stream
        _native.check(_native.lib().htgs_forward_visibility(ctypes.byref(scene), ctypes.byref(blobs), visible.data_ptr(), stream))
    return visible.view(torch.bool)


def backward(densification_info, grad_image, image, positions, scales, rotations, opacities, sh_rest, per_primitive_buffers, per_tile_buffers,
             per_instance_buffers, per_pixel_buffers, M, VPM, cam_position, rasterizer_mode, K, active_sh_bases, width, height, near_plane,
             far_plane, scale_modifier, n_instances, instance_primitive_indices_selector, use_distance_scaling, ranges=None, after_range=None,
             split_pass=True, compact=None):
    """`_C.backward` (rasterization/include/rasterization_api.h:28-55): returns the six gradients; `densification_info`
    ([2|3, N, 1] or empty) is updated in place.  `image` / `opacities` may be empty tensors, as the reference's autograd
    function passes them (torch_bindings/rasterization.py:72-76).

    Beyond the reference: with `ranges` (a list of (first Gaussian, count) that tiles [0, N)) the pass runs range by range
    (`htgs_backward_range`) and `after_range(k, first, count, grads)` is called after range k has been queued, with the six
    gradient tensors whose rows [first, first + count) are final once the stream gets there; a multi-GPU trainer starts
    summing those rows over the ranks while the next range is computed (htgs_b200.parallel.BackwardExchange).  With
    `split_pass=False` the per-tile pass runs once for all Gaussians (`htgs_backward_accumulate`) and only the per-Gaussian
    chain rule runs range by range (`htgs_backward_finish_range`): less to hide the exchange behind, but no cost for the split.

    With `compact` (an object with `capacity(n)` and `exchange(rows)`, e.g. htgs_b200.parallel.CompactExchange) the pass writes
    compact rows (`htgs_backward_compact`: 64 bytes per Gaussian the view kept instead of dense rows), `compact.exchange(rows)`
    returns the row buffers of all ranks in rank order, and the six tensors returned are the sums over those buffers
    (`htgs_expand_add_rows`), identical on every rank."""
    device = positions.device
    if device.type != "cuda":
        raise ValueError("htgs_b200 rasterizer: tensors must live on a CUDA device")
    n = positions.shape[0]
    total_sh = sh_rest.shape[1]
    for name, t in (("grad_image", grad_image), ("positions", positions), ("scales", scales), ("rotations", rotations), ("sh_rest", sh_rest)):
        if t.dtype != torch.float32 or t.device != device:
            raise TypeError(f"{name} must be a float32 tensor on {device}")
    if tuple(grad_image.shape) != (3, height, width):
        raise ValueError(f"grad_image must have shape (3, {height}, {width}), got {tuple(grad_image.shape)}")
    grad_image = grad_image.contiguous()
    positions, scales, rotations, sh_rest = positions.contiguous(), scales.contiguous(), rotations.contiguous(), sh_rest.contiguous()
    M, VPM, cam_position = M.contiguous(), VPM.contiguous(), cam_position.contiguous()
    lib = _native.lib()
    with torch.cuda.device(device):
        ctx = _native.context(_device_index(device))
        f32 = dict(dtype=torch.float32, device=device)
        grad_positions = torch.empty((n, 3), **f32)
        grad_scales = torch.empty((n, 3), **f32)
        grad_rotations = torch.empty((n, 4), **f32)
        grad_opacities = torch.empty((n, 1), **f32)
        grad_sh_0 = torch.empty((n, 1, 3), **f32)
        grad_sh_rest = torch.empty((n, total_sh, 3), **f32)
        # opacities / sh_0 are not read by the backward kernels (the forward's records hold what is needed)
        scene = HtgsScene(positions.data_ptr(), scales.data_ptr(), rotations.data_ptr(), positions.data_ptr(), positions.data_ptr(),
                          sh_rest.data_ptr() if sh_rest.numel() else None, n, total_sh)
        view = HtgsView(M.data_ptr(), VPM.data_ptr(), cam_position.data_ptr(), int(rasterizer_mode), int(K), int(active_sh_bases), int(width), int(height),
                        float(near_plane), float(far_plane), 1.0)
        scratch = torch.empty(lib.htgs_backward_scratch_bytes(ctypes.byref(scene)), dtype=torch.uint8, device=device)
        rows_d = int(densification_info.shape[0]) if densification_info.numel() > 0 else 0
        if rows_d not in (0, 2, 3):
            raise ValueError("densification_info must be empty or have 2 or 3 rows")
        if rows_d and (densification_info.dtype != torch.float32 or densification_info.device != device or not densification_info.is_contiguous()
                       or densification_info.numel() != rows_d * n):
            raise ValueError("densification_info must be a contiguous float32 tensor of shape [rows, N, 1] on the same device")
        grads = _native.HtgsGradients(grad_positions.data_ptr(), grad_scales.data_ptr(), grad_rotations.data_ptr(), grad_opacities.data_ptr(),
                                      grad_sh_0.data_ptr(), grad_sh_rest.data_ptr() if grad_sh_rest.numel() else None, scratch.data_ptr(), scratch.numel(),
                                      densification_info.data_ptr() if rows_d else None, rows_d, int(bool(use_distance_scaling)))
        blobs = _native.HtgsTrainBlobs(per_primitive_buffers.data_ptr(), per_primitive_buffers.numel(), per_tile_buffers.data_ptr(),
                                       per_tile_buffers.numel(), per_instance_buffers.data_ptr(), per_instance_buffers.numel(),
                                       per_pixel_buffers.data_ptr(), per_pixel_buffers.numel())
        image_ptr = image.contiguous().data_ptr() if image.numel() else None
        stream = torch.cuda.current_stream(device).cuda_stream
        outs = (grad_positions, grad_scales, grad_rotations, grad_opacities, grad_sh_0, grad_sh_rest)
        if compact is not None:
            capacity = int(compact.capacity(n))
            rows = compact.buffer(lib.htgs_compact_rows_bytes(capacity), device)
            # "sum": all buffers are local memory and one pass writes every dense row once (htgs_expand_sum_rows; nothing to clear);
            # "add": buffer after buffer into tensors the backward call cleared (htgs_expand_add_rows; reads a peer's buffer in place)
            one_pass = getattr(compact, "expansion", lambda: "add")() == "sum"
            no_dense = _native.HtgsGradients(None, None, None, None, None, None, scratch.data_ptr(), scratch.numel(),
                                             densification_info.data_ptr() if rows_d else None, rows_d, int(bool(use_distance_scaling)))
            _native.check(lib.htgs_backward_compact(ctx, ctypes.byref(scene), ctypes.byref(view), ctypes.byref(blobs), int(n_instances), grad_image.data_ptr(),
                                                    image_ptr, ctypes.byref(no_dense if one_pass else grads), rows.data_ptr(), capacity, stream))
            parts = compact.exchange(rows, capacity)
            if one_pass:
                addresses = (ctypes.c_void_p * len(parts))(*[int(address) for address, _, _ in parts])
                table = torch.empty(lib.htgs_expand_sum_scratch_bytes(ctypes.byref(scene), len(parts)), dtype=torch.uint8, device=device)
                _native.check(lib.htgs_expand_sum_rows(ctypes.byref(scene), addresses, len(parts), capacity, table.data_ptr(), table.numel(), ctypes.byref(grads), stream))
                table.record_stream(torch.cuda.current_stream(device))
            else:
                for address, rows_capacity, keep_alive in parts:
                    _native.check(lib.htgs_expand_add_rows(ctypes.byref(scene), address, int(rows_capacity), ctypes.byref(grads), stream))
            scratch.record_stream(torch.cuda.current_stream(device))
            return outs
        if ranges is None:
            _native.check(lib.htgs_backward(ctx, ctypes.byref(scene), ctypes.byref(view), ctypes.byref(blobs), int(n_instances), grad_image.data_ptr(),
                                            image_ptr, ctypes.byref(grads), stream))
        else:
            covered = 0
            if not split_pass:
                _native.check(lib.htgs_backward_accumulate(ctx, ctypes.byref(scene), ctypes.byref(view), ctypes.byref(blobs), int(n_instances),
                                                           grad_image.data_ptr(), image_ptr, ctypes.byref(grads), stream))
            for k, (first, count) in enumerate(ranges):
                if first != covered:
                    raise ValueError("ranges must tile [0, N) in ascending order")
                covered += count
                if split_pass:
                    _native.check(lib.htgs_backward_range(ctx, ctypes.byref(scene), ctypes.byref(view), ctypes.byref(blobs), int(n_instances),
                                                          grad_image.data_ptr(), image_ptr, ctypes.byref(grads), int(first), int(count), stream))
                else:
                    _native.check(lib.htgs_backward_finish_range(ctx, ctypes.byref(scene), ctypes.byref(view), ctypes.byref(blobs), ctypes.byref(grads),
                                                                 int(first), int(count), stream))
                if after_range is not None:
                    after_range(k, int(first), int(count), outs)
            if covered != n:
                raise ValueError("ranges must tile [0, N)")
        scratch.record_stream(torch.cuda.current_stream(device))
    return outs


# HYBRID_BLEND `update_max_weights`: False (default) reproduces the reference extension's output, which credits K-buffer (core)
# weights only; True also performs the second walk of the reference's kernel SOURCE that credits `alpha * tail weight` to
# every fragment (torch_bindings.rasterization.set_max_weights_tail_credit).
max_weights_tail_credit = False


def update_max_weights(max_weights, positions, scales, rotations, opacities, M, VPM, cam_position, rasterizer_mode, K, active_sh_bases,
                       width, height, near_plane, far_plane, scale_modifier, weight_threshold):
    """`_C.update_max_weights` (rasterization/include/rasterization_api.h:79-97): raises `max_weights` [N,1] in place."""
    device = positions.device
    if device.type != "cuda":
        raise ValueError("htgs_b200 rasterizer: tensors must live on a CUDA device")
    n = positions.shape[0]
    for name, t in (("max_weights", max_weights), ("positions", positions), ("scales", scales), ("rotations", rotations), ("opacities", opacities),
                    ("M", M), ("VPM", VPM), ("cam_position", cam_position)):
        if t.dtype != torch.float32 or t.device != device:
            raise TypeError(f"{name} must be a float32 tensor on {device}")
    if tuple(positions.shape) != (n, 3) or tuple(scales.shape) != (n, 3) or tuple(rotations.shape) != (n, 4) or opacities.numel() != n:
        raise ValueError("expected positions [N,3], scales [N,3], rotations [N,4], opacities [N,1]")
    if max_weights.numel() != n or not max_weights.is_contiguous():
        raise ValueError("max_weights is updated in place and must be a contiguous tensor of N values")
    tensors = [t.contiguous() for t in (positions, scales, rotations, opacities)]
    M, VPM, cam_position = M.contiguous(), VPM.contiguous(), cam_position.contiguous()
    with torch.cuda.device(device):
        scene = HtgsScene(tensors[0].data_ptr(), tensors[1].data_ptr(), tensors[2].data_ptr(), tensors[3].data_ptr(), None, None, n, 0)
        view = HtgsView(M.data_ptr(), VPM.data_ptr(), cam_position.data_ptr(), int(rasterizer_mode), int(K), int(active_sh_bases), int(width), int(height),
                        float(near_plane), float(far_plane), float(scale_modifier))
        info = HtgsFrameInfo()
        _native.check(_native.lib().htgs_set_max_weights_tail_credit(_native.context(_device_index(device)), int(max_weights_tail_credit)))
        rc = _native.lib().htgs_update_max_weights(_native.context(_device_index(device)), ctypes.byref(scene), ctypes.byref(view), max_weights.data_ptr(),
                                                   float(weight_threshold), None, 0, torch.cuda.current_stream(device).cuda_stream, ctypes.byref(info))
    _native.check(rc)
    _set_info(info)


def update_3d_filter_cuda(positions, w2c, filter_3d, visibility_mask, width, height, focal_x, focal_y, center_x, center_y, near_plane,
                          clipping_tolerance, distance2filter):
    """`_C.update_3d_filter_cuda` (filter3d/include/filter3d_api.h:7-20): updates `filter_3d` and `visibility_mask` in place."""
    device = positions.device
    if device.type != "cuda":
        raise ValueError("htgs_b200: tensors must live on a CUDA device")
    n = positions.shape[0]
    if positions.dtype != torch.float32 or w2c.dtype != torch.float32 or filter_3d.dtype != torch.float32 or visibility_mask.dtype != torch.bool:
        raise TypeError("positions, w2c, filter_3d must be float32 and visibility_mask bool")
    if tuple(positions.shape) != (n, 3) or w2c.numel() != 16 or filter_3d.numel() != n or visibility_mask.numel() != n:
        raise ValueError("expected positions [N,3], w2c [4,4], filter_3d [N,1], visibility_mask [N]")
    if not (filter_3d.is_contiguous() and visibility_mask.is_contiguous()):
        raise ValueError("filter_3d and visibility_mask are updated in place and must be contiguous")
    positions, w2c = positions.contiguous(), w2c.contiguous()
    with torch.cuda.device(device):
        rc = _native.lib().htgs_update_3d_filter(positions.data_ptr(), w2c.data_ptr(), filter_3d.data_ptr(), visibility_mask.data_ptr(), n, int(width),
                                                 int(height), float(focal_x), float(focal_y), float(center_x), float(center_y), float(near_plane),
                                                 float(clipping_tolerance), float(distance2filter), torch.cuda.current_stream(device).cuda_stream)
    _native.check(rc)


def update_3d_filter_views_cuda(positions, w2cs, filter_3d, visibility_mask, widths, heights, focal_xs, focal_ys, center_xs, center_ys, near_planes,
                                clipping_tolerance, distance2filter):
    """All views of a dataset in one pass over the points (`htgs_update_3d_filter_views`): equal, bit for bit, to
    `update_3d_filter_cuda` called once per view in order.  `w2cs` is [V,4,4] (any device: the matrices travel as kernel
    arguments); the per-view camera parameters are sequences of length V."""
    import numpy as np
    device = positions.device
    if device.type != "cuda":
        raise ValueError("htgs_b200: tensors must live on a CUDA device")
    n = positions.shape[0]
    if positions.dtype != torch.float32 or filter_3d.dtype != torch.float32 or visibility_mask.dtype != torch.bool:
        raise TypeError("positions, filter_3d must be float32 and visibility_mask bool")
    if tuple(positions.shape) != (n, 3) or filter_3d.numel() != n or visibility_mask.numel() != n:
        raise ValueError("expected positions [N,3], filter_3d [N,1], visibility_mask [N]")
    if not (filter_3d.is_contiguous() and visibility_mask.is_contiguous()):
        raise ValueError("filter_3d and visibility_mask are updated in place and must be contiguous")
    mats = (w2cs.detach().cpu().numpy() if isinstance(w2cs, torch.Tensor) else np.asarray(w2cs)).astype(np.float32).reshape(-1, 16)
    n_views = mats.shape[0]
    per_view = [widths, heights, focal_xs, focal_ys, center_xs, center_ys, near_planes]
    if any(len(x) != n_views for x in per_view):
        raise ValueError("one camera parameter per view expected")
    # the host array of HtgsFilterView (16 floats, 2 ints, 5 floats), filled column-wise
    packed = np.zeros(max(n_views, 1), dtype=np.dtype([("w2c", np.float32, 16), ("width", np.int32), ("height", np.int32), ("focal_x", np.float32),
                                                       ("focal_y", np.float32), ("center_x", np.float32), ("center_y", np.float32),
                                                       ("near_plane", np.float32)], align=False))
    assert packed.dtype.itemsize == ctypes.sizeof(_native.HtgsFilterView)
    if n_views:
        packed["w2c"][:n_views] = mats
        for name, values in zip(("width", "height", "focal_x", "focal_y", "center_x", "center_y", "near_plane"), per_view):
            packed[name][:n_views] = np.asarray(values)
    views = packed.ctypes.data_as(ctypes.POINTER(_native.HtgsFilterView))
    positions = positions.contiguous()
    with torch.cuda.device(device):
        rc = _native.lib().htgs_update_3d_filter_views(positions.data_ptr(), views, n_views, filter_3d.data_ptr(), visibility_mask.data_ptr(), n,
                                                       float(clipping_tolerance), float(distance2filter), torch.cuda.current_stream(device).cuda_stream)
    _native.check(rc)
