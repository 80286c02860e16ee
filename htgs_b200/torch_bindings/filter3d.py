"""`update_3d_filter`, name for name the reference's `HTGSCudaBackend.torch_bindings.filter3d` (torch_bindings/filter3d.py)."""
import torch

from .. import _native
from . import _C

_mods = _native.pybind_modules()
_impl = _mods[0] if _mods else _C     # the compiled extension module when it has been built, else the ctypes binding


def update_3d_filter(positions: torch.Tensor, w2c: torch.Tensor, filter_3d: torch.Tensor, visibility_mask: torch.Tensor, width: int, height: int,
                     focal_x: float, focal_y: float, center_x: float, center_y: float, near_plane: float, clipping_tolerance: float,
                     distance2filter: float) -> None:
    return _impl.update_3d_filter_cuda(positions, w2c, filter_3d, visibility_mask, width, height, focal_x, focal_y, center_x, center_y, near_plane,
                                    clipping_tolerance, distance2filter)


def update_3d_filter_views(positions: torch.Tensor, w2cs, filter_3d: torch.Tensor, visibility_mask: torch.Tensor, widths, heights, focal_xs, focal_ys,
                           center_xs, center_ys, near_planes, clipping_tolerance: float, distance2filter: float) -> None:
    """The loop over a dataset's views (Model.py:126-145 of the reference) as one call: same result, bit for bit, as
    `update_3d_filter` once per view, with the positions read once per 48 views."""
    return _C.update_3d_filter_views_cuda(positions, w2cs, filter_3d, visibility_mask, widths, heights, focal_xs, focal_ys, center_xs, center_ys,
                                          near_planes, clipping_tolerance, distance2filter)
