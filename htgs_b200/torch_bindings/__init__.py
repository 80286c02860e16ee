from .rasterization import diff_rasterize, rasterize, fast_rasterize, update_max_weights, RasterizerSettings, RasterizerMode
from .filter3d import update_3d_filter, update_3d_filter_views

__all__ = ['diff_rasterize', 'rasterize', 'fast_rasterize', 'update_max_weights', 'RasterizerSettings', 'RasterizerMode', 'update_3d_filter',
           'update_3d_filter_views']   # the last one has no counterpart in the reference (all views in one pass)
