from .rasterization import diff_rasterize, rasterize, fast_rasterize, update_max_weights, RasterizerSettings, RasterizerMode

__all__ = ['diff_rasterize', 'rasterize', 'fast_rasterize', 'update_max_weights', 'RasterizerSettings', 'RasterizerMode']
