"""htgs_b200: a B200-native (sm_100a) rasterizer for hybrid-transparency Gaussian splatting.

`htgs_b200.torch_bindings` mirrors `HTGSCudaBackend.torch_bindings` of the reference;
the work happens in libhtgs_b200.so (C-ABI in include/htgs_b200.h).
"""
__version__ = "0.1.0"
