"""The compiled torch extension modules of the rasterizer: `_C` and `_C_benchmarking`, with the function names and
signatures of the reference's pybind modules `HTGSCudaBackend._C` / `HTGSCudaBackend._C_benchmarking`
(torch_bindings/bindings.cpp:8-16, torch_bindings/bindings_benchmarking.cpp:6-8).  Built by `python -m htgs_b200.build`
from htgs_b200/csrc/bindings.cpp over libhtgs_b200.so.  The reference's own `torch_bindings/rasterization.py` runs unchanged
when these two modules stand in for its `_C` and `_C_benchmarking`.
"""
from __future__ import annotations


def load():
    """Returns (_C, _C_benchmarking), or raises ImportError when the modules have not been built."""
    import torch  # noqa: F401  (the modules link against torch's libraries)
    from . import _C, _C_benchmarking
    return _C, _C_benchmarking
