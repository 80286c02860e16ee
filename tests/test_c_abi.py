"""CPU: the shared library loads and exports every symbol include/htgs_b200.h declares; host-side
argument checks of the Python surface reject bad input before anything is launched."""
import ctypes

import pytest


def test_library_exports_all_declared_symbols():
    from htgs_b200 import _native, build
    build.build()
    lib = _native.lib()
    names = _native.exported_symbols()
    assert "htgs_render" in names and "htgs_create" in names and len(names) >= 8
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/htgs_b200.h but not exported"


def test_library_exports_nothing_the_header_does_not_declare():
    """The reverse direction: every `htgs_*` C symbol the library exports is declared in include/htgs_b200.h."""
    import subprocess
    from htgs_b200 import _native, build
    build.build()
    out = subprocess.run(["nm", "-D", "--defined-only", _native.LIB_PATH], stdout=subprocess.PIPE, text=True, check=True).stdout
    exported = {line.split()[-1] for line in out.splitlines() if len(line.split()) >= 3 and line.split()[-2] in ("T", "W")}
    c_symbols = {name for name in exported if name.startswith("htgs_")}          # C++ internals are mangled (_ZN4htgs...)
    declared = set(_native.exported_symbols())
    assert c_symbols, "nm found no htgs_* symbol: is the library stripped?"
    assert c_symbols <= declared, f"exported but not declared in the header: {sorted(c_symbols - declared)}"
    assert declared <= c_symbols, f"declared but not exported: {sorted(declared - c_symbols)}"


def test_version_and_error_string():
    from htgs_b200 import _native
    lib = _native.lib()
    assert lib.htgs_version() >= 100
    assert isinstance(_native.last_error(), str)


def test_surface_mirrors_reference_names():
    import htgs_b200.torch_bindings as tb
    for name in ("diff_rasterize", "rasterize", "fast_rasterize", "update_max_weights", "RasterizerSettings", "RasterizerMode"):
        assert hasattr(tb, name)
    assert [m.value for m in tb.RasterizerMode] == [0, 1, 2, 3]
    assert tb.RasterizerSettings._fields == ("M", "VPM", "cam_position", "mode", "K", "active_sh_bases", "width", "height",
                                              "near_plane", "far_plane", "scale_modifier")


def test_cpu_tensors_are_rejected():
    import torch
    import htgs_b200.torch_bindings as tb
    n = 4
    args = [torch.zeros(n, 3), torch.ones(n, 3), torch.zeros(n, 4), torch.ones(n, 1), torch.zeros(n, 1, 3), torch.zeros(n, 0, 3)]
    st = tb.RasterizerSettings(torch.eye(4), torch.eye(4), torch.zeros(3), tb.RasterizerMode.HYBRID_BLEND, 16, 1, 32, 32, 0.2, 100.0, 1.0)
    with pytest.raises(ValueError):
        tb.rasterize(*args, st, True, False)


def test_wrong_dtype_is_rejected():
    import torch
    from htgs_b200.torch_bindings import _C
    n = 4
    bad = [torch.zeros(n, 3, dtype=torch.float64), torch.ones(n, 3), torch.zeros(n, 4), torch.ones(n, 1), torch.zeros(n, 1, 3), torch.zeros(n, 0, 3)]
    with pytest.raises((TypeError, ValueError)):
        _C._check_inputs(*bad, torch.eye(4), torch.eye(4), torch.zeros(3))


def test_training_visibility_needs_tracking():
    """Asking for the visibility of a training forward that was never tracked is an error, not an empty answer."""
    import pytest
    from htgs_b200.torch_bindings import rasterization
    rasterization.track_training_visibility(False)
    with pytest.raises(RuntimeError):
        rasterization.last_training_visibility("cuda:0")


def test_extension_modules_expose_the_reference_entry_points():
    """The compiled torch extension modules import without a GPU and carry the names the reference's pybind modules bind
    (torch_bindings/bindings.cpp:8-16, bindings_benchmarking.cpp:6-8)."""
    from htgs_b200 import build
    build.build_bindings()
    from htgs_b200 import pybind
    mod_c, mod_b = pybind.load()
    for name in ("update_3d_filter_cuda", "forward", "backward", "render", "update_max_weights"):
        assert callable(getattr(mod_c, name)), name
    assert callable(mod_b.benchmark)
    assert [n for n in dir(mod_b) if not n.startswith("_")] == ["benchmark"]
    assert "arg18: bool) -> tuple[torch.Tensor, torch.Tensor]" in mod_c.render.__doc__      # 17 settings-order arguments + to_chw + use_median_depth


def test_instance_capacity_rounds_up_to_two_sizes_per_power_of_two():
    """`htgs_forward_instance_capacity` (host arithmetic only): never below the request, at most half more, stable under repetition,
    monotone, and only 2^k or 1.5 * 2^k above the floor of 4096."""
    import ctypes
    from htgs_b200 import _native
    lib = _native.lib()
    previous = 0
    for n in [0, 1, 4095, 4096, 4097, 6143, 6144, 6145, 8192, 8193, 1_000_000, 7_872_978, 12_582_912, 12_582_913, 150_000_000, 2**32 - 1]:
        c = int(lib.htgs_forward_instance_capacity(n))
        assert c >= max(n, 4096) and c >= previous
        assert c <= max(4096, n + n // 2 + 1)
        assert int(lib.htgs_forward_instance_capacity(c)) == c
        top = c.bit_length() - 1
        assert c in (1 << top, 3 << (top - 1))
        previous = c
