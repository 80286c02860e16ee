"""ctypes binding of libhtgs_b200.so (the C-ABI declared in include/htgs_b200.h).

The library is the product: there is no CPU or PyTorch fallback.  Importing this
module without the built library, or using it without a B200, raises.
"""
from __future__ import annotations

import ctypes
import os
import threading
from typing import Dict, Optional

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("HTGS_B200_LIB") or os.path.join(_HERE, "libhtgs_b200.so")

HTGS_OK = 0
HTGS_ERR_INVALID_ARGUMENT = 1
HTGS_ERR_UNSUPPORTED_MODE = 2
HTGS_ERR_WORKSPACE_TOO_SMALL = 3
HTGS_ERR_CUDA = 4
HTGS_ERR_DEVICE_FLAG = 5


class HtgsScene(ctypes.Structure):
    _fields_ = [
        ("positions", ctypes.c_void_p), ("scales", ctypes.c_void_p), ("rotations", ctypes.c_void_p),
        ("opacities", ctypes.c_void_p), ("sh_0", ctypes.c_void_p), ("sh_rest", ctypes.c_void_p),
        ("n_primitives", ctypes.c_int32), ("total_sh_bases", ctypes.c_int32),
    ]


class HtgsRowTensors(ctypes.Structure):
    _fields_ = [("data", ctypes.c_void_p * 8), ("width", ctypes.c_int32 * 8), ("n_tensors", ctypes.c_int32)]


class HtgsView(ctypes.Structure):
    _fields_ = [
        ("M", ctypes.c_void_p), ("VPM", ctypes.c_void_p), ("cam_position", ctypes.c_void_p),
        ("mode", ctypes.c_int32), ("K", ctypes.c_int32), ("active_sh_bases", ctypes.c_int32),
        ("width", ctypes.c_int32), ("height", ctypes.c_int32),
        ("near_plane", ctypes.c_float), ("far_plane", ctypes.c_float), ("scale_modifier", ctypes.c_float),
    ]


class HtgsFrameInfo(ctypes.Structure):
    _fields_ = [
        ("n_instances", ctypes.c_uint32), ("n_visible", ctypes.c_uint32), ("key_bytes", ctypes.c_uint32),
        ("end_bit", ctypes.c_uint32), ("reruns", ctypes.c_uint32), ("device_error", ctypes.c_uint32),
        ("kernel_launches", ctypes.c_uint32), ("reserved", ctypes.c_uint32),
        ("workspace_bytes", ctypes.c_uint64), ("candidate_pairs", ctypes.c_uint64), ("accepted_fragments", ctypes.c_uint64),
        ("warp_trips", ctypes.c_uint64), ("warp_trips_inserting", ctypes.c_uint64), ("lane_insertions", ctypes.c_uint64),
    ]


class HtgsIntermediates(ctypes.Structure):
    _fields_ = [
        ("n_touched", ctypes.c_void_p), ("bounds", ctypes.c_void_p), ("eval_records", ctypes.c_void_p),
        ("cull_records", ctypes.c_void_p), ("keys_unsorted", ctypes.c_void_p), ("prims_unsorted", ctypes.c_void_p),
        ("keys_sorted", ctypes.c_void_p), ("prims_sorted", ctypes.c_void_p), ("tile_ranges", ctypes.c_void_p),
        ("n_tiles", ctypes.c_uint32), ("grid_width", ctypes.c_uint32), ("grid_height", ctypes.c_uint32),
        ("key_bytes", ctypes.c_uint32),
    ]


class HtgsTrainBlobs(ctypes.Structure):
    _fields_ = [
        ("per_primitive", ctypes.c_void_p), ("per_primitive_bytes", ctypes.c_size_t),
        ("per_tile", ctypes.c_void_p), ("per_tile_bytes", ctypes.c_size_t),
        ("per_instance", ctypes.c_void_p), ("per_instance_bytes", ctypes.c_size_t),
        ("per_pixel", ctypes.c_void_p), ("per_pixel_bytes", ctypes.c_size_t),
    ]


class HtgsGradients(ctypes.Structure):
    _fields_ = [
        ("grad_positions", ctypes.c_void_p), ("grad_scales", ctypes.c_void_p), ("grad_rotations", ctypes.c_void_p),
        ("grad_opacities", ctypes.c_void_p), ("grad_sh_0", ctypes.c_void_p), ("grad_sh_rest", ctypes.c_void_p),
        ("scratch", ctypes.c_void_p), ("scratch_bytes", ctypes.c_size_t),
        ("densification_info", ctypes.c_void_p), ("densification_rows", ctypes.c_int32), ("use_distance_scaling", ctypes.c_int32),
    ]


class HtgsFilterView(ctypes.Structure):
    _fields_ = [("w2c", ctypes.c_float * 16), ("width", ctypes.c_int32), ("height", ctypes.c_int32), ("focal_x", ctypes.c_float),
                ("focal_y", ctypes.c_float), ("center_x", ctypes.c_float), ("center_y", ctypes.c_float), ("near_plane", ctypes.c_float)]


class HtgsError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(message)
        self.code = code


_lib = None
_lib_lock = threading.Lock()


def lib():
    """Loads the shared library (once).  Fails loudly if it has not been built."""
    global _lib
    if _lib is None:
        with _lib_lock:
            if _lib is None:
                if not os.path.exists(LIB_PATH):
                    raise ImportError(
                        f"{LIB_PATH} is missing: build it with `python -m htgs_b200.build` (needs nvcc). "
                        "htgs_b200 has no CPU or PyTorch fallback.")
                l = ctypes.CDLL(LIB_PATH)
                l.htgs_create.restype = ctypes.c_void_p
                l.htgs_create.argtypes = [ctypes.c_int]
                l.htgs_destroy.argtypes = [ctypes.c_void_p]
                l.htgs_last_error.restype = ctypes.c_char_p
                l.htgs_render_workspace_bytes.restype = ctypes.c_size_t
                l.htgs_render_workspace_bytes.argtypes = [ctypes.POINTER(HtgsScene), ctypes.POINTER(HtgsView), ctypes.c_uint64]
                l.htgs_render.restype = ctypes.c_int
                l.htgs_render.argtypes = [ctypes.c_void_p, ctypes.POINTER(HtgsScene), ctypes.POINTER(HtgsView), ctypes.c_void_p, ctypes.c_void_p,
                                          ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p,
                                          ctypes.POINTER(HtgsFrameInfo)]
                l.htgs_render_async.restype = ctypes.c_int
                l.htgs_render_async.argtypes = [ctypes.c_void_p, ctypes.POINTER(HtgsScene), ctypes.POINTER(HtgsView), ctypes.c_void_p, ctypes.c_void_p,
                                                ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
                l.htgs_render_fast_async.argtypes = [ctypes.c_void_p, ctypes.POINTER(HtgsScene), ctypes.POINTER(HtgsView), ctypes.c_void_p, ctypes.c_int,
                                                     ctypes.c_void_p]
                l.htgs_frame_result.argtypes = [ctypes.c_void_p, ctypes.POINTER(HtgsFrameInfo)]
                l.htgs_set_max_weights_tail_credit.argtypes = [ctypes.c_void_p, ctypes.c_int]
                l.htgs_render_host.restype = ctypes.c_int
                l.htgs_render_host.argtypes = [ctypes.c_void_p, ctypes.POINTER(HtgsScene), ctypes.POINTER(HtgsView), ctypes.c_void_p, ctypes.c_void_p,
                                               ctypes.c_int, ctypes.c_int, ctypes.POINTER(HtgsFrameInfo)]
                l.htgs_get_intermediates.restype = ctypes.c_int
                l.htgs_get_intermediates.argtypes = [ctypes.c_void_p, ctypes.POINTER(HtgsIntermediates)]
                l.htgs_forward_blob_sizes.argtypes = [ctypes.POINTER(HtgsScene), ctypes.POINTER(HtgsView), ctypes.POINTER(ctypes.c_size_t),
                                                      ctypes.POINTER(ctypes.c_size_t), ctypes.POINTER(ctypes.c_size_t)]
                l.htgs_forward_instance_capacity.restype = ctypes.c_uint64
                l.htgs_forward_instance_capacity.argtypes = [ctypes.c_uint64]
                l.htgs_forward_instance_bytes.restype = ctypes.c_size_t
                l.htgs_forward_instance_bytes.argtypes = [ctypes.POINTER(HtgsView), ctypes.c_uint64]
                l.htgs_forward_begin.argtypes = [ctypes.c_void_p, ctypes.POINTER(HtgsScene), ctypes.POINTER(HtgsView), ctypes.c_void_p, ctypes.c_size_t,
                                                 ctypes.c_void_p, ctypes.POINTER(ctypes.c_uint32)]
                l.htgs_forward_finish.argtypes = [ctypes.c_void_p, ctypes.POINTER(HtgsScene), ctypes.POINTER(HtgsView), ctypes.POINTER(HtgsTrainBlobs),
                                                  ctypes.c_uint32, ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(HtgsFrameInfo)]
                l.htgs_backward_scratch_bytes.restype = ctypes.c_size_t
                l.htgs_backward_scratch_bytes.argtypes = [ctypes.POINTER(HtgsScene)]
                l.htgs_backward.argtypes = [ctypes.c_void_p, ctypes.POINTER(HtgsScene), ctypes.POINTER(HtgsView), ctypes.POINTER(HtgsTrainBlobs),
                                            ctypes.c_uint32, ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(HtgsGradients), ctypes.c_void_p]
                l.htgs_backward_static.argtypes = l.htgs_backward.argtypes
                l.htgs_backward_range.argtypes = l.htgs_backward.argtypes[:8] + [ctypes.c_uint32, ctypes.c_uint32, ctypes.c_void_p]
                l.htgs_backward_accumulate.argtypes = l.htgs_backward.argtypes
                l.htgs_backward_finish_range.argtypes = [ctypes.c_void_p, ctypes.POINTER(HtgsScene), ctypes.POINTER(HtgsView), ctypes.POINTER(HtgsTrainBlobs),
                                                         ctypes.POINTER(HtgsGradients), ctypes.c_uint32, ctypes.c_uint32, ctypes.c_void_p]
                l.htgs_compact_rows_bytes.restype = ctypes.c_size_t
                l.htgs_compact_rows_bytes.argtypes = [ctypes.c_uint32]
                l.htgs_backward_compact.argtypes = l.htgs_backward.argtypes[:8] + [ctypes.c_void_p, ctypes.c_uint32, ctypes.c_void_p]
                l.htgs_expand_add_rows.argtypes = [ctypes.POINTER(HtgsScene), ctypes.c_void_p, ctypes.c_uint32, ctypes.POINTER(HtgsGradients), ctypes.c_void_p]
                l.htgs_expand_sum_scratch_bytes.restype = ctypes.c_size_t
                l.htgs_expand_sum_scratch_bytes.argtypes = [ctypes.POINTER(HtgsScene), ctypes.c_int]
                l.htgs_expand_sum_rows.argtypes = [ctypes.POINTER(HtgsScene), ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.c_uint32, ctypes.c_void_p,
                                                   ctypes.c_size_t, ctypes.POINTER(HtgsGradients), ctypes.c_void_p]
                l.htgs_copy_rows.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint32, ctypes.c_void_p]
                l.htgs_peer_buffer_create.argtypes = [ctypes.c_int, ctypes.c_size_t, ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p]
                l.htgs_peer_buffer_open.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p)]
                l.htgs_peer_buffer_close.argtypes = [ctypes.c_int, ctypes.c_void_p]
                l.htgs_peer_buffer_destroy.argtypes = [ctypes.c_int, ctypes.c_void_p]
                l.htgs_gather_rows.argtypes = [ctypes.POINTER(HtgsRowTensors), ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p]
                l.htgs_scatter_rows.argtypes = l.htgs_gather_rows.argtypes
                l.htgs_forward_visibility.argtypes = [ctypes.POINTER(HtgsScene), ctypes.POINTER(HtgsTrainBlobs), ctypes.c_void_p, ctypes.c_void_p]
                l.htgs_update_max_weights.argtypes = [ctypes.c_void_p, ctypes.POINTER(HtgsScene), ctypes.POINTER(HtgsView), ctypes.c_void_p, ctypes.c_float,
                                                      ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p, ctypes.POINTER(HtgsFrameInfo)]
                l.htgs_render_fast.argtypes = [ctypes.c_void_p, ctypes.POINTER(HtgsScene), ctypes.POINTER(HtgsView), ctypes.c_void_p, ctypes.c_int,
                                               ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p, ctypes.POINTER(HtgsFrameInfo)]
                l.htgs_update_3d_filter.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32,
                                                    ctypes.c_int32] + [ctypes.c_float] * 7 + [ctypes.c_void_p]
                l.htgs_update_3d_filter_views.argtypes = [ctypes.c_void_p, ctypes.POINTER(HtgsFilterView), ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p,
                                                          ctypes.c_int32, ctypes.c_float, ctypes.c_float, ctypes.c_void_p]
                l.htgs_activate.argtypes = [ctypes.c_void_p] * 7 + [ctypes.c_int32, ctypes.c_void_p]
                l.htgs_activate_backward.argtypes = [ctypes.c_void_p] * 10 + [ctypes.c_int32, ctypes.c_void_p]
                l.htgs_set_profiling.argtypes = [ctypes.c_void_p, ctypes.c_int]
                l.htgs_set_collect_stats.argtypes = [ctypes.c_void_p, ctypes.c_int]
                l.htgs_set_fast_deterministic.argtypes = [ctypes.c_void_p, ctypes.c_int]
                l.htgs_set_front_priority.argtypes = [ctypes.c_void_p, ctypes.c_int]
                l.htgs_get_stage_ms.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_float)]
                l.htgs_memcpy_d2h.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t]
                l.htgs_memcpy_h2d.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t]
                _lib = l
    return _lib


def last_error() -> str:
    msg = lib().htgs_last_error()
    return msg.decode("utf-8", "replace") if msg else ""


def check(code: int) -> None:
    if code != HTGS_OK:
        msg = last_error()
        if code == HTGS_ERR_UNSUPPORTED_MODE:
            raise RuntimeError(msg or "unsupported rasterizer mode")
        raise HtgsError(code, f"htgs_b200 error {code}: {msg}")


_contexts: Dict[tuple, int] = {}
_ctx_lock = threading.Lock()

# Which binding serves the Python surface: the compiled torch extension modules (htgs_b200/pybind, the default when they
# have been built) or this ctypes binding (no compile step beyond the core library).  HTGS_B200_BINDING=pybind|ctypes|auto.
_pybind_modules = None


def pybind_modules():
    """(_C, _C_benchmarking) of htgs_b200.pybind when they are the active binding, else None."""
    global _pybind_modules
    if _pybind_modules is None:
        choice = os.environ.get("HTGS_B200_BINDING", "auto").lower()
        if choice not in ("auto", "pybind", "ctypes"):
            raise ValueError("HTGS_B200_BINDING must be auto, pybind or ctypes")
        _pybind_modules = False
        if choice != "ctypes":
            try:
                from . import pybind
                _pybind_modules = pybind.load()
            except ImportError:
                if choice == "pybind":
                    raise
    return _pybind_modules or None


def active_binding() -> str:
    return "pybind" if pybind_modules() else "ctypes"



def context(device_index: int, stream: int = 0) -> int:
    """One library context per (CUDA device, host thread, stream key) of this process, created on first use.  A context owns
    its workspace and its pinned status word, so two frames that are in flight at once - two host threads rendering
    concurrently, or one thread queueing frames on two CUDA streams without waiting (`htgs_render_async`) - must not share
    one.  Blocking calls pass no stream key and share the thread's context; the non-blocking path passes the handle of the
    stream it queues on."""
    mods = pybind_modules()
    if mods:     # both bindings use one set of contexts: the extension module's (per host thread, like this table)
        return mods[0].context_handle(int(device_index), int(stream))
    key = (int(device_index), threading.get_ident(), int(stream))
    ctx = _contexts.get(key)
    if ctx is None:
        with _ctx_lock:
            ctx = _contexts.get(key)
            if ctx is None:
                ctx = lib().htgs_create(int(device_index))
                if not ctx:
                    raise RuntimeError(f"htgs_create({device_index}) failed: {last_error()}")
                _contexts[key] = ctx
    return ctx


def contexts_of_thread(device_index: Optional[int] = None):
    """Contexts the calling host thread has created (on one device, or on all)."""
    mods = pybind_modules()
    if mods:
        return list(mods[0].context_handles(-1 if device_index is None else int(device_index)))
    me = threading.get_ident()
    with _ctx_lock:
        return [ctx for (dev, thread, _), ctx in _contexts.items() if thread == me and (device_index is None or dev == int(device_index))]


def exported_symbols():
    """Names include/htgs_b200.h declares; used by the CPU-side test that the library exports them all."""
    import re
    header = os.path.join(os.path.dirname(_HERE), "include", "htgs_b200.h")
    text = open(header).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(htgs_[a-z0-9_]+)\s*\(", text)))
