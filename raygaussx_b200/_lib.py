"""ctypes binding of librgx.so (the C ABI declared in include/rgx.h).

There is no fallback: if the library is missing or fails to load, importing
this module's :func:`lib` raises.  Build it with ``python -m raygaussx_b200.build``.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# the in-tree build; RGX_LIBRARY names another build of the same library (a differently tuned one, say)
LIB_PATH = os.environ.get("RGX_LIBRARY") or os.path.join(_HERE, "librgx.so")

RGX_OK, RGX_E_INVALID, RGX_E_CUDA, RGX_E_NOT_BUILT, RGX_E_TOO_LARGE = 0, -1, -2, -3, -4
CURVE_MORTON, CURVE_HILBERT = 0, 1
FLAG_COUNT_WORK, FLAG_BRUTE_FORCE, FLAG_EXACT_SH_GRAD, FLAG_ACCUMULATE, FLAG_PER_RAY_SEARCH, FLAG_SAVE_HITS = 1, 2, 4, 8, 16, 32

_fp = C.c_void_p  # device pointers travel as integers


class Scene(C.Structure):
    _fields_ = [("n", C.c_int32), ("sh_coeffs", C.c_int32), ("num_lobes", C.c_int32),
                ("positions", _fp), ("scales", _fp), ("quaternions", _fp), ("densities", _fp),
                ("color_features", _fp), ("sg_features", _fp), ("sharpness", _fp), ("lobe_axis", _fp)]


class Camera(C.Structure):
    _fields_ = [("eye", C.c_float * 3), ("u", C.c_float * 3), ("v", C.c_float * 3), ("w", C.c_float * 3),
                ("tan_half_fov", C.c_float * 2), ("pp", C.c_float * 2), ("width", C.c_int32), ("height", C.c_int32)]


class March(C.Structure):
    _fields_ = [("dt_step", C.c_float), ("dynamic_sampling", C.c_int32), ("max_prim_slice", C.c_int32),
                ("white_background", C.c_int32), ("transmittance_eps", C.c_float), ("row_begin", C.c_int32),
                ("row_end", C.c_int32), ("flags", C.c_int32)]


class Grads(C.Structure):
    _fields_ = [("positions", _fp), ("scales", _fp), ("quaternions", _fp), ("densities", _fp),
                ("color_features", _fp), ("sg_features", _fp), ("sharpness", _fp), ("lobe_axis", _fp)]


class Counters(C.Structure):
    _fields_ = [(k, C.c_uint64) for k in ("rays", "slabs", "slabs_hit", "closest_queries", "hits", "pairs_inside",
                                          "overflow_slabs", "node_tests", "prim_tests", "ellipsoid_tests",
                                          "stack_overflows", "hits_hash", "candidates", "cycles_window", "cycles_seek",
                                          "cycles_search", "cycles_eval", "cycles_composite", "cycles_wait",
                                          "cycles_total")]

    def as_dict(self):
        return {k: int(getattr(self, k)) for k, _ in self._fields_}


# every symbol include/rgx.h declares: name -> (restype, argtypes)
SYMBOLS = {
    "rgx_create": (C.c_int, [C.c_int, C.POINTER(C.c_void_p)]),
    "rgx_destroy": (None, [C.c_void_p]),
    "rgx_last_error": (C.c_char_p, [C.c_void_p]),
    "rgx_build": (C.c_int, [C.c_void_p, C.POINTER(Scene), C.c_float, C.c_int, C.c_int, C.c_void_p]),
    "rgx_forward": (C.c_int, [C.c_void_p, C.POINTER(Scene), C.POINTER(Camera), C.POINTER(March), _fp, _fp, _fp,
                              C.c_void_p]),
    "rgx_forward_frame": (C.c_int, [C.c_void_p, C.POINTER(Scene), C.POINTER(Camera), C.POINTER(March), _fp, _fp,
                                    C.c_void_p]),
    "rgx_backward": (C.c_int, [C.c_void_p, C.POINTER(Scene), C.POINTER(Camera), C.POINTER(March), _fp, _fp,
                               C.POINTER(Grads), C.c_void_p]),
    "rgx_hint_next_view": (C.c_int, [C.c_void_p, C.POINTER(Camera), C.POINTER(March)]),
    "rgx_lists_made_ahead": (C.c_int, [C.c_void_p]),
    "rgx_gaussian_colors": (C.c_int, [C.c_void_p, C.POINTER(Scene), C.POINTER(C.c_float), _fp, C.c_void_p]),
    "rgx_scene_box": (C.c_int, [C.c_void_p, C.POINTER(C.c_float), C.POINTER(C.c_float), C.c_void_p]),
    "rgx_debug_fail_allocation": (C.c_int, [C.c_void_p, C.c_int]),
    "rgx_debug_cap_recording": (C.c_int, [C.c_void_p, C.c_longlong]),
    "rgx_debug_two_depth": (C.c_int, [C.c_void_p, C.c_int, C.c_int]),
    "rgx_read_two_depth": (C.c_int, [C.c_void_p, C.POINTER(C.c_longlong)]),
    "rgx_debug_near_lists": (C.c_int, [C.c_void_p, C.c_int, C.c_longlong]),
    "rgx_read_near_lists": (C.c_int, [C.c_void_p, C.POINTER(C.c_longlong)]),
    "rgx_measure_peaks": (C.c_int, [C.c_int, C.POINTER(C.c_float), C.POINTER(C.c_float)]),
    "rgx_knn_mean_dist2": (C.c_int, [C.c_int, _fp, C.c_int, _fp, C.c_void_p]),
    "rgx_reset_counters": (C.c_int, [C.c_void_p, C.c_void_p]),
    "rgx_read_counters": (C.c_int, [C.c_void_p, C.POINTER(Counters), C.c_void_p]),
    "rgx_workspace_bytes": (C.c_size_t, [C.c_void_p]),
    "rgx_kernel_launches": (C.c_ulonglong, []),
    "rgx_forward_static": (C.c_int, [C.c_int, C.POINTER(Scene), C.POINTER(Camera), C.POINTER(March), C.c_float, _fp, _fp,
                                     _fp, C.c_void_p]),
    "rgx_set_profiling": (C.c_int, [C.c_void_p, C.c_int]),
    "rgx_read_binning": (C.c_int, [C.c_void_p, C.POINTER(C.c_float), C.POINTER(C.c_int), C.POINTER(C.c_longlong)]),
    "rgx_read_kernel_times": (C.c_int, [C.c_void_p, C.POINTER(C.c_float), C.POINTER(C.c_int), C.POINTER(C.c_float),
                                        C.POINTER(C.c_int)]),
}

_lib = None


def lib():
    """The loaded library with argument types set.  Raises if it is not built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: run `python -m raygaussx_b200.build` (needs nvcc); "
                               "there is no fallback path")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(handle, name)   # AttributeError if the symbol is not exported
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


class RgxError(RuntimeError):
    def __init__(self, code, message):
        super().__init__(f"rgx error {code}: {message}")
        self.code = code


def check(ctx, code):
    if code != RGX_OK:
        msg = lib().rgx_last_error(ctx)
        raise RgxError(code, msg.decode() if msg else "")
