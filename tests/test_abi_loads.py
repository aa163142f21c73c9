"""The C-ABI library loads and exports exactly what include/rgx.h declares (no compute calls)."""
import ctypes
import os
import re

from raygaussx_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "rgx.h")).read()
    return sorted(set(re.findall(r"RGX_API\s+[\w\s\*]+?\b(rgx_\w+)\s*\(", text)))


def test_header_and_binding_agree():
    names = declared_symbols()
    assert len(names) >= 12
    assert sorted(_lib.SYMBOLS) == names


def test_library_exports_every_declared_symbol():
    handle = _lib.lib()
    for name in declared_symbols():
        assert getattr(handle, name) is not None


def test_struct_layouts_match_the_header():
    # sizes implied by the field lists of include/rgx.h on LP64
    assert ctypes.sizeof(_lib.Scene) == 3 * 4 + 4 + 8 * 8          # three int32, padding, eight pointers
    assert ctypes.sizeof(_lib.Camera) == (3 * 4 + 2 + 2) * 4 + 2 * 4
    assert ctypes.sizeof(_lib.March) == 8 * 4
    assert ctypes.sizeof(_lib.Grads) == 8 * 8
    assert ctypes.sizeof(_lib.Counters) == 20 * 8


def test_error_paths_without_a_gpu():
    handle = _lib.lib()
    assert handle.rgx_last_error(None) == b"null context"
    assert handle.rgx_workspace_bytes(None) == 0
    assert handle.rgx_create(0, None) == _lib.RGX_E_INVALID


def test_misaligned_vector_loaded_tensors_are_refused_before_any_launch():
    """The kernels load quaternions (and 16-coefficient colour rows) 16 bytes at a time; a pointer off that
    boundary -- a row slice of a larger buffer -- must be turned down as an invalid argument on the host, not
    found out by a misaligned-address fault on the device.  rgx_forward_static validates before it touches
    CUDA, so the refusal can be checked without a GPU (the addresses below are never dereferenced)."""
    handle = _lib.lib()
    sc = _lib.Scene()
    sc.n, sc.sh_coeffs, sc.num_lobes = 8, 16, 0
    sc.positions, sc.scales, sc.densities = 0x10000, 0x20000, 0x30000
    sc.quaternions, sc.color_features = 0x40000 + 4, 0x50000          # quaternions[1:]-style offset
    cam = _lib.Camera()
    cam.width, cam.height = 4, 4
    m = _lib.March()
    m.dt_step, m.max_prim_slice, m.transmittance_eps, m.row_begin, m.row_end = 0.01, 16, 1e-3, 0, 4
    args = (0, ctypes.byref(sc), ctypes.byref(cam), ctypes.byref(m), ctypes.c_float(0.1), 0x60000, None, None, None)
    assert handle.rgx_forward_static(*args) == _lib.RGX_E_INVALID
    sc.quaternions, sc.color_features = 0x40000, 0x50000 + 8          # aligned quaternions, misaligned colour rows
    assert handle.rgx_forward_static(*args) == _lib.RGX_E_INVALID
    sc.n = 40000                                                      # size beyond the fixed scratch comes first
    assert handle.rgx_forward_static(*args) == _lib.RGX_E_TOO_LARGE
