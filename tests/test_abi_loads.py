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
    assert ctypes.sizeof(_lib.Counters) == 24 * 8


def test_error_paths_without_a_gpu():
    handle = _lib.lib()
    assert handle.rgx_last_error(None) == b"null context"
    assert handle.rgx_workspace_bytes(None) == 0
    assert handle.rgx_create(0, None) == _lib.RGX_E_INVALID
