"""The C-ABI library loads and exports every symbol include/*.h declares.  No GPU needed."""
import ctypes
import glob
import os
import re

from conftest import ROOT
from hingetreefortorch_b200 import _build, _cabi


def declared_symbols():
    names = set()
    for header in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = open(header).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b(ht_[a-z0-9_]+)\s*\(", text))
    return names


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(_build.library_path())
    declared = declared_symbols()
    assert declared, "no declarations found"
    for name in declared:
        assert hasattr(lib, name), name
    assert declared == set(_cabi.SYMBOLS)


def test_status_strings_and_version():
    lib = _cabi.library()
    assert lib.ht_version() >= 100
    for status in range(0, -6, -1):
        assert lib.ht_status_string(status)
    assert b"unknown" in lib.ht_status_string(-99)


def test_workspace_query_and_argument_screening():
    lib = _cabi.library()
    p = _cabi.ForestProblem(0, 8, 1024, 128, 1, 1024, 1, 0, 0)
    need = lib.ht_forest_workspace_bytes(ctypes.byref(p))
    assert need >= 1024 * 255 * 4
    bad_depth = _cabi.ForestProblem(0, 32, 1, 1, 1, 1, 1, 0, 0)
    assert lib.ht_forest_workspace_bytes(ctypes.byref(bad_depth)) == 0
    # bad arguments are refused before anything touches a device
    rc = lib.ht_forest_forward_f32(ctypes.byref(bad_depth), None, None, None, None, None, None, ctypes.c_size_t(0), None, None)
    assert rc == -2
    rc = lib.ht_forest_forward_f32(ctypes.byref(p), None, None, None, None, None, None, ctypes.c_size_t(0), None, None)
    assert rc == -1
    rc = lib.ht_forest_forward_f32(None, None, None, None, None, None, None, ctypes.c_size_t(0), None, None)
    assert rc == -1
