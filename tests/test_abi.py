"""The shared library loads without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

import pytest

from flashlib_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "flashlib_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fl_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    assert declared_symbols() == sorted(_lib.SIGNATURES)


def test_library_exports_every_symbol():
    lib = ctypes.CDLL(str(_lib.lib_path()))
    for name in declared_symbols():
        assert hasattr(lib, name), name


def test_version_and_queries_without_gpu():
    lib = _lib.load()
    assert lib.fl_version() >= 100
    assert lib.fl_knn_plane_bytes(1000, 128) >= 1024 * 128 * 2 + 1024 * 4
    assert lib.fl_knn_workspace_bytes(100, 1000, 64, 10, _lib.FL_KNN_EXACT_SIMT) > 0
    assert lib.fl_kmeans_assign_workspace_bytes(1000, 64, 32) >= 64 * 4
    assert lib.fl_ivf_fine_scan_workspace_bytes(100, 4, 32, 5000, 32, 10) > 0


def test_bad_arguments_map_to_exceptions():
    lib = _lib.load()
    rc = lib.fl_knn_f32(None, 10, 8, None, 100, 8, 8, 0, 0, None, 0, None, None, None, 0, None, None)
    assert rc == _lib.FL_EINVAL
    with pytest.raises(ValueError):
        _lib.check(rc)
    assert "k must be" in _lib.last_error()
    rc = lib.fl_knn_f32(None, 10, 8, None, 100, 8, 8, 600, 0, None, 0, None, None, None, 0, None, None)
    assert rc == _lib.FL_EINVAL  # k > m
    rc = lib.fl_knn_f32(None, 10, 8, None, 1000, 8, 8, 600, 0, None, 0, None, None, None, 0, None, None)
    with pytest.raises(NotImplementedError):
        _lib.check(rc)
