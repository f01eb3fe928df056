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


BENCH_SHAPES = [  # (queries, database rows, features, k): the benchmark configurations and the size limits
    (10_000, 1_000_000, 128, 10), (10_000, 1_000_000, 128, 100), (10_000, 12_500_000, 128, 10),
    (10_000, 100_000_000, 128, 10), (10_000, 1_000_000, 512, 10), (2_000_000, 2_000_000, 64, 16), (1, 1, 1, 1),
]


@pytest.mark.parametrize("nq,m,d,k", BENCH_SHAPES)
def test_size_queries_are_64_bit_and_aligned(nq, m, d, k):
    """Workspace and plane sizes are host arithmetic: positive, 256-byte multiples, no 32-bit wrap."""
    lib = _lib.load()
    plane = lib.fl_knn_plane_bytes(m, d)
    d_pad = (d + 15) // 16 * 16
    assert plane >= m * d_pad * 2 + m * 4 and plane % 256 == 0     # bf16 rows + fp32 half norms
    for mode in (_lib.FL_KNN_AUTO, _lib.FL_KNN_EXACT_SIMT, _lib.FL_KNN_BF16_RERANK):
        ws = lib.fl_knn_workspace_bytes(nq, m, d, k, mode)
        assert ws > 0 and ws % 256 == 0, (mode, ws, _lib.last_error())
        # more queries never need less
        assert lib.fl_knn_workspace_bytes(2 * nq, m, d, k, mode) >= ws
    assert lib.fl_knn_seed_floats(nq) >= 32 * nq
    assert lib.fl_knn_pack_ints(nq, k, 8, 0) >= 2 * nq * k


def test_auto_mode_takes_the_tensor_cores_for_the_benchmark_shapes():
    lib = _lib.load()
    assert lib.fl_knn_resolve_mode(10_000, 1_000_000, 128, 10) == _lib.FL_KNN_BF16_RERANK
    assert lib.fl_knn_resolve_mode(10_000, 1_000_000, 512, 10) == _lib.FL_KNN_BF16_RERANK
    assert lib.fl_knn_resolve_mode(1, 1, 1, 1) == _lib.FL_KNN_EXACT_SIMT
    assert lib.fl_knn_resolve_mode(10_000, 1_000_000, 1024, 10) == _lib.FL_KNN_EXACT_SIMT   # d > 512
