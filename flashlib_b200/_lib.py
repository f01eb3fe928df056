"""ctypes binding of ``libflashlib_b200.so`` (the C ABI in ``include/flashlib_b200.h``).

This module is the only place that touches the shared library.  There is no CPU
fallback: when the library has not been built, or when a call is made without an
sm_100 device, the call raises.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_int32, c_int64, c_void_p
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent / "lib" / "libflashlib_b200.so"

FL_OK = 0
FL_EINVAL = -1
FL_EUNSUPPORTED = -2
FL_ECUDA = -3
FL_ETIMEOUT = -4
FL_EWORKSPACE = -5

FL_KNN_AUTO = -1
FL_KNN_EXACT_SIMT = 0
FL_KNN_BF16_RERANK = 1

FL_STATUS_WORDS = 8
FL_STATUS_ERROR = 0
FL_STATUS_WHERE = 1
FL_STATUS_FALLBACK = 2
FL_STATUS_POOL = 3
FL_STATUS_STAGE2 = 4
FL_DTYPE_F32, FL_DTYPE_BF16, FL_DTYPE_F16 = 0, 1, 2

# name -> (restype, argtypes); mirrors include/flashlib_b200.h one to one.
SIGNATURES = {
    "fl_version": (c_int, []),
    "fl_last_error": (c_char_p, []),
    "fl_device_ok": (c_int, []),
    "fl_launch_count": (ctypes.c_ulonglong, []),
    "fl_profile_enable": (c_int, [c_int]),
    "fl_profile_count": (c_int, []),
    "fl_profile_read_ms": (c_int, [c_int, c_void_p]),
    "fl_rownorm_f32": (c_int, [c_void_p, c_int64, c_int, c_int64, c_void_p, c_void_p]),
    "fl_knn_plane_bytes": (c_int64, [c_int64, c_int]),
    "fl_knn_prepare_db_f32": (c_int, [c_void_p, c_int64, c_int, c_int64, c_void_p, c_int64, c_void_p]),
    "fl_knn_workspace_bytes": (c_int64, [c_int64, c_int64, c_int, c_int, c_int]),
    "fl_knn_f32": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int, c_int, c_int,
                           c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p]),
    "fl_knn_prepare_db_rows": (c_int, [c_void_p, c_int, c_int64, c_int, c_int64, c_void_p, c_int64, c_void_p]),
    "fl_knn_rows": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int, c_int, c_int, c_int,
                            c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p]),
    "fl_knn_batch_workspace_bytes": (c_int64, [c_int, c_int64, c_int64, c_int, c_int]),
    "fl_knn_batch_f32": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64, c_int, c_int,
                                 c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
    "fl_knn_split_plane_bytes": (c_int64, [c_int64, c_int]),
    "fl_knn_prepare_split_f32": (c_int, [c_void_p, c_int64, c_int, c_int64, c_void_p, c_int64, c_void_p]),
    "fl_knn_staged_workspace_bytes": (c_int64, [c_int64, c_int64, c_int, c_int]),
    "fl_knn_staged_f32": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int, c_int,
                                  c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p]),
    "fl_knn_seed_floats": (c_int64, [c_int64]),
    "fl_knn_seed_f32": (c_int, [c_void_p, c_int64, c_int64, c_int, c_int, c_void_p, c_int64, c_void_p,
                                c_void_p, c_int64, c_void_p, c_void_p]),
    "fl_knn_plane_maxnorm_offset": (c_int64, [c_int64, c_int]),
    "fl_knn_seeded_f32": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int, c_int,
                                  c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                  c_void_p, c_void_p]),
    "fl_debug_tc_experiment": (c_int, [c_int, ctypes.c_uint]),
    "fl_debug_tc_prof_read": (c_int, [c_void_p, c_int]),
    "fl_knn_resolve_mode": (c_int, [c_int64, c_int64, c_int, c_int]),
    "fl_debug_knn_tc_scores": (c_int, [c_void_p, c_int64, c_int64, c_int, c_void_p, c_int64, c_void_p, c_int64,
                                       c_void_p, c_int64, c_void_p, c_void_p]),
    "fl_topk_merge_f32": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "fl_knn_pack_ints": (c_int64, [c_int64, c_int, c_int, c_int]),
    "fl_knn_pack_f32": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "fl_knn_merge_packed_f32": (c_int, [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "fl_f32_to_bf16_down": (c_int, [c_void_p, c_void_p, c_int64, c_void_p]),
    "fl_bf16_to_f32": (c_int, [c_void_p, c_void_p, c_int64, c_void_p]),
    "fl_gather_l2sq_f32": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int,
                                   c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "fl_kmeans_assign_workspace_bytes": (c_int64, [c_int64, c_int, c_int]),
    "fl_kmeans_assign_f32": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int, c_int64, c_int,
                                     c_void_p, c_void_p, c_int64, c_void_p]),
    "fl_kmeans_xplane_bytes": (c_int64, [c_int64, c_int]),
    "fl_kmeans_prepare_x_f32": (c_int, [c_void_p, c_int64, c_int, c_int64, c_void_p, c_int64, c_void_p]),
    "fl_kmeans_assign_tc_workspace_bytes": (c_int64, [c_int64, c_int, c_int, c_int]),
    "fl_kmeans_assign_tc_f32": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_int, c_int64, c_int,
                                        c_void_p, c_void_p, c_int64, c_void_p, c_void_p]),
    "fl_kmeans_assign_noalloc_f32": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int, c_int64, c_int,
                                             c_void_p, c_void_p]),
    "fl_kmeans_update_f32": (c_int, [c_void_p, c_int64, c_int64, c_int, c_void_p, c_int,
                                     c_void_p, c_void_p, c_void_p]),
    "fl_kmeans_update_delta_f32": (c_int, [c_void_p, c_int64, c_int64, c_int, c_void_p, c_void_p, c_int,
                                           c_void_p, c_void_p, c_void_p]),
    "fl_kmeans_assign_batch_workspace_bytes": (c_int64, [c_int, c_int64, c_int, c_int]),
    "fl_kmeans_assign_batch_f32": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_int, c_int64, c_int64,
                                           c_int, c_void_p, c_void_p, c_int64, c_void_p]),
    "fl_kmeans_update_batch_f32": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int, c_void_p, c_int,
                                           c_void_p, c_void_p, c_void_p]),
    "fl_kmeans_finalize_f32": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                       c_void_p]),
    "fl_ivf_fine_scan_workspace_bytes": (c_int64, [c_int64, c_int, c_int, c_int64, c_int, c_int]),
    "fl_ivf_fine_scan_f32": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int,
                                     c_void_p, c_int, c_void_p, c_int, c_int, c_void_p,
                                     c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
    "fl_ivf_build_workspace_bytes": (c_int64, [c_int64, c_int]),
    "fl_ivf_build_csr_f32": (c_int, [c_void_p, c_int64, c_int64, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                     c_void_p, c_void_p, c_int64, c_void_p]),
    "fl_ivf_map_ids": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p]),
    "fl_ivf_plane_bytes": (c_int64, [c_int64, c_int, c_int]),
    "fl_ivf_prepare_f32": (c_int, [c_void_p, c_int64, c_int64, c_int, c_void_p, c_int, c_void_p, c_int64, c_void_p]),
    "fl_ivf_fine_scan_tc_workspace_bytes": (c_int64, [c_int64, c_int, c_int, c_int64, c_int, c_int]),
    "fl_ivf_fine_scan_tc_f32": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int,
                                        c_void_p, c_int, c_void_p, c_int, c_int, c_void_p,
                                        c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p]),
}

_lib = None


class FlashlibError(RuntimeError):
    """A call into libflashlib_b200.so failed (CUDA error, timeout or workspace problem)."""


def lib_path() -> Path:
    return _LIB_PATH


def load() -> ctypes.CDLL:
    """Load the shared library (once) and declare every entry point's signature."""
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists():
        raise RuntimeError(
            f"{_LIB_PATH} is missing: build it with `python -m flashlib_b200._build` "
            "(flashlib_b200 has no CPU or PyTorch fallback)")
    lib = ctypes.CDLL(str(_LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def last_error() -> str:
    msg = load().fl_last_error()
    return msg.decode("utf-8", "replace") if msg else ""


def check(rc: int, what: str = "") -> None:
    """Map a C status code to the exception type the reference raises for that case."""
    if rc == FL_OK:
        return
    msg = last_error() or what or f"flashlib_b200 call failed with code {rc}"
    if rc == FL_EINVAL:
        raise ValueError(msg)
    if rc == FL_EUNSUPPORTED:
        raise NotImplementedError(msg)
    raise FlashlibError(msg)


def require_device() -> None:
    """Raise unless an sm_100 device is visible; there is nothing to fall back to."""
    if not load().fl_device_ok():
        raise RuntimeError("flashlib_b200 needs an NVIDIA B200 (sm_100) device; "
                           "no CPU or other-GPU fallback exists")
