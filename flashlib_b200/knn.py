"""Fused exact brute-force kNN behind flashlib's ``flash_knn`` signature.

Mirrors ``flashlib/primitives/knn/impl.py:199-287`` (``flash_knn_dispatch``): same
arguments, same return dtypes on CUDA (``vals`` fp32 true squared L2, ``idxs`` int32),
same error behaviour for unknown backends.  The reference's multi-backend routing is
gone: every call goes through the C ABI into the sm_100a kernels, and CPU tensors are
rejected because this library has no CPU path.
"""
from __future__ import annotations

import os
import weakref
from collections import OrderedDict, deque
from typing import Optional

import torch

from . import _lib

_VALID_BACKENDS = ("triton", "cutedsl", "torch")
_MODES = {None: _lib.FL_KNN_AUTO, "auto": _lib.FL_KNN_AUTO, "exact": _lib.FL_KNN_EXACT_SIMT,
          "simt": _lib.FL_KNN_EXACT_SIMT, "bf16": _lib.FL_KNN_BF16_RERANK,
          "tc": _lib.FL_KNN_BF16_RERANK}


def _stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _as_f32_rows(t: torch.Tensor) -> torch.Tensor:
    """fp32 tensor whose last dimension is contiguous (rows may be strided)."""
    if t.dtype != torch.float32:
        t = t.float()
    if t.stride(-1) != 1 or (t.dim() == 2 and t.stride(0) < t.shape[1]):
        t = t.contiguous()
    return t


_DTYPE_CODES = {torch.float32: _lib.FL_DTYPE_F32, torch.bfloat16: _lib.FL_DTYPE_BF16, torch.float16: _lib.FL_DTYPE_F16}


def _as_rows(t: torch.Tensor) -> torch.Tensor:
    """Rows the kernels read as they are: fp32, bf16 or fp16 (anything else is converted to fp32),
    last dimension contiguous."""
    if t.dtype not in _DTYPE_CODES:
        t = t.float()
    if t.stride(-1) != 1 or (t.dim() == 2 and t.stride(0) < t.shape[1]):
        t = t.contiguous()
    return t


# Restatement of the reference's tol -> storage dtype rule (flashlib/linalg/gemm/__init__.py:114-207):
# among the GEMM variants whose declared residual is <= tol the one with the highest listed throughput
# is chosen, and only "fp16" / "bf16" name a storage dtype.  fp16 (residual 4e-4, 892 TF) beats bf16
# (3e-3, 816 TF) whenever both qualify, and tf32 (3e-4, 386 TF) qualifies alone below 4e-4.
_TOL_VARIANTS = (("fp16", 4e-4, 892.0, torch.float16), ("bf16", 3e-3, 816.0, torch.bfloat16), ("tf32", 3e-4, 386.0, None))


def storage_dtype_for(tol: Optional[float]):
    """16-bit dtype the inputs may be stored in for this ``tol`` (``None``: keep them as given)."""
    if tol is None or tol <= 0:
        return None
    ok = [v for v in _TOL_VARIANTS if v[1] <= tol]
    if not ok:
        return None
    return max(ok, key=lambda v: v[2])[3]


_CAST_CACHE: "OrderedDict[tuple, torch.Tensor]" = OrderedDict()


def _cast_rows_cached(c: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """``c.to(dtype)``, kept while ``c`` is alive and unchanged: the database is stored in 16 bits once,
    and its operand plane is found again on the next call."""
    key = _plane_key(c) + (dtype,)
    hit = _CAST_CACHE.get(key)
    if hit is not None:
        _CAST_CACHE.move_to_end(key)
        return hit
    out = c.to(dtype)
    _CAST_CACHE[key] = out
    _evict_when_freed(_CAST_CACHE, key, c)
    while len(_CAST_CACHE) > _PLANE_CACHE_SIZE:
        _CAST_CACHE.popitem(last=False)
    return out


def _mode_from(mode: Optional[str]) -> int:
    if mode is None:
        mode = os.environ.get("FLASHLIB_B200_KNN_MODE") or None
    if mode not in _MODES:
        raise ValueError(f"mode must be one of {sorted(k for k in _MODES if k)} or None, got {mode!r}")
    return _MODES[mode]


class DbPlane:
    """The bf16 operand plane (+ half norms) of one fp32 database, built once per database.

    The reference caches ``||c||^2`` per ``data_ptr`` in the same spirit
    (``flashlib/primitives/knn/triton/_row_norm.py:82-93``).
    """

    def __init__(self, db: torch.Tensor):
        lib = _lib.load()
        m, d = db.shape
        nbytes = lib.fl_knn_plane_bytes(m, d)
        self.buf = torch.empty(nbytes, dtype=torch.uint8, device=db.device)
        _lib.check(lib.fl_knn_prepare_db_rows(db.data_ptr(), _DTYPE_CODES[db.dtype], m, d, db.stride(0),
                                              self.buf.data_ptr(), nbytes, _stream_ptr(db.device)))
        self.key = _plane_key(db)
        self.split_buf = None

    @property
    def ptr(self) -> int:
        return self.buf.data_ptr()

    def split_ptr(self, db: torch.Tensor):
        """Address of the split (hi/lo bf16) plane of the same database, built on first use; ``None``
        when the shape has none (d > 128) or it would exceed the size limit."""
        if self.split_buf is None:
            lib = _lib.load()
            m, d = db.shape
            nbytes = lib.fl_knn_split_plane_bytes(m, d) if db.dtype == torch.float32 else 0
            if nbytes == 0 or nbytes > _split_plane_limit():
                self.split_buf = False
            else:
                self.split_buf = torch.empty(nbytes, dtype=torch.uint8, device=db.device)
                _lib.check(lib.fl_knn_prepare_split_f32(db.data_ptr(), m, d, db.stride(0), self.split_buf.data_ptr(),
                                                        nbytes, _stream_ptr(db.device)))
        return self.split_buf.data_ptr() if self.split_buf is not False else None


def _split_plane_limit() -> int:
    """Largest split plane (bytes) built without being asked for: it takes 6.25x the fp32 rows'
    memory at d = 128 -> on for databases of a few million rows, off for the 100M-row shards."""
    return int(os.environ.get("FLASHLIB_B200_SPLIT_MAX_MB", "4096")) << 20


def _second_stage_default() -> bool:
    return os.environ.get("FLASHLIB_B200_KNN_STAGE2", "1") != "0"


def _plane_key(db: torch.Tensor):
    return (db.data_ptr(), tuple(db.shape), db.stride(0), db._version, db.device.index, db.dtype)


def _evict_when_freed(cache, key, t: torch.Tensor) -> None:
    """Drops ``cache[key]`` when the tensor that owns ``t``'s memory dies: a later tensor can
    be given the same address, shape and version, and must not meet the old entry."""
    owner = t._base if t._base is not None else t
    weakref.finalize(owner, cache.pop, key, None)


_PLANE_CACHE: "OrderedDict[tuple, DbPlane]" = OrderedDict()
_PLANE_CACHE_SIZE = 4


def get_plane(db: torch.Tensor) -> DbPlane:
    key = _plane_key(db)
    hit = _PLANE_CACHE.get(key)
    if hit is not None:
        _PLANE_CACHE.move_to_end(key)
        return hit
    plane = DbPlane(db)
    _PLANE_CACHE[key] = plane
    _evict_when_freed(_PLANE_CACHE, key, db)
    while len(_PLANE_CACHE) > _PLANE_CACHE_SIZE:
        _PLANE_CACHE.popitem(last=False)
    return plane


def clear_plane_cache() -> None:
    _PLANE_CACHE.clear()


# Status words of calls whose check was deferred: (pinned host copy, event of the copy).  The
# tensor-core kernel reports a timed-out wait there; reading it right after the call would
# serialise host and device once per call, so the public entry points look at the words of
# EARLIER calls instead (and ``check_pending()`` looks at all of them).
_PENDING_STATUS: deque = deque()


_STATUS_TEXT = {_lib.FL_ETIMEOUT: "a bounded device-side wait ran out",
                _lib.FL_EUNSUPPORTED: "the call ran with timing-experiment flags set",
                _lib.FL_EWORKSPACE: "the fallback list overflowed"}


def _raise_on_status(st) -> None:
    err = st[_lib.FL_STATUS_ERROR]
    if err != 0:
        raise _lib.FlashlibError(
            f"tensor-core kernel reported status {err} ({_STATUS_TEXT.get(err, 'unknown')}; "
            f"where={st[_lib.FL_STATUS_WHERE]:#x}): the results of that call are invalid")


def check_pending(block: bool = True) -> None:
    """Raises if an earlier call whose status check was deferred reported an error.  With
    ``block=False`` only calls that have already finished on the device are looked at."""
    while _PENDING_STATUS:
        host, ev = _PENDING_STATUS[0]
        if not block and not ev.query():
            return
        ev.synchronize()
        _PENDING_STATUS.popleft()
        _raise_on_status(host.tolist())


def _defer_status_check(status: torch.Tensor) -> None:
    check_pending(block=False)
    host = torch.empty(_lib.FL_STATUS_WORDS, dtype=torch.int32).pin_memory()
    host.copy_(status, non_blocking=True)
    ev = torch.cuda.Event()
    ev.record(torch.cuda.current_stream(status.device))
    _PENDING_STATUS.append((host, ev))
    while len(_PENDING_STATUS) > 64:              # bounded: the oldest calls have long finished
        check_pending_one = _PENDING_STATUS[0]
        check_pending_one[1].synchronize()
        _PENDING_STATUS.popleft()
        _raise_on_status(check_pending_one[0].tolist())


def knn_f32(q: torch.Tensor, db: torch.Tensor, k: int, *, mode: int = _lib.FL_KNN_AUTO,
            row_offset: int = 0, plane: Optional[DbPlane] = None, check_status=True,
            second_stage: Optional[bool] = None):
    """One 2-D problem through ``fl_knn_f32`` / ``fl_knn_staged_f32`` (fp32 rows) or ``fl_knn_rows``
    (bf16 / fp16 rows, read as stored): returns ``(dist fp32 (nq,k), idx int32 (nq,k), info)``.
    ``check_status=True`` reads the kernel's status words before returning (one host/device
    round trip; ``info["fallback_rows"]`` and ``info["stage2_rows"]`` are filled), ``"deferred"``
    leaves that to a later call or to ``check_pending()``, ``False`` skips it.
    ``second_stage`` (tensor-core mode): rows the bf16 proof rejects are scored again on the
    tensor cores with split hi/lo operands before anything takes the exact CUDA-core pass;
    ``None`` = when the database's split plane exists or is small enough to build."""
    lib = _lib.load()
    _lib.require_device()
    nq, d = q.shape
    m = db.shape[0]
    dev = q.device
    if q.dtype != db.dtype or db.dtype not in _DTYPE_CODES:
        raise TypeError(f"knn_f32 takes q and db of one dtype out of fp32 / bf16 / fp16, got {q.dtype} and {db.dtype}")
    resolved = lib.fl_knn_resolve_mode(nq, m, d, k) if mode == _lib.FL_KNN_AUTO else mode
    if resolved == _lib.FL_KNN_BF16_RERANK and plane is None:
        plane = get_plane(db)
    out_d = torch.empty((nq, k), dtype=torch.float32, device=dev)
    out_i = torch.empty((nq, k), dtype=torch.int32, device=dev)
    split = None
    if resolved == _lib.FL_KNN_BF16_RERANK and nq > 0:
        if second_stage is None:
            second_stage = _second_stage_default()
        if second_stage:
            split = plane.split_ptr(db)
    status = torch.zeros(_lib.FL_STATUS_WORDS, dtype=torch.int32, device=dev)
    if split is not None:
        ws_bytes = lib.fl_knn_staged_workspace_bytes(nq, m, d, k)
        ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=dev)
        rc = lib.fl_knn_staged_f32(q.data_ptr(), nq, q.stride(0), db.data_ptr(), m, db.stride(0), d, k,
                                   plane.ptr, split, row_offset, out_d.data_ptr(), out_i.data_ptr(),
                                   ws.data_ptr(), ws_bytes, status.data_ptr(), _stream_ptr(dev))
    else:
        ws_bytes = lib.fl_knn_workspace_bytes(max(nq, 1), m, d, k, resolved)
        ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=dev)
        rc = lib.fl_knn_rows(q.data_ptr(), nq, q.stride(0) if nq else d, db.data_ptr(), m, db.stride(0), d, k,
                             _DTYPE_CODES[db.dtype], resolved, plane.ptr if plane is not None else None, row_offset,
                             out_d.data_ptr(), out_i.data_ptr(), ws.data_ptr(), ws_bytes,
                             status.data_ptr(), _stream_ptr(dev))
    _lib.check(rc)
    info = {"mode": resolved, "status": status, "second_stage": split is not None}
    if check_status == "deferred" and resolved == _lib.FL_KNN_BF16_RERANK:
        _defer_status_check(status)
    elif check_status and resolved == _lib.FL_KNN_BF16_RERANK:
        st = status.tolist()
        info["fallback_rows"] = st[_lib.FL_STATUS_FALLBACK]
        info["stage2_rows"] = st[_lib.FL_STATUS_STAGE2]
        _raise_on_status(st)
    return out_d, out_i, info


def flash_knn_dispatch(x: torch.Tensor, c: torch.Tensor, k: int, *, tol: Optional[float] = None,
                       backend: Optional[str] = None, return_distances: bool = True,
                       mode: Optional[str] = None, **kwargs):
    """Exact k nearest rows of ``c`` for every row of ``x`` by squared L2.

    Parameters follow ``flashlib/primitives/knn/impl.py:199-247``: ``x`` is ``(B, N, D)`` or
    ``(N, D)``, ``c`` has the same rank and dtype, ``backend`` may be ``None`` or one of the
    reference's names (validated, then ignored: there is one implementation).  bf16 / fp16
    inputs are read as stored (no fp32 copy); ``tol`` follows the reference's rule
    (``storage_dtype_for``): when it allows 16-bit storage, fp32 inputs are cast to it -- the
    database once, cached -- and the result is the exact kNN of the stored values, as in the
    reference (``knn/impl.py:257-261``).  ``mode`` (``"exact"`` | ``"bf16"`` | ``None`` = auto)
    picks the scoring kernel.

    Returns ``(vals, idxs)`` -- fp32 true squared distances ascending and int32 indices --
    or just ``idxs`` with ``return_distances=False``.
    """
    if backend is not None and backend not in _VALID_BACKENDS:
        raise ValueError(f"backend must be one of {_VALID_BACKENDS} or None, got {backend!r}")
    if x.dim() not in (2, 3) or c.dim() != x.dim():
        raise ValueError("flash_knn expects x and c of the same rank: (N, D)/(M, D) or (B, N, D)/(B, M, D)")
    if x.dtype != c.dtype:
        raise AssertionError("x and c must share a dtype")
    if not (x.is_cuda and c.is_cuda):
        raise RuntimeError("flashlib_b200.flash_knn needs CUDA tensors (no CPU fallback)")
    squeeze = x.dim() == 2
    if squeeze:
        x = x.unsqueeze(0)
        c = c.unsqueeze(0)
    B, N, D = x.shape
    Bc, M, Dc = c.shape
    if Bc != B or Dc != D:
        raise AssertionError("x and c must agree on batch and feature dimensions")
    if not (1 <= int(k) <= M):
        raise AssertionError(f"k must be in [1, M={M}] (got {k})")
    k = int(k)
    m = _mode_from(mode)
    vals = torch.empty((B, N, k), dtype=torch.float32, device=x.device)
    idxs = torch.empty((B, N, k), dtype=torch.int32, device=x.device)
    target = storage_dtype_for(tol)
    lib = _lib.load()
    batched = (B > 1 and N > 0 and target is None and x.dtype == torch.float32 and m != _lib.FL_KNN_BF16_RERANK
               and lib.fl_knn_resolve_mode(N, M, D, k) == _lib.FL_KNN_EXACT_SIMT
               and x.stride(2) == 1 and c.stride(2) == 1 and x.stride(1) >= D and c.stride(1) >= D)
    if batched:
        # many small problems: one launch sequence for the whole batch
        _lib.require_device()
        with torch.cuda.device(x.device):
            ws_bytes = lib.fl_knn_batch_workspace_bytes(B, N, M, D, k)
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=x.device)
            _lib.check(lib.fl_knn_batch_f32(x.data_ptr(), B, N, x.stride(1), x.stride(0), c.data_ptr(), M, c.stride(1),
                                            c.stride(0), D, k, vals.data_ptr(), idxs.data_ptr(), ws.data_ptr(), ws_bytes,
                                            _stream_ptr(x.device)))
        if not return_distances:
            return idxs
        return vals, idxs
    with torch.cuda.device(x.device):
        for b in range(B):
            qb, cb = x[b], c[b]
            if target is not None and qb.dtype != target:
                qb, cb = qb.to(target), _cast_rows_cached(cb, target)
            qb, cb = _as_rows(qb), _as_rows(cb)
            d_b, i_b, _ = knn_f32(qb, cb, k, mode=m, check_status="deferred")
            vals[b] = d_b
            idxs[b] = i_b
    if not return_distances:
        return idxs[0] if squeeze else idxs
    if squeeze:
        return vals[0], idxs[0]
    return vals, idxs


flash_knn = flash_knn_dispatch
flash_knn_triton = flash_knn_dispatch  # name kept for callers of the reference's Triton entry


def triton_knn_gather_sqdist(x: torch.Tensor, c: torch.Tensor, idx: torch.Tensor,
                             out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[b,n,j] = sum_d (x[b,n,d] - c[b,idx[b,n,j],d])^2`` in fp32.

    Same contract as ``flashlib/kernels/distance/triton/knn_gather_l2sq.py:173-229``
    (3-D inputs, int32 or int64 indices).
    """
    assert x.is_cuda and c.is_cuda and idx.is_cuda
    assert x.dim() == 3 and c.dim() == 3 and idx.dim() == 3
    B, N, D = x.shape
    Bc, M, Dc = c.shape
    Bi, Ni, K = idx.shape
    assert B == Bc == Bi and N == Ni and D == Dc
    assert idx.dtype in (torch.int32, torch.int64)
    lib = _lib.load()
    _lib.require_device()
    if out is None:
        out = torch.empty((B, N, K), dtype=torch.float32, device=x.device)
    else:
        assert out.shape == (B, N, K) and out.dtype == torch.float32 and out.is_contiguous()
    with torch.cuda.device(x.device):
        for b in range(B):
            xb = _as_f32_rows(x[b])
            cb = _as_f32_rows(c[b])
            ib = idx[b].contiguous()
            _lib.check(lib.fl_gather_l2sq_f32(xb.data_ptr(), N, xb.stride(0), cb.data_ptr(), M, cb.stride(0), D,
                                              ib.data_ptr(), 1 if ib.dtype == torch.int64 else 0, K,
                                              out[b].data_ptr(), _stream_ptr(x.device)))
    return out


def row_sqnorm(x: torch.Tensor) -> torch.Tensor:
    """fp32 ``||row||^2`` of a 2-D CUDA tensor (``knn/triton/_row_norm.py:59-93``)."""
    lib = _lib.load()
    _lib.require_device()
    xb = _as_f32_rows(x)
    out = torch.empty(xb.shape[0], dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(lib.fl_rownorm_f32(xb.data_ptr(), xb.shape[0], xb.shape[1], xb.stride(0), out.data_ptr(),
                                      _stream_ptr(x.device)))
    return out


def topk_merge(cand_dist: torch.Tensor, cand_idx: torch.Tensor, k: int):
    """k smallest ``(dist, idx)`` per row of ``(nq, ncand)`` candidates (idx < 0 ignored)."""
    lib = _lib.load()
    _lib.require_device()
    cand_dist = cand_dist.contiguous().float()
    cand_idx = cand_idx.contiguous().to(torch.int32)
    nq, ncand = cand_dist.shape
    out_d = torch.empty((nq, k), dtype=torch.float32, device=cand_dist.device)
    out_i = torch.empty((nq, k), dtype=torch.int32, device=cand_dist.device)
    with torch.cuda.device(cand_dist.device):
        _lib.check(lib.fl_topk_merge_f32(cand_dist.data_ptr(), cand_idx.data_ptr(), nq, ncand, k,
                                         out_d.data_ptr(), out_i.data_ptr(), _stream_ptr(cand_dist.device)))
    return out_d, out_i
