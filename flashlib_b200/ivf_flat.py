"""IVF-Flat index build and search behind flashlib's ``flash_ivf_flat_*`` API.

Mirrors ``flashlib/primitives/ivf_flat/impl.py:69-159``, the container of
``ivf_flat/index.py:27-78``, the build of ``ivf_flat/triton/build.py:34-95`` and the search
of ``ivf_flat/triton/search.py:52-108``.  The fine scan (grouping of (query, probe) pairs by
list, list scan, per-query merge, exact re-rank) runs in one C-ABI call; nothing on the
search path synchronises the host.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from . import _lib
from .kmeans import euclid_assign_triton, flash_kmeans
from .knn import _as_f32_rows, _defer_status_check, _mode_from, _stream_ptr, knn_f32, row_sqnorm


@dataclass
class IvfFlatIndex:
    """A built IVF-Flat index; field for field the reference's ``IvfFlatIndex``.

    ``data`` holds the database rows cell-contiguously: list ``c`` owns rows
    ``list_offsets[c] .. list_offsets[c+1]``; ``ids[p]`` is the caller's row id of stored
    row ``p``.
    """

    centroids: torch.Tensor
    data: torch.Tensor
    ids: torch.Tensor
    list_offsets: torch.Tensor
    metric: str
    D: int
    Dp: int
    nlist: int
    nprobe: int
    max_list_len: int = 0      # may be given as a 1-element device tensor: read back (one sync) on first use
    _hnorm: Optional[torch.Tensor] = field(default=None, repr=False, compare=False)
    _tc_plane: Optional[torch.Tensor] = field(default=None, repr=False, compare=False)
    _last_status: Optional[torch.Tensor] = field(default=None, repr=False, compare=False)

    @property
    def M(self) -> int:
        return int(self.data.shape[0])

    @property
    def device(self) -> torch.device:
        return self.data.device

    @property
    def dtype(self) -> torch.dtype:
        return self.data.dtype

    def list_lengths(self) -> torch.Tensor:
        return self.list_offsets[1:] - self.list_offsets[:-1]

    def half_norms(self) -> torch.Tensor:
        """fp32 ``||row||^2 / 2`` of the stored rows, computed once per index."""
        if self._hnorm is None or self._hnorm.device != self.data.device:
            self._hnorm = row_sqnorm(self.data).mul_(0.5)
        return self._hnorm


_INDEX_FORMAT = "flashlib_b200.IvfFlatIndex/1"


def save_ivf_flat_index(index: IvfFlatIndex, path) -> None:
    """Writes the index to ``path`` with ``torch.save``: the reference's ``IvfFlatIndex`` fields
    (``ivf_flat/index.py:27-55``; the reference itself defines no on-disk format) as CPU tensors
    plus a format tag.  Derived data -- the half norms and the tensor-core operand plane -- is
    not stored: it is rebuilt from ``data`` on first use after loading."""
    torch.save({"format": _INDEX_FORMAT,
                "centroids": index.centroids.cpu(), "data": index.data.cpu(), "ids": index.ids.cpu(),
                "list_offsets": index.list_offsets.cpu(), "metric": index.metric, "D": int(index.D),
                "Dp": int(index.Dp), "nlist": int(index.nlist), "nprobe": int(index.nprobe),
                "max_list_len": int(index.max_list_len)}, path)


def load_ivf_flat_index(path, device=None) -> IvfFlatIndex:
    """Reads an index written by :func:`save_ivf_flat_index` and moves it to ``device`` (default:
    the tensors stay on the CPU; searching needs a CUDA device)."""
    blob = torch.load(path, map_location="cpu", weights_only=True)
    if not isinstance(blob, dict) or blob.get("format") != _INDEX_FORMAT:
        raise ValueError(f"{path!s} is not a flashlib_b200 IVF-Flat index (format tag {blob.get('format') if isinstance(blob, dict) else None!r})")
    t = {k: (blob[k].to(device) if device is not None else blob[k]) for k in ("centroids", "data", "ids", "list_offsets")}
    if t["data"].shape[0] != t["ids"].shape[0] or t["list_offsets"].shape[0] != blob["nlist"] + 1 \
            or int(t["list_offsets"][-1]) != t["data"].shape[0]:
        raise ValueError(f"{path!s}: inconsistent index (rows, ids and list offsets do not agree)")
    return IvfFlatIndex(centroids=t["centroids"], data=t["data"], ids=t["ids"], list_offsets=t["list_offsets"],
                        metric=blob["metric"], D=blob["D"], Dp=blob["Dp"], nlist=blob["nlist"], nprobe=blob["nprobe"],
                        max_list_len=blob["max_list_len"])


IvfFlatIndex.save = save_ivf_flat_index
IvfFlatIndex.load = staticmethod(load_ivf_flat_index)


def _get_max_list_len(self) -> int:
    v = self.__dict__.get("_max_list_len", 0)
    if isinstance(v, torch.Tensor):
        v = int(v.item())
        self.__dict__["_max_list_len"] = v
    return v


def _set_max_list_len(self, v) -> None:
    self.__dict__["_max_list_len"] = v


# The device-side build leaves the longest list's length on the device; nothing on the build or
# search path needs it, so it is only fetched when somebody reads the attribute.
IvfFlatIndex.max_list_len = property(_get_max_list_len, _set_max_list_len)


def _pad_features(x: torch.Tensor, Dp: int) -> torch.Tensor:
    D = x.shape[-1]
    if D >= Dp:
        return x
    pad = torch.zeros((*x.shape[:-1], Dp - D), device=x.device, dtype=x.dtype)
    return torch.cat([x, pad], dim=-1)


def flash_ivf_flat_build(X: torch.Tensor, nlist: int, *, metric: str = "l2", nprobe: int = 8,
                         niter: int = 20, train_size: Optional[int] = None, seed: int = 0,
                         backend: Optional[str] = None) -> IvfFlatIndex:
    """Train the coarse quantiser on a sample and lay the rows out cell-contiguously.

    Same steps and the same torch random draws as ``ivf_flat/triton/build.py:34-95``:
    ``randperm`` from a device generator seeded with ``seed`` picks the sample,
    ``flash_kmeans`` (global-generator ``randint`` init) trains ``nlist`` centroids, one
    assignment pass labels every row, and ``bincount`` / ``cumsum`` / stable ``argsort`` build
    the CSR layout.
    """
    if metric != "l2":
        raise NotImplementedError(f"ivf_flat currently supports metric='l2' only (got {metric!r})")
    if not X.is_cuda or X.ndim != 2:
        raise ValueError("flash_ivf_flat_build requires a 2D CUDA tensor")
    M, D = X.shape
    nlist = int(min(nlist, M))
    if nlist < 1:
        raise ValueError("nlist must be >= 1")
    Dp = max(int(D), 16)
    Xp = _pad_features(X, Dp).contiguous()

    train_size = int(train_size or min(M, nlist * 256))
    train_size = max(min(train_size, M), nlist)
    g = torch.Generator(device=X.device).manual_seed(seed)
    sample_idx = torch.randperm(M, generator=g, device=X.device)[:train_size]
    sample = Xp.index_select(0, sample_idx)

    _, centroids, _ = flash_kmeans(sample, nlist, max_iters=niter, metric="euclidean")
    centroids = centroids.contiguous()
    return index_from_centroids(Xp, centroids, D=int(D), nprobe=nprobe, metric=metric)


def index_from_centroids(Xp: torch.Tensor, centroids: torch.Tensor, *, D: int, nprobe: int,
                         metric: str = "l2") -> IvfFlatIndex:
    """Assign every (padded) row to its nearest centroid and build the cell-contiguous layout on
    the device: per-list histogram, exclusive scan, stable partition of the rows (the order of the
    reference's stable ``argsort`` by list, ``ivf_flat/triton/build.py:59-95``) -- one C-ABI call,
    no host synchronisation."""
    lib = _lib.load()
    nlist = centroids.shape[0]
    M, Dp = Xp.shape
    x32 = _as_f32_rows(Xp)
    assign = euclid_assign_triton(x32.unsqueeze(0), centroids.float().unsqueeze(0)).squeeze(0)
    dev = Xp.device
    data = torch.empty((M, Dp), dtype=torch.float32, device=dev)
    ids = torch.empty(M, dtype=torch.int64, device=dev)
    offsets = torch.empty(nlist + 1, dtype=torch.int64, device=dev)
    longest = torch.empty(1, dtype=torch.int32, device=dev)
    ws_bytes = lib.fl_ivf_build_workspace_bytes(M, nlist)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.fl_ivf_build_csr_f32(x32.data_ptr(), M, x32.stride(0), Dp, assign.data_ptr(), nlist,
                                            data.data_ptr(), ids.data_ptr(), offsets.data_ptr(), longest.data_ptr(),
                                            ws.data_ptr(), ws_bytes, _stream_ptr(dev)))
    if Xp.dtype != torch.float32:
        data = data.to(Xp.dtype)
    return IvfFlatIndex(centroids=centroids, data=data, ids=ids, list_offsets=offsets, metric=metric, D=int(D),
                        Dp=int(Dp), nlist=int(nlist), nprobe=int(nprobe), max_list_len=longest)


def _tc_plane(index: IvfFlatIndex, data: torch.Tensor, offs: torch.Tensor) -> torch.Tensor:
    """bf16 operand plane of the stored rows for the tensor-core fine scan, built on first use."""
    if index._tc_plane is None or index._tc_plane.device != data.device:
        lib = _lib.load()
        m, d = data.shape
        nbytes = lib.fl_ivf_plane_bytes(m, index.nlist, d)
        buf = torch.empty(nbytes, dtype=torch.uint8, device=data.device)
        with torch.cuda.device(data.device):
            _lib.check(lib.fl_ivf_prepare_f32(data.data_ptr(), m, data.stride(0), d, offs.data_ptr(), index.nlist,
                                              buf.data_ptr(), nbytes, _stream_ptr(data.device)))
        index._tc_plane = buf
    return index._tc_plane


def ivf_fine_scan(Qp: torch.Tensor, index: IvfFlatIndex, probed: torch.Tensor, k: int, mode: Optional[str] = None):
    """Fine scan of the probed lists: ``(vals fp32 (nq,k), pos int32 (nq,k))``, ``+inf`` / ``-1``
    padded when a query's lists hold fewer than ``k`` rows.  ``mode`` ``"exact"`` forces the
    CUDA-core scan, ``"bf16"`` the tensor-core scan (k <= 16, d <= 256); ``None`` takes the
    tensor cores for k <= 16 when the batch has at least 2,048 (query, probe) pairs.  Both
    return the same neighbours."""
    lib = _lib.load()
    _lib.require_device()
    q = _as_f32_rows(Qp)
    data = _as_f32_rows(index.data)
    nq, d = q.shape
    m = data.shape[0]
    probed = probed.to(torch.int32).contiguous()
    nprobe = probed.shape[1]
    offs = index.list_offsets.to(torch.int64).contiguous()
    vals = torch.empty((nq, k), dtype=torch.float32, device=q.device)
    pos = torch.empty((nq, k), dtype=torch.int32, device=q.device)
    if mode not in (None, "auto", "exact", "simt", "bf16", "tc"):
        raise ValueError(f"unknown fine-scan mode {mode!r} (exact|bf16|None)")
    same_data = data.data_ptr() == index.data.data_ptr()
    tc_bytes = lib.fl_ivf_fine_scan_tc_workspace_bytes(max(nq, 1), nprobe, index.nlist, m, d, k) if same_data else 0
    if mode in ("bf16", "tc") and tc_bytes == 0:
        raise NotImplementedError("tensor-core fine scan needs k <= 16, d <= 256 and fp32 rows stored in the index")
    # auto: every k the tensor-core scan takes (the pools keep 24 entries per (pair, half list): k <= 12
    # proves every query of the 1M-row benchmark, k = 16 leaves a handful to the exact scan)
    if nq > 0 and tc_bytes > 0 and (mode in ("bf16", "tc") or
                                    (mode in (None, "auto") and k <= 16 and nq * nprobe >= 2048)):
        plane = _tc_plane(index, data, offs)
        ws = torch.empty(tc_bytes, dtype=torch.uint8, device=q.device)
        status = torch.zeros(_lib.FL_STATUS_WORDS, dtype=torch.int32, device=q.device)
        with torch.cuda.device(q.device):
            _lib.check(lib.fl_ivf_fine_scan_tc_f32(q.data_ptr(), nq, q.stride(0), data.data_ptr(), m, data.stride(0), d,
                                                   offs.data_ptr(), index.nlist, probed.data_ptr(), nprobe, k,
                                                   plane.data_ptr(), vals.data_ptr(), pos.data_ptr(),
                                                   ws.data_ptr(), tc_bytes, status.data_ptr(), _stream_ptr(q.device)))
        index._last_status = status     # status[FL_STATUS_FALLBACK]: queries recomputed by the exact scan
        _defer_status_check(status)     # an error word raises at a later call or in check_pending()
        return vals, pos
    ws_bytes = lib.fl_ivf_fine_scan_workspace_bytes(max(nq, 1), nprobe, index.nlist, m, d, k)
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=q.device)
    hn = index.half_norms() if data.data_ptr() == index.data.data_ptr() else None
    with torch.cuda.device(q.device):
        _lib.check(lib.fl_ivf_fine_scan_f32(q.data_ptr(), nq, q.stride(0) if nq else d, data.data_ptr(), m,
                                            data.stride(0), d, offs.data_ptr(), index.nlist,
                                            probed.data_ptr(), nprobe, k,
                                            hn.data_ptr() if hn is not None else None,
                                            vals.data_ptr(), pos.data_ptr(), ws.data_ptr(), ws_bytes,
                                            _stream_ptr(q.device)))
    return vals, pos


def flash_ivf_flat_search(index: IvfFlatIndex, Q: torch.Tensor, k: int, *, nprobe: Optional[int] = None,
                          backend: Optional[str] = None, variant: str = "auto"):
    """``(vals fp32, ids int64)`` of the ``k`` nearest probed rows per query, ``-1`` / ``+inf``
    padded (``ivf_flat/triton/search.py:52-108``).  ``variant`` is validated like the
    reference's: ``"gemm"`` asks for the tensor-core fine scan (taken when k <= 16 and
    d <= 256, where its candidate pools prove nearly every query; the CUDA-core scan
    otherwise), ``"elementwise"`` for the CUDA-core scan, ``"auto"`` picks by batch size.
    All variants return the same neighbours."""
    if variant not in ("auto", "gemm", "elementwise"):
        raise ValueError(f"unknown variant {variant!r} (auto|gemm|elementwise)")
    if not Q.is_cuda or Q.ndim != 2:
        raise ValueError("flash_ivf_flat_search requires a 2D CUDA tensor")
    nprobe = int(nprobe or index.nprobe)
    nprobe = max(1, min(nprobe, index.nlist))
    if not (1 <= k <= index.M):
        raise ValueError(f"k must be in [1, M={index.M}] (got {k})")
    Qp = _pad_features(Q.to(index.data.dtype), index.Dp).contiguous()
    # Coarse probe: near-tied centroids must rank as in fp32, which both kNN modes guarantee (the
    # tensor-core mode proves every row's list of centroids or recomputes it exactly); large
    # batches take the tensor cores, where the 2 nq nlist D contraction costs next to nothing.
    coarse = "bf16" if (Q.shape[0] * index.nlist >= (1 << 22) and nprobe <= 16 and index.Dp <= 256
                        and index.centroids.dtype == torch.float32) else "exact"
    # (no second tensor-core stage here: on a database of a few tiles the exact pass for a handful of
    # unproven rows costs less than the stage's three launches cost every call)
    _, probed, _ = knn_f32(_as_f32_rows(Qp), _as_f32_rows(index.centroids), nprobe, mode=_mode_from(coarse),
                           check_status="deferred", second_stage=False)
    mode = {"auto": None, "elementwise": "exact", "gemm": "bf16"}[variant]
    if mode == "bf16" and (k > 16 or index.Dp > 256):
        mode = "exact"
    vals, pos = ivf_fine_scan(Qp, index, probed, k, mode=mode)
    if index.ids.dtype == torch.int64 and index.ids.is_contiguous():
        ids = torch.empty(pos.shape, dtype=torch.int64, device=pos.device)
        with torch.cuda.device(pos.device):
            _lib.check(_lib.load().fl_ivf_map_ids(pos.data_ptr(), index.ids.data_ptr(), pos.numel(), index.ids.shape[0],
                                                  ids.data_ptr(), _stream_ptr(pos.device)))
    else:
        valid = pos >= 0
        pos_safe = pos.clamp_min(0).to(torch.int64)
        ids = torch.where(valid, index.ids[pos_safe], torch.full_like(pos_safe, -1))
    return vals, ids


def flash_ivf_flat(X: torch.Tensor, Q: torch.Tensor, k: int, *, nlist: int = 1024, nprobe: int = 8,
                   metric: str = "l2", niter: int = 20, train_size: Optional[int] = None, seed: int = 0,
                   backend: Optional[str] = None):
    """One-shot build + search (``ivf_flat/impl.py:132-150``)."""
    index = flash_ivf_flat_build(X, nlist, metric=metric, nprobe=nprobe, niter=niter,
                                 train_size=train_size, seed=seed, backend=backend)
    return flash_ivf_flat_search(index, Q, k, nprobe=nprobe, backend=backend)
