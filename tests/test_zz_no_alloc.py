"""The workspace-free assignment entry point, for hosts that may launch kernels but not
allocate device memory (no allocator handed to a plugin, a memory pool that owns the whole
GPU, or a loop that cannot afford cudaMalloc's synchronisation).

It must give exactly the labels of the regular entry point, on two calls in a row: the
second call reuses the library's built-in scratch array, which still holds the first call's
half norms.  This file sorts last on purpose, so every other test has already run when a
run that stops at the first failure reaches it.
"""
import ctypes

import pytest
import torch

from flashlib_b200 import _lib

MAX_K = 16384


def _assign(lib, fn_noalloc, x, c):
    n, d = x.shape
    K = c.shape[0]
    labels = torch.full((n,), -1, dtype=torch.int32, device=x.device)
    stream = torch.cuda.current_stream().cuda_stream
    if fn_noalloc:
        rc = lib.fl_kmeans_assign_noalloc_f32(x.data_ptr(), n, x.stride(0), c.data_ptr(), K, c.stride(0), d,
                                              labels.data_ptr(), stream)
    else:
        ws_bytes = lib.fl_kmeans_assign_workspace_bytes(n, K, d)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=x.device)
        rc = lib.fl_kmeans_assign_f32(x.data_ptr(), n, x.stride(0), c.data_ptr(), K, c.stride(0), d,
                                      labels.data_ptr(), ws.data_ptr(), ws_bytes, stream)
    _lib.check(rc)
    torch.cuda.synchronize()
    return labels


@pytest.mark.gpu
def test_noalloc_assign_matches_workspace_assign_twice():
    lib = _lib.load()
    g = torch.Generator().manual_seed(77)
    x = torch.randn(5000, 48, generator=g).cuda()
    c1 = torch.randn(300, 48, generator=g).cuda()
    c2 = (3.0 * torch.randn(37, 48, generator=g)).cuda()      # fewer, larger centroids: stale norms would show
    for c in (c1, c2):
        ref = _assign(lib, False, x, c)
        got = _assign(lib, True, x, c)
        assert torch.equal(got, ref)
        assert int(got.min()) >= 0 and int(got.max()) < c.shape[0]


def test_noalloc_assign_rejects_oversized_k():
    lib = _lib.load()
    rc = lib.fl_kmeans_assign_noalloc_f32(None, 10, 8, None, MAX_K + 1, 8, 8, None, None)
    assert rc == _lib.FL_EUNSUPPORTED
    assert "exceeds the built-in scratch" in _lib.last_error()
    with pytest.raises(NotImplementedError):
        _lib.check(rc)
