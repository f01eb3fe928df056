"""Timed CPU baseline: the reference's chunked kNN restated with the same torch CPU operators
it calls (``bmm`` / ``topk`` / ``gather``), so the baseline runs on the same multi-threaded
ATen/MKL kernels as the reference's own CPU path.

TEST / BENCHMARK INFRASTRUCTURE ONLY -- never imported by ``flashlib_b200``.  The checker used
for parity is ``oracle/oracle.py``; ``tests/test_oracle_golden.py`` checks this file against it
and against the reference fixtures.
"""
from __future__ import annotations

import torch


def knn_chunked(x: torch.Tensor, c: torch.Tensor, k: int, chunk_size: int = 8192):
    """``knn_torch_chunked`` -- flashlib/primitives/knn/torch_fallback.py:33-79, for one batch:
    per database chunk ``x_sq + c_sq^T - 2 x c^T`` clamped at 0, then ``topk`` over the
    concatenation of the kept candidates and the chunk."""
    x = x.float()
    c = c.float()
    n = x.shape[0]
    m = c.shape[0]
    x_sq = (x ** 2).sum(-1, keepdim=True)
    top_v = torch.full((n, k), float("inf"), dtype=torch.float32)
    top_i = torch.full((n, k), -1, dtype=torch.int64)
    for s in range(0, m, chunk_size):
        e = min(s + chunk_size, m)
        cc = c[s:e]
        c_sq = (cc ** 2).sum(-1, keepdim=True)
        dist = x_sq + c_sq.T - 2.0 * (x @ cc.T)
        dist.clamp_min_(0.0)
        comb_v = torch.cat([top_v, dist], dim=-1)
        comb_i = torch.cat([top_i, torch.arange(s, e).view(1, -1).expand(n, -1)], dim=-1)
        _, sel = comb_v.topk(k, dim=-1, largest=False, sorted=True)
        top_v = comb_v.gather(-1, sel)
        top_i = comb_i.gather(-1, sel)
    return top_v, top_i
