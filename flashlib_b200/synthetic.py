"""Seeded synthetic inputs with the shapes and value distributions of the benchmark
configurations (standing in for SIFT-1M-style public data, which is not available offline).

Everything is drawn with a CPU ``torch.Generator`` so the CPU checker and the GPU path see
identical bits.
"""
from __future__ import annotations

import torch


def _gen(seed: int) -> torch.Generator:
    return torch.Generator(device="cpu").manual_seed(int(seed))


def randn_knn(m: int, d: int, nq: int, seed: int):
    """Database ``(m, d)`` and queries ``(nq, d)`` ~ N(0, 1) (configuration: 20 000 x 64,
    1 000 queries, seed 0; sharded configuration: 96 features)."""
    g = _gen(seed)
    db = torch.randn(m, d, generator=g)
    q = torch.randn(nq, d, generator=g)
    return db, q


def mixture(n: int, d: int, n_comp: int, seed: int, *, nq: int = 0, clamp: bool = False):
    """Gaussian mixture: component means ~ N(0, 4 I), equal weights, unit noise; optionally
    clamped at >= 0 (SIFT-like non-negative values).  Returns ``(X, Q)`` (``Q`` is ``None``
    when ``nq == 0``); queries come from the same mixture."""
    g = _gen(seed)
    means = 2.0 * torch.randn(n_comp, d, generator=g)

    def draw(rows: int) -> torch.Tensor:
        out = torch.empty(rows, d)
        step = 1 << 18
        for s in range(0, rows, step):
            e = min(rows, s + step)
            comp = torch.randint(0, n_comp, (e - s,), generator=g)
            out[s:e] = means[comp] + torch.randn(e - s, d, generator=g)
        return out.clamp_min_(0.0) if clamp else out

    X = draw(n)
    Q = draw(nq) if nq > 0 else None
    return X, Q


CONFIGS = {
    # name: generator arguments of the five benchmark configurations
    "knn_cpu_small": dict(kind="randn", m=20_000, d=64, nq=1_000, k=10, seed=0),
    "kmeans_1m": dict(kind="mixture", n=1_000_000, d=128, n_comp=1024, K=1024, iters=20, seed=1),
    "knn_1m": dict(kind="mixture", n=1_000_000, d=128, n_comp=4096, nq=10_000, clamp=True, seed=2),
    "ivf_1m": dict(kind="mixture", n=1_000_000, d=128, n_comp=4096, nq=10_000, clamp=True,
                   nlist=1024, nprobe=16, k=10, seed=3),
    "knn_sharded_100m": dict(kind="randn", m=100_000_000, d=96, nq=100_000, k=100, seed=4),
}
