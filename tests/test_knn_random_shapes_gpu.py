"""Seeded random sweep over the kNN entry points: shapes (tiny to a few tile rows, features up to 520,
k up to 64), element types (fp32 / bf16 / fp16), modes (exact CUDA-core, tensor-core, auto), row
strides and batches -- every case against fp64 brute force on the values as stored."""
import numpy as np
import pytest
import torch

import flashlib_b200 as fl
from flashlib_b200 import _lib
from flashlib_b200.knn import knn_f32
from tests import parity

pytestmark = pytest.mark.gpu


def _fp64_neighbours(q, db, k):
    qd, dbd = q.double(), db.double()
    d64 = (qd * qd).sum(-1, keepdim=True) + (dbd * dbd).sum(-1)[None, :] - 2.0 * qd @ dbd.T
    return d64.topk(k, dim=1, largest=False).indices.cpu().numpy()


def _case(seed):
    r = np.random.RandomState(seed)
    d = int(r.choice([1, 2, 3, 7, 16, 31, 64, 65, 96, 100, 128, 129, 160, 200, 256, 257, 300, 384, 512, 520]))
    m = int(r.choice([1, 2, 17, 255, 256, 257, 1000, 4097, 20_000, 70_000]))
    nq = int(r.choice([1, 2, 31, 128, 129, 500, 1000]))
    k = int(min(m, r.choice([1, 2, 5, 10, 16, 17, 33, 64])))
    dtype = [torch.float32, torch.bfloat16, torch.float16][int(r.randint(3))]
    mode = ["exact", "bf16", None][int(r.randint(3))]
    strided = bool(r.randint(2))
    spread = float(r.choice([1.0, 0.05]))        # 0.05: near-duplicate rows around a few centres
    return d, m, nq, k, dtype, mode, strided, spread


@pytest.mark.parametrize("seed", range(150))
def test_random_shape(seed):
    d, m, nq, k, dtype, mode, strided, spread = _case(seed)
    lib = _lib.load()
    if mode == "bf16" and (d > 512 or k > 112):
        mode = None
    g = torch.Generator().manual_seed(1000 + seed)
    centres = torch.randn(8, d, generator=g)
    db = (centres[torch.randint(0, 8, (m,), generator=g)] * (1.0 if spread < 1 else 0.0) + spread * torch.randn(m, d, generator=g))
    q = (centres[torch.randint(0, 8, (nq,), generator=g)] * (1.0 if spread < 1 else 0.0) + spread * torch.randn(nq, d, generator=g))
    db, q = db.to(dtype).cuda(), q.to(dtype).cuda()
    if strided:                                   # rows inside a wider buffer
        wide = torch.zeros(m, d + 8, dtype=dtype, device="cuda")
        wide[:, :d] = db
        db = wide[:, :d]
    vals, idxs = fl.flash_knn(q, db, k, mode=mode)
    fl.check_pending()
    assert vals.shape == (nq, k) and vals.dtype == torch.float32 and idxs.dtype == torch.int32
    ref_i = _fp64_neighbours(q, db, k)
    res = parity.knn_parity(q.float().cpu().numpy(), db.float().cpu().numpy(), vals.cpu().numpy(), idxs.cpu().numpy(), ref_i)
    assert res["ok"], (seed, d, m, nq, k, dtype, mode, strided, spread, res)


@pytest.mark.parametrize("seed", range(8))
def test_random_batch(seed):
    r = np.random.RandomState(100 + seed)
    B, N, M = int(r.choice([2, 5, 33])), int(r.choice([1, 64, 300])), int(r.choice([16, 300, 2000]))
    d, k = int(r.choice([2, 8, 33, 128])), int(r.choice([1, 4, 16]))
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, N, d, generator=g).cuda()
    c = torch.randn(B, M, d, generator=g).cuda()
    vals, idxs = fl.flash_knn(x, c, k)
    for b in range(B):
        ref_i = _fp64_neighbours(x[b], c[b], k)
        res = parity.knn_parity(x[b].cpu().numpy(), c[b].cpu().numpy(), vals[b].cpu().numpy(), idxs[b].cpu().numpy(), ref_i)
        assert res["ok"], (seed, B, N, M, d, k, b, res)
