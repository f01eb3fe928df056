"""Seeded random sweep over the IVF-Flat search: sizes, feature counts, list counts (more lists than
the data fills included), probes and k, all three fine-scan variants -- each against the exact top-k
of the rows of the probed lists, computed in fp64 from the same index and the same probe lists."""
import numpy as np
import pytest
import torch

import flashlib_b200 as fl
from flashlib_b200.ivf_flat import ivf_fine_scan
from tests import parity

pytestmark = pytest.mark.gpu


def _case(seed):
    r = np.random.RandomState(seed)
    n = int(r.choice([300, 5_000, 40_000]))
    d = int(r.choice([2, 17, 64, 96, 128, 200, 256, 300]))
    nlist = int(r.choice([1, 7, 64, 300]))
    nprobe = int(min(nlist, r.choice([1, 4, 16, 33])))
    k = int(r.choice([1, 5, 10, 16, 40]))
    nq = int(r.choice([1, 130, 1500]))
    variant = ["exact", "bf16", None][int(r.randint(3))]
    return n, d, nlist, nprobe, k, nq, variant


@pytest.mark.parametrize("seed", range(100))
def test_random_ivf_fine_scan(seed):
    n, d, nlist, nprobe, k, nq, variant = _case(seed)
    g = torch.Generator().manual_seed(300 + seed)
    means = 3 * torch.randn(20, d, generator=g)
    X = (means[torch.randint(0, 20, (n,), generator=g)] + torch.randn(n, d, generator=g)).cuda()
    Q = (means[torch.randint(0, 20, (nq,), generator=g)] + torch.randn(nq, d, generator=g)).cuda()
    index = fl.flash_ivf_flat_build(X, nlist, nprobe=nprobe, niter=3, seed=seed)
    Qp = torch.nn.functional.pad(Q, (0, index.Dp - d)) if index.Dp > d else Q
    probed = fl.flash_knn(Qp, index.centroids, nprobe, return_distances=False, mode="exact")
    if variant == "bf16" and (k > 16 or index.Dp > 256):
        variant = None
    vals, pos = ivf_fine_scan(Qp, index, probed, k, mode=variant)
    fl.check_pending()
    offs = index.list_offsets.cpu().numpy()
    data64 = index.data.double()
    pr = probed.cpu().numpy()
    v, p = vals.cpu().numpy(), pos.cpu().numpy()
    rows_checked = 0
    for qi in range(0, nq, max(1, nq // 25)):
        rows = np.concatenate([np.arange(offs[c], offs[c + 1]) for c in pr[qi]]) if nprobe else np.zeros(0, dtype=np.int64)
        kk = min(k, rows.size)
        assert np.all(p[qi, kk:] == -1) and np.all(np.isinf(v[qi, kk:]))
        if kk == 0:
            continue
        rt = torch.from_numpy(rows).cuda()
        d64 = ((data64[rt] - Qp[qi].double()) ** 2).sum(-1)
        ref_pos = rows[d64.topk(kk, largest=False).indices.cpu().numpy()]
        res = parity.knn_parity(Qp[qi:qi + 1].cpu().numpy(), index.data.cpu().numpy(), v[qi:qi + 1, :kk], p[qi:qi + 1, :kk],
                                ref_pos[None, :])
        assert res["ok"], (seed, n, d, nlist, nprobe, k, nq, variant, qi, res)
        rows_checked += 1
    assert rows_checked > 0 or n == 0
