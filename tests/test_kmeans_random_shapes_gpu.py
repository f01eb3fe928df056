"""Seeded random sweep over the k-means entry points: assignment (exact CUDA-core, tensor-core,
by size; single problems and batches) against the fp64 argmin within the tie band, and the centroid
update (full and incremental) against fp64 sums."""
import numpy as np
import pytest
import torch

import flashlib_b200 as fl
from flashlib_b200 import kmeans as km
from tests import parity

pytestmark = pytest.mark.gpu


def _case(seed):
    r = np.random.RandomState(seed)
    n = int(r.choice([1, 2, 127, 128, 129, 5000, 60_000]))
    K = int(r.choice([1, 2, 37, 255, 256, 257, 1024, 3000]))
    d = int(r.choice([1, 3, 8, 64, 65, 100, 128, 129, 200, 256, 300]))
    mode = ["exact", "bf16", None][int(r.randint(3))]
    B = int(r.choice([1, 1, 1, 3]))
    spread = float(r.choice([1.0, 0.02]))      # 0.02: points hug the centroids, near-duplicate centroids
    return n, K, d, mode, B, spread


@pytest.mark.parametrize("seed", range(80))
def test_random_assignment(seed):
    n, K, d, mode, B, spread = _case(seed)
    if mode == "bf16" and d > 256:
        mode = None
    g = torch.Generator().manual_seed(500 + seed)
    c = torch.randn(B, K, d, generator=g)
    if spread < 1.0 and K > 4:
        c[:, K - K // 2:] = c[:, :K // 2] + 1e-3 * torch.randn(B, K // 2, d, generator=g)   # near-duplicate centroids
    pick = torch.randint(0, K, (B, n), generator=g)
    x = torch.gather(c, 1, pick[..., None].expand(-1, -1, d)) * (1.0 if spread < 1 else 0.0) + spread * torch.randn(B, n, d, generator=g)
    xd, cd = x.cuda(), c.cuda()
    lab = fl.euclid_assign_triton(xd, cd, mode=mode)
    fl.check_pending()
    assert lab.shape == (B, n) and lab.dtype == torch.int32
    for b in range(B):
        d64 = torch.cdist(xd[b].double(), cd[b].double()) ** 2
        ref = d64.argmin(dim=1).cpu().numpy()
        res = parity.label_parity(x[b].numpy(), c[b].numpy(), lab[b].cpu().numpy(), ref)
        assert res["ok"], (seed, n, K, d, mode, B, spread, res)


@pytest.mark.parametrize("seed", range(20))
def test_random_update(seed):
    n, K, d, _, _, _ = _case(1000 + seed)
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(1, n, d, generator=g).cuda()
    lab = torch.randint(0, K, (1, n), generator=g, dtype=torch.int32).cuda()
    cents = torch.zeros(1, K, d, device="cuda")
    sums, cnts = km.triton_centroid_update_euclid(x, lab, cents, calculate_new=False)
    want_c = torch.bincount(lab[0].long(), minlength=K)
    want_s = torch.zeros(K, d, dtype=torch.float64, device="cuda").index_add_(0, lab[0].long(), x[0].double())
    assert torch.equal(cnts[0].long(), want_c)
    scale = max(want_s.abs().max().item(), 1.0)
    assert (sums[0].double() - want_s).abs().max().item() <= 1e-5 * scale
    # incremental form from a different labelling
    lab2 = torch.randint(0, K, (1, n), generator=g, dtype=torch.int32).cuda()
    prev = lab2.clone()
    s2, c2 = km.triton_centroid_update_euclid(x, lab2, cents, calculate_new=False)
    km.centroid_update_delta(x, lab, prev, s2, c2)
    assert torch.equal(c2[0].long(), want_c) and torch.equal(prev, lab)
    assert (s2[0].double() - want_s).abs().max().item() <= 3e-5 * scale
