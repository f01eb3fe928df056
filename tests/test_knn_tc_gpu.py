"""The tensor-core (tcgen05) kNN path: raw scores of the MMA pipeline against a plain matrix
product, and end-to-end parity of mode="bf16" against the oracle, including the verified
fallback to the exact path."""
import numpy as np
import pytest
import torch

import flashlib_b200 as fl
from flashlib_b200 import _lib
from flashlib_b200.knn import DbPlane, _stream_ptr, knn_f32
from oracle import oracle
from tests import parity

pytestmark = pytest.mark.gpu


def tc_scores(q, db):
    lib = _lib.load()
    nq, d = q.shape
    m = db.shape[0]
    plane = DbPlane(db)
    m_pad = (m + 255) // 256 * 256
    scores = torch.full((128, m_pad), float("nan"), device="cuda")
    ws_bytes = lib.fl_knn_workspace_bytes(nq, m, d, 10, _lib.FL_KNN_BF16_RERANK)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
    status = torch.zeros(_lib.FL_STATUS_WORDS, dtype=torch.int32, device="cuda")
    _lib.check(lib.fl_debug_knn_tc_scores(q.data_ptr(), nq, q.stride(0), d, plane.ptr, m, scores.data_ptr(), m_pad,
                                          ws.data_ptr(), ws_bytes, status.data_ptr(), _stream_ptr(q.device)))
    torch.cuda.synchronize()
    assert status[_lib.FL_STATUS_ERROR].item() == 0, status.tolist()
    return scores


@pytest.mark.parametrize("nq,m,d", [(128, 256, 64), (100, 1000, 128), (128, 5000, 128), (37, 3000, 96), (128, 2048, 256),
                                    (128, 70_000, 128)])
def test_mma_pipeline_scores(nq, m, d):
    g = torch.Generator().manual_seed(m + d)
    db = torch.randn(m, d, generator=g).cuda()
    q = torch.randn(nq, d, generator=g).cuda()
    got = tc_scores(q, db)
    ref = q.bfloat16().float() @ db.bfloat16().float().T - 0.5 * (db * db).sum(-1)[None, :]
    err = (got[:nq, :m] - ref).abs().max().item()
    assert err < 2e-3, err
    assert torch.all(got[:nq, m:] < -1e37)                    # padding rows can never be candidates


SHAPES = [(1, 300, 16, 1), (129, 5000, 128, 10), (300, 40_000, 128, 16), (64, 9_000, 200, 10), (500, 100_000, 64, 10),
          (257, 30_001, 96, 5)]


@pytest.mark.parametrize("nq,m,d,k", SHAPES)
def test_bf16_mode_vs_oracle(nq, m, d, k):
    g = torch.Generator().manual_seed(nq + m)
    db = torch.randn(m, d, generator=g)
    q = torch.randn(nq, d, generator=g)
    _, ref_i = oracle.knn_naive(q.numpy(), db.numpy(), k)
    vals, idxs = fl.flash_knn(q.cuda(), db.cuda(), k, mode="bf16")
    res = parity.knn_parity(q.numpy(), db.numpy(), vals.cpu().numpy(), idxs.cpu().numpy(), ref_i)
    assert res["ok"], res


def test_bf16_mode_equals_exact_mode_and_reports_fallbacks():
    """Clustered, near-duplicate data makes many candidate pools unprovable: those rows must
    come back through the exact path with identical results."""
    g = torch.Generator().manual_seed(9)
    base = torch.randn(200, 128, generator=g)
    db = (base[torch.randint(0, 200, (60_000,), generator=g)] + 0.1 * torch.randn(60_000, 128, generator=g)).cuda()
    q = (base[torch.randint(0, 200, (512,), generator=g)] + 0.1 * torch.randn(512, 128, generator=g)).cuda()
    d_tc, i_tc, info = knn_f32(q, db, 10, mode=_lib.FL_KNN_BF16_RERANK, second_stage=False)
    d_ex, i_ex, _ = knn_f32(q, db, 10, mode=_lib.FL_KNN_EXACT_SIMT)
    # Neighbours here are ~2.5 apart from the query at norms ~128, where the fp32 expansion the
    # oracle uses is itself only good to ~1e-5 relative; the yardstick is fp64 brute force.
    qd, dbd = q.double(), db.double()
    d64 = (qd * qd).sum(-1, keepdim=True) + (dbd * dbd).sum(-1)[None, :] - 2.0 * qd @ dbd.T
    ref_i = d64.topk(10, dim=1, largest=False).indices.cpu().numpy()
    res = parity.knn_parity(q.cpu().numpy(), db.cpu().numpy(), d_tc.cpu().numpy(), i_tc.cpu().numpy(), ref_i)
    assert res["ok"], res
    assert info["fallback_rows"] > 0
    same = (i_tc == i_ex).all(dim=1).float().mean().item()
    assert same > 0.99, same


def _near_duplicates(m, nq, d, seed, spread=0.1, centres=200):
    g = torch.Generator().manual_seed(seed)
    base = torch.randn(centres, d, generator=g)
    db = base[torch.randint(0, centres, (m,), generator=g)] + spread * torch.randn(m, d, generator=g)
    q = base[torch.randint(0, centres, (nq,), generator=g)] + spread * torch.randn(nq, d, generator=g)
    return q.cuda(), db.cuda()


def _fp64_neighbours(q, db, k):
    qd, dbd = q.double(), db.double()
    d64 = (qd * qd).sum(-1, keepdim=True) + (dbd * dbd).sum(-1)[None, :] - 2.0 * qd @ dbd.T
    return d64.topk(k, dim=1, largest=False).indices.cpu().numpy()


@pytest.mark.parametrize("m,nq,d,k", [(60_000, 512, 128, 10), (90_000, 700, 64, 5), (50_000, 300, 100, 32),
                                      (150_000, 2000, 128, 16)])
def test_second_stage_proves_what_the_bf16_pass_cannot(m, nq, d, k):
    """Near-duplicate data: the bf16 proof rejects many rows; the split-plane tensor-core stage
    (error bound a hundred times smaller) proves nearly all of them, the exact CUDA-core pass
    takes what is left, and the neighbours equal fp64 brute force either way."""
    q, db = _near_duplicates(m, nq, d, seed=m + k)
    d_1, i_1, info1 = knn_f32(q, db, k, mode=_lib.FL_KNN_BF16_RERANK, second_stage=False)
    d_2, i_2, info2 = knn_f32(q, db, k, mode=_lib.FL_KNN_BF16_RERANK, second_stage=True)
    assert info2["second_stage"] and not info1["second_stage"]
    ref_i = _fp64_neighbours(q, db, k)
    for d_, i_ in ((d_1, i_1), (d_2, i_2)):
        res = parity.knn_parity(q.cpu().numpy(), db.cpu().numpy(), d_.cpu().numpy(), i_.cpu().numpy(), ref_i)
        assert res["ok"], res
    assert info1["fallback_rows"] > 0, "the generator no longer defeats the bf16 proof"
    assert info2["stage2_rows"] == info1["fallback_rows"]
    assert info2["fallback_rows"] <= max(1, info1["fallback_rows"] // 50), (info1, info2)


def test_second_stage_overflow_goes_to_the_exact_pass():
    """More rejected rows than the second stage holds (every query up to 65 536, a quarter of them
    beyond): the surplus takes the exact pass directly and every row is still correct."""
    q, db = _near_duplicates(20_000, 70_000, 64, seed=77, centres=20)
    d_2, i_2, info = knn_f32(q, db, 5, mode=_lib.FL_KNN_BF16_RERANK, second_stage=True)
    assert info["stage2_rows"] == 65_536, info
    assert info["fallback_rows"] > 0
    sub = torch.arange(0, 70_000, 35, device="cuda")
    ref_i = _fp64_neighbours(q[sub], db, 5)
    res = parity.knn_parity(q[sub].cpu().numpy(), db.cpu().numpy(), d_2[sub].cpu().numpy(), i_2[sub].cpu().numpy(), ref_i)
    assert res["ok"], res


def test_second_stage_idle_on_well_separated_data():
    g = torch.Generator().manual_seed(5)
    db = torch.randn(100_000, 128, generator=g).cuda()
    q = torch.randn(400, 128, generator=g).cuda()
    d_1, i_1, _ = knn_f32(q, db, 10, mode=_lib.FL_KNN_BF16_RERANK, second_stage=False)
    d_2, i_2, info = knn_f32(q, db, 10, mode=_lib.FL_KNN_BF16_RERANK, second_stage=True)
    assert info["stage2_rows"] == 0 and info["fallback_rows"] == 0
    assert torch.equal(i_1, i_2) and torch.equal(d_1, d_2)


def test_no_split_plane_beyond_128_features():
    lib = _lib.load()
    assert lib.fl_knn_split_plane_bytes(1000, 129) == 0
    assert lib.fl_knn_split_plane_bytes(1000, 128) > 0
    g = torch.Generator().manual_seed(6)
    db = torch.randn(30_000, 200, generator=g).cuda()
    q = torch.randn(600, 200, generator=g).cuda()
    _, _, info = knn_f32(q, db, 10, mode=_lib.FL_KNN_BF16_RERANK, second_stage=True)
    assert not info["second_stage"]


@pytest.mark.parametrize("nq,m,d,k", [(200, 60_000, 384, 10), (129, 30_000, 512, 10), (100, 20_000, 300, 32), (300, 70_000, 512, 1),
                                      (64, 9_000, 257, 16)])
def test_bf16_mode_up_to_512_features(nq, m, d, k):
    """256 < d <= 512: the resident query tile leaves no room for pools in shared memory, so every k takes
    the global-memory pools of the large-k mode; same proof, same result as the oracle."""
    g = torch.Generator().manual_seed(nq + m + d)
    db = torch.randn(m, d, generator=g)
    q = torch.randn(nq, d, generator=g)
    _, ref_i = oracle.knn_naive(q.numpy(), db.numpy(), k)
    d_tc, i_tc, info = knn_f32(q.cuda(), db.cuda(), k, mode=_lib.FL_KNN_BF16_RERANK)
    res = parity.knn_parity(q.numpy(), db.numpy(), d_tc.cpu().numpy(), i_tc.cpu().numpy(), ref_i)
    assert res["ok"], (res, info)
    assert info["fallback_rows"] <= nq // 10, info
    lib = _lib.load()
    assert lib.fl_knn_workspace_bytes(nq, m, 513, k, _lib.FL_KNN_BF16_RERANK) >= 0
    with pytest.raises(NotImplementedError):
        knn_f32(q.cuda()[:, :1].expand(nq, 513).contiguous(), db.cuda()[:, :1].expand(m, 513).contiguous(), k,
                mode=_lib.FL_KNN_BF16_RERANK)


BIG_K_SHAPES = [(64, 3000, 64, 17), (129, 20_000, 128, 32), (300, 60_000, 128, 100), (500, 150_000, 64, 64),
                (100, 400, 96, 112), (257, 300_001, 96, 100), (33, 50_000, 200, 50)]


@pytest.mark.parametrize("nq,m,d,k", BIG_K_SHAPES)
def test_bf16_mode_large_k_vs_oracle(nq, m, d, k):
    """16 < k <= 112: pools of 256 entries in global memory, block-per-query finalisation."""
    g = torch.Generator().manual_seed(nq + m + k)
    db = torch.randn(m, d, generator=g)
    q = torch.randn(nq, d, generator=g)
    _, ref_i = oracle.knn_naive(q.numpy(), db.numpy(), k)
    d_tc, i_tc, info = knn_f32(q.cuda(), db.cuda(), k, mode=_lib.FL_KNN_BF16_RERANK)
    res = parity.knn_parity(q.numpy(), db.numpy(), d_tc.cpu().numpy(), i_tc.cpu().numpy(), ref_i)
    assert res["ok"], (res, info)
    dn = d_tc.cpu().numpy()
    assert (np.diff(dn, axis=1) >= 0).all()


def test_large_k_mixture_matches_exact_mode():
    """Clustered non-negative data (the benchmark's distribution), k = 100: tensor-core mode and
    exact mode agree, and most rows are proven without the exact path."""
    from flashlib_b200 import synthetic
    X, Q = synthetic.mixture(200_000, 128, 512, 5, nq=600, clamp=True)
    X, Q = X.cuda(), Q.cuda()
    d_tc, i_tc, info = knn_f32(Q, X, 100, mode=_lib.FL_KNN_BF16_RERANK)
    d_ex, i_ex, _ = knn_f32(Q, X, 100, mode=_lib.FL_KNN_EXACT_SIMT)
    assert info["fallback_rows"] < 60, info
    torch.testing.assert_close(d_tc, d_ex, rtol=1e-4, atol=1e-4)
    same = (i_tc == i_ex).float().mean().item()
    assert same > 0.999, same


def test_plane_cache_does_not_outlive_its_tensor():
    """A new database that the allocator places at the address of a freed one (same shape) must
    get its own operand plane."""
    g = torch.Generator().manual_seed(3)
    q = torch.randn(64, 64, generator=g).cuda()
    for _ in range(3):
        db = torch.randn(20_000, 64, generator=g).cuda()
        d_tc, i_tc, info = knn_f32(q, db, 10, mode=_lib.FL_KNN_BF16_RERANK)
        d_ex, i_ex, _ = knn_f32(q, db, 10, mode=_lib.FL_KNN_EXACT_SIMT)
        assert info["fallback_rows"] < 8, info
        assert (i_tc == i_ex).float().mean().item() > 0.999
        del db


def test_unsupported_k_raises_and_auto_falls_back():
    g = torch.Generator().manual_seed(1)
    db = torch.randn(5000, 32, generator=g).cuda()
    q = torch.randn(10, 32, generator=g).cuda()
    with pytest.raises(NotImplementedError):
        fl.flash_knn(q, db, 200, mode="bf16")
    vals, idxs = fl.flash_knn(q, db, 200)        # auto: exact path
    assert vals.shape == (10, 200)


def test_cta_pair_variant_in_a_subprocess():
    """The cta_group::2 variant of the scoring kernel (two CTAs share every database tile) is
    switched on by an environment variable that the library reads once, so it runs in its own
    process: same neighbours as the exact mode, no rows on the exact path beyond a handful."""
    import os
    import subprocess
    import sys
    code = (
        "import torch\n"
        "from flashlib_b200 import _lib\n"
        "from flashlib_b200.knn import knn_f32\n"
        "g = torch.Generator().manual_seed(11)\n"
        "db = torch.randn(150_000, 128, generator=g).cuda(); q = torch.randn(1000, 128, generator=g).cuda()\n"
        "d1, i1, info = knn_f32(q, db, 10, mode=_lib.FL_KNN_BF16_RERANK)\n"
        "d0, i0, _ = knn_f32(q, db, 10, mode=_lib.FL_KNN_EXACT_SIMT)\n"
        "assert info['status'][0].item() == 0, info\n"
        "assert info['fallback_rows'] < 20, info\n"
        "assert (i1 == i0).float().mean().item() > 0.999\n"
        "torch.testing.assert_close(d1, d0, rtol=1e-4, atol=1e-4)\n"
        "print('pair ok')\n")
    env = dict(os.environ, FLASHLIB_B200_TC_PAIR="1")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, "-c", code], cwd=root, env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and "pair ok" in out.stdout, out.stdout + out.stderr


def test_every_query_can_take_the_exact_path():
    """A large common offset makes the scoring error bound swamp every gap: all 9,000 queries fail
    their proof, more than the fallback list once held, and every one must come back exact."""
    g = torch.Generator().manual_seed(17)
    db = (torch.randn(40_000, 64, generator=g) + 30.0).cuda()
    q = (torch.randn(9_000, 64, generator=g) + 30.0).cuda()
    d_tc, i_tc, info = knn_f32(q, db, 10, mode=_lib.FL_KNN_BF16_RERANK, second_stage=False)
    assert info["status"][_lib.FL_STATUS_ERROR].item() == 0
    assert info["fallback_rows"] > 8_000, info["fallback_rows"]
    qd, dbd = q.double(), db.double()
    d64 = (qd * qd).sum(-1, keepdim=True) + (dbd * dbd).sum(-1)[None, :] - 2.0 * qd @ dbd.T
    ref_i = d64.topk(10, dim=1, largest=False).indices.cpu().numpy()
    res = parity.knn_parity(q.cpu().numpy(), db.cpu().numpy(), d_tc.cpu().numpy(), i_tc.cpu().numpy(), ref_i)
    assert res["ok"], res


def test_bounded_wait_runs_out_and_the_gpu_stays_usable():
    """The producer leaves out one operand load (experiment flag 32) and the wait limit is 1 ms:
    the MMA lane's wait for that load runs out, the kernel ends by itself, the status words say
    where, the Python mirror raises -- and the next ordinary call returns correct neighbours."""
    from flashlib_b200.knn import _raise_on_status
    lib = _lib.load()
    g = torch.Generator().manual_seed(23)
    db = torch.randn(100_000, 128, generator=g).cuda()
    q = torch.randn(512, 128, generator=g).cuda()
    try:
        _lib.check(lib.fl_debug_tc_experiment(32, 1000))
        _, _, info = knn_f32(q, db, 10, mode=_lib.FL_KNN_BF16_RERANK, check_status=False)
        torch.cuda.synchronize()
        st = info["status"].tolist()
    finally:
        _lib.check(lib.fl_debug_tc_experiment(0, 0))
    assert st[_lib.FL_STATUS_ERROR] == _lib.FL_ETIMEOUT, st
    assert st[_lib.FL_STATUS_WHERE] >> 16 == 5, hex(st[_lib.FL_STATUS_WHERE])      # role 5: the MMA lane
    with pytest.raises(_lib.FlashlibError):
        _raise_on_status(st)
    d_tc, i_tc, info = knn_f32(q, db, 10, mode=_lib.FL_KNN_BF16_RERANK)
    d_ex, i_ex, _ = knn_f32(q, db, 10, mode=_lib.FL_KNN_EXACT_SIMT)
    assert info["status"][_lib.FL_STATUS_ERROR].item() == 0
    torch.testing.assert_close(d_tc, d_ex, rtol=1e-4, atol=1e-4)
    assert (i_tc == i_ex).float().mean().item() > 0.999


def test_timing_experiment_flags_invalidate_the_status():
    """A launch that leaves work out for a timing run says so in its status words."""
    from flashlib_b200.knn import _raise_on_status
    lib = _lib.load()
    g = torch.Generator().manual_seed(24)
    db = torch.randn(100_000, 64, generator=g).cuda()
    q = torch.randn(256, 64, generator=g).cuda()
    try:
        _lib.check(lib.fl_debug_tc_experiment(1, 0))
        _, _, info = knn_f32(q, db, 10, mode=_lib.FL_KNN_BF16_RERANK, check_status=False)
        torch.cuda.synchronize()
        st = info["status"].tolist()
    finally:
        _lib.check(lib.fl_debug_tc_experiment(0, 0))
    assert st[_lib.FL_STATUS_ERROR] == _lib.FL_EUNSUPPORTED, st
    with pytest.raises(_lib.FlashlibError):
        _raise_on_status(st)
