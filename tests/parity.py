"""Tie-tolerant comparators used by the parity tests.

Rules (from the task statement): neighbour index sets must be identical per row except
where the competing distances differ by <= 1e-5 relative; distances within 1e-4 relative;
k-means labels identical outside the same tie band.  The reference's own tie-tolerant
comparator is tests/test_knn_blackwell_search_tc.py:27-43.
"""
from __future__ import annotations

import numpy as np

REL_TIE = 1e-5
REL_DIST = 1e-4


def _exact_d(q_row, rows):
    diff = rows.astype(np.float64) - q_row.astype(np.float64)[None, :]
    return (diff * diff).sum(-1)


def knn_parity(q, db, got_d, got_i, ref_i, *, rel_tie=REL_TIE, rel_dist=REL_DIST):
    """Returns a dict with the number of rows whose sets differ outside the tie band and the
    worst relative distance error of ``got_d`` against fp64 ``sum (q-x)^2``."""
    q = np.asarray(q, dtype=np.float32)
    db = np.asarray(db, dtype=np.float32)
    got_i = np.asarray(got_i).astype(np.int64)
    ref_i = np.asarray(ref_i).astype(np.int64)
    got_d = np.asarray(got_d, dtype=np.float64)
    n, k = got_i.shape
    bad_rows = []
    set_mismatch = 0
    worst_rel = 0.0
    not_sorted = 0
    for r in range(n):
        gi, ri = got_i[r], ref_i[r]
        ex = _exact_d(q[r], db[np.clip(gi, 0, db.shape[0] - 1)])
        scale = float((q[r].astype(np.float64) ** 2).sum()) + 1e-30
        rel = np.abs(got_d[r] - ex) / np.maximum(ex, 1e-6 * scale)
        worst_rel = max(worst_rel, float(rel.max()))
        if np.any(np.diff(got_d[r]) < -1e-6 * scale):
            not_sorted += 1
        sg, sr = set(gi.tolist()), set(ri.tolist())
        if len(sg) != k:
            bad_rows.append(r)
            continue
        if sg == sr:
            continue
        set_mismatch += 1
        only_g = np.array(sorted(sg - sr))
        only_r = np.array(sorted(sr - sg))
        dg = _exact_d(q[r], db[only_g])
        dr = _exact_d(q[r], db[only_r])
        lo = min(dg.min(), dr.min())
        hi = max(dg.max(), dr.max())
        if hi - lo > rel_tie * max(hi, 1e-30) + 1e-7 * scale:
            bad_rows.append(r)
    return {"rows": n, "set_mismatch_rows": set_mismatch, "bad_rows": bad_rows,
            "worst_rel_dist_err": worst_rel, "unsorted_rows": not_sorted,
            "ok": not bad_rows and worst_rel <= rel_dist and not_sorted == 0}


def label_parity(x, centroids, got, ref, *, rel_tie=REL_TIE):
    """k-means labels: every differing label must point at a centroid whose true squared
    distance is within the tie band of the best one."""
    got = np.asarray(got).astype(np.int64)
    ref = np.asarray(ref).astype(np.int64)
    diff = np.nonzero(got != ref)[0]
    bad = 0
    if diff.size:
        xs = np.asarray(x, dtype=np.float64)[diff]
        c = np.asarray(centroids, dtype=np.float64)
        dg = ((xs - c[got[diff]]) ** 2).sum(-1)
        dr = ((xs - c[ref[diff]]) ** 2).sum(-1)
        scale = (xs * xs).sum(-1)
        bad = int(np.sum(np.abs(dg - dr) > rel_tie * np.maximum(dg, dr) + 1e-7 * scale))
    return {"n": int(got.size), "differ": int(diff.size), "bad": bad, "ok": bad == 0}


def rel_close(a, b, rel=REL_DIST, atol=0.0):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return bool(np.all(np.abs(a - b) <= rel * np.abs(b) + atol))
