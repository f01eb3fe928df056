#!/usr/bin/env python
"""Benchmark of the fused exact-kNN hot path: queries/s on the 1,000,000 x 128 fp32, k=10
configuration, database row-sharded over the GPUs of one box.

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # CPU restatement of the reference's torch path

A step is one batch of queries through the hot path.  Scaling is weak: every rank brings
10,000 queries per step (global batch 10,000 x N) and holds 1/N of the database rows; the ranks
share their threshold seeds (one all-reduce), score, exchange their candidates (all-to-all, or
all-gather with --result replicated) and merge.  One JSON line is printed by rank 0; it carries
a "parity" object (a sample of the last step's results against the CPU oracle, at every N),
and at N = 1 a "secondary" object (the k-means, IVF-Flat and k=100 configurations, timed and
checked the same way) and a "sustained" object (the same loop run for seconds).

``--workload knn_100m`` runs the same flow on the sharded configuration (100,000,000 x 96 rows
~ N(0,1) split over the ranks, 100,000 queries per step, k = 100; strong scaling: the total work
is fixed).  The other ``--workload`` names time the remaining configurations on one GPU.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

K_NEIGHBOURS = 10
DB_ROWS = 1_000_000
DIM = 128
QUERIES_PER_GPU = 10_000
N_COMP = 4096
SEED = 2
# dram__bytes_read.sum + dram__bytes_write.sum of one knn_tc_kernel launch on this workload (ncu capture
# of the 1M x 128, 10,000-query case)
TC_KERNEL_DRAM_BYTES_PER_LAUNCH = 563_872_768
METRIC = "exact_knn_queries_per_sec"
UNIT = "queries/s"


SCALING = "weak"
WORKLOAD = "knn_1m"


def workload_name(n_gpus: int) -> str:
    if WORKLOAD == "knn_100m":
        return (f"knn_100m: exact kNN, database {DB_ROWS}x{DIM} fp32 ~ N(0,1) row-sharded over the ranks (drawn on "
                f"each device, seed {SEED} + rank), {QUERIES_PER_GPU} queries ~ N(0,1) per step in total, "
                f"k={K_NEIGHBOURS}, squared L2")
    return (f"knn_1m: exact kNN, database {DB_ROWS}x{DIM} fp32 (4096-component gaussian mixture, "
            f"clamped >= 0, seed {SEED}), {QUERIES_PER_GPU} queries per GPU per step, k={K_NEIGHBOURS}, squared L2")


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"source": "measured", "hbm_gbs": p.get("hbm_gbs"), "bf16_tflops": p.get("bf16_tflops"),
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained")}
    return {"source": "fallback", "hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


class ClockSampler:
    """Samples the SM clock and the throttle reasons of one GPU through NVML (read-only)
    every few milliseconds while the timed region runs."""
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown"}

    def __init__(self, cuda_index: int):
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = False
        self._thread = None
        self.error = None
        try:
            import pynvml
            self.nv = pynvml
            pynvml.nvmlInit()
            pr = torch.cuda.get_device_properties(cuda_index)
            bus = f"{getattr(pr, 'pci_domain_id', 0):08x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
            self.h = pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception as e:  # noqa: BLE001
            self.error = f"NVML unavailable: {e}"

    def _run(self):
        nv = self.nv
        while not self._stop:
            try:
                self.samples.append(float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:  # noqa: BLE001
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception as e:  # noqa: BLE001
                self.error = str(e)
                break
            time.sleep(0.004)

    def start(self):
        if self.error:
            return
        import threading
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def stop(self):
        if self._thread is not None:
            self._stop = True
            self._thread.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "samples": 0,
                    "reasons": [self.error or "no samples"]}
        return {"sm_mhz": statistics.median(self.samples), "sm_min_mhz": min(self.samples),
                "sm_max_mhz": self.max_mhz, "samples": len(self.samples), "reasons": sorted(self.reasons)}


def make_workload(rank: int, world: int):
    from flashlib_b200 import synthetic
    from flashlib_b200.sharded import shard_bounds
    if WORKLOAD == "knn_100m":
        # too large to draw on the host in bench time: every rank draws its own rows on its device
        s, e = shard_bounds(DB_ROWS, world, rank)
        g = torch.Generator(device="cuda").manual_seed(SEED + 1000 * (rank + 1))
        X = torch.randn(e - s, DIM, generator=g, device="cuda")
        Q = torch.randn(QUERIES_PER_GPU, DIM, generator=torch.Generator().manual_seed(SEED))
        return X, Q, s, e
    X, Q = synthetic.mixture(DB_ROWS, DIM, N_COMP, SEED, nq=QUERIES_PER_GPU * world, clamp=True)
    s, e = shard_bounds(DB_ROWS, world, rank)
    return X, Q, s, e


def config_dict(world: int, result: str, resolved_tc: bool, nq: int) -> dict:
    """The `config` object of the JSON line: the same for both arms (the reference arm reports the
    configuration it stands in for; what it ran itself is in its `cpu_baseline.sample`)."""
    from flashlib_b200.sharded import shard_bounds
    rows_local = shard_bounds(DB_ROWS, world, 0)
    plane_bytes = (rows_local[1] - rows_local[0]) * (((DIM + 63) // 64) * 64 + 16) * 2
    owned = shard_bounds(nq, world, 0)
    flushes = plane_bytes < (256 << 20)
    return {"workload": workload_name(world), "db_rows": DB_ROWS, "dim": DIM, "k": K_NEIGHBOURS,
            "queries_per_step": nq,
            "sharding": (f"database rows over {world} ranks; every rank scores all of the step's queries; "
                         + ("threshold seeds shared by one all-reduce; " if K_NEIGHBOURS <= 16 else "")
                         + ("candidates exchanged all-to-all, every rank merges and returns its own "
                            f"{owned[1] - owned[0]} queries" if result == "owner" else
                            "candidates all-gathered, every rank merges and returns all queries"))
            if world > 1 else "single GPU",
            "mode": ("tcgen05 bf16 candidates + exact fp32 re-rank + verified fallback" if resolved_tc else
                     "exact fp32 CUDA-core scoring + exact re-rank"),
            "l2": ("a 160 MB buffer (larger than the 126 MB L2) is overwritten before every step (inside the timed region): a rank's "
                   f"operand plane is {plane_bytes >> 20} MB" if flushes else
                   f"no flush needed: each step streams the rank's operand plane ({plane_bytes >> 20} MB), "
                   "larger than the 126 MB L2")}


def knn_rows_agree(q, got_d, got_i, ref_d, ref_i, rel_tie=1e-5, rel_dist=1e-4):
    """Number of rows of (got_d, got_i) that disagree with the oracle's (ref_d, ref_i) when the
    database rows are not at hand to recompute distances in fp64: index sets must be equal except
    between candidates whose distances differ by <= rel_tie relative, distances within rel_dist
    relative.  The oracle's distances come from the fp32 expansion ||q||^2 + ||x||^2 - 2 q.x, whose
    round-off (about 1e-6 of the norms) is added to both bands."""
    q = np.asarray(q, np.float64)
    got_d, ref_d = np.asarray(got_d, np.float64), np.asarray(ref_d, np.float64)
    got_i, ref_i = np.asarray(got_i, np.int64), np.asarray(ref_i, np.int64)
    bad = 0
    for r in range(got_i.shape[0]):
        hi_all = float(max(ref_d[r].max(), got_d[r].max()))
        noise = 1e-6 * (2.0 * float((q[r] * q[r]).sum()) + hi_all)
        if np.any(np.abs(np.sort(got_d[r]) - np.sort(ref_d[r])) > rel_dist * hi_all + noise):
            bad += 1
            continue
        sg, sr = set(got_i[r].tolist()), set(ref_i[r].tolist())
        if sg == sr:
            continue
        dg = [got_d[r][j] for j in range(got_i.shape[1]) if got_i[r][j] not in sr]
        dr = [ref_d[r][j] for j in range(ref_i.shape[1]) if ref_i[r][j] not in sg]
        lo, hi = min(dg + dr), max(dg + dr)
        if len(sg) != got_i.shape[1] or hi - lo > rel_tie * hi + noise:
            bad += 1
    return bad


def cpu_baseline_run(X: torch.Tensor, Q: torch.Tensor, n_queries: int, repeats: int = 1):
    """Times the torch-CPU restatement of the reference's chunked path (`oracle/oracle_torch.py`,
    the same ATen operators the reference calls) on `n_queries` queries against the whole
    database; returns (queries/s, threads)."""
    from oracle import oracle_torch
    torch.set_num_threads(os.cpu_count() or 1)
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        oracle_torch.knn_chunked(Q[:n_queries], X, K_NEIGHBOURS, chunk_size=8192)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return n_queries / best, torch.get_num_threads()


def run_reference(args, rank: int, world: int):
    if rank != 0:
        return
    # torch.distributed.run exports OMP_NUM_THREADS=1: the CPU arm takes every host core it can get
    torch.set_num_threads(os.cpu_count() or 1)
    from flashlib_b200 import _lib, synthetic
    X, Q = synthetic.mixture(DB_ROWS, DIM, N_COMP, SEED, nq=QUERIES_PER_GPU, clamp=True)
    from oracle import oracle_torch
    sample = 1024
    for _ in range(min(args.warmup, 1)):
        oracle_torch.knn_chunked(Q[:64], X, K_NEIGHBOURS, chunk_size=8192)
    t0 = time.perf_counter()
    for s in range(args.steps):
        lo = (s * sample) % (QUERIES_PER_GPU - sample + 1)
        oracle_torch.knn_chunked(Q[lo:lo + sample], X, K_NEIGHBOURS, chunk_size=8192)
    dt = time.perf_counter() - t0
    qps = args.steps * sample / dt
    cores = torch.get_num_threads()
    nq = QUERIES_PER_GPU * args.gpus
    rows0 = DB_ROWS // max(args.gpus, 1)
    tc = _lib.load().fl_knn_resolve_mode(nq, rows0, DIM, K_NEIGHBOURS) == _lib.FL_KNN_BF16_RERANK
    line = {
        "impl": "reference", "metric": METRIC, "value": qps, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_dict(args.gpus, args.result, tc, nq),
        "cpu_baseline": {"value": qps, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"{sample} queries per step against all {DB_ROWS} rows on {cores} host threads "
                                   "(os.cpu_count()); torch-CPU restatement of knn_torch_chunked, chunk 8192"},
        "e2e": {"value": qps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def _reference_gpu_child(dtype_name: str, backend):
    """One measurement of the UNMODIFIED reference's GPU kernels (installed under baseline/_ref by
    `python -m pip install --no-index --no-build-isolation --no-deps --target baseline/_ref
    <reference tree>`) through its public `flashlib.flash_knn`, on the headline shape, in a process
    of its own.  Prints one JSON line: time per 10,000 queries and recall@10 against this library's
    exact result."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    out = {"impl": "reference-gpu", "dtype": dtype_name, "backend": backend or "auto"}
    if not os.path.isdir(os.path.join(ref_dir, "flashlib")):
        out["unavailable"] = "baseline/_ref holds no installed reference"
        print(json.dumps(out), flush=True)
        return
    from flashlib_b200 import flash_knn as ours, synthetic
    sys.path.insert(0, ref_dir)
    try:
        import flashlib                      # noqa: F401  (the reference)
        from flashlib import flash_knn as theirs
    except Exception as e:  # noqa: BLE001
        out["unavailable"] = f"import of the reference failed: {type(e).__name__}: {e}"[:300]
        print(json.dumps(out), flush=True)
        return
    X, Q = synthetic.mixture(DB_ROWS, DIM, N_COMP, SEED, nq=QUERIES_PER_GPU, clamp=True)
    Xd, Qd = X.cuda(), Q.cuda()
    _, exact_i = ours(Qd, Xd, K_NEIGHBOURS)
    dt = {"fp32": torch.float32, "bf16": torch.bfloat16}[dtype_name]
    xq, xc = Qd.to(dt), Xd.to(dt)
    try:
        t0 = time.perf_counter()
        vals, idxs = theirs(xq, xc, K_NEIGHBOURS, backend=backend)
        torch.cuda.synchronize()
        out["first_call_s"] = time.perf_counter() - t0           # includes the JIT compilation
        ms = _time_steps(lambda: theirs(xq, xc, K_NEIGHBOURS, backend=backend), 10, 3)
    except Exception as e:  # noqa: BLE001
        out["unavailable"] = f"the reference's kernel did not run: {type(e).__name__}: {e}"[:300]
        print(json.dumps(out), flush=True)
        return
    a, b = idxs.cpu().numpy(), exact_i.cpu().numpy()
    recall = float(np.mean([len(set(r.tolist()) & set(t.tolist())) / K_NEIGHBOURS for r, t in zip(a, b)]))
    same_rows = float(np.mean([set(r.tolist()) == set(t.tolist()) for r, t in zip(a, b)]))
    out.update({"ms_per_step": ms, "value": QUERIES_PER_GPU / (ms * 1e-3), "unit": UNIT,
                "tensor_tflops_algorithmic": 2.0 * QUERIES_PER_GPU * DB_ROWS * DIM / (ms * 1e-3) / 1e12,
                "recall_at_10_vs_exact": recall, "rows_with_the_exact_set": same_rows,
                "note": "exact = this library's result for the fp32 inputs; the bf16 legs search the bf16-rounded data"})
    print(json.dumps(out), flush=True)


def _reference_gpu_child_other(which: str, dtype_name: str):
    """Same for the other two configurations: `kmeans` = the reference's `flash_kmeans` on 1,000,000 x 128,
    K = 1024, 20 Lloyd iterations from the first K rows; `ivf` = its `IVFFlat(nlist=1024, nprobe=16,
    niter=10)` fitted and searched with 10,000 queries, k = 10.  Quality beside the time: inertia
    against this library's run from the same start; recall@10 against this library's exact kNN."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    out = {"impl": "reference-gpu", "workload": {"kmeans": "kmeans_1m", "ivf": "ivf_1m"}[which], "dtype": dtype_name}
    if not os.path.isdir(os.path.join(ref_dir, "flashlib")):
        out["unavailable"] = "baseline/_ref holds no installed reference"
        print(json.dumps(out), flush=True)
        return
    import flashlib_b200 as ours
    from flashlib_b200 import synthetic
    sys.path.insert(0, ref_dir)
    try:
        import flashlib as theirs
    except Exception as e:  # noqa: BLE001
        out["unavailable"] = f"import of the reference failed: {type(e).__name__}: {e}"[:300]
        print(json.dumps(out), flush=True)
        return
    dt = {"fp32": torch.float32, "bf16": torch.bfloat16}[dtype_name]
    try:
        if which == "kmeans":
            cfg = synthetic.CONFIGS["kmeans_1m"]
            X, _ = synthetic.mixture(cfg["n"], cfg["d"], cfg["n_comp"], cfg["seed"])
            Xd = X.cuda()
            init = Xd[:cfg["K"]].clone()

            def inertia(c):
                lab = ours.euclid_assign_triton(Xd[None], c.float().reshape(1, cfg["K"], -1))[0].long()
                return float(((Xd - c.float().reshape(cfg["K"], -1)[lab]) ** 2).sum())
            _, c_ours, _ = ours.flash_kmeans(Xd, cfg["K"], max_iters=cfg["iters"], init_centroids=init)
            ms_ours = _time_steps(lambda: ours.flash_kmeans(Xd, cfg["K"], max_iters=cfg["iters"], init_centroids=init), 3, 1)
            xr, ir = Xd.to(dt), init.to(dt)
            run = lambda: theirs.flash_kmeans(xr, cfg["K"], max_iters=cfg["iters"], tol=0.0, init_centroids=ir)   # noqa: E731
            t0 = time.perf_counter()
            _, c_ref, _ = run()
            torch.cuda.synchronize()
            out["first_call_s"] = time.perf_counter() - t0
            ms = _time_steps(run, 3, 1)
            out.update({"ms_per_step": ms, "unit": "ms per 20 Lloyd iterations", "ours_ms_per_step": ms_ours,
                        "inertia_over_ours": inertia(c_ref) / inertia(c_ours)})
        else:
            cfg = synthetic.CONFIGS["ivf_1m"]
            X, Q = synthetic.mixture(cfg["n"], cfg["d"], cfg["n_comp"], cfg["seed"], nq=cfg["nq"], clamp=True)
            Xd, Qd = X.cuda(), Q.cuda()
            _, exact_i = ours.flash_knn(Qd[:2000], Xd, cfg["k"])
            mine = ours.IVFFlat(nlist=cfg["nlist"], nprobe=cfg["nprobe"], niter=10, seed=cfg["seed"]).fit(Xd)
            ms_ours = _time_steps(lambda: mine.kneighbors(Qd, cfg["k"]), 5, 2)
            _, i_ours = mine.kneighbors(Qd, cfg["k"])
            xr, qr = Xd.to(dt), Qd.to(dt)
            t0 = time.perf_counter()
            ref = theirs.IVFFlat(nlist=cfg["nlist"], nprobe=cfg["nprobe"], niter=10, seed=cfg["seed"]).fit(xr)
            torch.cuda.synchronize()
            out["build_s_first_call"] = time.perf_counter() - t0
            _, i_ref = ref.kneighbors(qr, cfg["k"])
            torch.cuda.synchronize()
            ms = _time_steps(lambda: ref.kneighbors(qr, cfg["k"]), 5, 2)

            def recall(i_):
                a, b = i_[:2000].cpu().numpy(), exact_i.cpu().numpy()
                return float(np.mean([len(set(r.tolist()) & set(t.tolist())) / cfg["k"] for r, t in zip(a, b)]))
            out.update({"ms_per_step": ms, "unit": "ms per 10,000 queries", "ours_ms_per_step": ms_ours,
                        "recall_at_10_vs_exact": recall(i_ref), "ours_recall_at_10_vs_exact": recall(i_ours)})
    except Exception as e:  # noqa: BLE001
        out["unavailable"] = f"the reference did not run: {type(e).__name__}: {e}"[:300]
    print(json.dumps(out), flush=True)


def run_reference_gpu(args):
    """The reference's own GPU kernels on this box, beside ours: every leg in a child process with a
    time limit (a leg that does not come back is reported, not retried)."""
    legs = [("fp32", "triton"), ("bf16", "triton"), ("bf16", None), ("fp32", "kmeans"), ("bf16", "kmeans"), ("fp32", "ivf")]
    if args.ref_leg:
        d_, b_ = args.ref_leg.split(":")
        if b_ in ("kmeans", "ivf"):
            _reference_gpu_child_other(b_, d_)
        else:
            _reference_gpu_child(d_, None if b_ == "auto" else b_)
        return
    for d_, b_ in legs:
        cmd = [sys.executable, os.path.abspath(__file__), "--impl", "reference-gpu", "--ref-leg", f"{d_}:{b_ or 'auto'}"]
        try:
            res = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=420)
            lines = [l for l in res.stdout.splitlines() if l.startswith("{")]
            print(lines[-1] if lines else json.dumps({"impl": "reference-gpu", "dtype": d_, "backend": b_ or "auto",
                                                      "unavailable": (res.stderr or "no output")[-300:]}), flush=True)
        except subprocess.TimeoutExpired:
            print(json.dumps({"impl": "reference-gpu", "dtype": d_, "backend": b_ or "auto",
                              "unavailable": "no result within 420 s"}), flush=True)
    # ours, same process layout, for the table
    import flashlib_b200 as fl
    from flashlib_b200 import synthetic
    X, Q = synthetic.mixture(DB_ROWS, DIM, N_COMP, SEED, nq=QUERIES_PER_GPU, clamp=True)
    Xd, Qd = X.cuda(), Q.cuda()
    ms = _time_steps(lambda: fl.flash_knn(Qd, Xd, K_NEIGHBOURS), 10, 3)
    print(json.dumps({"impl": "ours", "dtype": "fp32 in, exact fp32 out", "ms_per_step": ms,
                      "value": QUERIES_PER_GPU / (ms * 1e-3), "unit": UNIT, "recall_at_10_vs_exact": 1.0}), flush=True)


def _time_steps(fn, steps, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def _roof(bound: str, work: float, ms: float, peaks: dict) -> dict:
    """Roofline entry of a secondary workload: algorithmic FLOP (tensor) or bytes (hbm) per step
    over the step time, against the measured burst peak."""
    if bound == "tensor":
        achieved, peak, unit = work / (ms * 1e-3) / 1e12, peaks["bf16_tflops"], "TFLOP/s"
    else:
        achieved, peak, unit = work / (ms * 1e-3) / 1e9, peaks["hbm_gbs"], "GB/s"
    return {"bound": bound, "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak,
            "algorithmic_work_per_step": work, "peak_source": peaks["source"]}


def secondary_knn_k100(Xd, Qd, X, Q, steps, warm, mode_name, peaks):
    import flashlib_b200 as fl
    from flashlib_b200.knn import _mode_from, knn_f32
    from oracle import oracle_torch
    from tests import parity
    ms = _time_steps(lambda: fl.flash_knn(Qd, Xd, 100, mode=mode_name), steps, warm)
    d_, i_, info = knn_f32(Qd, Xd, 100, mode=_mode_from(mode_name))
    n_chk = 64
    _, ref_i = oracle_torch.knn_chunked(Q[:n_chk], X, 100, chunk_size=8192)
    res = parity.knn_parity(Q[:n_chk].numpy(), X.numpy(), d_[:n_chk].cpu().numpy(), i_[:n_chk].cpu().numpy(), ref_i.numpy())
    path = {0: "exact fp32 CUDA-core scoring", 1: "tcgen05 bf16 candidates (pools of 256) + exact fp32 re-rank + verified fallback"}
    nq, m, d = Qd.shape[0], Xd.shape[0], Xd.shape[1]
    return {"workload": "knn_1m_k100", "metric": "exact_knn_queries_per_sec", "value": nq / (ms * 1e-3),
            "unit": "queries/s", "ms_per_step": ms, "roofline": _roof("tensor", 2.0 * nq * m * d, ms, peaks),
            "parity_ok": bool(res["ok"]), "parity": {"rows": n_chk, "bad_rows": len(res["bad_rows"]),
                                                     "worst_rel_dist_err": res["worst_rel_dist_err"]},
            "config": {"k": 100, "path": path.get(int(info["mode"]), str(info["mode"])),
                       "rows_recomputed_on_exact_path": int(info.get("fallback_rows", 0))}}


def secondary_kmeans(steps, warm, peaks):
    """k-means 1,000,000 x 128, K = 1024, 20 Lloyd iterations from the first K rows.  Parity: the
    assignment under the final centroids against the oracle on 8,192 points (tie band), and the
    centroid update from those labels against the oracle's over all points."""
    import flashlib_b200 as fl
    from flashlib_b200 import synthetic
    from oracle import oracle
    from tests import parity
    cfg = synthetic.CONFIGS["kmeans_1m"]
    X, _ = synthetic.mixture(cfg["n"], cfg["d"], cfg["n_comp"], cfg["seed"])
    Xd = X.cuda()
    init = Xd[:cfg["K"]].clone()
    ms = _time_steps(lambda: fl.flash_kmeans(Xd, cfg["K"], max_iters=cfg["iters"], init_centroids=init), steps, warm)
    _, cents, _ = fl.flash_kmeans(Xd, cfg["K"], max_iters=cfg["iters"], init_centroids=init)
    lab = fl.euclid_assign_triton(Xd[None], cents[None])[0]
    new, _, _ = fl.triton_lloyd_centroid_step_euclid(Xd[None], lab[None], cents[None])
    sub = torch.randperm(cfg["n"], generator=torch.Generator().manual_seed(0))[:8192]
    cn = cents.cpu().numpy()
    ref_lab = oracle.kmeans_assign(X[sub].numpy(), cn)
    lp = parity.label_parity(X[sub].numpy(), cn, lab.cpu()[sub].numpy(), ref_lab)
    new_ref, _, _ = oracle.kmeans_update(X.numpy(), lab.cpu().numpy().astype(np.int64), cn)
    upd_ok = parity.rel_close(new[0].cpu().numpy(), new_ref, rel=1e-4, atol=1e-5)
    flop = 2.0 * cfg["n"] * cfg["K"] * cfg["d"] * cfg["iters"]
    return {"workload": "kmeans_1m", "metric": "kmeans_20_iterations_ms", "value": ms, "unit": "ms", "ms_per_step": ms,
            "higher_is_better": False, "roofline": _roof("tensor", flop, ms, peaks),
            "parity_ok": bool(lp["ok"] and upd_ok),
            "parity": {"labels_checked": lp["n"], "labels_differ": lp["differ"], "labels_bad": lp["bad"],
                       "centroid_update_within_1e-4": bool(upd_ok)},
            "config": {"n": cfg["n"], "d": cfg["d"], "K": cfg["K"], "iters": cfg["iters"], "init": "first K rows"}}


def secondary_ivf(steps, warm, peaks):
    """IVF-Flat 1,000,000 x 128, nlist 1024 (10 Lloyd iterations), nprobe 16, 10,000 queries, k = 10.
    Parity: the oracle's search of the SAME index for 128 queries."""
    import flashlib_b200 as fl
    from flashlib_b200 import synthetic
    from oracle import oracle
    from tests import parity
    cfg = synthetic.CONFIGS["ivf_1m"]
    X, Q = synthetic.mixture(cfg["n"], cfg["d"], cfg["n_comp"], cfg["seed"], nq=cfg["nq"], clamp=True)
    Xd, Qd = X.cuda(), Q.cuda()
    ivf = fl.IVFFlat(nlist=cfg["nlist"], nprobe=cfg["nprobe"], niter=10, seed=cfg["seed"]).fit(Xd)
    ms = _time_steps(lambda: ivf.kneighbors(Qd, cfg["k"]), steps, warm)
    _, bi = fl.flash_knn(Qd[:1000], Xd, cfg["k"])
    vals, ii = ivf.kneighbors(Qd, cfg["k"])
    recall = float(np.mean([len(set(a.tolist()) & set(b.tolist())) / cfg["k"]
                            for a, b in zip(ii[:1000].cpu().numpy(), bi.cpu().numpy())]))
    idx = ivf.index_
    n_chk = 128
    ov, oi, _ = oracle.ivf_search(idx.centroids.cpu().numpy(), idx.data.cpu().numpy(), idx.ids.cpu().numpy(),
                                  idx.list_offsets.cpu().numpy(), Q[:n_chk].numpy(), cfg["k"], cfg["nprobe"])
    v, i = vals[:n_chk].cpu().numpy(), ii[:n_chk].cpu().numpy()
    fin = np.isfinite(ov)
    same_rows = float(np.mean([set(a[f].tolist()) == set(b[f].tolist()) for a, b, f in zip(i, oi, fin)]))
    ok = bool(np.array_equal(np.isfinite(v), fin) and parity.rel_close(v[fin], ov[fin], rel=1e-4, atol=1e-4)
              and same_rows >= 0.99)
    # every probed list streamed once (fp32 rows) + the gathered queries + the results
    lens = idx.list_lengths().cpu().numpy()
    work = float(cfg["n"] * cfg["d"] * 4 + cfg["nq"] * cfg["nprobe"] * cfg["d"] * 4 + cfg["nq"] * cfg["k"] * 12)
    return {"workload": "ivf_1m", "metric": "ivf_flat_queries_per_sec", "value": cfg["nq"] / (ms * 1e-3), "unit": "queries/s",
            "ms_per_step": ms, "recall_at_10_vs_exact": recall, "roofline": _roof("hbm", work, ms, peaks),
            "parity_ok": ok, "parity": {"rows": n_chk, "rows_with_identical_sets": same_rows},
            "config": {"nlist": cfg["nlist"], "nprobe": cfg["nprobe"], "k": cfg["k"], "max_list_len": int(lens.max())}}


def secondary_knn_100m_shard(steps, warm, mode_name, peaks, rows=None, nq=None):
    """One GPU's share of the sharded configuration: 12,500,000 of the 100,000,000 rows x 96 features
    ~ N(0,1) (drawn on the device: 4.8 GB of rows), all 100,000 queries, k = 100.  Parity: the CPU
    restatement on 16 of the queries against all of this GPU's rows (copied to the host in blocks)."""
    import flashlib_b200 as fl
    from flashlib_b200 import synthetic
    from flashlib_b200.knn import _mode_from, knn_f32
    from oracle import oracle_torch
    from tests import parity
    cfg = synthetic.CONFIGS["knn_sharded_100m"]
    rows = rows or cfg["m"] // 8
    nq = nq or cfg["nq"]
    g = torch.Generator(device="cuda").manual_seed(cfg["seed"])
    Xd = torch.randn(rows, cfg["d"], generator=g, device="cuda")
    Qd = torch.randn(nq, cfg["d"], generator=g, device="cuda")
    ms = _time_steps(lambda: fl.flash_knn(Qd, Xd, cfg["k"], mode=mode_name), steps, warm)
    d_, i_, info = knn_f32(Qd, Xd, cfg["k"], mode=_mode_from(mode_name))
    n_chk = 16
    Xh = torch.empty((rows, cfg["d"]), dtype=torch.float32)
    for r0 in range(0, rows, 2_000_000):
        Xh[r0:r0 + 2_000_000] = Xd[r0:r0 + 2_000_000].cpu()
    Qh = Qd[:n_chk].cpu()
    _, ref_i = oracle_torch.knn_chunked(Qh, Xh, cfg["k"], chunk_size=65536)
    res = parity.knn_parity(Qh.numpy(), Xh.numpy(), d_[:n_chk].cpu().numpy(), i_[:n_chk].cpu().numpy(), ref_i.numpy())
    flop = 2.0 * nq * rows * cfg["d"]
    del Xd, Xh
    torch.cuda.empty_cache()
    return {"workload": "knn_100m_shard", "metric": "exact_knn_queries_per_sec", "value": nq / (ms * 1e-3),
            "unit": "queries/s", "ms_per_step": ms, "roofline": _roof("tensor", flop, ms, peaks),
            "parity_ok": bool(res["ok"]), "parity": {"rows": n_chk, "bad_rows": len(res["bad_rows"]),
                                                     "worst_rel_dist_err": res["worst_rel_dist_err"]},
            "config": {"rows_on_this_gpu": rows, "of_rows": cfg["m"], "dim": cfg["d"], "queries": nq, "k": cfg["k"],
                       "mode": int(info["mode"]), "rows_recomputed_on_exact_path": int(info.get("fallback_rows", 0))}}


def run_secondary(args):
    """Single-GPU timings of the other configurations (k-means 1M x 128 / K=1024 / 20 Lloyd
    iterations; IVF-Flat search nlist=1024, nprobe=16; exact kNN with k=100)."""
    import flashlib_b200 as fl
    from flashlib_b200 import synthetic
    torch.cuda.set_device(0)
    peaks = load_peaks()
    steps, warm = max(1, min(args.steps, 5)), max(1, min(args.warmup, 2))
    if args.workload == "knn_1m_k100":
        X, Q = synthetic.mixture(DB_ROWS, DIM, N_COMP, SEED, nq=QUERIES_PER_GPU, clamp=True)
        line = secondary_knn_k100(X.cuda(), Q.cuda(), X, Q, steps, warm, args.mode, peaks)
    elif args.workload == "knn_self_1m":
        # the "graph build" regime of flash_knn's internal callers: every row of the 1M x 128
        # database is a query against the same database
        X, _ = synthetic.mixture(DB_ROWS, DIM, N_COMP, SEED, clamp=True)
        Xd = X.cuda()
        from flashlib_b200.knn import _mode_from, knn_f32
        mode = _mode_from(args.mode)
        ms = _time_steps(lambda: fl.flash_knn(Xd, Xd, K_NEIGHBOURS, mode=args.mode), min(steps, 2), 1)
        _, _, info = knn_f32(Xd, Xd, K_NEIGHBOURS, mode=mode)
        line = {"workload": "knn_self_1m", "metric": "exact_knn_queries_per_sec", "value": DB_ROWS / (ms * 1e-3),
                "unit": "queries/s", "ms_per_step": ms,
                "algorithmic_tflops": 2.0 * DB_ROWS * DB_ROWS * DIM / (ms * 1e-3) / 1e12,
                "config": {"rows": DB_ROWS, "dim": DIM, "k": K_NEIGHBOURS, "mode": int(info["mode"]),
                           "rows_recomputed_on_exact_path": int(info.get("fallback_rows", 0))}}
    elif args.workload == "knn_neardup":
        # Near-duplicate data (200 centres, every row and query a centre plus N(0, 0.1^2) noise): rows
        # of one centre lie within the bf16 scoring error of each other, so the bf16 proof rejects
        # most queries and the split-plane stage (or, without it, the exact CUDA-core pass) decides.
        g = torch.Generator().manual_seed(9)
        base = torch.randn(200, DIM, generator=g)
        X = base[torch.randint(0, 200, (DB_ROWS,), generator=g)] + 0.1 * torch.randn(DB_ROWS, DIM, generator=g)
        Q = base[torch.randint(0, 200, (QUERIES_PER_GPU,), generator=g)] + 0.1 * torch.randn(QUERIES_PER_GPU, DIM, generator=g)
        Xd, Qd = X.cuda(), Q.cuda()
        from flashlib_b200.knn import _mode_from, knn_f32
        from tests import parity
        mode = _mode_from(args.mode or "bf16")
        ms = _time_steps(lambda: knn_f32(Qd, Xd, K_NEIGHBOURS, mode=mode, check_status=False), steps, warm)
        d_, i_, info = knn_f32(Qd, Xd, K_NEIGHBOURS, mode=mode)
        ms1 = _time_steps(lambda: knn_f32(Qd, Xd, K_NEIGHBOURS, mode=mode, check_status=False, second_stage=False), 1, 1)
        _, _, info1 = knn_f32(Qd, Xd, K_NEIGHBOURS, mode=mode, second_stage=False)
        # yardstick: fp64 brute force on the device for a sample (the fp32 expansion of the CPU
        # restatement is itself only good to about 1e-5 relative on such data)
        n_chk = 128
        qd, xd = Qd[:n_chk].double(), Xd.double()
        d64 = (qd * qd).sum(-1, keepdim=True) + (xd * xd).sum(-1)[None, :] - 2.0 * qd @ xd.T
        ref_i = d64.topk(K_NEIGHBOURS, dim=1, largest=False).indices.cpu().numpy()
        res = parity.knn_parity(Q[:n_chk].numpy(), X.numpy(), d_[:n_chk].cpu().numpy(), i_[:n_chk].cpu().numpy(), ref_i)
        nq = QUERIES_PER_GPU
        line = {"workload": "knn_neardup", "metric": "exact_knn_queries_per_sec", "value": nq / (ms * 1e-3),
                "unit": "queries/s", "ms_per_step": ms,
                "parity_ok": bool(res["ok"]), "parity": {"rows": n_chk, "bad_rows": len(res["bad_rows"]), "against": "fp64 brute force"},
                "rows_rejected_by_the_bf16_proof": int(info.get("stage2_rows", 0)) + (0 if info["second_stage"] else int(info["fallback_rows"])),
                "rows_on_the_split_plane_stage": int(info.get("stage2_rows", 0)),
                "rows_on_the_exact_cuda_core_pass": int(info.get("fallback_rows", 0)),
                "without_second_stage": {"ms_per_step": ms1, "rows_on_the_exact_cuda_core_pass": int(info1.get("fallback_rows", 0))},
                "config": {"rows": DB_ROWS, "dim": DIM, "queries": nq, "k": K_NEIGHBOURS, "centres": 200, "spread": 0.1,
                           "mode": int(info["mode"]), "second_stage": bool(info["second_stage"])}}
    elif args.workload == "knn_100m_shard":
        line = secondary_knn_100m_shard(steps, warm, args.mode, peaks, rows=args.db_rows, nq=args.queries)
    elif args.workload == "kmeans_1m":
        line = secondary_kmeans(steps, warm, peaks)
    else:
        line = secondary_ivf(steps, warm, peaks)
    line.update({"n_gpus": 1, "steps": steps, "warmup": warm, "data": "synthetic"})
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-gpu"],
                    help="reference: the reference's CPU path (oracle port) on the host cores; reference-gpu: the "
                         "unmodified reference's own GPU kernels from baseline/_ref, one GPU, for the comparison table")
    ap.add_argument("--ref-leg", default=None, help="internal: one leg of --impl reference-gpu, 'dtype:backend'")
    ap.add_argument("--mode", default=None, help="kNN scoring mode: exact | bf16 | None (auto)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true", help="N = 1: skip the k-means / IVF-Flat / k=100 legs")
    ap.add_argument("--result", default="owner", choices=["owner", "replicated"],
                    help="N > 1: 'owner' = all-to-all, every rank merges and returns its own slice of the step's queries; "
                         "'replicated' = all-gather, every rank merges and returns all of them")
    ap.add_argument("--workload", default="knn_1m", choices=["knn_1m", "knn_100m", "knn_1m_k100", "knn_self_1m", "knn_neardup", "knn_100m_shard", "kmeans_1m", "ivf_1m"],
                    help="knn_1m is the headline benchmark; the others time the remaining configurations on one GPU "
                         "and print a shorter JSON line")
    ap.add_argument("--db-rows", type=int, default=None, help="with --profile-case: database rows")
    ap.add_argument("--queries", type=int, default=None, help="with --profile-case: queries per GPU")
    ap.add_argument("--profile-case", action="store_true",
                    help="small case for profiler captures: 524,288 rows, 2,048 queries, no warm-up floor, "
                         "no end-to-end or CPU legs (its numbers are not benchmark values)")
    args = ap.parse_args()

    global DB_ROWS, QUERIES_PER_GPU, DIM, K_NEIGHBOURS, SEED, SCALING, WORKLOAD
    if args.workload == "knn_100m":
        from flashlib_b200 import synthetic as _syn
        c5 = _syn.CONFIGS["knn_sharded_100m"]
        WORKLOAD, SCALING = "knn_100m", "strong"
        DB_ROWS, DIM, K_NEIGHBOURS, SEED = args.db_rows or c5["m"], c5["d"], c5["k"], c5["seed"]
        QUERIES_PER_GPU = args.queries or c5["nq"]      # per step in total: every rank scores all of them
        args.no_cpu_baseline = True
    if args.profile_case:
        DB_ROWS, QUERIES_PER_GPU = args.db_rows or 524_288, args.queries or 2_048
        args.no_cpu_baseline = True
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.impl == "reference-gpu":
        if rank == 0:
            run_reference_gpu(args)
        return
    if args.workload not in ("knn_1m", "knn_100m"):
        run_secondary(args)
        return
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from flashlib_b200 import _lib
    from flashlib_b200.knn import _mode_from, check_pending, flash_knn, get_plane
    from flashlib_b200.sharded import sharded_knn
    lib = _lib.load()
    _lib.require_device()
    mode = _mode_from(args.mode)

    X, Q, s, e = make_workload(rank, world)
    nq = Q.shape[0]
    db = X if WORKLOAD == "knn_100m" else X[s:e].contiguous().to(dev)
    q_host = Q.contiguous().pin_memory()
    q_dev = q_host.to(dev)
    resolved = lib.fl_knn_resolve_mode(nq, db.shape[0], DIM, K_NEIGHBOURS) if mode == _lib.FL_KNN_AUTO else mode
    plane = get_plane(db) if resolved == _lib.FL_KNN_BF16_RERANK else None   # index-build-time work
    # the sharded index (a collective: global max norm, smallest shard) is index-build-time work too
    from flashlib_b200.sharded import ShardedKnnIndex
    index = ShardedKnnIndex(db, s, plane=plane) if world > 1 else None
    torch.cuda.synchronize()

    # Timing hygiene: when this rank's operand plane is not well above the 126 MB L2 it would stay
    # cache-resident from step to step, so a 160 MB buffer (larger than the L2) is overwritten before every step
    # (inside the timed region).
    plane_bytes = db.shape[0] * (((DIM + 63) // 64) * 64 + 16) * 2
    flush = torch.empty(160 << 20, dtype=torch.uint8, device=dev) if plane_bytes < (256 << 20) else None

    def step_device():
        if flush is not None:
            flush.zero_()
        return sharded_knn(q_dev, db, K_NEIGHBOURS, row_offset=s, mode=args.mode, plane=plane, result=args.result,
                           index=index)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing ----------------------------------------------------------
    n_warm = args.warmup if args.profile_case else max(args.warmup, 3)
    for _ in range(n_warm):
        out = step_device()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    lib.fl_profile_enable(1)
    launches0 = lib.fl_launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for _ in range(args.steps):
        out = step_device()
    ev1.record()
    barrier()
    launches = lib.fl_launch_count() - launches0
    ms_total = ev0.elapsed_time(ev1)
    check_pending()              # raises if any timed step reported a kernel error
    kernel_ms = []
    tmp = ctypes.c_float()
    for i in range(lib.fl_profile_count()):
        if lib.fl_profile_read_ms(i, ctypes.byref(tmp)) == 0:
            kernel_ms.append(tmp.value)
    lib.fl_profile_enable(0)
    clocks = sampler.stop() if rank == 0 else None
    t = torch.tensor([ms_total], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total = float(t.item())
    value = nq * args.steps / (ms_total * 1e-3)

    # ---- end to end: pinned host queries in, host results out, through the public API -----
    # Every step copies its queries from pinned host memory and its results back to pinned host
    # memory.  The copies run on their own streams, two steps deep, so the transfer of one step
    # overlaps the scoring of its neighbour (as a serving loop would); the host reads a step's
    # results (waits for its copy-out event) before it reuses that slot two steps later, and
    # everything is drained before the clock stops.
    from flashlib_b200.sharded import shard_bounds
    qs_, qe_ = shard_bounds(nq, world, rank) if (world > 1 and args.result == "owner") else (0, nq)
    out_d_host = [torch.empty((qe_ - qs_, K_NEIGHBOURS), dtype=torch.float32).pin_memory() for _ in range(2)]
    out_i_host = [torch.empty((qe_ - qs_, K_NEIGHBOURS), dtype=torch.int32).pin_memory() for _ in range(2)]
    q_slots = [torch.empty_like(q_dev) for _ in range(2)]
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    main = torch.cuda.current_stream(dev)
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_used = [torch.cuda.Event() for _ in range(2)]
    ev_done = [torch.cuda.Event() for _ in range(2)]
    ev_out = [None, None]
    keep = [None, None]            # device results stay referenced until their copy-out is done

    def step_e2e(i):
        j = i % 2
        if ev_out[j] is not None:
            ev_out[j].synchronize()                      # the host "reads" the results of step i - 2
        with torch.cuda.stream(s_in):
            if i >= 2:
                s_in.wait_event(ev_used[j])              # step i - 2 no longer reads this query slot
            q_slots[j].copy_(q_host, non_blocking=True)
            ev_in[j].record(s_in)
        main.wait_event(ev_in[j])
        if flush is not None:
            flush.zero_()
        if world == 1:
            d_, i_ = flash_knn(q_slots[j], db, K_NEIGHBOURS, mode=args.mode)
        else:
            d_, i_ = sharded_knn(q_slots[j], db, K_NEIGHBOURS, row_offset=s, mode=args.mode, plane=plane,
                                 result=args.result, index=index)
        ev_used[j].record(main)
        ev_done[j].record(main)
        keep[j] = (d_, i_)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_done[j])
            out_d_host[j].copy_(d_, non_blocking=True)
            out_i_host[j].copy_(i_, non_blocking=True)
            ev_out[j] = torch.cuda.Event()
            ev_out[j].record(s_out)

    def drain():
        for e_ in ev_out:
            if e_ is not None:
                e_.synchronize()
        torch.cuda.synchronize()

    e2e_steps = 0 if args.profile_case else args.steps
    for i in range(2 if e2e_steps else 0):
        step_e2e(i)
    drain()
    ev_out[0] = ev_out[1] = None
    barrier()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        step_e2e(i)
    drain()
    barrier()
    check_pending()
    e2e_s = max(time.perf_counter() - t0, 1e-9)
    t = torch.tensor([e2e_s], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_s = float(t.item())
    e2e_value = nq * e2e_steps / e2e_s

    # ---- parity of the last timed step's results, outside the timed region ---------------------
    # Every rank checks a sample of the queries whose results it holds against the CPU oracle on the
    # WHOLE database; the counts are summed over the ranks.  This is the check the real NCCL
    # exchange gets at every N.
    parity_line = None
    if not args.profile_case:
        from oracle import oracle_torch
        torch.set_num_threads(max(1, (os.cpu_count() or 1) // max(1, world)))
        out_d, out_i = out
        n_chk = min(out_d.shape[0], max(16, 128 // world))
        q_chk = Q[qs_:qs_ + n_chk]
        got_d, got_i = out_d[:n_chk].cpu().numpy(), out_i[:n_chk].cpu().numpy()
        if WORKLOAD == "knn_100m":
            # the rows live on the devices only: every rank runs the oracle on its shard for the first
            # queries of the batch, the per-shard lists are gathered and merged on the host
            n_chk = 32
            ld = torch.full((n_chk, K_NEIGHBOURS), float("inf"))
            li = torch.full((n_chk, K_NEIGHBOURS), -1, dtype=torch.int64)
            piece = 2_000_000                      # rows copied to the host at a time (0.8 GB)
            for p0 in range(0, db.shape[0], piece):
                pd, pi = oracle_torch.knn_chunked(Q[:n_chk], db[p0:p0 + piece].cpu(), K_NEIGHBOURS, chunk_size=65536)
                cv, ci_ = torch.cat([ld, pd], 1), torch.cat([li, pi + (s + p0)], 1)
                sel = cv.argsort(dim=1, stable=True)[:, :K_NEIGHBOURS]
                ld, li = cv.gather(1, sel), ci_.gather(1, sel)
            if world > 1:
                gl = [None] * world
                dist.all_gather_object(gl, (ld.numpy(), li.numpy()))
            else:
                gl = [(ld.numpy(), li.numpy())]
            cd = np.concatenate([g_[0] for g_ in gl], 1)
            ci = np.concatenate([g_[1] for g_ in gl], 1)
            order = np.argsort(cd, axis=1, kind="stable")[:, :K_NEIGHBOURS]
            ref_d, ref_i = np.take_along_axis(cd, order, 1), np.take_along_axis(ci, order, 1)
            # ... and compared with the rows of the distributed result this rank holds
            lo, hi = max(qs_, 0), min(qe_, n_chk)
            rows_chk = max(0, hi - lo)
            bad = knn_rows_agree(Q[lo:hi].numpy(), out_d[lo - qs_:hi - qs_].cpu().numpy(), out_i[lo - qs_:hi - qs_].cpu().numpy(),
                                 ref_d[lo:hi], ref_i[lo:hi]) if rows_chk else 0
            worst = 0.0
        else:
            from tests import parity as tparity
            _, ref_i = oracle_torch.knn_chunked(q_chk, X, K_NEIGHBOURS, chunk_size=8192)
            res = tparity.knn_parity(q_chk.numpy(), X.numpy(), got_d, got_i, ref_i.numpy())
            rows_chk, bad, worst = n_chk, len(res["bad_rows"]) + res["unsorted_rows"], res["worst_rel_dist_err"]
            if worst > tparity.REL_DIST:
                bad = max(bad, 1)
        t = torch.tensor([rows_chk, bad, worst], device=dev, dtype=torch.float64)
        if world > 1:
            tm = t.clone()
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
            dist.all_reduce(tm, op=dist.ReduceOp.MAX)
            t[2] = tm[2]
        parity_line = {"rows": int(t[0].item()), "bad_rows": int(t[1].item()), "ok": int(t[1].item()) == 0 and int(t[0].item()) > 0,
                       "worst_rel_dist_err": float(t[2].item()),
                       "against": "oracle_torch.knn_chunked on the whole database, every rank a sample of the queries it holds"}

    # ---- sustained: the same device-resident loop for seconds (what a serving loop gets) ---------
    sustained_line = None
    if world == 1 and not args.profile_case and WORKLOAD == "knn_1m":
        per_chunk = 20
        chunks = int(max(3.0 / max(ms_total * 1e-3 / args.steps * per_chunk, 1e-6), 5))
        samp2 = ClockSampler(local_rank)
        samp2.start()
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(chunks + 1)]
        evs[0].record()
        for c in range(chunks):
            for _ in range(per_chunk):
                step_device()
            evs[c + 1].record()
        torch.cuda.synchronize()
        check_pending()
        clk2 = samp2.stop()
        qps = [nq * per_chunk / (evs[c].elapsed_time(evs[c + 1]) * 1e-3) for c in range(chunks)]
        tail = qps[len(qps) // 2:]                  # the second half: clocks have settled under the power cap
        peaks_ = load_peaks()
        med = statistics.median(tail)
        tf = 2.0 * DB_ROWS * DIM * med / 1e12
        sustained_line = {"value": med, "unit": UNIT, "seconds": sum(evs[c].elapsed_time(evs[c + 1]) for c in range(chunks)) * 1e-3,
                          "steps": chunks * per_chunk, "first_chunk_value": qps[0],
                          "tensor_tflops_algorithmic": tf, "peak": peaks_.get("bf16_tflops_sustained"),
                          "frac": tf / peaks_["bf16_tflops_sustained"] if peaks_.get("bf16_tflops_sustained") else None,
                          "clocks": clk2}

    # ---- the other configurations, on the driver's clock (N = 1 only) ------------------------------
    secondary = None
    if world == 1 and not args.profile_case and WORKLOAD == "knn_1m" and not args.no_secondary:
        peaks_ = load_peaks()
        secondary = {}
        secondary["knn_1m_k100"] = secondary_knn_k100(db, q_dev, X, Q, 5, 2, args.mode, peaks_)
        del out
        secondary["kmeans_1m"] = secondary_kmeans(3, 1, peaks_)
        torch.cuda.empty_cache()
        secondary["ivf_1m"] = secondary_ivf(5, 2, peaks_)
        torch.cuda.empty_cache()
        # one GPU's share of the 100M-row sharded configuration (the 8-GPU run of it: --workload knn_100m)
        secondary["knn_100m_shard"] = secondary_knn_100m_shard(2, 1, args.mode, peaks_)

    if rank == 0:
        peaks = load_peaks()
        rows_local = e - s
        flop_per_launch = 2.0 * nq * rows_local * DIM
        k_ms = statistics.mean(kernel_ms) if kernel_ms else None
        achieved = flop_per_launch / (k_ms * 1e-3) / 1e12 if k_ms else None
        # a kernel timed alone for a few ms runs at burst clocks; the seconds-long launches of the
        # 100M-row workload run under the power cap: sustained figure
        sustained = WORKLOAD == "knn_100m" and peaks.get("bf16_tflops_sustained")
        peak = peaks["bf16_tflops_sustained"] if sustained else peaks["bf16_tflops"]
        roofline = {
            "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
            "frac": (achieved / peak) if achieved else None, "traffic": TC_KERNEL_DRAM_BYTES_PER_LAUNCH if resolved == _lib.FL_KNN_BF16_RERANK and not args.profile_case and world == 1 and WORKLOAD == "knn_1m" else None,
            "kernel": "knn_tc_kernel" if resolved == _lib.FL_KNN_BF16_RERANK else "knn_simt_kernel",
            "kernel_ms": k_ms, "launches_timed": len(kernel_ms),
            "algorithmic_flop_per_launch": flop_per_launch,
            "peak_source": (f"{peaks['source']} bf16 {'sustained' if sustained else 'burst'} (MEASURED_PEAKS.json)"
                            if peaks["source"] == "measured" else "fallback 1.59 PFLOP/s burst / 1.4 sustained"),
        }
        cpu_base = None
        if not args.no_cpu_baseline and world == 1:
            n_cpu_q = 2048
            v, cores = cpu_baseline_run(X, Q, n_cpu_q)
            cpu_base = {"value": v, "unit": UNIT, "cores": cores, "kind": "port",
                        "sample": f"{n_cpu_q} of the {QUERIES_PER_GPU} queries against all {DB_ROWS} rows; "
                                  "torch-CPU restatement of knn_torch_chunked, chunk 8192"}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": n_warm, "ms_per_step": ms_total / args.steps, "higher_is_better": True,
            "scaling": SCALING, "vs_baseline": None, "dtype": "bf16" if resolved == _lib.FL_KNN_BF16_RERANK else "f32",
            "data": "synthetic",
            "config": config_dict(world, args.result, resolved == _lib.FL_KNN_BF16_RERANK, nq),
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": int(q_host.numel() * 4),
                    "d2h_bytes_per_step": int(out_d_host[0].numel() * 4 + out_i_host[0].numel() * 4),
                    "note": "every step: queries from pinned host memory, results to pinned host memory, copies on "
                            "their own streams two steps deep; the database is the fitted index and stays resident"},
            "gpu_launches": int(launches),
            "roofline": roofline,
            "cpu_baseline": cpu_base,
            "parity": parity_line,
            "sustained": sustained_line,
            "secondary": secondary,
            "clocks": clocks,
            "tensor_tflops_algorithmic": 2.0 * nq * DB_ROWS * DIM * args.steps / (ms_total * 1e-3) / 1e12 / world,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
