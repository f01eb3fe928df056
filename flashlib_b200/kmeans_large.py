"""Lloyd k-means for sample sets that live in host memory (too large for one GPU).

Mirrors ``flashlib/primitives/kmeans/large.py:35-410`` (``kmeans_largeN`` /
``kmeans_largeN_assign``): ``x`` stays on the CPU and is streamed to the GPU in blocks of
``BLOCK_N`` rows through two device buffers on two CUDA streams, so the copy of one block
overlaps the assignment and the centroid sums of the other; the per-cluster sums and counts
are accumulated over the blocks and the centroids are finalised once per iteration.

The reference drives several GPUs from one process and reduces their partial sums on GPU 0.
Here one process drives one GPU; under ``torch.distributed`` (one process per GPU) every rank
streams its own contiguous share of the blocks and the sums and counts are all-reduced, so
all ranks hold the same centroids (``flashlib/primitives/kmeans/large.py:73-82`` partitions
the blocks the same way).
"""
from __future__ import annotations

import warnings
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from . import kmeans as km


def block_range(num_blocks: int, world: int, rank: int) -> Tuple[int, int]:
    """Blocks ``[first, last)`` of ``rank``: the first ``num_blocks % world`` ranks take one extra
    (``flashlib/primitives/kmeans/large.py:74-78``)."""
    base, rem = divmod(int(num_blocks), int(world))
    first = rank * base + min(rank, rem)
    return first, first + base + (1 if rank < rem else 0)


def _resolve_device(device) -> torch.device:
    if device is None:
        if not torch.cuda.is_available():
            raise RuntimeError("No CUDA devices available")
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device(device)


def _stream_blocks(x: torch.Tensor, first_row: int, last_row: int, BLOCK_N: int, dev: torch.device, dtype, bufs, streams):
    """Yields ``(row0, rows, device_block, stream)`` for the blocks of ``x[first_row:last_row]``;
    block i is copied on ``streams[i % 2]`` into ``bufs[i % 2]`` and must be consumed on that
    stream (the next use of the buffer is ordered behind it)."""
    i = 0
    for row0 in range(first_row, last_row, BLOCK_N):
        rows = min(BLOCK_N, last_row - row0)
        s = streams[i % 2]
        with torch.cuda.stream(s):
            blk = bufs[i % 2][:rows]
            blk.copy_(x[row0:row0 + rows].to(dtype), non_blocking=True)
            yield row0, rows, blk, s
        i += 1


def kmeans_largeN(x: torch.Tensor, n_clusters: int, max_iters: int = 100, tol: float = 0.0, verbose: bool = False,
                  BLOCK_N: int = 1048576, init_centroids: Optional[torch.Tensor] = None,
                  device: Optional[torch.device] = None, dtype: Optional[torch.dtype] = None, group=None):
    """k-means of a CPU-resident ``x (N, D)``.  Returns ``(cluster_ids int32 (N,) on the CPU,
    centroids (K, D) on the GPU)``; under ``torch.distributed`` a rank's ``cluster_ids`` are filled
    for its own rows only (the others are -1)."""
    if x.is_cuda or x.ndim != 2:
        raise ValueError("kmeans_largeN expects a 2D CPU tensor; use flash_kmeans for GPU-resident data")
    dev = _resolve_device(device)
    dtype = dtype or x.dtype
    if dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise ValueError(f"unsupported dtype {dtype}")
    multi = dist.is_initialized() and dist.get_world_size(group) > 1
    world = dist.get_world_size(group) if multi else 1
    rank = dist.get_rank(group) if multi else 0
    if not x.is_pinned():
        warnings.warn("x is not in pinned memory: host-to-device copies will not overlap with compute "
                      "(use x = x.pin_memory())", stacklevel=2)
    N, D = x.shape
    K = int(n_clusters)
    BLOCK_N = int(BLOCK_N)
    num_blocks = (N + BLOCK_N - 1) // BLOCK_N
    b0, b1 = block_range(num_blocks, world, rank)
    first_row, last_row = min(b0 * BLOCK_N, N), min(b1 * BLOCK_N, N)

    with torch.cuda.device(dev):
        if init_centroids is not None:
            cur = init_centroids.reshape(K, D).to(device=dev, dtype=torch.float32).contiguous().clone()
        else:
            idx = torch.randint(0, N, (K,), device="cpu")
            cur = x[idx].to(device=dev, dtype=torch.float32).contiguous()
            if multi:
                dist.broadcast(cur, src=0, group=group)
        streams = [torch.cuda.Stream(device=dev) for _ in range(2)]
        bufs = [torch.empty((min(BLOCK_N, max(last_row - first_row, 1)), D), device=dev, dtype=torch.float32)
                for _ in range(2)]
        ids_dev = torch.full((max(last_row - first_row, 1),), -1, device=dev, dtype=torch.int32)
        sums = [torch.zeros((1, K, D), device=dev, dtype=torch.float32) for _ in range(2)]
        cnts = [torch.zeros((1, K), device=dev, dtype=torch.int32) for _ in range(2)]
        part_s = [torch.empty((1, K, D), device=dev, dtype=torch.float32) for _ in range(2)]
        part_c = [torch.empty((1, K), device=dev, dtype=torch.int32) for _ in range(2)]
        main = torch.cuda.current_stream(dev)
        n_iter = 0
        for n_iter in range(1, max_iters + 1):
            for s in streams:
                s.wait_stream(main)            # centroids of this iteration are ready
            for j in range(2):
                with torch.cuda.stream(streams[j]):
                    sums[j].zero_()
                    cnts[j].zero_()
            i = 0
            for row0, rows, blk, s in _stream_blocks(x, first_row, last_row, BLOCK_N, dev, torch.float32, bufs, streams):
                j = i % 2
                lab = ids_dev[row0 - first_row:row0 - first_row + rows]
                km.euclid_assign_triton(blk[None], cur[None], out=lab[None])
                km.triton_centroid_update_euclid(blk[None], lab[None], cur[None], centroid_sums=part_s[j],
                                                 centroid_cnts=part_c[j], calculate_new=False)
                sums[j] += part_s[j]
                cnts[j] += part_c[j]
                i += 1
            for s in streams:
                main.wait_stream(s)
            tot_s = sums[0] + sums[1]
            tot_c = cnts[0] + cnts[1]
            if multi:
                from .sharded import all_reduce_sums_counts
                all_reduce_sums_counts(tot_s, tot_c, group)
            new, shift = km.triton_centroid_finalize(tot_s, tot_c, cur[None])
            cur = new[0].float().contiguous()
            if verbose:
                print(f"kmeans_largeN iteration {n_iter}: max shift {float(shift.max()):.6g}")
            if tol > 0.0 and float(shift.max()) < tol:
                break
        cluster_ids = torch.full((N,), -1, dtype=torch.int32)
        if last_row > first_row:
            cluster_ids[first_row:last_row] = ids_dev[:last_row - first_row].cpu()
    return cluster_ids, cur.to(dtype)


def kmeans_largeN_assign(x: torch.Tensor, centroids: torch.Tensor, BLOCK_N: int = 1048576,
                         device: Optional[torch.device] = None) -> torch.Tensor:
    """Labels ``int32 (N,)`` (CPU) of a CPU-resident ``x`` for fixed centroids, streamed block by
    block (``flashlib/primitives/kmeans/large.py:283-410``)."""
    if x.is_cuda or x.ndim != 2:
        raise ValueError("kmeans_largeN_assign expects a 2D CPU tensor")
    dev = _resolve_device(device)
    N, D = x.shape
    BLOCK_N = int(BLOCK_N)
    with torch.cuda.device(dev):
        cur = centroids.reshape(-1, D).to(device=dev, dtype=torch.float32).contiguous()
        streams = [torch.cuda.Stream(device=dev) for _ in range(2)]
        bufs = [torch.empty((min(BLOCK_N, max(N, 1)), D), device=dev, dtype=torch.float32) for _ in range(2)]
        ids_dev = torch.empty((max(N, 1),), device=dev, dtype=torch.int32)
        main = torch.cuda.current_stream(dev)
        for s in streams:
            s.wait_stream(main)
        for row0, rows, blk, s in _stream_blocks(x, 0, N, BLOCK_N, dev, torch.float32, bufs, streams):
            km.euclid_assign_triton(blk[None], cur[None], out=ids_dev[row0:row0 + rows][None])
        for s in streams:
            main.wait_stream(s)
        return ids_dev[:N].cpu()
