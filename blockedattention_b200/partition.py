"""Sharding of a packed batch across GPUs: segments are independent, so a rank
takes a contiguous range of them (its packed strips and rebased offsets are
plain slices) chosen to balance ``max(flops/peak, bytes/peak)``; there is no
collective on the data path.  The upstream project is single-GPU; this module
has no counterpart there.
"""
from __future__ import annotations

import ctypes as C
from typing import Tuple

import numpy as np

from . import _lib as L

# Default denominators of the cost model: nominal dense 16-bit tensor throughput and HBM bandwidth of a B200.
# Only their ratio matters for the split; callers that have measured both on their machine pass those instead
# (the benchmark passes the measured copy bandwidth and cuBLAS throughput).
PEAK_FLOPS = 2.25e15
PEAK_BYTES = 7.7e12


def segment_cost(M, N, K, H: int, in_bytes: int = 2, out_bytes: int = 2,
                 flops_per_s: float = PEAK_FLOPS, bytes_per_s: float = PEAK_BYTES) -> np.ndarray:
    M = np.ascontiguousarray(M, dtype=np.int64); N = np.ascontiguousarray(N, dtype=np.int64)
    K = np.ascontiguousarray(K, dtype=np.int64)
    cost = np.empty(len(M), np.float64)
    L.check(L.lib.blk_segment_cost(L.i64(M), L.i64(N), L.i64(K), len(M), H, in_bytes, out_bytes,
                                   flops_per_s, bytes_per_s, cost.ctypes.data_as(C.POINTER(C.c_double))))
    return cost


def partition_contiguous(cost, world: int) -> np.ndarray:
    """bounds[r]..bounds[r+1] is rank r's segment range; minimises the largest range cost."""
    cost = np.ascontiguousarray(cost, dtype=np.float64)
    bounds = np.empty(world + 1, np.int64)
    L.check(L.lib.blk_partition_contiguous(cost.ctypes.data_as(C.POINTER(C.c_double)), len(cost), world,
                                           L.i64(bounds)))
    return bounds


def partition_lpt(cost, world: int) -> np.ndarray:
    """owner[s] by longest-processing-time greedy (not contiguous)."""
    cost = np.ascontiguousarray(cost, dtype=np.float64)
    owner = np.empty(len(cost), np.int32)
    L.check(L.lib.blk_partition_lpt(cost.ctypes.data_as(C.POINTER(C.c_double)), len(cost), world,
                                    owner.ctypes.data_as(C.POINTER(C.c_int32))))
    return owner


def imbalance(cost, bounds) -> float:
    """max range cost / mean range cost (1.0 = perfect)."""
    cost = np.asarray(cost, dtype=np.float64)
    loads = np.array([cost[bounds[r]:bounds[r + 1]].sum() for r in range(len(bounds) - 1)])
    return float(loads.max() / max(loads.mean(), 1e-300))


def shard_range(M, N, K, H: int, rank: int, world: int, in_bytes: int = 2, out_bytes: int = 2) -> Tuple[int, int]:
    """Segment range [lo, hi) of ``rank`` under the balanced contiguous split."""
    b = partition_contiguous(segment_cost(M, N, K, H, in_bytes, out_bytes), world)
    return int(b[rank]), int(b[rank + 1])


def shard(M, N, K, H: int, world: int, in_bytes: int = 2, out_bytes: int = 2,
          flops_per_s: float = PEAK_FLOPS, bytes_per_s: float = PEAK_BYTES, max_imbalance: float = 1.05):
    """Ownership of every segment for ``world`` ranks: ``(owner, info)`` with ``owner[s]`` the rank of segment s.

    The balanced contiguous split is used when its largest range is within ``max_imbalance`` of the mean (each
    rank's strips are then plain slices of the packed buffers); otherwise the longest-processing-time assignment,
    whose ranges are not contiguous.  ``info`` = {"kind", "imbalance", "bounds" (contiguous only)}."""
    cost = segment_cost(M, N, K, H, in_bytes, out_bytes, flops_per_s, bytes_per_s)
    bounds = partition_contiguous(cost, world)
    imb = imbalance(cost, bounds) if len(cost) else 1.0
    if imb <= max_imbalance:
        owner = np.repeat(np.arange(world, dtype=np.int32), np.diff(bounds))
        return owner, {"kind": "contiguous", "imbalance": imb, "bounds": [int(b) for b in bounds]}
    owner = partition_lpt(cost, world)
    loads = np.bincount(owner, weights=cost, minlength=world)
    return owner, {"kind": "lpt", "imbalance": float(loads.max() / max(loads.mean(), 1e-300)),
                   "contiguous_imbalance": imb}


def _runs(owner: np.ndarray):
    """Maximal runs of consecutive segments with one owner: (rank, first segment, one past the last)."""
    out, s, S = [], 0, len(owner)
    while s < S:
        e = s
        while e < S and owner[e] == owner[s]:
            e += 1
        out.append((int(owner[s]), s, e))
        s = e
    return out


# gather_output sends run by run up to this many runs per rank and all-gathers beyond
GATHER_MAX_RUNS_PER_RANK = 4


def gather_output(local, block_elems, owner, H: int, group=None, out=None):
    """Every rank ends with the whole packed head-major result.

    ``local`` is this rank's result ``(H, D_rank)``: the blocks of the segments it owns, in batch order, packed;
    ``block_elems[s]`` is the number of elements of segment s's block in one head strip (``M_s * N_s`` for scores
    and probabilities, ``M_s * d`` for attention results); ``owner`` as returned by :func:`shard`.  Returns
    ``(H, sum(block_elems))`` with segment s of head h at ``h * D + offset[s]``, ``offset = cumsum(block_elems)``
    -- the layout a single process produces (upstream csrc/cuda/spBlkGEMM.cu:453-455).

    Ownership in a few runs of consecutive segments (contiguous ranges): one grouped set of point-to-point transfers
    (``torch.distributed.batch_isend_irecv``: NCCL send/recv between ``ncclGroupStart`` and ``ncclGroupEnd`` on GPUs,
    gloo on CPU).  A rank's strips have unequal lengths and are not contiguous in the result, so this is H transfers
    per run, received in place: no staging buffer, no equal-size padding.  Ownership scattered over many runs (the
    longest-processing-time assignment): thousands of point-to-point transfers in one group are not something to rely
    on, so the ranks all-gather their packed strips, padded to the longest, and every rank copies the runs into place
    itself.  The upstream project is single-GPU; no counterpart there."""
    import torch
    import torch.distributed as dist
    owner = np.asarray(owner)
    be = np.asarray(block_elems, dtype=np.int64)
    off = np.concatenate([[0], np.cumsum(be)])
    D = int(off[-1])
    rank = dist.get_rank(group)
    if out is None:
        out = torch.empty((H, D), dtype=local.dtype, device=local.device)
    mine = int(be[owner == rank].sum())
    if local.shape != (H, mine):
        raise RuntimeError(f"local result has shape {tuple(local.shape)}, this rank owns ({H}, {mine})")
    world = dist.get_world_size(group)
    runs = [(r, s, e) for r, s, e in _runs(owner) if off[e] > off[s]]
    if len(runs) > GATHER_MAX_RUNS_PER_RANK * world:
        per_rank = [int(be[owner == r].sum()) for r in range(world)]
        longest = max(per_rank)
        padded = local if mine == longest else torch.cat(
            [local, torch.zeros((H, longest - mine), dtype=local.dtype, device=local.device)], dim=1)
        parts = [torch.empty((H, longest), dtype=local.dtype, device=local.device) for _ in range(world)]
        dist.all_gather(parts, padded.contiguous(), group=group)
        pos = [0] * world
        for r, s, e in runs:
            lo, hi = int(off[s]), int(off[e])
            out[:, lo:hi].copy_(parts[r][:, pos[r]:pos[r] + (hi - lo)])
            pos[r] += hi - lo
        return out
    peers = [r for r in range(world) if r != rank]
    ops, lpos = [], 0
    for r, s, e in runs:
        lo, hi = int(off[s]), int(off[e])
        if hi == lo:
            continue
        if r == rank:
            piece = local[:, lpos:lpos + (hi - lo)]
            out[:, lo:hi].copy_(piece)
            for h in range(H):
                for q in peers:
                    ops.append(dist.P2POp(dist.isend, piece[h], q if group is None else dist.get_global_rank(group, q),
                                          group))
            lpos += hi - lo
        else:
            src = r if group is None else dist.get_global_rank(group, r)
            for h in range(H):
                ops.append(dist.P2POp(dist.irecv, out[h, lo:hi], src, group))
    if ops:
        for req in dist.batch_isend_irecv(ops):
            req.wait()
    return out
