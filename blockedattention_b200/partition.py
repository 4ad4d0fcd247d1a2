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

# Denominators of the cost model: dense 16-bit tensor throughput and HBM bandwidth of a B200.
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
