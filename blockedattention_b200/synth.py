"""Seeded synthetic workloads: the segment-size draws and value distributions
of the benchmark configurations (no dataset is involved anywhere; sizes come
from ``numpy.random.RandomState(seed)`` so they are identical on every
machine, values from a ``torch.Generator`` on the device that holds them).

Buffers are produced directly in the packed head-major layout ``(H, sum n*d)``
the operators take; for i.i.d. random values this is the same distribution as
drawing ``[sum n, H, d]`` and permuting.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional

import numpy as np
import torch


@dataclass
class Workload:
    name: str
    M: np.ndarray
    N: np.ndarray
    K: np.ndarray
    H: int
    dtype: torch.dtype
    out_dtype: torch.dtype
    scale: float
    softmax: bool
    dist: str                      # "normal" or "uniform"
    std: float = 1.0
    d_v: int = 0                   # > 0: a P @ V product follows (full forward)
    note: str = ""
    extra: dict = field(default_factory=dict)

    @property
    def S(self) -> int:
        return len(self.M)

    @property
    def Dm1(self) -> int:
        return int((self.M * self.K).sum())

    @property
    def Dm2(self) -> int:
        return int((self.N * self.K).sum())

    @property
    def Dout(self) -> int:
        return int((self.M * self.N).sum())

    def flops(self) -> float:
        if self.extra.get("softmax_only"):
            return 0.0
        f = 2.0 * self.H * float((self.M * self.N * self.K).sum())
        if self.d_v:
            f += 2.0 * self.H * float((self.M * self.N).sum()) * self.d_v
        return f

    def bytes(self) -> float:
        ei = torch.empty((), dtype=self.dtype).element_size()
        eo = torch.empty((), dtype=self.out_dtype).element_size()
        if self.extra.get("softmax_only"):     # the score buffer read once and written once
            return 2.0 * self.H * float((self.M * self.N).sum()) * eo
        if self.extra.get("fused_attention"):  # q, k, v read, O written; P never exists
            return self.H * ei * (float(((self.M + self.N) * self.K).sum()) + float((self.N + self.M).sum()) * self.d_v)
        b = self.H * (float(((self.M + self.N) * self.K).sum()) * ei + float((self.M * self.N).sum()) * eo)
        if self.d_v:  # P read, V read, O written
            b += self.H * (float((self.M * self.N).sum()) * eo + float((self.N + self.M).sum()) * self.d_v * ei)
        return b

    def slice(self, lo: int, hi: int) -> "Workload":
        """Segments [lo, hi) as a workload of their own (a rank's shard)."""
        w = Workload(**{**self.__dict__})
        w.M, w.N, w.K = self.M[lo:hi].copy(), self.N[lo:hi].copy(), self.K[lo:hi].copy()
        return w

    def take(self, idx) -> "Workload":
        """The segments ``idx`` (in that order) as a workload of their own (a sample, or a non-contiguous shard)."""
        idx = np.asarray(idx, dtype=np.int64)
        w = Workload(**{**self.__dict__})
        w.M, w.N, w.K = self.M[idx].copy(), self.N[idx].copy(), self.K[idx].copy()
        return w

    def make_inputs(self, device, seed: int = 0):
        """(mat1, mat2) -- and v when d_v > 0 -- packed head-major on ``device``."""
        g = torch.Generator(device=device)
        g.manual_seed(seed)

        def draw(numel):
            if self.dist == "uniform":
                x = torch.rand((self.H, numel), generator=g, device=device, dtype=torch.float32) * 2 - 1
            else:
                x = torch.randn((self.H, numel), generator=g, device=device, dtype=torch.float32) * self.std
            return x.to(self.dtype)

        outs = [draw(self.Dm1), draw(self.Dm2)]
        if self.d_v:
            outs.append(draw(int(self.N.sum()) * self.d_v))
        return tuple(outs)


def _i64(x):
    return np.asarray(x, dtype=np.int64)


def workload(name: str, seed: int = 0, segments: Optional[int] = None) -> Workload:
    """Named configurations; ``segments`` overrides the segment count (same distributions)."""
    rs = np.random.RandomState(seed)
    if name == "cpu_plumbing":
        S = segments or 32
        n = _i64(rs.randint(4, 33, size=S))
        return Workload(name, n, n.copy(), np.full(S, 32, np.int64), 1, torch.float32, torch.float32,
                        1 / math.sqrt(32), True, "normal", note="32 segments, n~U{4..32}, j=32, fp32")
    if name == "molecular":
        S = segments or 4096
        n = _i64(np.clip(np.rint(rs.normal(25.0, 10.0, size=S)), 2, 128))
        return Workload(name, n, n.copy(), np.full(S, 64, np.int64), 8, torch.float16, torch.float16, 1 / 8.0, True,
                        "normal", note="4096 graphs, n~clip(round(N(25,10)),2,128), 8 heads, d=64, fp16")
    if name == "molecular_attention":
        # the molecular batch with graphs capped at 64 nodes, values added: softmax(QK^T) V in one kernel
        S = segments or 4096
        n = _i64(np.clip(np.rint(rs.normal(25.0, 10.0, size=S)), 2, 64))
        return Workload(name, n, n.copy(), np.full(S, 64, np.int64), 8, torch.float16, torch.float16, 1 / 8.0, True,
                        "normal", d_v=64, note="4096 graphs, n~clip(round(N(25,10)),2,64), 8 heads, d=64, fp16, "
                        "fused softmax(QK^T)V without materialising P", extra={"fused_attention": True})
    if name == "general_gemm":
        S = segments or 2048
        M = _i64(rs.randint(1, 257, size=S)); N = _i64(rs.randint(1, 257, size=S))
        K = _i64(rs.choice([16, 32, 48, 64, 96, 128], size=S))
        return Workload(name, M, N, K, 1, torch.float16, torch.float32, 1.0, False, "uniform",
                        note="2048 segments, i,k~U{1..256}, j in {16,32,48,64,96,128}, fp16 in, fp32 out")
    if name == "long_tail":
        S = segments or 512
        n = _i64(np.rint(np.exp(rs.uniform(math.log(16), math.log(2048), size=S))))
        return Workload(name, n, n.copy(), np.full(S, 64, np.int64), 4, torch.bfloat16, torch.bfloat16, 1 / 8.0, True,
                        "normal", std=0.5, note="512 segments, n log-uniform in [16,2048], 4 heads, d=64, bf16")
    if name == "full_forward":
        S = segments or 1024
        n = _i64(np.concatenate([rs.randint(64, 513, size=S), np.ones(max(1, S // 16), np.int64)]))
        return Workload(name, n, n.copy(), np.full(len(n), 128, np.int64), 16, torch.bfloat16, torch.bfloat16,
                        1 / math.sqrt(128), True, "normal", d_v=128,
                        note="1024 graphs n~U{64..512} + 64 graphs n=1, 16 heads, d=128, bf16, P then P@V")
    if name in ("long_tail_attention", "full_forward_attention"):
        # the same batches with the product with V fused in: one kernel, P never stored
        b = workload(name[:-len("_attention")], seed, segments)
        dv = int(b.K[0])
        return Workload(name, b.M, b.N, b.K, b.H, b.dtype, b.dtype, b.scale, True, "normal", std=b.std, d_v=dv,
                        note=b.note.replace(", P then P@V", "") + ", fused softmax(QK^T)V without materialising P",
                        extra={"fused_attention": True})
    if name.endswith("_softmax"):
        # the standalone row softmax over the score buffer of a batch (the second of upstream's two operators)
        b = workload(name[:-len("_softmax")], seed, segments)
        return Workload(name, b.M, b.N, b.K, b.H, b.out_dtype, b.out_dtype, 1.0, True, "normal", std=2.0,
                        note=b.note + ", standalone row softmax of its score buffer", extra={"softmax_only": True})
    if name == "large_k":
        S = segments or 64
        n = _i64(rs.randint(1024, 2049, size=S))
        K = _i64(rs.choice([1024, 2048, 4096], size=S))
        return Workload(name, n, n.copy(), K, 1, torch.float16, torch.float16, 1.0, False, "uniform",
                        note="64 segments, M=N~U{1024..2048}, K in {1024,2048,4096}, fp16, GEMM only (compute-bound)")
    raise ValueError(f"unknown workload {name!r}")


WORKLOADS = ("cpu_plumbing", "molecular", "molecular_attention", "general_gemm", "long_tail", "full_forward", "large_k",
             "long_tail_attention", "full_forward_attention", "long_tail_softmax", "full_forward_softmax",
             "molecular_softmax")
