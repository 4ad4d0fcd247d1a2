"""Python surface: ``blockGEMM`` and ``blockSoftmax`` with the upstream
signatures (``blockedAttention/apply.py:6-11`` and ``:27-30``), plus the fused
``blockAttnScores``.

Differences from upstream, all at the boundary:

* keyword-only extensions ``scale``, ``out_dtype`` and ``softmax`` (defaults
  reproduce upstream behaviour: no scale, output dtype = input dtype, separate
  softmax call);
* lists/offsets are read to the host once per distinct (tensor, version) and
  the resulting plan is cached, where upstream synchronises seven to eleven
  times per call;
* the shape checks upstream leaves to ``assert`` raise ``RuntimeError``;
* ``blockSoftmax`` passes its arguments by name, so ``srcAccum`` reaches the
  offsets parameter (upstream ``apply.py:41`` hands it to ``rowList``);
* forward only: outputs do not carry autograd history.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Optional

import numpy as np
import torch

from . import _lib as L
from .plan import GemmPlan, SoftmaxPlan, _host_i64

_CACHE: "OrderedDict[tuple, object]" = OrderedDict()
_CACHE_MAX = 32


def _key_of(x):
    if x is None:
        return None
    if isinstance(x, torch.Tensor):
        return ("t", x.data_ptr(), x._version, x.numel(), str(x.device))
    a = np.asarray(x, dtype=np.int64)
    return ("h", a.tobytes())


def _cached(key, build):
    plan = _CACHE.get(key)
    if plan is None:
        plan = build()
        _CACHE[key] = plan
        while len(_CACHE) > _CACHE_MAX:
            _CACHE.popitem(last=False)[1].close()
    else:
        _CACHE.move_to_end(key)
    return plan


def clear_plan_cache() -> None:
    while _CACHE:
        _CACHE.popitem()[1].close()


def _check_operand(name: str, t: torch.Tensor) -> None:
    # the two TORCH_CHECKs of upstream csrc/sparseBlockedAttention.h:6-8
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise RuntimeError(f"{name} must be CUDA Tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous Tensor")


def _lists_from_offsets(a1, a2, ao):
    a1, a2, ao = _host_i64(a1), _host_i64(a2), _host_i64(ao)
    S = len(a1) - 1
    M = np.empty(S, np.int64); N = np.empty(S, np.int64); K = np.empty(S, np.int64)
    L.check(L.lib.blk_lists_from_offsets(L.i64(a1), L.i64(a2), L.i64(ao), S, L.i64(M), L.i64(N), L.i64(K)))
    return M, N, K


def blockGEMM(mat1: torch.Tensor, mat2: torch.Tensor,
              mat1Accum: Optional[torch.Tensor] = None, mat2Accum: Optional[torch.Tensor] = None,
              outAccum: Optional[torch.Tensor] = None,
              MList: Optional[torch.Tensor] = None, NList: Optional[torch.Tensor] = None,
              KList: Optional[torch.Tensor] = None,
              transpose1: Optional[bool] = False, transpose2: Optional[bool] = False,
              *, scale: float = 1.0, out_dtype: Optional[torch.dtype] = None,
              softmax: bool = False) -> torch.Tensor:
    """Varlen blocked GEMM over a packed, head-major batch.

    ``mat1 -> (H, sum m_s*k_s)``, ``mat2 -> (H, sum n_s*k_s)``, result
    ``(H, sum m_s*n_s)`` with ``out_s = mat1_s @ mat2_s^T``.  Give either the
    three offset tensors (``mat1Accum = (0, m1*k1, m1*k1+m2*k2, ...)`` and so
    on) or the three lists (``MList = (m1, m2, ...)``), or both.
    ``transpose1``: mat1_s is stored (k, m); ``transpose2``: mat2_s is stored
    (k, n).  Any leading shape of mat1 flattens to H.
    """
    _check_operand("mat1", mat1)
    _check_operand("mat2", mat2)
    have_acc = mat1Accum is not None and mat2Accum is not None and outAccum is not None
    have_lists = MList is not None and NList is not None and KList is not None
    if not (have_acc or have_lists):
        raise RuntimeError("blockGEMM needs either mat1Accum/mat2Accum/outAccum or MList/NList/KList")
    if mat1.dtype != mat2.dtype:
        raise RuntimeError("mat1 and mat2 must have the same dtype")
    odt = out_dtype if out_dtype is not None else mat1.dtype
    key = ("gemm", _key_of(mat1Accum) if have_acc else None, _key_of(mat2Accum) if have_acc else None,
           _key_of(outAccum) if have_acc else None, _key_of(MList) if have_lists else None,
           _key_of(NList) if have_lists else None, _key_of(KList) if have_lists else None,
           mat1.numel(), mat1.dtype, odt, bool(transpose1), bool(transpose2), bool(softmax), str(mat1.device))

    def build():
        if have_lists:
            M, N, K = _host_i64(MList), _host_i64(NList), _host_i64(KList)
        else:
            M, N, K = _lists_from_offsets(mat1Accum, mat2Accum, outAccum)
        accum = (mat1Accum, mat2Accum, outAccum) if have_acc else None
        Dm1 = int(_host_i64(mat1Accum)[-1]) if have_acc else int((M * K).sum())
        if Dm1 <= 0 or mat1.numel() % Dm1:
            raise RuntimeError(f"mat1 has {mat1.numel()} elements, not a multiple of the packed extent {Dm1}")
        H = mat1.numel() // Dm1
        return GemmPlan(M, N, K, H, mat1.dtype, odt, bool(transpose1), bool(transpose2), bool(softmax),
                        accum=accum, device=mat1.device)

    plan = _cached(key, build)
    if mat1.shape[-1] != plan.Dm1 and mat1.numel() != plan.H * plan.Dm1:
        raise RuntimeError(f"mat1.size(-1) = {mat1.shape[-1]} does not match mat1Accum[-1] = {plan.Dm1}")
    return plan.run(mat1, mat2, scale=scale)


def blockSoftmax(src: torch.Tensor, rowList: torch.Tensor, colList: torch.Tensor,
                 srcAccum: Optional[torch.Tensor] = None, *, scale: float = 1.0,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Row softmax (last dim) of every packed block.

    ``src -> (H, sum rows_s*cols_s)``, result has the same shape; ``rowList =
    (rows_1, rows_2, ...)``, ``colList = (cols_1, ...)``; ``srcAccum = (0,
    rows_1*cols_1, ...)`` is optional.  ``out=src`` runs in place.
    """
    _check_operand("src", src)
    if rowList is None or colList is None:
        raise RuntimeError("blockSoftmax needs rowList and colList")
    key = ("smx", _key_of(rowList), _key_of(colList), _key_of(srcAccum), src.numel(), src.dtype, str(src.device))

    def build():
        rows, cols = _host_i64(rowList), _host_i64(colList)
        D = int(_host_i64(srcAccum)[-1]) if srcAccum is not None else int((rows * cols).sum())
        if D <= 0 or src.numel() % D:
            raise RuntimeError(f"src has {src.numel()} elements, not a multiple of the packed extent {D}")
        return SoftmaxPlan(rows, cols, src.numel() // D, src.dtype, accum=srcAccum, device=src.device)

    plan = _cached(key, build)
    return plan.run(src, out=out, scale=scale)


def blockAttnScores(q: torch.Tensor, k: torch.Tensor, MList, NList, KList, scale: float = 1.0,
                    out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``softmax_rows(scale * Q_s K_s^T)`` for every segment in one pass: the
    fused form of ``blockSoftmax(blockGEMM(q, k, ...), MList, NList)``; the raw
    scores are never written to memory."""
    return blockGEMM(q, k, None, None, None, MList, NList, KList, False, False,
                     scale=scale, out_dtype=out_dtype, softmax=True)
