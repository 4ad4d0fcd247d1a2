"""CPU oracle for the varlen blocked GEMM and the varlen row softmax.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this file;
only the tests, the smoke check and the benchmark's CPU-baseline leg do, and
only as the checker / the timed CPU baseline.

The upstream project has no CPU implementation (its launchers reject non-CUDA
tensors, ``csrc/sparseBlockedAttention.h:6-8``).  What it has is a per-segment
torch check loop, and this file restates that loop:

* packed head-major layout: ``blockedAttention/apply.py:12-23`` and ``:31-39``;
* per-segment ``matmul`` + ``cat`` check: ``csrc/sparseBlockedAttention.cpp:197``;
* per-segment ``reshape -> softmax(-1) -> cat`` check: ``test/pytest.py:55-59``;
* offsets from lists (``cat([0], M*K).cumsum``): ``csrc/sparseBlockedAttention.cpp:22-29``
  and ``:85-91``;
* lists from offsets (float32 ``sqrt`` formula): ``csrc/sparseBlockedAttention.cpp:30-40``;
* device addressing the loop must agree with: ``csrc/cuda/spBlkGEMM.cu:141-150``
  (segment start = head * D + accum[seg]) and ``csrc/cuda/spBlkSoftmax.cu:107``;
* backward pair: the argument permutation of ``csrc/sparseBlockedAttention.cpp:52-72`` and
  the row arithmetic of ``csrc/cuda/spBlkSoftmax.cu:140-180``; these two are additionally
  checked against torch autograd of the forward restatement (``tests/test_oracle.py``).

Parity pin: the upstream repository holds no golden vectors or known-answer
files (its only checks are run-time comparisons with torch on unseeded data),
so the pin is the upstream CUDA kernels themselves, compiled unmodified by
``oracle/build_ref.py`` and compared with this oracle by the GPU tests
(``tests/test_reference_ext.py``).  On a machine without a GPU that pin cannot
run and this oracle is "parity unpinned" there; the committed fixtures under
``tests/golden/`` then only guard it against drift.

All arithmetic is float32 on the CPU (float64 available for the tests that
want a tighter yard-stick); index arithmetic is int64 numpy.
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import numpy as np
import torch


# --------------------------------------------------------------------------
# index / offset derivation
# --------------------------------------------------------------------------
def offsets_from_lists(MList, NList, KList) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """``cat([0], M*K).cumsum(0)`` etc. -- csrc/sparseBlockedAttention.cpp:22-29."""
    M = np.asarray(MList, dtype=np.int64)
    N = np.asarray(NList, dtype=np.int64)
    K = np.asarray(KList, dtype=np.int64)
    z = np.zeros(1, dtype=np.int64)
    a1 = np.concatenate([z, M * K]).cumsum(dtype=np.int64)
    a2 = np.concatenate([z, N * K]).cumsum(dtype=np.int64)
    ao = np.concatenate([z, M * N]).cumsum(dtype=np.int64)
    return a1, a2, ao


def softmax_offsets(rowList, colList) -> np.ndarray:
    """``cat([0], rows*cols).cumsum(0)`` -- csrc/sparseBlockedAttention.cpp:85-91."""
    r = np.asarray(rowList, dtype=np.int64)
    c = np.asarray(colList, dtype=np.int64)
    return np.concatenate([np.zeros(1, dtype=np.int64), r * c]).cumsum(dtype=np.int64)


def lists_from_offsets_float32(a1, a2, ao) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """The upstream formula, bit for bit: csrc/sparseBlockedAttention.cpp:30-40.

    ``M = int64(sqrt(float32(mk*mn) / float32(nk)))``, ``N = int64(float32(mn) /
    float32(M))``, ``K = int64(float32(mk) / float32(M))`` -- torch's true
    division of int64 tensors promotes to float32.  Exact only while the
    products fit float32's 24-bit mantissa; beyond that it can truncate to
    M-1 (see ``lists_from_offsets_exact``).
    """
    a1 = np.asarray(a1, dtype=np.int64)
    a2 = np.asarray(a2, dtype=np.int64)
    ao = np.asarray(ao, dtype=np.int64)
    mk = a1[1:] - a1[:-1]
    nk = a2[1:] - a2[:-1]
    mn = ao[1:] - ao[:-1]
    with np.errstate(divide="ignore", invalid="ignore"):
        q = (mk * mn).astype(np.float32) / nk.astype(np.float32)
        M = np.sqrt(q).astype(np.int64)
        N = (mn.astype(np.float32) / M.astype(np.float32)).astype(np.int64)
        K = (mk.astype(np.float32) / M.astype(np.float32)).astype(np.int64)
    return M, N, K


def lists_from_offsets_exact(a1, a2, ao) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """Exact-integer statement of the same derivation (M^2 = mk*mn/nk).

    Agrees with ``lists_from_offsets_float32`` wherever that one is
    self-consistent (M*K == mk, N*K == nk, M*N == mn); raises ValueError where
    no integer solution exists.
    """
    import math
    a1 = [int(x) for x in np.asarray(a1).tolist()]
    a2 = [int(x) for x in np.asarray(a2).tolist()]
    ao = [int(x) for x in np.asarray(ao).tolist()]
    Ms, Ns, Ks = [], [], []
    for s in range(len(a1) - 1):
        mk, nk, mn = a1[s + 1] - a1[s], a2[s + 1] - a2[s], ao[s + 1] - ao[s]
        if mk <= 0 or nk <= 0 or mn <= 0:
            raise ValueError(f"segment {s}: empty extents cannot be inverted")
        num = mk * mn
        if num % nk:
            raise ValueError(f"segment {s}: offsets are not those of an (M,N,K) segment")
        m = math.isqrt(num // nk)
        if m * m != num // nk or mn % m or mk % m or (mn // m) * (mk // m) != nk:
            raise ValueError(f"segment {s}: offsets are not those of an (M,N,K) segment")
        Ms.append(m); Ns.append(mn // m); Ks.append(mk // m)
    return (np.asarray(Ms, dtype=np.int64), np.asarray(Ns, dtype=np.int64),
            np.asarray(Ks, dtype=np.int64))


# --------------------------------------------------------------------------
# the per-segment loops
# --------------------------------------------------------------------------
def _as2d(x: torch.Tensor, D: int) -> torch.Tensor:
    # any leading shape flattens to H (csrc/cuda/spBlkGEMM.cu:999)
    return x.reshape(-1, D)


def block_gemm(mat1: torch.Tensor, mat2: torch.Tensor, MList, NList, KList,
               accum1=None, accum2=None, accumOut=None,
               transpose1: bool = False, transpose2: bool = False,
               scale: float = 1.0, compute_dtype=torch.float32) -> torch.Tensor:
    """out[h, accumOut[s] + m*N_s + n] = scale * sum_k A_s[h,m,k] * B_s[h,n,k].

    A_s is stored (M_s, K_s) row-major, or (K_s, M_s) when ``transpose1``;
    B_s is stored (N_s, K_s), or (K_s, N_s) when ``transpose2``
    (blockedAttention/apply.py:21-22).  Returns ``compute_dtype`` (float32) on
    the CPU; the caller rounds to the dtype it compares with.
    """
    M = np.asarray(MList, dtype=np.int64); N = np.asarray(NList, dtype=np.int64)
    K = np.asarray(KList, dtype=np.int64)
    d1, d2, do = offsets_from_lists(M, N, K)
    a1 = d1 if accum1 is None else np.asarray(accum1, dtype=np.int64)
    a2 = d2 if accum2 is None else np.asarray(accum2, dtype=np.int64)
    ao = do if accumOut is None else np.asarray(accumOut, dtype=np.int64)
    m1 = _as2d(mat1.detach().cpu(), int(a1[-1])).to(compute_dtype)
    m2 = _as2d(mat2.detach().cpu(), int(a2[-1])).to(compute_dtype)
    H = m1.shape[0]
    out = torch.zeros((H, int(ao[-1])), dtype=compute_dtype)
    for s in range(len(M)):
        m, n, k = int(M[s]), int(N[s]), int(K[s])
        if m == 0 or n == 0:
            continue
        A = m1[:, a1[s]:a1[s] + m * k]
        B = m2[:, a2[s]:a2[s] + n * k]
        A = A.reshape(H, k, m).transpose(1, 2) if transpose1 else A.reshape(H, m, k)
        B = B.reshape(H, k, n).transpose(1, 2) if transpose2 else B.reshape(H, n, k)
        C = torch.matmul(A, B.transpose(1, 2))
        if scale != 1.0:
            C = C * scale
        out[:, ao[s]:ao[s] + m * n] = C.reshape(H, m * n)
    return out


def block_softmax(src: torch.Tensor, rowList, colList, srcAccum=None,
                  scale: float = 1.0, compute_dtype=torch.float32) -> torch.Tensor:
    """Row softmax of every (rows_s, cols_s) block -- test/pytest.py:55-59."""
    r = np.asarray(rowList, dtype=np.int64); c = np.asarray(colList, dtype=np.int64)
    acc = softmax_offsets(r, c) if srcAccum is None else np.asarray(srcAccum, dtype=np.int64)
    x = _as2d(src.detach().cpu(), int(acc[-1])).to(compute_dtype)
    H = x.shape[0]
    out = torch.zeros_like(x)
    for s in range(len(r)):
        rows, cols = int(r[s]), int(c[s])
        if rows == 0 or cols == 0:
            continue
        blk = x[:, acc[s]:acc[s] + rows * cols].reshape(H, rows, cols)
        if scale != 1.0:
            blk = blk * scale
        out[:, acc[s]:acc[s] + rows * cols] = blk.softmax(-1).reshape(H, rows * cols)
    return out


def block_scores(q: torch.Tensor, k: torch.Tensor, MList, NList, KList, scale: float = 1.0,
                 compute_dtype=torch.float32) -> torch.Tensor:
    """softmax_rows(scale * Q_s K_s^T) per segment, no rounding in between."""
    s = block_gemm(q, k, MList, NList, KList, scale=scale, compute_dtype=compute_dtype)
    return block_softmax(s, MList, NList, compute_dtype=compute_dtype)


def block_attention(q, k, v, nList, d: int, scale: float, p_dtype=None,
                    compute_dtype=torch.float32) -> Tuple[torch.Tensor, torch.Tensor]:
    """P = softmax(scale Q K^T); O = P V with V stored (n_s, d) = the (K, N)
    layout of ``transpose2=True``.  ``p_dtype`` rounds P before the second
    product, as a materialised 16-bit P buffer does."""
    n = np.asarray(nList, dtype=np.int64)
    dl = np.full_like(n, d)
    P = block_scores(q, k, n, n, dl, scale=scale, compute_dtype=compute_dtype)
    Pr = P.to(p_dtype).to(compute_dtype) if p_dtype is not None else P
    O = block_gemm(Pr, v, n, dl, n, transpose2=True, compute_dtype=compute_dtype)
    return P, O


def block_softmax_backward(out: torch.Tensor, grad_out: torch.Tensor, rowList, colList, srcAccum=None,
                           scale: float = 1.0, compute_dtype=torch.float32) -> torch.Tensor:
    """grad_src = scale * (grad_out - rowsum(out * grad_out)) * out per row of every block: the arithmetic of
    upstream sparseBlockedSoftmaxBackward_warp (csrc/cuda/spBlkSoftmax.cu:140-180: fp32 dot product of the two
    rows, then ``(dsrc - sum) * src``), with the forward scale folded in (upstream has none)."""
    r = np.asarray(rowList, dtype=np.int64); c = np.asarray(colList, dtype=np.int64)
    acc = softmax_offsets(r, c) if srcAccum is None else np.asarray(srcAccum, dtype=np.int64)
    P = _as2d(out.detach().cpu(), int(acc[-1])).to(compute_dtype)
    G = _as2d(grad_out.detach().cpu(), int(acc[-1])).to(compute_dtype)
    H = P.shape[0]
    res = torch.zeros_like(P)
    for s in range(len(r)):
        rows, cols = int(r[s]), int(c[s])
        if rows == 0 or cols == 0:
            continue
        p = P[:, acc[s]:acc[s] + rows * cols].reshape(H, rows, cols)
        g = G[:, acc[s]:acc[s] + rows * cols].reshape(H, rows, cols)
        dot = (p * g).sum(-1, keepdim=True)
        res[:, acc[s]:acc[s] + rows * cols] = ((g - dot) * p * scale).reshape(H, rows * cols)
    return res


def block_gemm_backward(mat1: torch.Tensor, mat2: torch.Tensor, grad_out: torch.Tensor, MList, NList, KList,
                        accum1=None, accum2=None, accumOut=None, transpose1: bool = False,
                        transpose2: bool = False, scale: float = 1.0,
                        compute_dtype=torch.float32) -> Tuple[torch.Tensor, torch.Tensor]:
    """The two launches of upstream sparseBlockedGEMM::backward (csrc/sparseBlockedAttention.cpp:52-72), each
    restated through :func:`block_gemm` with upstream's permuted arguments:
    mat1Grad = gemm(outGrad, mat2; offsets (out, mat2, mat1); lists (M, K, N); False, not transpose2),
    mat2Grad = gemm(outGrad, mat1; offsets (out, mat1, mat2); lists (N, K, M); True, not transpose1)."""
    M = np.asarray(MList, dtype=np.int64); N = np.asarray(NList, dtype=np.int64)
    K = np.asarray(KList, dtype=np.int64)
    d1, d2, do = offsets_from_lists(M, N, K)
    a1 = d1 if accum1 is None else np.asarray(accum1, dtype=np.int64)
    a2 = d2 if accum2 is None else np.asarray(accum2, dtype=np.int64)
    ao = do if accumOut is None else np.asarray(accumOut, dtype=np.int64)
    g1 = block_gemm(grad_out, mat2, M, K, N, ao, a2, a1, False, not transpose2, scale=scale, compute_dtype=compute_dtype)
    g2 = block_gemm(grad_out, mat1, N, K, M, ao, a1, a2, True, not transpose1, scale=scale, compute_dtype=compute_dtype)
    return g1, g2


# --------------------------------------------------------------------------
# timed CPU baseline (the benchmark's cpu_baseline / reference arm)
# --------------------------------------------------------------------------
def timed_scores_loop(q: torch.Tensor, k: torch.Tensor, nList: Sequence[int], d: int,
                      scale: float, threads: Optional[int] = None) -> Tuple[float, torch.Tensor]:
    """One pass of the per-segment torch loop on the host cores; returns
    (seconds, packed probabilities).  Inputs are float32 CPU tensors (H, sum n*d)."""
    import time
    if threads:
        torch.set_num_threads(threads)
    n = np.asarray(nList, dtype=np.int64)
    dl = np.full_like(n, d)
    t0 = time.perf_counter()
    out = block_scores(q, k, n, n, dl, scale=scale)
    return time.perf_counter() - t0, out
