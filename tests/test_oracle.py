"""CPU: the oracle against the committed golden vectors, and its index helpers."""
import glob
import os

import numpy as np
import pytest
import torch

from helpers import O, assert_probs_close, assert_scores_close

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz")))
_DT = {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}


def load_golden(path):
    z = np.load(path)
    d = {k: z[k] for k in z.files}
    dt = _DT[str(d["dtype"])]

    def t(a):
        x = torch.from_numpy(np.ascontiguousarray(a))
        return x.view(torch.bfloat16) if dt == torch.bfloat16 else x
    d["torch_dtype"] = dt
    for k in ("A", "B", "X"):
        if k in d:
            d[k] = t(d[k])
    d["out"] = torch.from_numpy(d["out"])
    return d


def test_golden_present():
    assert len(GOLDEN) >= 8


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_oracle_matches_golden(path):
    d = load_golden(path)
    if str(d["kind"]) == "gemm":
        out = O.block_gemm(d["A"], d["B"], d["M"], d["N"], d["K"], transpose1=bool(d["ta"]),
                           transpose2=bool(d["tb"]), scale=float(d["scale"]))
        if bool(d["softmax"]):
            out = O.block_softmax(out, d["M"], d["N"])
        a1, a2, ao = O.offsets_from_lists(d["M"], d["N"], d["K"])
        assert (a1 == d["a1"]).all() and (a2 == d["a2"]).all() and (ao == d["ao"]).all()
    elif str(d["kind"]) == "attention":
        dl = np.full_like(d["M"], int(d["d"]))
        out = O.block_gemm(O.block_scores(d["A"], d["B"], d["M"], d["N"], dl, scale=float(d["scale"])), d["X"],
                           d["M"], dl, d["N"], transpose2=True)
    else:
        out = O.block_softmax(d["X"], d["rows"], d["cols"])
        assert (O.softmax_offsets(d["rows"], d["cols"]) == d["acc"]).all()
    # same machine arithmetic up to BLAS summation order
    torch.testing.assert_close(out, d["out"], rtol=1e-5, atol=1e-5)


def test_arange_case_is_exact_integers():
    d = load_golden([p for p in GOLDEN if "arange" in p][0])
    A = d["A"].double().reshape(11, 5); B = d["B"].double().reshape(13, 5)
    assert torch.equal((A @ B.T).reshape(1, -1).float(), d["out"])


def test_oracle_float64_agrees():
    rs = np.random.RandomState(3)
    M = rs.randint(1, 40, 6); N = rs.randint(1, 40, 6); K = rs.randint(1, 70, 6)
    g = torch.Generator().manual_seed(0)
    A = torch.randn((3, int((M * K).sum())), generator=g)
    B = torch.randn((3, int((N * K).sum())), generator=g)
    for ta in (False, True):
        for tb in (False, True):
            s32 = O.block_gemm(A, B, M, N, K, transpose1=ta, transpose2=tb, scale=0.25)
            s64 = O.block_gemm(A, B, M, N, K, transpose1=ta, transpose2=tb, scale=0.25, compute_dtype=torch.float64)
            torch.testing.assert_close(s32.double(), s64, rtol=1e-4, atol=1e-4)
    p32 = O.block_scores(A, A, M, M, K, scale=0.3)
    p64 = O.block_scores(A, A, M, M, K, scale=0.3, compute_dtype=torch.float64)
    assert_probs_close(p32, p64.float())
    # rows of a softmax block sum to one
    acc = O.softmax_offsets(M, M)
    for s in range(len(M)):
        blk = p32[:, acc[s]:acc[s + 1]].reshape(3, M[s], M[s])
        torch.testing.assert_close(blk.sum(-1), torch.ones(3, M[s]), rtol=1e-5, atol=1e-5)


def test_offsets_against_torch_cumsum():
    # the literal upstream expression (csrc/sparseBlockedAttention.cpp:24-28) in torch
    M = torch.tensor([33, 99, 64, 1, 0, 7]); N = torch.tensor([33, 99, 64, 5, 3, 0]); K = torch.tensor([64, 64, 64, 9, 2, 4])
    z = torch.zeros(1, dtype=M.dtype)
    a1, a2, ao = O.offsets_from_lists(M.numpy(), N.numpy(), K.numpy())
    assert a1.dtype == np.int64
    assert (torch.cat([z, M * K]).cumsum(0).numpy() == a1).all()
    assert (torch.cat([z, N * K]).cumsum(0).numpy() == a2).all()
    assert (torch.cat([z, M * N]).cumsum(0).numpy() == ao).all()


def test_lists_from_offsets_float32_is_the_upstream_expression():
    M = torch.tensor([33, 127, 11, 60, 5]); N = torch.tensor([33, 127, 13, 60, 5]); K = torch.tensor([61, 61, 5, 32, 32])
    a1, a2, ao = (torch.from_numpy(a) for a in O.offsets_from_lists(M.numpy(), N.numpy(), K.numpy()))
    mk, nk, mn = a1[1:] - a1[:-1], a2[1:] - a2[:-1], ao[1:] - ao[:-1]
    Mt = ((mk * mn) / nk).sqrt().to(torch.int64)           # csrc/sparseBlockedAttention.cpp:37
    Nt = (mn / Mt).to(torch.int64); Kt = (mk / Mt).to(torch.int64)
    Mo, No, Ko = O.lists_from_offsets_float32(a1.numpy(), a2.numpy(), ao.numpy())
    assert (Mo == Mt.numpy()).all() and (No == Nt.numpy()).all() and (Ko == Kt.numpy()).all()
    assert (Mo == M.numpy()).all() and (No == N.numpy()).all() and (Ko == K.numpy()).all()
    Me, Ne, Ke = O.lists_from_offsets_exact(a1.numpy(), a2.numpy(), ao.numpy())
    assert (Me == Mo).all() and (Ne == No).all() and (Ke == Ko).all()


def test_exact_inverse_where_float32_formula_fails():
    # products beyond float32's mantissa: the upstream formula can land on M-1; the exact one cannot
    rs = np.random.RandomState(0)
    M = rs.randint(200, 3000, 400); N = rs.randint(200, 3000, 400); K = rs.randint(1, 300, 400)
    a1, a2, ao = O.offsets_from_lists(M, N, K)
    Me, Ne, Ke = O.lists_from_offsets_exact(a1, a2, ao)
    assert (Me == M).all() and (Ne == N).all() and (Ke == K).all()
    Mf, Nf, Kf = O.lists_from_offsets_float32(a1, a2, ao)
    consistent = (Mf * Kf == a1[1:] - a1[:-1]) & (Nf * Kf == a2[1:] - a2[:-1]) & (Mf * Nf == ao[1:] - ao[:-1])
    assert ((Mf == M) | ~consistent).all()       # wherever upstream is self-consistent it equals the truth
    with pytest.raises(ValueError):
        O.lists_from_offsets_exact([0, 6], [0, 6], [0, 5])


@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False)])
def test_backward_restatements_against_autograd(ta, tb):
    # the oracle's backward pair (upstream's permuted launches, upstream's softmax-backward arithmetic) against
    # torch autograd of the forward restatement, float64
    rs = np.random.RandomState(3)
    M = rs.randint(1, 9, size=5); N = rs.randint(1, 9, size=5); K = rs.randint(1, 7, size=5)
    H = 3
    A = torch.randn(H, int((M * K).sum()), dtype=torch.float64, requires_grad=True)
    B = torch.randn(H, int((N * K).sum()), dtype=torch.float64, requires_grad=True)

    def fwd(a, b):
        outs = []
        o1 = o2 = 0
        for m, n, k in zip(M, N, K):
            m, n, k = int(m), int(n), int(k)
            x = a[:, o1:o1 + m * k]; y = b[:, o2:o2 + n * k]
            x = x.reshape(H, k, m).transpose(1, 2) if ta else x.reshape(H, m, k)
            y = y.reshape(H, k, n).transpose(1, 2) if tb else y.reshape(H, n, k)
            outs.append((0.7 * x @ y.transpose(1, 2)).reshape(H, m * n))
            o1 += m * k; o2 += n * k
        return torch.cat(outs, 1)

    C = fwd(A, B)
    g = torch.randn_like(C)
    C.backward(g)
    g1, g2 = O.block_gemm_backward(A, B, g, M, N, K, transpose1=ta, transpose2=tb, scale=0.7,
                                   compute_dtype=torch.float64)
    # upstream lays both gradients out (m, k) / (n, k) row-major whatever the forward flags were
    def relayout(grad, rows, cols, transposed):
        if not transposed:
            return grad
        parts, o = [], 0
        for r, c in zip(rows, cols):
            r, c = int(r), int(c)
            parts.append(grad[:, o:o + r * c].reshape(H, c, r).transpose(1, 2).reshape(H, r * c)); o += r * c
        return torch.cat(parts, 1)
    assert torch.allclose(g1, relayout(A.grad, M, K, ta), atol=1e-10)
    assert torch.allclose(g2, relayout(B.grad, N, K, tb), atol=1e-10)

    # softmax backward
    X = torch.randn(H, int((M * N).sum()), dtype=torch.float64, requires_grad=True)
    outs, o = [], 0
    for m, n in zip(M, N):
        m, n = int(m), int(n)
        outs.append((1.3 * X[:, o:o + m * n].reshape(H, m, n)).softmax(-1).reshape(H, m * n)); o += m * n
    P = torch.cat(outs, 1)
    gp = torch.randn_like(P)
    P.backward(gp)
    got = O.block_softmax_backward(P, gp, M, N, scale=1.3, compute_dtype=torch.float64)
    assert torch.allclose(got, X.grad, atol=1e-10)
