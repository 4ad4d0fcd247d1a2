"""GPU: every benchmark configuration at its full size, seed 0, every segment checked.

The CPU oracle needs minutes for these batches, so each one is compared twice:
all segments against the per-segment fp32 ``matmul`` (+ ``softmax``) loop run on
the device -- the loop of upstream test/pytest.py:55-59 and
csrc/sparseBlockedAttention.cpp:197 -- and a seeded sample of at least 32
segments (the smallest, the largest, every degenerate one-node graph, random
others) against ``oracle/blk_oracle.py`` on the CPU.  Tolerances are those of
the parity contract (helpers.py): probabilities 2e-3 max-abs, raw scores 1e-2
relative with a floor of 1e-3 rms for cancellation.
"""
import numpy as np
import pytest
import torch

from helpers import O, PROB_ATOL, SCORE_RTOL, assert_probs_close, assert_scores_close
from blockedattention_b200 import blockAttention, blockAttnScores, blockGEMM
from blockedattention_b200.synth import workload

pytestmark = pytest.mark.gpu


def sample_segments(w, count=32, seed=0):
    order = np.argsort(w.M * w.N, kind="stable")
    pick = {int(order[0]), int(order[-1])}
    pick |= {int(s) for s in np.nonzero((w.M == 1) | (w.N == 1))[0]}
    rs = np.random.RandomState(seed)
    for s in rs.permutation(w.S):
        if len(pick) >= max(count, 2):
            break
        pick.add(int(s))
    return sorted(pick)


def offsets(w):
    return O.offsets_from_lists(w.M, w.N, w.K)


def seg(t, acc, s, H, rows, cols):
    return t[:, acc[s]:acc[s + 1]].reshape(H, rows, cols)


def device_scores_check(w, q, k, out, softmax):
    """All segments against the fp32 loop on the device; returns (worst probability error or count of scores out of
    tolerance) as a Python number after one synchronisation."""
    a1, a2, ao = offsets(w)
    worst = torch.zeros((), device=q.device)
    bad = torch.zeros((), dtype=torch.int64, device=q.device)
    for s in range(w.S):
        m, n, kk = int(w.M[s]), int(w.N[s]), int(w.K[s])
        if m == 0 or n == 0:
            continue
        ref = seg(q, a1, s, w.H, m, kk).float() @ seg(k, a2, s, w.H, n, kk).float().mT * w.scale
        got = seg(out, ao, s, w.H, m, n).float()
        if softmax:
            worst = torch.maximum(worst, (got - torch.softmax(ref, dim=-1)).abs().max())
        else:
            rms = ref.pow(2).mean().sqrt()
            bad += ((got - ref).abs() > SCORE_RTOL * ref.abs() + 1e-3 * rms).sum()
    return float(worst), int(bad)


def test_general_gemm_full_size(cuda_device):
    w = workload("general_gemm")
    dev = cuda_device
    q, k = w.make_inputs(dev, seed=0)
    out = blockGEMM(q, k, None, None, None, w.M, w.N, w.K, scale=w.scale, out_dtype=w.out_dtype)
    torch.cuda.synchronize()
    assert out.shape == (w.H, w.Dout) and out.dtype == torch.float32
    _, bad = device_scores_check(w, q, k, out, softmax=False)
    assert bad == 0, f"{bad} scores out of tolerance against the fp32 loop on the device"
    a1, a2, ao = offsets(w)
    qc, kc, oc = q.cpu(), k.cpu(), out.cpu()
    for s in sample_segments(w, 48):
        ref = O.block_gemm(qc[:, a1[s]:a1[s + 1]], kc[:, a2[s]:a2[s + 1]], w.M[s:s + 1], w.N[s:s + 1], w.K[s:s + 1],
                           scale=w.scale)
        assert_scores_close(oc[:, ao[s]:ao[s + 1]], ref, f"segment {s} vs oracle")
    # the drop-in variant (output in the input dtype, as upstream csrc/cuda/spBlkGEMM.cu:1008)
    out16 = blockGEMM(q, k, None, None, None, w.M, w.N, w.K)
    assert out16.dtype == torch.float16
    _, bad = device_scores_check(w, q, k, out16, softmax=False)
    assert bad == 0


def test_long_tail_full_size(cuda_device):
    w = workload("long_tail")
    dev = cuda_device
    q, k = w.make_inputs(dev, seed=0)
    P = blockAttnScores(q, k, w.M, w.N, w.K, scale=w.scale)
    torch.cuda.synchronize()
    worst, _ = device_scores_check(w, q, k, P, softmax=True)
    assert worst <= PROB_ATOL, f"worst probability error over all {w.S} segments {worst:.3e}"
    a1, a2, ao = offsets(w)
    for s in sample_segments(w, 32):
        ref = O.block_scores(q[:, a1[s]:a1[s + 1]].cpu(), k[:, a2[s]:a2[s + 1]].cpu(), w.M[s:s + 1], w.N[s:s + 1],
                             w.K[s:s + 1], scale=w.scale)
        assert_probs_close(P[:, ao[s]:ao[s + 1]], ref, f"segment {s} (n={int(w.M[s])}) vs oracle")


def attention_bound(ref, v):
    # relative tolerance of the raw-score contract plus a floor for cancellation: a result element is a sum of
    # products of probabilities (rounded to 16 bits before the second product) and values, so its absolute error
    # scales with the largest value, not with the element
    return SCORE_RTOL * ref.abs() + 1e-3 * v.abs().max()


def test_full_forward_full_size_p_then_pv(cuda_device):
    # configuration 5 as specified: P = softmax(QK^T/sqrt(d)) fused, then O = P V through the same blocked GEMM
    w = workload("full_forward")
    dev = cuda_device
    q, k, v = w.make_inputs(dev, seed=0)
    d = int(w.K[0])
    dl = np.full_like(w.M, d)
    P = blockAttnScores(q, k, w.M, w.N, w.K, scale=w.scale)
    Oout = blockGEMM(P, v, None, None, None, w.M, dl, w.N, False, True)
    torch.cuda.synchronize()
    assert Oout.shape == (w.H, int(w.M.sum()) * d)
    worst, _ = device_scores_check(w, q, k, P, softmax=True)
    assert worst <= PROB_ATOL, f"worst probability error over all {w.S} segments {worst:.3e}"
    # second product, every segment: against fp32 P V on the P it was given
    a1, a2, ao = offsets(w)
    bad = torch.zeros((), dtype=torch.int64, device=dev)
    for s in range(w.S):
        n = int(w.M[s])
        ref = seg(P, ao, s, w.H, n, n).float() @ seg(v, a2, s, w.H, n, d).float()
        got = seg(Oout, a1, s, w.H, n, d).float()
        rms = ref.pow(2).mean().sqrt()
        bad += ((got - ref).abs() > SCORE_RTOL * ref.abs() + 1e-3 * rms).sum()
    assert int(bad) == 0, f"{int(bad)} elements of O = P V out of tolerance"
    for s in sample_segments(w, 32):      # includes the 64 one-node graphs
        sl = slice(s, s + 1)
        qs, ks, vs = (t[:, a1[s]:a1[s + 1]].cpu() for t in (q, k, v))
        Pref, Oref = O.block_attention(qs, ks, vs, w.M[sl], d, w.scale, p_dtype=w.dtype)
        assert_probs_close(P[:, ao[s]:ao[s + 1]], Pref, f"P of segment {s} vs oracle")
        got = Oout[:, a1[s]:a1[s + 1]].float().cpu()
        assert bool(((got - Oref).abs() <= attention_bound(Oref, vs.float())).all()), f"O of segment {s} vs oracle"


@pytest.mark.parametrize("name", ["full_forward_attention", "long_tail_attention"])
def test_fused_attention_full_size(cuda_device, name):
    w = workload(name)
    dev = cuda_device
    q, k, v = w.make_inputs(dev, seed=0)
    d = int(w.K[0])
    out = blockAttention(q, k, v, w.M, w.N, scale=w.scale, d=d)
    torch.cuda.synchronize()
    a1, a2, _ = offsets(w)
    vmax = v.float().abs().max()
    bad = torch.zeros((), dtype=torch.int64, device=dev)
    worst = torch.zeros((), device=dev)
    for s in range(w.S):
        n = int(w.M[s])
        qs, ks, vs = (seg(t, a1, s, w.H, n, d).float() for t in (q, k, v))
        ref = torch.softmax(qs @ ks.mT * w.scale, dim=-1) @ vs
        err = (seg(out, a1, s, w.H, n, d).float() - ref).abs()
        bad += (err > SCORE_RTOL * ref.abs() + 1e-3 * vmax).sum()
        worst = torch.maximum(worst, (err / (SCORE_RTOL * ref.abs() + 1e-3 * vmax)).max())
    assert int(bad) == 0, f"{int(bad)} result elements out of tolerance (worst {float(worst):.2f}x the bound)"
    for s in sample_segments(w, 32):
        qs, ks, vs = (t[:, a1[s]:a1[s + 1]].cpu() for t in (q, k, v))
        _, Oref = O.block_attention(qs, ks, vs, w.M[s:s + 1], d, w.scale)
        got = out[:, a1[s]:a1[s + 1]].float().cpu()
        assert bool(((got - Oref).abs() <= attention_bound(Oref, vs.float())).all()), f"segment {s} vs oracle"
