"""GPU parity of the varlen blocked GEMM (all kernels behind blk_gemm_run) with
the CPU oracle, through the C ABI (GemmPlan -> ctypes -> libblkattn)."""
import os

import numpy as np
import pytest
import torch

from helpers import O, assert_probs_close, assert_scores_close, packed_inputs
from blockedattention_b200 import (blockAttnScores, blockAttnScoresHost, blockAttnScoresTokenMajor, blockGEMM,
                                   blockSoftmax)
from blockedattention_b200 import _lib as L
from blockedattention_b200.plan import GemmPlan
from blockedattention_b200.synth import workload

pytestmark = pytest.mark.gpu
F16, BF16, F32 = torch.float16, torch.bfloat16, torch.float32


def run_case(dev, M, N, K, H, dtype, ta=False, tb=False, softmax=False, scale=1.0, out_dtype=None, seed=0,
             dist="normal", std=1.0, accum=None, env=None, what=""):
    M = np.asarray(M, np.int64); N = np.asarray(N, np.int64); K = np.asarray(K, np.int64)
    a1 = a2 = ao = None
    if accum is not None:
        a1, a2, ao = accum
    A, B = packed_inputs(M, N, K, H, dtype, seed, dist, std, a1, a2)
    ref = O.block_gemm(A, B, M, N, K, a1, a2, ao, ta, tb, scale)
    if softmax:
        ref = O.block_softmax(ref, M, N, ao)
    old = {}
    for k, v in (env or {}).items():
        old[k] = os.environ.get(k); os.environ[k] = v
    try:
        plan = GemmPlan(M, N, K, H, dtype, out_dtype, ta, tb, softmax, accum=accum, device=dev)
    finally:
        for k, v in old.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v
    out = torch.full((H, plan.Dout), float("nan"), dtype=plan.dtype_out, device=dev)
    plan.run(A.to(dev), B.to(dev), out=out, scale=scale)
    torch.cuda.synchronize()
    got = out.float().cpu()
    if accum is not None:  # gaps between segments are not written: compare segment by segment
        keep = torch.zeros(plan.Dout, dtype=torch.bool)
        for s in range(len(M)):
            keep[ao[s]:ao[s] + M[s] * N[s]] = True
        assert torch.isnan(got[:, ~keep]).all(), f"{what}: wrote outside the segments"
        got, ref = got[:, keep], ref[:, keep]
    (assert_probs_close if softmax else assert_scores_close)(got, ref, what)
    return plan


def test_upstream_author_shapes(cuda_device):
    # csrc/sparseBlockedAttention.cpp:170-199 (odd K), :216-255, :147-155; test/pytest.py:7-19
    run_case(cuda_device, [33, 127], [33, 127], [61, 61], 8, F16, what="odd K fp16")
    run_case(cuda_device, [33, 127], [33, 127], [61, 61], 8, BF16, what="odd K bf16")
    run_case(cuda_device, [11], [13], [5], 1, F16, what="11x13x5")
    run_case(cuda_device, [10, 5, 20, 5, 60], [10, 5, 20, 5, 60], [32] * 5, 8, F16, softmax=True,
             scale=1 / np.sqrt(32), what="graph lengths d=32")
    run_case(cuda_device, [33, 99, 64], [33, 99, 64], [64] * 3, 16, F32, what="script shapes fp32")
    run_case(cuda_device, [33, 99, 64], [33, 99, 64], [64] * 3, 16, F16, softmax=True, what="script shapes fp16 fused")


@pytest.mark.parametrize("dtype", [F16, BF16])
@pytest.mark.parametrize("K", [1, 2, 3, 5, 8, 15, 16, 17, 31, 32, 33, 61, 64])
def test_exhaustive_small_extents(cuda_device, dtype, K):
    # every (M, N) in [1, 40]^2 as one packed batch: ragged tile edges, every alignment class
    g = np.arange(1, 41)
    M, N = [a.ravel() for a in np.meshgrid(g, g, indexing="ij")]
    run_case(cuda_device, M, N, np.full(M.size, K), 2, dtype, seed=K, what=f"grid K={K}")


@pytest.mark.parametrize("K", [32, 64])
def test_exhaustive_small_fused_softmax(cuda_device, K):
    g = np.arange(1, 41)
    M, N = [a.ravel() for a in np.meshgrid(g, g, indexing="ij")]
    # default (K = 64: pipelined pack kernel, K = 32: register-fed small kernel), staged kernel only, register-fed only
    for env in (None, {"BLK_DISABLE_SMALL": "1"}, {"BLK_DISABLE_PIPE": "1"}):
        p = run_case(cuda_device, M, N, np.full(M.size, K), 2, F16, softmax=True, scale=0.3, seed=K, env=env,
                     what=f"fused grid K={K} env={env}")
        assert (p.summary["small_items"] > 0) == (env is None or "BLK_DISABLE_PIPE" in env)
        pipe_off = bool(env) or os.environ.get("BLK_DISABLE_PIPE", "0") not in ("", "0")
        assert (p.summary["packs"] > 0) == (K == 64 and not pipe_off)
        p.check()
    # scores only and bf16 through the same kernels, a negative scale on the fused path
    for env in (None, {"BLK_DISABLE_PIPE": "1"}):
        run_case(cuda_device, M, N, np.full(M.size, K), 2, BF16, scale=0.5, seed=K, env=env, what=f"scores grid K={K}")
        run_case(cuda_device, M, N, np.full(M.size, K), 3, BF16, softmax=True, scale=-0.7, seed=K + 1, env=env,
                 what=f"fused grid negative scale K={K}")


UMMA_SHAPES = dict(
    M=[65, 128, 129, 100, 300, 7, 512, 640, 1, 200],
    N=[70, 256, 257, 65, 513, 300, 512, 1030, 129, 96],
)


@pytest.mark.parametrize("dtype", [F16, BF16])
@pytest.mark.parametrize("K", [64, 128, 256])
@pytest.mark.parametrize("mode", ["scores", "scores32", "softmax"])
def test_tcgen05_path(cuda_device, dtype, K, mode):
    # segments too big for the packed kernel with K a multiple of 64: the TMA + tcgen05 kernel.
    # N <= 256: one accumulator; N <= 512: whole row in tensor memory; N > 512: two sweeps.
    M, N = UMMA_SHAPES["M"], UMMA_SHAPES["N"]
    kw = dict(softmax=mode == "softmax", out_dtype=F32 if mode == "scores32" else None,
              scale=0.125 if mode == "softmax" else 0.5, seed=K)
    p = run_case(cuda_device, M, N, [K] * len(M), 3, dtype, what=f"tcgen05 {mode} K={K}", **kw)
    assert p.summary["umma_items"] == int(np.ceil(np.array(M) / 128).sum())
    p.check()
    # same problem on the staged mma.sync kernel
    p2 = run_case(cuda_device, M, N, [K] * len(M), 3, dtype, env={"BLK_DISABLE_UMMA": "1"},
                  what=f"tile kernel {mode} K={K}", **kw)
    assert p2.summary["umma_items"] == 0 and p2.summary["tile_items"] > 0


def test_tcgen05_mixed_batch_and_negative_scale(cuda_device):
    # small, tcgen05 and staged-kernel segments in one batch: K = 64 and K = 48 go to the tcgen05 kernel (two views per
    # operand), K = 44 -- rows of 88 bytes, which no tensor map takes -- to the staged kernel.
    # The small segments get a launch of their own only when asked to (there are too few of them otherwise).
    M = [20, 300, 64, 130, 33, 500, 90, 70]; N = [20, 300, 64, 70, 40, 600, 200, 50]; K = [64, 64, 64, 64, 48, 64, 44, 64]
    p = run_case(cuda_device, M, N, K, 2, BF16, softmax=True, scale=-0.2, what="mixed batch",
                 env={"BLK_SMALL_MIN_PAIRS": "0"})
    s = p.summary
    assert s["umma_items"] > 0 and s["small_items"] == 2 and s["tile_items"] > 0
    p = run_case(cuda_device, M, N, K, 2, BF16, softmax=True, scale=-0.2, what="mixed batch, small segments riding along")
    assert p.summary["small_items"] == 0 and p.summary["umma_items"] > s["umma_items"]
    run_case(cuda_device, M, N, K, 2, F16, scale=-1.5, what="mixed batch scores")


@pytest.mark.parametrize("out32", [False, True])
@pytest.mark.parametrize("softmax", [False, True])
def test_tcgen05_several_contraction_lengths(cuda_device, out32, softmax):
    # one launch of the tcgen05 kernel for contraction lengths from 16 to 320 (short last k-blocks, k-blocks the tensor
    # map fills with zeros past K) and offsets that are not whole rows of the segment's own (rows, K) view
    rs = np.random.RandomState(5)
    S = 60
    M = rs.randint(1, 300, size=S); N = rs.randint(1, 700, size=S)
    K = rs.choice([16, 24, 32, 48, 64, 72, 96, 128, 200, 320], size=S)
    p = run_case(cuda_device, M, N, K, 3, F16, softmax=softmax, scale=0.07 if softmax else 0.5,
                 out_dtype=torch.float32 if out32 and not softmax else None, what=f"many K out32={out32} softmax={softmax}")
    s = p.summary
    assert s["umma_items"] > 0 and s["launches"] <= 2


def test_tcgen05_more_views_than_slots(cuda_device):
    # more (K, offset modulo K) combinations than tensor-map slots: the lightest go to the staged kernel
    rs = np.random.RandomState(6)
    S = 120
    M = rs.randint(65, 200, size=S); N = rs.randint(65, 200, size=S)
    K = rs.choice(np.arange(16, 400, 8), size=S)
    p = run_case(cuda_device, M, N, K, 2, BF16, what="views overflow")
    assert p.summary["umma_items"] > 0 and p.summary["tile_items"] > 0


@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("dtype", [F16, BF16, F32])
def test_transposes(cuda_device, dtype, ta, tb):
    rs = np.random.RandomState(7)
    M = rs.randint(1, 200, 24); N = rs.randint(1, 300, 24); K = rs.randint(1, 150, 24)
    M[:4] = [8, 16, 64, 128]; N[:4] = [8, 24, 128, 256]; K[:4] = [8, 32, 64, 128]   # fully aligned ones too
    run_case(cuda_device, M, N, K, 3, dtype, ta, tb, seed=11, what=f"transposes {ta},{tb}")


@pytest.mark.parametrize("dtype", [F16, BF16])
def test_fp32_output_and_scale(cuda_device, dtype):
    rs = np.random.RandomState(9)
    M = rs.randint(1, 257, 40); N = rs.randint(1, 257, 40); K = rs.choice([16, 32, 48, 64, 96, 128], 40)
    run_case(cuda_device, M, N, K, 1, dtype, out_dtype=F32, scale=0.125, dist="uniform", what="fp32 out")


@pytest.mark.parametrize("dtype", [F16, BF16, F32])
def test_fused_softmax_long_rows(cuda_device, dtype):
    # N > 128 takes the two-sweep path of the tile kernel; K uniform and ragged
    M = [1, 130, 64, 300, 65, 7]; N = [129, 130, 1000, 257, 2049, 512]; K = [64, 64, 64, 40, 33, 128]
    run_case(cuda_device, M, N, K, 2, dtype, softmax=True, scale=0.125, what="two-sweep softmax")
    # large logits: the running max must do its job
    run_case(cuda_device, M, N, K, 2, dtype, softmax=True, scale=4.0, seed=3, what="two-sweep softmax, hot")


def test_degenerate_segments(cuda_device):
    # empty segments, n = 1 graphs, K = 0 (a product over nothing is zero; its softmax is uniform)
    M = [0, 1, 5, 0, 1, 3]; N = [4, 1, 0, 0, 7, 3]; K = [8, 64, 8, 0, 1, 0]
    for sm in (False, True):
        run_case(cuda_device, M, N, K, 3, F16, softmax=sm, what=f"degenerate softmax={sm}")
        run_case(cuda_device, M, N, K, 3, F32, softmax=sm, what=f"degenerate fp32 softmax={sm}")
    p = GemmPlan([], [], [], 4, F16, device=cuda_device)
    out = p.run(torch.empty((4, 0), dtype=F16, device=cuda_device), torch.empty((4, 0), dtype=F16, device=cuda_device))
    assert out.shape == (4, 0)


def test_offsets_with_gaps_and_odd_strides(cuda_device):
    M = np.array([5, 16, 33]); N = np.array([7, 16, 20]); K = np.array([9, 32, 64])
    a1 = np.array([3, 60, 700, 3000]); a2 = np.array([0, 100, 800, 2500]); ao = np.array([1, 50, 400, 1201])
    for dtype in (F16, F32):
        run_case(cuda_device, M, N, K, 3, dtype, accum=(a1, a2, ao), what="gapped offsets")
        run_case(cuda_device, M, N, K, 3, dtype, softmax=True, accum=(a1, a2, ao), what="gapped offsets fused")
    # packed, but odd strip lengths: head 1 starts on an odd element
    run_case(cuda_device, [3, 5], [5, 3], [7, 9], 5, BF16, what="odd strips")


@pytest.mark.parametrize("name,segments", [("molecular", 512), ("general_gemm", 192), ("long_tail", 20)])
def test_workload_shapes_reduced(cuda_device, name, segments):
    w = workload(name, seed=1, segments=segments)
    run_case(cuda_device, w.M, w.N, w.K, w.H, w.dtype, softmax=w.softmax, scale=w.scale, out_dtype=w.out_dtype,
             dist=w.dist, std=w.std, what=name)


def test_molecular_full_size_against_oracle(cuda_device):
    # the headline configuration at its full size: the oracle still finishes in seconds
    w = workload("molecular")
    run_case(cuda_device, w.M, w.N, w.K, w.H, w.dtype, softmax=True, scale=w.scale, what="molecular full")


def test_full_forward_reduced_p_then_pv(cuda_device):
    # P = softmax(Q K^T / sqrt(d)) fused, then O = P @ V through the same GEMM with transpose2
    rs = np.random.RandomState(5)
    n = np.concatenate([rs.randint(64, 513, 6), np.ones(3, np.int64)])
    H, d = 4, 128
    dl = np.full_like(n, d)
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn((H, int(n.sum()) * d), generator=g).to(BF16) for _ in range(3))
    Pref, Oref = O.block_attention(q, k, v, n, d, 1 / np.sqrt(d), p_dtype=BF16)
    dev = cuda_device
    P = blockAttnScores(q.to(dev), k.to(dev), n, n, dl, scale=1 / np.sqrt(d))
    assert_probs_close(P, Pref, "P")
    out = blockGEMM(P, v.to(dev), None, None, None, n, dl, n, False, True)
    assert out.shape == (H, int(n.sum()) * d)
    # the second product is checked on the P it was given (a one-ulp difference in a bf16 probability
    # is within the contract but moves O), then loosely against the all-oracle O
    assert_scores_close(out, O.block_gemm(P.cpu(), v, n, dl, n, transpose2=True), "O = P V")
    assert float((out.float().cpu() - Oref).abs().max()) < 1e-2 * float(Oref.abs().max())
    # unfused chain gives the same probabilities within tolerance (scores rounded to bf16 in between)
    S = blockGEMM(q.to(dev), k.to(dev), None, None, None, n, n, dl, out_dtype=F32, scale=1 / np.sqrt(d))
    P2 = blockSoftmax(S, n, n)
    assert_probs_close(P2, Pref, "unfused chain")


def test_long_tail_full_size_properties(cuda_device):
    # full size: rows sum to one, values in [0,1], sampled segments against the oracle
    w = workload("long_tail")
    dev = cuda_device
    q, k = w.make_inputs(dev, seed=0)
    P = blockAttnScores(q, k, w.M, w.N, w.K, scale=w.scale)
    torch.cuda.synchronize()
    assert P.shape == (w.H, w.Dout)
    ao = O.offsets_from_lists(w.M, w.N, w.K)[2]
    a1 = O.offsets_from_lists(w.M, w.N, w.K)[0]
    worst = 0.0
    for s in range(w.S):
        blk = P[:, ao[s]:ao[s + 1]].reshape(w.H, w.M[s], w.N[s]).float()
        worst = max(worst, float((blk.sum(-1) - 1).abs().max()))
    assert worst < 2e-2, worst          # bf16 rounding of up to 2048 terms
    assert float(P.float().min()) >= 0 and float(P.float().max()) <= 1.0
    order = np.argsort(w.M)
    for s in [order[0], order[len(order) // 2], order[-1]]:
        n = int(w.M[s])
        qs = q[:, a1[s]:a1[s + 1]].cpu(); ks = k[:, a1[s]:a1[s + 1]].cpu()
        ref = O.block_scores(qs, ks, [n], [n], [64], scale=w.scale)
        assert_probs_close(P[:, ao[s]:ao[s + 1]], ref, f"segment {s} (n={n})")


def test_output_larger_than_2_to_31_elements(cuda_device):
    # one head strip of more than 2^31 output elements (upstream truncates such offsets to int,
    # csrc/cuda/spBlkGEMM.cu:996-998): 64-bit addressing in the tcgen05 kernel, the pack kernel behind it in the
    # same strip and the pipelined softmax; sampled rows against torch on the device
    dev = cuda_device
    n_big, n_small = 46400, 40
    n = np.array([n_big, n_small]); K = np.array([64, 64])
    g = torch.Generator(device=dev).manual_seed(3)
    q = (torch.randn((1, int(n.sum()) * 64), generator=g, device=dev) * 0.5).to(BF16)
    k = (torch.randn((1, int(n.sum()) * 64), generator=g, device=dev) * 0.5).to(BF16)
    P = blockAttnScores(q, k, n, n, K, scale=0.125)
    torch.cuda.synchronize()
    assert P.numel() == n_big * n_big + n_small * n_small and P.numel() > 2 ** 31
    qb = q[0, :n_big * 64].reshape(n_big, 64).float(); kb = k[0, :n_big * 64].reshape(n_big, 64).float()
    for r in (0, 1, 12345, 46271, n_big - 1):
        want = torch.softmax((qb[r] @ kb.T) * 0.125, dim=-1)
        got = P[0, r * n_big:(r + 1) * n_big].float()
        assert float((got - want).abs().max()) <= 2e-3, r
    # the small segment sits behind the 2^31-th element of the strip
    off = n_big * n_big
    qs = q[0, n_big * 64:].reshape(n_small, 64).float(); ks = k[0, n_big * 64:].reshape(n_small, 64).float()
    want = torch.softmax((qs @ ks.T) * 0.125, dim=-1)
    got = P[0, off:].reshape(n_small, n_small).float()
    assert float((got - want).abs().max()) <= 2e-3
    # standalone softmax over the same strip, in place: a probability row of n equal... rows still sum to one
    S = blockSoftmax(P, n, n, out=P)
    torch.cuda.synchronize()
    for r in (0, 30000, n_big - 1):
        assert abs(float(S[0, r * n_big:(r + 1) * n_big].float().sum()) - 1.0) < 2e-2
    assert abs(float(S[0, off:off + n_small].float().sum()) - 1.0) < 2e-2
    del P, S, q, k
    torch.cuda.empty_cache()


def test_python_surface_matches_upstream_contract(cuda_device):
    dev = cuda_device
    M = torch.tensor([33, 99, 64], device=dev); K = torch.tensor([64, 64, 64], device=dev)
    A, B = packed_inputs(M.cpu(), M.cpu(), K.cpu(), 6, F16, 1)
    ref = O.block_gemm(A, B, M.cpu(), M.cpu(), K.cpu())
    res = blockGEMM(A.to(dev), B.to(dev), None, None, None, M, M, K)
    assert res.dtype == F16 and res.shape == (6, int((M * M).sum()))       # dtype = input dtype, 2-D (H, Dout)
    assert_scores_close(res, ref)
    # offsets only: lists are derived (upstream csrc/sparseBlockedAttention.cpp:30-40)
    a1, a2, ao = (torch.from_numpy(a).to(dev) for a in O.offsets_from_lists(M.cpu(), M.cpu(), K.cpu()))
    res2 = blockGEMM(A.to(dev), B.to(dev), a1, a2, ao)
    assert torch.equal(res, res2)
    # any leading shape flattens to H
    res3 = blockGEMM(A.to(dev).reshape(2, 3, -1), B.to(dev).reshape(2, 3, -1), None, None, None, M, M, K)
    assert torch.equal(res, res3)
    # chained softmax, upstream test/pytest.py:36-38
    sm = blockSoftmax(res, M, M)
    assert_probs_close(sm, O.block_softmax(res.cpu(), M.cpu(), M.cpu()))
    # error behaviour: RuntimeError like TORCH_CHECK
    with pytest.raises(RuntimeError):
        blockGEMM(A, B.to(dev), None, None, None, M, M, K)                 # CPU tensor
    with pytest.raises(RuntimeError):
        blockGEMM(A.to(dev).t(), B.to(dev), None, None, None, M, M, K)     # not contiguous
    with pytest.raises(RuntimeError):
        blockGEMM(A.to(dev), B.to(dev))                                    # neither lists nor offsets
    with pytest.raises(RuntimeError):
        blockGEMM(A.to(dev)[:, :-1].contiguous(), B.to(dev), None, None, None, M, M, K)


@pytest.mark.parametrize("groups", [None, 1, 2, 3])
def test_host_entry_point_matches_device_call(cuda_device, groups):
    # host operands in, host result out, head groups pipelined over three streams: same bits as the device call
    dev = cuda_device
    rs = np.random.RandomState(5)
    M = rs.randint(1, 60, size=40); K = np.full(40, 64)
    H = 6
    A, B = packed_inputs(M, M, K, H, F16, 3)
    want = blockAttnScores(A.to(dev), B.to(dev), M, M, K, scale=0.125)
    for pinned in (True, False):
        q, k = (A.pin_memory(), B.pin_memory()) if pinned else (A, B)
        for rep in range(3):  # repeated calls reuse the staging buffers: later groups must wait for earlier copies
            got = blockAttnScoresHost(q, k, M, M, K, scale=0.125, device=dev, head_groups=groups)
            torch.cuda.current_stream(dev).synchronize()
            assert not got.is_cuda and got.shape == want.shape
            assert torch.equal(got, want.cpu())
    with pytest.raises(RuntimeError):
        blockAttnScoresHost(A.to(dev), B, M, M, K, device=dev)              # device operand
    with pytest.raises(RuntimeError):
        blockAttnScoresHost(A, B, M, M, K, device=dev, head_groups=4)       # 4 does not divide 6 heads


@pytest.mark.parametrize("dtype,d,lo,hi", [(F16, 64, 2, 64), (BF16, 64, 2, 300), (F16, 128, 65, 400)])
def test_token_major_entry_matches_head_major(cuda_device, dtype, d, lo, hi):
    # (sum n, H, d) operands read in place through strided tensor maps: same bits as permuting into strips first
    dev = cuda_device
    rs = np.random.RandomState(d + hi)
    n = rs.randint(lo, hi + 1, size=24)
    H = 3
    T = int(n.sum())
    g = torch.Generator().manual_seed(4)
    q = torch.randn((T, H, d), generator=g).to(dtype).to(dev)
    k = torch.randn((T, H, d), generator=g).to(dtype).to(dev)
    got = blockAttnScoresTokenMajor(q, k, n, scale=0.1)
    qs = q.permute(1, 0, 2).reshape(H, T * d).contiguous(); ks = k.permute(1, 0, 2).reshape(H, T * d).contiguous()
    want = blockAttnScores(qs, ks, n, n, np.full_like(n, d), scale=0.1)
    assert got.shape == want.shape and torch.equal(got, want)
    assert_probs_close(got, O.block_scores(qs.cpu(), ks.cpu(), n, n, np.full_like(n, d), scale=0.1), "token-major vs oracle")
    # scores only through the same path
    got_s = blockAttnScoresTokenMajor(q, k, n, scale=0.1, softmax=False)
    assert torch.equal(got_s, blockGEMM(qs, ks, None, None, None, n, n, np.full_like(n, d), scale=0.1))


def test_token_major_entry_refuses_what_it_cannot_take(cuda_device):
    dev = cuda_device
    n = np.array([5, 9, 70])
    # d = 32 and d = 128 with a few small segments: everything rides on the tcgen05 kernel, which reads token-major rows
    for d in (32, 128):
        q = torch.randn((int(n.sum()), 2, d), device=dev).half()
        qs = q.permute(1, 0, 2).reshape(2, int(n.sum()) * d).contiguous()
        assert torch.equal(blockAttnScoresTokenMajor(q, q, n), blockAttnScores(qs, qs, n, n, np.full_like(n, d)))
    q = torch.randn((int(n.sum()), 2, 20), device=dev).half()       # d = 20: rows of 40 bytes, no tensor map takes them
    with pytest.raises(RuntimeError):
        blockAttnScoresTokenMajor(q, q, n)
    q = torch.randn((int(n.sum()), 2, 64), device=dev)              # fp32 operands: no tensor-map kernel
    with pytest.raises(RuntimeError):
        blockAttnScoresTokenMajor(q, q, n)
    q = torch.randn((int(n.sum()), 2, 128), device=dev).half()
    with pytest.raises(RuntimeError):
        blockAttnScoresTokenMajor(q[:, :, :64], q[:, :, :64], n)    # not contiguous


def test_unaligned_pointer_is_handled(cuda_device):
    dev = cuda_device
    M = [5, 9]; N = [6, 4]; K = [8, 8]
    A, B = packed_inputs(M, N, K, 1, F16, 2)
    big = torch.zeros(A.numel() + 1, dtype=F16, device=dev)
    big[1:] = A.to(dev).reshape(-1)
    Au = big[1:].reshape(1, -1)            # data pointer off by two bytes
    assert Au.data_ptr() % 16 != 0
    plan = GemmPlan(M, N, K, 1, F16, device=dev)
    out = plan.run(Au, B.to(dev))
    assert_scores_close(out, O.block_gemm(A, B, M, N, K))
    # the raw ABI refuses it rather than faulting
    import ctypes as C
    rc = L.lib.blk_gemm_run(plan._h, C.c_void_p(Au.data_ptr()), C.c_void_p(B.to(dev).data_ptr()),
                            C.c_void_p(out.data_ptr()), C.c_float(1.0), None)
    assert rc == L.BLK_ERR_UNALIGNED
