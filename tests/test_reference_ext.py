"""GPU: the upstream project's own CUDA kernels (built unmodified by
oracle/build_ref.py into oracle/_ref/) as a second checker -- they pin the CPU
oracle, and the new kernels are compared with them directly.

Inputs stay inside what the upstream kernels handle: even K and even packed
offsets for 16-bit types (their vector loads assume it,
csrc/cuda/spBlkGEMM.cu:293-304), N odd or a multiple of 8 (an even N sends full
sub-tiles through wmma::store_matrix_sync with ldm = N, csrc/cuda/spBlkGEMM.cu:599,
and that call documents ldm as a multiple of 8), cols < 8192
(csrc/cuda/spBlkSoftmax.cu:392)."""
import glob
import os
import sys

import numpy as np
import pytest
import torch

from helpers import O, ROOT, assert_probs_close, assert_scores_close, packed_inputs
from blockedattention_b200 import blockGEMM, blockSoftmax
from blockedattention_b200.plan import SoftmaxPlan

pytestmark = pytest.mark.gpu
REF_DIR = os.path.join(ROOT, "oracle", "_ref")


@pytest.fixture(scope="module")
def ref():
    if not glob.glob(os.path.join(REF_DIR, "blk_ref_ext*.so")):
        pytest.skip("oracle/_ref is not built (python oracle/build_ref.py needs the upstream checkout)")
    sys.path.insert(0, REF_DIR)
    import blk_ref_ext
    return blk_ref_ext


def padded(t, dev):
    """The tensor as a contiguous view at the start of a larger zeroed allocation: the upstream
    loaders read whole tiles before masking (csrc/cuda/spBlkGEMM.cu:294-308), i.e. up to a tile
    past the end of the last segment; the padding keeps those reads inside memory this test owns."""
    buf = torch.zeros(t.numel() + (1 << 19), dtype=t.dtype, device=dev)
    buf[:t.numel()] = t.reshape(-1).to(dev)
    return buf[:t.numel()].view(t.shape)


def dev_lists(dev, *ls):
    return [torch.as_tensor(np.asarray(l, np.int64), device=dev) for l in ls]


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_gemm_three_way(cuda_device, ref, dtype):
    dev = cuda_device
    rs = np.random.RandomState(2)
    M = rs.randint(1, 50, 12) * 8; N = rs.randint(1, 50, 12) * 8; K = rs.choice([16, 32, 64, 128, 30, 62], 12)
    N[::3] += 1                                       # odd N: the upstream scalar store path
    M[1::3] += 3
    A, B = packed_inputs(M, N, K, 4, dtype, 3)
    a1, a2, ao = O.offsets_from_lists(M, N, K)
    oracle = O.block_gemm(A, B, M, N, K)
    tM, tN, tK, t1, t2, to = dev_lists(dev, M, N, K, a1, a2, ao)
    theirs = ref.gemm_launch(padded(A, dev), padded(B, dev), t1, t2, to, tM, tN, tK, False, False)
    torch.cuda.synchronize()
    ours = blockGEMM(A.to(dev), B.to(dev), t1, t2, to, tM, tN, tK)
    assert theirs.shape == ours.shape and theirs.dtype == ours.dtype
    assert_scores_close(theirs, oracle, "upstream kernels vs oracle")      # pins the oracle
    assert_scores_close(ours, oracle, "new kernels vs oracle")
    assert_scores_close(ours, theirs.float(), "new kernels vs upstream kernels")


@pytest.mark.parametrize("ta,tb", [(False, True), (True, False)])
def test_gemm_transposed_three_way(cuda_device, ref, ta, tb):
    dev = cuda_device
    M = np.array([64, 32, 128]); N = np.array([32, 64, 96]); K = np.array([64, 128, 32])
    A, B = packed_inputs(M, N, K, 2, torch.float16, 5)
    a1, a2, ao = O.offsets_from_lists(M, N, K)
    oracle = O.block_gemm(A, B, M, N, K, transpose1=ta, transpose2=tb)
    tM, tN, tK, t1, t2, to = dev_lists(dev, M, N, K, a1, a2, ao)
    theirs = ref.gemm_launch(padded(A, dev), padded(B, dev), t1, t2, to, tM, tN, tK, ta, tb)
    ours = blockGEMM(A.to(dev), B.to(dev), t1, t2, to, tM, tN, tK, ta, tb)
    assert_scores_close(theirs, oracle, "upstream kernels vs oracle")
    assert_scores_close(ours, theirs.float(), "new kernels vs upstream kernels")


@pytest.mark.parametrize("dtype,rows,cols,H", [
    (torch.float16, [127] * 3, [2047] * 3, 7),        # csrc/sparseBlockedAttention.cpp:265-294
    (torch.float32, [33, 99, 64], [64, 64, 64], 16),  # test/pytest.py:54-62
    (torch.bfloat16, [40, 7, 200], [24, 128, 1000], 3),
])
def test_softmax_three_way(cuda_device, ref, dtype, rows, cols, H):
    dev = cuda_device
    rows = np.asarray(rows, np.int64); cols = np.asarray(cols, np.int64)
    g = torch.Generator().manual_seed(1)
    X = torch.randn((H, int((rows * cols).sum())), generator=g).to(dtype)
    acc = O.softmax_offsets(rows, cols)
    oracle = O.block_softmax(X, rows, cols)
    tr, tc, ta = dev_lists(dev, rows, cols, acc)
    theirs = ref.softmax_launch(X.to(dev), ta, tr, tc)
    torch.cuda.synchronize()
    ours = blockSoftmax(X.to(dev), tr, tc, ta)
    assert_probs_close(theirs, oracle, "upstream kernels vs oracle")       # pins the oracle
    assert_probs_close(ours, oracle, "new kernels vs oracle")
    assert_probs_close(ours, theirs.float(), "new kernels vs upstream kernels")


@pytest.mark.parametrize("dtype,rows,cols,H", [
    (torch.float32, [33, 99, 64], [64, 64, 64], 16),
    (torch.float16, [40, 7, 200, 3], [24, 128, 1000, 2], 3),   # at most 1024 columns: upstream's warp kernel
])
def test_softmax_backward_three_way(cuda_device, ref, dtype, rows, cols, H):
    if not hasattr(ref, "softmax_backward_launch"):
        pytest.skip("oracle/_ref was built before the backward launcher was bound: rerun python oracle/build_ref.py")
    dev = cuda_device
    rows = np.asarray(rows, np.int64); cols = np.asarray(cols, np.int64)
    g = torch.Generator().manual_seed(2)
    X = torch.randn((H, int((rows * cols).sum())), generator=g)
    P = O.block_softmax(X, rows, cols).to(dtype)
    G = torch.randn(P.shape, generator=g).to(dtype)
    acc = O.softmax_offsets(rows, cols)
    oracle = O.block_softmax_backward(P, G, rows, cols)
    tr, tc, ta = dev_lists(dev, rows, cols, acc)
    theirs = ref.softmax_backward_launch(P.to(dev), G.to(dev), ta, tr, tc)
    torch.cuda.synchronize()
    ours = SoftmaxPlan(rows, cols, H, dtype, device=dev).run_backward(P.to(dev), G.to(dev))
    tol = 1e-5 if dtype == torch.float32 else 4e-3   # upstream multiplies the two 16-bit rows in 16 bits
    for name, got in (("upstream kernel vs oracle", theirs), ("new kernel vs oracle", ours)):
        err = float((got.float().cpu() - oracle).abs().max())
        assert err <= tol, f"{name}: {err}"
    assert float((ours.float() - theirs.float()).abs().max()) <= tol


def test_molecular_chain_three_way(cuda_device, ref):
    # GEMM then softmax as upstream chains them (test/pytest.py:36-38), on a reduced molecular batch
    from blockedattention_b200.synth import workload
    dev = cuda_device
    w = workload("molecular", seed=2, segments=300)
    # N odd or a multiple of 8 (see the module docstring), and every multiple-of-8 graph before the
    # first odd one: upstream's wmma store of an even-N segment also assumes an even output offset
    # (csrc/cuda/spBlkGEMM.cu:599), which a preceding odd n*n block would break
    n = np.where(w.M % 8 == 0, w.M, w.M | 1)
    n = np.concatenate([n[n % 8 == 0], n[n % 8 != 0]])
    w.M, w.N = n, n.copy()
    # one head: with H > 1 upstream adds head * Dout to that offset (csrc/cuda/spBlkGEMM.cu:455), and
    # Dout = sum n*n is odd for a typical mixed batch -- the wmma store then faults on every other head
    w.H = 1
    A, B = packed_inputs(w.M, w.N, w.K, w.H, w.dtype, 0)
    A = (A.float() * w.scale).to(w.dtype)             # upstream has no scale argument: fold it into q
    a1, a2, ao = O.offsets_from_lists(w.M, w.N, w.K)
    tM, tN, tK, t1, t2, to = dev_lists(dev, w.M, w.N, w.K, a1, a2, ao)
    s_ref = ref.gemm_launch(padded(A, dev), padded(B, dev), t1, t2, to, tM, tN, tK, False, False)
    p_ref = ref.softmax_launch(s_ref, to, tM, tN)
    torch.cuda.synchronize()
    p_ours = blockGEMM(A.to(dev), B.to(dev), None, None, None, tM, tN, tK, softmax=True)
    oracle = O.block_scores(A, B, w.M, w.N, w.K)
    assert_probs_close(p_ref, oracle, "upstream chain vs oracle")
    assert_probs_close(p_ours, oracle, "fused kernel vs oracle")
    assert_probs_close(p_ours, p_ref.float(), "fused kernel vs upstream chain")
