"""GPU: the compiled extension module ``blockAttention`` (upstream's operator names and argument order,
upstream csrc/sparseBlockedAttention.cpp:118-138) against the oracle, and bit for bit against the ctypes path
of ``blockedattention_b200`` -- both sit on the same library, so any difference is a boundary defect."""
import numpy as np
import pytest
import torch

import blockAttention
from helpers import O, assert_probs_close, assert_scores_close, packed_inputs
from blockedattention_b200 import blockGEMM, blockSoftmax

pytestmark = pytest.mark.gpu


def lists(dev, *ls):
    return [torch.as_tensor(np.asarray(l, np.int64), device=dev) for l in ls]


def test_extension_is_the_compiled_module():
    assert blockAttention.COMPILED, "blockAttention fell back to the Python alias: build blockAttention/_C"
    assert type(blockAttention.sparseBlockedGEMM).__name__ == "builtin_function_or_method"


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_gemm_then_softmax_like_the_upstream_script(cuda_device, dtype):
    # upstream test/pytest.py:35-38: res = blockGEMM(A, B, None, None, None, M, N, K); res = blockSoftmax(res, M, N)
    dev = cuda_device
    M = [33, 99, 64, 1, 130]; N = [33, 99, 64, 7, 300]; K = [64, 64, 64, 61, 64]
    A, B = packed_inputs(M, N, K, 5, dtype, 1)
    tM, tN, tK = lists(dev, M, N, K)
    got = blockAttention.sparseBlockedGEMM(A.to(dev), B.to(dev), None, None, None, tM, tN, tK, False, False)
    assert got.dtype == dtype and got.shape == (5, int((np.array(M) * np.array(N)).sum()))
    assert_scores_close(got, O.block_gemm(A, B, M, N, K), "extension GEMM vs oracle")
    assert torch.equal(got, blockGEMM(A.to(dev), B.to(dev), None, None, None, tM, tN, tK))
    sm = blockAttention.sparseBlockedSoftmax(got, tM, tN)                     # (src, rowList, colList, srcAccum)
    assert_probs_close(sm, O.block_softmax(got.cpu(), M, N), "extension softmax vs oracle")
    assert torch.equal(sm, blockSoftmax(got, tM, tN))
    # keyword form and explicit offsets, lists on the host
    a1, a2, ao = (torch.from_numpy(a) for a in O.offsets_from_lists(M, N, K))
    got2 = blockAttention.sparseBlockedGEMM(mat1=A.to(dev), mat2=B.to(dev), mat1Accum=a1, mat2Accum=a2, outAccum=ao)
    assert torch.equal(got, got2), "lists derived from the offsets give the same result"
    sm2 = blockAttention.sparseBlockedSoftmax(got, rowList=tM, colList=tN, srcAccum=ao.to(dev))
    assert torch.equal(sm, sm2)


@pytest.mark.parametrize("ta,tb", [(False, True), (True, False), (True, True)])
def test_transposed_operands_and_leading_shape(cuda_device, ta, tb):
    dev = cuda_device
    M = [64, 32, 127]; N = [32, 64, 96]; K = [64, 128, 33]
    A, B = packed_inputs(M, N, K, 6, torch.float16, 5)
    tM, tN, tK = lists(dev, M, N, K)
    got = blockAttention.sparseBlockedGEMM(A.to(dev).reshape(2, 3, -1), B.to(dev).reshape(2, 3, -1), None, None, None,
                                           tM, tN, tK, ta, tb)
    assert got.dim() == 2 and got.shape[0] == 6
    assert_scores_close(got, O.block_gemm(A, B, M, N, K, transpose1=ta, transpose2=tb), f"transposes {ta},{tb}")


def test_autograd_through_the_extension(cuda_device):
    # upstream test/pytest.py:43-46: res.mean().backward() through both operators
    dev = cuda_device
    M = [11, 40, 5]; N = [13, 24, 70]; K = [5, 32, 64]
    A, B = packed_inputs(M, N, K, 2, torch.float32, 3)
    tM, tN, tK = lists(dev, M, N, K)
    a = A.to(dev).requires_grad_(); b = B.to(dev).requires_grad_()
    res = blockAttention.sparseBlockedSoftmax(blockAttention.sparseBlockedGEMM(a, b, None, None, None, tM, tN, tK), tM, tN)
    w = torch.randn(res.shape, generator=torch.Generator().manual_seed(0)).to(dev)
    (res * w).sum().backward()
    # reference gradients: the same chain per segment with torch autograd on the CPU in float64
    a64 = A.double().requires_grad_(); b64 = B.double().requires_grad_()
    outs, oa, ob = [], 0, 0
    for m, n, k in zip(M, N, K):
        x = a64[:, oa:oa + m * k].reshape(2, m, k); y = b64[:, ob:ob + n * k].reshape(2, n, k)
        outs.append((x @ y.transpose(1, 2)).softmax(-1).reshape(2, m * n))
        oa += m * k; ob += n * k
    (torch.cat(outs, 1) * w.cpu().double()).sum().backward()
    assert float((a.grad.cpu() - a64.grad.float()).abs().max()) <= 1e-4
    assert float((b.grad.cpu() - b64.grad.float()).abs().max()) <= 1e-4
    assert a.grad.shape == a.shape and b.grad.shape == b.shape


def test_error_behaviour_matches_torch_check(cuda_device):
    dev = cuda_device
    M, K = lists(dev, [4, 5], [8, 8])
    A = torch.zeros((1, 72), dtype=torch.float16)
    with pytest.raises(RuntimeError, match="must be CUDA Tensor"):
        blockAttention.sparseBlockedGEMM(A, A.to(dev), None, None, None, M, M, K)
    with pytest.raises(RuntimeError, match="contiguous"):
        blockAttention.sparseBlockedGEMM(A.to(dev).expand(2, 72).t(), A.to(dev), None, None, None, M, M, K)
    with pytest.raises(RuntimeError):
        blockAttention.sparseBlockedGEMM(A.to(dev), A.to(dev))                        # neither lists nor offsets
    with pytest.raises(RuntimeError):
        blockAttention.sparseBlockedSoftmax(A.to(dev), M, None)                       # colList missing


def test_fresh_list_tensors_with_other_values_get_their_own_plan(cuda_device):
    # two batches whose list tensors have equal length and equal packed totals, allocated one after the other
    # (the second may reuse the first one's address): each must be computed with its own lists
    dev = cuda_device
    for mod_gemm in (blockAttention.sparseBlockedGEMM, blockGEMM):
        for M in ([10, 50], [50, 10], [30, 30], [20, 40]):
            K = [16, 16]
            A, B = packed_inputs(M, M, K, 2, torch.float16, sum(M) + M[0])
            tM, tK = lists(dev, M, K)
            got = mod_gemm(A.to(dev), B.to(dev), None, None, None, tM, tM, tK)
            assert_scores_close(got, O.block_gemm(A, B, M, M, K), f"lists {M}")
            del tM, tK
