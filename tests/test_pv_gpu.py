"""GPU: the tcgen05 kernel for a second operand stored (K, D) -- the product of a packed probability block with the
values, blockGEMM(P, V, ..., transpose2=True) of upstream blockedAttention/apply.py:6-25 -- against the oracle and
against the staged mma.sync kernel on the same inputs."""
import os

import numpy as np
import pytest
import torch

from helpers import O, assert_scores_close
from blockedattention_b200 import _lib as L
from blockedattention_b200.plan import GemmPlan

pytestmark = pytest.mark.gpu
F16, BF16 = torch.float16, torch.bfloat16


def run_pv(dev, M, K, D, H, dtype, scale=1.0, seed=0, env=None, probs=True):
    M = np.asarray(M, np.int64); K = np.asarray(K, np.int64); N = np.full_like(M, D)
    g = torch.Generator().manual_seed(seed)
    D1, D2 = int((M * K).sum()), int((K * N).sum())
    A = torch.rand((H, D1), generator=g) if probs else torch.randn((H, D1), generator=g)
    B = torch.randn((H, D2), generator=g)
    A, B = A.to(dtype), B.to(dtype)
    ref = O.block_gemm(A, B, M, N, K, transpose2=True, scale=scale)
    old = {}
    for k, v in (env or {}).items():
        old[k] = os.environ.get(k); os.environ[k] = v
    try:
        plan = GemmPlan(M, N, K, H, dtype, dtype, False, True, False, device=dev)
    finally:
        for k, v in old.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v
    out = torch.full((H, plan.Dout), float("nan"), dtype=dtype, device=dev)
    plan.run(A.to(dev), B.to(dev), out=out, scale=scale)
    plan.check()
    return plan, out, ref


@pytest.mark.parametrize("dtype", [F16, BF16])
@pytest.mark.parametrize("D", [64, 128])
def test_pv_every_alignment_and_tail(cuda_device, dtype, D):
    # row lengths around the tile (128), the MMA step (16) and the 16-byte vector (8), odd ones included, so that the
    # rows of the first operand start at every 2-byte offset; row counts around the 128-row block
    M = [1, 7, 33, 127, 128, 129, 200, 64, 300, 5, 16, 90]
    K = [1, 7, 33, 127, 128, 129, 200, 257, 300, 513, 16, 1031]
    plan, out, ref = run_pv(cuda_device, M, K, D, 3, dtype, seed=D)
    assert plan.summary["umma_items"] == int(np.ceil(np.array(M) / 128).sum()) and plan.summary["tile_items"] == 0
    assert_scores_close(out, ref, f"tcgen05 P V D={D}")
    # the staged mma.sync kernel on the same problem
    plan2, out2, _ = run_pv(cuda_device, M, K, D, 3, dtype, seed=D, env={"BLK_DISABLE_UMMA": "1"})
    assert plan2.summary["umma_items"] == 0 and plan2.summary["tile_items"] > 0
    assert_scores_close(out2, ref, "staged kernel P V")


def test_pv_scale_and_values_of_either_sign(cuda_device):
    plan, out, ref = run_pv(cuda_device, [150, 40, 260], [70, 333, 129], 128, 2, BF16, scale=-0.37, probs=False, seed=5)
    assert plan.summary["umma_items"] > 0
    assert_scores_close(out, ref, "scaled P V")


def test_pv_neighbour_values_do_not_leak(cuda_device):
    # infinite and NaN values in the segment behind: the value rows a tile reads past the end of a segment must not
    # reach the result (they are cleared in shared memory, and the first operand's columns past the row end are zeros)
    dev = cuda_device
    M = np.array([130, 20]); K = np.array([77, 50]); D = 64
    N = np.full_like(M, D)
    g = torch.Generator().manual_seed(2)
    A = torch.rand((2, int((M * K).sum())), generator=g).to(F16)
    B = torch.randn((2, int((K * N).sum())), generator=g).to(F16)
    B[:, 77 * 64:] = float("inf")           # all of segment 1's values
    B[:, 77 * 64 + 5] = float("nan")
    plan = GemmPlan(M, N, K, 2, F16, F16, False, True, False, device=dev)
    assert plan.summary["umma_items"] == 3
    out = plan.run(A.to(dev), B.to(dev))
    plan.check()
    ref = O.block_gemm(A[:, :130 * 77], B[:, :77 * 64], M[:1], N[:1], K[:1], transpose2=True)
    assert_scores_close(out[:, :130 * 64], ref, "segment in front of infinite values")


def test_pv_mixed_batch_sends_the_rest_to_the_staged_kernel(cuda_device):
    # second operands of 128 columns go to the tcgen05 kernel, the segment with 96 columns stays on the staged
    # kernel, and so does the empty contraction, which writes zeros
    dev = cuda_device
    M = np.array([100, 50, 3, 260, 9]); N = np.array([128, 96, 128, 128, 128]); K = np.array([300, 40, 0, 129, 64])
    g = torch.Generator().manual_seed(9)
    A = torch.rand((2, int((M * K).sum())), generator=g).to(BF16)
    B = torch.randn((2, int((K * N).sum())), generator=g).to(BF16)
    plan = GemmPlan(M, N, K, 2, BF16, BF16, False, True, False, device=dev)
    s = plan.summary
    assert s["umma_items"] == 1 + 3 + 1 and s["tile_items"] > 0
    out = torch.full((2, plan.Dout), float("nan"), dtype=BF16, device=dev)
    plan.run(A.to(dev), B.to(dev), out=out)
    plan.check()
    assert_scores_close(out, O.block_gemm(A, B, M, N, K, transpose2=True), "mixed batch")
