"""GPU: a bounded device-side wait that runs out.

Every wait of the pipelined kernels (on an mbarrier, on a rendezvous counter) has an iteration limit; when it is
hit the kernel records a status code in the plan's status word, every role leaves its loop, tensor memory is
released and the kernel returns -- it never traps and never spins for ever.  The test makes a wait run out the
harmless way: under ``BLK_TEST_STALL_PRODUCER=1`` the producer role of the tcgen05 GEMM kernel issues no copies at
all (so nothing is in flight when the kernel ends) and the limit is a few thousand polls; the MMA role's wait for
operands then gives up, ``blk_plan_check`` reports ``BLK_ERR_TIMEOUT``, and the next ordinary run of the same
plan is correct.
"""
import numpy as np
import pytest
import torch

from helpers import O, assert_probs_close, packed_inputs
from blockedattention_b200 import _lib as L
from blockedattention_b200.plan import GemmPlan

pytestmark = pytest.mark.gpu


def test_wait_runs_out_status_is_reported_and_the_plan_recovers(cuda_device, monkeypatch):
    dev = cuda_device
    M = [300, 200, 129]; N = [300, 600, 70]; K = [64, 64, 64]
    H = 2
    A, B = packed_inputs(M, N, K, H, torch.bfloat16, 7, std=0.5)
    plan = GemmPlan(M, N, K, H, torch.bfloat16, softmax=True, device=dev)
    assert plan.summary["umma_items"] == 3 + 2 + 2 and plan.summary["tile_items"] == 0
    a, b = A.to(dev), B.to(dev)
    out = torch.full((H, plan.Dout), float("nan"), dtype=torch.bfloat16, device=dev)

    monkeypatch.setenv("BLK_TEST_STALL_PRODUCER", "1")
    plan.run(a, b, out=out, scale=0.125)
    with pytest.raises(L.BlkError) as e:
        plan.check()
    assert e.value.code == L.BLK_ERR_TIMEOUT
    assert bool(torch.isnan(out.float()).all()), "a kernel that gave up before its first product stores nothing"
    plan.check()                                        # the status word was cleared by the failed check

    monkeypatch.delenv("BLK_TEST_STALL_PRODUCER")
    plan.run(a, b, out=out, scale=0.125)
    plan.check()
    assert_probs_close(out, O.block_scores(A, B, M, N, K, scale=0.125), "run after a timed-out run")


def test_blk_check_env_raises_from_the_operator_call(cuda_device, monkeypatch):
    # BLK_CHECK=1 makes every run read the status word, so a timeout surfaces at the call that caused it
    dev = cuda_device
    M = [256]; N = [256]; K = [64]
    A, B = packed_inputs(M, N, K, 1, torch.float16, 1)
    plan = GemmPlan(M, N, K, 1, torch.float16, device=dev)
    monkeypatch.setenv("BLK_CHECK", "1")
    monkeypatch.setenv("BLK_TEST_STALL_PRODUCER", "1")
    with pytest.raises(L.BlkError) as e:
        plan.run(A.to(dev), B.to(dev))
    assert e.value.code == L.BLK_ERR_TIMEOUT
    monkeypatch.delenv("BLK_TEST_STALL_PRODUCER")
    out = plan.run(A.to(dev), B.to(dev))
    ref = O.block_gemm(A, B, M, N, K)
    assert float((out.float().cpu() - ref).abs().max()) <= 1e-2 * float(ref.abs().max())
