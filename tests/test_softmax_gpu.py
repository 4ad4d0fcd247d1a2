"""GPU parity of the standalone varlen row softmax (blk_softmax_run) with the CPU oracle."""
import numpy as np
import pytest
import torch

from helpers import O, assert_probs_close
from blockedattention_b200 import blockSoftmax
from blockedattention_b200.plan import SoftmaxPlan

pytestmark = pytest.mark.gpu
F16, BF16, F32 = torch.float16, torch.bfloat16, torch.float32


def run_softmax(dev, rows, cols, H, dtype, scale=1.0, seed=0, accum=None, inplace=False, std=1.0, what=""):
    rows = np.asarray(rows, np.int64); cols = np.asarray(cols, np.int64)
    D = int((rows * cols).sum()) if accum is None else int(accum[-1])
    g = torch.Generator().manual_seed(seed)
    X = (torch.randn((H, D), generator=g) * std).to(dtype)
    ref = O.block_softmax(X, rows, cols, accum, scale)
    plan = SoftmaxPlan(rows, cols, H, dtype, accum=accum, device=dev)
    x = X.to(dev)
    if inplace:
        out = plan.run(x, out=x, scale=scale)
    else:
        out = torch.full_like(x, float("nan"))
        plan.run(x, out=out, scale=scale)
    torch.cuda.synchronize()
    got = out.float().cpu()
    if accum is not None:
        keep = torch.zeros(D, dtype=torch.bool)
        for s in range(len(rows)):
            keep[accum[s]:accum[s] + rows[s] * cols[s]] = True
        if not inplace:
            assert torch.isnan(got[:, ~keep]).all(), f"{what}: wrote outside the blocks"
        got, ref = got[:, keep], ref[:, keep]
    assert_probs_close(got, ref, what)


COLS = [1, 2, 3, 4, 5, 7, 8, 9, 16, 25, 31, 32, 33, 63, 64, 65, 127, 128, 129, 255, 511, 512, 513, 1023, 1025, 2047]


@pytest.mark.parametrize("dtype", [F16, BF16, F32])
def test_every_column_class(cuda_device, dtype):
    rows = [3 + (i * 7) % 40 for i in range(len(COLS))]
    for inplace in (False, True):
        run_softmax(cuda_device, rows, COLS, 3, dtype, inplace=inplace, what=f"cols sweep inplace={inplace}")
    run_softmax(cuda_device, rows, COLS, 2, dtype, scale=3.0, std=4.0, seed=1, what="hot logits")


def test_upstream_shapes(cuda_device):
    # csrc/sparseBlockedAttention.cpp:265-294: half, rows 127, cols 2047, 3 blocks, 7 heads
    run_softmax(cuda_device, [127] * 3, [2047] * 3, 7, F16, what="127x2047 half")
    # test/pytest.py:54-62: fp32 blocks (33,64), (99,64), (64,64)
    run_softmax(cuda_device, [33, 99, 64], [64, 64, 64], 16, F32, what="script softmax")


@pytest.mark.parametrize("dtype", [F16, F32])
def test_rows_longer_than_the_window_and_upstream_limit(cuda_device, dtype):
    # upstream refuses cols >= 8192 (csrc/cuda/spBlkSoftmax.cu:392); here there is no limit
    run_softmax(cuda_device, [2, 3, 1, 2], [8191, 8193, 40000, 4097], 2, dtype, what="long rows")
    run_softmax(cuda_device, [2, 1], [8193, 16385], 1, dtype, inplace=True, what="long rows in place")


def test_degenerate_and_gapped(cuda_device):
    run_softmax(cuda_device, [0, 4, 3, 0], [5, 0, 1, 0], 2, F16, what="empty blocks")
    acc = np.array([3, 40, 41, 2000])
    run_softmax(cuda_device, [5, 1, 30], [7, 1, 64], 3, BF16, accum=acc, what="gapped")
    run_softmax(cuda_device, [5, 1, 30], [7, 1, 64], 3, F32, accum=acc, inplace=True, what="gapped in place")
    plan = SoftmaxPlan([], [], 4, F16, device=cuda_device)
    assert plan.run(torch.empty((4, 0), dtype=F16, device=cuda_device)).shape == (4, 0)


def test_odd_strips_many_heads(cuda_device):
    # odd D: every other head starts on an odd element; edge vectors of neighbouring chunks interleave
    run_softmax(cuda_device, [37, 11, 300], [25, 3, 33], 9, F16, what="odd strips")
    run_softmax(cuda_device, [37, 11, 300], [25, 3, 33], 9, BF16, inplace=True, what="odd strips in place")


def test_python_surface(cuda_device):
    dev = cuda_device
    rows = torch.tensor([33, 99, 64], device=dev); cols = torch.tensor([64, 64, 64], device=dev)
    g = torch.Generator().manual_seed(0)
    X = torch.randn((8, int((rows * cols).sum())), generator=g)
    out = blockSoftmax(X.to(dev), rows, cols)                          # upstream call shape, test/pytest.py:54
    assert out.shape == X.shape and out.dtype == F32
    assert_probs_close(out, O.block_softmax(X, rows.cpu(), cols.cpu()))
    acc = torch.from_numpy(O.softmax_offsets(rows.cpu(), cols.cpu())).to(dev)
    out2 = blockSoftmax(X.to(dev), rows, cols, acc)                    # srcAccum reaches the offsets parameter
    assert torch.equal(out, out2)
    with pytest.raises(RuntimeError):
        blockSoftmax(X, rows, cols)
    with pytest.raises(RuntimeError):
        blockSoftmax(X.to(dev), None, cols)
