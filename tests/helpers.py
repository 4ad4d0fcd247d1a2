"""Shared helpers of the test-suite: seeded packed inputs, the oracle call and
the tolerances of the parity contract."""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle"))

import blk_oracle as O  # noqa: E402

PROB_ATOL = 2e-3     # max-abs error on softmax probabilities
SCORE_RTOL = 1e-2    # relative error on raw 16-bit scores


def packed_inputs(M, N, K, H, dtype, seed=0, dist="normal", std=1.0, a1=None, a2=None):
    """CPU tensors (H, D1), (H, D2) already rounded to ``dtype``."""
    M = np.asarray(M, np.int64); N = np.asarray(N, np.int64); K = np.asarray(K, np.int64)
    D1 = int((M * K).sum()) if a1 is None else int(a1[-1])
    D2 = int((N * K).sum()) if a2 is None else int(a2[-1])
    g = torch.Generator().manual_seed(seed)
    if dist == "normal":
        A = torch.randn((H, D1), generator=g) * std
        B = torch.randn((H, D2), generator=g) * std
    else:
        A = torch.rand((H, D1), generator=g) * 2 - 1
        B = torch.rand((H, D2), generator=g) * 2 - 1
    return A.to(dtype), B.to(dtype)


def assert_scores_close(got, ref, what=""):
    got = got.detach().float().cpu(); ref = ref.detach().float().cpu()
    assert got.shape == ref.shape, (got.shape, ref.shape)
    if ref.numel() == 0:
        return
    assert torch.isfinite(got).all(), f"{what}: non-finite output"
    rms = float(ref.pow(2).mean().sqrt())
    err = (got - ref).abs()
    bound = SCORE_RTOL * ref.abs() + 1e-3 * max(rms, 1e-30)
    bad = err > bound
    assert not bad.any(), (f"{what}: {int(bad.sum())} of {ref.numel()} scores off; worst abs err "
                           f"{float(err.max()):.3e} (rms {rms:.3e})")


def assert_probs_close(got, ref, what=""):
    got = got.detach().float().cpu(); ref = ref.detach().float().cpu()
    assert got.shape == ref.shape, (got.shape, ref.shape)
    if ref.numel() == 0:
        return
    assert torch.isfinite(got).all(), f"{what}: non-finite output"
    err = float((got - ref).abs().max())
    assert err <= PROB_ATOL, f"{what}: max-abs error {err:.3e} > {PROB_ATOL}"
