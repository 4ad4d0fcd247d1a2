"""GPU: the tcgen05 attention kernel (segments of any length, head dimension 64 or 128) against the oracle
(softmax(scale Q K^T) V per segment in float32) and against the two-operator composition it replaces."""
import numpy as np
import pytest
import torch

from helpers import O, packed_inputs
from blockedattention_b200 import blockAttention, blockAttentionTokenMajor, blockAttnScores, blockGEMM
from blockedattention_b200.plan import AttentionPlan

pytestmark = pytest.mark.gpu
F16, BF16 = torch.float16, torch.bfloat16
TOL = {F16: 2e-3, BF16: 1.6e-2}


def oracle_attention(q, k, v, M, N, d, scale):
    dl = np.full_like(M, d)
    P = O.block_scores(q, k, M, N, dl, scale=scale)
    return O.block_gemm(P, v, M, dl, N, transpose2=True)


def close(got, want, dtype, what):
    got = got.detach().float().cpu(); want = want.float()
    assert not bool(torch.isnan(got).any()), f"{what}: NaN in the result"
    scale = max(1.0, float(want.abs().max()))
    err = float((got - want).abs().max())
    assert err <= TOL[dtype] * scale, f"{what}: max abs err {err} (scale {scale})"


def inputs(M, N, d, H, dtype, seed, amp=1.0):
    q, k = packed_inputs(M, N, np.full_like(M, d), H, dtype, seed)
    v = packed_inputs(N, N, np.full_like(M, d), H, dtype, seed + 1)[0]
    if amp != 1.0:
        q = (q.float() * amp).to(dtype)
    return q, k, v


@pytest.mark.parametrize("dtype", [F16, BF16])
@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("scale", [0.1, -0.07])
def test_attention_every_edge_of_the_tiling(cuda_device, dtype, d, scale):
    # query counts around the 128-row block, key counts around the 128-row tile and the 16-row MMA step, a segment
    # without queries, single rows; M != N throughout
    dev = cuda_device
    M = np.array([1, 127, 128, 129, 5, 0, 300, 64, 257, 16, 31, 200])
    N = np.array([1, 128, 127, 129, 300, 7, 5, 15, 17, 256, 385, 113])
    H = 3
    q, k, v = inputs(M, N, d, H, dtype, 11)
    plan = AttentionPlan(M, N, H, dtype, device=dev, d=d)
    big = (M > 64) | (N > 64) if d == 64 else np.ones(len(M), bool)   # at d = 64 the small segments go into packs
    assert plan.summary["umma_items"] == int(np.ceil(M[big] / 128).sum())
    assert plan.summary["launches"] == 1 + int(d == 64)
    out = torch.full((H, int(M.sum()) * d), float("nan"), dtype=dtype, device=dev)
    plan.run(q.to(dev), k.to(dev), v.to(dev), out=out, scale=scale)
    plan.check()
    close(out, oracle_attention(q, k, v, M, N, d, scale), dtype, "attention, tiling edges")


@pytest.mark.parametrize("d", [64, 128])
def test_attention_moving_row_maximum(cuda_device, d):
    # keys grow along the segment, so the row maximum moves by far more than the lazy threshold several times during
    # the sweep and the accumulated result is rescaled in tensor memory; some rows (negative dot products) never move
    dev = cuda_device
    M = np.array([200, 70]); N = np.array([1500, 900])
    H = 2
    q, k, v = inputs(M, N, d, H, F16, 21)
    ramp = torch.cat([torch.linspace(0.2, 3.0, int(n)).repeat_interleave(d) for n in N])
    k = (k.float() * ramp).to(F16)
    got = blockAttention(q.to(dev), k.to(dev), v.to(dev), M, N, scale=0.5, d=d)
    close(got, oracle_attention(q, k, v, M, N, d, 0.5), F16, "attention, moving maximum")


def test_attention_long_tail_batch_and_composition(cuda_device):
    dev = cuda_device
    rs = np.random.RandomState(4)
    n = np.rint(np.exp(rs.uniform(np.log(16), np.log(1500), 40))).astype(np.int64)
    H, d = 4, 64
    q, k, v = inputs(n, n, d, H, BF16, 31)
    qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
    got = blockAttention(qd, kd, vd, n, n, scale=0.125)
    close(got, oracle_attention(q, k, v, n, n, d, 0.125), BF16, "attention, long-tail batch")
    dl = np.full_like(n, d)
    comp = blockGEMM(blockAttnScores(qd, kd, n, n, dl, scale=0.125), vd, None, None, None, n, dl, n, False, True)
    close(got, comp.float().cpu(), BF16, "fused vs composed")


def test_attention_mixed_batch_uses_both_kernels(cuda_device):
    # molecular sizes with a few graphs beyond 64 nodes (d = 64): the small graphs go into packs of the small-segment
    # kernel, the large ones to the tcgen05 kernel; two launches write disjoint rows of one result
    dev = cuda_device
    rs = np.random.RandomState(7)
    n = np.clip(np.rint(rs.normal(25, 10, 500)), 2, 64).astype(np.int64)
    n[::50] = rs.randint(65, 400, size=len(n[::50]))
    M = n.copy(); N = n.copy()
    N[5] = 100                                       # few queries, many keys: not a small segment either
    H, d = 4, 64
    q, k, v = inputs(M, N, d, H, F16, 51)
    plan = AttentionPlan(M, N, H, F16, device=dev, d=d)
    s = plan.summary
    big = (M > 64) | (N > 64)
    assert s["packs"] > 0 and s["launches"] == 2 and s["umma_items"] == int(np.ceil(M[big] / 128).sum())
    out = torch.full((H, int(M.sum()) * d), float("nan"), dtype=F16, device=dev)
    plan.run(q.to(dev), k.to(dev), v.to(dev), out=out, scale=0.125)
    plan.check()
    close(out, oracle_attention(q, k, v, M, N, d, 0.125), F16, "attention, mixed batch")


def test_attention_values_of_a_neighbour_do_not_leak(cuda_device):
    # the value tile of a segment's last keys also holds rows of the next segment; they must not reach the result,
    # not even as 0 * inf: the next segment's values are infinite here
    dev = cuda_device
    M = np.array([50, 40]); N = np.array([37, 60])
    H, d = 2, 128
    q, k, v = inputs(M, N, d, H, F16, 41)
    v = v.clone()
    v.view(H, -1, d)[:, 37:, :] = float("inf")
    got = blockAttention(q.to(dev), k.to(dev), v.to(dev), M, N, scale=0.09)   # d = 128 read off the (H, rows * d) shape
    first = got.view(H, -1, d)[:, :50, :].float().cpu()
    want = oracle_attention(q, k, torch.nan_to_num(v, posinf=0.0), M, N, d, 0.09).view(H, -1, d)[:, :50, :]
    assert bool(torch.isfinite(first).all())
    assert float((first - want).abs().max()) <= TOL[F16] * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("d", [64, 128])
def test_token_major_attention_long_segments(cuda_device, d):
    # (sum n, H, d) tensors in and out: same bits as permuting into strips and back
    dev = cuda_device
    n = np.array([300, 5, 128, 77, 1000])
    H, T = 3, int(n.sum())
    g = torch.Generator().manual_seed(9)
    q, k, v = (torch.randn((T, H, d), generator=g).to(BF16).to(dev) for _ in range(3))
    got = blockAttentionTokenMajor(q, k, v, n, scale=0.1)
    assert got.shape == (T, H, d)
    strips = [t.permute(1, 0, 2).reshape(H, T * d).contiguous() for t in (q, k, v)]
    want = blockAttention(*strips, n, n, scale=0.1, d=d).reshape(H, T, d).permute(1, 0, 2)
    assert torch.equal(got, want)


def test_attention_very_long_key_sweep_and_single_query(cuda_device):
    # 40 key tiles per query block, one query row against thousands of keys, one head: the rings, the two score
    # buffers and the two result buffers wrap many times inside one item
    dev = cuda_device
    M = np.array([1, 130, 3]); N = np.array([5000, 4100, 129])
    H, d = 1, 128
    q, k, v = inputs(M, N, d, H, BF16, 61)
    plan = AttentionPlan(M, N, H, BF16, device=dev, d=d)
    out = torch.full((H, int(M.sum()) * d), float("nan"), dtype=BF16, device=dev)
    for _ in range(2):                                 # a second run of the same plan: barriers start afresh
        plan.run(q.to(dev), k.to(dev), v.to(dev), out=out, scale=0.09)
        plan.check()
    close(out, oracle_attention(q, k, v, M, N, d, 0.09), BF16, "attention, very long key sweep")
