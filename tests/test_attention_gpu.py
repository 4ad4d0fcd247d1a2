"""GPU: the fused small-segment attention kernel against the oracle (softmax(scale Q K^T) V per segment) and against
the two-operator composition it replaces."""
import numpy as np
import pytest
import torch

from helpers import O, packed_inputs
from blockedattention_b200 import blockAttention, blockAttentionTokenMajor, blockAttnScores, blockGEMM
from blockedattention_b200.plan import AttentionPlan

pytestmark = pytest.mark.gpu
F16, BF16 = torch.float16, torch.bfloat16
TOL = {F16: 2e-3, BF16: 1.6e-2}


def oracle_attention(q, k, v, M, N, scale):
    # per segment: P = softmax(scale Q K^T), O = P V, float32 throughout (oracle GEMM restatements)
    d = np.full_like(M, 64)
    P = O.block_scores(q, k, M, N, d, scale=scale)
    return O.block_gemm(P, v, M, d, N, transpose2=True)


def close(got, want, dtype, what):
    got = got.detach().float().cpu(); want = want.float()
    scale = max(1.0, float(want.abs().max()))
    err = float((got - want).abs().max())
    assert err <= TOL[dtype] * scale, f"{what}: max abs err {err} (scale {scale})"


@pytest.mark.parametrize("dtype", [F16, BF16])
@pytest.mark.parametrize("scale", [0.125, -0.3])
def test_fused_attention_every_small_extent(cuda_device, dtype, scale):
    # every (m, n) in a grid up to 64 x 64, including single rows and columns and the 16-row block boundaries
    dev = cuda_device
    g = np.array([1, 2, 7, 8, 9, 15, 16, 17, 25, 31, 32, 33, 47, 48, 49, 63, 64])
    M, N = [a.ravel() for a in np.meshgrid(g, g, indexing="ij")]
    H = 2
    q, k = packed_inputs(M, N, np.full_like(M, 64), H, dtype, 1)
    v = packed_inputs(N, N, np.full_like(M, 64), H, dtype, 2)[0]
    out = torch.full((H, int(M.sum()) * 64), float("nan"), dtype=dtype, device=dev)
    plan = AttentionPlan(M, N, H, dtype, device=dev, small_only=True)
    assert plan.summary["packs"] > 0 and plan.summary["tile_items"] == 0
    plan.run(q.to(dev), k.to(dev), v.to(dev), out=out, scale=scale)
    plan.check()
    assert not bool(torch.isnan(out.float()).any())
    close(out, oracle_attention(q, k, v, M, N, scale), dtype, "fused attention grid")


def test_fused_attention_molecular_sizes_and_composition(cuda_device):
    dev = cuda_device
    rs = np.random.RandomState(0)
    n = np.clip(np.rint(rs.normal(25, 10, 600)), 2, 64).astype(np.int64)
    H = 8
    q, k = packed_inputs(n, n, np.full_like(n, 64), H, F16, 3)
    v = packed_inputs(n, n, np.full_like(n, 64), H, F16, 4)[0]
    qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
    got = blockAttention(qd, kd, vd, n, n, scale=0.125)
    close(got, oracle_attention(q, k, v, n, n, 0.125), F16, "fused attention, molecular sizes")
    # the composition of the two operators it replaces (rounds the probabilities to fp16 in between)
    d = np.full_like(n, 64)
    comp = blockGEMM(blockAttnScores(qd, kd, n, n, d, scale=0.125), vd, None, None, None, n, d, n, False, True)
    close(got, comp.float().cpu(), F16, "fused vs composed")
    # values left over in shared memory from other segments must not leak in: zero values give a zero result
    z = blockAttention(qd, kd, torch.zeros_like(vd), n, n, scale=0.125)
    assert float(z.float().abs().max()) == 0.0


def test_attention_falls_back_to_the_composition(cuda_device):
    # a head dimension neither fused kernel takes runs as scores + P V; same operator, same result
    dev = cuda_device
    n = np.array([10, 100, 64, 200])
    H = 2
    q, k = packed_inputs(n, n, np.full_like(n, 32), H, BF16, 5)
    v = packed_inputs(n, n, np.full_like(n, 32), H, BF16, 6)[0]
    got = blockAttention(q.to(dev), k.to(dev), v.to(dev), n, n, scale=0.125, d=32)
    d = np.full_like(n, 32)
    P = O.block_scores(q, k, n, n, d, scale=0.125)
    close(got, O.block_gemm(P, v, n, d, n, transpose2=True), BF16, "composed attention")
    with pytest.raises(RuntimeError):
        AttentionPlan(n, n, H, BF16, device=dev, small_only=True)   # the pack kernel refuses segments beyond 64 rows
    with pytest.raises(RuntimeError):
        AttentionPlan(n, n, H, BF16, device=dev, d=32)              # and neither kernel has this head dimension
    with pytest.raises(RuntimeError):
        blockAttention(q, k.to(dev), v.to(dev), n, n)  # CPU tensor


@pytest.mark.parametrize("dtype", [F16, BF16])
def test_token_major_attention_matches_packed(cuda_device, dtype):
    # (sum n, H, 64) tensors in and out, read and written in place: same bits as permuting into strips and back
    dev = cuda_device
    rs = np.random.RandomState(8)
    n = rs.randint(1, 65, size=300)
    H, T = 5, int(n.sum())
    g = torch.Generator().manual_seed(9)
    q, k, v = (torch.randn((T, H, 64), generator=g).to(dtype).to(dev) for _ in range(3))
    got = blockAttentionTokenMajor(q, k, v, n, scale=0.125)
    assert got.shape == (T, H, 64)
    strips = [t.permute(1, 0, 2).reshape(H, T * 64).contiguous() for t in (q, k, v)]
    want = blockAttention(*strips, n, n, scale=0.125).reshape(H, T, 64).permute(1, 0, 2)
    assert torch.equal(got, want)
    with pytest.raises(RuntimeError):
        blockAttentionTokenMajor(q[:, :, :32], k[:, :, :32], v[:, :, :32], n)
