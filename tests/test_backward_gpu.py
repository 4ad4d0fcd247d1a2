"""GPU: the backward pair -- softmax backward kernel and the two permuted GEMM launches -- against the oracle,
and the autograd surface of the Python operators (upstream test/pytest.py:43-46 runs ``res.mean().backward()``)."""
import numpy as np
import pytest
import torch

from helpers import O, packed_inputs
from blockedattention_b200 import blockAttention, blockAttnScores, blockGEMM, blockSoftmax
from blockedattention_b200.plan import SoftmaxPlan

pytestmark = pytest.mark.gpu
F16, BF16, F32 = torch.float16, torch.bfloat16, torch.float32
TOL = {F32: 2e-5, F16: 2e-3, BF16: 1.6e-2}


def close(got, want, dtype, what):
    got = got.detach().float().cpu(); want = want.float()
    scale = max(1.0, float(want.abs().max()))
    err = float((got - want).abs().max())
    assert err <= TOL[dtype] * scale, f"{what}: max abs err {err} (scale {scale})"


@pytest.mark.parametrize("dtype", [F32, F16, BF16])
def test_softmax_backward_kernel(cuda_device, dtype):
    dev = cuda_device
    rs = np.random.RandomState(11)
    # short rows (sub-warp groups), rows of a few hundred columns, a row longer than the 16 KB window, odd offsets
    rows = np.array([5, 1, 17, 3, 2, 40, 1, 7]); cols = np.array([3, 1, 33, 700, 9000, 64, 5000, 129])
    H = 3
    D = int((rows * cols).sum())
    X = torch.randn(H, D) * 2
    P = O.block_softmax(X, rows, cols, scale=0.9).to(dtype)
    G = torch.randn(H, D).to(dtype)
    plan = SoftmaxPlan(rows, cols, H, dtype, device=dev)
    got = plan.run_backward(P.to(dev), G.to(dev), scale=0.9)
    want = O.block_softmax_backward(P, G, rows, cols, scale=0.9)
    close(got, want, dtype, "softmax backward")
    # in place on the gradient
    g2 = G.to(dev).clone()
    res = plan.run_backward(P.to(dev), g2, grad_src=g2, scale=0.9)
    assert res.data_ptr() == g2.data_ptr() and torch.equal(res, got)
    # offsets with gaps: untouched elements keep their canary
    acc = np.concatenate([[0], np.cumsum(rows * cols + 3)])
    Dg = int(acc[-1])
    Pg = torch.zeros(H, Dg, dtype=dtype); Gg = torch.zeros(H, Dg, dtype=dtype)
    for s in range(len(rows)):
        n = int(rows[s] * cols[s]); o = int((rows[:s] * cols[:s]).sum())
        Pg[:, acc[s]:acc[s] + n] = P[:, o:o + n]; Gg[:, acc[s]:acc[s] + n] = G[:, o:o + n]
    plan_g = SoftmaxPlan(rows, cols, H, dtype, accum=acc, device=dev)
    out = torch.full((H, Dg), 7.0, dtype=dtype, device=dev)
    plan_g.run_backward(Pg.to(dev), Gg.to(dev), grad_src=out, scale=0.9)
    want_g = O.block_softmax_backward(Pg, Gg, rows, cols, srcAccum=acc, scale=0.9)
    for s in range(len(rows)):
        n = int(rows[s] * cols[s])
        close(out[:, acc[s]:acc[s] + n], want_g[:, acc[s]:acc[s] + n], dtype, f"gapped segment {s}")
        assert bool((out[:, acc[s] + n:acc[s + 1]] == 7.0).all())


@pytest.mark.parametrize("dtype,K", [(F32, 24), (F16, 64), (BF16, 40)])
def test_gemm_autograd_matches_upstream_backward(cuda_device, dtype, K):
    dev = cuda_device
    rs = np.random.RandomState(7)
    M = rs.randint(1, 90, size=12); N = rs.randint(1, 90, size=12); Kl = np.full(12, K)
    H = 2
    A, B = packed_inputs(M, N, Kl, H, dtype, 4)
    a = A.to(dev).requires_grad_(); b = B.to(dev).requires_grad_()
    out = blockGEMM(a, b, None, None, None, M, N, Kl, scale=0.5)
    assert out.requires_grad
    g = (torch.randn(out.shape) * 0.5).to(dtype)
    out.backward(g.to(dev))
    w1, w2 = O.block_gemm_backward(A, B, g, M, N, Kl, scale=0.5)
    close(a.grad, w1, dtype, "mat1 grad")
    close(b.grad, w2, dtype, "mat2 grad")
    assert a.grad.shape == a.shape and b.grad.shape == b.shape and a.grad.dtype == dtype


def test_chained_operators_backward_like_upstream_script(cuda_device):
    # blockGEMM -> blockSoftmax -> mean().backward(), fp32, the upstream script's sizes (test/pytest.py:7-46)
    dev = cuda_device
    h, m, n, k = 8, 33, 99, 64
    M = torch.tensor([m, n, k], device=dev); Kl = torch.tensor([k, k, k], device=dev)
    torch.manual_seed(0)
    A = torch.randn(h, m * k + n * k + k * k); B = torch.randn(h, m * k + n * k + k * k)
    a = A.to(dev).requires_grad_(); b = B.to(dev).requires_grad_()
    res = blockSoftmax(blockGEMM(a, b, None, None, None, M, M, Kl), M, M)
    res.mean().backward()
    # the same chain with torch autograd on the CPU, float64
    a64 = A.double().requires_grad_(); b64 = B.double().requires_grad_()
    outs, o = [], 0
    for r in (m, n, k):
        x = a64[:, o:o + r * k].reshape(h, r, k); y = b64[:, o:o + r * k].reshape(h, r, k)
        outs.append((x @ y.transpose(1, 2)).softmax(-1).reshape(h, r * r)); o += r * k
    torch.cat(outs, 1).mean().backward()
    close(a.grad, a64.grad, F32, "chained mat1 grad")
    close(b.grad, b64.grad, F32, "chained mat2 grad")


@pytest.mark.parametrize("dtype", [F16, BF16])
def test_fused_scores_backward(cuda_device, dtype):
    dev = cuda_device
    rs = np.random.RandomState(2)
    n = rs.randint(2, 70, size=20); Kl = np.full(20, 64)
    H = 4
    Q, Kt = packed_inputs(n, n, Kl, H, dtype, 9)
    q = Q.to(dev).requires_grad_(); k = Kt.to(dev).requires_grad_()
    p = blockAttnScores(q, k, n, n, Kl, scale=0.125)
    g = torch.randn(p.shape).to(dtype)
    p.backward(g.to(dev))
    # oracle: softmax backward on the rounded probabilities, then the two permuted GEMMs with the scale
    ds = O.block_softmax_backward(p.detach().cpu(), g, n, n).to(dtype)
    w1, w2 = O.block_gemm_backward(Q, Kt, ds, n, n, Kl, scale=0.125)
    close(q.grad, w1, dtype, "dq")
    close(k.grad, w2, dtype, "dk")


@pytest.mark.parametrize("d,sizes", [(64, [5, 33, 64, 17]),          # packs of the small-segment kernel
                                     (64, [5, 200, 64, 130]),        # packs and the tcgen05 attention kernel
                                     (128, [150, 7, 260])])          # the tcgen05 attention kernel
def test_fused_attention_backward(cuda_device, d, sizes):
    # forward on the fused kernels; backward recomputes the probabilities with the two-operator path.  Checked against
    # torch autograd of the per-segment formula in float64.
    dev = cuda_device
    n = np.array(sizes, np.int64)
    m = np.maximum(n - 3, 1)                      # fewer queries than keys
    H, scale = 2, 0.1
    g = torch.Generator().manual_seed(5)
    q0 = torch.randn((H, int(m.sum()) * d), generator=g).to(F16)
    k0 = torch.randn((H, int(n.sum()) * d), generator=g).to(F16)
    v0 = torch.randn((H, int(n.sum()) * d), generator=g).to(F16)
    go = torch.randn((H, int(m.sum()) * d), generator=g).to(F16)
    q, k, v = (t.to(dev).requires_grad_(True) for t in (q0, k0, v0))
    out = blockAttention(q, k, v, m, n, scale=scale, d=d)
    out.backward(go.to(dev))
    # reference
    qr, kr, vr = (t.double().requires_grad_(True) for t in (q0, k0, v0))
    outs = []; oq = okv = 0
    for ms, ns in zip(m, n):
        ms, ns = int(ms), int(ns)
        Q = qr[:, oq * d:(oq + ms) * d].reshape(H, ms, d); K = kr[:, okv * d:(okv + ns) * d].reshape(H, ns, d)
        V = vr[:, okv * d:(okv + ns) * d].reshape(H, ns, d)
        outs.append((torch.softmax(scale * Q @ K.transpose(1, 2), dim=-1) @ V).reshape(H, ms * d))
        oq += ms; okv += ns
    ref = torch.cat(outs, dim=1)
    ref.backward(go.double())
    close(out, ref.detach(), F16, "fused attention forward")
    for name, got, want in (("dq", q.grad, qr.grad), ("dk", k.grad, kr.grad), ("dv", v.grad, vr.grad)):
        assert got is not None and got.shape == want.shape
        s = max(1.0, float(want.abs().max()))
        err = float((got.float().cpu() - want.float()).abs().max())
        assert err <= 1e-2 * s, f"{name}: max abs err {err} (scale {s})"
