"""Generates tests/golden/*.npz from the CPU oracle (oracle/blk_oracle.py).

Run from the repository root: ``python tests/golden/make_golden.py``.  The
upstream project ships no golden vectors; these fixtures freeze the oracle's
answers on the shapes the upstream author exercised
(csrc/sparseBlockedAttention.cpp:147-155, :170-199, :216-255, :265-294;
test/pytest.py:7-19) plus the 32-segment CPU configuration, so that the oracle
cannot drift silently and the CUDA path is checked against stored numbers as
well as against a live oracle run.  Inputs are stored with the outputs (as the
16-bit or fp32 values the operators receive) so nothing depends on a random
number generator at test time.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
sys.path.insert(0, ROOT)
import blk_oracle as O  # noqa: E402


def _np(t):
    if t.dtype == torch.bfloat16:  # numpy has no bf16: keep the bit pattern
        return t.view(torch.int16).numpy()
    return t.numpy()


def gemm_case(name, M, N, K, H, dtype, seed, ta=False, tb=False, scale=1.0, softmax=False, arange=False):
    M = np.asarray(M, np.int64); N = np.asarray(N, np.int64); K = np.asarray(K, np.int64)
    g = torch.Generator().manual_seed(seed)
    D1, D2 = int((M * K).sum()), int((N * K).sum())
    if arange:
        A = torch.arange(H * D1, dtype=torch.float32).reshape(H, D1).to(dtype)
        B = torch.arange(H * D2, dtype=torch.float32).reshape(H, D2).to(dtype)
    else:
        A = torch.randn((H, D1), generator=g).to(dtype)
        B = torch.randn((H, D2), generator=g).to(dtype)
    out = O.block_gemm(A, B, M, N, K, transpose1=ta, transpose2=tb, scale=scale)
    if softmax:
        out = O.block_softmax(out, M, N)
    a1, a2, ao = O.offsets_from_lists(M, N, K)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), kind="gemm", M=M, N=N, K=K, H=H,
                        dtype=str(dtype).split(".")[-1], ta=ta, tb=tb, scale=scale, softmax=softmax,
                        A=_np(A), B=_np(B), out=out.numpy().astype(np.float32), a1=a1, a2=a2, ao=ao)


def softmax_case(name, rows, cols, H, dtype, seed):
    rows = np.asarray(rows, np.int64); cols = np.asarray(cols, np.int64)
    g = torch.Generator().manual_seed(seed)
    X = torch.randn((H, int((rows * cols).sum())), generator=g).to(dtype)
    out = O.block_softmax(X, rows, cols)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), kind="softmax", rows=rows, cols=cols, H=H,
                        dtype=str(dtype).split(".")[-1], X=_np(X), out=out.numpy().astype(np.float32),
                        acc=O.softmax_offsets(rows, cols))


def attention_case(name, M, N, d, H, dtype, seed, scale):
    # softmax(scale Q K^T) V per segment: the composition of the two operators, all float32 in the oracle
    M = np.asarray(M, np.int64); N = np.asarray(N, np.int64)
    dl = np.full_like(M, d)
    g = torch.Generator().manual_seed(seed)
    Q = torch.randn((H, int(M.sum()) * d), generator=g).to(dtype)
    K = torch.randn((H, int(N.sum()) * d), generator=g).to(dtype)
    V = torch.randn((H, int(N.sum()) * d), generator=g).to(dtype)
    P = O.block_scores(Q, K, M, N, dl, scale=scale)
    out = O.block_gemm(P, V, M, dl, N, transpose2=True)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), kind="attention", M=M, N=N, d=d, H=H,
                        dtype=str(dtype).split(".")[-1], scale=scale, A=_np(Q), B=_np(K), X=_np(V),
                        out=out.numpy().astype(np.float32))


def main():
    rs = np.random.RandomState(0)
    n = rs.randint(4, 33, size=32)
    # the 32-segment CPU configuration: fp32, j = 32, scale 1/sqrt(32), scores + softmax
    gemm_case("cpu_plumbing_fp32", n, n, [32] * 32, 1, torch.float32, 0, scale=1 / np.sqrt(32.0), softmax=True)
    # odd-K shapes of csrc/sparseBlockedAttention.cpp:170-199 (H reduced from 128 to 2)
    gemm_case("oddk_33_127_fp16", [33, 127], [33, 127], [61, 61], 2, torch.float16, 1)
    # arange inputs of csrc/sparseBlockedAttention.cpp:216-255: exact integer answers
    gemm_case("arange_11_13_5_fp32", [11], [13], [5], 1, torch.float32, 2, arange=True)
    # graph lengths of csrc/sparseBlockedAttention.cpp:147-155, d = 32, 8 heads
    gemm_case("graphs_d32_bf16", [10, 5, 20, 5, 60], [10, 5, 20, 5, 60], [32] * 5, 8, torch.bfloat16, 3,
              scale=1 / np.sqrt(32.0), softmax=True)
    # the three fp32 segments of test/pytest.py:7-19 (H reduced from 128 to 2, k from 64 kept)
    gemm_case("script_33_99_64_fp32", [33, 99, 64], [33, 99, 64], [64, 64, 64], 2, torch.float32, 4)
    # transposed operands as the backward of csrc/sparseBlockedAttention.cpp:68-69 uses them
    gemm_case("transposed_fp16", [17, 40], [9, 33], [24, 50], 2, torch.float16, 5, ta=True, tb=True)
    # the half softmax of csrc/sparseBlockedAttention.cpp:265-294 (rows reduced from 127 to 5, H from 7 to 2)
    softmax_case("softmax_5x2047_fp16", [5, 5, 5], [2047, 2047, 2047], 2, torch.float16, 6)
    # the script's softmax check, test/pytest.py:54-62 (H reduced)
    softmax_case("softmax_script_fp32", [33, 99, 64], [64, 64, 64], 2, torch.float32, 7)
    # fused attention: graph sizes of csrc/sparseBlockedAttention.cpp:147-155 at d = 64 (the small-segment kernel),
    # and segments beyond one 128-row block / 128-key tile at d = 128 (the tcgen05 attention kernel)
    attention_case("attention_graphs_d64_fp16", [10, 5, 20, 5, 60], [10, 5, 20, 5, 60], 64, 2, torch.float16, 8, 0.125)
    attention_case("attention_long_d128_bf16", [130, 3, 40], [150, 257, 40], 128, 2, torch.bfloat16, 9,
                   1 / np.sqrt(128.0))
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
