"""CPU: the C ABI loads and exports what include/blkattn.h declares; host-side
index helpers are bit-exact with the oracle; scheduler and partitioners behave."""
import ctypes as C
import os
import re

import numpy as np
import pytest
import torch

from helpers import O, ROOT
from blockedattention_b200 import _lib as L
from blockedattention_b200 import partition as P
from blockedattention_b200.plan import AttentionPlan, GemmPlan, SoftmaxPlan
from blockedattention_b200.synth import WORKLOADS, workload


def declared_symbols():
    src = open(os.path.join(ROOT, "include", "blkattn.h")).read()
    return sorted(set(re.findall(r"BLK_API\s+[\w\s\*]+?\b(blk_\w+)\s*\(", src)))


def test_library_exports_every_declared_symbol():
    names = declared_symbols()
    assert len(names) >= 18
    lib = C.CDLL(L.LIB_PATH)
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/blkattn.h but not exported"
    assert set(names) == set(L.SIGNATURES), "ctypes table and header disagree"
    assert b"sm_100a" in L.lib.blk_version()


def _offsets(M, N, K):
    M = np.ascontiguousarray(M, np.int64); N = np.ascontiguousarray(N, np.int64); K = np.ascontiguousarray(K, np.int64)
    S = len(M)
    a1 = np.empty(S + 1, np.int64); a2 = np.empty_like(a1); ao = np.empty_like(a1)
    L.check(L.lib.blk_offsets_from_lists(L.i64(M), L.i64(N), L.i64(K), S, L.i64(a1), L.i64(a2), L.i64(ao)))
    return a1, a2, ao


@pytest.mark.parametrize("name", WORKLOADS)
def test_offsets_bit_exact_on_every_workload(name):
    w = workload(name)
    a1, a2, ao = _offsets(w.M, w.N, w.K)
    o1, o2, oo = O.offsets_from_lists(w.M, w.N, w.K)
    assert np.array_equal(a1, o1) and np.array_equal(a2, o2) and np.array_equal(ao, oo)
    # and the inverse recovers the lists exactly
    S = w.S
    M = np.empty(S, np.int64); N = np.empty(S, np.int64); K = np.empty(S, np.int64)
    L.check(L.lib.blk_lists_from_offsets(L.i64(a1), L.i64(a2), L.i64(ao), S, L.i64(M), L.i64(N), L.i64(K)))
    assert np.array_equal(M, w.M) and np.array_equal(N, w.N) and np.array_equal(K, w.K)


def test_offsets_empty_and_overflow():
    a1, a2, ao = _offsets([], [], [])
    assert a1.tolist() == [0] and a2.tolist() == [0] and ao.tolist() == [0]
    a1, a2, ao = _offsets([0, 3, 0], [4, 0, 0], [5, 6, 7])
    assert a1.tolist() == [0, 0, 18, 18] and a2.tolist() == [0, 20, 20, 20] and ao.tolist() == [0, 0, 0, 0]
    with pytest.raises(L.BlkError) as e:
        _offsets([2 ** 40], [2 ** 40], [2 ** 40])
    assert e.value.code == L.BLK_ERR_INVALID
    with pytest.raises(L.BlkError):
        _offsets([-1], [1], [1])


def test_lists_from_offsets_agrees_with_upstream_formula_where_that_is_consistent():
    rs = np.random.RandomState(1)
    M = rs.randint(1, 3000, 500); N = rs.randint(1, 3000, 500); K = rs.randint(1, 300, 500)
    a1, a2, ao = O.offsets_from_lists(M, N, K)
    Mo = np.empty(500, np.int64); No = np.empty_like(Mo); Ko = np.empty_like(Mo)
    L.check(L.lib.blk_lists_from_offsets(L.i64(a1), L.i64(a2), L.i64(ao), 500, L.i64(Mo), L.i64(No), L.i64(Ko)))
    assert np.array_equal(Mo, M) and np.array_equal(No, N) and np.array_equal(Ko, K)
    Mf, Nf, Kf = O.lists_from_offsets_float32(a1, a2, ao)
    ok = (Mf * Kf == a1[1:] - a1[:-1]) & (Nf * Kf == a2[1:] - a2[:-1]) & (Mf * Nf == ao[1:] - ao[:-1])
    assert ok.sum() > 100
    assert np.array_equal(Mo[ok], Mf[ok]) and np.array_equal(No[ok], Nf[ok]) and np.array_equal(Ko[ok], Kf[ok])
    bad = np.array([0, 6], np.int64), np.array([0, 6], np.int64), np.array([0, 5], np.int64)
    with pytest.raises(L.BlkError):
        L.check(L.lib.blk_lists_from_offsets(L.i64(bad[0]), L.i64(bad[1]), L.i64(bad[2]), 1, L.i64(Mo), L.i64(No), L.i64(Ko)))


def test_softmax_offsets():
    rows = np.array([127, 127, 127, 0, 3], np.int64); cols = np.array([2047, 2047, 2047, 9, 1], np.int64)
    acc = np.empty(6, np.int64)
    L.check(L.lib.blk_softmax_offsets(L.i64(rows), L.i64(cols), 5, L.i64(acc)))
    assert np.array_equal(acc, O.softmax_offsets(rows, cols))


# ---- scheduler ---------------------------------------------------------------
def test_attention_schedule_picks_the_kernel_by_batch():
    # graphs of at most 64 nodes with d = 64: packs of the small-segment kernel, one launch
    w = workload("molecular_attention")
    p = AttentionPlan(w.M, w.N, w.H, w.dtype, d=64)
    s = p.summary
    assert s["packs"] > 0 and s["umma_items"] == 0 and s["launches"] == 1
    assert p.work[0] == pytest.approx(w.flops()) and p.work[1] == pytest.approx(w.bytes())
    # longer segments, or d = 128: one item per 128-row block of queries on the tcgen05 attention kernel (at d = 64
    # the segments of at most 64 x 64 stay in packs: two launches)
    for name in ("long_tail_attention", "full_forward_attention"):
        w = workload(name)
        d = int(w.K[0])
        p = AttentionPlan(w.M, w.N, w.H, w.dtype, d=d)
        s = p.summary
        big = (w.M > 64) | (w.N > 64) if d == 64 else np.ones(w.S, bool)
        assert (s["packs"] > 0) == bool((~big).any()) and s["tile_items"] == 0
        assert s["launches"] == 1 + int((~big).any())
        assert s["umma_items"] == int(np.ceil(w.M[big] / 128).sum())
        assert p.work[0] == pytest.approx(w.flops()) and p.work[1] == pytest.approx(w.bytes())
        assert p.extents[0] == int(w.M.sum()) * int(w.K[0]) and p.extents[2] == p.extents[0]
    # d = 64 with a few long segments: packs for the small ones, tcgen05 items for the rest, two launches
    w = workload("molecular")
    M = w.M.copy(); N = w.N.copy()
    M[::97] = 150; N[::97] = 150
    N[5] = 100
    p = AttentionPlan(M, N, w.H, w.dtype, d=64)
    s = p.summary
    big = (M > 64) | (N > 64)
    assert s["packs"] > 0 and s["launches"] == 2
    assert s["umma_items"] == int(np.ceil(M[big] / 128).sum()) and s["small_items"] == int((~big).sum())
    # what neither kernel takes
    with pytest.raises(RuntimeError):
        AttentionPlan([4], [4], 1, torch.float16, d=32)
    with pytest.raises(RuntimeError):
        AttentionPlan([4], [0], 1, torch.float16, d=64)       # queries without keys
    with pytest.raises(RuntimeError):
        AttentionPlan([100], [100], 1, torch.float16, d=64, small_only=True)
    with pytest.raises(RuntimeError):
        AttentionPlan([4], [4], 1, torch.float32, d=64)
    assert AttentionPlan([0, 0], [0, 5], 2, torch.bfloat16, d=128).summary["launches"] == 0


def test_schedule_bins_and_work():
    w = workload("molecular")
    p = GemmPlan(w.M, w.N, w.K, w.H, w.dtype, softmax=True)
    s = p.summary
    assert s["segments"] == 4096 and s["small_items"] + s["tile_items"] > 0
    assert s["small_items"] == int((w.N <= 64).sum())
    fl, by = p.work
    assert fl == pytest.approx(w.flops()) and by == pytest.approx(w.bytes())
    assert p.extents == (w.Dm1, w.Dm2, w.Dout)

    w = workload("long_tail")
    p = GemmPlan(w.M, w.N, w.K, w.H, w.dtype, softmax=True)
    s = p.summary
    big = w.N > 64
    assert s["tile_items"] + s["umma_items"] >= int(np.ceil(w.M[big] / 128).sum())

    w = workload("general_gemm")
    p = GemmPlan(w.M, w.N, w.K, w.H, w.dtype, torch.float32)
    assert p.summary["launches"] >= 1 and p.work[0] == pytest.approx(w.flops())


def _with_env(env, fn):
    old = {k: os.environ.get(k) for k in env}
    os.environ.update(env)
    try:
        return fn()
    finally:
        for k, v in old.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v


def test_tcgen05_bin_takes_mixed_contraction_lengths():
    # six contraction lengths, offsets that are no whole rows of a segment's own (rows, K) view: 24 views per operand
    # cover all of them, every segment goes to the tcgen05 kernel (the handful of small ones ride along), one launch
    w = workload("general_gemm")
    s = GemmPlan(w.M, w.N, w.K, w.H, w.dtype, torch.float32).summary
    assert s["umma_items"] == int(np.ceil(w.M / 128).sum()) and s["tile_items"] == 0 and s["small_items"] == 0
    assert s["launches"] == 1
    # with the ride-along rule off the small segments of the small kernel's K get their own launches
    s0 = _with_env({"BLK_SMALL_MIN_PAIRS": "0"}, lambda: GemmPlan(w.M, w.N, w.K, w.H, w.dtype, torch.float32).summary)
    assert s0["small_items"] > 0 and s0["umma_items"] + s0["small_items"] <= s["umma_items"] and s0["launches"] > 1
    # a batch of small segments only keeps its small-segment launch: there is no tcgen05 launch to ride along with
    sm = GemmPlan([20, 30, 64], [20, 30, 64], [64, 64, 64], 2, torch.float16, softmax=True).summary
    assert sm["umma_items"] == 0 and sm["small_items"] == 3
    # more (K, offset) combinations than view slots: the lightest fall back to the staged kernel
    rs = np.random.RandomState(6)
    M = rs.randint(65, 200, size=120); N = rs.randint(65, 200, size=120); K = rs.choice(np.arange(16, 400, 8), size=120)
    s = GemmPlan(M, N, K, 2, torch.bfloat16).summary
    assert s["umma_items"] > 0 and s["tile_items"] > 0
    # K that is no multiple of 8: rows of the views would not be 16-byte multiples
    s = GemmPlan([200, 200], [300, 300], [36, 100], 1, torch.float16).summary
    assert s["umma_items"] == 0 and s["tile_items"] > 0


def test_tcgen05_items_per_tile_for_long_contractions():
    # scores only and K >= 512: one item per 128 x 256 tile; with the fused softmax, or a shorter K, one per row block
    w = workload("large_k")
    s = GemmPlan(w.M, w.N, w.K, w.H, w.dtype).summary
    assert s["umma_items"] == int((np.ceil(w.M / 128) * np.ceil(w.N / 256)).sum()) and s["launches"] == 1
    s = GemmPlan(w.M, w.N, w.K, w.H, w.dtype, softmax=True).summary
    assert s["umma_items"] == int(np.ceil(w.M / 128).sum())
    s = GemmPlan([300, 700], [900, 100], [256, 256], 2, torch.bfloat16).summary
    assert s["umma_items"] == 3 + 6

    w = workload("cpu_plumbing")
    p = GemmPlan(w.M, w.N, w.K, w.H, torch.float32, softmax=True)
    s = p.summary
    assert s["simt_items"] == w.S and s["softmax_chunks"] >= 1 and s["launches"] == 2


def test_schedule_rejects_bad_input():
    with pytest.raises(L.BlkError) as e:
        GemmPlan([4], [4], [8], 1, torch.float16, accum=([0, 31], [0, 32], [0, 16]))  # 4*8 = 32 > 31
    assert e.value.code == L.BLK_ERR_INVALID
    with pytest.raises(L.BlkError):
        GemmPlan([4, 4], [4, 4], [8, 8], 1, torch.float16, accum=([0, 32, 30], [0, 32, 64], [0, 16, 32]))
    with pytest.raises(L.BlkError) as e:
        GemmPlan([4], [4], [8], 1, torch.float32, torch.float16)
    assert e.value.code == L.BLK_ERR_UNSUPPORTED
    with pytest.raises(L.BlkError):
        GemmPlan([-1], [4], [8], 1, torch.float16)
    with pytest.raises(RuntimeError):
        GemmPlan([1, 2], [1], [1], 1, torch.float16)
    p = GemmPlan([4], [4], [8], 1, torch.float16)      # no device: cannot run
    with pytest.raises(RuntimeError):
        p.run(torch.zeros(1, 32, dtype=torch.float16), torch.zeros(1, 32, dtype=torch.float16))


def test_softmax_schedule_chunks():
    p = SoftmaxPlan([127] * 3, [2047] * 3, 7, torch.float16)
    # rows of 4094 bytes: three fit a 12 KB window, so 127 rows make 43 chunks
    assert p.summary["softmax_chunks"] == 3 * 43 and p.D == 3 * 127 * 2047
    p = SoftmaxPlan([3, 0, 2], [20000, 5, 0], 1, torch.float32)   # rows longer than the window: one chunk per row
    assert p.summary["softmax_chunks"] == 3
    p = SoftmaxPlan([], [], 4, torch.bfloat16)
    assert p.summary["softmax_chunks"] == 0 and p.D == 0
    assert p.work[1] == 0


# ---- partitioners --------------------------------------------------------------
def brute_force_bottleneck(cost, R):
    import itertools
    S = len(cost)
    best = float("inf")
    for cuts in itertools.combinations_with_replacement(range(S + 1), R - 1):
        b = (0,) + cuts + (S,)
        best = min(best, max(sum(cost[b[i]:b[i + 1]]) for i in range(R)))
    return best


def test_partition_contiguous_is_optimal_on_small_cases():
    rs = np.random.RandomState(0)
    for trial in range(30):
        S = rs.randint(1, 10); R = rs.randint(1, 5)
        cost = rs.rand(S) ** 3
        b = P.partition_contiguous(cost, R)
        assert b[0] == 0 and b[-1] == S and (np.diff(b) >= 0).all()
        got = max(cost[b[i]:b[i + 1]].sum() for i in range(R))
        assert got <= brute_force_bottleneck(cost.tolist(), R) * (1 + 1e-6)


@pytest.mark.parametrize("name", ["molecular", "long_tail", "full_forward"])
def test_partition_balance_on_workloads(name):
    w = workload(name)
    cost = P.segment_cost(w.M, w.N, w.K, w.H)
    assert (cost > 0).all()
    for R in (1, 2, 4, 8):
        b = P.partition_contiguous(cost, R)
        assert P.imbalance(cost, b) < 1.06
        owner = P.partition_lpt(cost, R)
        loads = np.bincount(owner, weights=cost, minlength=R)
        assert loads.max() / loads.mean() < 1.06
        lo, hi = P.shard_range(w.M, w.N, w.K, w.H, R - 1, R)
        assert (lo, hi) == (b[R - 1], b[R])


def test_partition_edge_cases():
    assert P.partition_contiguous([], 4).tolist() == [0, 0, 0, 0, 0]
    b = P.partition_contiguous([5.0], 3)
    assert b[0] == 0 and b[-1] == 1
    with pytest.raises(L.BlkError):
        P.partition_contiguous([1.0, -1.0], 2)
    with pytest.raises(L.BlkError):
        P.partition_contiguous([1.0], 0)


def test_plan_cache_is_keyed_on_list_values_not_addresses():
    # a freed list tensor's address comes back with other values: the key must follow the values
    from blockedattention_b200 import apply as A
    A.clear_plan_cache()
    keys, ptrs = set(), set()
    for i in range(40):
        t = torch.tensor([10 + i, 50 - i])
        ptrs.add(t.data_ptr())
        keys.add(A._key_of(t))
        A._LISTS.clear()          # the memo would keep t alive; without it the allocator reuses the block
        del t
    assert len(keys) == 40, "two lists with different values shared a key"
    # a remembered tensor is not read again, and an in-place write is seen
    t = torch.tensor([3, 4, 5])
    k1 = A._key_of(t)
    assert A._key_of(t) == k1 and len(A._LISTS) == 1
    t[1] = 9
    assert A._key_of(t) != k1
    # host sequences, arrays and tensors with equal values share one key
    assert A._key_of([3, 9, 5]) == A._key_of(np.array([3, 9, 5])) == A._key_of(t)
    A.clear_plan_cache()


def test_evicted_plans_stay_usable_for_their_holders():
    # the cache drops an evicted plan without closing it: whoever still holds it (an autograd context between
    # forward and backward, a queued host-pipe step) keeps a live handle
    from blockedattention_b200 import apply as A
    A.clear_plan_cache()
    first = A._cached(("t", 0), lambda: SoftmaxPlan([3], [4], 1, torch.float16))
    for i in range(1, A._CACHE_MAX + 5):
        A._cached(("t", i), lambda: SoftmaxPlan([3], [4 + i], 1, torch.float16))
    assert ("t", 0) not in A._CACHE and len(A._CACHE) == A._CACHE_MAX
    assert first._h and first.extents[0] == 12
    A.clear_plan_cache()
    assert first._h and first.extents[0] == 12


def test_softmax_schedule_refuses_by_count_before_building():
    # 2^30 rows of more than a window each would be 2^30 chunks (tens of GB of host memory): refused from the lists alone, quickly
    import time
    t0 = time.perf_counter()
    with pytest.raises(L.BlkError) as e:
        SoftmaxPlan([2 ** 29, 2 ** 29], [9000, 9000], 4, torch.float16)
    assert e.value.code == L.BLK_ERR_UNSUPPORTED and time.perf_counter() - t0 < 1.0
