"""CPU: the schedules themselves, read back through ``blk_plan_table``.  Every output element of a batch must belong
to exactly one work item, the items must address their operands where the offsets say, and the orderings and size
limits the kernels rely on must hold."""
import numpy as np
import pytest
import torch

from blockedattention_b200.plan import AttentionPlan, GemmPlan, SoftmaxPlan, TABLES
from blockedattention_b200.synth import workload

WINDOW = 12288  # bytes of a softmax window
PACK_ROWS, PACK_ROWS_ATTN, PACK_BLOCKS = 192, 128, 16


def _batch(mode, rs, S):
    ks = np.array([16, 32, 48, 64, 96, 128, 40, 72])
    if mode == "mixed":
        return rs.randint(1, 257, S), rs.randint(1, 257, S), ks[rs.randint(0, 6, S)]
    if mode == "graphs":
        n = rs.randint(2, 92, S)
        return n, n, np.full(S, 64)
    if mode == "long":
        n = rs.randint(16, 1500, S)
        return n, n, np.full(S, 64)
    if mode == "ragged":
        return rs.randint(0, 300, S), rs.randint(0, 700, S), 8 * rs.randint(1, 60, S)
    if mode == "deep":
        n = rs.randint(300, 700, S)
        return n, n, 512 << rs.randint(0, 2, S)
    if mode == "tiny":
        return rs.randint(0, 70, S), rs.randint(0, 70, S), ks[rs.randint(0, 8, S)]
    if mode == "oddk":
        return rs.randint(1, 200, S), rs.randint(1, 200, S), rs.randint(1, 131, S)
    raise KeyError(mode)


MODES = ["mixed", "graphs", "long", "ragged", "deep", "tiny", "oddk"]


def _cover_block(cover, off, M, N, r0, r1, c0, c1):
    cover[off:off + M * N].reshape(M, N)[r0:r1, c0:c1] += 1


def _gemm_cover(plan, M, N, ao):
    """Number of work items that write each output element of one head strip."""
    cover = np.zeros(int(ao[-1]), np.int32)
    seg_of = {int(ao[s]): s for s in range(len(M)) if M[s] > 0 and N[s] > 0}
    segs = plan.table("segments")
    for name, bm, bn in (("tile_items", 64, 128), ("simt_items", 64, 64)):
        for it in plan.table(name):
            s = int(it["seg"])
            _cover_block(cover, int(ao[s]), int(M[s]), int(N[s]), it["tm"] * bm, min((it["tm"] + 1) * bm, M[s]),
                         it["tn"] * bn, min((it["tn"] + it["ntn"]) * bn, N[s]))
    for name in ("small_items_32", "small_items_64"):
        for it in plan.table(name):
            s = seg_of[int(it["offC"])]
            assert (it["M"], it["N"]) == (M[s], N[s]) and it["offA"] == segs[s]["offA"] and it["offB"] == segs[s]["offB"]
            assert (it["N"] <= 32) == (name == "small_items_32")
            cover[int(ao[s]):int(ao[s + 1])] += 1
    for it in plan.table("umma_items"):
        s = seg_of[int(it["offC"])]
        assert (it["M"], it["N"]) == (M[s], N[s])
        c0, c1 = (0, int(N[s])) if it["nch"] == 0 else (it["ch0"] * 256, min((it["ch0"] + it["nch"]) * 256, int(N[s])))
        _cover_block(cover, int(ao[s]), int(M[s]), int(N[s]), it["tm"] * 128, min((it["tm"] + 1) * 128, M[s]), c0, c1)
    for it in plan.table("pv_items"):
        # offC is the block's first result row; the item holds min(M, 128) rows of the segment's D columns
        s = max(k for k in seg_of.values() if ao[k] <= it["offC"])
        rows = min(int(it["M"]), 128)
        tm, rem = divmod(int(it["offC"] - ao[s]), 128 * int(N[s]))
        assert rem == 0 and it["M"] == M[s] - 128 * tm and it["K"] == segs[s]["K"]
        assert it["offA"] == segs[s]["offA"] + tm * 128 * int(it["K"])   # first operand: rows of K elements
        assert int(it["rowB"]) * int(N[s]) == segs[s]["offB"]            # second operand: (rows, D) view of the strip
        cover[int(it["offC"]):int(it["offC"]) + rows * int(N[s])] += 1
    packs, blocks = plan.table("packs"), plan.table("pack_blocks")
    for pk in packs:
        for b in blocks[pk["first_block"]:pk["first_block"] + pk["nblocks"]]:
            cover[int(b["offC"]):int(b["offC"]) + int(b["M"]) * int(b["N"])] += 1
    return cover


@pytest.mark.parametrize("softmax", [False, True])
@pytest.mark.parametrize("mode", MODES)
def test_every_output_element_belongs_to_one_work_item(mode, softmax):
    rs = np.random.RandomState(MODES.index(mode) + 17 * softmax)
    for trial in range(3):
        S = int(rs.randint(1, 12 if mode in ("long", "deep") else 150))
        M, N, K = (np.asarray(x, np.int64) for x in _batch(mode, rs, S))
        for odt in (torch.float16, torch.float32):
            plan = GemmPlan(M, N, K, 1 + trial, torch.float16, odt, softmax=softmax)
            _, _, ao = plan.offsets
            cover = _gemm_cover(plan, M, N, ao)
            assert cover.size == 0 or (cover.min() == 1 and cover.max() == 1), (mode, softmax, trial, odt, plan.summary)
            if plan.summary["packs"]:
                assert plan.table("small_items_32").size == 0 and plan.table("small_items_64").size == 0
                assert plan.summary["small_items"] > 0


def test_transposed_and_fp32_batches_are_covered_too():
    rs = np.random.RandomState(5)
    M, N, K = rs.randint(1, 200, 40), rs.randint(1, 200, 40), rs.randint(1, 100, 40)
    for kw in (dict(transpose1=True), dict(transpose2=True), dict(transpose1=True, transpose2=True)):
        plan = GemmPlan(M, N, K, 2, torch.bfloat16, **kw)
        cover = _gemm_cover(plan, M, N, plan.offsets[2])
        assert cover.min() == 1 and cover.max() == 1
    plan = GemmPlan(M, N, K, 2, torch.float32, softmax=True)
    cover = _gemm_cover(plan, M, N, plan.offsets[2])
    assert cover.min() == 1 and cover.max() == 1 and plan.table("simt_items").size > 0
    # the product with a (K, D) second operand: D = 64 segments on the tcgen05 kernel for that layout
    Mv, Kv = rs.randint(1, 400, 30), rs.randint(1, 400, 30)
    plan = GemmPlan(Mv, np.full(30, 64), Kv, 3, torch.float16, transpose2=True)
    assert plan.table("pv_items").size == sum(-(-int(m) // 128) for m in Mv)
    cover = _gemm_cover(plan, Mv, np.full(30, 64), plan.offsets[2])
    assert cover.min() == 1 and cover.max() == 1


def _umma_cost(it, two_sweeps):
    chunks = int(it["nch"]) if it["nch"] else (int(it["N"]) + 255) // 256
    rows = min(int(it["M"]) - int(it["tm"]) * 128, 128)
    work = (2 * chunks if two_sweeps and chunks > 2 else chunks) * (4 + (int(it["K"]) + 63) // 64)
    return (work << 36) + (int(it["N"]) << 8) + rows


@pytest.mark.parametrize("softmax", [False, True])
@pytest.mark.parametrize("mode", ["mixed", "long", "ragged", "deep"])
def test_tcgen05_items_address_their_operands_and_come_heaviest_first(mode, softmax):
    rs = np.random.RandomState(100 + MODES.index(mode))
    S = 10 if mode in ("long", "deep") else 200
    M, N, K = (np.asarray(x, np.int64) for x in _batch(mode, rs, S))
    plan = GemmPlan(M, N, K, 2, torch.float16, softmax=softmax)
    a1, a2, ao = plan.offsets
    items, va, vb = plan.table("umma_items"), plan.table("umma_views_a"), plan.table("umma_views_b")
    assert items.size > 0 and 0 < va.size <= 24 and 0 < vb.size <= 24
    seg_of = {int(ao[s]): s for s in range(S) if M[s] > 0 and N[s] > 0}
    costs, gen = [], []
    for it in items:
        s = seg_of[int(it["offC"])]
        A, B = va[it["views"] & 255], vb[it["views"] >> 8]
        assert A["K"] == K[s] == B["K"] == it["K"] and A["residue"] < K[s] and A["residue"] % 8 == 0
        # row r of a view starts residue + r * K elements into the head strip
        assert A["residue"] + int(it["rowA"]) * K[s] == a1[s] + int(it["tm"]) * 128 * K[s]
        assert B["residue"] + int(it["rowB"]) * K[s] == a2[s]
        if softmax:
            assert it["nch"] == 0  # a fused softmax needs the whole row block
        costs.append(_umma_cost(it, softmax))
        gen.append((s, int(it["tm"]), int(it["ch0"])))
    for i in range(1, len(costs)):
        assert costs[i - 1] > costs[i] or (costs[i - 1] == costs[i] and gen[i - 1] < gen[i]), i
    if mode == "deep" and not softmax:
        assert (items["nch"] == 1).all()  # long contractions without softmax: one item per 128 x 256 tile


@pytest.mark.parametrize("attention", [False, True])
def test_packs_hold_contiguous_runs_within_their_limits(attention):
    rs = np.random.RandomState(3 + attention)
    S = 700
    n = np.clip(np.rint(rs.normal(25, 12, S)), 1, 64).astype(np.int64)
    m = n.copy()
    m[::7] = np.clip(m[::7] + rs.randint(-5, 6, m[::7].size), 1, 64)  # some rectangular segments
    if attention:
        plan = AttentionPlan(m, n, 4, torch.float16, d=64)
        a1 = np.concatenate([[0], np.cumsum(m * 64)]); a2 = np.concatenate([[0], np.cumsum(n * 64)]); ao = a1
        width = lambda s: 64
    else:
        plan = GemmPlan(m, n, np.full(S, 64), 4, torch.float16, softmax=True)
        a1, a2, ao = plan.offsets
        width = lambda s: int(n[s])
    packs, blocks = plan.table("packs"), plan.table("pack_blocks")
    assert packs.size > S // 16 and plan.summary["packs"] == packs.size
    assert blocks.size == sum(-(-int(x) // 16) for x in m) + PACK_BLOCKS
    assert not blocks[-PACK_BLOCKS:].view(np.uint8).any()   # the slack the kernel may read past the last pack
    rows_cap = PACK_ROWS_ATTN if attention else PACK_ROWS
    firstA = {int(a1[s]): s for s in range(S)}
    seen, cost_before, next_block = np.zeros(S, np.int32), None, 0
    for pk in packs:
        assert pk["first_block"] == next_block            # the tables follow the order of the packs
        next_block += int(pk["nblocks"])
        assert 0 < pk["rowsA"] <= rows_cap and 0 < pk["rowsB"] <= rows_cap and 0 < pk["nblocks"] <= PACK_BLOCKS
        # the pack is a run of consecutive segments, contiguous in both operands
        s0 = firstA[int(pk["offA"])]
        s1, ra, rb, cost = s0, 0, 0, 0.0
        members = {}
        while ra < pk["rowsA"]:
            members[s1] = (ra, rb)
            cost += float(m[s1] * n[s1] + (m[s1] + n[s1]) * 64)
            ra += int(m[s1]); rb += int(n[s1]); s1 += 1
        assert ra == pk["rowsA"] and rb == pk["rowsB"] and pk["offB"] == a2[s0]
        assert cost_before is None or cost <= cost_before  # heaviest pack first
        cost_before = cost
        mine = blocks[pk["first_block"]:pk["first_block"] + pk["nblocks"]]
        assert (mine["nblocks"] == pk["nblocks"]).all()
        assert (np.diff(mine["N"]) <= 0).all()            # widest blocks first
        rows_of = {s: 0 for s in members}
        for b in mine:
            s = max(k for k in members if ao[k] <= b["offC"])
            mb, rem = divmod(int(b["offC"] - ao[s]), 16 * width(s))
            assert rem == 0 and b["N"] == n[s] and b["M"] == min(16, m[s] - 16 * mb)
            assert b["rowA"] == members[s][0] + 16 * mb and b["rowB"] == members[s][1]
            rows_of[s] += int(b["M"])
        assert all(rows_of[s] == m[s] for s in members)
        seen[s0:s1] += 1
    assert (seen == 1).all()


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_softmax_chunks_and_windows(dtype):
    es = 2 if dtype == torch.float16 else 4
    rs = np.random.RandomState(11)
    rows = np.concatenate([rs.randint(0, 200, 60), rs.randint(1, 6, 10), [3, 1]])
    cols = np.concatenate([rs.randint(0, 900, 60), rs.randint(6000, 15000, 10), [WINDOW // es, WINDOW // es + 1]])
    gaps = rs.randint(0, 3, rows.size) * 5
    off = np.concatenate([[0], np.cumsum(rows * cols + gaps)])
    plan = SoftmaxPlan(rows, cols, 3, dtype, accum=off)
    chunks, windows = plan.table("softmax_chunks"), plan.table("softmax_windows")
    assert plan.summary["softmax_chunks"] == chunks.size
    cover = np.zeros(int(off[-1]), np.int32)
    for ch in chunks:
        nb = int(ch["rows"]) * int(ch["cols"]) * es
        assert ch["rows"] >= 1 and (nb <= WINDOW or ch["rows"] == 1)
        cover[int(ch["off"]):int(ch["off"]) + int(ch["rows"]) * int(ch["cols"])] += 1
    want = np.zeros_like(cover)
    for s in range(rows.size):
        want[int(off[s]):int(off[s]) + int(rows[s] * cols[s])] = 1
        first = chunks[chunks["off"] == off[s]]
        if rows[s] and cols[s]:
            assert first.size == 1 and first[0]["cols"] == cols[s]
            # as many whole rows as fit the window
            assert first[0]["rows"] == min(rows[s], max(1, WINDOW // es // cols[s]))
    assert np.array_equal(cover, want)
    nxt = 0
    for wd in windows:
        assert wd["first_piece"] == nxt and 1 <= wd["npieces"] <= 64
        mine = chunks[nxt:nxt + wd["npieces"]]
        nxt += int(wd["npieces"])
        assert wd["off"] == mine[0]["off"]
        sizes = mine["rows"].astype(np.int64) * mine["cols"] * es
        if wd["npieces"] == 1 and sizes[0] > WINDOW:
            assert wd["nbytes"] == WINDOW + 1              # a streamed row: only "longer than the window" matters
        else:
            assert wd["nbytes"] == sizes.sum() <= WINDOW
            ends = mine["off"] + mine["rows"].astype(np.int64) * mine["cols"]
            assert np.array_equal(ends[:-1], mine["off"][1:])   # the pieces of a window are contiguous
    assert nxt == chunks.size


def test_attention_items_cover_the_query_blocks_longest_sweeps_first():
    rs = np.random.RandomState(9)
    M = np.concatenate([rs.randint(1, 65, 40), rs.randint(65, 900, 25), [0]])
    N = np.concatenate([rs.randint(1, 65, 40), rs.randint(1, 900, 25), [7]])
    for d in (64, 128):
        plan = AttentionPlan(M, N, 2, torch.bfloat16, d=d)
        items, packs = plan.table("flash_items"), plan.table("packs")
        q0 = np.concatenate([[0], np.cumsum(M)]); k0 = np.concatenate([[0], np.cumsum(N)])
        small = (M <= 64) & (N <= 64) & (M > 0)
        in_items = (M > 0) & ~(small & (d == 64))
        assert (packs.size > 0) == (d == 64)
        assert items.size == sum(-(-int(m) // 128) for m in M[in_items])
        assert (np.diff(items["N"]) <= 0).all()
        rows = np.zeros(int(q0[-1]), np.int32)
        for it in items:
            s = int(np.searchsorted(q0, it["rowQ"], side="right") - 1)
            while M[s] == 0:
                s += 1
            assert in_items[s] and it["rowKV"] == k0[s] and it["N"] == N[s]
            assert (it["rowQ"] - q0[s]) % 128 == 0 and it["M"] == M[s] - (it["rowQ"] - q0[s])
            rows[int(it["rowQ"]):int(it["rowQ"]) + min(int(it["M"]), 128)] += 1
        want = np.zeros_like(rows)
        for s in np.nonzero(in_items)[0]:
            want[int(q0[s]):int(q0[s + 1])] = 1
        assert np.array_equal(rows, want)


@pytest.mark.parametrize("name", ["long_tail", "molecular", "general_gemm"])
def test_benchmark_batches_are_covered(name):
    w = workload(name, segments=96 if name == "long_tail" else 400)
    plan = GemmPlan(w.M, w.N, w.K, 1, torch.float16, torch.float32 if name == "general_gemm" else torch.float16,
                    softmax=name != "general_gemm")
    cover = _gemm_cover(plan, np.asarray(w.M), np.asarray(w.N), plan.offsets[2])
    assert cover.min() == 1 and cover.max() == 1


def test_table_names_and_refusals():
    plan = GemmPlan([3], [4], [5], 1, torch.float16)
    for name in TABLES:
        plan.table(name)
    from blockedattention_b200 import _lib as L
    import ctypes as C
    n = C.c_int64()
    assert L.lib.blk_plan_table(plan._h, 99, None, 0, C.byref(n), None) == L.BLK_ERR_INVALID
    buf = (C.c_char * 8)()
    assert L.lib.blk_plan_table(plan._h, 0, buf, 8, C.byref(n), None) == L.BLK_ERR_INVALID and n.value == 40
