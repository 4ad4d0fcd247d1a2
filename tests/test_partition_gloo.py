"""CPU, world size 2 over gloo: the sharded path -- every rank takes its
contiguous range of the balanced split, computes its share (with the CPU oracle
standing in for the kernels, which need a GPU) and the gathered strips rebuild
the single-process result bit for bit; offsets rebased per rank stay exact."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import O, ROOT


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from blockedattention_b200 import partition as P
        from blockedattention_b200.plan import GemmPlan
        from blockedattention_b200.synth import workload
        import blk_oracle as Or
        w = workload("molecular", seed=3, segments=96)
        w.H = 2
        cost = P.segment_cost(w.M, w.N, w.K, w.H)
        bounds = P.partition_contiguous(cost, world)
        lo, hi = int(bounds[rank]), int(bounds[rank + 1])
        assert (lo, hi) == P.shard_range(w.M, w.N, w.K, w.H, rank, world)
        q, k = w.make_inputs("cpu", seed=0)                       # same seed on every rank: same global batch
        a1, a2, ao = Or.offsets_from_lists(w.M, w.N, w.K)
        # the rank's strips are plain slices of the packed buffers
        ql = q[:, a1[lo]:a1[hi]].contiguous(); kl = k[:, a2[lo]:a2[hi]].contiguous()
        plan = GemmPlan(w.M[lo:hi], w.N[lo:hi], w.K[lo:hi], w.H, w.dtype, softmax=True)   # schedule only, no GPU
        r1, r2, ro = plan.offsets
        assert np.array_equal(r1, a1[lo:hi + 1] - a1[lo]) and np.array_equal(ro, ao[lo:hi + 1] - ao[lo])
        mine = Or.block_scores(ql, kl, w.M[lo:hi], w.N[lo:hi], w.K[lo:hi], scale=w.scale)
        sizes = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(sizes, torch.tensor([mine.shape[1]]))
        parts = [torch.zeros((w.H, int(s)), dtype=mine.dtype) for s in sizes]
        # unequal strip lengths: gather by broadcast from each owner
        for r in range(world):
            buf = mine.clone() if r == rank else parts[r]
            dist.broadcast(buf, src=r)
            parts[r] = buf
        full = torch.cat(parts, dim=1)
        ref = Or.block_scores(q, k, w.M, w.N, w.K, scale=w.scale)
        assert torch.equal(full, ref)
        # the library's gather: every rank ends with the single-process (H, Dout) layout, strips received in place
        owner, info = P.shard(w.M, w.N, w.K, w.H, world)
        assert info["kind"] == "contiguous" and info["bounds"] == [int(b) for b in bounds]
        got = P.gather_output(mine, w.M * w.N, owner, w.H)
        assert got.shape == ref.shape and torch.equal(got, ref)
        # an ownership that is not contiguous (what the longest-processing-time fallback produces)
        owner2 = (np.arange(w.S) // 5 % world).astype(np.int32)
        idx = np.nonzero(owner2 == rank)[0]
        ql2 = torch.cat([q[:, a1[s]:a1[s + 1]] for s in idx], dim=1)
        kl2 = torch.cat([k[:, a2[s]:a2[s + 1]] for s in idx], dim=1)
        mine2 = Or.block_scores(ql2, kl2, w.M[idx], w.N[idx], w.K[idx], scale=w.scale)
        got2 = P.gather_output(mine2, w.M * w.N, owner2, w.H)   # 20 runs: the all-gather path, unequal strips padded
        assert torch.equal(got2, ref)
        # a few runs that are not one range per rank: still point to point
        owner3 = (np.arange(w.S) // 24 % world).astype(np.int32)
        assert len(list(P._runs(owner3))) <= P.GATHER_MAX_RUNS_PER_RANK * world
        idx = np.nonzero(owner3 == rank)[0]
        ql3 = torch.cat([q[:, a1[s]:a1[s + 1]] for s in idx], dim=1)
        kl3 = torch.cat([k[:, a2[s]:a2[s + 1]] for s in idx], dim=1)
        mine3 = Or.block_scores(ql3, kl3, w.M[idx], w.N[idx], w.K[idx], scale=w.scale)
        assert torch.equal(P.gather_output(mine3, w.M * w.N, owner3, w.H), ref)
        # a heavy-tailed batch sends shard() to the fallback
        heavy = np.array([4, 4, 4, 4, 2000, 4, 4, 1500], np.int64)
        o3, i3 = P.shard(heavy, heavy, np.full(8, 64), 1, world, max_imbalance=1.0)
        assert i3["kind"] in ("contiguous", "lpt") and len(o3) == 8 and set(o3.tolist()) <= set(range(world))
        # timing reduction the benchmark uses: max over ranks
        t = torch.tensor([float(rank + 1)])
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        assert float(t) == world
        open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_two_rank_sharded_path(tmp_path):
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert sorted(os.listdir(tmp_path)) == ["ok0", "ok1"]
