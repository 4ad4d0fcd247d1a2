"""GPU, two ranks on two devices (skipped on a machine with one): the sharded run and the library's gather.

Each rank takes the segments `partition.shard` gives it, computes its share with the product kernels, and
`partition.gather_output` (grouped NCCL send/recv, strips received in place) must rebuild, on every rank, the packed
head-major result a single process produces, bit for bit.  Ranks are child processes; NVLS is off and nothing waits
across ranks inside a kernel.
"""
import os
import subprocess
import sys

import pytest
import torch

from helpers import ROOT

pytestmark = pytest.mark.gpu

WORKER = r'''
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.environ["BLK_ROOT"])
from blockedattention_b200 import blockAttnScores, partition
from blockedattention_b200.synth import workload
rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dev = torch.device("cuda", rank)
dist.init_process_group("nccl", device_id=dev)
w = workload("long_tail", seed=3, segments=40)
q, k = w.make_inputs("cpu", seed=0)
a1 = np.concatenate([[0], np.cumsum(w.M * w.K)])
for kind in ("balanced", "scattered"):
    if kind == "balanced":
        owner, info = partition.shard(w.M, w.N, w.K, w.H, world)
    else:
        owner = (np.arange(w.S) // 3 % world).astype(np.int32)      # what the longest-processing-time fallback looks like
    mine = np.nonzero(owner == rank)[0]
    ql = torch.cat([q[:, a1[s]:a1[s + 1]] for s in mine], dim=1).to(dev)
    kl = torch.cat([k[:, a1[s]:a1[s + 1]] for s in mine], dim=1).to(dev)
    local = blockAttnScores(ql, kl, w.M[mine], w.N[mine], w.K[mine], scale=w.scale)
    full = partition.gather_output(local, w.M * w.N, owner, w.H)
    ref = blockAttnScores(q.to(dev), k.to(dev), w.M, w.N, w.K, scale=w.scale)
    torch.cuda.synchronize()
    assert full.shape == ref.shape and torch.equal(full, ref), kind
dist.barrier()
dist.destroy_process_group()
print("rank", rank, "ok")
'''


def test_two_gpu_shard_and_gather_rebuild_the_single_process_result(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, BLK_ROOT=ROOT, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", str(29600 + os.getpid() % 300), str(script)],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "rank 0 ok" in r.stdout and "rank 1 ok" in r.stdout
