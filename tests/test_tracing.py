"""CPU: the library opens a named NVTX range around plan creation (and around every run; those need a GPU).  A small
injection library compiled here stands in for a profiler and records the ranges."""
import os
import shutil
import subprocess
import sys

import pytest

from helpers import ROOT

HERE = os.path.dirname(os.path.abspath(__file__))
CUDA_INC = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")

CHILD = """
import numpy as np, torch
from blockedattention_b200.plan import AttentionPlan, GemmPlan, SoftmaxPlan
GemmPlan([40, 300], [50, 300], [64, 64], 2, torch.float16, softmax=True)
SoftmaxPlan([5, 7], [9, 11], 2, torch.float16)
AttentionPlan([30, 200], [30, 200], 2, torch.bfloat16, d=64)
"""


@pytest.mark.skipif(shutil.which("gcc") is None or not os.path.exists(os.path.join(CUDA_INC, "nvtx3", "nvToolsExt.h")),
                    reason="needs gcc and the NVTX headers")
@pytest.mark.parametrize("switch", [None, "0"])
def test_plan_creation_is_an_nvtx_range(tmp_path, switch):
    so = tmp_path / "libnvtx_recorder.so"
    subprocess.run(["gcc", "-shared", "-fPIC", "-O1", f"-I{CUDA_INC}", os.path.join(HERE, "nvtx_recorder.c"), "-o", str(so)],
                   check=True)
    log = tmp_path / "ranges.txt"
    env = dict(os.environ, NVTX_INJECTION64_PATH=str(so), NVTX_RECORD_FILE=str(log), PYTHONPATH=ROOT)
    env.pop("BLK_NVTX", None)
    if switch is not None:
        env["BLK_NVTX"] = switch
    r = subprocess.run([sys.executable, "-c", CHILD], env=env, capture_output=True, text=True, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = log.read_text().split("\n") if log.exists() else []
    mine = [ln for ln in lines if ln.startswith("push blk_")]
    if switch == "0":
        assert mine == []
        return
    assert mine == ["push blk_gemm_plan_create", "push blk_softmax_plan_create", "push blk_attention_plan_create"]
    # every range is closed before the next opens
    seq = [ln.split()[0] for ln in lines if ln.startswith("push blk_") or ln.startswith("pop")]
    depth = 0
    for what in seq:
        depth += 1 if what == "push" else -1
        assert 0 <= depth <= 1
    assert depth == 0
