"""GPU: the CUDA path against the committed golden vectors (tests/golden/*.npz)."""
import os

import pytest
import torch

from helpers import assert_probs_close, assert_scores_close
from test_oracle import GOLDEN, load_golden
from blockedattention_b200.plan import AttentionPlan, GemmPlan, SoftmaxPlan

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_cuda_matches_golden(cuda_device, path):
    d = load_golden(path)
    dev = cuda_device
    dt = d["torch_dtype"]
    if str(d["kind"]) == "gemm":
        plan = GemmPlan(d["M"], d["N"], d["K"], int(d["H"]), dt, None, bool(d["ta"]), bool(d["tb"]),
                        bool(d["softmax"]), device=dev)
        a1, a2, ao = plan.offsets
        assert (a1 == d["a1"]).all() and (a2 == d["a2"]).all() and (ao == d["ao"]).all()   # bit-exact index outputs
        out = plan.run(d["A"].to(dev), d["B"].to(dev), scale=float(d["scale"]))
        if bool(d["softmax"]):
            assert_probs_close(out, d["out"], path)
        else:
            assert_scores_close(out, d["out"], path)
            if "arange" in path:   # integer-valued fp32 answers come out exactly
                assert torch.equal(out.cpu(), d["out"])
    elif str(d["kind"]) == "attention":
        plan = AttentionPlan(d["M"], d["N"], int(d["H"]), dt, device=dev, d=int(d["d"]))
        out = plan.run(d["A"].to(dev), d["B"].to(dev), d["X"].to(dev), scale=float(d["scale"]))
        plan.check()
        want = d["out"]
        tol = (2e-3 if dt == torch.float16 else 1.6e-2) * max(1.0, float(want.abs().max()))
        assert float((out.float().cpu() - want).abs().max()) <= tol, path
    else:
        plan = SoftmaxPlan(d["rows"], d["cols"], int(d["H"]), dt, device=dev)
        assert (plan.offsets == d["acc"]).all()
        assert_probs_close(plan.run(d["X"].to(dev)), d["out"], path)
