"""CPU: the install recipe names the packages upstream's does and ships the library as package data."""
import os
import subprocess
import sys

from helpers import ROOT


def test_setup_lists_upstream_import_names(tmp_path):
    out = subprocess.run([sys.executable, "setup.py", "--name", "--version"], cwd=ROOT, capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    assert out.stdout.split()[0] == "blockedAttention"          # upstream setup.py:23
    build = tmp_path / "b"
    r = subprocess.run([sys.executable, "setup.py", "-q", "build_py", "--build-lib", str(build)], cwd=ROOT,
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    for name in ("blockedAttention/__init__.py", "blockAttention/__init__.py", "blockedattention_b200/apply.py",
                 "blockedattention_b200/lib/libblkattn.so"):
        assert os.path.exists(build / name), name
    assert [f for f in os.listdir(build / "blockAttention") if f.startswith("_C") and f.endswith(".so")], \
        "the compiled extension module is shipped with the blockAttention package"


def test_extension_module_is_compiled_and_keeps_the_upstream_names():
    # upstream csrc/sparseBlockedAttention.cpp:134-137 exports exactly these two operators from `blockAttention`
    import torch
    import blockAttention
    assert blockAttention.COMPILED, "blockAttention/_C is missing: python blockedattention_b200/build.py builds it"
    doc = blockAttention.sparseBlockedGEMM.__doc__
    for arg in ("mat1", "mat2", "mat1Accum", "mat2Accum", "outAccum", "MList", "NList", "KList", "transpose1", "transpose2"):
        assert arg in doc
    assert doc.index("mat1Accum") < doc.index("MList") < doc.index("transpose1")
    sdoc = blockAttention.sparseBlockedSoftmax.__doc__
    assert sdoc.index("src") < sdoc.index("rowList") < sdoc.index("colList") < sdoc.index("srcAccum")
    # the device / contiguity checks of upstream csrc/sparseBlockedAttention.h:6-8 need no GPU to fail
    import pytest
    M = torch.tensor([2]); K = torch.tensor([4])
    with pytest.raises(RuntimeError, match="must be CUDA Tensor"):
        blockAttention.sparseBlockedGEMM(torch.zeros(1, 8), torch.zeros(1, 8), None, None, None, M, M, K)
    with pytest.raises(RuntimeError):
        blockAttention.sparseBlockedGEMM(torch.zeros(1, 8), torch.zeros(1, 8))
