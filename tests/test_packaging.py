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
