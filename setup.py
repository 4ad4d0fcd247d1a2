"""Install of the same two import names the upstream package provides (upstream setup.py:15-31):
``blockedAttention`` (operators ``blockGEMM`` / ``blockSoftmax``) and the extension-module name
``blockAttention`` (``sparseBlockedGEMM`` / ``sparseBlockedSoftmax``: the compiled torch extension
``blockAttention/_C``, a shim over the C-ABI library).  ``blockedattention_b200/build.py`` builds the
library ``lib/libblkattn.so`` with nvcc for sm_100a and the extension with g++ during ``build_py``;
both ship as package data.

    python setup.py build_py          # or: pip install --no-build-isolation .
"""
import os
import runpy

from setuptools import setup
from setuptools.command.build_py import build_py

ROOT = os.path.dirname(os.path.realpath(__file__))


class BuildWithLibrary(build_py):
    def run(self):
        # the build script runs without importing the package (which would look for the library it is about to make)
        b = runpy.run_path(os.path.join(ROOT, "blockedattention_b200", "build.py"))
        b["build"]()
        b["build_extension"]()
        super().run()


setup(
    name="blockedAttention",
    version="0.1.0",
    description="Varlen blocked GEMM and row softmax for NVIDIA B200 (sm_100a) behind the blockedAttention operator API",
    python_requires=">=3.9",
    install_requires=[],
    packages=["blockedattention_b200", "blockedAttention", "blockAttention"],
    package_data={"blockedattention_b200": ["lib/libblkattn.so"], "blockAttention": ["_C*.so"]},
    cmdclass={"build_py": BuildWithLibrary},
)
