"""Builds ``blockedattention_b200/lib/libblkattn.so`` for sm_100a with nvcc.

The library is built in-tree (no JIT cache) so that it travels with the source
tree.  ``python blockedattention_b200/build.py`` rebuilds what is out of date (run it
as a script: importing the package first would load the old library);
``--force`` rebuilds everything; ``--verbose`` adds ``-Xptxas -v``.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "build")
LIBDIR = os.path.join(PKG, "lib")
LIB = os.path.join(LIBDIR, "libblkattn.so")

SOURCES = ["blk_host.cpp", "blk_api.cu", "blk_gemm_tile.cu", "blk_gemm_simt.cu", "blk_scores_small.cu",
           "blk_softmax.cu", "blk_softmax_pipe.cu", "blk_gemm_umma.cu", "blk_scores_pipe.cu", "blk_attn_umma.cu"]
GENCODE = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc() -> str:
    return os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")


def _headers():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    hs.append(os.path.join(ROOT, "include", "blkattn.h"))
    return hs


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    os.makedirs(LIBDIR, exist_ok=True)
    hdrs = _headers()
    common = ["-std=c++17", "-O3", "-lineinfo", f"-I{os.path.join(ROOT, 'include')}", f"-I{CSRC}",
              "-Xcompiler", "-fPIC,-Wall,-fvisibility=hidden", "--expt-relaxed-constexpr",
              "-DBLK_BUILDING_LIB"]
    if verbose:
        common += ["-Xptxas", "-v"]

    def compile_one(src):
        path = os.path.join(CSRC, src)
        obj = os.path.join(OBJ, src + ".o")
        if force or _stale(obj, [path] + hdrs):
            cmd = [_nvcc(), *GENCODE, *common, "-x", "cu", "-c", path, "-o", obj]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if verbose or r.returncode:
                sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
            if r.returncode:
                raise RuntimeError(f"nvcc failed on {src}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(SOURCES))) as ex:
        objs = list(ex.map(compile_one, SOURCES))
    if force or _stale(LIB, objs):
        cmd = [_nvcc(), *GENCODE, "-shared", "-o", LIB, *objs, "-cudart", "static"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return LIB


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args(argv)
    print(build(a.force, a.verbose))
    return 0


if __name__ == "__main__":
    sys.exit(main())
