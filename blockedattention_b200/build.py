"""Builds ``blockedattention_b200/lib/libblkattn.so`` for sm_100a with nvcc.

The library is built in-tree (no JIT cache) so that it travels with the source
tree.  ``build()`` also compiles the torch-extension module ``blockAttention/_C``
(``csrc/sparseBlockedAttention.cpp``: the upstream extension's two operators as
a shim over the library) with g++ against the installed torch.  ``python blockedattention_b200/build.py`` rebuilds what is out of date (run it
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
           "blk_softmax.cu", "blk_softmax_pipe.cu", "blk_gemm_umma.cu", "blk_scores_pipe.cu", "blk_attn_umma.cu", "blk_pv_umma.cu"]
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


def build_extension(force: bool = False, verbose: bool = False) -> str:
    """``blockAttention/_C<ext suffix>``: the pybind/torch module with upstream's operator names, linked against
    libtorch and ``libblkattn.so`` only (no kernels of its own, so g++ compiles it)."""
    import sysconfig

    import torch
    from torch.utils import cpp_extension as ce

    src = os.path.join(CSRC, "sparseBlockedAttention.cpp")
    deps = [src, os.path.join(CSRC, "sparseBlockedAttention.h"), os.path.join(ROOT, "include", "blkattn.h")]
    outdir = os.path.join(ROOT, "blockAttention")
    target = os.path.join(outdir, "_C" + sysconfig.get_config_var("EXT_SUFFIX"))
    obj = os.path.join(OBJ, "sparseBlockedAttention.cpp.o")
    if not force and not _stale(target, deps + [LIB]):
        return target
    os.makedirs(OBJ, exist_ok=True)
    incs = ce.include_paths("cuda") + [sysconfig.get_paths()["include"], os.path.join(ROOT, "include"), CSRC]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-w", f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DTORCH_EXTENSION_NAME=_C",
           "-DTORCH_API_INCLUDE_EXTENSION_H", *[f"-I{p}" for p in incs], "-c", src, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
    if r.returncode:
        raise RuntimeError("g++ failed on sparseBlockedAttention.cpp")
    libdirs = ce.library_paths("cuda")
    link = ["g++", "-shared", "-o", target, obj, f"-L{LIBDIR}", "-lblkattn",
            "-Wl,-rpath,$ORIGIN/../blockedattention_b200/lib", *[f"-L{p}" for p in libdirs],
            *[f"-Wl,-rpath,{p}" for p in libdirs], "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch",
            "-ltorch_python", "-lcudart"]
    r = subprocess.run(link, capture_output=True, text=True)
    if r.returncode:
        sys.stderr.write(" ".join(link) + "\n" + r.stdout + r.stderr)
        raise RuntimeError("link of blockAttention/_C failed")
    return target


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--no-extension", action="store_true", help="build the C-ABI library only")
    a = ap.parse_args(argv)
    print(build(a.force, a.verbose))
    if not a.no_extension:
        print(build_extension(a.force, a.verbose))
    return 0


if __name__ == "__main__":
    sys.exit(main())
