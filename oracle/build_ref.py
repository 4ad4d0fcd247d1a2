"""Build recipe for ``oracle/_ref/blk_ref_ext*.so`` (TEST INFRASTRUCTURE ONLY).

Compiles the upstream CUDA translation units ``csrc/cuda/spBlkGEMM.cu`` and
``csrc/cuda/spBlkSoftmax.cu`` for sm_100a, unmodified and from where they lie,
plus ``oracle/ref_shim.cpp`` (a pybind binding of the launchers declared at
``csrc/sparseBlockedAttention.h:18-20``).  Nothing is copied into this
repository; objects and the shared library go to ``oracle/_ref/`` only, which
is git-ignored.  The upstream build system (setup.py / CMake) is not run.

Usage: ``python oracle/build_ref.py --ref /path/to/upstream/checkout`` (or the
environment variable ``BLK_REFERENCE_DIR``); without either nothing is built.
The result needs a GPU to do anything; it is used by the ``-m gpu`` parity
tests as a second checker beside the CPU oracle.
"""
import argparse
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("BLK_REFERENCE_DIR", ""))
    ap.add_argument("--force", action="store_true")
    args = ap.parse_args(argv)
    ref = args.ref
    if not ref or not os.path.isdir(os.path.join(ref, "csrc", "cuda")):
        print(f"no upstream checkout given (--ref or BLK_REFERENCE_DIR; got {ref!r}); nothing built")
        return 0
    import torch
    from torch.utils import cpp_extension as ce

    os.makedirs(OUT, exist_ok=True)
    ext_suffix = sysconfig.get_config_var("EXT_SUFFIX")
    target = os.path.join(OUT, "blk_ref_ext" + ext_suffix)
    srcs = [os.path.join(ref, "csrc", "cuda", "spBlkGEMM.cu"),
            os.path.join(ref, "csrc", "cuda", "spBlkSoftmax.cu"),
            os.path.join(HERE, "ref_shim.cpp")]
    if (not args.force and os.path.exists(target)
            and all(os.path.getmtime(target) >= os.path.getmtime(s) for s in srcs)):
        print("up to date:", target)
        return 0
    incs = ce.include_paths("cuda") + [sysconfig.get_paths()["include"],
                                       os.path.join(ref, "csrc"), os.path.join(ref, "csrc", "cuda")]
    inc_flags = [f"-I{p}" for p in incs]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    common = ["-std=c++17", "-O2", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
              "-DTORCH_EXTENSION_NAME=blk_ref_ext", "-DTORCH_API_INCLUDE_EXTENSION_H"]
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")

    def compile_one(src):
        obj = os.path.join(OUT, os.path.basename(src) + ".o")
        if src.endswith(".cu"):
            cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "--expt-relaxed-constexpr",
                   "-Xcompiler", "-fPIC", "-w", *common, *inc_flags, "-c", src, "-o", obj]
        else:
            cmd = ["g++", "-fPIC", "-w", *common, *inc_flags, "-c", src, "-o", obj]
        print(" ".join(cmd), flush=True)
        subprocess.check_call(cmd)
        return obj

    with ThreadPoolExecutor(3) as ex:
        objs = list(ex.map(compile_one, srcs))
    libdir = ce.library_paths("cuda")
    link = ["g++", "-shared", "-o", target, *objs, *[f"-L{p}" for p in libdir],
            *[f"-Wl,-rpath,{p}" for p in libdir],
            "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"]
    print(" ".join(link), flush=True)
    subprocess.check_call(link)
    print("built", target)
    return 0


if __name__ == "__main__":
    sys.exit(main())
