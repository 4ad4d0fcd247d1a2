"""The upstream extension module ``blockAttention`` (upstream setup.py:16): ``sparseBlockedGEMM`` and
``sparseBlockedSoftmax`` with the C++ argument order of upstream csrc/sparseBlockedAttention.cpp:118-131.

The operators are the compiled torch extension ``blockAttention._C`` (``blockedattention_b200/csrc/
sparseBlockedAttention.cpp``, a shim over ``libblkattn``), built by ``python blockedattention_b200/build.py``.
Only where that module has not been built do the names fall back to the Python operators of
``blockedattention_b200`` (same library underneath); ``COMPILED`` tells which one is in use."""
try:
    from ._C import (sparseBlockedGEMM, sparseBlockedGEMMLaunch, sparseBlockedSoftmax,  # noqa: F401
                     sparseBlockedSoftmaxBackwardLaunch, sparseBlockedSoftmaxLaunch)
    COMPILED = True
except ImportError:
    COMPILED = False
    from blockedattention_b200.apply import blockGEMM as _gemm, blockSoftmax as _softmax

    def sparseBlockedGEMM(mat1, mat2, mat1Accum=None, mat2Accum=None, outAccum=None, MList=None, NList=None,
                          KList=None, transpose1=False, transpose2=False):
        """sparseBlockedGEMM forward (csrc/sparseBlockedAttention.cpp:118-125)."""
        return _gemm(mat1, mat2, mat1Accum, mat2Accum, outAccum, MList, NList, KList, transpose1, transpose2)

    def sparseBlockedSoftmax(src, rowList=None, colList=None, srcAccum=None):
        """sparseBlockedSoftmax forward (csrc/sparseBlockedAttention.cpp:127-131): (src, rowList, colList, srcAccum)."""
        return _softmax(src, rowList, colList, srcAccum)
