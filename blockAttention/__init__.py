"""Import-name alias of the upstream extension module ``blockAttention``
(setup.py:16): the two operators the upstream pybind block exports
(csrc/sparseBlockedAttention.cpp:134-137), with the C++ argument order of
csrc/sparseBlockedAttention.cpp:118-131."""
from blockedattention_b200.apply import blockGEMM as _gemm, blockSoftmax as _softmax


def sparseBlockedGEMM(mat1, mat2, mat1Accum=None, mat2Accum=None, outAccum=None, MList=None, NList=None,
                      KList=None, transpose1=False, transpose2=False):
    """sparseBlockedGEMM forward (csrc/sparseBlockedAttention.cpp:118-125)."""
    return _gemm(mat1, mat2, mat1Accum, mat2Accum, outAccum, MList, NList, KList, transpose1, transpose2)


def sparseBlockedSoftmax(src, rowList=None, colList=None, srcAccum=None):
    """sparseBlockedSoftmax forward (csrc/sparseBlockedAttention.cpp:127-131): (src, rowList, colList, srcAccum)."""
    return _softmax(src, rowList, colList, srcAccum)
