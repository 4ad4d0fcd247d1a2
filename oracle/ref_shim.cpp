// TEST INFRASTRUCTURE ONLY -- never linked into, imported by or called from the product.
//
// Python binding for the upstream project's own CUDA launchers, so that the GPU
// parity tests can compare the new kernels with the original WMMA kernels on
// the same inputs.  The upstream translation units csrc/cuda/spBlkGEMM.cu and
// csrc/cuda/spBlkSoftmax.cu are compiled unmodified from where they lie; this
// file only replaces the upstream csrc/sparseBlockedAttention.cpp, whose
// pybind block is compiled out by a hard-coded macro
// (csrc/sparseBlockedAttention.h:10) and which defines a debugging main().
//
// Exposed functions take the arguments of the launchers declared at
// csrc/sparseBlockedAttention.h:18-21 in the same order.
#include "sparseBlockedAttention.h"

PYBIND11_MODULE(blk_ref_ext, m) {
    m.doc() = "upstream blockedAttention CUDA launchers (parity checker only)";
    m.def("gemm_launch", &sparseBlockedGEMMLaunch,
          "sparseBlockedGEMMLaunch(mat1, mat2, mat1Accum, mat2Accum, outAccum, MList, NList, KList, transpose1, transpose2)");
    m.def("softmax_launch", &sparseBlockedSoftmaxLaunch,
          "sparseBlockedSoftmaxLaunch(src, accumSrc, rowList, colList)");
    m.def("softmax_backward_launch", &sparseBlockedSoftmaxBackwardLaunch,
          "sparseBlockedSoftmaxBackwardLaunch(out, dout, accumSrc, rowList, colList)");
}
