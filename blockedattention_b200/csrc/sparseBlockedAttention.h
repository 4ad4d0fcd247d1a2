// Torch-extension boundary of the upstream project, kept by name and signature, over libblkattn.
//
// Upstream's extension module `blockAttention` exports two operators, sparseBlockedGEMM and sparseBlockedSoftmax
// (upstream csrc/sparseBlockedAttention.cpp:118-138), which sit on three launchers declared at upstream
// csrc/sparseBlockedAttention.h:18-21.  This header declares the same five functions with the same argument
// lists; sparseBlockedAttention.cpp implements them as a thin layer over the C ABI of include/blkattn.h (plans
// cached per list set, kernels on torch's current stream, the tensor's device made current).  Nothing here
// contains a kernel: the only link dependencies are libtorch and libblkattn.
#pragma once
#include <torch/extension.h>

#include <optional>

// out(H, Dout) = mat1 mat2^T per segment and head, dtype of the inputs (upstream sparseBlockedGEMMLaunch,
// csrc/cuda/spBlkGEMM.cu:985-1033).  Offsets and lists: int64 tensors on any device.
torch::Tensor sparseBlockedGEMMLaunch(const torch::Tensor& mat1, const torch::Tensor& mat2, const torch::Tensor& mat1Accum,
                                      const torch::Tensor& mat2Accum, const torch::Tensor& outAccum,
                                      const torch::Tensor& MList, const torch::Tensor& NList, const torch::Tensor& KList,
                                      const bool transpose1 = false, const bool transpose2 = false);

// Row softmax of every packed block (upstream sparseBlockedSoftmaxLaunch, csrc/cuda/spBlkSoftmax.cu:375-416).
torch::Tensor sparseBlockedSoftmaxLaunch(const torch::Tensor& src, const torch::Tensor& accumSrc,
                                         const torch::Tensor& rowList, const torch::Tensor& colList);

// (dout - rowsum(out * dout)) * out (upstream sparseBlockedSoftmaxBackwardLaunch, csrc/cuda/spBlkSoftmax.cu:418-459).
torch::Tensor sparseBlockedSoftmaxBackwardLaunch(const torch::Tensor& out, const torch::Tensor& dout,
                                                 const torch::Tensor& accumSrc, const torch::Tensor& rowList,
                                                 const torch::Tensor& colList);

// The two exported operators (upstream csrc/sparseBlockedAttention.cpp:118-131): either the three offset tensors or
// the three lists may be absent and are then derived from the others; both carry autograd history.
torch::Tensor sparseBlockedGEMM_op(const torch::Tensor& mat1, const torch::Tensor& mat2,
                                   const std::optional<torch::Tensor>& mat1Accum,
                                   const std::optional<torch::Tensor>& mat2Accum,
                                   const std::optional<torch::Tensor>& outAccum, const std::optional<torch::Tensor>& MList,
                                   const std::optional<torch::Tensor>& NList, const std::optional<torch::Tensor>& KList,
                                   const bool transpose1, const bool transpose2);
torch::Tensor sparseBlockedSoftmax_op(const torch::Tensor& src, const std::optional<torch::Tensor>& rowList,
                                      const std::optional<torch::Tensor>& colList,
                                      const std::optional<torch::Tensor>& srcAccum);
