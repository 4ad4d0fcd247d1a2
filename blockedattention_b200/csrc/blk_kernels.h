// Kernel parameter blocks and launcher prototypes (internal).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "blk_internal.h"

struct BlkGemmParams {
    const uint16_t* A;
    const uint16_t* B;
    void* C;
    const BlkSeg* segs;
    const BlkTileItem* items;
    int64_t Dm1, Dm2, Dout;
    int num_items;
    int H;
    int out_f32;
    int epi;
    float scale;
};

struct BlkSimtParams {
    const float* A;
    const float* B;
    float* C;
    const BlkSeg* segs;
    const BlkTileItem* items;
    int64_t Dm1, Dm2, Dout;
    int num_items;
    int H;
    int ta, tb;
    float scale;
};

struct BlkSmallParams {
    const uint16_t* A;
    const uint16_t* B;
    void* C;
    const BlkSmallItem* items;
    int64_t Dm1, Dm2, Dout;
    int num_items;
    int H;
    int out_f32;
    int epi;
    float scale;
};

struct BlkUmmaParams {
    void* C;
    const BlkUmmaItem* items;
    int64_t Dout;
    int num_items;
    int H;
    int K;
    int bf16;
    int out_f32;
    int epi;
    float scale;
    int* status;
};

struct BlkPackParams {
    const uint16_t* A;
    const uint16_t* B;
    void* C;
    const BlkPack* packs;
    const BlkPackBlock* blocks;
    int64_t Dm1, Dm2, Dout;
    int num_packs;
    int H;
    int epi;
    float scale;
    int* status;
};

struct BlkSmxParams {
    const void* src;
    void* dst;
    const BlkSmxChunk* chunks;
    int64_t D;
    int num_chunks;
    int H;
    float scale;
};

// Backward of the row softmax: grad_src = scale * (grad_out - rowsum(out * grad_out)) * out.
struct BlkSmxBwdParams {
    const void* out;       // forward result (probabilities)
    const void* grad_out;  // gradient with respect to the forward result
    void* grad_src;        // may alias grad_out
    const BlkSmxChunk* chunks;
    int64_t D;
    int num_chunks;
    int H;
    float scale;
};

// Tensor map (128-byte swizzle) over a packed 16-bit operand viewed as (k, row, head): K contiguous elements per
// row, D elements per head, boxes of box_k x box_rows x 1.  False when the driver's encoder is unavailable or
// rejects the view.  Defined in blk_gemm_umma.cu.
struct CUtensorMap_st;
bool blk_make_row_map(CUtensorMap_st* map, const void* base, int bf16, int64_t K, int64_t rows, int64_t H, int64_t D,
                      int box_k, int box_rows);

cudaError_t blk_launch_gemm_tile(const BlkGemmParams& p, int dtype_in, int ta, int tb, cudaStream_t st);
cudaError_t blk_launch_softmax_bwd(const BlkSmxBwdParams& p, int dtype, cudaStream_t st);
cudaError_t blk_launch_gemm_simt(const BlkSimtParams& p, cudaStream_t st);
cudaError_t blk_launch_scores_small(const BlkSmallParams& p, int dtype_in, int K, int bucket, int sms,
                                    cudaStream_t st);
cudaError_t blk_launch_gemm_umma(const BlkUmmaParams& p, const void* A, const void* B, int64_t Dm1, int64_t Dm2,
                                 int sms, cudaStream_t st);
cudaError_t blk_launch_scores_pipe(const BlkPackParams& p, int dtype_in, int sms, cudaStream_t st);
cudaError_t blk_launch_softmax(const BlkSmxParams& p, int dtype, cudaStream_t st);
