// Kernel parameter blocks and launcher prototypes (internal).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "blk_internal.h"

// Where the rows of one 16-bit operand live: element (head h, row r, k) is at base[r * row_stride +
// h * head_stride + k].  Packed head-major strips: row_stride = K, head_stride = elements per strip;
// token-major [rows, H, K]: row_stride = H * K, head_stride = K.
struct BlkOperandLayout {
    int64_t rows;         // rows per head
    int64_t row_stride;   // elements
    int64_t head_stride;  // elements
};

struct BlkGemmParams {
    const uint16_t* A;
    const uint16_t* B;
    void* C;
    const BlkSeg* segs;
    const BlkTileItem* items;
    const BlkTileRec* recs;  // items[i] and its segment side by side
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
    int bf16;
    int out_f32;
    int epi;
    float scale;
    int* status;
    int head_firstA, head_firstB;  // coordinate order of the operands' tensor maps
    int long_rows;                 // some item has more than 512 columns (a fused softmax takes two sweeps there)
    // Test hook for the bounded waits: stall != 0 makes the producer role issue no copies at all (nothing is ever
    // in flight), so the first wait for operands runs out after spin_limit polls (0: the normal limit), the kernel
    // records BLK_ERR_TIMEOUT's status code and returns.
    int stall;
    uint32_t spin_limit;
};

struct BlkPvParams {
    const void* A;  // first operand: rows of K elements at arbitrary 2-byte offsets
    void* C;
    const BlkPvItem* items;
    int64_t Dm1, Dm2, Dout;
    int num_items;
    int H;
    int D;  // columns of the second operand and of the result: 64 or 128
    int bf16;
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
    BlkOperandLayout layA, layB;   // where the operands' rows are (filled by the caller)
    int head_firstA, head_firstB;  // coordinate order of the tensor maps (filled by the launcher)
    // attention variant (V != null): C receives softmax(scale A B^T) V, 64 columns per first-operand row
    const uint16_t* V;
    BlkOperandLayout layV;
    int head_firstV;
    int64_t out_row_stride, out_head_stride;  // elements; result row r of head h at C[h * head_stride + r * row_stride]
};

struct BlkFlashParams {
    void* out;
    const BlkFlashItem* items;
    int num_items;
    int H;
    int D;  // head dimension: 64 or 128
    int bf16;
    float scale;
    int* status;
    BlkOperandLayout layQ, layK, layV;
    int head_firstQ, head_firstK, head_firstV;  // coordinate order of the tensor maps (filled by the launcher)
    int64_t out_row_stride, out_head_stride;    // elements; result row r of head h at out[h * head_stride + r * row_stride]
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

// Tensor map (128-byte swizzle) over such an operand, boxes of box_k x box_rows of one head.  The dimension
// with the smaller stride comes second: *head_first = 0 means coordinates (k, row, head), 1 means (k, head, row).
// False when the driver's encoder is unavailable or rejects the view.  Defined in blk_gemm_umma.cu.
struct CUtensorMap_st;
bool blk_make_row_map(CUtensorMap_st* map, const void* base, int bf16, int64_t K, int64_t H, const BlkOperandLayout& lay,
                      int box_k, int box_rows, int* head_first);

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per kernel and device.  Defined in blk_gemm_umma.cu.
cudaError_t blk_func_smem(const void* kern, int bytes);

cudaError_t blk_launch_gemm_tile(const BlkGemmParams& p, int dtype_in, int ta, int tb, cudaStream_t st);
// Pipelined softmax kernels (blk_softmax_pipe.cu).  Forward: in0 = src, in1 unused; backward: in0 = forward
// result, in1 = its gradient (out may alias in1).
struct BlkSmxPipeParams {
    const void* in0;
    const void* in1;
    void* out;
    const BlkSmxWindow* windows;
    const BlkSmxChunk* pieces;
    int64_t D;
    int num_windows;
    int H;
    float scale;
    int* status;
};
cudaError_t blk_launch_softmax_pipe(const BlkSmxPipeParams& p, int dtype, int backward, int sms, cudaStream_t st);
cudaError_t blk_launch_gemm_simt(const BlkSimtParams& p, cudaStream_t st);
cudaError_t blk_launch_scores_small(const BlkSmallParams& p, int dtype_in, int K, int bucket, int sms,
                                    cudaStream_t st);
// An operand of the tcgen05 GEMM kernel: the buffer, the length of a head strip, and the views the plan's items refer
// to.  given != nullptr (strided operands): the one view, which starts at the buffer, has this layout instead of the
// packed one.
struct BlkUmmaOperand {
    const void* base;
    int64_t D;
    const BlkUmmaView* views;
    int num_views;
    const BlkOperandLayout* given;
};
cudaError_t blk_launch_gemm_umma(const BlkUmmaParams& p, const BlkUmmaOperand& A, const BlkUmmaOperand& B, int sms,
                                 cudaStream_t st);
cudaError_t blk_launch_pv_umma(const BlkPvParams& p, const void* V, int sms, cudaStream_t st);
cudaError_t blk_launch_attn_umma(const BlkFlashParams& p, const void* q, const void* k, const void* v, int sms,
                                 cudaStream_t st);
cudaError_t blk_launch_scores_pipe(const BlkPackParams& p, int dtype_in, int sms, cudaStream_t st);
cudaError_t blk_launch_softmax(const BlkSmxParams& p, int dtype, cudaStream_t st);
