/*
 * blkattn.h -- C ABI of libblkattn: variable-length blocked GEMM and
 * variable-length row softmax over packed, head-major buffers, for NVIDIA
 * B200 (sm_100a).
 *
 * Layout (upstream blockedAttention/apply.py:12-23, :31-39): every operand is
 * a 2-D buffer (H, D).  Head h owns the strip [h*D, (h+1)*D); inside a strip
 * segment s starts at element offset accum[s] and is a dense row-major
 * matrix: mat1 (M_s, K_s) [or (K_s, M_s) if transpose1], mat2 (N_s, K_s)
 * [or (K_s, N_s) if transpose2], out (M_s, N_s); softmax blocks are
 * (rows_s, cols_s).  Offsets and lists are int64.
 *
 * Every function returns BLK_OK (0) or a negative blk_status_t; none throws.
 * blk_last_error() gives a thread-local message for the last failure.
 * "host" pointers are ordinary memory; "dev" pointers are CUDA device memory
 * of the device the plan was created on.  Inputs are borrowed, outputs are
 * caller-allocated.  Plan creation allocates (cudaMalloc) and uploads the
 * schedule once; blk_*_run only launch kernels on the given stream and
 * neither allocate nor synchronise.
 */
#ifndef BLKATTN_H_
#define BLKATTN_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define BLK_API __attribute__((visibility("default")))
#else
#define BLK_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    BLK_OK = 0,
    BLK_ERR_INVALID = -1,     /* bad argument / inconsistent lists or offsets   */
    BLK_ERR_CUDA = -2,        /* a CUDA runtime call failed                      */
    BLK_ERR_UNSUPPORTED = -3, /* dtype / shape outside what the kernels cover   */
    BLK_ERR_UNALIGNED = -4,   /* a device pointer is not 16-byte aligned         */
    BLK_ERR_NOMEM = -5,
    BLK_ERR_TIMEOUT = -6      /* a bounded device-side wait gave up              */
} blk_status_t;

typedef enum { BLK_F16 = 0, BLK_BF16 = 1, BLK_F32 = 2 } blk_dtype_t;

/* What the GEMM writes. */
typedef enum {
    BLK_EPI_SCORES = 0,  /* out = scale * A B^T                                  */
    BLK_EPI_SOFTMAX = 1  /* out = softmax_rows(scale * A B^T), never materialising the scores */
} blk_epilogue_t;

typedef struct blk_plan blk_plan_t;

BLK_API const char* blk_last_error(void);
BLK_API const char* blk_version(void);

/* ---- index helpers (host only, no CUDA) ---------------------------------- */

/* accum1 = cumsum([0, M*K]), accum2 = cumsum([0, N*K]), accumOut = cumsum([0, M*N]);
 * each output has S+1 entries.  Replaces the cat+cumsum at upstream
 * csrc/sparseBlockedAttention.cpp:22-29. */
BLK_API int blk_offsets_from_lists(const int64_t* M, const int64_t* N, const int64_t* K, int64_t S,
                           int64_t* accum1, int64_t* accum2, int64_t* accumOut);

/* accum = cumsum([0, rows*cols]) (S+1 entries).  Replaces upstream
 * csrc/sparseBlockedAttention.cpp:85-91. */
BLK_API int blk_softmax_offsets(const int64_t* rows, const int64_t* cols, int64_t S, int64_t* accum);

/* Inverse: M = sqrt(mk*mn/nk), N = mn/M, K = mk/M from consecutive differences
 * of the three offset arrays.  Replaces the float32 formula at upstream
 * csrc/sparseBlockedAttention.cpp:30-40 with exact integer arithmetic: same
 * values wherever the upstream formula is self-consistent, BLK_ERR_INVALID
 * where no integer (M,N,K) exists or a segment is empty. */
BLK_API int blk_lists_from_offsets(const int64_t* accum1, const int64_t* accum2, const int64_t* accumOut,
                           int64_t S, int64_t* M, int64_t* N, int64_t* K);

/* ---- multi-GPU partitioning (host only, no CUDA) -------------------------- */

/* Per-segment cost = H * max(flops / flops_per_s, bytes / bytes_per_s) with
 * flops = 2 M N K and bytes = (M+N) K in_bytes + M N out_bytes.  No upstream
 * counterpart (the upstream project is single-GPU). */
BLK_API int blk_segment_cost(const int64_t* M, const int64_t* N, const int64_t* K, int64_t S, int64_t H,
                     int in_bytes, int out_bytes, double flops_per_s, double bytes_per_s,
                     double* cost);

/* Split segments [0,S) into R contiguous ranges [bounds[r], bounds[r+1])
 * minimising the largest range cost (bounds has R+1 entries). */
BLK_API int blk_partition_contiguous(const double* cost, int64_t S, int R, int64_t* bounds);

/* Longest-processing-time greedy: owner[s] in [0,R).  Use when the best
 * contiguous split is too far off balance. */
BLK_API int blk_partition_lpt(const double* cost, int64_t S, int R, int32_t* owner);

/* ---- varlen blocked GEMM --------------------------------------------------- */

/* Builds the segment schedule for one (lists, offsets, dtype, flags) problem.
 * Replaces the host tiling at upstream csrc/cuda/spBlkGEMM.cu:943-983 and the
 * dispatch at :826-941.  M,N,K: host, S entries.  accum1/accum2/accumOut:
 * host, S+1 entries, or all three NULL for the packed offsets of
 * blk_offsets_from_lists.  device >= 0: the CUDA device that will run the
 * plan (tables are uploaded there); device = -1: schedule only, for
 * inspection on a machine without a GPU (blk_*_run then fails).
 * dtype_in: BLK_F16 / BLK_BF16 / BLK_F32.  dtype_out: any of the three for
 * 16-bit inputs, BLK_F32 for BLK_F32 inputs.  epilogue: blk_epilogue_t. */
BLK_API int blk_gemm_plan_create(blk_plan_t** plan,
                         const int64_t* M, const int64_t* N, const int64_t* K,
                         const int64_t* accum1, const int64_t* accum2, const int64_t* accumOut,
                         int64_t S, int64_t H, int dtype_in, int dtype_out,
                         int transpose1, int transpose2, int epilogue, int device);

/* out(H, Dout) = epilogue(scale * mat1 mat2^T) per segment and head.
 * Replaces upstream sparseBlockedGEMMLaunch, csrc/cuda/spBlkGEMM.cu:985-1033
 * (declared csrc/sparseBlockedAttention.h:18), and with BLK_EPI_SOFTMAX also
 * the following sparseBlockedSoftmaxLaunch call.  mat1, mat2, out: dev
 * pointers, 16-byte aligned, H strips of Dm1 / Dm2 / Dout elements.  Elements
 * of out between segments (if the offsets leave gaps) are not written. */
BLK_API int blk_gemm_run(const blk_plan_t* plan, const void* mat1, const void* mat2, void* out,
                 float scale, void* cuda_stream);

/* blk_gemm_run for operands that are not packed head-major strips: element
 * (head h, row r, k) of mat1 is at mat1[r * row_stride1 + h * head_stride1 + k],
 * r counting the rows of all segments in batch order (same for mat2); strides
 * in elements, multiples of 8.  A token-major [rows, H, d] tensor, the layout
 * attention inputs usually have before upstream's callers permute them into
 * strips, is row_stride = H * d, head_stride = d.  The result is packed
 * head-major as always.  Only batches whose every segment runs on a kernel
 * that fetches operands through tensor maps qualify: 16-bit inputs, not
 * transposed, packed offsets, one contraction length d that is a multiple of
 * 8 (with d = 32, a batch with hundreds of segments of at most 64 rows and
 * columns runs those on a kernel that reads packed strips only and is
 * refused); otherwise BLK_ERR_UNSUPPORTED.  No counterpart upstream. */
BLK_API int blk_gemm_run_strided(const blk_plan_t* plan, const void* mat1, int64_t row_stride1, int64_t head_stride1,
                         const void* mat2, int64_t row_stride2, int64_t head_stride2, void* out, float scale,
                         void* cuda_stream);

/* ---- fused attention --------------------------------------------------------- */

/* out_s = softmax_rows(scale * Q_s K_s^T) V_s for segments of at most 64 query
 * rows and 64 key rows, head dimension 64, fp16 or bf16, in one kernel: the
 * scores and probabilities stay in registers.  q (H, sum M_s * 64), k and v
 * (H, sum N_s * 64) and out (H, sum M_s * 64) are packed head-major strips like
 * the operands of blk_gemm_run.  Equals, up to the rounding of the
 * probabilities that the two-call form stores in between,
 *   P = blk_gemm_run(BLK_EPI_SOFTMAX)(q, k);  out = blk_gemm_run(P, v; lists (M, 64, N), transpose2).
 * Any other batch gets BLK_ERR_UNSUPPORTED from the plan call: compose the two
 * operators for it.  No counterpart upstream (upstream materialises P). */
BLK_API int blk_attention_plan_create(blk_plan_t** plan, const int64_t* M, const int64_t* N, int64_t S, int64_t H,
                              int dtype, int device);
/* The same operator for any batch: segments of any length (M_s >= 0 queries,
 * N_s >= 1 keys where M_s > 0), head dimension 64 or 128.  At head dimension
 * 64 the segments the kernel above can take run on it (a first launch); every
 * other segment -- every segment at head dimension 128 -- runs on one tcgen05 kernel that
 * sweeps a segment's keys and values in tiles of 128 rows with an online
 * softmax, the scores in tensor memory and the probabilities written over them
 * for the second product: neither is ever stored.  q (H, sum M_s * d),
 * k, v (H, sum N_s * d), out (H, sum M_s * d).  Replaces the upstream chain
 * blockGEMM -> blockSoftmax -> blockGEMM (blockedAttention/apply.py:6-41,
 * test/pytest.py:35-38) where its result feeds the product with V.
 * blk_plan_summary reports this kernel's work items in counts[3]. */
BLK_API int blk_attention_plan_create_dim(blk_plan_t** plan, const int64_t* M, const int64_t* N, int64_t S, int64_t H,
                                  int64_t head_dim, int dtype, int device);
BLK_API int blk_attention_run(const blk_plan_t* plan, const void* q, const void* k, const void* v, void* out,
                      float scale, void* cuda_stream);
/* The same for q, k, v and out that are not packed strips: row r (counted over
 * all segments in batch order) of head h of each of the four tensors starts at
 * element r * row_stride + h * head_stride; strides in elements, multiples of 8.
 * Token-major [rows, H, d] tensors -- the layout attention layers hold their
 * activations in -- are row_stride = H * d, head_stride = d: no permuted copy
 * on the way in or out. */
BLK_API int blk_attention_run_strided(const blk_plan_t* plan, const void* q, const void* k, const void* v, void* out,
                              int64_t row_stride, int64_t head_stride, float scale, void* cuda_stream);

/* ---- varlen row softmax ---------------------------------------------------- */

/* Replaces the per-row host table at upstream csrc/cuda/spBlkSoftmax.cu:358-373
 * and the kernel choice at :389-396.  rows, cols: host, S entries; accum:
 * host, S+1 entries or NULL for packed.  No limit on cols. */
BLK_API int blk_softmax_plan_create(blk_plan_t** plan, const int64_t* rows, const int64_t* cols,
                            const int64_t* accum, int64_t S, int64_t H, int dtype, int device);

/* out = softmax_rows(scale * src), fp32 arithmetic, one rounding to dtype.
 * Replaces upstream sparseBlockedSoftmaxLaunch, csrc/cuda/spBlkSoftmax.cu:375-416
 * (declared csrc/sparseBlockedAttention.h:20).  src may equal out. */
BLK_API int blk_softmax_run(const blk_plan_t* plan, const void* src, void* out, float scale,
                    void* cuda_stream);

/* Backward of blk_softmax_run: grad_src = scale * (grad_out - rowsum(out *
 * grad_out)) * out, with `out` the forward result, fp32 arithmetic, one
 * rounding to dtype; `plan` is the forward call's plan.  Replaces upstream
 * sparseBlockedSoftmaxBackwardLaunch, csrc/cuda/spBlkSoftmax.cu:418-459
 * (declared csrc/sparseBlockedAttention.h:21; upstream has no scale, i.e.
 * scale = 1).  grad_src may equal grad_out. */
BLK_API int blk_softmax_backward_run(const blk_plan_t* plan, const void* out, const void* grad_out,
                             void* grad_src, float scale, void* cuda_stream);

/* The row softmax for callers that cannot allocate device memory when they
 * need it: a host whose runtime owns all device memory through its own arena,
 * a plugin running inside another component's pool, a caller that must not
 * stall other streams (cudaMalloc and cudaFree synchronise the device).  No
 * plan: rows and cols are host lists (packed offsets), and the chunk table a
 * plan would upload into allocated memory goes into a fixed 1 MB array that
 * every GPU loading the library carries until exit.  Limit: the batch may need
 * at most 65536 chunks (a chunk covers up to 12 KB of one head's rows; a row
 * longer than 12 KB is one chunk) -- larger batches get BLK_ERR_UNSUPPORTED,
 * decided from the lists before anything is built, and should use the plan
 * entry points.  The call performs no cudaMalloc/cudaFree: it copies the table
 * with cudaMemcpyAsync from ordinary host memory (the runtime stages that copy
 * before the call returns, which may wait for earlier work on the stream) and
 * launches on cuda_stream.  A stream that is being captured is refused with
 * BLK_ERR_UNSUPPORTED, nothing issued.  The first call on each device also
 * resolves the array's device address, so make that first call outside any
 * stream capture, with the device current.  All calls on a device share the
 * one array: calls whose GPU work may overlap (different streams, no
 * dependency between them) race on it; calls on one stream are safe.  src/out
 * as for blk_softmax_run.  This entry point has no counterpart in the upstream
 * project. */
BLK_API int blk_softmax_noalloc(const void* src, void* out, const int64_t* rows, const int64_t* cols,
                        int64_t S, int64_t H, int dtype, float scale, void* cuda_stream);

/* ---- plan queries ---------------------------------------------------------- */

BLK_API void blk_plan_destroy(blk_plan_t* plan);

/* D extents in elements (what upstream reads back with .item() at
 * csrc/cuda/spBlkGEMM.cu:996-998 and csrc/cuda/spBlkSoftmax.cu:381).  For a
 * softmax plan Dm1 = Dout = D and Dm2 = 0. */
BLK_API int blk_plan_extents(const blk_plan_t* plan, int64_t* Dm1, int64_t* Dm2, int64_t* Dout);

/* Copies the plan's offsets (S+1 entries each; any pointer may be NULL).
 * These are the bit-exact index outputs of the boundary. */
BLK_API int blk_plan_offsets(const blk_plan_t* plan, int64_t* accum1, int64_t* accum2, int64_t* accumOut);

/* Schedule summary: counts[0] = segments, [1] = work items of the packed
 * small-segment kernel, [2] = tiles of the staged mma.sync kernel, [3] = tiles
 * of the tcgen05 kernel, [4] = softmax chunks, [5] = kernels launched per
 * run, [6] = tiles of the fp32 SIMT kernel, [7] = packs of the pipelined
 * small-segment kernel (0 unless it was enabled). */
BLK_API int blk_plan_summary(const blk_plan_t* plan, int64_t counts[8]);

/* The schedule itself, for tests and debugging: copies the host copy of one of the plan's tables into dst
 * (capacity bytes; dst may be NULL to ask for the size only), *bytes = size of the table, *record_bytes = size of
 * one record.  The record layouts are the library's own (csrc/blk_internal.h) and may change between versions; no
 * run-time caller needs them. */
typedef enum {
    BLK_TABLE_SEGMENTS = 0,      /* BlkSeg: one per segment, batch order */
    BLK_TABLE_TILE_ITEMS = 1,    /* BlkTileItem: staged mma.sync kernel */
    BLK_TABLE_SIMT_ITEMS = 2,    /* BlkTileItem: fp32 SIMT kernel */
    BLK_TABLE_SMALL_ITEMS_32 = 3,/* BlkSmallItem: per-warp small-segment kernel, at most 32 columns */
    BLK_TABLE_SMALL_ITEMS_64 = 4,/* BlkSmallItem: ... 33 to 64 columns */
    BLK_TABLE_UMMA_ITEMS = 5,    /* BlkUmmaItem: tcgen05 kernel, in the order the CTAs take them */
    BLK_TABLE_PV_ITEMS = 6,      /* BlkPvItem: tcgen05 kernel for (K, D) second operands */
    BLK_TABLE_PACKS = 7,         /* BlkPack: pipelined small-segment kernel */
    BLK_TABLE_PACK_BLOCKS = 8,   /* BlkPackBlock */
    BLK_TABLE_SMX_CHUNKS = 9,    /* BlkSmxChunk */
    BLK_TABLE_SMX_WINDOWS = 10,  /* BlkSmxWindow */
    BLK_TABLE_FLASH_ITEMS = 11,  /* BlkFlashItem: tcgen05 attention kernel */
    BLK_TABLE_UMMA_VIEWS_A = 12, /* BlkUmmaView: views of the first operand the tcgen05 items refer to */
    BLK_TABLE_UMMA_VIEWS_B = 13  /* BlkUmmaView: ... of the second operand */
} blk_table_t;
BLK_API int blk_plan_table(const blk_plan_t* plan, int table, void* dst, int64_t capacity, int64_t* bytes,
                           int64_t* record_bytes);

/* Algorithmic work of one run over all heads: flops = 2 H sum(M N K) (0 for a
 * softmax plan), bytes = inputs read once + outputs written once. */
BLK_API int blk_plan_work(const blk_plan_t* plan, double* flops, double* bytes);

/* Kernel-side status word of the plan's device (0 = fine).  Synchronises the
 * stream it is given. */
BLK_API int blk_plan_check(const blk_plan_t* plan, void* cuda_stream);

#ifdef __cplusplus
}
#endif
#endif /* BLKATTN_H_ */
