// Internal declarations shared by the host scheduler and the kernels of
// libblkattn.  Not part of the public ABI (that is include/blkattn.h).
#pragma once
#include <stdint.h>
#include <string>
#include <vector>

#include "blkattn.h"

// ---- device-visible schedule records ---------------------------------------

// One segment of the packed batch.  Offsets are in elements inside a head
// strip.  cls is the widest access the kernels may use for this segment on
// every head: 2 -> 16-byte vectors, 1 -> 4-byte pairs, 0 -> single elements.
struct BlkSeg {
    int64_t offA, offB, offC;
    int32_t M, N, K;
    uint8_t clsIn;   // min over both inputs
    uint8_t clsOut;  // output
    uint8_t pad[2];
};
static_assert(sizeof(BlkSeg) == 40, "BlkSeg layout");

// One CTA of the staged mma.sync kernel: rows [tm*BM, ...) of segment seg and
// column tiles tn .. tn+ntn-1 (ntn > 1 only when the softmax epilogue sweeps
// the whole row).
struct BlkTileItem {
    int32_t seg;
    int32_t tm;
    int32_t tn;
    int32_t ntn;
};

// What a CTA of the staged mma.sync kernel reads first: its item and the item's segment in one 64-byte record, so
// that the operand addresses depend on one global load instead of two in a row.
struct BlkTileRec {
    BlkSeg sd;
    BlkTileItem it;
    int64_t pad;
};
static_assert(sizeof(BlkTileRec) == 64, "BlkTileRec layout");

// One warp of the packed small-segment kernel: a whole (segment, head) score
// block with N <= 64, K a multiple of 32, everything 16-byte aligned.
struct BlkSmallItem {
    int64_t offA, offB, offC;
    int32_t M, N;
};
static_assert(sizeof(BlkSmallItem) == 32, "BlkSmallItem layout");

// Pipelined small-segment kernel: a pack is a run of consecutive small segments whose first operands, and
// whose second operands, are each one contiguous piece of a head strip (<= BLK_PACK_ROWS rows), fetched by one
// bulk copy each; its blocks (<= BLK_PACK_BLOCKS) are the 16-row pieces of the segments' first operands.
struct BlkPack {
    int64_t offA, offB;  // element offsets of the run inside the head strips
    int32_t rowsA, rowsB;
    int32_t first_block, nblocks;
};
static_assert(sizeof(BlkPack) == 32, "BlkPack layout");
struct BlkPackBlock {
    int64_t offC;        // element offset of the block's output inside a head strip
    int32_t rowA, rowB;  // first row of the block inside the pack's operand runs
    int32_t M, N;
    int32_t nblocks;     // blocks in this pack (repeated in every record)
    int32_t pad;
};
static_assert(sizeof(BlkPackBlock) == 32, "BlkPackBlock layout");

// One CTA of the softmax kernel: `rows` consecutive rows of `cols` elements
// starting at element `off` of the head strip.  rows*cols fits the CTA's
// shared-memory window, or rows == 1 for a row longer than the window.
struct BlkSmxChunk {
    int64_t off;
    int32_t rows;
    int32_t cols;
};

// One window of the pipelined softmax kernels: npieces consecutive chunks (pieces) that are contiguous in
// memory and together at most BLK_SMX_WINDOW_BYTES long, or a single one-row piece longer than that.
struct BlkSmxWindow {
    int64_t off;          // element offset of the first piece inside the head strip
    int32_t nbytes;       // bytes of all pieces
    int32_t first_piece;  // index into the chunk table
    int32_t npieces;
    int32_t pad;
};
static_assert(sizeof(BlkSmxWindow) == 24, "BlkSmxWindow layout");
constexpr int BLK_SMX_WINDOW_PIECES = 64;  // pieces a window may hold

// The tcgen05 kernel reads an operand through (K, rows, heads) views of the packed buffer, one tensor map per view.
// A segment with contraction length K whose offset inside a head strip is r modulo K starts on row (offset - r) / K of
// the view that begins r elements into the strip, so a batch of several contraction lengths (or of offsets that are
// not whole rows of one view) needs a handful of views per operand; BLK_UMMA_VIEWS bounds them.
constexpr int BLK_UMMA_VIEWS = 24;
struct BlkUmmaView {
    int64_t K;        // row length = contraction length
    int64_t residue;  // elements from the start of a head strip to row 0 of the view (< K, a multiple of 8)
};

// Per-CTA tile of the tcgen05 kernel (filled in by the scheduler).
struct BlkUmmaItem {
    int32_t views;    // view of the first operand | view of the second << 8
    int32_t tm;       // 128-row block inside the segment
    int32_t rowA;     // first row of that block in its view of the first operand
    int32_t rowB;     // first row of the segment in its view of the second operand
    int64_t offC;     // element offset of the segment's output block
    int32_t M, N;     // extents of the whole segment
    int32_t K;        // contraction length
    int32_t ch0;      // first 256-column chunk of the item ...
    int32_t nch;      // ... and how many (0: all the chunks of the row block, which a fused softmax needs)
    int32_t pad;
};
static_assert(sizeof(BlkUmmaItem) == 48, "BlkUmmaItem layout");

// One work item of the tcgen05 kernel for the product with a (K, D) second operand (P V): a 128-row block of the
// first operand of one segment.
struct BlkPvItem {
    int64_t offA;   // element offset of the block's first row inside a head strip of the first operand
    int64_t offC;   // element offset of the block's first result row inside a head strip of the output
    int32_t rowB;   // first row of the segment in the (rows, D) view of the second operand
    int32_t M;      // rows of the segment from this block on (the block holds min(M, 128))
    int32_t K;      // contraction length = row pitch of the first operand
    int32_t pad;
};
static_assert(sizeof(BlkPvItem) == 32, "BlkPvItem layout");

// One work item of the fused attention kernel for long segments: a 128-row block of the queries of a segment.
struct BlkFlashItem {
    int32_t rowQ;   // first query row of the block in the (rows, d) view of q (and of the result)
    int32_t rowKV;  // first key / value row of the segment
    int32_t M;      // query rows of the segment from this block on (the block holds min(M, 128))
    int32_t N;      // key / value rows of the segment
};
static_assert(sizeof(BlkFlashItem) == 16, "BlkFlashItem layout");

// ---- kernel geometry constants the scheduler must agree with ----------------
constexpr int BLK_TILE_BM = 64;
constexpr int BLK_TILE_BN = 128;
constexpr int BLK_TILE_BK = 32;
constexpr int BLK_SIMT_BM = 64;
constexpr int BLK_SIMT_BN = 64;
constexpr int BLK_SMALL_MAXN = 64;
constexpr int BLK_SMALL_WARPS = 4;
constexpr int BLK_SMALL_MAXM = 64;
constexpr int BLK_SMALL_BUCKETS = 2;  // N <= 32, N <= 64
constexpr int BLK_PACK_ROWS = 192;    // rows of each operand a pack may hold
constexpr int BLK_PACK_ROWS_ATTN = 128;  // same for the attention variant, whose slots hold a third operand
constexpr int BLK_PACK_BLOCKS = 16;   // segments a pack may hold
// Shared-memory window of the softmax kernels: 12 KB lets eight CTAs of the pipelined forward kernel (two windows each)
// and four of the backward kernel (four) share an SM; with 16 KB and six / three the CTA-wide barriers of a window were
// hidden less well (5 to 10 % slower on every buffer but the longest rows).
constexpr int BLK_SMX_WINDOW_BYTES = 12288;
constexpr int BLK_UMMA_BM = 128;
constexpr int BLK_FLASH_BM = 128;
constexpr int BLK_NOALLOC_MAX_CHUNKS = 65536;  // entries of the built-in chunk table of blk_softmax_noalloc

// ---- the plan ----------------------------------------------------------------
struct blk_plan {
    int kind = 0;  // 0 GEMM, 1 softmax
    int64_t S = 0, H = 0;
    int dtype_in = 0, dtype_out = 0, ta = 0, tb = 0, epi = 0, device = -1;
    std::vector<int64_t> M, N, K, a1, a2, ao;
    int64_t Dm1 = 0, Dm2 = 0, Dout = 0;
    double flops = 0, bytes = 0;

    std::vector<BlkSeg> segs;
    std::vector<BlkTileItem> tile_items;    // staged mma.sync kernel (16-bit inputs)
    std::vector<BlkTileItem> simt_items;    // fp32 SIMT kernel
    std::vector<BlkSmallItem> small_items[BLK_SMALL_BUCKETS];  // packed small-segment kernel, by column count (empty when small_pipe)
    std::vector<BlkUmmaItem> umma_items;    // tcgen05 kernel
    std::vector<BlkPvItem> pv_items;        // tcgen05 kernel for transposed second operands of 64 or 128 columns
    int pv_D = 0;                           // columns of that second operand
    std::vector<BlkSmxChunk> smx_chunks;    // softmax kernel (also second pass of fp32 scores)
    std::vector<BlkSmxWindow> smx_windows;  // pipelined softmax kernels: groups of chunks
    int64_t max_chunks = 0;                 // > 0: the softmax scheduler refuses batches that need more chunks
    int umma_K = 0;                         // K of the tcgen05 bin when it has one view per operand that starts at the
                                            // strip (the only case the strided entry takes); 0: no such bin; -1: several views
    int umma_long_rows = 0;                 // a tcgen05 item has more than 512 columns
    std::vector<BlkUmmaView> umma_viewsA, umma_viewsB;  // views of the operands the tcgen05 items refer to
    int small_K = 0;                        // uniform K of the small bin
    int64_t small_segments = 0;             // segments of the small bin (as packs when small_pipe, else one item each)
    int small_pipe = 0;                     // 1: the small segments run as packs on the pipelined kernel
    int attn = 0;                           // attention plan (result = softmax(QK^T) V): 1 every segment in packs,
                                            // 2 every segment on the tcgen05 attention kernel
    int head_dim = 64;                      // attention plans: columns of q, k, v and result rows
    std::vector<BlkFlashItem> flash_items;
    BlkFlashItem* d_flash_items = nullptr;
    std::vector<BlkPack> packs;
    std::vector<BlkPackBlock> pack_blocks;
    BlkPack* d_packs = nullptr;
    BlkPackBlock* d_pack_blocks = nullptr;

    // device copies: pieces of the one allocation d_pool
    void* d_pool = nullptr;
    BlkSeg* d_segs = nullptr;
    BlkTileItem* d_tile_items = nullptr;
    BlkTileRec* d_tile_recs = nullptr;
    BlkTileItem* d_simt_items = nullptr;
    BlkSmallItem* d_small_items[BLK_SMALL_BUCKETS] = {nullptr, nullptr};
    int num_sms = 148;
    BlkUmmaItem* d_umma_items = nullptr;
    BlkPvItem* d_pv_items = nullptr;
    BlkSmxChunk* d_smx_chunks = nullptr;
    BlkSmxWindow* d_smx_windows = nullptr;
    int* d_status = nullptr;
    int* d_counter = nullptr;  // persistent-kernel tile counter
};

void blk_set_error(const std::string& msg);

// Host scheduling (blk_host.cpp) -- no CUDA calls.
int blk_build_gemm_schedule(blk_plan* p);
int blk_build_softmax_schedule(blk_plan* p);

// Environment overrides used by the benchmark harness to force a path:
// BLK_DISABLE_SMALL=1, BLK_DISABLE_UMMA=1.
bool blk_env_flag(const char* name);
