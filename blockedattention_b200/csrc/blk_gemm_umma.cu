// Large-segment kernel of the varlen blocked GEMM on the 5th-generation tensor
// cores: TMA-fed tcgen05.mma with the accumulator in tensor memory.
//
// A persistent CTA (one per SM; 22 warps for the two-sweep fused softmax, 14 otherwise) walks a static list of work
// items, an item being a 128-row block of one segment of one head (or one 256-column chunk of it).  Roles:
//   warp 0   producer: one lane issues 3-D tiled TMA loads (k, row, head) of a
//            128 x 64 tile of the first operand and a 256 x 64 tile of the
//            second into a 3-stage ring of 128-byte-swizzled shared memory;
//   warp 1   MMA: allocates the 512 tensor-memory columns, and one lane issues
//            tcgen05.mma (M = 128, N up to 256, K = 16 per instruction) into
//            one of two 256-column accumulators; tcgen05.commit hands shared
//            memory stages back to the producer and accumulators to the epilogue;
//   next 16 or 8 warps  epilogue arithmetic: a warp may read the 32 accumulator lanes (= rows)
//            of its quarter; the four or two warps of a quarter (SPLIT) each take an equal share of every
//            staged piece's columns and exchange partial row statistics through
//            shared memory.  A thread reads its row 32 columns at a time
//            (tcgen05.ld), applies the epilogue and writes the packed words into
//            one of the quarter's two strips (32 rows x 128 16-bit or 64 fp32 columns each, used
//            alternately), at the position the row has in global memory modulo
//            one 32-bit word;
//   last 4 warps  stores: one warp per quarter.  It waits for a strip to
//            be filled, writes its 32 rows to global memory -- a row piece is 256
//            contiguous bytes stored as two fully coalesced 128-byte word stores;
//            an odd first or last element goes out as a 16-bit store -- and hands
//            the strip back.  Keeping the stores in warps of their own matters:
//            a warp that alternates between exponentials and stores leaves the
//            special-function unit idle whenever the memory system pushes back
//            on its stores, and all warps of a CTA reach that point together;
//            with separate warps the exponentials of one piece run while the
//            previous piece drains.  Wide contiguous row pieces matter as well:
//            the same data written as 128-byte pieces with element-wise ragged
//            edges runs at little more than half the rate.
//
// Epilogues.  Scores: scale and round.  Softmax with N <= 512: both
// accumulators hold the whole row; pass 1 takes the row maximum, pass 2 writes
// exp2 back into tensor memory while summing, pass 3 normalises and stores, so
// the exponential is evaluated once per element and the scores never leave the
// SM.  Softmax with N > 512: the products are computed twice -- a first sweep
// over the 256-column chunks keeps only a running (max, sum) per row, a second
// sweep recomputes each chunk and stores normalised probabilities; when the CTA's next item is of the same kind and
// length, its first sweep is interleaved chunk by chunk with this item's second.
//
// Rows of the operand views past the end of a segment belong to its neighbour
// (or are zero-filled past the end of the buffer); they only reach accumulator
// rows/columns the epilogue never stores, and columns >= N are masked before
// any row reduction.
//
// Every wait on an mbarrier is bounded: when the bound is hit the kernel
// records a status code, all roles leave their loops, tensor memory is
// released and the kernel returns.
//
// Replaces upstream sparseBlockedHGEMM_half / _bf16 with the 128 x 128 x 16
// WMMA tile (csrc/cuda/spBlkGEMM.cu:424-817, :866-868) and, fused, the softmax
// kernels (csrc/cuda/spBlkSoftmax.cu:88-269).
#include <cuda.h>

#include <mutex>

#include "blk_device.cuh"
#include "blk_kernels.h"
#include "blk_umma_ptx.cuh"

namespace {

constexpr int UM_BM = BLK_UMMA_BM;      // 128 rows per work item
constexpr int UM_BN = 256;              // columns per accumulator
constexpr int UM_BK = 64;               // k elements per shared-memory stage (one 128-byte swizzle row)
constexpr int UM_STAGES = 3;
constexpr int UM_A_BYTES = UM_BM * UM_BK * 2;  // 16 KB
constexpr int UM_B_BYTES = UM_BN * UM_BK * 2;  // 32 KB
constexpr int UM_STAGE_BYTES = UM_A_BYTES + UM_B_BYTES;
// Arithmetic warps per accumulator-lane quarter (SPLIT, a template parameter of the kernel): four for the fused
// softmax over rows too long for tensor memory (each converts 32 of every 128 columns: with two warps per scheduler
// partition the special-function unit idles half the time in the two-sweep scheme), two otherwise -- rows that stay
// resident, scores only (both a few per cent faster with fewer, fatter warps) and fp32 results (a staged piece is 64
// columns there, and a warp's share must be whole 32-column loads).
constexpr int UM_SPLIT_MAX = 4;
constexpr int UM_STORE_WARPS = 4;                     // one per quarter
constexpr int um_threads(int split) { return 64 + 32 * (4 * split + UM_STORE_WARPS); }
constexpr int UM_PIECE = 32;                          // columns per tcgen05.ld
constexpr int UM_PW = 64;                             // 32-bit words of a staged row piece (128 x 16-bit, 64 x fp32)
// Strip row pitch in words: odd, so that the 32 row-owning lanes of a store (same word, consecutive rows) hit 32
// different banks; a row holds UM_PW words plus the half word an odd first element pushes past the end.
constexpr int UM_STRIP_PITCHW = UM_PW + 5;
constexpr int UM_STRIP_BYTES = 32 * UM_STRIP_PITCHW * 4;  // one strip; a quarter has two
// What the arithmetic warps tell the store warp about the piece in a strip.
struct UmPiece {
    int64_t g0;   // element index in the output of the piece's first element in the quarter's first row
    int32_t N;    // row pitch of the output block
    int32_t pcols;  // columns of the piece
    int32_t rows;   // rows of the quarter inside the block (0..32)
    int32_t halves; // a row may start or end on half a word
    int32_t stop;   // no more pieces: the store warp leaves
    int32_t pad;
};
static_assert(sizeof(UmPiece) == 32, "UmPiece layout");
constexpr int PCOLS16 = UM_PW * 2;                    // columns of a whole 16-bit piece
constexpr int UM_XCH_BYTES = 2 * 2 * UM_SPLIT_MAX * 128 * 4;  // row statistics exchanged between the two halves, double-buffered
constexpr int UM_SMEM_BYTES = UM_STAGES * UM_STAGE_BYTES + 8 * UM_STRIP_BYTES + UM_XCH_BYTES + 8 * 32 + 512;
static_assert(UM_SMEM_BYTES <= 227 * 1024, "shared memory budget");
static_assert(UM_STAGES <= 4, "barrier slots");

struct Work {
    BlkUmmaItem it;
    int head;
    int nchunks;
    int sweeps;
    int nkb;     // k-blocks of UM_BK; the last may be short (the tensor map fills what lies past K with zeros)
};

// The tensor maps of the operands' views (BlkUmmaView), passed as one kernel parameter.
struct UmMaps {
    CUtensorMap a[BLK_UMMA_VIEWS];
    CUtensorMap b[BLK_UMMA_VIEWS];
};

// Work w of a CTA's walk (w = blockIdx.x + k gridDim.x in round k).  Odd rounds run through the CTAs backwards, so
// that with the items sorted by cost no CTA always gets the heaviest of a round.  Only the last round can point past
// the end, so a CTA that gets nothing there has nothing left either.
__device__ __forceinline__ bool next_work(const BlkUmmaParams& p, uint32_t w, Work& wk) {
    const uint32_t total = (uint32_t)p.num_items * (uint32_t)p.H;
    const uint32_t round = w / gridDim.x;
    if (round & 1u) w = round * gridDim.x + (gridDim.x - 1u - (w - round * gridDim.x));
    if (w >= total) return false;
    const uint32_t item = w / (uint32_t)p.H;
    wk.head = (int)(w - item * (uint32_t)p.H);
    wk.it = p.items[item];
    wk.nchunks = wk.it.nch ? wk.it.nch : (wk.it.N + UM_BN - 1) / UM_BN;  // chunks [it.ch0, it.ch0 + nchunks)
    wk.nkb = (wk.it.K + UM_BK - 1) / UM_BK;
    wk.sweeps = (p.epi == BLK_EPI_SOFTMAX && wk.nchunks > 2) ? 2 : 1;
    return true;
}

// Two consecutive items of a CTA's walk pair up when both take the two-sweep softmax over the same number of chunks:
// then the first sweep of the later one (special-function bound, stores nothing) is interleaved chunk by chunk with the
// second sweep of the earlier one (bound by the stores).  nx receives the later item.
__device__ __forceinline__ bool pairs_with_next(const BlkUmmaParams& p, uint32_t w, const Work& wk, Work& nx) {
#ifdef UM_NO_PAIRING
    return false;
#else
    return wk.sweeps == 2 && next_work(p, w + gridDim.x, nx) && nx.sweeps == 2 && nx.nchunks == wk.nchunks;
#endif
}

// Predicated global stores as single instructions (no branch around them).
__device__ __forceinline__ void stg_b32_if(void* p, uint32_t v, bool ok) {
    asm volatile("{\n .reg .pred q;\n setp.ne.b32 q, %2, 0;\n @q st.global.b32 [%0], %1;\n}\n" ::"l"(p), "r"(v), "r"((int)ok)
                 : "memory");
}
__device__ __forceinline__ void stg_b16_if(void* p, uint32_t v, bool ok) {
    asm volatile("{\n .reg .pred q;\n setp.ne.b32 q, %2, 0;\n @q st.global.b16 [%0], %1;\n}\n" ::"l"(p), "h"((uint16_t)v),
                 "r"((int)ok)
                 : "memory");
}
__device__ __forceinline__ uint32_t lds_b32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.b32 %0, [%1];\n" : "=r"(v) : "r"(addr));
    return v;
}

template <typename Tag, bool OUT32, int SPLIT>
__global__ void __launch_bounds__(um_threads(SPLIT), 1)
blk_gemm_umma_kernel(const BlkUmmaParams p, const __grid_constant__ UmMaps maps) {
    extern __shared__ __align__(1024) unsigned char um_smem_raw[];  // the swizzled tiles need a 1024-byte aligned base
    unsigned char* smem = um_smem_raw;
    if (blk_smem_u32(smem) & 1023u) {  // cannot happen with the alignment above; checked because the swizzle relies on it
        if (threadIdx.x == 0) atomicCAS(p.status, 0, 9);
        return;
    }
    constexpr int UM_SPLIT = SPLIT;
    static_assert(!OUT32 || SPLIT == 2, "fp32 results: two arithmetic warps per quarter");
    constexpr int UM_EPI_WARPS = 4 * UM_SPLIT;
    unsigned char* strips = smem + UM_STAGES * UM_STAGE_BYTES;
    float* xch = reinterpret_cast<float*>(strips + 8 * UM_STRIP_BYTES);
    UmPiece* pieces_desc = reinterpret_cast<UmPiece*>(strips + 8 * UM_STRIP_BYTES + UM_XCH_BYTES);  // [quarter][strip]
    uint64_t* bars = reinterpret_cast<uint64_t*>(strips + 8 * UM_STRIP_BYTES + UM_XCH_BYTES + 8 * 32);
    // bars[0..3] full (UM_STAGES used), [4..7] empty, [8..9] tmem_full, [10..11] tmem_empty; per quarter q:
    // [16+q] rendezvous for the row statistics; per quarter and strip: [20 + 2q + b] strip filled, [28 + 2q + b] strip drained
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 13);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t smem_u32 = blk_smem_u32(smem);
    const uint32_t bar0 = blk_smem_u32(bars);
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (4 + s); };
    auto tfull_bar = [&](int b) { return bar0 + 8u * (8 + b); };
    auto tempty_bar = [&](int b) { return bar0 + 8u * (10 + b); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < UM_STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(tfull_bar(b), 1);
            mbar_init(tempty_bar(b), UM_EPI_WARPS);
        }
        *abort_flag = 0;
        for (int i = 0; i < 4; ++i) mbar_init(bar0 + 8u * (16 + i), UM_SPLIT);   // one arrival per arithmetic warp of the quarter
        for (int i = 0; i < 8; ++i) mbar_init(bar0 + 8u * (20 + i), UM_SPLIT);   // strip filled: the quarter's arithmetic warps
        for (int i = 0; i < 8; ++i) mbar_init(bar0 + 8u * (28 + i), 1);          // strip drained: its store warp
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(blk_smem_u32(tmem_slot)),
                     "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t lim = p.spin_limit ? p.spin_limit : BLK_UMMA_SPIN_LIMIT;

    if (warp == 0) {
        // ---------------- producer ----------------
        if (lane == 0 && !p.stall) {
            int stage = 0;
            uint32_t phase = 0;
            Work wk;
            bool ok = true;
            // the operand tiles of chunk ch of an item
            auto load_chunk = [&](const Work& k, int ch) {
                for (int kb = 0; kb < k.nkb; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, 1, lim)) { ok = false; return; }
                    const uint32_t sA = smem_u32 + stage * UM_STAGE_BYTES, sB = sA + UM_A_BYTES;
                    mbar_expect_tx(full_bar(stage), UM_STAGE_BYTES);
                    // coordinates (k, row, head), or (k, head, row) for a token-major operand
                    const int rA = k.it.rowA, rB = k.it.rowB + ch * UM_BN;
                    tma_load_3d(sA, &maps.a[k.it.views & 255], full_bar(stage), kb * UM_BK, p.head_firstA ? k.head : rA,
                                p.head_firstA ? rA : k.head);
                    tma_load_3d(sB, &maps.b[k.it.views >> 8], full_bar(stage), kb * UM_BK, p.head_firstB ? k.head : rB,
                                p.head_firstB ? rB : k.head);
                    if (++stage == UM_STAGES) { stage = 0; phase ^= 1u; }
                }
            };
            // the order of the chunks is that of the arithmetic warps (see there): first sweep (unless it ran alongside
            // the previous item), then the storing chunks, each followed by a first-sweep chunk of the next item when
            // the two items pair up
            Work nx;
            bool pre = false;
            for (uint32_t w = blockIdx.x; ok && next_work(p, w, wk); w += gridDim.x) {
                const bool pair = pairs_with_next(p, w, wk, nx);
                if (wk.sweeps == 2 && !pre)
                    for (int ch = 0; ok && ch < wk.nchunks; ++ch) load_chunk(wk, ch);
                for (int ch = wk.it.ch0; ok && ch < wk.it.ch0 + wk.nchunks; ++ch) {
                    load_chunk(wk, ch);
                    if (ok && pair) load_chunk(nx, ch);
                }
                pre = pair;
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issue ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0, slot = 0;
            Work wk;
            bool ok = true;
            // the products of chunk ch of an item into the next accumulator
            auto mma_chunk = [&](const Work& k, int ch) {
                const int buf = slot & 1;
                if (!mbar_wait(tempty_bar(buf), ((slot >> 1) & 1u) ^ 1u, abort_flag, p.status, 2, lim)) { ok = false; return; }
                tc_fence_after();
                const int ncols = min(k.it.N - ch * UM_BN, UM_BN);
                const uint32_t idesc = instr_desc(p.bf16, (ncols + 15) & ~15, p.epi == BLK_EPI_SOFTMAX && p.scale < 0.f);
                const uint32_t d_tmem = tmem_base + (uint32_t)(buf * UM_BN);
                for (int kb = 0; kb < k.nkb; ++kb) {
                    if (!mbar_wait(full_bar(stage), phase, abort_flag, p.status, 3, lim)) { ok = false; return; }
                    tc_fence_after();
                    const uint32_t sA = smem_u32 + stage * UM_STAGE_BYTES, sB = sA + UM_A_BYTES;
                    // steps of 16 along k in this block: all four, or as many as reach the end of a short last block
                    const int ksteps = min(UM_BK / 16, (k.it.K - kb * UM_BK + 15) / 16);
#pragma unroll
                    for (int j = 0; j < UM_BK / 16; ++j)
                        if (j < ksteps)
                            tc_mma_f16(d_tmem, smem_desc_sw128(sA + 32 * j), smem_desc_sw128(sB + 32 * j), idesc, (kb | j) != 0);
                    tc_commit(empty_bar(stage));  // stage reusable once these products have read it
                    if (++stage == UM_STAGES) { stage = 0; phase ^= 1u; }
                }
                tc_commit(tfull_bar(buf));
                ++slot;
            };
            Work nx;
            bool pre = false;
            for (uint32_t w = blockIdx.x; ok && next_work(p, w, wk); w += gridDim.x) {
                const bool pair = pairs_with_next(p, w, wk, nx);
                if (wk.sweeps == 2 && !pre)
                    for (int ch = 0; ok && ch < wk.nchunks; ++ch) mma_chunk(wk, ch);
                for (int ch = wk.it.ch0; ok && ch < wk.it.ch0 + wk.nchunks; ++ch) {
                    mma_chunk(wk, ch);
                    if (ok && pair) mma_chunk(nx, ch);
                }
                pre = pair;
            }
        }
    } else if (warp >= 2 + UM_EPI_WARPS) {
        // ---------------- stores: the last four warps, one per quarter ----------------
        const int sq = warp & 3;
        unsigned char* const C = reinterpret_cast<unsigned char*>(p.C);
        constexpr int ES = OUT32 ? 4 : 2;
        for (uint32_t n = 0;; ++n) {
            // the quarter's pieces in order, piece m from strip m & 1
            const int sb = (int)(n & 1u);
            const uint32_t use = n >> 1;   // how often the strip has been used before
            const uint32_t strip = blk_smem_u32(strips + (sq * 2 + sb) * UM_STRIP_BYTES);
            const uint32_t filled_bar = bar0 + 8u * (20 + sq * 2 + sb), drained_bar = bar0 + 8u * (28 + sq * 2 + sb);
            const volatile UmPiece* desc = pieces_desc + sq * 2 + sb;
            if (!mbar_wait(filled_bar, use & 1u, abort_flag, p.status, 10, lim)) break;
            if (desc->stop) break;
            const int64_t g0 = desc->g0;
            const int N = desc->N, pcols = desc->pcols, rows = desc->rows;
            const bool halves = desc->halves != 0;
            // lane l carries words l and l + 32 of a row: two stores of 128 contiguous bytes per row, four rows a batch
            const uint32_t rbase = strip + 4u * lane;
            if (!OUT32 && pcols == PCOLS16 && rows == 32) {
                // A whole piece (the common case), with as few instructions per row as it takes: the store warps share
                // their scheduler's issue slots with the arithmetic warps, and a row costing twenty instructions here
                // made the second sweep issue bound.  Row k starts at element g0 + k N: at word (t >> 1) past the word
                // of g0 with t = (g0 & 1) + k N, on its odd half when t is odd.  Words 1..63 of the row are whole; word 0
                // is whole when the row starts on an even element (its upper half goes out below otherwise), and so does
                // the lower half of word 64.
                uint32_t* const w0 = reinterpret_cast<uint32_t*>(C) + (g0 >> 1) + lane;
                uint32_t t = (uint32_t)(g0 & 1);
#pragma unroll 2
                for (int kb = 0; kb < 32; kb += 4) {
                    uint32_t v[4][2];
#pragma unroll
                    for (int k = 0; k < 4; ++k)
#pragma unroll
                        for (int i = 0; i < 2; ++i) v[k][i] = lds_b32(rbase + (uint32_t)(kb + k) * (UM_STRIP_PITCHW * 4) + 128u * i);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        uint32_t* wp = w0 + (t >> 1);
                        stg_b32_if(wp, v[k][0], lane >= (int)(t & 1u));
                        asm volatile("st.global.b32 [%0], %1;\n" ::"l"(wp + 32), "r"(v[k][1]) : "memory");
                        t += (uint32_t)N;
                    }
                }
            } else if (OUT32 && pcols == UM_PW && rows == 32) {
                // the same for a whole piece of fp32 results: row k is the 64 words from word g0 + k N on
                uint32_t* wp = reinterpret_cast<uint32_t*>(C) + g0 + lane;
#pragma unroll 2
                for (int kb = 0; kb < 32; kb += 4) {
                    uint32_t v[4][2];
#pragma unroll
                    for (int k = 0; k < 4; ++k)
#pragma unroll
                        for (int i = 0; i < 2; ++i) v[k][i] = lds_b32(rbase + (uint32_t)(kb + k) * (UM_STRIP_PITCHW * 4) + 128u * i);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        asm volatile("st.global.b32 [%0], %1;\n" ::"l"(wp), "r"(v[k][0]) : "memory");
                        asm volatile("st.global.b32 [%0], %1;\n" ::"l"(wp + 32), "r"(v[k][1]) : "memory");
                        wp += N;
                    }
                }
            } else if constexpr (OUT32) {
                // a partial piece of fp32 results (fewer rows or columns): the same walk with the bounds as predicates
                uint32_t* wp = reinterpret_cast<uint32_t*>(C) + g0 + lane;
#pragma unroll 2
                for (int kb = 0; kb < 32; kb += 4) {
                    if (kb >= rows) break;
                    uint32_t v[4][2];
#pragma unroll
                    for (int k = 0; k < 4; ++k)
#pragma unroll
                        for (int i = 0; i < 2; ++i) v[k][i] = lds_b32(rbase + (uint32_t)(kb + k) * (UM_STRIP_PITCHW * 4) + 128u * i);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const bool row_ok = kb + k < rows;
#pragma unroll
                        for (int i = 0; i < 2; ++i) stg_b32_if(wp + 32 * i, v[k][i], row_ok && lane + 32 * i < pcols);
                        wp += N;
                    }
                }
            } else
#pragma unroll 2
            for (int kb = 0; kb < 32; kb += 4) {
                if (kb >= rows) break;
                uint32_t v[4][2];
#pragma unroll
                for (int k = 0; k < 4; ++k)
#pragma unroll
                    for (int i = 0; i < 2; ++i) v[k][i] = lds_b32(rbase + (uint32_t)(kb + k) * (UM_STRIP_PITCHW * 4) + 128u * i);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int64_t gr = g0 + (int64_t)(kb + k) * N;
                    const int pr = OUT32 ? 0 : (int)(gr & 1);
                    const bool row_ok = kb + k < rows;
                    // whole words of the piece: [pr, (pr + pcols) / 2) for 16-bit elements, [0, pcols) for fp32
                    const int wl = OUT32 ? pcols : ((pr + pcols) >> 1);
                    uint32_t* wp = reinterpret_cast<uint32_t*>(C + (gr - pr) * ES);
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const int wi = lane + 32 * i;
                        stg_b32_if(wp + wi, v[k][i], row_ok && wi >= pr && wi < wl);
                    }
                }
            }
            if (!OUT32 && halves) {
                // half words at the ends: lane k the odd first element of row k, then the last element of row k when the
                // piece ends on half a word
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    const bool tail = t != 0;
                    const int64_t gr = g0 + (int64_t)lane * N;
                    const int pr = (int)(gr & 1);
                    const int endh = pr + pcols;                 // half words [pr, endh) of the row's words are the piece
                    const int wi = tail ? (endh >> 1) : 0;       // word that is only half inside the piece
                    const bool need = lane < rows && (tail ? (endh & 1) != 0 : pr != 0);
                    const uint32_t word = lds_b32(strip + (uint32_t)lane * (UM_STRIP_PITCHW * 4) + 4u * (need ? wi : 0));
                    unsigned char* dst = C + (gr - pr) * 2 + 4 * (int64_t)wi + (tail ? 0 : 2);
                    stg_b16_if(dst, tail ? (word & 0xffffu) : (word >> 16), need);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(drained_bar);
        }
    } else {
        // ---------------- epilogue arithmetic: warps 2 .. 2 + 4 SPLIT - 1 ----------------
        // lane quarter q = warp % 4 (the 32 accumulator lanes a warp may read); the SPLIT warps of a quarter split the
        // columns (share h: the columns c of a chunk with (c mod PC) / SH == h) and exchange their partial row
        // statistics.
        const int q = warp & 3, h = (warp - 2) >> 2;  // h in [0, UM_SPLIT)
        const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
        const int myrow = q * 32 + lane;
        uint32_t slot = 0, seq = 0;
        Work wk;
        bool ok = true;
        const bool softmax = p.epi == BLK_EPI_SOFTMAX;
        const float sl = softmax ? fabsf(p.scale) * BLK_LOG2E : p.scale;  // a negative softmax scale is applied by
                                                                          // the MMA (negated A), see instr_desc
        constexpr int ES = OUT32 ? 4 : 2;
        constexpr int PC = UM_PW * 4 / ES;   // columns of a staged row piece: 128 x 16-bit or 64 x fp32
        constexpr int SH = PC / UM_SPLIT;    // columns of a piece this warp converts (32 words)
        // Rendezvous of the two warps of a quarter: an mbarrier that one lane of each warp arrives on, waited for like
        // every other barrier (suspended, bounded), so that a warp whose partner gave up cannot wait for ever.
        const uint32_t stat_bar = bar0 + 8u * (16 + q);
        uint32_t stat_phase = 0;
        auto pair_sync = [&]() -> bool {
            __syncwarp();
            if (lane == 0) mbar_arrive(stat_bar);
            const bool good = mbar_wait(stat_bar, stat_phase, abort_flag, p.status, 8, lim);
            stat_phase ^= 1u;
            __syncwarp();
            return good;
        };
        uint32_t pieces = 0;  // pieces staged so far by this quarter: piece n goes into strip n & 1

        // Stage the piece of up to PC columns starting at column c0 of the 32 rows of this quarter for its store warp.
        // tcol(c) gives the tensor-memory column of row column c; pack(r, w) turns 32 raw accumulator words into
        // output words (32 fp32 words, or 16 words of 16-bit pairs); loaded() runs right after this warp's last
        // tensor-memory load of the piece, where the caller hands the accumulator back to the MMA role.  This warp
        // converts columns [c0 + h SH, c0 + (h + 1) SH) of its lane's row and writes the words into the row of the
        // strip, at the word the element has in global memory: strip word j of a row holds the output's 32-bit word
        // (first word of the piece) + j.  A 16-bit piece that starts on an odd element is shifted by half a word with
        // a funnel shift through the previous pair; its first and last half words are written as 16-bit stores, since
        // the other half of those words belongs to the other warp.
        auto store_piece = [&](int c0, int pcols, auto tcol, auto pack, int64_t cbase, int M, int N, bool anyodd,
                               auto loaded) -> bool {
            uint32_t r[32];
            const int sb = (int)(pieces & 1u);
            const uint32_t strip = blk_smem_u32(strips + (q * 2 + sb) * UM_STRIP_BYTES);
            const uint32_t filled_bar = bar0 + 8u * (20 + q * 2 + sb), drained_bar = bar0 + 8u * (28 + q * 2 + sb);
            const int64_t g = cbase + (int64_t)myrow * N + c0;       // element index of this lane's piece in the output
            const uint32_t par = OUT32 ? 0u : (uint32_t)(g & 1);
            [[maybe_unused]] const uint32_t par16 = par * 16u;
            const uint32_t srow = strip + (uint32_t)lane * (UM_STRIP_PITCHW * 4) + (uint32_t)h * (SH * ES);  // word 32 h of my row
            const int mycols = min(SH, pcols - h * SH);              // columns of the piece this warp converts (<= 0: none)
            // the strip's previous piece (two pieces ago) has been written out
            if (!mbar_wait(drained_bar, ((pieces >> 1) & 1u) ^ 1u, abort_flag, p.status, 8, lim)) return false;
            if (mycols <= 0) {
                loaded();
            } else if constexpr (OUT32) {
                uint32_t w[32];
                tc_ld32(lane_addr + tcol(c0 + h * SH), r);
                loaded();
                pack(r, w);
#pragma unroll
                for (int i = 0; i < 32; ++i) blk_sts_b32(srow + 4 * i, w[i]);
            } else {
                uint32_t w[16];
                uint32_t prev = 0;
                const int nu = (mycols + UM_PIECE - 1) / UM_PIECE;
                for (int u = 0; u < nu; ++u) {
                    tc_ld32(lane_addr + tcol(c0 + h * SH + u * UM_PIECE), r);
                    if (u == nu - 1) loaded();
                    pack(r, w);
                    const uint32_t a = srow + 64 * u;
                    if (!anyodd) {
#pragma unroll
                        for (int i = 0; i < 16; ++i) blk_sts_b32(a + 4 * i, w[i]);
                    } else {
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const uint32_t v = __funnelshift_l(prev, w[i], par16);
                            if (u == 0 && i == 0) {
                                // the low half of my first word is the other warp's last element when the piece is odd
                                if (par) blk_sts_b16(a + 2, v >> 16);
                                else blk_sts_b32(a, v);
                            } else {
                                blk_sts_b32(a + 4 * i, v);
                            }
                            prev = w[i];
                        }
                    }
                }
                if (anyodd && par) blk_sts_b16(srow + 64 * nu, prev >> 16);  // my last element: low half of the next word
            }
            if (h == 0 && lane == 0) {
                volatile UmPiece* d = pieces_desc + q * 2 + sb;
                d->g0 = cbase + (int64_t)(q * 32) * N + c0;
                d->N = N;
                d->pcols = pcols;
                d->rows = max(0, min(M - q * 32, 32));
                d->halves = (anyodd || (pcols & 1)) ? 1 : 0;
                d->stop = 0;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(filled_bar);
            ++pieces;
            return true;
        };
        // the pieces of columns [c_lo, c_hi) of a chunk
        auto store_cols = [&](int c_lo, int c_hi, auto tcol, auto pack, int64_t cbase, int M, int N, bool anyodd,
                              auto loaded) -> bool {
            for (int c0 = c_lo; c0 < c_hi; c0 += PC) {
                const bool last = c0 + PC >= c_hi;
                if (!store_piece(c0, min(PC, c_hi - c0), tcol, pack, cbase, M, N, anyodd, [&]() { if (last) loaded(); }))
                    return false;
            }
            return true;
        };
        // pack(r, w) for an elementwise map of the accumulator values
        auto pack_with = [](auto xform) {
            return [xform](const uint32_t (&r)[32], auto& w) {
                if constexpr (OUT32) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) w[i] = __float_as_uint(xform(__uint_as_float(r[i])));
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        w[i] = BlkCvt<Tag>::pack2(xform(__uint_as_float(r[2 * i])), xform(__uint_as_float(r[2 * i + 1])));
                }
            };
        };
        // First sweep of a row too long for tensor memory, one chunk: running (maximum, sum) over this warp's blocks.
        float mx1 = -INFINITY, sum1 = 0.f;
        auto first_sweep_chunk = [&](int N, int ch) {
            uint32_t r[32];
            const int buf = slot & 1;
            if (!mbar_wait(tfull_bar(buf), (slot >> 1) & 1u, abort_flag, p.status, 6, lim)) { ok = false; return; }
            tc_fence_after();
            const int ncols = min(N - ch * UM_BN, UM_BN);
            for (int b0 = h * SH; b0 < ncols; b0 += PC) {
                const int hi = min(b0 + SH, ncols);
                for (int c = b0; c < hi; c += UM_PIECE) {
                    tc_ld32(lane_addr + (uint32_t)(buf * UM_BN + c), r);
                    const bool part = c + 32 > hi;
                    if (part) {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (c + i >= hi) r[i] = 0xff800000u;  // -inf
                    }
                    float pm = -INFINITY;
#pragma unroll
                    for (int i = 0; i < 32; i += 2) pm = blk_max3(pm, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
                    const float mnew = fmaxf(mx1, pm);  // finite: column c of the piece is inside the row
                    const float nm = -mnew * sl;
                    float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int i = 0; i < 32; ++i) s4[i & 3] += blk_exp2(fmaf(__uint_as_float(r[i]), sl, nm));
                    sum1 = sum1 * blk_exp2((mx1 - mnew) * sl) + ((s4[0] + s4[1]) + (s4[2] + s4[3]));
                    mx1 = mnew;
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(buf));
            ++slot;
        };
        // The quarter's warps combine their (maximum, sum) of a finished first sweep; the result is the offset with which
        // exp2(x * sl + off) = exp2((x - max) * sl) / sum: no multiply after the exponential in the second sweep.
        float off_next = 0.f;
        auto first_sweep_done = [&]() {
            volatile float* xm = xch + (seq++ & 1) * (2 * UM_SPLIT * 128);  // [part][row] maxima, then [UM_SPLIT + part][row] sums
            xm[h * 128 + myrow] = mx1;
            xm[(UM_SPLIT + h) * 128 + myrow] = sum1;
            if (!pair_sync()) { ok = false; return; }
            // a warp whose share held no column of the row (a last chunk of at most 64 columns) has maximum -inf
            // and sum 0: its term is skipped
            float m = -INFINITY;
#pragma unroll
            for (int o = 0; o < UM_SPLIT; ++o) m = fmaxf(m, xm[o * 128 + myrow]);
            float l = 0.f;
#pragma unroll
            for (int o = 0; o < UM_SPLIT; ++o) {
                const float mo = xm[o * 128 + myrow];
                if (mo != -INFINITY) l += xm[(UM_SPLIT + o) * 128 + myrow] * blk_exp2((mo - m) * sl);
            }
            off_next = -m * sl - __log2f(l);
        };
        Work nx;
        bool pre = false;  // this item's first sweep ran alongside the previous item's second
        for (uint32_t w = blockIdx.x; ok && next_work(p, w, wk); w += gridDim.x) {
            const bool pair = pairs_with_next(p, w, wk, nx);
            const bool had_first = pre;
            pre = pair;
            const int M = wk.it.M - wk.it.tm * UM_BM;  // rows of the segment from this block on
            const int N = wk.it.N;
            const int64_t cbase = (int64_t)wk.head * p.Dout + wk.it.offC + (int64_t)wk.it.tm * UM_BM * N;
            // 16-bit rows that start on an odd element need the half-word shift while staging (chunks and pieces start
            // on even columns, so a row's parity is the same for all of them); the quarter's warps hold the same rows
            const bool anyodd = !OUT32 && __any_sync(0xffffffffu, (int)((cbase + (int64_t)myrow * N) & 1));
            if (!softmax) {
                for (int ch = wk.it.ch0; ok && ch < wk.it.ch0 + wk.nchunks; ++ch, ++slot) {
                    const int buf = slot & 1;
                    if (!mbar_wait(tfull_bar(buf), (slot >> 1) & 1u, abort_flag, p.status, 4, lim)) { ok = false; break; }
                    tc_fence_after();
                    const int ncols = min(N - ch * UM_BN, UM_BN);
                    auto release = [&]() {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(tempty_bar(buf));
                    };
                    ok = store_cols(ch * UM_BN, ch * UM_BN + ncols,
                                    [&](int c) { return (uint32_t)(buf * UM_BN + (c - ch * UM_BN)); },
                                    pack_with([sl](float x) { return x * sl; }), cbase, M, N, anyodd, release);
                }
            } else if (wk.sweeps == 1) {
                // whole row resident: chunk k of the row sits in accumulator (slot + k) & 1
                volatile float* xm = xch + (seq++ & 1) * (2 * UM_SPLIT * 128);  // [part][row] maxima, then [UM_SPLIT + part][row] sums
                for (int ch = 0; ok && ch < wk.nchunks; ++ch)
                    if (!mbar_wait(tfull_bar((slot + ch) & 1), ((slot + ch) >> 1) & 1u, abort_flag, p.status, 5, lim)) ok = false;
                if (!ok) break;
                tc_fence_after();
                auto tcol = [&](int c) {  // tensor-memory column of row column c
                    return (uint32_t)((((slot + (c >> 8)) & 1) * UM_BN) + (c & (UM_BN - 1)));
                };
                uint32_t r[32];
                // pass 1: maximum over this warp's blocks
                float mx = -INFINITY;
                for (int b0 = h * SH; b0 < N; b0 += PC) {
                    const int bend = min(b0 + SH, N);
                    for (int c = b0; c < bend; c += UM_PIECE) {
                        tc_ld32(lane_addr + tcol(c), r);
                        if (c + 32 <= bend) {
#pragma unroll
                            for (int i = 0; i < 32; i += 2) mx = blk_max3(mx, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
                        } else {
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                if (c + i < bend) mx = fmaxf(mx, __uint_as_float(r[i]));
                        }
                    }
                }
                xm[h * 128 + myrow] = mx;
                if (!pair_sync()) { ok = false; break; }
#pragma unroll
                for (int o = 0; o < UM_SPLIT; ++o) mx = fmaxf(mx, xm[o * 128 + myrow]);
                const float nm = -mx * sl;
                // pass 2: exponentials back into tensor memory, partial sum
                float s4[4] = {0.f, 0.f, 0.f, 0.f};
                for (int b0 = h * SH; b0 < N; b0 += PC) {
                    const int bend = min(b0 + SH, N);
                    for (int c = b0; c < bend; c += UM_PIECE) {
                        tc_ld32(lane_addr + tcol(c), r);
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            float e = blk_exp2(fmaf(__uint_as_float(r[i]), sl, nm));
                            if (c + 32 > bend) e = (c + i < bend) ? e : 0.f;
                            s4[i & 3] += e;
                            r[i] = __float_as_uint(e);
                        }
                        tc_st32(lane_addr + tcol(c), r);
                    }
                }
                tc_wait_st();
                float sum = (s4[0] + s4[1]) + (s4[2] + s4[3]);
                xm[(UM_SPLIT + h) * 128 + myrow] = sum;
                if (!pair_sync()) { ok = false; break; }
                sum = 0.f;
#pragma unroll
                for (int o = 0; o < UM_SPLIT; ++o) sum += xm[(UM_SPLIT + o) * 128 + myrow];
                const float inv = __frcp_rn(sum);
                // pass 3: normalise and stage (this warp reads back the columns it wrote in pass 2); an accumulator goes
                // back to the MMA role as soon as this warp has read its share of it, so the next item's products overlap
                // the rest of this item's epilogue
                for (int ch = 0; ok && ch < wk.nchunks; ++ch) {
                    auto release = [&]() {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(tempty_bar((slot + ch) & 1));
                    };
                    ok = store_cols(ch * UM_BN, min((ch + 1) * UM_BN, N), tcol, pack_with([inv](float x) { return x * inv; }),
                                    cbase, M, N, anyodd, release);
                }
                slot += wk.nchunks;
            } else {
                // two sweeps: running (max, sum) over this warp's blocks, then recompute and stage; when the next item
                // pairs with this one, each storing chunk is followed by a first-sweep chunk of the next item, whose
                // exponentials run while this chunk's pieces drain
                if (!had_first) {
                    mx1 = -INFINITY; sum1 = 0.f;
                    for (int ch = 0; ok && ch < wk.nchunks; ++ch) first_sweep_chunk(N, ch);
                    if (ok) first_sweep_done();
                    if (!ok) break;
                }
                const float off = off_next;
                if (pair) { mx1 = -INFINITY; sum1 = 0.f; }
                for (int ch = 0; ok && ch < wk.nchunks; ++ch) {
                    const int buf = slot & 1;
                    if (!mbar_wait(tfull_bar(buf), (slot >> 1) & 1u, abort_flag, p.status, 7, lim)) { ok = false; break; }
                    tc_fence_after();
                    const int ncols = min(N - ch * UM_BN, UM_BN);
                    auto release = [&]() {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(tempty_bar(buf));
                    };
                    ok = store_cols(ch * UM_BN, ch * UM_BN + ncols,
                                    [&](int c) { return (uint32_t)(buf * UM_BN + (c - ch * UM_BN)); },
                                    pack_with([sl, off](float x) { return blk_exp2(fmaf(x, sl, off)); }), cbase, M, N, anyodd,
                                    release);
                    ++slot;
                    if (ok && pair) first_sweep_chunk(nx.it.N, ch);
                }
                if (ok && pair) first_sweep_done();
            }
        }
        // tell the quarter's store warp that nothing follows: one more "piece" that only says stop (posted on both strips;
        // the store warp leaves at the first)
        for (int t = 0; t < 2; ++t) {
            const int sb = (int)(pieces & 1u);
            const uint32_t filled_bar = bar0 + 8u * (20 + q * 2 + sb), drained_bar = bar0 + 8u * (28 + q * 2 + sb);
            if (ok && !mbar_wait(drained_bar, ((pieces >> 1) & 1u) ^ 1u, abort_flag, p.status, 8, lim)) ok = false;
            if (h == 0 && lane == 0) (pieces_desc + q * 2 + sb)->stop = 1;
            __syncwarp();
            if (lane == 0) mbar_arrive(filled_bar);
            ++pieces;
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        // a role gave up: let copies that may still be in flight land before the CTA's memory is released
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512));
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qr) == cudaSuccess &&
            qr == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

template <typename Tag, bool OUT32, int SPLIT>
cudaError_t launch(const BlkUmmaParams& p, const UmMaps& maps, int sms, cudaStream_t st) {
    auto kern = blk_gemm_umma_kernel<Tag, OUT32, SPLIT>;
    cudaError_t e = blk_func_smem(reinterpret_cast<const void*>(kern), UM_SMEM_BYTES);
    if (e != cudaSuccess) return e;
    const int64_t total = (int64_t)p.num_items * p.H;
    const dim3 grid((unsigned)(total < sms ? total : sms)), block(um_threads(SPLIT));
    kern<<<grid, block, UM_SMEM_BYTES, st>>>(p, maps);
    return cudaGetLastError();
}

}  // namespace

// Encoded maps are remembered: a map depends only on the arguments below (never on the memory it describes), and a
// plan is run many times on the same buffers, so the driver's encoder is called once per distinct view.
namespace {
struct MapKey {
    const void* base; int64_t K, H, rows, row_stride, head_stride; int bf16, box_k, box_rows;
    bool operator==(const MapKey& o) const {
        return base == o.base && K == o.K && H == o.H && rows == o.rows && row_stride == o.row_stride &&
               head_stride == o.head_stride && bf16 == o.bf16 && box_k == o.box_k && box_rows == o.box_rows;
    }
};
struct MapSlot { MapKey key; CUtensorMap map; int head_first; uint64_t stamp; bool used; };
constexpr int MAP_SLOTS = 64;
MapSlot g_map_slots[MAP_SLOTS];
uint64_t g_map_clock = 0;
std::mutex g_map_mu;
}  // namespace

bool blk_make_row_map(CUtensorMap_st* map, const void* base, int bf16, int64_t K, int64_t H, const BlkOperandLayout& lay,
                      int box_k, int box_rows, int* head_first) {
    EncodeTiledFn fn = encode_fn();
    if (!fn || lay.rows <= 0 || H <= 0) return false;
    if (lay.row_stride % 8 || lay.head_stride % 8 || lay.row_stride < K) return false;  // 16-byte strides
    const MapKey key{base, K, H, lay.rows, lay.row_stride, lay.head_stride, bf16, box_k, box_rows};
    {
        std::lock_guard<std::mutex> g(g_map_mu);
        for (MapSlot& sl : g_map_slots)
            if (sl.used && sl.key == key) {
                sl.stamp = ++g_map_clock;
                *map = sl.map;
                *head_first = sl.head_first;
                return true;
            }
    }
    const bool hf = lay.head_stride < lay.row_stride;  // token-major: heads are the closer dimension
    *head_first = hf ? 1 : 0;
    const cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)(hf ? H : lay.rows), (cuuint64_t)(hf ? lay.rows : H)};
    const cuuint64_t strides[2] = {(cuuint64_t)(hf ? lay.head_stride : lay.row_stride) * 2,
                                   (cuuint64_t)(hf ? lay.row_stride : lay.head_stride) * 2};
    const cuuint32_t box[3] = {(cuuint32_t)box_k, (cuuint32_t)(hf ? 1 : box_rows), (cuuint32_t)(hf ? box_rows : 1)};
    const cuuint32_t estr[3] = {1, 1, 1};
    if (fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
           const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    std::lock_guard<std::mutex> g(g_map_mu);
    MapSlot* victim = &g_map_slots[0];
    for (MapSlot& sl : g_map_slots) {
        if (!sl.used) { victim = &sl; break; }
        if (sl.stamp < victim->stamp) victim = &sl;
    }
    victim->key = key;
    victim->map = *map;
    victim->head_first = *head_first;
    victim->stamp = ++g_map_clock;
    victim->used = true;
    return true;
}

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per kernel and device instead of before every launch.
cudaError_t blk_func_smem(const void* kern, int bytes) {
    constexpr int SLOTS = 256;
    static struct { const void* kern; int dev; } done[SLOTS];
    static int ndone = 0;
    static std::mutex mu;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    {
        std::lock_guard<std::mutex> g(mu);
        for (int i = 0; i < ndone; ++i)
            if (done[i].kern == kern && done[i].dev == dev) return cudaSuccess;
    }
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return e;
    std::lock_guard<std::mutex> g(mu);
    if (ndone < SLOTS) { done[ndone].kern = kern; done[ndone].dev = dev; ++ndone; }
    return cudaSuccess;
}

// The maps of a launch are remembered as a set under everything they depend on (buffers, strip lengths, views,
// layouts): a plan is run many times on a few sets of buffers, and encoding up to 48 maps costs more than the launch.
namespace {
struct LaunchKey {
    const void *a, *b;
    int64_t Da, Db, H;
    int na, nb, bf16, ga, gb;
    BlkOperandLayout layA, layB;
    BlkUmmaView va[BLK_UMMA_VIEWS], vb[BLK_UMMA_VIEWS];
};
struct LaunchSlot { LaunchKey key; UmMaps maps; int hfA, hfB; uint64_t stamp; bool used; };
constexpr int LAUNCH_SLOTS = 8;
LaunchSlot g_launch_slots[LAUNCH_SLOTS];
uint64_t g_launch_clock = 0;
std::mutex g_launch_mu;
bool same_key(const LaunchKey& x, const LaunchKey& y) {
    if (x.a != y.a || x.b != y.b || x.Da != y.Da || x.Db != y.Db || x.H != y.H || x.na != y.na || x.nb != y.nb ||
        x.bf16 != y.bf16 || x.ga != y.ga || x.gb != y.gb)
        return false;
    auto lay_eq = [](const BlkOperandLayout& p, const BlkOperandLayout& q) {
        return p.rows == q.rows && p.row_stride == q.row_stride && p.head_stride == q.head_stride;
    };
    if ((x.ga && !lay_eq(x.layA, y.layA)) || (x.gb && !lay_eq(x.layB, y.layB))) return false;
    for (int i = 0; i < x.na; ++i)
        if (x.va[i].K != y.va[i].K || x.va[i].residue != y.va[i].residue) return false;
    for (int i = 0; i < x.nb; ++i)
        if (x.vb[i].K != y.vb[i].K || x.vb[i].residue != y.vb[i].residue) return false;
    return true;
}
}  // namespace

cudaError_t blk_launch_gemm_umma(const BlkUmmaParams& p_in, const BlkUmmaOperand& A, const BlkUmmaOperand& B, int sms,
                                 cudaStream_t st) {
    if ((int64_t)p_in.num_items * p_in.H == 0) return cudaSuccess;
    if (A.num_views < 1 || B.num_views < 1 || A.num_views > BLK_UMMA_VIEWS || B.num_views > BLK_UMMA_VIEWS) return cudaErrorInvalidValue;
    BlkUmmaParams p = p_in;
    static thread_local LaunchKey key;   // these are kilobytes: not on the stack of a caller's thread
    static thread_local UmMaps maps;
    key.a = A.base; key.b = B.base; key.Da = A.D; key.Db = B.D; key.H = p.H;
    key.na = A.num_views; key.nb = B.num_views; key.bf16 = p.bf16;
    key.ga = A.given != nullptr; key.gb = B.given != nullptr;
    if (A.given) key.layA = *A.given;
    if (B.given) key.layB = *B.given;
    for (int i = 0; i < A.num_views; ++i) key.va[i] = A.views[i];
    for (int i = 0; i < B.num_views; ++i) key.vb[i] = B.views[i];
    bool hit = false;
    {
        std::lock_guard<std::mutex> g(g_launch_mu);
        for (LaunchSlot& sl : g_launch_slots)
            if (sl.used && same_key(sl.key, key)) {
                sl.stamp = ++g_launch_clock;
                maps = sl.maps;
                p.head_firstA = sl.hfA;
                p.head_firstB = sl.hfB;
                hit = true;
                break;
            }
    }
    if (!hit) {
        // every view of an operand has the same order of its strides, so the same order of coordinates
        auto encode = [&](const BlkUmmaOperand& op, CUtensorMap* out, int box_rows, int* head_first) {
            if (op.given && (op.num_views != 1 || op.views[0].residue != 0)) return false;
            for (int v = 0; v < op.num_views; ++v) {
                const BlkUmmaView& vw = op.views[v];
                const BlkOperandLayout lay = op.given ? *op.given : BlkOperandLayout{(op.D - vw.residue) / vw.K, vw.K, op.D};
                int hf = 0;
                if (!blk_make_row_map(&out[v], static_cast<const unsigned char*>(op.base) + 2 * vw.residue, p.bf16, vw.K, p.H, lay,
                                      UM_BK, box_rows, &hf))
                    return false;
                if (v > 0 && hf != *head_first) return false;
                *head_first = hf;
            }
            return true;
        };
        if (!encode(A, maps.a, UM_BM, &p.head_firstA) || !encode(B, maps.b, UM_BN, &p.head_firstB)) return cudaErrorInvalidValue;
        std::lock_guard<std::mutex> g(g_launch_mu);
        LaunchSlot* victim = &g_launch_slots[0];
        for (LaunchSlot& sl : g_launch_slots) {
            if (!sl.used) { victim = &sl; break; }
            if (sl.stamp < victim->stamp) victim = &sl;
        }
        victim->key = key;
        victim->maps = maps;
        victim->hfA = p.head_firstA;
        victim->hfB = p.head_firstB;
        victim->stamp = ++g_launch_clock;
        victim->used = true;
    }
    const bool four = !p.out_f32 && p.epi == BLK_EPI_SOFTMAX && p.long_rows;
    if (p.bf16)
        return p.out_f32 ? launch<BlkBf16Tag, true, 2>(p, maps, sms, st)
                         : (four ? launch<BlkBf16Tag, false, 4>(p, maps, sms, st) : launch<BlkBf16Tag, false, 2>(p, maps, sms, st));
    return p.out_f32 ? launch<BlkHalfTag, true, 2>(p, maps, sms, st)
                     : (four ? launch<BlkHalfTag, false, 4>(p, maps, sms, st) : launch<BlkHalfTag, false, 2>(p, maps, sms, st));
}
