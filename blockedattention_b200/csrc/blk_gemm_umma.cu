// Large-segment kernel of the varlen blocked GEMM on the 5th-generation tensor
// cores: TMA-fed tcgen05.mma with the accumulator in tensor memory.
//
// A persistent CTA (one per SM, 18 warps) walks a static list of work items, an
// item being a 128-row block of one segment of one head.  Roles:
//   warp 0   producer: one lane issues 3-D tiled TMA loads (k, row, head) of a
//            128 x 64 tile of the first operand and a 256 x 64 tile of the
//            second into a 3-stage ring of 128-byte-swizzled shared memory;
//   warp 1   MMA: allocates the 512 tensor-memory columns, and one lane issues
//            tcgen05.mma (M = 128, N up to 256, K = 16 per instruction) into
//            one of two 256-column accumulators; tcgen05.commit hands shared
//            memory stages back to the producer and accumulators to the epilogue;
//   warps 2-17 epilogue: a warp may read the 32 accumulator lanes (= rows) of its
//            quarter; the four warps of a quarter each take 64 of every 256
//            columns of the row and exchange partial row statistics through
//            shared memory.  A thread reads its row 32 columns at a time
//            (tcgen05.ld), applies the epilogue and the warp writes the piece
//            out through a padded shared-memory strip so that lanes store
//            consecutive addresses with the widest store the row allows.
//
// Epilogues.  Scores: scale and round.  Softmax with N <= 512: both
// accumulators hold the whole row; pass 1 takes the row maximum, pass 2 writes
// exp2 back into tensor memory while summing, pass 3 normalises and stores, so
// the exponential is evaluated once per element and the scores never leave the
// SM.  Softmax with N > 512: the products are computed twice -- a first sweep
// over the 256-column chunks keeps only a running (max, sum) per row, a second
// sweep recomputes each chunk and stores normalised probabilities.
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
constexpr int UM_SPLIT = 4;                           // epilogue warps per accumulator-lane quarter
constexpr int UM_EPI_WARPS = 4 * UM_SPLIT;
constexpr int UM_THREADS = 64 + 32 * UM_EPI_WARPS;
constexpr int UM_CB = UM_BN / UM_SPLIT;               // columns of a chunk owned by one of them
constexpr int UM_PIECE = 32;                          // columns per tcgen05.ld
constexpr int UM_ROWPIECE_BYTES = 128;                // bytes of an output row staged per flush (64 x 16-bit, 32 x fp32)
constexpr int UM_STRIP_PITCH = UM_ROWPIECE_BYTES + 20;  // bytes per strip row: 37 words, odd, so lanes on one column hit 32 banks
constexpr int UM_STRIP_BYTES = 32 * UM_STRIP_PITCH;   // per epilogue warp
constexpr int UM_XCH_BYTES = 2 * 2 * UM_SPLIT * 128 * 4;  // row statistics exchanged between the two halves, double-buffered
constexpr int UM_SMEM_BYTES = UM_STAGES * UM_STAGE_BYTES + UM_EPI_WARPS * UM_STRIP_BYTES + UM_XCH_BYTES + 256;
static_assert(UM_SMEM_BYTES <= 227 * 1024, "shared memory budget");
static_assert(UM_STAGES <= 4, "barrier slots");

struct Work {
    BlkUmmaItem it;
    int head;
    int nchunks;
    int sweeps;
};

__device__ __forceinline__ bool next_work(const BlkUmmaParams& p, uint32_t w, Work& wk) {
    const uint32_t total = (uint32_t)p.num_items * (uint32_t)p.H;
    if (w >= total) return false;
    const uint32_t item = w / (uint32_t)p.H;
    wk.head = (int)(w - item * (uint32_t)p.H);
    wk.it = p.items[item];
    wk.nchunks = (wk.it.N + UM_BN - 1) / UM_BN;
    wk.sweeps = (p.epi == BLK_EPI_SOFTMAX && wk.nchunks > 2) ? 2 : 1;
    return true;
}

// Stage 32 consecutive columns of this thread's row (strip row = lane) at column offset `sub` * 32 of the
// current row piece.  The strip pitch is an odd number of words (37), so the 32 lanes of a store hit 32
// different banks.
template <typename Tag, bool OUT32>
__device__ __forceinline__ void emit32(const float (&v)[32], unsigned char* strip, int sub, int lane) {
    const uint32_t base = blk_smem_u32(strip) + lane * UM_STRIP_PITCH + sub * (UM_PIECE * (OUT32 ? 4 : 2));
    if (OUT32) {
#pragma unroll
        for (int i = 0; i < 32; ++i) blk_sts_f32(base + 4 * i, v[i]);
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) blk_sts_b32(base + 4 * i, BlkCvt<Tag>::pack2(v[2 * i], v[2 * i + 1]));
    }
}

// Predicated global stores as single instructions (no branch around them).
__device__ __forceinline__ void stg_v4_if(void* p, const uint4& v, bool ok) {
    asm volatile("{\n .reg .pred q;\n setp.ne.b32 q, %5, 0;\n @q st.global.v4.b32 [%0], {%1, %2, %3, %4};\n}\n" ::"l"(p),
                 "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w), "r"((int)ok)
                 : "memory");
}
__device__ __forceinline__ void stg_b16_if(void* p, uint16_t v, bool ok) {
    asm volatile("{\n .reg .pred q;\n setp.ne.b32 q, %2, 0;\n @q st.global.b16 [%0], %1;\n}\n" ::"l"(p), "h"(v), "r"((int)ok)
                 : "memory");
}
__device__ __forceinline__ void stg_b32_if(void* p, uint32_t v, bool ok) {
    asm volatile("{\n .reg .pred q;\n setp.ne.b32 q, %2, 0;\n @q st.global.b32 [%0], %1;\n}\n" ::"l"(p), "r"(v), "r"((int)ok)
                 : "memory");
}

// Strip -> global for the warp's 32 rows x `ncols` columns starting at column col0.  Four rows per pass,
// eight lanes per row; lane hl owns the 16-byte vector hl of the row piece *as aligned in global memory*.
// A row piece starts at an arbitrary 2-byte (4-byte for fp32) offset sh inside its first vector, so the
// lane gathers its 16 bytes from the strip as five words and funnel-shifts them into place; only the
// ragged first and last vector of a row piece go out as single elements, one per lane.  Branch-free.
template <bool OUT32>
__device__ __forceinline__ void flush_piece(const BlkUmmaParams& p, unsigned char* strip, int64_t cbase, int row0,
                                            int M, int N, int col0, int ncols, int lane) {
    constexpr int ES = OUT32 ? 4 : 2;
    constexpr int LPR = UM_ROWPIECE_BYTES / 16;  // lanes (vectors) per row
    constexpr int RPP = 32 / LPR;                // rows per pass
    __syncwarp();
    const int hl = lane % LPR, rsel = lane / LPR;
    const int nbytes = ncols * ES;
    const int eoff = ES * hl;  // byte of this lane's edge elements inside the first / last vector
    int64_t b0 = (cbase + (int64_t)(row0 + rsel) * N + col0) * ES;  // byte offset of this lane's row piece
    const int64_t bstep = (int64_t)RPP * N * ES;
    const unsigned char* src = strip + rsel * UM_STRIP_PITCH;  // byte 0 of src <-> byte b0 of the output
    unsigned char* C = reinterpret_cast<unsigned char*>(p.C);
#pragma unroll 4
    for (int r = rsel; r < 32; r += RPP, b0 += bstep, src += RPP * UM_STRIP_PITCH) {
        const bool row_ok = row0 + r < M;
        const int sh = (int)(b0 & 15);
        unsigned char* dst = C + (b0 - sh);  // 16-byte aligned
        const int end = sh + nbytes;         // the row piece is bytes [sh, end) counted from dst
        // vector [16 hl, 16 hl + 16) if it lies inside [sh, end): strip bytes [x, x + 16), x = 16 hl - sh
        const int lo = 16 * hl, x = lo - sh;
        const int xw = x > 0 ? (x & ~3) : 0;
        const int sb = (x & 2) * 8;
        const uint32_t* wp = reinterpret_cast<const uint32_t*>(src + xw);
        const uint32_t w0 = wp[0], w1 = wp[1], w2 = wp[2], w3 = wp[3], w4 = wp[4];
        uint4 vec;
        vec.x = __funnelshift_r(w0, w1, sb);
        vec.y = __funnelshift_r(w1, w2, sb);
        vec.z = __funnelshift_r(w2, w3, sb);
        vec.w = __funnelshift_r(w3, w4, sb);
        stg_v4_if(dst + lo, vec, row_ok && lo >= sh && lo + 16 <= end);
        // ragged first and last vector: lane hl takes element hl of each
        const int tail = end & ~15;
        const bool in_vec = eoff < 16;
        const bool first_full = sh == 0 && end >= 16;
        const bool ok_h = row_ok && in_vec && !first_full && eoff >= sh && eoff < end;
        const int bt = tail + eoff;
        const bool ok_t = row_ok && in_vec && tail != 0 && bt < end;
        const int sh_h = ok_h ? eoff - sh : 0, sh_t = ok_t ? bt - sh : 0;  // strip bytes of the two elements
        if (OUT32) {
            stg_b32_if(dst + eoff, *reinterpret_cast<const uint32_t*>(src + sh_h), ok_h);
            stg_b32_if(dst + bt, *reinterpret_cast<const uint32_t*>(src + sh_t), ok_t);
        } else {
            stg_b16_if(dst + eoff, *reinterpret_cast<const uint16_t*>(src + sh_h), ok_h);
            stg_b16_if(dst + bt, *reinterpret_cast<const uint16_t*>(src + sh_t), ok_t);
        }
    }
    __syncwarp();
}

template <typename Tag, bool OUT32>
__global__ void __launch_bounds__(UM_THREADS, 1)
blk_gemm_umma_kernel(const BlkUmmaParams p, const __grid_constant__ CUtensorMap mapA,
                     const __grid_constant__ CUtensorMap mapB) {
    extern __shared__ __align__(1024) unsigned char um_smem_raw[];  // the swizzled tiles need a 1024-byte aligned base
    unsigned char* smem = um_smem_raw;
    if (blk_smem_u32(smem) & 1023u) {  // cannot happen with the alignment above; checked because the swizzle relies on it
        if (threadIdx.x == 0) atomicCAS(p.status, 0, 9);
        return;
    }
    unsigned char* strips = smem + UM_STAGES * UM_STAGE_BYTES;
    float* xch = reinterpret_cast<float*>(strips + UM_EPI_WARPS * UM_STRIP_BYTES);
    uint64_t* bars = reinterpret_cast<uint64_t*>(strips + UM_EPI_WARPS * UM_STRIP_BYTES + UM_XCH_BYTES);
    // bars[0..3] full (UM_STAGES used), [4..7] empty, [8..9] tmem_full, [10..11] tmem_empty
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
        for (int i = 0; i < 4; ++i) reinterpret_cast<volatile uint32_t*>(bars + 14)[i] = 0;
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
    const int nkb = p.K / UM_BK;
    const uint32_t lim = p.spin_limit ? p.spin_limit : BLK_UMMA_SPIN_LIMIT;

    if (warp == 0) {
        // ---------------- producer ----------------
        if (lane == 0 && !p.stall) {
            int stage = 0;
            uint32_t phase = 0;
            Work wk;
            bool ok = true;
            for (uint32_t w = blockIdx.x; ok && next_work(p, w, wk); w += gridDim.x) {
                for (int sw = 0; ok && sw < wk.sweeps; ++sw)
                    for (int ch = 0; ok && ch < wk.nchunks; ++ch)
                        for (int kb = 0; kb < nkb; ++kb) {
                            if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, 1, lim)) { ok = false; break; }
                            const uint32_t sA = smem_u32 + stage * UM_STAGE_BYTES, sB = sA + UM_A_BYTES;
                            mbar_expect_tx(full_bar(stage), UM_STAGE_BYTES);
                            // coordinates (k, row, head), or (k, head, row) for a token-major operand
                            const int rA = wk.it.rowA, rB = wk.it.rowB + ch * UM_BN;
                            tma_load_3d(sA, &mapA, full_bar(stage), kb * UM_BK, p.head_firstA ? wk.head : rA,
                                        p.head_firstA ? rA : wk.head);
                            tma_load_3d(sB, &mapB, full_bar(stage), kb * UM_BK, p.head_firstB ? wk.head : rB,
                                        p.head_firstB ? rB : wk.head);
                            if (++stage == UM_STAGES) { stage = 0; phase ^= 1u; }
                        }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issue ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0, slot = 0;
            Work wk;
            bool ok = true;
            for (uint32_t w = blockIdx.x; ok && next_work(p, w, wk); w += gridDim.x) {
                for (int sw = 0; ok && sw < wk.sweeps; ++sw)
                    for (int ch = 0; ok && ch < wk.nchunks; ++ch) {
                        const int buf = slot & 1;
                        if (!mbar_wait(tempty_bar(buf), ((slot >> 1) & 1u) ^ 1u, abort_flag, p.status, 2, lim)) { ok = false; break; }
                        tc_fence_after();
                        const int ncols = min(wk.it.N - ch * UM_BN, UM_BN);
                        const uint32_t idesc = instr_desc(p.bf16, (ncols + 15) & ~15, p.epi == BLK_EPI_SOFTMAX && p.scale < 0.f);
                        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * UM_BN);
                        for (int kb = 0; kb < nkb; ++kb) {
                            if (!mbar_wait(full_bar(stage), phase, abort_flag, p.status, 3, lim)) { ok = false; break; }
                            tc_fence_after();
                            const uint32_t sA = smem_u32 + stage * UM_STAGE_BYTES, sB = sA + UM_A_BYTES;
#pragma unroll
                            for (int k = 0; k < UM_BK / 16; ++k)
                                tc_mma_f16(d_tmem, smem_desc_sw128(sA + 32 * k), smem_desc_sw128(sB + 32 * k), idesc,
                                           (kb | k) != 0);
                            tc_commit(empty_bar(stage));  // stage reusable once these products have read it
                            if (++stage == UM_STAGES) { stage = 0; phase ^= 1u; }
                        }
                        if (!ok) break;
                        tc_commit(tfull_bar(buf));
                        ++slot;
                    }
            }
        }
    } else {
        // ---------------- epilogue: warps 2..17 ----------------
        // lane quarter q = warp % 4 (the 32 accumulator lanes a warp may read); the UM_SPLIT warps of a quarter
        // split the row's 128-column blocks by parity (half h) and exchange their partial row statistics.
        const int q = warp & 3, h = (warp - 2) >> 2;  // h in [0, UM_SPLIT)
        unsigned char* strip = strips + (warp - 2) * UM_STRIP_BYTES;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
        const int myrow = q * 32 + lane;
        uint32_t slot = 0, seq = 0;
        Work wk;
        bool ok = true;
        const bool softmax = p.epi == BLK_EPI_SOFTMAX;
        const float sl = softmax ? fabsf(p.scale) * BLK_LOG2E : p.scale;  // a negative softmax scale is applied by
                                                                          // the MMA (negated A), see instr_desc
        constexpr int RP = UM_ROWPIECE_BYTES / (OUT32 ? 4 : 2);  // columns per staged row piece
        constexpr int CB = UM_CB;                                // columns of a chunk owned by this warp
        // Rendezvous of the warps of a quarter (after each has published its row statistics): a shared
        // counter and a bounded spin, so that a warp whose partner gave up cannot wait for ever.
        volatile uint32_t* pair_cnt = reinterpret_cast<volatile uint32_t*>(bars + 14) + q;
        uint32_t pair_target = 0;
        auto pair_sync = [&]() -> bool {
            pair_target += UM_SPLIT;
            __threadfence_block();
            __syncwarp();
            if (lane == 0) atomicAdd(const_cast<uint32_t*>(pair_cnt), 1u);
            bool good = false;
            for (uint32_t i = 0; i < BLK_UMMA_SPIN_LIMIT; ++i) {
                if ((int32_t)(*pair_cnt - pair_target) >= 0) { good = true; break; }
                if (i > 64) __nanosleep(32);
                if ((i & 255u) == 255u && *abort_flag) break;
            }
            if (!good) {
                *abort_flag = 1;
                atomicCAS(p.status, 0, 8);
            }
            __syncwarp();
            __threadfence_block();
            return good;
        };
        // scale, round and store columns [c_lo, c_hi) of the row; tcol(c) gives the tensor-memory column
        auto store_cols = [&](int c_lo, int c_hi, auto tcol, auto xform, int64_t cbase, int M, int N) {
            uint32_t r[32];
            float v[32];
            for (int c0 = c_lo; c0 < c_hi; c0 += RP) {
                const int pc = min(RP, c_hi - c0);
                for (int c = 0; c < pc; c += UM_PIECE) {
                    tc_ld32(lane_addr + tcol(c0 + c), r);
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = xform(__uint_as_float(r[i]));
                    emit32<Tag, OUT32>(v, strip, c / UM_PIECE, lane);
                }
                flush_piece<OUT32>(p, strip, cbase, q * 32, M, N, c0, pc, lane);
            }
        };
        for (uint32_t w = blockIdx.x; ok && next_work(p, w, wk); w += gridDim.x, ++seq) {
            const int M = wk.it.M - wk.it.tm * UM_BM;  // rows of the segment from this block on
            const int N = wk.it.N;
            const int64_t cbase = (int64_t)wk.head * p.Dout + wk.it.offC + (int64_t)wk.it.tm * UM_BM * N;
            volatile float* xm = xch + (seq & 1) * (2 * UM_SPLIT * 128);  // [part][row] maxima, then [UM_SPLIT + part][row] sums
            if (!softmax) {
                for (int ch = 0; ok && ch < wk.nchunks; ++ch, ++slot) {
                    const int buf = slot & 1;
                    if (!mbar_wait(tfull_bar(buf), (slot >> 1) & 1u, abort_flag, p.status, 4, lim)) { ok = false; break; }
                    tc_fence_after();
                    const int ncols = min(N - ch * UM_BN, UM_BN);
                    const int lo = h * CB, hi = min(lo + CB, ncols);
                    if (lo < hi)
                        store_cols(ch * UM_BN + lo, ch * UM_BN + hi,
                                   [&](int c) { return (uint32_t)(buf * UM_BN + (c - ch * UM_BN)); },
                                   [&](float x) { return x * sl; }, cbase, M, N);
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(tempty_bar(buf));
                }
            } else if (wk.sweeps == 1) {
                // whole row resident: chunk k of the row sits in accumulator (slot + k) & 1
                for (int ch = 0; ok && ch < wk.nchunks; ++ch)
                    if (!mbar_wait(tfull_bar((slot + ch) & 1), ((slot + ch) >> 1) & 1u, abort_flag, p.status, 5, lim)) ok = false;
                if (!ok) break;
                tc_fence_after();
                auto tcol = [&](int c) {  // tensor-memory column of row column c
                    return (uint32_t)((((slot + (c >> 8)) & 1) * UM_BN) + (c & (UM_BN - 1)));
                };
                uint32_t r[32];
                // pass 1: maximum over this half's blocks
                float mx = -INFINITY;
                for (int b0 = h * CB; b0 < N; b0 += UM_BN) {
                    const int bend = min(b0 + CB, N);
                    for (int c = b0; c < bend; c += UM_PIECE) {
                        tc_ld32(lane_addr + tcol(c), r);
                        if (c + 32 <= bend) {
#pragma unroll
                            for (int i = 0; i < 32; i += 2)
                                mx = fmaxf(mx, fmaxf(__uint_as_float(r[i]), __uint_as_float(r[i + 1])));
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
                for (int b0 = h * CB; b0 < N; b0 += UM_BN) {
                    const int bend = min(b0 + CB, N);
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
                // pass 3: normalise and store
                for (int b0 = h * CB; b0 < N; b0 += UM_BN)
                    store_cols(b0, min(b0 + CB, N), tcol, [&](float x) { return x * inv; }, cbase, M, N);
                tc_fence_before();
                __syncwarp();
                for (int ch = 0; ch < wk.nchunks; ++ch)
                    if (lane == 0) mbar_arrive(tempty_bar((slot + ch) & 1));
                slot += wk.nchunks;
            } else {
                // two sweeps: running (max, sum) over this half's blocks, then recompute and store
                float mx = -INFINITY, sum = 0.f;
                uint32_t r[32];
                for (int ch = 0; ok && ch < wk.nchunks; ++ch, ++slot) {
                    const int buf = slot & 1;
                    if (!mbar_wait(tfull_bar(buf), (slot >> 1) & 1u, abort_flag, p.status, 6, lim)) { ok = false; break; }
                    tc_fence_after();
                    const int ncols = min(N - ch * UM_BN, UM_BN);
                    const int lo = h * CB, hi = min(lo + CB, ncols);
                    for (int c = lo; c < hi; c += UM_PIECE) {
                        tc_ld32(lane_addr + (uint32_t)(buf * UM_BN + c), r);
                        const bool part = c + 32 > hi;
                        if (part) {
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                if (c + i >= hi) r[i] = 0xff800000u;  // -inf
                        }
                        float pm = -INFINITY;
#pragma unroll
                        for (int i = 0; i < 32; i += 2)
                            pm = fmaxf(pm, fmaxf(__uint_as_float(r[i]), __uint_as_float(r[i + 1])));
                        const float mnew = fmaxf(mx, pm);  // finite: column c of the piece is inside the row
                        const float nm = -mnew * sl;
                        float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                        for (int i = 0; i < 32; ++i) s4[i & 3] += blk_exp2(fmaf(__uint_as_float(r[i]), sl, nm));
                        sum = sum * blk_exp2((mx - mnew) * sl) + ((s4[0] + s4[1]) + (s4[2] + s4[3]));
                        mx = mnew;
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(tempty_bar(buf));
                }
                if (!ok) break;
                xm[h * 128 + myrow] = mx;
                xm[(UM_SPLIT + h) * 128 + myrow] = sum;
                if (!pair_sync()) break;
                {
                    float m = -INFINITY;
#pragma unroll
                    for (int o = 0; o < UM_SPLIT; ++o) m = fmaxf(m, xm[o * 128 + myrow]);
                    float l = 0.f;
#pragma unroll
                    for (int o = 0; o < UM_SPLIT; ++o)
                        l += xm[(UM_SPLIT + o) * 128 + myrow] * blk_exp2((xm[o * 128 + myrow] - m) * sl);
                    mx = m;
                    sum = l;
                }
                const float off = -mx * sl - __log2f(sum);  // exp2(x * sl + off) = exp2((x - max) * sl) / sum: no multiply after the exponential
                for (int ch = 0; ok && ch < wk.nchunks; ++ch, ++slot) {
                    const int buf = slot & 1;
                    if (!mbar_wait(tfull_bar(buf), (slot >> 1) & 1u, abort_flag, p.status, 7, lim)) { ok = false; break; }
                    tc_fence_after();
                    const int ncols = min(N - ch * UM_BN, UM_BN);
                    const int lo = h * CB, hi = min(lo + CB, ncols);
                    if (lo < hi)
                        store_cols(ch * UM_BN + lo, ch * UM_BN + hi,
                                   [&](int c) { return (uint32_t)(buf * UM_BN + (c - ch * UM_BN)); },
                                   [&](float x) { return blk_exp2(fmaf(x, sl, off)); }, cbase, M, N);
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(tempty_bar(buf));
                }
            }
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

template <typename Tag, bool OUT32>
cudaError_t launch(const BlkUmmaParams& p, const CUtensorMap& a, const CUtensorMap& b, int sms, cudaStream_t st) {
    auto kern = blk_gemm_umma_kernel<Tag, OUT32>;
    cudaError_t e = blk_func_smem(reinterpret_cast<const void*>(kern), UM_SMEM_BYTES);
    if (e != cudaSuccess) return e;
    const int64_t total = (int64_t)p.num_items * p.H;
    const dim3 grid((unsigned)(total < sms ? total : sms)), block(UM_THREADS);
    kern<<<grid, block, UM_SMEM_BYTES, st>>>(p, a, b);
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

cudaError_t blk_launch_gemm_umma(const BlkUmmaParams& p_in, const void* A, const void* B, const BlkOperandLayout& layA,
                                 const BlkOperandLayout& layB, int sms, cudaStream_t st) {
    if ((int64_t)p_in.num_items * p_in.H == 0) return cudaSuccess;
    BlkUmmaParams p = p_in;
    CUtensorMap mapA, mapB;
    if (!blk_make_row_map(&mapA, A, p.bf16, p.K, p.H, layA, UM_BK, UM_BM, &p.head_firstA) ||
        !blk_make_row_map(&mapB, B, p.bf16, p.K, p.H, layB, UM_BK, UM_BN, &p.head_firstB))
        return cudaErrorInvalidValue;
    if (p.bf16) return p.out_f32 ? launch<BlkBf16Tag, true>(p, mapA, mapB, sms, st) : launch<BlkBf16Tag, false>(p, mapA, mapB, sms, st);
    return p.out_f32 ? launch<BlkHalfTag, true>(p, mapA, mapB, sms, st) : launch<BlkHalfTag, false>(p, mapA, mapB, sms, st);
}
