// Fused attention for segments of any length on the 5th-generation tensor cores:
// out_s = softmax(scale * Q_s K_s^T) V_s per segment and head, head dimension 64 or
// 128, without the probabilities ever leaving the SM.
//
// A persistent CTA (one per SM, 14 warps) walks a static list of work items, an item
// being a 128-row block of the queries of one segment of one head; it sweeps the
// segment's keys and values in tiles of 128 rows.  Roles:
//   warp 0      producer: one lane issues tiled TMA loads (128-byte swizzle) of the query
//               block and, into two rings of stages, of the key tiles and value tiles;
//   warp 1      MMA: one lane issues tcgen05.mma.  S = Q K^T (both operands K-major from
//               shared memory) goes to one of two 128-column score buffers in tensor
//               memory; O += P V takes P from tensor memory (first operand [tmem], two
//               16-bit elements per column, row = lane) and V from shared memory as
//               loaded, i.e. MN-major, and accumulates in one of two result buffers
//               (items alternate).  The products of tile g+1 are issued before P V of
//               tile g, across item boundaries, so the tensor pipe has work while the
//               softmax warps are busy with tile g;
//   warps 2-9   softmax: thread (quarter q, lane) owns row 32 q + lane of the block; the
//               two warps of a quarter each take 64 of the 128 columns of a tile and meet
//               on an mbarrier to exchange row maxima.  Online softmax with a lazy
//               reference: the running row maximum is only moved (and O rescaled in
//               tensor memory) when the new maximum exceeds it by more than 8 in the
//               exponent, so P <= 2^8 and the rescale is rare.  P, rounded to the input
//               type, overwrites the first 64 columns of the tile's score buffer (Q K^T
//               of tile g+2 is issued after P V of tile g and overwrites it in pipe
//               order).  After an item's last tile the warps leave the row sums in shared
//               memory and go on to the next item;
//   warps 10-13 output: wait for the item's last P V and the row sums, read O, divide and
//               store the rows, then hand the result buffer back.
//
// Rows of the tiles past the end of a segment belong to its neighbour (or are zero
// past the end of the buffer): extra query rows are never stored, extra key columns
// are masked before the row maximum, and the value rows of the last partial group of
// 16 are cleared in shared memory, so nothing outside the segment reaches a result.
//
// Every wait is bounded: when the bound is hit the kernel records a status code, all
// roles leave their loops, tensor memory is released and the kernel returns.
//
// Upstream has no fused operator; this replaces the chain blockGEMM -> blockSoftmax ->
// blockGEMM(P, V) of its two operators (blockedAttention/apply.py:6-41) for the
// attention use they are built for.
#include <cuda.h>

#include "blk_device.cuh"
#include "blk_kernels.h"
#include "blk_umma_ptx.cuh"

namespace {

constexpr int FA_BM = BLK_FLASH_BM;  // query rows per work item
constexpr int FA_BN = 128;           // key / value rows per tile
// Softmax warps per accumulator-lane quarter: each takes 128 / FA_SPLIT key columns of a tile.  Two; four (22 warps of 80
// registers) measured the same on the long batches and 2 % slower at d = 128 -- this kernel waits on the chain
// QK^T -> softmax -> PV of a tile, not on the softmax warps' throughput.
#ifndef FA_SPLIT_N
#define FA_SPLIT_N 2
#endif
constexpr int FA_SPLIT = FA_SPLIT_N;
constexpr int FA_SOFT_WARPS = 4 * FA_SPLIT;
constexpr int FA_OUT_WARPS = 4;
constexpr int FA_THREADS = 64 + 32 * (FA_SOFT_WARPS + FA_OUT_WARPS);
constexpr int FA_BLOCK_BYTES = 128 * 128;  // 128 rows of one 64-column block: 16 KB
constexpr int FA_O_COL = 256;              // tensor-memory columns of the two result accumulators: 256 and 384
constexpr float FA_LAZY = 8.f;             // exponent slack before the running maximum moves

template <int D>
struct FL {
    static constexpr int NB = D / 64;                       // 64-column blocks of an operand row
    static constexpr int KS = D == 64 ? 5 : 3;              // key ring
    static constexpr int VS = D == 64 ? 5 : 2;              // value ring (a deeper one measured slower)
    static constexpr int OPER_BYTES = NB * FA_BLOCK_BYTES;  // a 128 x D tile
    static constexpr int Q_OFF = 0;
    static constexpr int K_OFF = OPER_BYTES;
    static constexpr int V_OFF = K_OFF + KS * OPER_BYTES;
    static constexpr int XCH_OFF = V_OFF + VS * OPER_BYTES;
    static constexpr int XCH_BYTES = 2 * FA_SPLIT * 128 * 4;  // row maxima: [exchange parity][part][row]
    static constexpr int LSUM_OFF = XCH_OFF + XCH_BYTES;
    static constexpr int LSUM_BYTES = 2 * FA_SPLIT * 128 * 4; // row sums for the output warps: [result buffer][part][row]
    static constexpr int BAR_OFF = LSUM_OFF + LSUM_BYTES;
    static constexpr int SMEM_BYTES = BAR_OFF + 512;
    static_assert(KS <= 6 && VS <= 6, "barrier slots");
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
};

struct FaWork {
    BlkFlashItem it;
    int head;
    int T;  // key/value tiles
};

__device__ __forceinline__ bool fa_work(const BlkFlashParams& p, uint32_t w, FaWork& wk) {
    const uint32_t total = (uint32_t)p.num_items * (uint32_t)p.H;
    if (w >= total) return false;
    const uint32_t item = w / (uint32_t)p.H;
    wk.head = (int)(w - item * (uint32_t)p.H);
    wk.it = p.items[item];
    wk.T = (wk.it.N + FA_BN - 1) / FA_BN;
    return true;
}

template <typename Tag, int D>
__global__ void __launch_bounds__(FA_THREADS, 1)
blk_attn_umma_kernel(const BlkFlashParams p, const __grid_constant__ CUtensorMap mapQ,
                     const __grid_constant__ CUtensorMap mapK, const __grid_constant__ CUtensorMap mapV) {
    using L = FL<D>;
    constexpr int KS = L::KS, VS = L::VS;
    extern __shared__ __align__(1024) unsigned char fa_smem_raw[];
    unsigned char* smem = fa_smem_raw;
    if (blk_smem_u32(smem) & 1023u) {  // the swizzled tiles rely on a 1024-byte aligned base
        if (threadIdx.x == 0) atomicCAS(p.status, 0, 29);
        return;
    }
    float* xch = reinterpret_cast<float*>(smem + L::XCH_OFF);
    float* lsum = reinterpret_cast<float*>(smem + L::LSUM_OFF);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
    // barriers: 0 q_full, 1 q_empty, 2.. p_full[2], 4.. pv_done[2], 6.. s_full[2], 8.. o_ready[2], 10.. o_free[2],
    // 12.. l_ready[2], 14.. one per accumulator-lane quarter, on which its two softmax warps meet, 18.. k_full[KS],
    // 24.. k_empty[KS], 30.. v_full[VS], 36.. v_empty[VS]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 42);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 43);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t smem_u32 = blk_smem_u32(smem);
    const uint32_t bar0 = blk_smem_u32(bars);
    const uint32_t q_full = bar0, q_empty = bar0 + 8;
    auto p_full = [&](int b) { return bar0 + 8u * (2 + b); };
    auto pv_done = [&](int b) { return bar0 + 8u * (4 + b); };
    auto s_full = [&](int b) { return bar0 + 8u * (6 + b); };
    auto o_ready = [&](int b) { return bar0 + 8u * (8 + b); };
    auto o_free = [&](int b) { return bar0 + 8u * (10 + b); };
    auto l_ready = [&](int b) { return bar0 + 8u * (12 + b); };
    auto k_full = [&](int s) { return bar0 + 8u * (18 + s); };
    auto k_empty = [&](int s) { return bar0 + 8u * (24 + s); };
    auto v_full = [&](int s) { return bar0 + 8u * (30 + s); };
    auto v_empty = [&](int s) { return bar0 + 8u * (36 + s); };
    const uint32_t sQ = smem_u32 + L::Q_OFF;
    auto sK = [&](int s) { return smem_u32 + L::K_OFF + s * L::OPER_BYTES; };
    auto sV = [&](int s) { return smem_u32 + L::V_OFF + s * L::OPER_BYTES; };

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        mbar_init(q_empty, 1);
        for (int b = 0; b < 2; ++b) {
            mbar_init(p_full(b), FA_SOFT_WARPS);
            mbar_init(pv_done(b), 1);
            mbar_init(s_full(b), 1);
            mbar_init(o_ready(b), 1);
            mbar_init(o_free(b), FA_OUT_WARPS);
            mbar_init(l_ready(b), FA_SOFT_WARPS);
        }
        for (int i = 0; i < 4; ++i) mbar_init(bar0 + 8u * (14 + i), FA_SPLIT);
        for (int s = 0; s < KS; ++s) {
            mbar_init(k_full(s), 1);
            mbar_init(k_empty(s), 1);
        }
        for (int s = 0; s < VS; ++s) {
            mbar_init(v_full(s), 1);
            mbar_init(v_empty(s), 1);
        }
        *abort_flag = 0;
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

    if (warp == 0) {
        // ---------------- producer ----------------
        if (lane == 0) {
            uint32_t g = 0, itc = 0;
            FaWork wk;
            bool ok = true;
            auto load_tile = [&](uint32_t dst, const CUtensorMap* map, uint32_t bar, int row, int head, int hf) {
                mbar_expect_tx(bar, L::OPER_BYTES);
#pragma unroll
                for (int b = 0; b < L::NB; ++b)  // coordinates (k, row, head), or (k, head, row) for a token-major operand
                    tma_load_3d(dst + b * FA_BLOCK_BYTES, map, bar, 64 * b, hf ? head : row, hf ? row : head);
            };
            for (uint32_t w = blockIdx.x; ok && fa_work(p, w, wk); w += gridDim.x, ++itc) {
                if (!mbar_wait(q_empty, (itc & 1u) ^ 1u, abort_flag, p.status, 21)) break;
                load_tile(sQ, &mapQ, q_full, wk.it.rowQ, wk.head, p.head_firstQ);
                for (int j = 0; j < wk.T; ++j, ++g) {
                    const int ks = (int)(g % KS), vs = (int)(g % VS);
                    if (!mbar_wait(k_empty(ks), ((g / KS) & 1u) ^ 1u, abort_flag, p.status, 22)) { ok = false; break; }
                    load_tile(sK(ks), &mapK, k_full(ks), wk.it.rowKV + j * FA_BN, wk.head, p.head_firstK);
                    if (!mbar_wait(v_empty(vs), ((g / VS) & 1u) ^ 1u, abort_flag, p.status, 20)) { ok = false; break; }
                    load_tile(sV(vs), &mapV, v_full(vs), wk.it.rowKV + j * FA_BN, wk.head, p.head_firstV);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issue ----------------
        if (lane == 0) {
            struct Cur {
                uint32_t w, g, itc;
                int j;
                FaWork wk;
                bool valid;
            };
            auto start = [&](Cur& c) { c.valid = fa_work(p, c.w, c.wk); c.j = 0; };
            auto advance = [&](Cur& c) {
                ++c.g;
                if (++c.j == c.wk.T) {
                    c.w += gridDim.x;
                    ++c.itc;
                    start(c);
                }
            };
            const int neg = p.scale < 0.f;
            const uint32_t idesc_pv = instr_desc(p.bf16, D, 0, 1);
            const uint64_t desc_q = smem_desc_sw128(sQ);
            bool ok = true;
            // S = Q K^T of tile c.g into score buffer g & 1.  The buffer is free: its previous user, tile g - 2, was
            // read by all softmax warps before P V of that tile (issued earlier, executed in order) read the
            // probabilities that overlay it.
            auto issue_qk = [&](const Cur& c) {
                const int ks = (int)(c.g % KS), buf = (int)(c.g & 1u);
                if (c.j == 0 && !mbar_wait(q_full, c.itc & 1u, abort_flag, p.status, 23)) { ok = false; return; }
                if (!mbar_wait(k_full(ks), (c.g / KS) & 1u, abort_flag, p.status, 24)) { ok = false; return; }
                tc_fence_after();
                const int ncols = min(c.wk.it.N - c.j * FA_BN, FA_BN);
                const uint32_t idesc = instr_desc(p.bf16, (ncols + 15) & ~15, neg);
                const uint32_t d_tmem = tmem_base + (uint32_t)(buf * FA_BN);
                // descriptors of the k-th step: the start-address field (16-byte units) moves by 2 per 32 bytes
                // inside a 64-column block and by 1024 per block
                const uint64_t da0 = desc_q, db0 = smem_desc_sw128(sK(ks));
#pragma unroll
                for (int k = 0; k < D / 16; ++k) {
                    const uint64_t o = (uint64_t)((k >> 2) * (FA_BLOCK_BYTES >> 4) + 2 * (k & 3));
                    tc_mma_f16(d_tmem, da0 + o, db0 + o, idesc, k != 0);
                }
                tc_commit(s_full(buf));
                tc_commit(k_empty(ks));                     // key tile reusable
                if (c.j == c.wk.T - 1) tc_commit(q_empty);  // the query block is free once these products have read it
            };
            // O[item & 1] += P V of tile c.g; P sits in the first 64 columns of the tile's score buffer
            auto issue_pv = [&](const Cur& c) {
                const int vs = (int)(c.g % VS), buf = (int)(c.g & 1u), ob = (int)(c.itc & 1u);
                if (c.j == 0 && !mbar_wait(o_free(ob), ((c.itc >> 1) & 1u) ^ 1u, abort_flag, p.status, 19)) { ok = false; return; }
                if (!mbar_wait(p_full(buf), (c.g >> 1) & 1u, abort_flag, p.status, 26)) { ok = false; return; }
                if (!mbar_wait(v_full(vs), (c.g / VS) & 1u, abort_flag, p.status, 27)) { ok = false; return; }
                tc_fence_after();
                const int ncols = min(c.wk.it.N - c.j * FA_BN, FA_BN);
                const int ksteps = (ncols + 15) >> 4;
                const uint32_t d_tmem = tmem_base + (uint32_t)(FA_O_COL + 128 * ob);
                const uint32_t a_tmem = tmem_base + (uint32_t)(buf * FA_BN);
                const uint64_t db0 = smem_desc_sw128_mn(sV(vs), FA_BLOCK_BYTES);
#pragma unroll
                for (int k = 0; k < FA_BN / 16; ++k)  // 16 probabilities of a row are 8 columns; 16 value rows are 2048 bytes
                    if (k < ksteps)
                        tc_mma_f16_ts(d_tmem, a_tmem + 8u * k, db0 + (uint64_t)(128 * k), idesc_pv, (c.j | k) != 0);
                tc_commit(v_empty(vs));                             // value tile reusable
                tc_commit(pv_done(buf));                            // O at rest until the next P V
                if (c.j == c.wk.T - 1) tc_commit(o_ready(ob));     // the item's result is complete
            };
            Cur a, b;
            a.w = b.w = blockIdx.x;
            a.g = b.g = a.itc = b.itc = 0;
            start(a);
            start(b);
            if (a.valid) {
                issue_qk(a);
                advance(a);
            }
            while (ok && b.valid) {
                if (a.valid) {
                    issue_qk(a);
                    if (!ok) break;
                    advance(a);
                }
                issue_pv(b);
                advance(b);
            }
        }
    } else if (warp < 2 + FA_SOFT_WARPS) {
        // ---------------- softmax: warps 2..9 ----------------
        const int q = warp & 3, h = (warp - 2) >> 2;
        const int row = q * 32 + lane;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
        const float sl = fabsf(p.scale) * BLK_LOG2E;  // a negative scale is applied by the MMA (negated Q)
        const uint32_t pair_bar = bar0 + 8u * (14 + q);
        uint32_t xc = 0;
        constexpr int CW = (FA_BN + 0 * D) / FA_SPLIT;  // key columns of a tile this warp owns: 64 or 32 (written as depending on D so that the branches not taken are not instantiated)
        // value a of this row to the other warps of the quarter, the maximum of theirs back
        auto exchange = [&](float a, float& other) -> bool {
            volatile float* x = xch + (xc & 1u) * (FA_SPLIT * 128);
            x[h * 128 + row] = a;
            __syncwarp();
            if (lane == 0) mbar_arrive(pair_bar);  // release: the warp's values are visible to whoever sees the phase end
            const bool good = mbar_wait(pair_bar, xc & 1u, abort_flag, p.status, 28);
            ++xc;
            if (good) {
                other = -INFINITY;
#pragma unroll
                for (int o = 0; o < FA_SPLIT; ++o)
                    if (o != h) other = fmaxf(other, x[o * 128 + row]);
            }
            return good;
        };
        uint32_t g = 0, itc = 0;
        FaWork wk;
        bool ok = true;
        uint32_t ra[32];
        [[maybe_unused]] uint32_t rb[CW == 64 ? 32 : 1];
        for (uint32_t w = blockIdx.x; ok && fa_work(p, w, wk); w += gridDim.x, ++itc) {
            const int ob = (int)(itc & 1u);
            float m_run = -INFINITY, l_run = 0.f;
            for (int j = 0; ok && j < wk.T; ++j, ++g) {
                const int buf = (int)(g & 1u), vs = (int)(g % VS);
                if (!mbar_wait(s_full(buf), (g >> 1) & 1u, abort_flag, p.status, 30)) { ok = false; break; }
                tc_fence_after();
                const uint32_t scol = lane_addr + (uint32_t)(buf * FA_BN + CW * h);
                tc_ld32_nowait(scol, ra);
                if constexpr (CW == 64) tc_ld32_nowait(scol + 32, rb);
                tc_ld_wait();
                const int ncols = min(wk.it.N - j * FA_BN, FA_BN);
                const int lim = ncols - CW * h;  // valid columns of this warp's share
                if (lim < CW) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        if (i >= lim) ra[i] = 0xff800000u;  // -inf
                        if constexpr (CW == 64)
                            if (32 + i >= lim) rb[i] = 0xff800000u;
                    }
                }
                float pm = -INFINITY;
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    pm = fmaxf(pm, fmaxf(__uint_as_float(ra[i]), __uint_as_float(ra[i + 1])));
                    if constexpr (CW == 64) pm = fmaxf(pm, fmaxf(__uint_as_float(rb[i]), __uint_as_float(rb[i + 1])));
                }
                // after this rendezvous all warps of the quarter have their scores in registers, so the
                // probabilities may overwrite the first 64 columns of the score buffer
                float other;
                if (!exchange(pm, other)) { ok = false; break; }
                pm = fmaxf(pm, other);
                const float m_new = fmaxf(m_run, pm);
                const bool move = (m_new - m_run) * sl > FA_LAZY;  // always at the first tile (m_run = -inf)
                float f = 1.f;
                if (move) {
                    f = blk_exp2((m_run - m_new) * sl);
                    m_run = m_new;
                }
                const float nm = -m_run * sl;
                float s4[4] = {0.f, 0.f, 0.f, 0.f};
                uint32_t pk[CW / 2];  // the probabilities, two per word
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    const float e0 = blk_exp2(fmaf(__uint_as_float(ra[i]), sl, nm));
                    const float e1 = blk_exp2(fmaf(__uint_as_float(ra[i + 1]), sl, nm));
                    s4[i & 3] += e0;
                    s4[(i + 1) & 3] += e1;
                    pk[i >> 1] = BlkCvt<Tag>::pack2(e0, e1);
                }
                if constexpr (CW == 64) {
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float e0 = blk_exp2(fmaf(__uint_as_float(rb[i]), sl, nm));
                        const float e1 = blk_exp2(fmaf(__uint_as_float(rb[i + 1]), sl, nm));
                        s4[i & 3] += e0;
                        s4[(i + 1) & 3] += e1;
                        pk[16 + (i >> 1)] = BlkCvt<Tag>::pack2(e0, e1);
                    }
                }
                l_run = l_run * f + ((s4[0] + s4[1]) + (s4[2] + s4[3]));
                // P V of tile g - 2 (long done: the scores of tile g were computed after it); waited for on every
                // tile so that each warp sees the phases of these two barriers in order
                if (g >= 2u && !mbar_wait(pv_done(buf), ((g >> 1) - 1u) & 1u, abort_flag, p.status, 31)) { ok = false; break; }
                if (j > 0 && __any_sync(0xffffffffu, move)) {
                    // a row's reference moved: rescale O, at rest once P V of the previous tile is done
                    if (!mbar_wait(pv_done(buf ^ 1), ((g - 1u) >> 1) & 1u, abort_flag, p.status, 34)) { ok = false; break; }
                    tc_fence_after();
                    // this warp's D / FA_SPLIT columns of the result
                    constexpr int OC = D / FA_SPLIT;
                    if constexpr (OC >= 32) {
#pragma unroll 1
                        for (int c = 0; c < OC; c += 32) {
                            const uint32_t ocol = lane_addr + (uint32_t)(FA_O_COL + 128 * ob + h * OC + c);
                            tc_ld32(ocol, ra);
#pragma unroll
                            for (int i = 0; i < 32; ++i) ra[i] = __float_as_uint(__uint_as_float(ra[i]) * f);
                            tc_st32(ocol, ra);
                        }
                    } else {
                        static_assert(OC == 16 || OC >= 32, "result columns per softmax warp");
                        uint32_t ro[16];
                        const uint32_t ocol = lane_addr + (uint32_t)(FA_O_COL + 128 * ob + h * OC);
                        tc_ld16(ocol, ro);
#pragma unroll
                        for (int i = 0; i < 16; ++i) ro[i] = __float_as_uint(__uint_as_float(ro[i]) * f);
                        tc_st16(ocol, ro);
                    }
                }
                // probabilities of this row, key columns [CW h, CW h + CW): columns [CW/2 h, CW/2 h + CW/2) of the score buffer
                if constexpr (CW == 64) tc_st32(lane_addr + (uint32_t)(buf * FA_BN + 32 * h), pk);
                else tc_st16(lane_addr + (uint32_t)(buf * FA_BN + 16 * h), pk);
                tc_wait_st();
                if (ncols & 15) {
                    // last tile of the segment: clear the value rows between its end and the next multiple of 16
                    if (!mbar_wait(v_full(vs), (g / VS) & 1u, abort_flag, p.status, 32)) { ok = false; break; }
                    const int nz = (16 - (ncols & 15)) * L::NB * 8;  // 16-byte pieces to clear
                    const int t = (warp - 2) * 32 + lane;
                    if (t < nz) {
                        const int rr = t / (L::NB * 8), rem = t % (L::NB * 8);
                        tc_sts_v4(sV(vs) + (rem >> 3) * FA_BLOCK_BYTES + (ncols + rr) * 128 + (rem & 7) * 16, 0u, 0u, 0u, 0u);
                    }
                    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // generic-proxy writes before the MMA's reads
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(p_full(buf));
            }
            if (!ok) break;
            // row sums to the output warps; the slot is free once they have stored the item two before this one
            if (!mbar_wait(o_free(ob), ((itc >> 1) & 1u) ^ 1u, abort_flag, p.status, 33)) break;
            lsum[(ob * FA_SPLIT + h) * 128 + row] = l_run;
            __syncwarp();
            if (lane == 0) mbar_arrive(l_ready(ob));
        }
    } else {
        // ---------------- output: warps 10..13 ----------------
        const int q = warp & 3;
        const int row = q * 32 + lane;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
        uint32_t itc = 0;
        FaWork wk;
        uint32_t r[32];
        for (uint32_t w = blockIdx.x; fa_work(p, w, wk); w += gridDim.x, ++itc) {
            const int ob = (int)(itc & 1u);
            const uint32_t par = (itc >> 1) & 1u;
            if (!mbar_wait(l_ready(ob), par, abort_flag, p.status, 35)) break;
            if (!mbar_wait(o_ready(ob), par, abort_flag, p.status, 36)) break;
            tc_fence_after();
            float lrow = 0.f;
#pragma unroll
            for (int o = 0; o < FA_SPLIT; ++o) lrow += lsum[(ob * FA_SPLIT + o) * 128 + row];
            const float inv = __frcp_rn(lrow);
            // a thread stores its row, 64 bytes at a time
            uint16_t* orow = reinterpret_cast<uint16_t*>(p.out) + (int64_t)wk.head * p.out_head_stride +
                             (int64_t)(wk.it.rowQ + row) * p.out_row_stride;
#pragma unroll 1
            for (int c = 0; c < D; c += 32) {
                tc_ld32(lane_addr + (uint32_t)(FA_O_COL + 128 * ob + c), r);
#pragma unroll
                for (int i = 0; i < 32; i += 2)
                    r[i >> 1] = BlkCvt<Tag>::pack2(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv);
                if (row < wk.it.M) {
                    uint4* dst = reinterpret_cast<uint4*>(orow + c);
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc) dst[cc] = make_uint4(r[4 * cc], r[4 * cc + 1], r[4 * cc + 2], r[4 * cc + 3]);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(o_free(ob));  // result buffer and row-sum slot reusable
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

template <typename Tag, int D>
cudaError_t launch(const BlkFlashParams& p, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, int sms,
                   cudaStream_t st) {
    auto kern = blk_attn_umma_kernel<Tag, D>;
    cudaError_t e = blk_func_smem(reinterpret_cast<const void*>(kern), FL<D>::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    const int64_t total = (int64_t)p.num_items * p.H;
    const dim3 grid((unsigned)(total < sms ? total : sms)), block(FA_THREADS);
    kern<<<grid, block, FL<D>::SMEM_BYTES, st>>>(p, mq, mk, mv);
    return cudaGetLastError();
}

}  // namespace

cudaError_t blk_launch_attn_umma(const BlkFlashParams& p_in, const void* q, const void* k, const void* v, int sms,
                                 cudaStream_t st) {
    if ((int64_t)p_in.num_items * p_in.H == 0) return cudaSuccess;
    if (p_in.D != 64 && p_in.D != 128) return cudaErrorInvalidValue;
    BlkFlashParams p = p_in;
    CUtensorMap mq, mk, mv;
    if (!blk_make_row_map(&mq, q, p.bf16, p.D, p.H, p.layQ, 64, FA_BM, &p.head_firstQ) ||
        !blk_make_row_map(&mk, k, p.bf16, p.D, p.H, p.layK, 64, FA_BN, &p.head_firstK) ||
        !blk_make_row_map(&mv, v, p.bf16, p.D, p.H, p.layV, 64, FA_BN, &p.head_firstV))
        return cudaErrorInvalidValue;
    if (p.D == 64) return p.bf16 ? launch<BlkBf16Tag, 64>(p, mq, mk, mv, sms, st) : launch<BlkHalfTag, 64>(p, mq, mk, mv, sms, st);
    return p.bf16 ? launch<BlkBf16Tag, 128>(p, mq, mk, mv, sms, st) : launch<BlkHalfTag, 128>(p, mq, mk, mv, sms, st);
}
