// Second product of blocked attention on the 5th-generation tensor cores:
// out_s (M x D) = scale * A_s (M x K) B_s (K x D) per segment and head, where the rows of
// the first operand have an arbitrary length K and start at arbitrary 2-byte
// offsets (a block of probabilities P_s of a packed (M_s, N_s) score buffer, K =
// N_s) and the second operand is stored (K, D) with D = 64 or 128 (the values V_s
// of a segment: upstream's transpose2 = true).
//
// The rows of P cannot be fetched by TMA (a tensor map needs 16-byte aligned row
// pitches; a packed score block has whatever pitch its segment has), so they take
// another road into the tensor core: loader warps read them with aligned 16-byte
// loads, shift them into place in registers and store them into tensor memory,
// from where tcgen05.mma takes them as its first operand ([tmem], 16-bit elements,
// two per column, row = lane).  The values are fetched by tiled TMA exactly as
// they lie (MN-major second operand, 128-byte swizzle).
//
// A persistent CTA (one per SM, 22 warps) walks a static list of work items, an
// item being a 128-row block of the first operand of one segment of one head; it
// sweeps the contraction index in tiles of 128.  Roles:
//   warp 0      producer: one lane issues the TMA loads of the value tiles into a ring;
//   warp 1      MMA: one lane issues O += P V for each tile, P from one of two
//               64-column buffers in tensor memory, O in one of two accumulators
//               (items alternate); tcgen05.commit frees the value stage and the P
//               buffer and, after an item's last tile, hands O to the output warps;
//   warps 2-17  loaders, two groups of eight, one per P buffer (so a group takes every other
//               tile and the global loads of two tiles are in flight at a time): thread
//               (quarter q, lane) owns row 32 q + lane of the block; the two warps of a
//               quarter in a group each bring 64 of the 128 columns of a tile;
//   warps 18-21 output: read O, scale, round and store the rows (a row of the result is
//               D contiguous, 16-byte aligned elements).
//
// Columns of a tile past the end of a row (K) and rows past the end of the block
// (M) are loaded as zeros, and the value rows between K and the next multiple of
// 16 are cleared in shared memory, so nothing outside the segment reaches a result.
// Every wait is bounded: when the bound is hit the kernel records a status code,
// all roles leave their loops, tensor memory is released and the kernel returns.
//
// Replaces upstream sparseBlockedHGEMM_half / _bf16 with transpose2 = true
// (csrc/cuda/spBlkGEMM.cu:424-817) for the product it is used for after the
// softmax, blockGEMM(P, V, ..., transpose2=True) (blockedAttention/apply.py:6-25).
#include <cuda.h>

#include "blk_device.cuh"
#include "blk_kernels.h"
#include "blk_umma_ptx.cuh"

namespace {

static_assert(BLK_UMMA_BM == 128, "a work item is a block of 128 rows: one accumulator lane per row");
constexpr int PV_BK = 128;           // contraction elements per tile
constexpr int PV_LOAD_WARPS = 8;     // loader warps of a group: four lane quarters x two halves of a tile's 128 columns
#ifndef PV_GROUPS_N
#define PV_GROUPS_N 2
#endif
constexpr int PV_GROUPS = PV_GROUPS_N;  // groups of loader warps, one per tensor-memory buffer: their loads are in flight together
                                        // (two: 13 % faster than one; three measured the same as two)
constexpr int PV_PBUFS = PV_GROUPS > 2 ? PV_GROUPS : 2;  // buffers of the first operand in tensor memory, 64 columns each
static_assert(PV_PBUFS <= 4, "the first-operand buffers lie below the result accumulators (column 256)");
constexpr int PV_OUT_WARPS = 4;
constexpr int PV_THREADS = 64 + 32 * (PV_LOAD_WARPS * PV_GROUPS + PV_OUT_WARPS);
constexpr int PV_BLOCK_BYTES = 128 * 128;  // 128 value rows of one 64-column block: 16 KB
constexpr int PV_O_COL = 256;              // tensor-memory columns of the two result accumulators: 256 and 384

template <int D>
struct PVL {
    static constexpr int NB = D / 64;                       // 64-column blocks of a value row
    static constexpr int VS = D == 64 ? 6 : 4;              // value ring
    static constexpr int OPER_BYTES = NB * PV_BLOCK_BYTES;  // a 128 x D tile
    static constexpr int V_OFF = 0;
    static constexpr int BAR_OFF = VS * OPER_BYTES;
    static constexpr int SMEM_BYTES = BAR_OFF + 512;
    static_assert(VS <= 6, "barrier slots");
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
};

struct PvWork {
    BlkPvItem it;
    int head;
    int T;  // tiles of the contraction index
};

__device__ __forceinline__ bool pv_work(const BlkPvParams& p, uint32_t w, PvWork& wk) {
    const uint32_t total = (uint32_t)p.num_items * (uint32_t)p.H;
    if (w >= total) return false;
    const uint32_t item = w / (uint32_t)p.H;
    wk.head = (int)(w - item * (uint32_t)p.H);
    wk.it = p.items[item];
    wk.T = (wk.it.K + PV_BK - 1) / PV_BK;
    return true;
}

__device__ __forceinline__ uint4 ldg_v4_if(const void* ptr, bool ok) {
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (ok) v = __ldg(reinterpret_cast<const uint4*>(ptr));
    return v;
}

template <typename Tag, int D>
__global__ void __launch_bounds__(PV_THREADS, 1)
blk_pv_umma_kernel(const BlkPvParams p, const __grid_constant__ CUtensorMap mapV) {
    using L = PVL<D>;
    constexpr int VS = L::VS;
    extern __shared__ __align__(1024) unsigned char pv_smem_raw[];
    unsigned char* smem = pv_smem_raw;
    if (blk_smem_u32(smem) & 1023u) {  // the swizzled tiles rely on a 1024-byte aligned base
        if (threadIdx.x == 0) atomicCAS(p.status, 0, 49);
        return;
    }
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
    // barriers: 0.. p_full[4], 4.. p_free[4], 8.. o_ready[2], 10.. o_free[2], 12.. v_full[VS], 18.. v_empty[VS]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 24);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 25);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t smem_u32 = blk_smem_u32(smem);
    const uint32_t bar0 = blk_smem_u32(bars);
    auto p_full = [&](int b) { return bar0 + 8u * (0 + b); };
    auto p_free = [&](int b) { return bar0 + 8u * (4 + b); };
    auto o_ready = [&](int b) { return bar0 + 8u * (8 + b); };
    auto o_free = [&](int b) { return bar0 + 8u * (10 + b); };
    auto v_full = [&](int s) { return bar0 + 8u * (12 + s); };
    auto v_empty = [&](int s) { return bar0 + 8u * (18 + s); };
    auto sV = [&](int s) { return smem_u32 + L::V_OFF + s * L::OPER_BYTES; };

    if (threadIdx.x == 0) {
        for (int b = 0; b < PV_PBUFS; ++b) {
            mbar_init(p_full(b), PV_LOAD_WARPS);
            mbar_init(p_free(b), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(o_ready(b), 1);
            mbar_init(o_free(b), PV_OUT_WARPS);
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
        // ---------------- producer: value tiles ----------------
        if (lane == 0) {
            uint32_t g = 0;
            PvWork wk;
            bool ok = true;
            for (uint32_t w = blockIdx.x; ok && pv_work(p, w, wk); w += gridDim.x) {
                for (int j = 0; j < wk.T; ++j, ++g) {
                    const int vs = (int)(g % VS);
                    if (!mbar_wait(v_empty(vs), ((g / VS) & 1u) ^ 1u, abort_flag, p.status, 41)) { ok = false; break; }
                    mbar_expect_tx(v_full(vs), L::OPER_BYTES);
                    const int row = wk.it.rowB + j * PV_BK;
#pragma unroll
                    for (int b = 0; b < L::NB; ++b)  // coordinates (column, row, head)
                        tma_load_3d(sV(vs) + b * PV_BLOCK_BYTES, &mapV, v_full(vs), 64 * b, row, wk.head);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issue ----------------
        if (lane == 0) {
            const uint32_t idesc = instr_desc(p.bf16, D, 0, 1);  // second operand MN-major
            uint32_t g = 0, itc = 0;
            PvWork wk;
            bool ok = true;
            for (uint32_t w = blockIdx.x; ok && pv_work(p, w, wk); w += gridDim.x, ++itc) {
                const int ob = (int)(itc & 1u);
                if (!mbar_wait(o_free(ob), ((itc >> 1) & 1u) ^ 1u, abort_flag, p.status, 42)) break;
                for (int j = 0; j < wk.T; ++j, ++g) {
                    const int vs = (int)(g % VS), buf = (int)(g % PV_PBUFS);
                    if (!mbar_wait(p_full(buf), (g / PV_PBUFS) & 1u, abort_flag, p.status, 43)) { ok = false; break; }
                    if (!mbar_wait(v_full(vs), (g / VS) & 1u, abort_flag, p.status, 44)) { ok = false; break; }
                    tc_fence_after();
                    const int ncols = min(wk.it.K - j * PV_BK, PV_BK);
                    const int ksteps = (ncols + 15) >> 4;
                    const uint32_t d_tmem = tmem_base + (uint32_t)(PV_O_COL + 128 * ob);
                    const uint32_t a_tmem = tmem_base + (uint32_t)(buf * 64);
                    const uint64_t db0 = smem_desc_sw128_mn(sV(vs), PV_BLOCK_BYTES);
#pragma unroll
                    for (int k = 0; k < PV_BK / 16; ++k)  // 16 elements of a row are 8 columns; 16 value rows are 2048 bytes
                        if (k < ksteps) tc_mma_f16_ts(d_tmem, a_tmem + 8u * k, db0 + (uint64_t)(128 * k), idesc, (j | k) != 0);
                    tc_commit(v_empty(vs));                         // value tile reusable
                    tc_commit(p_free(buf));                         // first-operand buffer reusable
                    if (j == wk.T - 1) tc_commit(o_ready(ob));     // the item's result is complete
                }
            }
        }
    } else if (warp < 2 + PV_LOAD_WARPS * PV_GROUPS) {
        // ---------------- loaders: warps 2..17, group grp fills buffer grp (every other tile) ----------------
        const int lw = (warp - 2) % PV_LOAD_WARPS, grp = (warp - 2) / PV_LOAD_WARPS;
        const int q = warp & 3, h = lw >> 2;
        const int row = q * 32 + lane;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
        const unsigned char* A = reinterpret_cast<const unsigned char*>(p.A);
        uint32_t g = 0;
        PvWork wk;
        bool ok = true;
        for (uint32_t w = blockIdx.x; ok && pv_work(p, w, wk); w += gridDim.x) {
            const int K = wk.it.K;
            const bool row_ok = row < wk.it.M;
            // byte address of this lane's row of the block
            const int64_t rowb = ((int64_t)wk.head * p.Dm1 + wk.it.offA + (int64_t)row * K) * 2;
            for (int j = 0; ok && j < wk.T; ++j, ++g) {
                if (PV_GROUPS > 1 && (int)(g % PV_GROUPS) != grp) continue;  // another group's tile
                const int buf = (int)(g % PV_PBUFS), vs = (int)(g % VS);
                const int ncols = min(K - j * PV_BK, PV_BK);
                const int ksteps = (ncols + 15) >> 4;
                const int nv = row_ok ? max(0, min(ncols - 64 * h, 64)) : 0;   // elements of this lane's 64 that exist
                // 64 elements from byte address b: the aligned 16-byte vectors that hold at least one of them
                const int64_t b = rowb + (int64_t)(j * PV_BK + 64 * h) * 2;
                const int sh = (int)(b & 15);
                const unsigned char* base = A + (b - sh);
                const int need = sh + 2 * nv;  // bytes [sh, need) of the vectors are wanted
                uint32_t v[36];
#pragma unroll
                for (int i = 0; i < 9; ++i) {
                    const uint4 t = ldg_v4_if(base + 16 * i, nv > 0 && 16 * i < need);
                    v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
                }
                // shift by sh bytes: whole words by the case, the odd half word with a funnel shift
                uint32_t pk[32];
                const uint32_t hs = (uint32_t)(sh & 2) * 8u;
                switch (sh >> 2) {
                    case 0:
#pragma unroll
                        for (int i = 0; i < 32; ++i) pk[i] = __funnelshift_r(v[i], v[i + 1], hs);
                        break;
                    case 1:
#pragma unroll
                        for (int i = 0; i < 32; ++i) pk[i] = __funnelshift_r(v[i + 1], v[i + 2], hs);
                        break;
                    case 2:
#pragma unroll
                        for (int i = 0; i < 32; ++i) pk[i] = __funnelshift_r(v[i + 2], v[i + 3], hs);
                        break;
                    default:
#pragma unroll
                        for (int i = 0; i < 32; ++i) pk[i] = __funnelshift_r(v[i + 3], v[i + 4], hs);
                        break;
                }
                if (nv < 64) {
                    // elements past the end of the row (or a row past the end of the block) count as zeros
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        if (2 * i >= nv) pk[i] = 0u;
                        else if (2 * i + 1 >= nv) pk[i] &= 0xffffu;
                    }
                }
                if (!mbar_wait(p_free(buf), ((g / PV_PBUFS) & 1u) ^ 1u, abort_flag, p.status, 45)) { ok = false; break; }
                tc_fence_after();
                // this row's elements [64 h, 64 h + 64) of the tile: columns [32 h, 32 h + 32) of the buffer (only the
                // columns the products of this tile read)
                if (64 * h < 16 * ksteps) {
                    tc_st32(lane_addr + (uint32_t)(buf * 64 + 32 * h), pk);
                    tc_wait_st();
                }
                if (ncols & 15) {
                    // last tile of the row: clear the value rows between its end and the next multiple of 16
                    if (!mbar_wait(v_full(vs), (g / VS) & 1u, abort_flag, p.status, 46)) { ok = false; break; }
                    const int nz = (16 - (ncols & 15)) * L::NB * 8;  // 16-byte pieces to clear
                    const int t = lw * 32 + lane;
                    if (t < nz) {
                        const int rr = t / (L::NB * 8), rem = t % (L::NB * 8);
                        tc_sts_v4(sV(vs) + (rem >> 3) * PV_BLOCK_BYTES + (ncols + rr) * 128 + (rem & 7) * 16, 0u, 0u, 0u, 0u);
                    }
                    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // generic-proxy writes before the MMA's reads
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(p_full(buf));
            }
        }
    } else {
        // ---------------- output: the last four warps ----------------
        const int q = warp & 3;
        const int row = q * 32 + lane;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
        uint32_t itc = 0;
        PvWork wk;
        uint32_t r[32];
        for (uint32_t w = blockIdx.x; pv_work(p, w, wk); w += gridDim.x, ++itc) {
            const int ob = (int)(itc & 1u);
            if (!mbar_wait(o_ready(ob), (itc >> 1) & 1u, abort_flag, p.status, 47)) break;
            tc_fence_after();
            // a thread stores its row, 64 bytes at a time
            uint16_t* orow = reinterpret_cast<uint16_t*>(p.C) + (int64_t)wk.head * p.Dout + wk.it.offC + (int64_t)row * D;
#pragma unroll 1
            for (int c = 0; c < D; c += 32) {
                tc_ld32(lane_addr + (uint32_t)(PV_O_COL + 128 * ob + c), r);
#pragma unroll
                for (int i = 0; i < 32; i += 2)
                    r[i >> 1] = BlkCvt<Tag>::pack2(__uint_as_float(r[i]) * p.scale, __uint_as_float(r[i + 1]) * p.scale);
                if (row < wk.it.M) {
                    uint4* dst = reinterpret_cast<uint4*>(orow + c);
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc) dst[cc] = make_uint4(r[4 * cc], r[4 * cc + 1], r[4 * cc + 2], r[4 * cc + 3]);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(o_free(ob));  // result accumulator reusable
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
cudaError_t launch(const BlkPvParams& p, const CUtensorMap& mv, int sms, cudaStream_t st) {
    auto kern = blk_pv_umma_kernel<Tag, D>;
    cudaError_t e = blk_func_smem(reinterpret_cast<const void*>(kern), PVL<D>::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    const int64_t total = (int64_t)p.num_items * p.H;
    const dim3 grid((unsigned)(total < sms ? total : sms)), block(PV_THREADS);
    kern<<<grid, block, PVL<D>::SMEM_BYTES, st>>>(p, mv);
    return cudaGetLastError();
}

}  // namespace

cudaError_t blk_launch_pv_umma(const BlkPvParams& p, const void* V, int sms, cudaStream_t st) {
    if ((int64_t)p.num_items * p.H == 0) return cudaSuccess;
    if (p.D != 64 && p.D != 128) return cudaErrorInvalidValue;
    CUtensorMap mv;
    int head_first = 0;
    const BlkOperandLayout lay{p.Dm2 / p.D, p.D, p.Dm2};  // the values as a (rows, D) matrix per head strip
    if (!blk_make_row_map(&mv, V, p.bf16, p.D, p.H, lay, 64, PV_BK, &head_first) || head_first) return cudaErrorInvalidValue;
    if (p.D == 64) return p.bf16 ? launch<BlkBf16Tag, 64>(p, mv, sms, st) : launch<BlkHalfTag, 64>(p, mv, sms, st);
    return p.bf16 ? launch<BlkBf16Tag, 128>(p, mv, sms, st) : launch<BlkHalfTag, 128>(p, mv, sms, st);
}
