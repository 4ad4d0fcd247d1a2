// Staged mma.sync kernel of the varlen blocked GEMM: the path that takes every
// 16-bit segment the specialised kernels do not (any M, N, K, any element
// alignment, either operand transposed, fp16/bf16 or fp32 output, scores or
// fused row softmax).
//
// One CTA owns a 64-row block of one segment of one head and a 128-column tile
// of it.  With the softmax epilogue it has 4 warps and warp w owns rows
// 16w..16w+15 across all 128 columns, so a row's reduction never leaves a quad;
// for scores only it has 8 warps (each 16 rows x 64 columns), which doubles the
// resident warps that hide the load latency of short contractions.  Operands are staged through
// shared memory (register-staged double buffer; per operand, segment and head
// either plain 16-byte global loads or, for rows that start at odd element
// offsets, aligned 16-byte loads shifted into place in registers) and fed to
// mma.sync.m16n8k16 through ldmatrix.  With the softmax epilogue the CTA
// sweeps the column tiles of its rows twice -- first keeping only a running
// (max, sum) per row, then recomputing the products and writing normalised
// probabilities -- so the scores never reach global memory; a segment with
// N <= 128 needs one sweep.
//
// Replaces upstream sparseBlockedHGEMM_half / _bf16 (csrc/cuda/spBlkGEMM.cu:424-817)
// and, when fused, sparseBlockedSoftmax_warp/_block (csrc/cuda/spBlkSoftmax.cu:88-269).
#include <type_traits>

#include "blk_device.cuh"
#include "blk_kernels.h"

namespace {

constexpr int BM = BLK_TILE_BM, BN = BLK_TILE_BN, BK = BLK_TILE_BK, NT = 128;
constexpr int A_PITCH_N = BK + 8, A_PITCH_T = BM + 8, B_PITCH_N = BK + 8, B_PITCH_T = BN + 8;
constexpr int A_STAGE = (BM * A_PITCH_N > BK * A_PITCH_T) ? BM * A_PITCH_N : BK * A_PITCH_T;
constexpr int B_STAGE = (BN * B_PITCH_N > BK * B_PITCH_T) ? BN * B_PITCH_N : BK * B_PITCH_T;
constexpr int NJ = BN / 8;  // n8 tiles per warp row block

// Eight consecutive 16-bit elements starting at any element address: the two 16-byte aligned vectors that
// cover them are loaded and the wanted bytes shifted into place.  Elements from nvalid (1..8) on read as zero;
// the second vector is fetched only when a wanted byte lies in it, so no vector without a valid byte is touched.
__device__ __forceinline__ uint4 ldg8_any(const uint16_t* src, int nvalid) {
    const uintptr_t a = reinterpret_cast<uintptr_t>(src);
    const uint4* base = reinterpret_cast<const uint4*>(a & ~static_cast<uintptr_t>(15));
    const uint32_t m = static_cast<uint32_t>(a) & 15u;  // even
    const uint4 v0 = __ldg(base);
    uint4 v1 = make_uint4(0u, 0u, 0u, 0u);
    if ((int)m + 2 * nvalid > 16) v1 = __ldg(base + 1);
    uint32_t w0 = v0.x, w1 = v0.y, w2 = v0.z, w3 = v0.w, w4 = v1.x, w5 = v1.y;
    if (m & 8u) {
        w0 = w2; w1 = w3; w2 = w4; w3 = w5; w4 = v1.z; w5 = v1.w;
    }
    if (m & 4u) {
        w0 = w1; w1 = w2; w2 = w3; w3 = w4; w4 = w5;
    }
    const uint32_t sh = (m & 2u) * 8u;
    uint4 r;
    r.x = __funnelshift_r(w0, w1, sh);
    r.y = __funnelshift_r(w1, w2, sh);
    r.z = __funnelshift_r(w2, w3, sh);
    r.w = __funnelshift_r(w3, w4, sh);
    if (nvalid < 8) {
        auto keep = [&](uint32_t w, int j) { return nvalid >= 2 * j + 2 ? w : (nvalid == 2 * j + 1 ? (w & 0xffffu) : 0u); };
        r.x = keep(r.x, 0); r.y = keep(r.y, 1); r.z = keep(r.z, 2); r.w = keep(r.w, 3);
    }
    return r;
}

// Register staging of an OUTER x INNER tile of a row-major matrix in units of eight 16-bit elements: one
// 16-byte load per unit when the matrix is ALIGNED (16-byte aligned base and a pitch that is a multiple of
// eight elements, so the inner extent is one too), the shifting load above otherwise.
template <int OUTER, int INNER, bool ALIGNED, int NTHR>
struct TileStage {
    static constexpr int UPR = INNER / 8;
    static constexpr int UNITS = OUTER * UPR;
    static constexpr int PT = UNITS / NTHR;
    static_assert(UNITS % NTHR == 0, "tile must divide among the threads");
    uint4 r[PT];

    __device__ __forceinline__ void load(const uint16_t* __restrict__ g, int64_t ld, int o0, int i0, int o_lim,
                                         int i_lim, int tid) {
#pragma unroll
        for (int j = 0; j < PT; ++j) {
            const int u = tid + j * NTHR;
            const int o = o0 + u / UPR, i = i0 + (u % UPR) * 8;
            const uint16_t* src = g + (int64_t)o * ld + i;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (o < o_lim && i < i_lim) {
                if constexpr (ALIGNED) v = blk_ldg16(src);
                else v = ldg8_any(src, min(8, i_lim - i));
            }
            r[j] = v;
        }
    }
    __device__ __forceinline__ void store(uint16_t* s, int pitch, int tid) const {
#pragma unroll
        for (int j = 0; j < PT; ++j) {
            const int u = tid + j * NTHR;
            *reinterpret_cast<uint4*>(s + (u / UPR) * pitch + (u % UPR) * 8) = r[j];
        }
    }
};

// One BK-deep step of a warp's 16 x (8 NJW) block from shared memory: rows 16 wrow.., columns wcol0.. of the tile.
template <typename Tag, bool TA, bool TB, int NJW>
__device__ __forceinline__ void mma_stage(float (&acc)[NJW][4], const uint16_t* sA, const uint16_t* sB, int wrow,
                                          int wcol0, int lane, int ncols) {
#pragma unroll
    for (int ks = 0; ks < BK / 16; ++ks) {
        const int k0 = ks * 16;
        uint32_t a[4];
        if constexpr (!TA) {
            blk_ldmatrix_x4(a, blk_smem_u32(sA + (wrow * 16 + (lane & 15)) * A_PITCH_N + k0 + (lane >> 4) * 8));
        } else {
            blk_ldmatrix_x4_trans(a, blk_smem_u32(sA + (k0 + (lane & 7) + ((lane >> 4) << 3)) * A_PITCH_T +
                                                  wrow * 16 + ((lane >> 3) & 1) * 8));
        }
#pragma unroll
        for (int jp = 0; jp < NJW / 2; ++jp) {
            const int c0 = wcol0 + jp * 16;
            if (c0 < ncols) {
                uint32_t b[4];
                if constexpr (!TB) {
                    blk_ldmatrix_x4(b, blk_smem_u32(sB + (c0 + (lane & 7) + ((lane >> 4) << 3)) * B_PITCH_N + k0 +
                                                    ((lane >> 3) & 1) * 8));
                } else {
                    blk_ldmatrix_x4_trans(b, blk_smem_u32(sB + (k0 + (lane & 7) + ((lane >> 3) & 1) * 8) * B_PITCH_T +
                                                          c0 + ((lane >> 4) << 3)));
                }
                blk_mma16816<Tag>(acc[2 * jp], a[0], a[1], a[2], a[3], b[0], b[1]);
                blk_mma16816<Tag>(acc[2 * jp + 1], a[0], a[1], a[2], a[3], b[2], b[3]);
            }
        }
    }
}

// acc = A[m0.., :] * B[n0.., :]^T for the CTA's 64 x 128 tile.
// NTHR threads: NTHR / 128 warp columns, each warp 16 rows x (BN / warp columns) columns.
template <typename Tag, bool TA, bool TB, bool AA, bool AB, int NTHR>
__device__ __forceinline__ void compute_tile(float (&acc)[NJ * 128 / NTHR][4], const uint16_t* __restrict__ gA,
                                             const uint16_t* __restrict__ gB, int M, int N, int K, int m0, int n0,
                                             uint16_t (*sA)[A_STAGE], uint16_t (*sB)[B_STAGE], int tid) {
    constexpr int NJW = NJ * 128 / NTHR;
#pragma unroll
    for (int j = 0; j < NJW; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    const int nk = (K + BK - 1) / BK;
    if (nk == 0) return;
    const int warp = tid >> 5, lane = tid & 31;
    const int wrow = warp & 3, wcol0 = (warp >> 2) * (8 * NJW);
    const int ncols = min(N - n0, BN);
    const bool active = m0 + wrow * 16 < M && wcol0 < ncols;

    TileStage<TA ? BK : BM, TA ? BM : BK, AA, NTHR> stA;
    TileStage<TB ? BK : BN, TB ? BN : BK, AB, NTHR> stB;
    auto loadA = [&](int k0) {
        if constexpr (!TA) stA.load(gA, K, m0, k0, M, K, tid); else stA.load(gA, M, k0, m0, K, M, tid);
    };
    auto loadB = [&](int k0) {
        if constexpr (!TB) stB.load(gB, K, n0, k0, N, K, tid); else stB.load(gB, N, k0, n0, K, N, tid);
    };
    constexpr int pA = TA ? A_PITCH_T : A_PITCH_N, pB = TB ? B_PITCH_T : B_PITCH_N;

    loadA(0);
    loadB(0);
    stA.store(sA[0], pA, tid);
    stB.store(sB[0], pB, tid);
    __syncthreads();
    for (int kt = 0; kt < nk; ++kt) {
        const int cur = kt & 1;
        const bool more = kt + 1 < nk;
        if (more) {
            loadA((kt + 1) * BK);
            loadB((kt + 1) * BK);
        }
        if (active) mma_stage<Tag, TA, TB, NJW>(acc, sA[cur], sB[cur], wrow, wcol0, lane, ncols);
        if (more) {
            stA.store(sA[cur ^ 1], pA, tid);
            stB.store(sB[cur ^ 1], pB, tid);
        }
        __syncthreads();
    }
}

// Writes the thread's fragment (rows r0 and r0+8, columns n0 + 8j + 2t, +1).
template <typename Tag, int NJW, bool F32>
__device__ __forceinline__ void store_frag_t(void* C, int64_t cbase, const float (&v)[NJW][4], int r0, int M, int N,
                                             int n0, int t, bool pair_ok) {
    typedef typename std::conditional<F32, float, uint16_t>::type E;
    const int c0 = n0 + 2 * t;  // this thread's first column
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = r0 + 8 * h;
        if (r >= M) continue;
        E* row = reinterpret_cast<E*>(C) + (cbase + (int64_t)r * N + c0);  // columns c0 + 8 j, + 1 at row[8 j], [8 j + 1]
        if (pair_ok) {
#pragma unroll
            for (int j = 0; j < NJW; ++j) {
                const float x = v[j][2 * h], y = v[j][2 * h + 1];
                if (c0 + 8 * j + 1 < N) {
                    if constexpr (F32) *reinterpret_cast<float2*>(row + 8 * j) = make_float2(x, y);
                    else *reinterpret_cast<uint32_t*>(row + 8 * j) = BlkCvt<Tag>::pack2(x, y);
                } else if (c0 + 8 * j < N) {
                    if constexpr (F32) row[8 * j] = x;
                    else row[8 * j] = BlkCvt<Tag>::pack1(x);
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < NJW; ++j) {
                const float x = v[j][2 * h], y = v[j][2 * h + 1];
                if (c0 + 8 * j < N) {
                    if constexpr (F32) row[8 * j] = x;
                    else row[8 * j] = BlkCvt<Tag>::pack1(x);
                }
                if (c0 + 8 * j + 1 < N) {
                    if constexpr (F32) row[8 * j + 1] = y;
                    else row[8 * j + 1] = BlkCvt<Tag>::pack1(y);
                }
            }
        }
    }
}
template <typename Tag, int NJW>
__device__ __forceinline__ void store_frag(void* C, int out_f32, int64_t cbase, const float (&v)[NJW][4], int r0, int M,
                                           int N, int n0, int t, bool pair_ok) {
    if (out_f32) store_frag_t<Tag, NJW, true>(C, cbase, v, r0, M, N, n0, t, pair_ok);
    else store_frag_t<Tag, NJW, false>(C, cbase, v, r0, M, N, n0, t, pair_ok);
}

template <typename Tag, bool TA, bool TB, bool AA, bool AB>
__device__ __forceinline__ void tile_body(const BlkGemmParams& p, const BlkSeg& sd, const BlkTileItem& it,
                                          const uint16_t* gA, const uint16_t* gB, int64_t cbase,
                                          uint16_t (*sA)[A_STAGE], uint16_t (*sB)[B_STAGE]) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int M = sd.M, N = sd.N, K = sd.K;
    const int m0 = it.tm * BM;
    const int r0 = m0 + warp * 16 + g;
    const bool pair_ok = ((cbase & 1) == 0) && ((N & 1) == 0);
    float acc[NJ][4];

    // softmax epilogue, base-2 domain
    const float sl = p.scale * BLK_LOG2E;
    float mrun[2] = {-INFINITY, -INFINITY}, lrun[2] = {0.f, 0.f};
    for (int tn = 0; tn < it.ntn; ++tn) {
        const int n0 = tn * BN;
        compute_tile<Tag, TA, TB, AA, AB, NT>(acc, gA, gB, M, N, K, m0, n0, sA, sB, tid);
        float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            const int col = n0 + 8 * j + 2 * t;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float s = (col + (e & 1) < N) ? acc[j][e] * sl : -INFINITY;
                acc[j][e] = s;
                tmax[e >> 1] = fmaxf(tmax[e >> 1], s);
            }
        }
        if (it.ntn == 1) {
            // whole row in this tile: finish in registers
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const float mx = blk_quad_max(tmax[h]);
                float sum = 0.f;
#pragma unroll
                for (int j = 0; j < NJ; ++j) {
                    acc[j][2 * h] = blk_exp2(acc[j][2 * h] - mx);
                    acc[j][2 * h + 1] = blk_exp2(acc[j][2 * h + 1] - mx);
                    sum += acc[j][2 * h] + acc[j][2 * h + 1];
                }
                const float inv = 1.f / blk_quad_sum(sum);
#pragma unroll
                for (int j = 0; j < NJ; ++j) {
                    acc[j][2 * h] *= inv;
                    acc[j][2 * h + 1] *= inv;
                }
            }
            store_frag<Tag, NJ>(p.C, p.out_f32, cbase, acc, r0, M, N, 0, t, pair_ok);
            return;
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const float mnew = fmaxf(mrun[h], tmax[h]);
            if (mnew > -INFINITY) {
                float sum = 0.f;
#pragma unroll
                for (int j = 0; j < NJ; ++j) sum += blk_exp2(acc[j][2 * h] - mnew) + blk_exp2(acc[j][2 * h + 1] - mnew);
                lrun[h] = lrun[h] * blk_exp2(mrun[h] - mnew) + sum;
                mrun[h] = mnew;
            }
        }
    }
    float inv[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const float mx = blk_quad_max(mrun[h]);
        const float part = (mrun[h] > -INFINITY) ? lrun[h] * blk_exp2(mrun[h] - mx) : 0.f;
        inv[h] = 1.f / blk_quad_sum(part);
        mrun[h] = mx;
    }
    for (int tn = 0; tn < it.ntn; ++tn) {
        const int n0 = tn * BN;
        compute_tile<Tag, TA, TB, AA, AB, NT>(acc, gA, gB, M, N, K, m0, n0, sA, sB, tid);
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[j][e] = blk_exp2(acc[j][e] * sl - mrun[e >> 1]) * inv[e >> 1];
        }
        store_frag<Tag, NJ>(p.C, p.out_f32, cbase, acc, r0, M, N, n0, t, pair_ok);
    }
}

// Scores only: eight warps per tile (four row blocks x two column halves), so twice the warps of the softmax
// layout are resident per SM to hide the global-load latency of short contractions.
constexpr int NT_SC = 256;
template <typename Tag, bool TA, bool TB, bool AA, bool AB>
__device__ __forceinline__ void scores_body(const BlkGemmParams& p, const BlkSeg& sd, const BlkTileItem& it,
                                            const uint16_t* gA, const uint16_t* gB, int64_t cbase,
                                            uint16_t (*sA)[A_STAGE], uint16_t (*sB)[B_STAGE]) {
    constexpr int NJW = NJ * 128 / NT_SC;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int M = sd.M, N = sd.N, K = sd.K;
    const int m0 = it.tm * BM, n0 = it.tn * BN;
    const int r0 = m0 + (warp & 3) * 16 + g;
    const bool pair_ok = ((cbase & 1) == 0) && ((N & 1) == 0);
    float acc[NJW][4];
    compute_tile<Tag, TA, TB, AA, AB, NT_SC>(acc, gA, gB, M, N, K, m0, n0, sA, sB, tid);
#pragma unroll
    for (int j = 0; j < NJW; ++j) {
        acc[j][0] *= p.scale; acc[j][1] *= p.scale; acc[j][2] *= p.scale; acc[j][3] *= p.scale;
    }
    store_frag<Tag, NJW>(p.C, p.out_f32, cbase, acc, r0, M, N, n0 + (warp >> 2) * (8 * NJW), t, pair_ok);
}

// SOFTMAX: the fused two-sweep kernel (four warps); otherwise the scores kernel (eight warps).  The scores kernel
// without transposed operands is held to 64 registers (a few spills) for a fourth resident CTA: its tiles are bound
// by the latency of their load chain, and one more tile in flight measured 8 % faster; the transposed variants
// measured slower that way.
template <typename Tag, bool TA, bool TB, bool SOFTMAX>
__global__ void __launch_bounds__(SOFTMAX ? NT : NT_SC, (SOFTMAX || TA || TB) ? 3 : 4) blk_gemm_tile_kernel(const BlkGemmParams p) {
    __shared__ __align__(16) uint16_t sA[2][A_STAGE];
    __shared__ __align__(16) uint16_t sB[2][B_STAGE];
    const int64_t bid = blockIdx.x;
    const int head = (int)(bid / p.num_items);
    const BlkTileRec rec = p.recs[bid % p.num_items];
    const BlkTileItem it = rec.it;
    const BlkSeg sd = rec.sd;
    const int64_t baseA = (int64_t)head * p.Dm1 + sd.offA, baseB = (int64_t)head * p.Dm2 + sd.offB;
    const int64_t cbase = (int64_t)head * p.Dout + sd.offC;
    const uint16_t* gA = p.A + baseA;
    const uint16_t* gB = p.B + baseB;
    const int64_t pitchA = TA ? sd.M : sd.K, pitchB = TB ? sd.N : sd.K;
    // per operand: plain 16-byte loads when every row of this (segment, head) starts on a 16-byte boundary
    const bool alignedA = ((baseA | pitchA) & 7) == 0, alignedB = ((baseB | pitchB) & 7) == 0;
    auto body = [&](auto aa, auto ab) {
        if constexpr (SOFTMAX) tile_body<Tag, TA, TB, decltype(aa)::value, decltype(ab)::value>(p, sd, it, gA, gB, cbase, sA, sB);
        else scores_body<Tag, TA, TB, decltype(aa)::value, decltype(ab)::value>(p, sd, it, gA, gB, cbase, sA, sB);
    };
    if (alignedA) {
        if (alignedB) body(std::true_type{}, std::true_type{});
        else body(std::true_type{}, std::false_type{});
    } else {
        if (alignedB) body(std::false_type{}, std::true_type{});
        else body(std::false_type{}, std::false_type{});
    }
}

template <typename Tag, bool SOFTMAX>
cudaError_t launch_epi(const BlkGemmParams& p, int ta, int tb, cudaStream_t st) {
    const int64_t blocks = (int64_t)p.num_items * p.H;
    const dim3 grid((unsigned)blocks), block(SOFTMAX ? NT : NT_SC);
    if (!ta && !tb) blk_gemm_tile_kernel<Tag, false, false, SOFTMAX><<<grid, block, 0, st>>>(p);
    else if (!ta && tb) blk_gemm_tile_kernel<Tag, false, true, SOFTMAX><<<grid, block, 0, st>>>(p);
    else if (ta && !tb) blk_gemm_tile_kernel<Tag, true, false, SOFTMAX><<<grid, block, 0, st>>>(p);
    else blk_gemm_tile_kernel<Tag, true, true, SOFTMAX><<<grid, block, 0, st>>>(p);
    return cudaGetLastError();
}

template <typename Tag>
cudaError_t launch_tag(const BlkGemmParams& p, int ta, int tb, cudaStream_t st) {
    if ((int64_t)p.num_items * p.H == 0) return cudaSuccess;
    return p.epi == BLK_EPI_SOFTMAX ? launch_epi<Tag, true>(p, ta, tb, st) : launch_epi<Tag, false>(p, ta, tb, st);
}

}  // namespace

cudaError_t blk_launch_gemm_tile(const BlkGemmParams& p, int dtype_in, int ta, int tb, cudaStream_t st) {
    return dtype_in == BLK_F16 ? launch_tag<BlkHalfTag>(p, ta, tb, st) : launch_tag<BlkBf16Tag>(p, ta, tb, st);
}
