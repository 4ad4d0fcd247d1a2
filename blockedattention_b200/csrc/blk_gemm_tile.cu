// Staged mma.sync kernel of the varlen blocked GEMM: the path that takes every
// 16-bit segment the specialised kernels do not (any M, N, K, any element
// alignment, either operand transposed, fp16/bf16 or fp32 output, scores or
// fused row softmax).
//
// One CTA (4 warps) owns a 64-row block of one segment of one head and a
// 128-column tile of it; warp w owns rows 16w..16w+15 across all 128 columns,
// so a row's reduction never leaves a quad.  Operands are staged through
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
template <int OUTER, int INNER, bool ALIGNED>
struct TileStage {
    static constexpr int UPR = INNER / 8;
    static constexpr int UNITS = OUTER * UPR;
    static constexpr int PT = UNITS / NT;
    static_assert(UNITS % NT == 0, "tile must divide among the threads");
    uint4 r[PT];

    __device__ __forceinline__ void load(const uint16_t* __restrict__ g, int64_t ld, int o0, int i0, int o_lim,
                                         int i_lim, int tid) {
#pragma unroll
        for (int j = 0; j < PT; ++j) {
            const int u = tid + j * NT;
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
            const int u = tid + j * NT;
            *reinterpret_cast<uint4*>(s + (u / UPR) * pitch + (u % UPR) * 8) = r[j];
        }
    }
};

// One BK-deep step of the warp's 16 x 128 block from shared memory.
template <typename Tag, bool TA, bool TB>
__device__ __forceinline__ void mma_stage(float (&acc)[NJ][4], const uint16_t* sA, const uint16_t* sB, int warp,
                                          int lane, int ncols) {
#pragma unroll
    for (int ks = 0; ks < BK / 16; ++ks) {
        const int k0 = ks * 16;
        uint32_t a[4];
        if constexpr (!TA) {
            blk_ldmatrix_x4(a, blk_smem_u32(sA + (warp * 16 + (lane & 15)) * A_PITCH_N + k0 + (lane >> 4) * 8));
        } else {
            blk_ldmatrix_x4_trans(a, blk_smem_u32(sA + (k0 + (lane & 7) + ((lane >> 4) << 3)) * A_PITCH_T +
                                                  warp * 16 + ((lane >> 3) & 1) * 8));
        }
#pragma unroll
        for (int jp = 0; jp < NJ / 2; ++jp) {
            if (jp * 16 < ncols) {
                uint32_t b[4];
                if constexpr (!TB) {
                    blk_ldmatrix_x4(b, blk_smem_u32(sB + (jp * 16 + (lane & 7) + ((lane >> 4) << 3)) * B_PITCH_N + k0 +
                                                    ((lane >> 3) & 1) * 8));
                } else {
                    blk_ldmatrix_x4_trans(b, blk_smem_u32(sB + (k0 + (lane & 7) + ((lane >> 3) & 1) * 8) * B_PITCH_T +
                                                          jp * 16 + ((lane >> 4) << 3)));
                }
                blk_mma16816<Tag>(acc[2 * jp], a[0], a[1], a[2], a[3], b[0], b[1]);
                blk_mma16816<Tag>(acc[2 * jp + 1], a[0], a[1], a[2], a[3], b[2], b[3]);
            }
        }
    }
}

// acc = A[m0.., :] * B[n0.., :]^T for the CTA's 64 x 128 tile.
template <typename Tag, bool TA, bool TB, bool AA, bool AB>
__device__ __forceinline__ void compute_tile(float (&acc)[NJ][4], const uint16_t* __restrict__ gA,
                                             const uint16_t* __restrict__ gB, int M, int N, int K, int m0, int n0,
                                             uint16_t (*sA)[A_STAGE], uint16_t (*sB)[B_STAGE], int tid) {
#pragma unroll
    for (int j = 0; j < NJ; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    const int nk = (K + BK - 1) / BK;
    if (nk == 0) return;
    const int warp = tid >> 5, lane = tid & 31;
    const bool active = m0 + warp * 16 < M;
    const int ncols = min(N - n0, BN);

    TileStage<TA ? BK : BM, TA ? BM : BK, AA> stA;
    TileStage<TB ? BK : BN, TB ? BN : BK, AB> stB;
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
        if (active) mma_stage<Tag, TA, TB>(acc, sA[cur], sB[cur], warp, lane, ncols);
        if (more) {
            stA.store(sA[cur ^ 1], pA, tid);
            stB.store(sB[cur ^ 1], pB, tid);
        }
        __syncthreads();
    }
}

// Writes the thread's fragment (rows r0 and r0+8, columns n0 + 8j + 2t, +1).
template <typename Tag>
__device__ __forceinline__ void store_frag(void* C, int out_f32, int64_t cbase, const float (&v)[NJ][4], int r0, int M,
                                           int N, int n0, int t, bool pair_ok) {
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        const int col = n0 + 8 * j + 2 * t;
        if (col < N) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int r = r0 + 8 * h;
                if (r < M) {
                    const int64_t e = cbase + (int64_t)r * N + col;
                    const float x = v[j][2 * h], y = v[j][2 * h + 1];
                    if (out_f32) {
                        float* c = reinterpret_cast<float*>(C) + e;
                        if (pair_ok && col + 1 < N) {
                            *reinterpret_cast<float2*>(c) = make_float2(x, y);
                        } else {
                            c[0] = x;
                            if (col + 1 < N) c[1] = y;
                        }
                    } else {
                        uint16_t* c = reinterpret_cast<uint16_t*>(C) + e;
                        if (pair_ok && col + 1 < N) {
                            *reinterpret_cast<uint32_t*>(c) = BlkCvt<Tag>::pack2(x, y);
                        } else {
                            c[0] = BlkCvt<Tag>::pack1(x);
                            if (col + 1 < N) c[1] = BlkCvt<Tag>::pack1(y);
                        }
                    }
                }
            }
        }
    }
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

    if (p.epi == BLK_EPI_SCORES) {
        const int n0 = it.tn * BN;
        compute_tile<Tag, TA, TB, AA, AB>(acc, gA, gB, M, N, K, m0, n0, sA, sB, tid);
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            acc[j][0] *= p.scale; acc[j][1] *= p.scale; acc[j][2] *= p.scale; acc[j][3] *= p.scale;
        }
        store_frag<Tag>(p.C, p.out_f32, cbase, acc, r0, M, N, n0, t, pair_ok);
        return;
    }

    // softmax epilogue, base-2 domain
    const float sl = p.scale * BLK_LOG2E;
    float mrun[2] = {-INFINITY, -INFINITY}, lrun[2] = {0.f, 0.f};
    for (int tn = 0; tn < it.ntn; ++tn) {
        const int n0 = tn * BN;
        compute_tile<Tag, TA, TB, AA, AB>(acc, gA, gB, M, N, K, m0, n0, sA, sB, tid);
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
            store_frag<Tag>(p.C, p.out_f32, cbase, acc, r0, M, N, 0, t, pair_ok);
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
        compute_tile<Tag, TA, TB, AA, AB>(acc, gA, gB, M, N, K, m0, n0, sA, sB, tid);
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[j][e] = blk_exp2(acc[j][e] * sl - mrun[e >> 1]) * inv[e >> 1];
        }
        store_frag<Tag>(p.C, p.out_f32, cbase, acc, r0, M, N, n0, t, pair_ok);
    }
}

template <typename Tag, bool TA, bool TB>
__global__ void __launch_bounds__(NT, 3) blk_gemm_tile_kernel(const BlkGemmParams p) {
    __shared__ __align__(16) uint16_t sA[2][A_STAGE];
    __shared__ __align__(16) uint16_t sB[2][B_STAGE];
    const int64_t bid = blockIdx.x;
    const int head = (int)(bid / p.num_items);
    const BlkTileItem it = p.items[bid % p.num_items];
    const BlkSeg sd = p.segs[it.seg];
    const int64_t baseA = (int64_t)head * p.Dm1 + sd.offA, baseB = (int64_t)head * p.Dm2 + sd.offB;
    const int64_t cbase = (int64_t)head * p.Dout + sd.offC;
    const uint16_t* gA = p.A + baseA;
    const uint16_t* gB = p.B + baseB;
    const int64_t pitchA = TA ? sd.M : sd.K, pitchB = TB ? sd.N : sd.K;
    // per operand: plain 16-byte loads when every row of this (segment, head) starts on a 16-byte boundary
    const bool alignedA = ((baseA | pitchA) & 7) == 0, alignedB = ((baseB | pitchB) & 7) == 0;
    if (alignedA) {
        if (alignedB) tile_body<Tag, TA, TB, true, true>(p, sd, it, gA, gB, cbase, sA, sB);
        else tile_body<Tag, TA, TB, true, false>(p, sd, it, gA, gB, cbase, sA, sB);
    } else {
        if (alignedB) tile_body<Tag, TA, TB, false, true>(p, sd, it, gA, gB, cbase, sA, sB);
        else tile_body<Tag, TA, TB, false, false>(p, sd, it, gA, gB, cbase, sA, sB);
    }
}

template <typename Tag>
cudaError_t launch_tag(const BlkGemmParams& p, int ta, int tb, cudaStream_t st) {
    const int64_t blocks = (int64_t)p.num_items * p.H;
    if (blocks == 0) return cudaSuccess;
    const dim3 grid((unsigned)blocks), block(NT);
    if (!ta && !tb) blk_gemm_tile_kernel<Tag, false, false><<<grid, block, 0, st>>>(p);
    else if (!ta && tb) blk_gemm_tile_kernel<Tag, false, true><<<grid, block, 0, st>>>(p);
    else if (ta && !tb) blk_gemm_tile_kernel<Tag, true, false><<<grid, block, 0, st>>>(p);
    else blk_gemm_tile_kernel<Tag, true, true><<<grid, block, 0, st>>>(p);
    return cudaGetLastError();
}

}  // namespace

cudaError_t blk_launch_gemm_tile(const BlkGemmParams& p, int dtype_in, int ta, int tb, cudaStream_t st) {
    return dtype_in == BLK_F16 ? launch_tag<BlkHalfTag>(p, ta, tb, st) : launch_tag<BlkBf16Tag>(p, ta, tb, st);
}
