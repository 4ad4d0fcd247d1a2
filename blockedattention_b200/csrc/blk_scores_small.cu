// Packed small-segment kernel: one warp computes the whole score block of one
// (segment, head) with N <= 64 columns and K in {32, 64}, four such blocks per
// CTA, with no shared memory at all.
//
// The contraction index may be permuted freely as long as both operands use
// the same permutation, so each lane reads its mma.sync fragments straight
// from global memory as 16-byte vectors: lane (g, t) of a quad takes elements
// k = 32c + 8t .. 8t+7 of row g, which are exactly the A (or B) fragment
// registers of two consecutive m16n8k16 steps under the permutation
// "slot (2t, 2t+1, 2t+8, 2t+9) of step h <- element 8t + 4h + (0, 1, 2, 3)".
// A quad therefore reads 64 contiguous bytes of a row and a warp-wide load
// covers eight rows: every load is 128-bit and uses whole 32-byte sectors.
// The segment's second operand (N x K) stays in registers while the warp walks
// the 16-row blocks of the first operand; scale, row softmax (quad shuffles
// only) and the store follow in registers.
//
// Replaces, for small segments, upstream sparseBlockedHGEMM_half/_bf16 with a
// 32 x 32 tile (csrc/cuda/spBlkGEMM.cu:842-846, :424-817) followed by
// sparseBlockedSoftmax_warp (csrc/cuda/spBlkSoftmax.cu:88-138).
#include "blk_device.cuh"
#include "blk_kernels.h"

namespace {

constexpr int SW = BLK_SMALL_WARPS;
constexpr int NT8 = BLK_SMALL_MAXN / 8;  // n8 tiles per row block

template <typename Tag, int KC>
__global__ void __launch_bounds__(SW * 32) blk_scores_small_kernel(const BlkSmallParams p) {
    constexpr int K = KC * 32;
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int64_t w = (int64_t)blockIdx.x * SW + (threadIdx.x >> 5);
    if (w >= (int64_t)p.num_items * p.H) return;
    const int head = (int)(w / p.num_items);
    const BlkSmallItem it = p.items[w % p.num_items];
    const int M = it.M, N = it.N;
    const uint16_t* gA = p.A + (int64_t)head * p.Dm1 + it.offA + 8 * t;
    const uint16_t* gB = p.B + (int64_t)head * p.Dm2 + it.offB + 8 * t;
    const int64_t cbase = (int64_t)head * p.Dout + it.offC;
    const bool pair_ok = ((cbase & 1) == 0) && ((N & 1) == 0);
    const int ntiles = (N + 7) >> 3;

    // second operand: row 8j+g of the segment, all of K, resident for the whole block
    uint4 b[NT8][KC];
#pragma unroll
    for (int j = 0; j < NT8; ++j) {
        const int n = 8 * j + g;
#pragma unroll
        for (int c = 0; c < KC; ++c) {
            b[j][c] = make_uint4(0u, 0u, 0u, 0u);
            if (n < N) b[j][c] = blk_ldg_stream16(gB + (int64_t)n * K + 32 * c);
        }
    }
    uint4 a[2][KC];
    auto load_a = [&](int mb) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = mb * 16 + g + 8 * h;
#pragma unroll
            for (int c = 0; c < KC; ++c) {
                a[h][c] = make_uint4(0u, 0u, 0u, 0u);
                if (r < M) a[h][c] = blk_ldg_stream16(gA + (int64_t)r * K + 32 * c);
            }
        }
    };
    load_a(0);
    const float sl = p.scale * BLK_LOG2E;
    const int nmb = (M + 15) >> 4;
    for (int mb = 0; mb < nmb; ++mb) {
        float acc[NT8][4];
#pragma unroll
        for (int j = 0; j < NT8; ++j) {
            acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
            if (j < ntiles) {
#pragma unroll
                for (int c = 0; c < KC; ++c) {
                    blk_mma16816<Tag>(acc[j], a[0][c].x, a[1][c].x, a[0][c].y, a[1][c].y, b[j][c].x, b[j][c].y);
                    blk_mma16816<Tag>(acc[j], a[0][c].z, a[1][c].z, a[0][c].w, a[1][c].w, b[j][c].z, b[j][c].w);
                }
            }
        }
        if (mb + 1 < nmb) load_a(mb + 1);  // in flight during the epilogue

        if (p.epi == BLK_EPI_SOFTMAX) {
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < NT8; ++j) {
                const int col = 8 * j + 2 * t;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float s = (col + (e & 1) < N) ? acc[j][e] * sl : -INFINITY;
                    acc[j][e] = s;
                    mx[e >> 1] = fmaxf(mx[e >> 1], s);
                }
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const float m = blk_quad_max(mx[h]);
                float sum = 0.f;
#pragma unroll
                for (int j = 0; j < NT8; ++j) {
                    acc[j][2 * h] = blk_exp2(acc[j][2 * h] - m);
                    acc[j][2 * h + 1] = blk_exp2(acc[j][2 * h + 1] - m);
                    sum += acc[j][2 * h] + acc[j][2 * h + 1];
                }
                const float inv = 1.f / blk_quad_sum(sum);
#pragma unroll
                for (int j = 0; j < NT8; ++j) {
                    acc[j][2 * h] *= inv;
                    acc[j][2 * h + 1] *= inv;
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < NT8; ++j) {
                acc[j][0] *= p.scale; acc[j][1] *= p.scale; acc[j][2] *= p.scale; acc[j][3] *= p.scale;
            }
        }
#pragma unroll
        for (int j = 0; j < NT8; ++j) {
            const int col = 8 * j + 2 * t;
            if (col < N) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int r = mb * 16 + g + 8 * h;
                    if (r < M) {
                        const int64_t e = cbase + (int64_t)r * N + col;
                        const float x = acc[j][2 * h], y = acc[j][2 * h + 1];
                        if (p.out_f32) {
                            float* c = reinterpret_cast<float*>(p.C) + e;
                            if (pair_ok && col + 1 < N) {
                                *reinterpret_cast<float2*>(c) = make_float2(x, y);
                            } else {
                                c[0] = x;
                                if (col + 1 < N) c[1] = y;
                            }
                        } else {
                            uint16_t* c = reinterpret_cast<uint16_t*>(p.C) + e;
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
}

template <typename Tag>
cudaError_t launch_tag(const BlkSmallParams& p, int K, cudaStream_t st) {
    const int64_t warps = (int64_t)p.num_items * p.H;
    if (warps == 0) return cudaSuccess;
    const dim3 grid((unsigned)((warps + SW - 1) / SW)), block(SW * 32);
    if (K == 32) blk_scores_small_kernel<Tag, 1><<<grid, block, 0, st>>>(p);
    else if (K == 64) blk_scores_small_kernel<Tag, 2><<<grid, block, 0, st>>>(p);
    else return cudaErrorInvalidValue;
    return cudaGetLastError();
}

}  // namespace

cudaError_t blk_launch_scores_small(const BlkSmallParams& p, int dtype_in, int K, cudaStream_t st) {
    return dtype_in == BLK_F16 ? launch_tag<BlkHalfTag>(p, K, st) : launch_tag<BlkBf16Tag>(p, K, st);
}
