// Packed small-segment kernel: one warp computes the whole score block of one
// (segment, head) with N <= 64 columns and K in {32, 64}; persistent warps walk
// a cost-sorted item list, several blocks in flight per CTA, no shared memory.
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
// the 16-row blocks of the first operand (the next block's loads are issued
// before the current block's epilogue); scale, row softmax (quad shuffles
// only) and the store follow in registers.  Segments are binned by column
// count (N <= 16, 32, 64) into separately compiled variants so that a short
// segment does not pay the registers and the epilogue of a long one.
//
// Replaces, for small segments, upstream sparseBlockedHGEMM_half/_bf16 with a
// 32 x 32 tile (csrc/cuda/spBlkGEMM.cu:842-846, :424-817) followed by
// sparseBlockedSoftmax_warp (csrc/cuda/spBlkSoftmax.cu:88-138).
#include "blk_device.cuh"
#include "blk_kernels.h"

namespace {

constexpr int SW = BLK_SMALL_WARPS;

template <typename Tag, bool OUT32>
struct OutT;
template <typename Tag>
struct OutT<Tag, true> {
    typedef float E;
    static __device__ __forceinline__ void pair(E* p, float x, float y) { *reinterpret_cast<float2*>(p) = make_float2(x, y); }
    static __device__ __forceinline__ void one(E* p, float x) { *p = x; }
};
template <typename Tag>
struct OutT<Tag, false> {
    typedef uint16_t E;
    static __device__ __forceinline__ void pair(E* p, float x, float y) {
        *reinterpret_cast<uint32_t*>(p) = BlkCvt<Tag>::pack2(x, y);
    }
    static __device__ __forceinline__ void one(E* p, float x) { *p = BlkCvt<Tag>::pack1(x); }
};

template <int NT8>
struct MinBlocks {
    static constexpr int value = NT8 <= 2 ? 6 : (NT8 <= 4 ? 5 : 3);
};

template <typename Tag, int KC, int NT8, bool SOFTMAX, bool OUT32>
__global__ void __launch_bounds__(SW * 32, MinBlocks<NT8>::value) blk_scores_small_kernel(const BlkSmallParams p) {
    constexpr int K = KC * 32;
    typedef OutT<Tag, OUT32> Out;
    typedef typename Out::E E;
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int64_t total = (int64_t)p.num_items * p.H;
    const int64_t stride = (int64_t)gridDim.x * SW;
    const float sl = SOFTMAX ? p.scale * BLK_LOG2E : p.scale;

    for (int64_t w = (int64_t)blockIdx.x * SW + (threadIdx.x >> 5); w < total; w += stride) {
        const int head = (int)(w % p.H);
        const BlkSmallItem it = p.items[w / p.H];
        const int M = it.M, N = it.N;
        const uint16_t* gA = p.A + (int64_t)head * p.Dm1 + it.offA + 8 * t;
        const uint16_t* gB = p.B + (int64_t)head * p.Dm2 + it.offB + 8 * t;
        const int64_t cbase = (int64_t)head * p.Dout + it.offC;
        const bool pair_ok = ((cbase & 1) == 0) && ((N & 1) == 0);
        const int ntiles = (N + 7) >> 3, nrem = N - 2 * t;

        // second operand: row 8j+g of the segment, all of K, resident for the whole block
        uint4 b[NT8][KC];
#pragma unroll
        for (int j = 0; j < NT8; ++j) {
            const int n = 8 * j + g;
#pragma unroll
            for (int c = 0; c < KC; ++c) {
                b[j][c] = make_uint4(0u, 0u, 0u, 0u);
                if (n < N) b[j][c] = blk_ldg_stream16(gB + n * K + 32 * c);
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

            if (SOFTMAX) {
                float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
                for (int j = 0; j < NT8; ++j) {
                    if (j < ntiles) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) acc[j][e] *= sl;
                        const bool in0 = 8 * j < nrem, in1 = 8 * j + 1 < nrem;  // columns 8j+2t, +1 inside N
                        acc[j][0] = in0 ? acc[j][0] : -INFINITY;
                        acc[j][2] = in0 ? acc[j][2] : -INFINITY;
                        acc[j][1] = in1 ? acc[j][1] : -INFINITY;
                        acc[j][3] = in1 ? acc[j][3] : -INFINITY;
                        mx0 = fmaxf(mx0, fmaxf(acc[j][0], acc[j][1]));
                        mx1 = fmaxf(mx1, fmaxf(acc[j][2], acc[j][3]));
                    }
                }
                mx0 = blk_quad_max(mx0);
                mx1 = blk_quad_max(mx1);
                float s0 = 0.f, s1 = 0.f;
#pragma unroll
                for (int j = 0; j < NT8; ++j) {
                    if (j < ntiles) {
                        acc[j][0] = blk_exp2(acc[j][0] - mx0);
                        acc[j][1] = blk_exp2(acc[j][1] - mx0);
                        acc[j][2] = blk_exp2(acc[j][2] - mx1);
                        acc[j][3] = blk_exp2(acc[j][3] - mx1);
                        s0 += acc[j][0] + acc[j][1];
                        s1 += acc[j][2] + acc[j][3];
                    }
                }
                const float i0 = 1.f / blk_quad_sum(s0), i1 = 1.f / blk_quad_sum(s1);
#pragma unroll
                for (int j = 0; j < NT8; ++j) {
                    if (j < ntiles) {
                        acc[j][0] *= i0; acc[j][1] *= i0; acc[j][2] *= i1; acc[j][3] *= i1;
                    }
                }
            } else {
#pragma unroll
                for (int j = 0; j < NT8; ++j) {
                    acc[j][0] *= sl; acc[j][1] *= sl; acc[j][2] *= sl; acc[j][3] *= sl;
                }
            }

            // store: rows r0 = 16 mb + g and r0 + 8, columns 8j + 2t, +1
            const int r0 = mb * 16 + g;
            E* c0 = reinterpret_cast<E*>(p.C) + cbase + (int64_t)r0 * N + 2 * t;
            E* c1 = c0 + 8 * N;
            const bool v0 = r0 < M, v1 = r0 + 8 < M;
            if (pair_ok) {
#pragma unroll
                for (int j = 0; j < NT8; ++j) {
                    if (8 * j + 2 * t < N) {  // N even: the pair is wholly inside or wholly outside
                        if (v0) Out::pair(c0 + 8 * j, acc[j][0], acc[j][1]);
                        if (v1) Out::pair(c1 + 8 * j, acc[j][2], acc[j][3]);
                    }
                }
            } else {
#pragma unroll
                for (int j = 0; j < NT8; ++j) {
                    const int col = 8 * j + 2 * t;
                    if (col < N) {
                        if (v0) Out::one(c0 + 8 * j, acc[j][0]);
                        if (v1) Out::one(c1 + 8 * j, acc[j][2]);
                        if (col + 1 < N) {
                            if (v0) Out::one(c0 + 8 * j + 1, acc[j][1]);
                            if (v1) Out::one(c1 + 8 * j + 1, acc[j][3]);
                        }
                    }
                }
            }
        }
    }
}

template <typename Tag, int KC, int NT8>
cudaError_t launch_variant(const BlkSmallParams& p, int sms, cudaStream_t st) {
    const int64_t warps = (int64_t)p.num_items * p.H;
    if (warps == 0) return cudaSuccess;
    const int64_t want = (warps + SW - 1) / SW;
    const int64_t cap = (int64_t)sms * MinBlocks<NT8>::value;
    const dim3 grid((unsigned)(want < cap ? want : cap)), block(SW * 32);
    const bool sm = p.epi == BLK_EPI_SOFTMAX, o32 = p.out_f32 != 0;
    if (sm && !o32) blk_scores_small_kernel<Tag, KC, NT8, true, false><<<grid, block, 0, st>>>(p);
    else if (sm && o32) blk_scores_small_kernel<Tag, KC, NT8, true, true><<<grid, block, 0, st>>>(p);
    else if (!sm && !o32) blk_scores_small_kernel<Tag, KC, NT8, false, false><<<grid, block, 0, st>>>(p);
    else blk_scores_small_kernel<Tag, KC, NT8, false, true><<<grid, block, 0, st>>>(p);
    return cudaGetLastError();
}

template <typename Tag>
cudaError_t launch_tag(const BlkSmallParams& p, int K, int bucket, int sms, cudaStream_t st) {
    if (K == 32) {
        if (bucket == 0) return launch_variant<Tag, 1, 2>(p, sms, st);
        if (bucket == 1) return launch_variant<Tag, 1, 4>(p, sms, st);
        return launch_variant<Tag, 1, 8>(p, sms, st);
    }
    if (K == 64) {
        if (bucket == 0) return launch_variant<Tag, 2, 2>(p, sms, st);
        if (bucket == 1) return launch_variant<Tag, 2, 4>(p, sms, st);
        return launch_variant<Tag, 2, 8>(p, sms, st);
    }
    return cudaErrorInvalidValue;
}

}  // namespace

cudaError_t blk_launch_scores_small(const BlkSmallParams& p, int dtype_in, int K, int bucket, int sms,
                                    cudaStream_t st) {
    return dtype_in == BLK_F16 ? launch_tag<BlkHalfTag>(p, K, bucket, sms, st)
                               : launch_tag<BlkBf16Tag>(p, K, bucket, sms, st);
}
