// Packed small-segment kernel: one warp computes the whole score block of one
// (segment, head) with M, N <= 64 and K in {32, 64}; persistent warps walk a
// cost-sorted item list, four blocks in flight per CTA.
//
// Loads.  The contraction index may be permuted freely as long as both
// operands use the same permutation, so each lane reads its mma.sync
// fragments straight from global memory as 16-byte vectors: lane (g, t) of a
// quad takes elements k = 32c + 8t .. 8t+7 of row g, which are exactly the
// fragment registers of two consecutive m16n8k16 steps under the permutation
// "slot (2t, 2t+1, 2t+8, 2t+9) of step h <- element 8t + 4h + (0, 1, 2, 3)".
// A quad reads 64 contiguous bytes of a row and a warp-wide load covers eight
// rows: every load is 128-bit and uses whole 32-byte sectors.  The segment's
// second operand (N x K) stays in registers while the warp walks the 16-row
// blocks of the first operand, whose next block is requested before the
// current block's epilogue.
//
// Epilogue.  Scale, row softmax (quad shuffles only, fp32, base-2 exponent) and
// rounding happen in registers.  The code is specialised on the exact number
// of 8-column tiles (a switch per block, 1..4 tiles in one kernel and 5..8 in
// another, so that short segments keep a small register footprint): only the
// last tile carries column masks and nothing is computed for tiles a segment
// does not have.
//
// Stores.  Rows of a packed block start at arbitrary element offsets, so the
// warp first lays the block out in its private shared-memory strip exactly as
// it lies in global memory (same offset modulo 16 bytes) and then copies it
// out as 16-byte vectors, with single elements only at the two ragged ends.
//
// Replaces, for small segments, upstream sparseBlockedHGEMM_half/_bf16 with a
// 32 x 32 tile (csrc/cuda/spBlkGEMM.cu:842-846, :424-817) followed by
// sparseBlockedSoftmax_warp (csrc/cuda/spBlkSoftmax.cu:88-138).
#include "blk_device.cuh"
#include "blk_kernels.h"

namespace {

constexpr int SW = BLK_SMALL_WARPS;
constexpr int MAXM = BLK_SMALL_MAXM;  // rows of a block handled here (a multiple of 16)

template <int NTMAX>
struct MinBlocks {
    static constexpr int value = NTMAX <= 4 ? 5 : 3;  // measured: more resident CTAs (with spills) ran slower
};

// One (segment, head) block with exactly NT column tiles.
template <typename Tag, int KC, int NT, bool SOFTMAX, bool OUT32>
__device__ __forceinline__ void small_block(const BlkSmallParams& p, const BlkSmallItem& it, uint32_t head,
                                            unsigned char* strip, float sl, bool flip, int lane) {
    constexpr int K = KC * 32;
    constexpr int ES = OUT32 ? 4 : 2;
    const int g = lane >> 2, t = lane & 3;
    const int M = it.M, N = it.N;
    const uint16_t* gA = p.A + ((int64_t)head * p.Dm1 + it.offA + 8 * t);
    const uint16_t* gB = p.B + ((int64_t)head * p.Dm2 + it.offB + 8 * t);
    const int64_t cbase = (int64_t)head * p.Dout + it.offC;
    const bool pair_ok = ((cbase & 1) == 0) && ((N & 1) == 0);
    const int mis = (int)((cbase * ES) & 15);  // the strip mirrors global memory modulo 16 bytes

    // Second operand: row 8j+g, all of K, resident for the whole block.  Rows past the end are
    // clamped to the last row instead of predicated; their columns are masked in the last tile.
    uint4 b[NT][KC];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const uint16_t* pb = gB + min(8 * j + g, N - 1) * K;
#pragma unroll
        for (int c = 0; c < KC; ++c) b[j][c] = blk_ldg_stream16(pb + 32 * c);
    }
    uint4 a[2][KC];
    auto load_a = [&](int mb) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint16_t* pa = gA + min(mb * 16 + g + 8 * h, M - 1) * K;
#pragma unroll
            for (int c = 0; c < KC; ++c) a[h][c] = blk_ldg_stream16(pa + 32 * c);
        }
    };
    load_a(0);
    // columns 8(NT-1) + 2t, +1 of the last tile
    const bool last0 = 8 * (NT - 1) + 2 * t < N, last1 = 8 * (NT - 1) + 2 * t + 1 < N;
    const uint32_t srow = blk_smem_u32(strip) + mis + (g * N + 2 * t) * ES;
    const int nmb = (M + 15) >> 4;
    for (int mb = 0; mb < nmb; ++mb) {
        // the four registers of each A fragment, contiguous: {row g lo, row g+8 lo, row g hi, row g+8 hi}
        uint32_t af[2 * KC][4];
#pragma unroll
        for (int c = 0; c < KC; ++c) {
            af[2 * c][0] = a[0][c].x; af[2 * c][1] = a[1][c].x; af[2 * c][2] = a[0][c].y; af[2 * c][3] = a[1][c].y;
            af[2 * c + 1][0] = a[0][c].z; af[2 * c + 1][1] = a[1][c].z;
            af[2 * c + 1][2] = a[0][c].w; af[2 * c + 1][3] = a[1][c].w;
        }
        if (SOFTMAX && flip) {  // negative scale: work with |scale| and -A
#pragma unroll
            for (int c = 0; c < 2 * KC; ++c)
#pragma unroll
                for (int e = 0; e < 4; ++e) af[c][e] ^= 0x80008000u;
        }
        if (mb + 1 < nmb) load_a(mb + 1);  // in flight during the products and the epilogue
        float acc[NT][4];
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
#pragma unroll
            for (int c = 0; c < KC; ++c) {
                blk_mma16816<Tag>(acc[j], af[2 * c][0], af[2 * c][1], af[2 * c][2], af[2 * c][3], b[j][c].x, b[j][c].y);
                blk_mma16816<Tag>(acc[j], af[2 * c + 1][0], af[2 * c + 1][1], af[2 * c + 1][2], af[2 * c + 1][3],
                                  b[j][c].z, b[j][c].w);
            }
        }
        if (SOFTMAX) {
            acc[NT - 1][0] = last0 ? acc[NT - 1][0] : -INFINITY;
            acc[NT - 1][2] = last0 ? acc[NT - 1][2] : -INFINITY;
            acc[NT - 1][1] = last1 ? acc[NT - 1][1] : -INFINITY;
            acc[NT - 1][3] = last1 ? acc[NT - 1][3] : -INFINITY;
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                mx0 = fmaxf(mx0, fmaxf(acc[j][0], acc[j][1]));
                mx1 = fmaxf(mx1, fmaxf(acc[j][2], acc[j][3]));
            }
            const float nm0 = -blk_quad_max(mx0) * sl, nm1 = -blk_quad_max(mx1) * sl;
            float s0 = 0.f, s1 = 0.f;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                acc[j][0] = blk_exp2(fmaf(acc[j][0], sl, nm0));
                acc[j][1] = blk_exp2(fmaf(acc[j][1], sl, nm0));
                acc[j][2] = blk_exp2(fmaf(acc[j][2], sl, nm1));
                acc[j][3] = blk_exp2(fmaf(acc[j][3], sl, nm1));
                s0 += acc[j][0] + acc[j][1];
                s1 += acc[j][2] + acc[j][3];
            }
            const float i0 = __frcp_rn(blk_quad_sum(s0)), i1 = __frcp_rn(blk_quad_sum(s1));
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                acc[j][0] *= i0; acc[j][1] *= i0; acc[j][2] *= i1; acc[j][3] *= i1;
            }
        } else {
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                acc[j][0] *= sl; acc[j][1] *= sl; acc[j][2] *= sl; acc[j][3] *= sl;
            }
        }
        // into the strip: rows 16 mb + g and + 8 (rows >= M land in the strip's padding), columns 8j + 2t, +1
        const uint32_t s0a = srow + (uint32_t)(mb * 16 * N * ES), s1a = s0a + 8 * N * ES;
        if (pair_ok) {  // N even: a pair of columns is wholly inside or wholly outside
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                if (j < NT - 1 || last0) {
                    if (OUT32) {
                        blk_sts_f32x2(s0a + 8 * j * ES, acc[j][0], acc[j][1]);
                        blk_sts_f32x2(s1a + 8 * j * ES, acc[j][2], acc[j][3]);
                    } else {
                        blk_sts_b32(s0a + 8 * j * ES, BlkCvt<Tag>::pack2(acc[j][0], acc[j][1]));
                        blk_sts_b32(s1a + 8 * j * ES, BlkCvt<Tag>::pack2(acc[j][2], acc[j][3]));
                    }
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const bool in0 = j < NT - 1 || last0, in1 = j < NT - 1 || last1;
                if (OUT32) {
                    if (in0) { blk_sts_f32(s0a + 8 * j * ES, acc[j][0]); blk_sts_f32(s1a + 8 * j * ES, acc[j][2]); }
                    if (in1) { blk_sts_f32(s0a + 8 * j * ES + ES, acc[j][1]); blk_sts_f32(s1a + 8 * j * ES + ES, acc[j][3]); }
                } else {
                    const uint32_t lo = BlkCvt<Tag>::pack2(acc[j][0], acc[j][1]);
                    const uint32_t hi = BlkCvt<Tag>::pack2(acc[j][2], acc[j][3]);
                    if (in0) { blk_sts_b16(s0a + 8 * j * ES, lo); blk_sts_b16(s1a + 8 * j * ES, hi); }
                    if (in1) { blk_sts_b16(s0a + 8 * j * ES + ES, lo >> 16); blk_sts_b16(s1a + 8 * j * ES + ES, hi >> 16); }
                }
            }
        }
    }
    __syncwarp();
    // strip -> global: the block is M*N contiguous elements
    {
        const int lo = mis, hi = mis + M * N * ES;
        const int vlo = (lo + 15) & ~15, vhi = hi & ~15;
        unsigned char* gdst = reinterpret_cast<unsigned char*>(p.C) + (cbase * ES - mis);  // 16-byte aligned
        for (int o = vlo + 16 * lane; o < vhi; o += 16 * 32)
            *reinterpret_cast<uint4*>(gdst + o) = *reinterpret_cast<const uint4*>(strip + o);
        const int head_end = vlo < hi ? vlo : hi;              // [lo, head_end): elements before the first full vector
        const int tail_beg = vhi > head_end ? vhi : head_end;  // [tail_beg, hi): elements after the last one
        const int oh = lo + lane * ES, ot = tail_beg + lane * ES;
        if (OUT32) {
            if (oh < head_end) *reinterpret_cast<float*>(gdst + oh) = *reinterpret_cast<const float*>(strip + oh);
            if (ot < hi) *reinterpret_cast<float*>(gdst + ot) = *reinterpret_cast<const float*>(strip + ot);
        } else {
            if (oh < head_end) *reinterpret_cast<uint16_t*>(gdst + oh) = *reinterpret_cast<const uint16_t*>(strip + oh);
            if (ot < hi) *reinterpret_cast<uint16_t*>(gdst + ot) = *reinterpret_cast<const uint16_t*>(strip + ot);
        }
    }
    __syncwarp();  // the strip is rewritten by the warp's next block
}

template <typename Tag, int KC, int NTMAX, bool SOFTMAX, bool OUT32>
__global__ void __launch_bounds__(SW * 32, MinBlocks<NTMAX>::value) blk_scores_small_kernel(const BlkSmallParams p) {
    constexpr int ES = OUT32 ? 4 : 2;
    constexpr int STRIP = MAXM * NTMAX * 8 * ES + 32;
    extern __shared__ __align__(16) unsigned char strips[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t total = (uint32_t)p.num_items * (uint32_t)p.H;  // < 2^31, checked at plan creation
    const uint32_t stride = gridDim.x * SW, H = (uint32_t)p.H;
    const bool flip = p.scale < 0.f;
    const float sl = SOFTMAX ? fabsf(p.scale) * BLK_LOG2E : p.scale;
    unsigned char* strip = strips + warp * STRIP;

    for (uint32_t w = blockIdx.x * SW + warp; w < total; w += stride) {
        const uint32_t item = w / H, head = w - item * H;
        const BlkSmallItem it = p.items[item];
        switch ((it.N + 7) >> 3) {
            case NTMAX - 3: small_block<Tag, KC, NTMAX - 3, SOFTMAX, OUT32>(p, it, head, strip, sl, flip, lane); break;
            case NTMAX - 2: small_block<Tag, KC, NTMAX - 2, SOFTMAX, OUT32>(p, it, head, strip, sl, flip, lane); break;
            case NTMAX - 1: small_block<Tag, KC, NTMAX - 1, SOFTMAX, OUT32>(p, it, head, strip, sl, flip, lane); break;
            default: small_block<Tag, KC, NTMAX, SOFTMAX, OUT32>(p, it, head, strip, sl, flip, lane); break;
        }
    }
}

template <typename Tag, int KC, int NTMAX>
cudaError_t launch_variant(const BlkSmallParams& p, int sms, cudaStream_t st) {
    const int64_t warps = (int64_t)p.num_items * p.H;
    if (warps == 0) return cudaSuccess;
    const int64_t want = (warps + SW - 1) / SW;
    const int64_t cap = (int64_t)sms * MinBlocks<NTMAX>::value;
    const dim3 grid((unsigned)(want < cap ? want : cap)), block(SW * 32);
    const bool sm = p.epi == BLK_EPI_SOFTMAX, o32 = p.out_f32 != 0;
    const size_t smem = (size_t)SW * (MAXM * NTMAX * 8 * (o32 ? 4 : 2) + 32);
    auto go = [&](auto kern) -> cudaError_t {
        if (smem > 48 * 1024) {
            cudaError_t e = blk_func_smem(reinterpret_cast<const void*>(kern), (int)smem);
            if (e != cudaSuccess) return e;
        }
        kern<<<grid, block, smem, st>>>(p);
        return cudaGetLastError();
    };
    if (sm && !o32) return go(blk_scores_small_kernel<Tag, KC, NTMAX, true, false>);
    if (sm && o32) return go(blk_scores_small_kernel<Tag, KC, NTMAX, true, true>);
    if (!sm && !o32) return go(blk_scores_small_kernel<Tag, KC, NTMAX, false, false>);
    return go(blk_scores_small_kernel<Tag, KC, NTMAX, false, true>);
}

template <typename Tag>
cudaError_t launch_tag(const BlkSmallParams& p, int K, int bucket, int sms, cudaStream_t st) {
    if (K == 32) return bucket == 0 ? launch_variant<Tag, 1, 4>(p, sms, st) : launch_variant<Tag, 1, 8>(p, sms, st);
    if (K == 64) return bucket == 0 ? launch_variant<Tag, 2, 4>(p, sms, st) : launch_variant<Tag, 2, 8>(p, sms, st);
    return cudaErrorInvalidValue;
}

}  // namespace

cudaError_t blk_launch_scores_small(const BlkSmallParams& p, int dtype_in, int K, int bucket, int sms,
                                    cudaStream_t st) {
    return dtype_in == BLK_F16 ? launch_tag<BlkHalfTag>(p, K, bucket, sms, st)
                               : launch_tag<BlkBf16Tag>(p, K, bucket, sms, st);
}
