// fp32 path of the varlen blocked GEMM: a plain FFMA tile kernel (64 x 64 x 16
// CTA tile, 256 threads, 4 x 4 outputs per thread), fp32 in, fp32 accumulate,
// fp32 out, either operand transposed, any alignment.  fp32 is the second
// priority of this library (the 16-bit paths carry the throughput), so this
// kernel favours exactness and simplicity.
//
// Replaces upstream sparseBlockedGEMM<float,...> (csrc/cuda/spBlkGEMM.cu:120-271).
#include "blk_device.cuh"
#include "blk_kernels.h"

namespace {

constexpr int SBM = BLK_SIMT_BM, SBN = BLK_SIMT_BN, SBK = 16, SNT = 256, SPAD = 4;

// Loads a (64 rows of the logical operand) x (16 k) tile into s[k][row].
// The logical operand X is (R, K) row-major, or stored (K, R) when TR.
template <bool TR>
__device__ __forceinline__ void load_tile(float (*s)[SBM + SPAD], const float* __restrict__ g, int R, int K, int r0,
                                          int k0, int tid) {
#pragma unroll
    for (int i = 0; i < (SBM * SBK) / SNT; ++i) {
        int r, k;
        if (!TR) {  // k contiguous in memory
            k = tid % SBK;
            r = tid / SBK + i * (SNT / SBK);
        } else {    // r contiguous in memory
            r = tid % SBM;
            k = tid / SBM + i * (SNT / SBM);
        }
        const int gr = r0 + r, gk = k0 + k;
        float v = 0.f;
        if (gr < R && gk < K) v = TR ? __ldg(g + (int64_t)gk * R + gr) : __ldg(g + (int64_t)gr * K + gk);
        s[k][r] = v;
    }
}

template <bool TA, bool TB>
__global__ void __launch_bounds__(SNT) blk_gemm_simt_kernel(const BlkSimtParams p) {
    __shared__ __align__(16) float sA[SBK][SBM + SPAD];
    __shared__ __align__(16) float sB[SBK][SBN + SPAD];
    const int tid = threadIdx.x;
    const int64_t bid = blockIdx.x;
    const int head = (int)(bid / p.num_items);
    const BlkTileItem it = p.items[bid % p.num_items];
    const BlkSeg sd = p.segs[it.seg];
    const float* gA = p.A + (int64_t)head * p.Dm1 + sd.offA;
    const float* gB = p.B + (int64_t)head * p.Dm2 + sd.offB;
    float* gC = p.C + (int64_t)head * p.Dout + sd.offC;
    const int M = sd.M, N = sd.N, K = sd.K;
    const int m0 = it.tm * SBM, n0 = it.tn * SBN;
    const int ty = tid / 16, tx = tid % 16;

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += SBK) {
        load_tile<TA>(sA, gA, M, K, m0, k0, tid);
        load_tile<TB>(sB, gB, N, K, n0, k0, tid);
        __syncthreads();
#pragma unroll
        for (int k = 0; k < SBK; ++k) {
            const float4 a = *reinterpret_cast<const float4*>(&sA[k][ty * 4]);
            const float4 b = *reinterpret_cast<const float4*>(&sB[k][tx * 4]);
            const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = m0 + ty * 4 + i;
        if (r < M) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int c = n0 + tx * 4 + j;
                if (c < N) gC[(int64_t)r * N + c] = acc[i][j] * p.scale;
            }
        }
    }
}

}  // namespace

cudaError_t blk_launch_gemm_simt(const BlkSimtParams& p, cudaStream_t st) {
    const int64_t blocks = (int64_t)p.num_items * p.H;
    if (blocks == 0) return cudaSuccess;
    const dim3 grid((unsigned)blocks), block(SNT);
    if (!p.ta && !p.tb) blk_gemm_simt_kernel<false, false><<<grid, block, 0, st>>>(p);
    else if (!p.ta && p.tb) blk_gemm_simt_kernel<false, true><<<grid, block, 0, st>>>(p);
    else if (p.ta && !p.tb) blk_gemm_simt_kernel<true, false><<<grid, block, 0, st>>>(p);
    else blk_gemm_simt_kernel<true, true><<<grid, block, 0, st>>>(p);
    return cudaGetLastError();
}
