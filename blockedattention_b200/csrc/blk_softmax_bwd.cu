// Backward of the varlen row softmax over a packed (H, D) buffer:
//   grad_src = scale * (grad_out - sum_row(out * grad_out)) * out
// where out = softmax_rows(scale * src) is the forward result.
//
// Same decomposition as the forward kernel (blk_softmax.cu): a CTA owns a chunk
// of consecutive rows of one segment of one head whose bytes fit a 16 KB
// window, and moves it as a flat byte range -- 16-byte vectors for every
// vector wholly inside the chunk, single elements for the ragged edges -- here
// for two inputs that sit at the same element offset of their buffers, so one
// alignment computation serves both.  The row arithmetic runs in fp32 out of
// shared memory: sub-warp groups for short rows, one warp per longer row; a row
// longer than the window is streamed twice by the whole CTA.
//
// Replaces upstream sparseBlockedSoftmaxBackward_warp / _block
// (csrc/cuda/spBlkSoftmax.cu:140-180, :271-332) and their launcher (:418-459).
#include "blk_device.cuh"
#include "blk_kernels.h"

namespace {

constexpr int SB_THREADS = 256;
constexpr int SB_WARPS = SB_THREADS / 32;
constexpr int SB_WINDOW = BLK_SMX_WINDOW_BYTES;

template <typename Tag>
struct BwdIO16 {
    typedef uint16_t E;
    static __device__ __forceinline__ float ld(E v) { return BlkCvt<Tag>::unpack1(v); }
    static __device__ __forceinline__ E st(float v) { return BlkCvt<Tag>::pack1(v); }
};
struct BwdIO32 {
    typedef float E;
    static __device__ __forceinline__ float ld(E v) { return v; }
    static __device__ __forceinline__ E st(float v) { return v; }
};

__device__ __forceinline__ float sb_group_sum(float v, int G) {
    for (int o = G >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// flat copy of `span` window bytes (the chunk is bytes [mis, span) of it) from global to shared memory
template <typename E>
__device__ __forceinline__ void window_in(unsigned char* sbuf, const unsigned char* src_al, int mis, int span, int tid) {
    const int nvec = (span + 15) >> 4;
    for (int v = tid; v < nvec; v += SB_THREADS) {
        const int lo = v << 4, hi = lo + 16;
        if (lo >= mis && hi <= span) {
            *reinterpret_cast<uint4*>(sbuf + lo) = blk_ldg_stream16(src_al + lo);
        } else {
            const int b0 = lo > mis ? lo : mis, b1 = hi < span ? hi : span;
            for (int b = b0; b < b1; b += (int)sizeof(E))
                *reinterpret_cast<E*>(sbuf + b) = *reinterpret_cast<const E*>(src_al + b);
        }
    }
}

template <typename IO>
__global__ void __launch_bounds__(SB_THREADS) blk_softmax_bwd_kernel(const BlkSmxBwdParams p) {
    typedef typename IO::E E;
    constexpr int ES = (int)sizeof(E);
    __shared__ __align__(16) unsigned char sP[SB_WINDOW + 32];
    __shared__ __align__(16) unsigned char sG[SB_WINDOW + 32];
    __shared__ float red[SB_WARPS];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t bid = blockIdx.x;
    const int head = (int)(bid / p.num_chunks);
    const BlkSmxChunk ch = p.chunks[bid % p.num_chunks];
    const int64_t e0 = (int64_t)head * p.D + ch.off;
    const E* gP = reinterpret_cast<const E*>(p.out) + e0;
    const E* gG = reinterpret_cast<const E*>(p.grad_out) + e0;
    E* gD = reinterpret_cast<E*>(p.grad_src) + e0;
    const int cols = ch.cols;

    const int64_t nbytes = (int64_t)ch.rows * cols * ES;
    if (nbytes > SB_WINDOW) {  // rows == 1 by construction: two streaming passes by the whole CTA
        float dot = 0.f;
        for (int c = tid; c < cols; c += SB_THREADS) dot += IO::ld(gP[c]) * IO::ld(gG[c]);
        dot = sb_group_sum(dot, 32);
        if (lane == 0) red[warp] = dot;
        __syncthreads();
        dot = 0.f;
#pragma unroll
        for (int w = 0; w < SB_WARPS; ++w) dot += red[w];
        for (int c = tid; c < cols; c += SB_THREADS) {
            const float pv = IO::ld(gP[c]), gv = IO::ld(gG[c]);
            gD[c] = IO::st((gv - dot) * pv * p.scale);
        }
        return;
    }
    const int mis = (int)((e0 * ES) & 15);
    const int span = mis + (int)nbytes;
    window_in<E>(sP, reinterpret_cast<const unsigned char*>(gP) - mis, mis, span, tid);
    window_in<E>(sG, reinterpret_cast<const unsigned char*>(gG) - mis, mis, span, tid);
    __syncthreads();

    const E* pw = reinterpret_cast<const E*>(sP + mis);
    E* gw = reinterpret_cast<E*>(sG + mis);  // overwritten with the result
    int G = 32;
    if (cols <= 64) {
        G = 1;
        while (G * 4 < cols) G <<= 1;  // G in {1,2,4,8,16}
    }
    const int rpw = 32 / G, gl = lane & (G - 1), gi = lane / G;
    for (int rb = warp * rpw; rb < ch.rows; rb += SB_WARPS * rpw) {
        const int r = rb + gi;
        const bool valid = r < ch.rows;
        const E* prow = pw + (size_t)(valid ? r : 0) * cols;
        E* grow = gw + (size_t)(valid ? r : 0) * cols;
        float dot = 0.f;
        if (valid)
            for (int c = gl; c < cols; c += G) dot += IO::ld(prow[c]) * IO::ld(grow[c]);
        dot = sb_group_sum(dot, G);
        if (valid)
            for (int c = gl; c < cols; c += G) grow[c] = IO::st((IO::ld(grow[c]) - dot) * IO::ld(prow[c]) * p.scale);
    }
    __syncthreads();

    unsigned char* dst_al = reinterpret_cast<unsigned char*>(gD) - mis;
    const int nvec = (span + 15) >> 4;
    for (int v = tid; v < nvec; v += SB_THREADS) {
        const int lo = v << 4, hi = lo + 16;
        if (lo >= mis && hi <= span) {
            *reinterpret_cast<uint4*>(dst_al + lo) = *reinterpret_cast<const uint4*>(sG + lo);
        } else {
            const int b0 = lo > mis ? lo : mis, b1 = hi < span ? hi : span;
            for (int b = b0; b < b1; b += ES) *reinterpret_cast<E*>(dst_al + b) = *reinterpret_cast<const E*>(sG + b);
        }
    }
}

}  // namespace

cudaError_t blk_launch_softmax_bwd(const BlkSmxBwdParams& p, int dtype, cudaStream_t st) {
    const int64_t blocks = (int64_t)p.num_chunks * p.H;
    if (blocks == 0) return cudaSuccess;
    const dim3 grid((unsigned)blocks), block(SB_THREADS);
    if (dtype == BLK_F16) blk_softmax_bwd_kernel<BwdIO16<BlkHalfTag>><<<grid, block, 0, st>>>(p);
    else if (dtype == BLK_BF16) blk_softmax_bwd_kernel<BwdIO16<BlkBf16Tag>><<<grid, block, 0, st>>>(p);
    else blk_softmax_bwd_kernel<BwdIO32><<<grid, block, 0, st>>>(p);
    return cudaGetLastError();
}
