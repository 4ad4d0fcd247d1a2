// Varlen row softmax over a packed (H, D) buffer: out = softmax_rows(scale * src).
//
// A CTA owns a chunk of consecutive rows of one segment of one head whose
// bytes fit a 12 KB shared-memory window.  Rows of a packed segment start at
// arbitrary element offsets, so the CTA moves the chunk as a flat byte range:
// 16-byte vectors for every vector that lies wholly inside the chunk, single
// elements for the (at most two) ragged edge vectors.  Global traffic is thus
// vectorised and coalesced whatever the row length, each element is read once
// and written once, and the row arithmetic (fp32, base-2 exponent, one
// rounding) runs out of shared memory: several short rows per warp through
// sub-warp groups, one warp per longer row, values held in registers between
// the max, sum and normalise steps when a row has at most 512 columns.  A row
// longer than the window is handled by one CTA in three streaming passes, so
// there is no limit on the column count.
//
// Replaces upstream sparseBlockedSoftmax_warp / _block
// (csrc/cuda/spBlkSoftmax.cu:88-138, :182-269) and the per-row host table
// (csrc/cuda/spBlkSoftmax.cu:358-373).
#include <string>

#include "blk_device.cuh"
#include "blk_kernels.h"

namespace {

constexpr int SMX_THREADS = 256;
constexpr int SMX_WARPS = SMX_THREADS / 32;
constexpr int WINDOW = BLK_SMX_WINDOW_BYTES;

template <typename Tag>
struct SmxIO16 {
    typedef uint16_t E;
    static __device__ __forceinline__ float ld(E v) { return BlkCvt<Tag>::unpack1(v); }
    static __device__ __forceinline__ E st(float v) { return BlkCvt<Tag>::pack1(v); }
};
struct SmxIO32 {
    typedef float E;
    static __device__ __forceinline__ float ld(E v) { return v; }
    static __device__ __forceinline__ E st(float v) { return v; }
};

__device__ __forceinline__ float group_max(float v, int G) {
    for (int o = G >> 1; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float group_sum(float v, int G) {
    for (int o = G >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Rows of at most EPL*G columns, G lanes per row, values kept in registers.
template <typename IO, int EPL>
__device__ __forceinline__ void rows_in_regs(typename IO::E* srow, int rows, int cols, int G, float sl, int warp,
                                             int lane) {
    const int rpw = 32 / G;  // rows a warp handles at once
    const int gl = lane & (G - 1), gi = lane / G;
    for (int rb = warp * rpw; rb < rows; rb += SMX_WARPS * rpw) {
        const int r = rb + gi;
        const bool valid = r < rows;
        typename IO::E* row = srow + (size_t)r * cols;
        float v[EPL];
        float mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            const int c = gl + i * G;
            v[i] = (valid && c < cols) ? IO::ld(row[c]) * sl : -INFINITY;
            mx = fmaxf(mx, v[i]);
        }
        mx = group_max(mx, G);
        if (!valid) mx = 0.f;
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            v[i] = blk_exp2(v[i] - mx);
            sum += v[i];
        }
        sum = group_sum(sum, G);
        const float inv = 1.f / sum;
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            const int c = gl + i * G;
            if (valid && c < cols) row[c] = IO::st(v[i] * inv);
        }
    }
}

// One warp per row, any column count that fits the window; exponent evaluated twice.
template <typename IO>
__device__ __forceinline__ void rows_streamed(typename IO::E* srow, int rows, int cols, float sl, int warp, int lane) {
    for (int r = warp; r < rows; r += SMX_WARPS) {
        typename IO::E* row = srow + (size_t)r * cols;
        float mx = -INFINITY;
        for (int c = lane; c < cols; c += 32) mx = fmaxf(mx, IO::ld(row[c]) * sl);
        mx = group_max(mx, 32);
        float sum = 0.f;
        for (int c = lane; c < cols; c += 32) sum += blk_exp2(IO::ld(row[c]) * sl - mx);
        sum = group_sum(sum, 32);
        const float inv = 1.f / sum;
        for (int c = lane; c < cols; c += 32) row[c] = IO::st(blk_exp2(IO::ld(row[c]) * sl - mx) * inv);
    }
}

__device__ __forceinline__ float cta_reduce(float v, bool is_max, float* red, int warp, int lane) {
    v = is_max ? group_max(v, 32) : group_sum(v, 32);
    __syncthreads();  // red may still be read from the previous reduction
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = red[0];
#pragma unroll
    for (int w = 1; w < SMX_WARPS; ++w) r = is_max ? fmaxf(r, red[w]) : r + red[w];
    return r;
}

// A single row longer than the window: three streaming passes by the whole CTA.
template <typename IO>
__device__ __forceinline__ void long_row(const typename IO::E* src, typename IO::E* dst, int cols,
                                         float sl, float* red, int tid) {
    const int warp = tid >> 5, lane = tid & 31;
    float mx = -INFINITY;
    for (int c = tid; c < cols; c += SMX_THREADS) mx = fmaxf(mx, IO::ld(src[c]) * sl);
    mx = cta_reduce(mx, true, red, warp, lane);
    float sum = 0.f;
    for (int c = tid; c < cols; c += SMX_THREADS) sum += blk_exp2(IO::ld(src[c]) * sl - mx);
    sum = cta_reduce(sum, false, red, warp, lane);
    const float inv = 1.f / sum;
    for (int c = tid; c < cols; c += SMX_THREADS) dst[c] = IO::st(blk_exp2(IO::ld(src[c]) * sl - mx) * inv);
}

template <typename IO>
__global__ void __launch_bounds__(SMX_THREADS) blk_softmax_kernel(const BlkSmxParams p) {
    typedef typename IO::E E;
    constexpr int ES = (int)sizeof(E);
    __shared__ __align__(16) unsigned char sbuf[WINDOW + 32];
    __shared__ float red[SMX_WARPS];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t bid = blockIdx.x;
    const int head = (int)(bid / p.num_chunks);
    const BlkSmxChunk ch = p.chunks[bid % p.num_chunks];
    const int64_t e0 = (int64_t)head * p.D + ch.off;
    const float sl = p.scale * BLK_LOG2E;
    const E* gsrc = reinterpret_cast<const E*>(p.src) + e0;
    E* gdst = reinterpret_cast<E*>(p.dst) + e0;

    const int64_t nbytes = (int64_t)ch.rows * ch.cols * ES;
    if (nbytes > WINDOW) {  // rows == 1 by construction
        long_row<IO>(gsrc, gdst, ch.cols, sl, red, tid);
        return;
    }
    // flat, aligned window: byte b of the window mirrors byte (a0 + b) of the strip
    const int mis = (int)((e0 * ES) & 15);
    const int span = mis + (int)nbytes;
    const int nvec = (span + 15) >> 4;
    const unsigned char* src_al = reinterpret_cast<const unsigned char*>(gsrc) - mis;
    unsigned char* dst_al = reinterpret_cast<unsigned char*>(gdst) - mis;
    for (int v = tid; v < nvec; v += SMX_THREADS) {
        const int lo = v << 4, hi = lo + 16;
        if (lo >= mis && hi <= span) {
            *reinterpret_cast<uint4*>(sbuf + lo) = blk_ldg_stream16(src_al + lo);
        } else {
            const int b0 = lo > mis ? lo : mis, b1 = hi < span ? hi : span;
            for (int b = b0; b < b1; b += ES)
                *reinterpret_cast<E*>(sbuf + b) = *reinterpret_cast<const E*>(src_al + b);
        }
    }
    __syncthreads();

    E* srow = reinterpret_cast<E*>(sbuf + mis);
    const int cols = ch.cols;
    if (cols <= 128) {
        int G = 1;
        while (G * 4 < cols) G <<= 1;  // G in {1,2,4,8,16,32}
        rows_in_regs<IO, 4>(srow, ch.rows, cols, G, sl, warp, lane);
    } else if (cols <= 512) {
        rows_in_regs<IO, 16>(srow, ch.rows, cols, 32, sl, warp, lane);
    } else {
        rows_streamed<IO>(srow, ch.rows, cols, sl, warp, lane);
    }
    __syncthreads();

    for (int v = tid; v < nvec; v += SMX_THREADS) {
        const int lo = v << 4, hi = lo + 16;
        if (lo >= mis && hi <= span) {
            *reinterpret_cast<uint4*>(dst_al + lo) = *reinterpret_cast<const uint4*>(sbuf + lo);
        } else {
            const int b0 = lo > mis ? lo : mis, b1 = hi < span ? hi : span;
            for (int b = b0; b < b1; b += ES) *reinterpret_cast<E*>(dst_al + b) = *reinterpret_cast<const E*>(sbuf + b);
        }
    }
}

}  // namespace

cudaError_t blk_launch_softmax(const BlkSmxParams& p, int dtype, cudaStream_t st) {
    const int64_t blocks = (int64_t)p.num_chunks * p.H;
    if (blocks == 0) return cudaSuccess;
    const dim3 grid((unsigned)blocks), block(SMX_THREADS);
    if (dtype == BLK_F16) blk_softmax_kernel<SmxIO16<BlkHalfTag>><<<grid, block, 0, st>>>(p);
    else if (dtype == BLK_BF16) blk_softmax_kernel<SmxIO16<BlkBf16Tag>><<<grid, block, 0, st>>>(p);
    else blk_softmax_kernel<SmxIO32><<<grid, block, 0, st>>>(p);
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// Softmax without a plan and without any device allocation.
//
// Some hosts of this library may not allocate device memory at the point where
// they need the operator: a runtime that has handed all device memory to its
// own arena, a plugin called inside someone else's memory pool, a caller that
// must not disturb other streams (cudaMalloc and cudaFree synchronise the
// whole device).  For them the chunk table that blk_softmax_plan_create would
// upload into a cudaMalloc'ed buffer lives instead in the fixed array below,
// which every GPU that loads the library carries (1 MB) until the process
// exits.  The table is copied from ordinary host memory, which the runtime
// stages before the call returns; that copy may make the call wait for earlier
// work on the same stream, and it is why the call refuses a capturing stream
// (a captured copy would read the host table again at every replay, after it
// has been freed).
// ---------------------------------------------------------------------------
static __device__ __align__(256) BlkSmxChunk g_noalloc_chunks[BLK_NOALLOC_MAX_CHUNKS];

namespace {
constexpr int NOALLOC_MAX_DEVICES = 64;
// Device address of g_noalloc_chunks per device; the symbol's name is only a host-side handle.
BlkSmxChunk* g_noalloc_dev_ptr[NOALLOC_MAX_DEVICES] = {};
}  // namespace

extern "C" int blk_softmax_noalloc(const void* src, void* out, const int64_t* rows, const int64_t* cols, int64_t S,
                                   int64_t H, int dtype, float scale, void* cuda_stream) {
    if (S < 0 || H < 0 || (S > 0 && (!rows || !cols))) {
        blk_set_error("blk_softmax_noalloc: negative count or null list");
        return BLK_ERR_INVALID;
    }
    if (dtype < BLK_F16 || dtype > BLK_F32) {
        blk_set_error("blk_softmax_noalloc: unsupported dtype");
        return BLK_ERR_UNSUPPORTED;
    }
    // host-side schedule only (device = -1: nothing is uploaded or allocated on the GPU)
    blk_plan plan;
    plan.kind = 1;
    plan.S = S;
    plan.H = H;
    plan.dtype_in = plan.dtype_out = dtype;
    plan.device = -1;
    plan.max_chunks = BLK_NOALLOC_MAX_CHUNKS;  // refused by count, before any chunk is made
    plan.M.assign(rows, rows + S);
    plan.N.assign(cols, cols + S);
    plan.a1.resize(S + 1);
    int rc = blk_softmax_offsets(rows, cols, S, plan.a1.data());
    if (rc == BLK_OK) rc = blk_build_softmax_schedule(&plan);
    if (rc != BLK_OK) return rc;
    const size_t nchunks = plan.smx_chunks.size();
    if (nchunks == 0 || H == 0) return BLK_OK;
    if (nchunks > (size_t)BLK_NOALLOC_MAX_CHUNKS) {  // the scheduler has already refused by count; kept as a guard
        blk_set_error("blk_softmax_noalloc: the built-in table holds " + std::to_string(BLK_NOALLOC_MAX_CHUNKS) + " chunks");
        return BLK_ERR_UNSUPPORTED;
    }
    if ((int64_t)nchunks * H > 0x7fffffffLL) {
        blk_set_error("blk_softmax_noalloc: chunks x heads exceeds 2^31-1 CTAs");
        return BLK_ERR_UNSUPPORTED;
    }
    if (!src || !out) {
        blk_set_error("blk_softmax_noalloc: null buffer");
        return BLK_ERR_INVALID;
    }
    if ((reinterpret_cast<uintptr_t>(src) & 15u) || (reinterpret_cast<uintptr_t>(out) & 15u)) {
        blk_set_error("blk_softmax_noalloc: device pointers must be 16-byte aligned");
        return BLK_ERR_UNALIGNED;
    }
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEVICES) {
        blk_set_error("blk_softmax_noalloc: cannot identify the current device");
        return BLK_ERR_CUDA;
    }
    if (!g_noalloc_dev_ptr[dev]) {
        // one-time set-up on this device (it is the current one): resolve the array's device address
        BlkSmxChunk* ptr = nullptr;
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_chunks);
        if (e != cudaSuccess || !ptr) {
            blk_set_error(std::string("blk_softmax_noalloc: cudaGetSymbolAddress failed: ") + cudaGetErrorString(e));
            return BLK_ERR_CUDA;
        }
        g_noalloc_dev_ptr[dev] = ptr;
    }
    BlkSmxChunk* table = g_noalloc_dev_ptr[dev];
    cudaStream_t st = reinterpret_cast<cudaStream_t>(cuda_stream);
    {
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        e = cudaStreamIsCapturing(st, &cap);
        if (e != cudaSuccess) {
            blk_set_error(std::string("blk_softmax_noalloc: cannot query the stream: ") + cudaGetErrorString(e));
            return BLK_ERR_CUDA;
        }
        if (cap != cudaStreamCaptureStatusNone) {
            blk_set_error("blk_softmax_noalloc: the stream is being captured; this entry point uploads its table from "
                          "temporary host memory and cannot be recorded -- capture blk_softmax_run on a plan instead");
            return BLK_ERR_UNSUPPORTED;
        }
    }
    // every call rewrites the entries it uses; nothing in the table has to start at zero
    e = cudaMemcpyAsync(table, plan.smx_chunks.data(), nchunks * sizeof(BlkSmxChunk), cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) {
        blk_set_error(std::string("blk_softmax_noalloc: table upload failed: ") + cudaGetErrorString(e));
        return BLK_ERR_CUDA;
    }
    BlkSmxParams xp{};
    xp.src = src;
    xp.dst = out;
    xp.chunks = table;
    xp.D = plan.Dm1;
    xp.num_chunks = (int)nchunks;
    xp.H = (int)H;
    xp.scale = scale;
    e = blk_launch_softmax(xp, dtype, st);
    if (e != cudaSuccess) {
        blk_set_error(std::string("blk_softmax_noalloc: launch failed: ") + cudaGetErrorString(e));
        return BLK_ERR_CUDA;
    }
    return BLK_OK;
}
