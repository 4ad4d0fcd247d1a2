// Pipelined varlen row softmax, forward and backward, over a packed (H, D) buffer.
//
// The host groups consecutive row pieces (blk_softmax.cu's chunks) whose bytes are contiguous in memory into
// windows of at most 12 KB -- many small segments, or a few rows of a wide one.  A persistent CTA walks windows
// w = blockIdx.x, + gridDim.x, ... of the (window, head) list with two shared-memory stages:
//   * one thread fetches the next window with a bulk asynchronous copy (cp.async.bulk, completion on the
//     stage's mbarrier) of the 16-byte aligned range that covers it -- no thread waits for a load it issued;
//   * all threads do the row arithmetic of the current window out of shared memory (fp32, base-2 exponent,
//     one rounding): one lane per short row (one warp per small segment); one warp per longer row, which reads and writes the row as
//     16-byte vectors between its first and last 16-byte boundary (the few elements outside go one per lane)
//     and keeps up to 1024 columns in registers between the maximum, the sum and the normalisation;
//   * one thread writes the window back with a bulk asynchronous store of the aligned vectors that lie wholly
//     inside it, a few lanes store the ragged edge elements, and the CTA moves on without waiting for either.
// Loads, arithmetic and stores of neighbouring windows overlap inside one CTA, so the kernel streams at memory
// speed with few resident CTAs.  A row longer than a window is streamed from global memory by the whole CTA.
// Every barrier wait is bounded and reports through the status word.
//
// Forward: out = softmax_rows(scale * src); replaces upstream sparseBlockedSoftmax_warp / _block
// (csrc/cuda/spBlkSoftmax.cu:88-138, :182-269).  Backward: grad_src = scale * (grad_out - rowsum(out *
// grad_out)) * out; replaces sparseBlockedSoftmaxBackward_warp / _block (:140-180, :271-332).
#include "blk_device.cuh"
#include "blk_kernels.h"

namespace {

constexpr int SP_THREADS = 128;
constexpr int SP_WARPS = SP_THREADS / 32;
constexpr int SP_WIN = BLK_SMX_WINDOW_BYTES;
constexpr int SP_BUF = SP_WIN + 32;  // a window plus the slack of its 16-byte aligned cover
constexpr uint32_t SP_SPIN_LIMIT = 1u << 22;

// Element types: E, scalar conversion, and the 16-byte vector of VE elements.
template <typename Tag>
struct SpIO16;
template <>
struct SpIO16<BlkHalfTag> {
    typedef uint16_t E;
    static constexpr int VE = 8;
    static __device__ __forceinline__ float ld(E v) { return BlkCvt<BlkHalfTag>::unpack1(v); }
    static __device__ __forceinline__ E st(float v) { return BlkCvt<BlkHalfTag>::pack1(v); }
    static __device__ __forceinline__ void unpack(const uint4& q, float (&f)[8]) {
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            f[2 * i] = t.x;
            f[2 * i + 1] = t.y;
        }
    }
    static __device__ __forceinline__ uint4 pack(const float (&f)[8]) {
        return make_uint4(BlkCvt<BlkHalfTag>::pack2(f[0], f[1]), BlkCvt<BlkHalfTag>::pack2(f[2], f[3]),
                          BlkCvt<BlkHalfTag>::pack2(f[4], f[5]), BlkCvt<BlkHalfTag>::pack2(f[6], f[7]));
    }
    // running extreme (maximum, or minimum for a negative scale) of a row, taken on the packed pairs as they lie in
    // memory: one instruction per two elements and no conversion
    typedef uint32_t X;
    template <bool NEG> static __device__ __forceinline__ X xinit() { return NEG ? 0x7c007c00u : 0xfc00fc00u; }
    template <bool NEG> static __device__ __forceinline__ X xacc(X a, const uint4& q) {
        X r;
        if (NEG) asm("{\n .reg .b32 t, u;\n min.f16x2 t, %1, %2;\n min.f16x2 u, %3, %4;\n min.f16x2 t, t, u;\n min.f16x2 %0, t, %5;\n}\n" : "=r"(r) : "r"(q.x), "r"(q.y), "r"(q.z), "r"(q.w), "r"(a));
        else asm("{\n .reg .b32 t, u;\n max.f16x2 t, %1, %2;\n max.f16x2 u, %3, %4;\n max.f16x2 t, t, u;\n max.f16x2 %0, t, %5;\n}\n" : "=r"(r) : "r"(q.x), "r"(q.y), "r"(q.z), "r"(q.w), "r"(a));
        return r;
    }
    template <bool NEG> static __device__ __forceinline__ float xfin(X a) {
        const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&a));
        return NEG ? fminf(t.x, t.y) : fmaxf(t.x, t.y);
    }
};
template <>
struct SpIO16<BlkBf16Tag> {
    typedef uint16_t E;
    static constexpr int VE = 8;
    static __device__ __forceinline__ float ld(E v) { return BlkCvt<BlkBf16Tag>::unpack1(v); }
    static __device__ __forceinline__ E st(float v) { return BlkCvt<BlkBf16Tag>::pack1(v); }
    static __device__ __forceinline__ void unpack(const uint4& q, float (&f)[8]) {
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    static __device__ __forceinline__ uint4 pack(const float (&f)[8]) {
        return make_uint4(BlkCvt<BlkBf16Tag>::pack2(f[0], f[1]), BlkCvt<BlkBf16Tag>::pack2(f[2], f[3]),
                          BlkCvt<BlkBf16Tag>::pack2(f[4], f[5]), BlkCvt<BlkBf16Tag>::pack2(f[6], f[7]));
    }
    typedef uint32_t X;
    template <bool NEG> static __device__ __forceinline__ X xinit() { return NEG ? 0x7f807f80u : 0xff80ff80u; }
    template <bool NEG> static __device__ __forceinline__ X xacc(X a, const uint4& q) {
        X r;
        if (NEG) asm("{\n .reg .b32 t, u;\n min.bf16x2 t, %1, %2;\n min.bf16x2 u, %3, %4;\n min.bf16x2 t, t, u;\n min.bf16x2 %0, t, %5;\n}\n" : "=r"(r) : "r"(q.x), "r"(q.y), "r"(q.z), "r"(q.w), "r"(a));
        else asm("{\n .reg .b32 t, u;\n max.bf16x2 t, %1, %2;\n max.bf16x2 u, %3, %4;\n max.bf16x2 t, t, u;\n max.bf16x2 %0, t, %5;\n}\n" : "=r"(r) : "r"(q.x), "r"(q.y), "r"(q.z), "r"(q.w), "r"(a));
        return r;
    }
    template <bool NEG> static __device__ __forceinline__ float xfin(X a) {
        const float lo = __uint_as_float(a << 16), hi = __uint_as_float(a & 0xffff0000u);
        return NEG ? fminf(lo, hi) : fmaxf(lo, hi);
    }
};
struct SpIO32 {
    typedef float E;
    static constexpr int VE = 4;
    static __device__ __forceinline__ float ld(E v) { return v; }
    static __device__ __forceinline__ E st(float v) { return v; }
    static __device__ __forceinline__ void unpack(const uint4& q, float (&f)[4]) {
        f[0] = __uint_as_float(q.x); f[1] = __uint_as_float(q.y); f[2] = __uint_as_float(q.z); f[3] = __uint_as_float(q.w);
    }
    static __device__ __forceinline__ uint4 pack(const float (&f)[4]) {
        return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
    }
    typedef float X;
    template <bool NEG> static __device__ __forceinline__ X xinit() { return NEG ? INFINITY : -INFINITY; }
    template <bool NEG> static __device__ __forceinline__ X xacc(X a, const uint4& q) {
        const float x = __uint_as_float(q.x), y = __uint_as_float(q.y), z = __uint_as_float(q.z), w = __uint_as_float(q.w);
        return NEG ? fminf(fminf(a, x), fminf(fminf(y, z), w)) : fmaxf(fmaxf(a, x), fmaxf(fmaxf(y, z), w));
    }
    template <bool NEG> static __device__ __forceinline__ float xfin(X a) { return a; }
};

__device__ __forceinline__ float sp_max(float v, int G) {
    for (int o = G >> 1; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float sp_sum(float v, int G) {
    for (int o = G >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ void sp_bar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void sp_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool sp_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred q;\n mbarrier.try_wait.parity.shared::cta.b64 q, [%1], %2;\n selp.u32 %0, 1, 0, q;\n}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool sp_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < SP_SPIN_LIMIT; ++i)
        if (sp_try(bar, parity)) return true;
    return false;
}
// contiguous bulk copies (16-byte aligned addresses and size)
__device__ __forceinline__ void sp_bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void sp_bulk_s2g(void* dst, uint32_t src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;\n" ::"l"(dst), "r"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void sp_bulk_commit() { asm volatile("cp.async.bulk.commit_group;\n" ::: "memory"); }
// all earlier bulk stores of this thread have finished reading shared memory
__device__ __forceinline__ void sp_bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory"); }
// ... and have completed
__device__ __forceinline__ void sp_bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory"); }

// ---- row arithmetic on a piece that sits in shared memory ---------------------------------------------------

// A row of at least 8 vectors' worth of columns, one warp per row: the row starts at an arbitrary element of
// shared memory, so it is split into the elements before the first 16-byte boundary (at most VE - 1, one per
// lane 0..7), whole 16-byte vectors (lane l takes vectors l, l + 32, ...) and the elements after the last
// whole vector (one per lane 8..15).
template <typename IO>
struct RowSplit {
    typename IO::E* row;
    uint4* body;
    int nv;  // whole vectors
    int xi;  // this lane's extra element, or -1
    __device__ __forceinline__ RowSplit(typename IO::E* r, int cols, int lane) : row(r) {
        constexpr int ES = (int)sizeof(typename IO::E);
        const int h = (int)((16u - (blk_smem_u32(r) & 15u)) & 15u) / ES;
        nv = (cols - h) / IO::VE;
        const int tail = cols - h - nv * IO::VE;
        body = reinterpret_cast<uint4*>(r + h);
        xi = -1;
        if (lane < 8) {
            if (lane < h) xi = lane;
        } else if (lane < 16) {
            if (lane - 8 < tail) xi = h + nv * IO::VE + lane - 8;
        }
    }
};

// forward, at most 32 EPV whole vectors per row, values kept in registers (one exponential per element)
template <typename IO, int EPV, int NW>
__device__ __forceinline__ void fwd_rows_vec(typename IO::E* piece, int rows, int cols, float sl, int warp, int lane) {
    constexpr int VE = IO::VE;
    for (int r = warp; r < rows; r += NW) {
        RowSplit<IO> rs(piece + (size_t)r * cols, cols, lane);
        float x = rs.xi >= 0 ? IO::ld(rs.row[rs.xi]) * sl : -INFINITY;
        float v[EPV][VE];
        float mx = x;
#pragma unroll
        for (int i = 0; i < EPV; ++i) {
            const int vi = lane + 32 * i;
            if (vi < rs.nv) {
                IO::unpack(rs.body[vi], v[i]);
#pragma unroll
                for (int e = 0; e < VE; ++e) {
                    v[i][e] *= sl;
                    mx = fmaxf(mx, v[i][e]);
                }
            } else {
#pragma unroll
                for (int e = 0; e < VE; ++e) v[i][e] = -INFINITY;
            }
        }
        mx = sp_max(mx, 32);
        x = blk_exp2(x - mx);
        float sum = x;
#pragma unroll
        for (int i = 0; i < EPV; ++i)
#pragma unroll
            for (int e = 0; e < VE; ++e) {
                v[i][e] = blk_exp2(v[i][e] - mx);
                sum += v[i][e];
            }
        sum = sp_sum(sum, 32);
        const float inv = 1.f / sum;
#pragma unroll
        for (int i = 0; i < EPV; ++i) {
            const int vi = lane + 32 * i;
            if (vi < rs.nv) {
#pragma unroll
                for (int e = 0; e < VE; ++e) v[i][e] *= inv;
                rs.body[vi] = IO::pack(v[i]);
            }
        }
        if (rs.xi >= 0) rs.row[rs.xi] = IO::st(x * inv);
    }
}
// forward, any column count that fits the window: three passes over the row, exponential evaluated twice.  The first
// pass takes the extreme of the raw packed elements; the third folds the normalisation into the exponent.
template <typename IO, int NW, bool NEG>
__device__ __forceinline__ void fwd_rows_vec_streamed_impl(typename IO::E* piece, int rows, int cols, float sl, int warp,
                                                           int lane) {
    constexpr int VE = IO::VE;
    for (int r = warp; r < rows; r += NW) {
        RowSplit<IO> rs(piece + (size_t)r * cols, cols, lane);
        const float x = rs.xi >= 0 ? IO::ld(rs.row[rs.xi]) * sl : -INFINITY;
        float f[VE];
        typename IO::X ex = IO::template xinit<NEG>();
        for (int vi = lane; vi < rs.nv; vi += 32) ex = IO::template xacc<NEG>(ex, rs.body[vi]);
        const float mx = sp_max(fmaxf(x, IO::template xfin<NEG>(ex) * sl), 32);
        float sum = blk_exp2(x - mx);
        for (int vi = lane; vi < rs.nv; vi += 32) {
            IO::unpack(rs.body[vi], f);
#pragma unroll
            for (int e = 0; e < VE; ++e) sum += blk_exp2(fmaf(f[e], sl, -mx));
        }
        sum = sp_sum(sum, 32);
        const float off = -mx - __log2f(sum);  // exp2(x * sl + off) = exp2(x * sl - max) / sum
        for (int vi = lane; vi < rs.nv; vi += 32) {
            IO::unpack(rs.body[vi], f);
#pragma unroll
            for (int e = 0; e < VE; ++e) f[e] = blk_exp2(fmaf(f[e], sl, off));
            rs.body[vi] = IO::pack(f);
        }
        if (rs.xi >= 0) rs.row[rs.xi] = IO::st(blk_exp2(x + off));
    }
}
template <typename IO, int NW>
__device__ __forceinline__ void fwd_rows_vec_streamed(typename IO::E* piece, int rows, int cols, float sl, int warp,
                                                      int lane) {
    if (sl < 0.f) fwd_rows_vec_streamed_impl<IO, NW, true>(piece, rows, cols, sl, warp, lane);
    else fwd_rows_vec_streamed_impl<IO, NW, false>(piece, rows, cols, sl, warp, lane);
}
// backward over whole vectors, two passes (dot product, then the result over the gradient)
template <typename IO, int NW>
__device__ __forceinline__ void bwd_rows_vec(const typename IO::E* ppiece, typename IO::E* gpiece, int rows, int cols,
                                             float scale, int warp, int lane) {
    constexpr int VE = IO::VE;
    for (int r = warp; r < rows; r += NW) {
        RowSplit<IO> rs(gpiece + (size_t)r * cols, cols, lane);  // both rows sit at the same offset of their buffers
        const typename IO::E* prow = ppiece + (size_t)r * cols;
        const uint4* pbody = reinterpret_cast<const uint4*>(prow + (reinterpret_cast<typename IO::E*>(rs.body) - rs.row));
        float px = 0.f, gx = 0.f;
        if (rs.xi >= 0) {
            px = IO::ld(prow[rs.xi]);
            gx = IO::ld(rs.row[rs.xi]);
        }
        float pf[VE], gf[VE];
        float dot = px * gx;
        for (int vi = lane; vi < rs.nv; vi += 32) {
            IO::unpack(pbody[vi], pf);
            IO::unpack(rs.body[vi], gf);
#pragma unroll
            for (int e = 0; e < VE; ++e) dot = fmaf(pf[e], gf[e], dot);
        }
        dot = sp_sum(dot, 32);
        for (int vi = lane; vi < rs.nv; vi += 32) {
            IO::unpack(pbody[vi], pf);
            IO::unpack(rs.body[vi], gf);
#pragma unroll
            for (int e = 0; e < VE; ++e) gf[e] = (gf[e] - dot) * pf[e] * scale;
            rs.body[vi] = IO::pack(gf);
        }
        if (rs.xi >= 0) rs.row[rs.xi] = IO::st((gx - dot) * px * scale);
    }
}

// Short rows (fewer columns than eight vectors): one lane per row, one warp per piece, so a window of many
// small segments keeps every warp busy and no shuffle is needed.  Up to 32 columns stay in registers.
template <typename IO>
__device__ __forceinline__ void fwd_rows_lane(typename IO::E* piece, int rows, int cols, float sl, int lane) {
    for (int r = lane; r < rows; r += 32) {
        typename IO::E* row = piece + (size_t)r * cols;
        if (cols <= 32) {
            float v[32];
            float mx = -INFINITY;
#pragma unroll
            for (int c = 0; c < 32; ++c) {
                v[c] = c < cols ? IO::ld(row[c]) * sl : -INFINITY;
                mx = fmaxf(mx, v[c]);
            }
            float sum = 0.f;
#pragma unroll
            for (int c = 0; c < 32; ++c) {
                v[c] = blk_exp2(v[c] - mx);
                sum += v[c];
            }
            const float inv = 1.f / sum;
#pragma unroll
            for (int c = 0; c < 32; ++c)
                if (c < cols) row[c] = IO::st(v[c] * inv);
        } else {
            float mx = -INFINITY;
            for (int c = 0; c < cols; ++c) mx = fmaxf(mx, IO::ld(row[c]) * sl);
            float sum = 0.f;
            for (int c = 0; c < cols; ++c) sum += blk_exp2(fmaf(IO::ld(row[c]), sl, -mx));
            const float inv = 1.f / sum;
            for (int c = 0; c < cols; ++c) row[c] = IO::st(blk_exp2(fmaf(IO::ld(row[c]), sl, -mx)) * inv);
        }
    }
}
template <typename IO>
__device__ __forceinline__ void bwd_rows_lane(const typename IO::E* ppiece, typename IO::E* gpiece, int rows, int cols,
                                              float scale, int lane) {
    for (int r = lane; r < rows; r += 32) {
        const typename IO::E* prow = ppiece + (size_t)r * cols;
        typename IO::E* grow = gpiece + (size_t)r * cols;
        float dot = 0.f;
        for (int c = 0; c < cols; ++c) dot = fmaf(IO::ld(prow[c]), IO::ld(grow[c]), dot);
        for (int c = 0; c < cols; ++c) grow[c] = IO::st((IO::ld(grow[c]) - dot) * IO::ld(prow[c]) * scale);
    }
}

// One piece.  Pieces of short rows are dealt out to the warps one piece each (piece index pi); the warps share
// the rows of a piece of longer rows.
template <typename IO>
__device__ __forceinline__ void fwd_piece(typename IO::E* srow, int rows, int cols, float sl, int pi, int warp, int lane) {
    constexpr int VE = IO::VE;
    if (cols < 8 * VE) {
        if (pi % SP_WARPS == warp) fwd_rows_lane<IO>(srow, rows, cols, sl, lane);
        return;
    }
    const int nvmax = cols / VE;  // whole vectors of a row never exceed this
    if (nvmax <= 32) fwd_rows_vec<IO, 1, SP_WARPS>(srow, rows, cols, sl, warp, lane);
    else if (nvmax <= 64) fwd_rows_vec<IO, 2, SP_WARPS>(srow, rows, cols, sl, warp, lane);
    else if (nvmax <= 128) fwd_rows_vec<IO, 4, SP_WARPS>(srow, rows, cols, sl, warp, lane);
    else fwd_rows_vec_streamed<IO, SP_WARPS>(srow, rows, cols, sl, warp, lane);
}
// backward: the result overwrites the gradient piece
template <typename IO>
__device__ __forceinline__ void bwd_piece(const typename IO::E* prow0, typename IO::E* grow0, int rows, int cols, float scale,
                                          int pi, int warp, int lane) {
    if (cols >= 8 * IO::VE) {
        bwd_rows_vec<IO, SP_WARPS>(prow0, grow0, rows, cols, scale, warp, lane);
        return;
    }
    if (pi % SP_WARPS == warp) bwd_rows_lane<IO>(prow0, grow0, rows, cols, scale, lane);
}

__device__ __forceinline__ float sp_cta_reduce(float v, bool is_max, float* red, int warp, int lane) {
    v = is_max ? sp_max(v, 32) : sp_sum(v, 32);
    __syncthreads();  // red may still be read from the previous reduction
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = red[0];
#pragma unroll
    for (int w = 1; w < SP_WARPS; ++w) r = is_max ? fmaxf(r, red[w]) : r + red[w];
    return r;
}

// BWD = false: in0 = src, result = softmax; BWD = true: in0 = forward result, in1 = its gradient.
template <typename IO, bool BWD>
__global__ void __launch_bounds__(SP_THREADS, BWD ? 4 : 8) blk_softmax_pipe_kernel(const BlkSmxPipeParams p) {
    typedef typename IO::E E;
    constexpr int ES = (int)sizeof(E);
    constexpr int NIN = BWD ? 2 : 1;
    extern __shared__ __align__(128) unsigned char sp_smem[];  // [2 stages][NIN][SP_BUF]
    __shared__ __align__(8) uint64_t bars[2];
    __shared__ float red[SP_WARPS];
    __shared__ __align__(16) BlkSmxChunk recs[2][BLK_SMX_WINDOW_PIECES];  // the windows' piece records, per stage

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t bar0 = blk_smem_u32(bars);
    auto buf = [&](int st, int in) { return sp_smem + (st * NIN + in) * SP_BUF; };
    if (tid == 0) {
        sp_bar_init(bar0, 1);
        sp_bar_init(bar0 + 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();

    const int64_t total = (int64_t)p.num_windows * p.H, G = gridDim.x;
    const E* g0 = reinterpret_cast<const E*>(p.in0);
    const E* g1 = reinterpret_cast<const E*>(p.in1);
    E* gd = reinterpret_cast<E*>(p.out);
    const float sl = BWD ? p.scale : p.scale * BLK_LOG2E;

    // thread 0: start the copies of window w into stage st (nothing for a row longer than a window)
    auto issue = [&](int64_t w, int st) {
        const BlkSmxWindow win = p.windows[w % p.num_windows];
        if (win.nbytes > SP_WIN) return;
        const int64_t a = ((w / p.num_windows) * p.D + win.off) * ES;  // byte offset of the window in each buffer
        const int mis = (int)(a & 15);
        const uint32_t bytes = (uint32_t)((mis + win.nbytes + 15) & ~15);
        const uint32_t bar = bar0 + 8u * st;
        const uint32_t rbytes = (uint32_t)win.npieces * (uint32_t)sizeof(BlkSmxChunk);
        sp_expect_tx(bar, NIN * bytes + rbytes);
        sp_bulk_g2s(blk_smem_u32(recs[st]), p.pieces + win.first_piece, rbytes, bar);
        sp_bulk_g2s(blk_smem_u32(buf(st, 0)), reinterpret_cast<const unsigned char*>(g0) + (a - mis), bytes, bar);
        if (BWD) sp_bulk_g2s(blk_smem_u32(buf(st, 1)), reinterpret_cast<const unsigned char*>(g1) + (a - mis), bytes, bar);
    };

    uint32_t phase0 = 0u, phase1 = 0u;  // parity of the next completion of each stage's barrier
    int64_t w = blockIdx.x;
    if (tid == 0 && w < total) issue(w, 0);
    for (int k = 0; w < total; w += G, ++k) {
        const int st = k & 1;
        // the other stage is free once the bulk store that read it (previous window) is done with shared memory
        if (tid == 0) sp_bulk_wait_read();
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // this thread's reads of that stage come first
        __syncthreads();
        if (tid == 0 && w + G < total) issue(w + G, st ^ 1);

        const BlkSmxWindow win = p.windows[w % p.num_windows];
        const int64_t e0 = (w / p.num_windows) * p.D + win.off;
        if (win.nbytes > SP_WIN) {
            // one row longer than a window: streamed from global memory by the whole CTA
            const int cols = p.pieces[win.first_piece].cols;
            if (!BWD) {
                float mx = -INFINITY;
                for (int c = tid; c < cols; c += SP_THREADS) mx = fmaxf(mx, IO::ld(g0[e0 + c]) * sl);
                mx = sp_cta_reduce(mx, true, red, warp, lane);
                float sum = 0.f;
                for (int c = tid; c < cols; c += SP_THREADS) sum += blk_exp2(IO::ld(g0[e0 + c]) * sl - mx);
                sum = sp_cta_reduce(sum, false, red, warp, lane);
                const float inv = 1.f / sum;
                for (int c = tid; c < cols; c += SP_THREADS) gd[e0 + c] = IO::st(blk_exp2(IO::ld(g0[e0 + c]) * sl - mx) * inv);
            } else {
                float dot = 0.f;
                for (int c = tid; c < cols; c += SP_THREADS) dot += IO::ld(g0[e0 + c]) * IO::ld(g1[e0 + c]);
                dot = sp_cta_reduce(dot, false, red, warp, lane);
                for (int c = tid; c < cols; c += SP_THREADS)
                    gd[e0 + c] = IO::st((IO::ld(g1[e0 + c]) - dot) * IO::ld(g0[e0 + c]) * sl);
            }
            continue;
        }
        const int mis = (int)((e0 * ES) & 15);
        bool arrived = true;
        if (lane == 0) arrived = sp_wait(bar0 + 8u * st, st ? phase1 : phase0);  // one lane per warp polls
        arrived = __shfl_sync(0xffffffffu, arrived, 0);
        if (st) phase1 ^= 1u;
        else phase0 ^= 1u;
        unsigned char* res = buf(st, BWD ? 1 : 0);  // the buffer that ends up holding the result
        if (arrived) {
            E* r0 = reinterpret_cast<E*>(res + mis);
            const E* p0 = reinterpret_cast<const E*>(buf(st, 0) + mis);
            int eo = 0;
            for (int pi = 0; pi < win.npieces; ++pi) {
                const BlkSmxChunk pc = recs[st][pi];
                if (!BWD) fwd_piece<IO>(r0 + eo, pc.rows, pc.cols, sl, pi, warp, lane);
                else bwd_piece<IO>(p0 + eo, r0 + eo, pc.rows, pc.cols, sl, pi, warp, lane);
                eo += pc.rows * pc.cols;
            }
        }
        // results (generic-proxy writes) must be visible to the bulk store (async proxy)
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        if (__syncthreads_or(!arrived)) {
            if (tid == 0) atomicCAS(p.status, 0, 21);
            break;
        }
        // aligned vectors wholly inside the window: one bulk store; ragged edges: single elements
        const int span = mis + win.nbytes;
        const int lo = mis ? 16 : 0, hi = span & ~15;
        unsigned char* dst_al = reinterpret_cast<unsigned char*>(gd) + (e0 * ES - mis);
        if (tid == 0 && hi > lo) {
            sp_bulk_s2g(dst_al + lo, blk_smem_u32(res + lo), (uint32_t)(hi - lo));
            sp_bulk_commit();
        }
        if (warp == 1 % SP_WARPS) {
            // head edge: bytes [mis, min(lo, span)); tail edge: bytes [max(hi, lo), span)  (hi >= lo or the window is tiny)
            const int h_end = lo < span ? lo : span;
            const int b = mis + lane * ES;
            if (lane < 16 / ES && b < h_end) *reinterpret_cast<E*>(dst_al + b) = *reinterpret_cast<const E*>(res + b);
            const int t0 = hi > h_end ? hi : h_end;
            const int bt = t0 + (lane - 16) * ES;
            if (lane >= 16 && lane < 16 + 16 / ES && bt < span) *reinterpret_cast<E*>(dst_al + bt) = *reinterpret_cast<const E*>(res + bt);
        }
    }
    if (tid == 0) sp_bulk_wait_all();
}

}  // namespace

cudaError_t blk_launch_softmax_pipe(const BlkSmxPipeParams& p, int dtype, int backward, int sms, cudaStream_t st) {
    const int64_t total = (int64_t)p.num_windows * p.H;
    if (total == 0) return cudaSuccess;
    auto go = [&](auto kern, int nin) -> cudaError_t {
        const int smem = 2 * nin * SP_BUF;
        cudaError_t e = blk_func_smem(reinterpret_cast<const void*>(kern), smem);
        if (e != cudaSuccess) return e;
        const int64_t resident = (int64_t)sms * (nin == 1 ? 8 : 4);
        const dim3 grid((unsigned)(total < resident ? total : resident)), block(SP_THREADS);
        kern<<<grid, block, smem, st>>>(p);
        return cudaGetLastError();
    };
    if (!backward) {
        if (dtype == BLK_F16) return go(blk_softmax_pipe_kernel<SpIO16<BlkHalfTag>, false>, 1);
        if (dtype == BLK_BF16) return go(blk_softmax_pipe_kernel<SpIO16<BlkBf16Tag>, false>, 1);
        return go(blk_softmax_pipe_kernel<SpIO32, false>, 1);
    }
    if (dtype == BLK_F16) return go(blk_softmax_pipe_kernel<SpIO16<BlkHalfTag>, true>, 2);
    if (dtype == BLK_BF16) return go(blk_softmax_pipe_kernel<SpIO16<BlkBf16Tag>, true>, 2);
    return go(blk_softmax_pipe_kernel<SpIO32, true>, 2);
}
