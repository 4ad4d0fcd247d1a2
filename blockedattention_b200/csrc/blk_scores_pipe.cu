// Pipelined packed small-segment kernel (K = 64, 16-bit output).
//
// Small segments are grouped on the host into packs: runs of up to 16
// consecutive segments whose first operands -- and whose second operands -- are
// one contiguous piece of a head strip of at most 192 rows (24 KB).  One
// persistent CTA per SM walks its share of the cost-sorted (pack, head) list:
//   warp 0      producer: one lane brings each pack into a 4-slot shared-memory
//               ring with three bulk asynchronous copies (first operands,
//               second operands, the pack's block records) that complete on
//               the slot's mbarrier -- few, large copies keep the copy engine
//               at memory speed, and the latency is paid by the ring instead of
//               by the registers and occupancy of the arithmetic warps;
//   warps 1-16  consumers: each takes one block (segment) of a pack, computes it
//               as the register-fed small kernel does (k-permuted 128-bit
//               fragment reads, here from shared memory; mma.sync.m16n8k16;
//               softmax in registers; exact tile-count specialisation), lays
//               the result out over the block's own first-operand rows (dead
//               once their fragments are in registers), and copies it to global
//               memory as aligned 16-byte vectors, re-aligning on the fly.
// Every consumer arrives on every slot's "empty" barrier, so a slot is reused
// only when all sixteen are done with it; every wait is bounded and reports
// through the status word.
//
// Same arithmetic and the same upstream counterparts as blk_scores_small.cu.
#include <cstdlib>

#include "blk_device.cuh"
#include "blk_kernels.h"

namespace {

constexpr int PK = 64;  // contraction length handled here
constexpr int PKC = PK / 32;
constexpr int ROWB = PK * 2;  // bytes per operand row
constexpr int P_CONSUMERS = 16;
constexpr int P_THREADS = 32 * (1 + P_CONSUMERS);
constexpr int P_OPER_BYTES = BLK_PACK_ROWS * ROWB;  // 24 KB per operand per slot
constexpr int P_REC_BYTES = BLK_PACK_BLOCKS * (int)sizeof(BlkPackBlock);
constexpr int P_SLOT_BYTES = 2 * P_OPER_BYTES + P_REC_BYTES;
constexpr int P_SLOTS = 4;
constexpr int P_SMEM_BYTES = P_SLOTS * P_SLOT_BYTES + 16 * P_SLOTS + 64;
constexpr uint32_t P_SPIN_LIMIT = 6u << 20;
static_assert(P_SMEM_BYTES <= 227 * 1024, "shared memory budget");
static_assert(BLK_PACK_BLOCKS == P_CONSUMERS, "one consumer per block of a pack");

__device__ __forceinline__ void pb_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void pb_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void pb_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool pb_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred q;\n mbarrier.test_wait.parity.shared::cta.b64 q, [%1], %2;\n selp.u32 %0, 1, 0, q;\n}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool pb_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
    for (uint32_t i = 0; i < P_SPIN_LIMIT; ++i) {
        if (pb_test(bar, parity)) return true;
        if (i > 64) __nanosleep(40);
        if ((i & 255u) == 255u && *abort_flag) return false;
    }
    *abort_flag = 1;
    atomicCAS(status, 0, code);
    return false;
}
// Contiguous global -> shared bulk copy completing on an mbarrier (16-byte aligned addresses and size).
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ uint4 lds16(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds4(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint16_t lds2(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];\n" : "=h"(v) : "r"(addr));
    return v;
}
// Predicated stores as single instructions.
__device__ __forceinline__ void sts_b32_if(uint32_t addr, uint32_t v, bool ok) {
    asm volatile("{\n .reg .pred q;\n setp.ne.b32 q, %2, 0;\n @q st.shared.b32 [%0], %1;\n}\n" ::"r"(addr), "r"(v), "r"((int)ok)
                 : "memory");
}
__device__ __forceinline__ void sts_b16_if(uint32_t addr, uint32_t v, bool ok) {
    asm volatile("{\n .reg .pred q;\n setp.ne.b32 q, %2, 0;\n @q st.shared.b16 [%0], %1;\n}\n" ::"r"(addr), "h"((uint16_t)v),
                 "r"((int)ok)
                 : "memory");
}
__device__ __forceinline__ void stg_v4_if(void* p, const uint4& v, bool ok) {
    asm volatile("{\n .reg .pred q;\n setp.ne.b32 q, %5, 0;\n @q st.global.v4.b32 [%0], {%1, %2, %3, %4};\n}\n" ::"l"(p),
                 "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w), "r"((int)ok)
                 : "memory");
}
__device__ __forceinline__ void stg_b16_if(void* p, uint16_t v, bool ok) {
    asm volatile("{\n .reg .pred q;\n setp.ne.b32 q, %2, 0;\n @q st.global.b16 [%0], %1;\n}\n" ::"l"(p), "h"(v), "r"((int)ok)
                 : "memory");
}

// One block with exactly NT column tiles: operands at shared-window addresses sA / sB, result staged over the
// block's own first-operand rows (M * N * 2 <= M * 128 bytes) and copied to the output at element cbase.
template <typename Tag, int NT, bool SOFTMAX>
__device__ __forceinline__ void pack_block(void* C, uint32_t sA, uint32_t sB, int64_t cbase, int M, int N, float sl,
                                           bool flip, int lane) {
    const int g = lane >> 2, t = lane & 3;
    const bool pair_ok = (N & 1) == 0;  // staged rows start on 4-byte boundaries

    uint4 a[2][PKC];
    auto load_a = [&](int mb) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t pa = sA + min(mb * 16 + g + 8 * h, M - 1) * ROWB + 16 * t;
#pragma unroll
            for (int c = 0; c < PKC; ++c) a[h][c] = lds16(pa + 64 * c);
        }
    };
    load_a(0);
    // rows of the second operand this lane reads (clamped past the end; their columns are masked below)
    uint32_t pb[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) pb[j] = sB + min(8 * j + g, N - 1) * ROWB + 16 * t;
    const bool last0 = 8 * (NT - 1) + 2 * t < N, last1 = 8 * (NT - 1) + 2 * t + 1 < N;
    const uint32_t srow = sA + (g * N + 2 * t) * 2;
    const int nmb = (M + 15) >> 4;
    for (int mb = 0; mb < nmb; ++mb) {
        uint32_t af[2 * PKC][4];
#pragma unroll
        for (int c = 0; c < PKC; ++c) {
            af[2 * c][0] = a[0][c].x; af[2 * c][1] = a[1][c].x; af[2 * c][2] = a[0][c].y; af[2 * c][3] = a[1][c].y;
            af[2 * c + 1][0] = a[0][c].z; af[2 * c + 1][1] = a[1][c].z;
            af[2 * c + 1][2] = a[0][c].w; af[2 * c + 1][3] = a[1][c].w;
        }
        if (SOFTMAX && flip) {
#pragma unroll
            for (int c = 0; c < 2 * PKC; ++c)
#pragma unroll
                for (int e = 0; e < 4; ++e) af[c][e] ^= 0x80008000u;
        }
        if (mb + 1 < nmb) load_a(mb + 1);  // the next rows are in registers before this block's output lands near them
        float acc[NT][4];
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
#pragma unroll
            for (int c = 0; c < PKC; ++c) {
                const uint4 b = lds16(pb[j] + 64 * c);
                blk_mma16816<Tag>(acc[j], af[2 * c][0], af[2 * c][1], af[2 * c][2], af[2 * c][3], b.x, b.y);
                blk_mma16816<Tag>(acc[j], af[2 * c + 1][0], af[2 * c + 1][1], af[2 * c + 1][2], af[2 * c + 1][3], b.z, b.w);
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
        // stage rows 16 mb + g and + 8 if they exist (the staged block must stay inside this block's own rows)
        const uint32_t s0a = srow + (uint32_t)(mb * 16 * N * 2), s1a = s0a + 8 * N * 2;
        const bool v0 = mb * 16 + g < M, v1 = mb * 16 + g + 8 < M;
        if (pair_ok) {
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const bool in = j < NT - 1 || last0;
                sts_b32_if(s0a + 16 * j, BlkCvt<Tag>::pack2(acc[j][0], acc[j][1]), in && v0);
                sts_b32_if(s1a + 16 * j, BlkCvt<Tag>::pack2(acc[j][2], acc[j][3]), in && v1);
            }
        } else {
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const bool in0 = j < NT - 1 || last0, in1 = j < NT - 1 || last1;
                const uint32_t lo = BlkCvt<Tag>::pack2(acc[j][0], acc[j][1]);
                const uint32_t hi = BlkCvt<Tag>::pack2(acc[j][2], acc[j][3]);
                sts_b16_if(s0a + 16 * j, lo, in0 && v0);
                sts_b16_if(s1a + 16 * j, hi, in0 && v1);
                sts_b16_if(s0a + 16 * j + 2, lo >> 16, in1 && v0);
                sts_b16_if(s1a + 16 * j + 2, hi >> 16, in1 && v1);
            }
        }
    }
    __syncwarp();
    // staged block (M * N contiguous elements at sA) -> global.  Lane j owns the 16-byte vector j of the block *as
    // aligned in global memory*; the block starts mis bytes into its first vector, so a lane gathers its bytes
    // from the staged copy as five words and funnel-shifts them into place.  The ragged first and last vector
    // go out as single elements (lanes 0-7 and 8-15).
    {
        const int nbytes = M * N * 2;
        const int64_t g0 = cbase * 2;
        const int mis = (int)(g0 & 15);
        unsigned char* dst = reinterpret_cast<unsigned char*>(C) + (g0 - mis);  // 16-byte aligned
        const int end = mis + nbytes;
        for (int lo = 16 * lane; lo < end; lo += 16 * 32) {
            const int x = lo - mis;  // staged byte that goes to dst + lo
            const int xw = x > 0 ? (x & ~3) : 0;
            const int sb = (x & 2) * 8;
            const uint32_t w0 = lds4(sA + xw), w1 = lds4(sA + xw + 4), w2 = lds4(sA + xw + 8), w3 = lds4(sA + xw + 12),
                           w4 = lds4(sA + xw + 16);
            uint4 v;
            v.x = __funnelshift_r(w0, w1, sb);
            v.y = __funnelshift_r(w1, w2, sb);
            v.z = __funnelshift_r(w2, w3, sb);
            v.w = __funnelshift_r(w3, w4, sb);
            stg_v4_if(dst + lo, v, lo >= mis && lo + 16 <= end);
        }
        const int tail = end & ~15;
        const bool is_tail = lane >= 8;
        const int b = (is_tail ? tail : 0) + 2 * (lane & 7);  // byte, counted from dst, of this lane's edge element
        const bool first_full = mis == 0 && end >= 16;
        const bool ok = lane < 16 && b >= mis && b < end && (is_tail ? tail != 0 : !first_full);
        const int sx = ok ? b - mis : 0;
        stg_b16_if(dst + b, lds2(sA + sx), ok);
    }
}

template <typename Tag, bool SOFTMAX>
__global__ void __launch_bounds__(P_THREADS, 1) blk_scores_pipe_kernel(const BlkPackParams p, int dbg) {
    extern __shared__ __align__(128) unsigned char pipe_smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(pipe_smem + P_SLOTS * P_SLOT_BYTES);  // [s] full, [P_SLOTS + s] empty
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * P_SLOTS);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t smem0 = blk_smem_u32(pipe_smem), bar0 = blk_smem_u32(bars);
    auto full_bar = [&](uint32_t s) { return bar0 + 8u * s; };
    auto empty_bar = [&](uint32_t s) { return bar0 + 8u * (P_SLOTS + s); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < P_SLOTS; ++s) {
            pb_init(full_bar(s), 1);
            pb_init(empty_bar(s), P_CONSUMERS);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();

    const uint32_t total = (uint32_t)p.num_packs * (uint32_t)p.H;  // < 2^31, checked at plan creation
    const uint32_t H = (uint32_t)p.H, G = gridDim.x;
    // the CTA's u-th unit is (pack, head) number w = blockIdx.x + u * G; it uses ring slot u % P_SLOTS
    if (warp == 0) {
        if (lane == 0) {
            uint32_t u = 0;
            BlkPack nxt = p.packs[blockIdx.x / H];  // blockIdx.x < total by the launch
            for (uint32_t w = blockIdx.x; w < total; w += G, ++u) {
                const BlkPack pk = nxt;
                const uint32_t pack = w / H, hd = w - pack * H;
                if (w + G < total) nxt = p.packs[(w + G) / H];  // next record in flight during this unit's wait
                const uint32_t s = u % P_SLOTS;
                if (!pb_wait(empty_bar(s), ((u / P_SLOTS) & 1u) ^ 1u, abort_flag, p.status, 11)) break;
                const uint32_t bytesA = (uint32_t)pk.rowsA * ROWB, bytesB = (uint32_t)pk.rowsB * ROWB;
                const uint32_t bytesR = (uint32_t)pk.nblocks * (uint32_t)sizeof(BlkPackBlock);
                const uint32_t dst = smem0 + s * P_SLOT_BYTES;
                pb_expect_tx(full_bar(s), bytesA + bytesB + bytesR);
                bulk_g2s(dst, p.A + ((int64_t)hd * p.Dm1 + pk.offA), bytesA, full_bar(s));
                bulk_g2s(dst + P_OPER_BYTES, p.B + ((int64_t)hd * p.Dm2 + pk.offB), bytesB, full_bar(s));
                bulk_g2s(dst + 2 * P_OPER_BYTES, p.blocks + pk.first_block, bytesR, full_bar(s));
            }
        }
    } else {
        const uint32_t cw = warp - 1;
        const bool flip = p.scale < 0.f;
        const float sl = SOFTMAX ? fabsf(p.scale) * BLK_LOG2E : p.scale;
        uint32_t u = 0;
        for (uint32_t w = blockIdx.x; w < total; w += G, ++u) {
            const uint32_t s = u % P_SLOTS;
            if (!pb_wait(full_bar(s), (u / P_SLOTS) & 1u, abort_flag, p.status, 12)) break;
            const unsigned char* slot = pipe_smem + s * P_SLOT_BYTES;
            const BlkPackBlock* recs = reinterpret_cast<const BlkPackBlock*>(slot + 2 * P_OPER_BYTES);
            // block b of unit u goes to consumer (b + 5 u) mod 16: spreads short packs over all consumers
            const uint32_t b = (cw - 5u * u) & (P_CONSUMERS - 1);
            if ((int)b < recs[0].nblocks && !(dbg & 1)) {
                const BlkPackBlock r = recs[b];
                const uint32_t hd = w - (w / H) * H;
                const uint32_t sA = smem0 + s * P_SLOT_BYTES + (uint32_t)r.rowA * ROWB;
                const uint32_t sB = smem0 + s * P_SLOT_BYTES + P_OPER_BYTES + (uint32_t)r.rowB * ROWB;
                const int64_t cbase = (int64_t)hd * p.Dout + r.offC;
                switch ((r.N + 7) >> 3) {
                    case 1: pack_block<Tag, 1, SOFTMAX>(p.C, sA, sB, cbase, r.M, r.N, sl, flip, lane); break;
                    case 2: pack_block<Tag, 2, SOFTMAX>(p.C, sA, sB, cbase, r.M, r.N, sl, flip, lane); break;
                    case 3: pack_block<Tag, 3, SOFTMAX>(p.C, sA, sB, cbase, r.M, r.N, sl, flip, lane); break;
                    case 4: pack_block<Tag, 4, SOFTMAX>(p.C, sA, sB, cbase, r.M, r.N, sl, flip, lane); break;
                    case 5: pack_block<Tag, 5, SOFTMAX>(p.C, sA, sB, cbase, r.M, r.N, sl, flip, lane); break;
                    case 6: pack_block<Tag, 6, SOFTMAX>(p.C, sA, sB, cbase, r.M, r.N, sl, flip, lane); break;
                    case 7: pack_block<Tag, 7, SOFTMAX>(p.C, sA, sB, cbase, r.M, r.N, sl, flip, lane); break;
                    default: pack_block<Tag, 8, SOFTMAX>(p.C, sA, sB, cbase, r.M, r.N, sl, flip, lane); break;
                }
                // this warp's reads and writes of the slot are done: order them before the next bulk copy into it
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            }
            __syncwarp();
            if (lane == 0) pb_arrive(empty_bar(s));
        }
    }
    __syncthreads();
    if (*abort_flag) {
        // a role gave up: let copies that may still be in flight land before the CTA's memory is released
        for (int k = 0; k < 64; ++k) __nanosleep(1000);
    }
}

template <typename Tag>
cudaError_t launch_pipe(const BlkPackParams& p, int sms, cudaStream_t st) {
    const int64_t total = (int64_t)p.num_packs * p.H;
    if (total == 0) return cudaSuccess;
    const dim3 grid((unsigned)(total < sms ? total : sms)), block(P_THREADS);
    auto go = [&](auto kern) -> cudaError_t {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM_BYTES);
        if (e != cudaSuccess) return e;
        kern<<<grid, block, P_SMEM_BYTES, st>>>(p, getenv("BLK_PIPE_DBG") ? atoi(getenv("BLK_PIPE_DBG")) : 0);
        return cudaGetLastError();
    };
    return p.epi == BLK_EPI_SOFTMAX ? go(blk_scores_pipe_kernel<Tag, true>) : go(blk_scores_pipe_kernel<Tag, false>);
}

}  // namespace

cudaError_t blk_launch_scores_pipe(const BlkPackParams& p, int dtype_in, int sms, cudaStream_t st) {
    return dtype_in == BLK_F16 ? launch_pipe<BlkHalfTag>(p, sms, st) : launch_pipe<BlkBf16Tag>(p, sms, st);
}
