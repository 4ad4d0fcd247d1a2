// Pipelined packed small-segment kernel (K = 64, 16-bit output).
//
// Small segments are grouped on the host into packs: runs of consecutive
// segments whose first operands -- and whose second operands -- are one
// contiguous piece of a head strip of at most 192 rows (24 KB), cut into at
// most 16 blocks of up to 16 first-operand rows of one segment each.  One
// persistent CTA per SM walks its share of the cost-sorted (pack, head) list:
//   warp 0      producer: one lane brings each pack into a 4-slot shared-memory
//               ring with tiled tensor-map copies (cp.async.bulk.tensor, boxes
//               of 64 / 32 / 16 rows of the (64, rows, heads) view of each
//               operand, 128-byte swizzle) plus one bulk copy of the pack's
//               block records, all completing on the slot's mbarrier -- the
//               memory latency is paid by the ring instead of by the registers
//               and occupancy of the arithmetic warps;
//   warps 1-16  consumers in two groups (a group owns two slots, so a warp
//               visits every other unit): each claims blocks of the pack
//               through a per-slot counter, heaviest first, reads mma.sync
//               fragments with ldmatrix (conflict-free under the swizzle),
//               does the softmax in registers (only the tile arithmetic is
//               specialised by tile count, behind one jump per block), lays the
//               result out over the block's own first-operand rows (dead once
//               their fragments are in registers) at the output's 16-byte
//               misalignment, and copies it to global memory as aligned 16-byte
//               vectors.
// Every consumer of a group arrives on the "empty" barrier of the group's
// slots, so a slot is reused only when all eight are done with it; every wait
// is bounded and reports through the status word.
//
// Same arithmetic and the same upstream counterparts as blk_scores_small.cu.
#include <cuda.h>

#include <type_traits>

#include "blk_device.cuh"
#include "blk_kernels.h"

namespace {

constexpr int PK = 64;  // contraction length handled here
constexpr int ROWB = PK * 2;  // bytes per operand row
#ifndef BLK_PIPE_CONSUMERS
#define BLK_PIPE_CONSUMERS 16
#endif
#ifndef BLK_PIPE_GROUPS
#define BLK_PIPE_GROUPS 2
#endif
constexpr int P_CONSUMERS = BLK_PIPE_CONSUMERS;
constexpr int P_THREADS = 32 * (1 + P_CONSUMERS);
constexpr int P_REC_BYTES = 1024;  // block records, padded so that every slot starts on a swizzle-atom boundary
static_assert(BLK_PACK_BLOCKS * (int)sizeof(BlkPackBlock) <= P_REC_BYTES, "record area");
constexpr int P_SLOTS = 4;
constexpr int P_TAIL_PAD = 1024;  // second-operand rows are read up to 7 rows past a run's end
constexpr int P_GROUPS = BLK_PIPE_GROUPS;        // consumer groups; unit u belongs to group u % P_GROUPS
constexpr int P_GROUP_WARPS = P_CONSUMERS / P_GROUPS;
constexpr int P_SCRATCH_BYTES = 128;  // target of staging stores that must not land
static_assert(P_SLOTS % P_GROUPS == 0 && P_CONSUMERS % P_GROUPS == 0, "groups own whole slots");
constexpr uint32_t P_SPIN_LIMIT = 1u << 22;
// Slot layout: the operand regions (first, second and, for the attention variant, the values), then the records.
template <bool ATTN>
struct PL {
    static constexpr int ROWS = ATTN ? BLK_PACK_ROWS_ATTN : BLK_PACK_ROWS;
    static constexpr int NOPER = ATTN ? 3 : 2;
    static constexpr int OPER_BYTES = ROWS * ROWB;
    // the 16-deep steps of P V read up to 15 value rows past a run's end: a cleared guard keeps them finite
    static constexpr int GUARD_BYTES = ATTN ? 16 * ROWB : 0;
    static constexpr int REC_OFF = NOPER * OPER_BYTES + GUARD_BYTES;
    static constexpr int SLOT_BYTES = REC_OFF + P_REC_BYTES;
    static constexpr int SMEM_BYTES = P_SLOTS * SLOT_BYTES + P_TAIL_PAD + 16 * P_SLOTS + 16 + 4 * P_SLOTS + P_SCRATCH_BYTES;
    static_assert(SLOT_BYTES % 1024 == 0 && OPER_BYTES % 1024 == 0, "128-byte swizzle needs 1024-byte aligned regions");
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
};

__device__ __forceinline__ void pb_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void pb_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void pb_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
// One attempt: the hardware suspends the thread for a bounded, implementation-defined time while the phase is pending.
__device__ __forceinline__ bool pb_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred q;\n mbarrier.try_wait.parity.shared::cta.b64 q, [%1], %2;\n selp.u32 %0, 1, 0, q;\n}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after P_SPIN_LIMIT attempts (or when another role gave up), recording `code`.
__device__ __forceinline__ bool pb_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
    for (uint32_t i = 0; i < P_SPIN_LIMIT; ++i) {
        if (pb_try(bar, parity)) return true;
        if ((i & 63u) == 63u && *abort_flag) return false;
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
// Tiled tensor-map copy global -> shared of one box at coordinates (k = 0, c1, c2), completing on an mbarrier.
__device__ __forceinline__ void tma_rows(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];\n"
        ::"r"(dst), "l"(map), "r"(bar), "r"(0), "r"(c1), "r"(c2)
        : "memory");
}
// Brings `rows` rows starting at row `row0` of a head's operand into shared memory at dst as boxes of 64, 32 and
// 16 rows (each box a whole number of 1024-byte swizzle atoms); returns the bytes that will arrive.
// The map's coordinates are (k, row, head), or (k, head, row) when head_first (token-major operand).
__device__ __forceinline__ uint32_t tma_run(uint32_t dst, const CUtensorMap* m64, const CUtensorMap* m32,
                                            const CUtensorMap* m16, uint32_t bar, int row0, int rows, int head,
                                            int head_first) {
    int r = 0;
    while (r < rows) {
        const int rem = rows - r;
        const int box = rem > 48 ? 64 : (rem > 16 ? 32 : 16);
        const CUtensorMap* m = box == 64 ? m64 : (box == 32 ? m32 : m16);
        tma_rows(dst + r * ROWB, m, bar, head_first ? head : row0 + r, head_first ? row0 + r : head);
        r += box;
    }
    return (uint32_t)r * ROWB;
}
// Shared-memory stores by 32-bit address, and predicated global stores as single instructions.
__device__ __forceinline__ void sts_b32(uint32_t addr, uint32_t v) {
    asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void sts_b16(uint32_t addr, uint32_t v) {
    asm volatile("st.shared.b16 [%0], %1;\n" ::"r"(addr), "h"((uint16_t)v) : "memory");
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

// Non-volatile mma wrappers: pure functions of their operands, so the compiler may interleave them with loads.
template <typename Tag>
__device__ __forceinline__ void pk_mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1);
template <>
__device__ __forceinline__ void pk_mma<BlkHalfTag>(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                   uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void pk_mma<BlkBf16Tag>(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                   uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// First product of a tile: the accumulator input is the constant zero, so no registers are cleared beforehand.
template <typename Tag>
__device__ __forceinline__ void pk_mma0(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1);
template <>
__device__ __forceinline__ void pk_mma0<BlkHalfTag>(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                    uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}
template <>
__device__ __forceinline__ void pk_mma0<BlkBf16Tag>(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                    uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

// The arithmetic of one block with exactly NT column tiles: products, optional row softmax, and the staging
// stores (rows g and g + 8 of the block at shared addresses s0a / s1a).  Columns 8 (NT - 1) + 2 t and + 1 of the
// last tile exist when last0 / last1; stores that must not land go to `scratch`.
// ATTN: the probabilities are not stored; they become the first operand of P V (the accumulator fragments of two
// neighbouring score tiles are exactly the first-operand fragment of one 16-deep step), the values' fragments come
// from shared memory through transposing ldmatrix loads (vb / vx address this lane's rows and swizzle), and the
// 16 x 64 result is staged at s0a / s1a (rows g and g + 8) with its 16-byte chunks swizzled by the row.
template <typename Tag, int NT, bool SOFTMAX, bool ATTN>
__device__ __forceinline__ void pack_tiles(const uint32_t (&af)[PK / 16][4], uint32_t b0, uint32_t b1, float sl, bool last0,
                                           bool last1, bool pairs, uint32_t s0a, uint32_t s1a, uint32_t scratch,
                                           uint32_t vb, uint32_t vx, int g, int t) {
    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        // rows 8 j .. 8 j + 7 of the second operand: k 0-31 through b0, k 32-63 through b1
        uint32_t m0[4], m1[4];
        blk_ldmatrix_x4(m0, b0 + j * 8 * ROWB);
        blk_ldmatrix_x4(m1, b1 + j * 8 * ROWB);
        pk_mma0<Tag>(acc[j], af[0][0], af[0][1], af[0][2], af[0][3], m0[0], m0[1]);
        pk_mma<Tag>(acc[j], af[1][0], af[1][1], af[1][2], af[1][3], m0[2], m0[3]);
        pk_mma<Tag>(acc[j], af[2][0], af[2][1], af[2][2], af[2][3], m1[0], m1[1]);
        pk_mma<Tag>(acc[j], af[3][0], af[3][1], af[3][2], af[3][3], m1[2], m1[3]);
    }
    float r0 = sl, r1 = sl;
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
        r0 = __frcp_rn(blk_quad_sum(s0));
        r1 = __frcp_rn(blk_quad_sum(s1));
    }
    if constexpr (ATTN) {
        constexpr int KK = (NT + 1) / 2;  // 16-deep steps over the columns of the scores = rows of the values
        float o[PK / 8][4];
#pragma unroll
        for (int kk = 0; kk < KK; ++kk) {
            const uint32_t a0 = BlkCvt<Tag>::pack2(acc[2 * kk][0] * r0, acc[2 * kk][1] * r0);
            const uint32_t a1 = BlkCvt<Tag>::pack2(acc[2 * kk][2] * r1, acc[2 * kk][3] * r1);
            uint32_t a2 = 0u, a3 = 0u;  // an odd tile count leaves the upper half of the last step empty
            if (2 * kk + 1 < NT) {
                a2 = BlkCvt<Tag>::pack2(acc[2 * kk + 1][0] * r0, acc[2 * kk + 1][1] * r0);
                a3 = BlkCvt<Tag>::pack2(acc[2 * kk + 1][2] * r1, acc[2 * kk + 1][3] * r1);
            }
#pragma unroll
            for (int nn = 0; nn < PK / 16; ++nn) {
                // value rows 16 kk .. 16 kk + 15, columns 16 nn .. 16 nn + 15, transposed into second-operand fragments
                uint32_t m[4];
                blk_ldmatrix_x4_trans(m, vb + kk * 16 * ROWB + (vx ^ (uint32_t)(nn << 5)));
                if (kk == 0) {
                    pk_mma0<Tag>(o[2 * nn], a0, a1, a2, a3, m[0], m[1]);
                    pk_mma0<Tag>(o[2 * nn + 1], a0, a1, a2, a3, m[2], m[3]);
                } else {
                    pk_mma<Tag>(o[2 * nn], a0, a1, a2, a3, m[0], m[1]);
                    pk_mma<Tag>(o[2 * nn + 1], a0, a1, a2, a3, m[2], m[3]);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < PK / 8; ++j) {
            const uint32_t off = (uint32_t)(((j ^ g) << 4) + 4 * t);  // chunk j of a row goes to chunk position j ^ (row & 7)
            sts_b32(s0a + off, BlkCvt<Tag>::pack2(o[j][0], o[j][1]));
            sts_b32(s1a + off, BlkCvt<Tag>::pack2(o[j][2], o[j][3]));
        }
        return;
    }
    // Rows that do not exist were given the address of a scratch area by the caller, so only the last tile's
    // columns need a per-store decision; it is made by choosing the address, which keeps the stores unpredicated.
    if (pairs) {  // every staged pair starts on a 4-byte boundary
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            const uint32_t lo = BlkCvt<Tag>::pack2(acc[j][0] * r0, acc[j][1] * r0);
            const uint32_t hi = BlkCvt<Tag>::pack2(acc[j][2] * r1, acc[j][3] * r1);
            sts_b32(j < NT - 1 || last0 ? s0a + 16 * j : scratch, lo);
            sts_b32(j < NT - 1 || last0 ? s1a + 16 * j : scratch, hi);
        }
    } else {
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            const uint32_t lo = BlkCvt<Tag>::pack2(acc[j][0] * r0, acc[j][1] * r0);
            const uint32_t hi = BlkCvt<Tag>::pack2(acc[j][2] * r1, acc[j][3] * r1);
            sts_b16(j < NT - 1 || last0 ? s0a + 16 * j : scratch, lo);
            sts_b16(j < NT - 1 || last0 ? s1a + 16 * j : scratch, hi);
            sts_b16(j < NT - 1 || last1 ? s0a + 16 * j + 2 : scratch, lo >> 16);
            sts_b16(j < NT - 1 || last1 ? s1a + 16 * j + 2 : scratch, hi >> 16);
        }
    }
}

// One block = up to 16 first-operand rows of one segment against that segment's N <= 64 second-operand rows.
// pA / pB point at the block's operand rows inside the slot.  Only the tile arithmetic is specialised by the
// number of 8-column tiles (one jump per block); fragment loads, staging layout and copy-out are shared, which
// keeps the code the sixteen warps run concurrently small enough for the instruction cache.
// Rows past M and past N are read as whatever follows in shared memory: such rows of the result are never
// stored and such columns are masked before the row reduction.  The result is staged over the block's own
// first-operand rows (M * N * 2 <= M * 128 bytes) and copied to the output at element cbase.
template <typename Tag, bool SOFTMAX, bool FLIP, bool ATTN>
__device__ __forceinline__ void pack_block(void* C, unsigned char* pA, uint32_t sA0, uint32_t sB0, uint32_t sV0, int rowA,
                                           int rowB, int64_t cbase, int64_t out_pitch, int M, int N, float sl,
                                           uint32_t scratch, int lane) {
    const int g = lane >> 2, t = lane & 3;
    const int nt = (N + 7) >> 3;

    // Operand rows sit in shared memory under the 128-byte swizzle of the tensor-map copy: the 16-byte chunk c of
    // row r (row counted from the 1024-byte aligned start of the operand's region) is at chunk c ^ (r & 7).
    // ldmatrix lane l addresses row l % 16 and k-chunk l / 16 of a 16 x 16 first-operand tile.
    uint32_t af[PK / 16][4];
    {
        const uint32_t ra = (uint32_t)rowA + (lane & 15);
        const uint32_t base = sA0 + ra * ROWB, x0 = (((uint32_t)lane >> 4) ^ (ra & 7u)) << 4;
#pragma unroll
        for (int ks = 0; ks < PK / 16; ++ks) blk_ldmatrix_x4(af[ks], base + (x0 ^ (uint32_t)(ks << 5)));
        if (SOFTMAX && FLIP) {  // negative scale: softmax of the negated scores
#pragma unroll
            for (int ks = 0; ks < PK / 16; ++ks)
#pragma unroll
                for (int e = 0; e < 4; ++e) af[ks][e] ^= 0x80008000u;
        }
    }
    // The block's M * N results are contiguous in the output, starting mis bytes into a 16-byte vector.  They
    // are staged at the same offset from the block's (128-byte aligned) rows when that fits, so that staged and
    // global vectors line up and the copy-out needs no shifting.
    const int nbytes = M * N * 2;
    const int64_t g0 = cbase * 2;
    const int mis = (int)(g0 & 15);
    const int so = mis + nbytes <= M * ROWB ? mis : 0;
    {
        // second operand: lane l addresses row l % 8 of an 8-row tile and k-chunk l / 8 (+ 4 for the upper half of k)
        const uint32_t rb = (uint32_t)rowB + (lane & 7);
        const uint32_t bx = (((uint32_t)lane >> 3) ^ (rb & 7u)) << 4;
        const uint32_t b0 = sB0 + rb * ROWB + bx, b1 = sB0 + rb * ROWB + (bx ^ 64u);
        const bool last0 = 8 * (nt - 1) + 2 * t < N, last1 = 8 * (nt - 1) + 2 * t + 1 < N;
        // rows g and g + 8 of the staged block; a row past M is pointed at the scratch area instead.  (Attention:
        // the staged block is the 16 x 64 result, one 128-byte row per first-operand row.)
        const uint32_t row0 = blk_smem_u32(pA) + (uint32_t)(ATTN ? g * ROWB : so + (g * N + 2 * t) * 2);
        const uint32_t s0a = g < M ? row0 : scratch, s1a = g + 8 < M ? row0 + 8 * (ATTN ? ROWB : N * 2) : scratch;
        const bool pairs = ((N | (so >> 1)) & 1) == 0;
        // values: lane l addresses row (l % 8) + 8 ((l / 8) % 2) of a 16-row step and column chunk l / 16 of a pair
        const uint32_t rv = (uint32_t)rowB + (lane & 7);
        const uint32_t vb = sV0 + (rv + ((lane >> 3) & 1) * 8) * ROWB, vx = (((uint32_t)lane >> 4) ^ (rv & 7u)) << 4;
        // one jump to the code for this tile count; only the tile arithmetic is specialised
        switch (nt) {
            case 1: pack_tiles<Tag, 1, SOFTMAX, ATTN>(af, b0, b1, sl, last0, last1, pairs, s0a, s1a, scratch, vb, vx, g, t); break;
            case 2: pack_tiles<Tag, 2, SOFTMAX, ATTN>(af, b0, b1, sl, last0, last1, pairs, s0a, s1a, scratch, vb, vx, g, t); break;
            case 3: pack_tiles<Tag, 3, SOFTMAX, ATTN>(af, b0, b1, sl, last0, last1, pairs, s0a, s1a, scratch, vb, vx, g, t); break;
            case 4: pack_tiles<Tag, 4, SOFTMAX, ATTN>(af, b0, b1, sl, last0, last1, pairs, s0a, s1a, scratch, vb, vx, g, t); break;
            case 5: pack_tiles<Tag, 5, SOFTMAX, ATTN>(af, b0, b1, sl, last0, last1, pairs, s0a, s1a, scratch, vb, vx, g, t); break;
            case 6: pack_tiles<Tag, 6, SOFTMAX, ATTN>(af, b0, b1, sl, last0, last1, pairs, s0a, s1a, scratch, vb, vx, g, t); break;
            case 7: pack_tiles<Tag, 7, SOFTMAX, ATTN>(af, b0, b1, sl, last0, last1, pairs, s0a, s1a, scratch, vb, vx, g, t); break;
            default: pack_tiles<Tag, 8, SOFTMAX, ATTN>(af, b0, b1, sl, last0, last1, pairs, s0a, s1a, scratch, vb, vx, g, t); break;
        }
    }
    __syncwarp();
    if constexpr (ATTN) {
        // the staged 16 x 64 result -> global: M rows of 128 bytes, out_pitch bytes apart, always 16-byte aligned; chunk c of row r sits at
        // chunk position c ^ (r & 7)
        unsigned char* dst = reinterpret_cast<unsigned char*>(C) + cbase * 2;  // row r of the block at dst + r * out_pitch
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int v = lane + 32 * i, r = v >> 3, c = v & 7;
            const uint4 q = *reinterpret_cast<const uint4*>(pA + r * ROWB + ((c ^ (r & 7)) << 4));
            stg_v4_if(dst + r * out_pitch + 16 * c, q, r < M);
        }
        return;
    }
    // staged block -> global.  Lane j owns the 16-byte vector j of the block as aligned in global memory.  The
    // ragged first and last vector go out as single elements (lanes 0-7 and 8-15).
    {
        unsigned char* dst = reinterpret_cast<unsigned char*>(C) + (g0 - mis);  // 16-byte aligned
        const int end = mis + nbytes;
        if (so == mis) {
            for (int lo = 16 * lane; lo < end; lo += 16 * 32)
                stg_v4_if(dst + lo, *reinterpret_cast<const uint4*>(pA + lo), lo >= mis && lo + 16 <= end);
        } else {
            // staged at offset 0: a lane gathers its bytes as five words and funnel-shifts them into place
            for (int lo = 16 * lane; lo < end; lo += 16 * 32) {
                const int x = lo - mis;  // staged byte that goes to dst + lo
                const int xw = x > 0 ? (x & ~3) : 0;
                const int sb = (x & 2) * 8;
                const uint32_t* w = reinterpret_cast<const uint32_t*>(pA + xw);
                const uint32_t w0 = w[0], w1 = w[1], w2 = w[2], w3 = w[3], w4 = w[4];
                uint4 v;
                v.x = __funnelshift_r(w0, w1, sb);
                v.y = __funnelshift_r(w1, w2, sb);
                v.z = __funnelshift_r(w2, w3, sb);
                v.w = __funnelshift_r(w3, w4, sb);
                stg_v4_if(dst + lo, v, lo >= mis && lo + 16 <= end);
            }
        }
        const int tail = end & ~15;
        const bool is_tail = lane >= 8;
        const int b = (is_tail ? tail : 0) + 2 * (lane & 7);  // byte, counted from dst, of this lane's edge element
        const bool first_full = mis == 0 && end >= 16;
        const bool ok = lane < 16 && b >= mis && b < end && (is_tail ? tail != 0 : !first_full);
        const int sx = ok ? b - mis + so : 0;
        stg_b16_if(dst + b, *reinterpret_cast<const uint16_t*>(pA + sx), ok);
    }
}

// The maps of one operand: boxes of 64, 32 and 16 rows.
struct PackMaps {
    CUtensorMap m64, m32, m16;
};

template <typename Tag, bool SOFTMAX, bool FLIP, bool ATTN>
__global__ void __launch_bounds__(P_THREADS, 1)
blk_scores_pipe_kernel(const BlkPackParams p, const __grid_constant__ PackMaps mA, const __grid_constant__ PackMaps mB,
                       const __grid_constant__ PackMaps mV) {
    constexpr int P_OPER_BYTES = PL<ATTN>::OPER_BYTES, P_SLOT_BYTES = PL<ATTN>::SLOT_BYTES;
    constexpr int P_REC_OFF = PL<ATTN>::REC_OFF;  // the block records follow the operand regions (and the guard)
    extern __shared__ __align__(1024) unsigned char pipe_smem[];  // the swizzled operand regions need this alignment
    if (blk_smem_u32(pipe_smem) & 1023u) {  // cannot happen with the alignment above; the swizzle relies on it
        if (threadIdx.x == 0) atomicCAS(p.status, 0, 13);
        return;
    }
    unsigned char* ctl = pipe_smem + P_SLOTS * P_SLOT_BYTES + P_TAIL_PAD;
    uint64_t* bars = reinterpret_cast<uint64_t*>(ctl);  // [s] full, [P_SLOTS + s] empty
    volatile int* abort_flag = reinterpret_cast<volatile int*>(ctl + 16 * P_SLOTS);
    int* next_block = reinterpret_cast<int*>(ctl + 16 * P_SLOTS + 16);  // [s]: next unclaimed block of the pack in slot s
    const uint32_t scratch = blk_smem_u32(ctl + 16 * P_SLOTS + 16 + 4 * P_SLOTS);  // P_SCRATCH_BYTES, written, never read
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t smem0 = blk_smem_u32(pipe_smem), bar0 = blk_smem_u32(bars);
    auto full_bar = [&](uint32_t s) { return bar0 + 8u * s; };
    auto empty_bar = [&](uint32_t s) { return bar0 + 8u * (P_SLOTS + s); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < P_SLOTS; ++s) {
            pb_init(full_bar(s), 1);
            pb_init(empty_bar(s), P_GROUP_WARPS);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (ATTN) {
        // value rows past a segment's end meet probabilities that are exactly zero, but zero times whatever an
        // unwritten region of shared memory holds need not be zero: clear the value regions and their guards once
        for (int s = 0; s < P_SLOTS; ++s) {
            uint4* vreg = reinterpret_cast<uint4*>(pipe_smem + s * P_SLOT_BYTES + 2 * P_OPER_BYTES);
            for (int i = threadIdx.x; i < (P_OPER_BYTES + PL<ATTN>::GUARD_BYTES) / 16; i += P_THREADS)
                vreg[i] = make_uint4(0u, 0u, 0u, 0u);
        }
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // before the first tensor-map copy lands there
    }
    __syncthreads();

    // The CTA's u-th unit is (pack, head) number w = blockIdx.x + u * G, pack = w / H, head = w % H; it uses ring
    // slot u % P_SLOTS and belongs to consumer group u % P_GROUPS (so each group owns P_SLOTS / P_GROUPS slots).
    const uint32_t total = (uint32_t)p.num_packs * (uint32_t)p.H;  // < 2^31, checked at plan creation
    const uint32_t H = (uint32_t)p.H, G = gridDim.x;
    if (warp == 0) {
        if (lane == 0) {
            const uint32_t dq = G / H, dr = G - dq * H;  // (pack, head) advance by (dq, dr) per unit
            uint32_t pack = blockIdx.x / H, hd = blockIdx.x - pack * H;  // blockIdx.x < total by the launch
            BlkPack nxt = p.packs[pack];
            uint32_t u = 0;
            for (uint32_t w = blockIdx.x; w < total; w += G, ++u) {
                const BlkPack pk = nxt;
                const uint32_t hd_now = hd;
                pack += dq;
                hd += dr;
                if (hd >= H) {
                    hd -= H;
                    ++pack;
                }
                if (w + G < total) nxt = p.packs[pack];  // next record in flight during this unit's wait
                const uint32_t s = u % P_SLOTS;
                if (!pb_wait(empty_bar(s), ((u / P_SLOTS) & 1u) ^ 1u, abort_flag, p.status, 11)) break;
                const uint32_t bytesR = (uint32_t)pk.nblocks * (uint32_t)sizeof(BlkPackBlock);
                const uint32_t dst = smem0 + s * P_SLOT_BYTES;
                *reinterpret_cast<volatile int*>(next_block + s) = 0;  // ordered before the consumers' claims by the barrier
                // rows are fetched in whole boxes: up to 15 rows past the run's end come along (zeros past the strip)
                const uint32_t bytesA = (uint32_t)((pk.rowsA + 15) & ~15) * ROWB, bytesB = (uint32_t)((pk.rowsB + 15) & ~15) * ROWB;
                pb_expect_tx(full_bar(s), bytesA + (ATTN ? 2 : 1) * bytesB + bytesR);
                tma_run(dst, &mA.m64, &mA.m32, &mA.m16, full_bar(s), (int)(pk.offA / PK), pk.rowsA, (int)hd_now, p.head_firstA);
                tma_run(dst + P_OPER_BYTES, &mB.m64, &mB.m32, &mB.m16, full_bar(s), (int)(pk.offB / PK), pk.rowsB, (int)hd_now,
                        p.head_firstB);
                if (ATTN)  // the values: one row per second-operand row
                    tma_run(dst + 2 * P_OPER_BYTES, &mV.m64, &mV.m32, &mV.m16, full_bar(s), (int)(pk.offB / PK), pk.rowsB,
                            (int)hd_now, p.head_firstV);
                bulk_g2s(dst + P_REC_OFF, p.blocks + pk.first_block, bytesR, full_bar(s));
            }
        }
    } else {
        const uint32_t group = (uint32_t)(warp - 1) % P_GROUPS;
        const float sl = SOFTMAX ? fabsf(p.scale) * BLK_LOG2E : p.scale;
        const uint32_t step = P_GROUPS * G, dq = step / H, dr = step - dq * H;
        uint32_t w = blockIdx.x + group * G;
        uint32_t hd = w % H;
        for (uint32_t u = group; w < total; w += step, u += P_GROUPS) {
            const uint32_t s = u % P_SLOTS;
            // scores: head strip + element offset; attention: result rows with their own row and head strides
            const int64_t hbase = ATTN ? (int64_t)hd * p.out_head_stride : (int64_t)hd * p.Dout;
            const int64_t out_pitch = ATTN ? p.out_row_stride * 2 : 0;
            hd += dr;
            if (hd >= H) hd -= H;
            if (!pb_wait(full_bar(s), (u / P_SLOTS) & 1u, abort_flag, p.status, 12)) break;
            unsigned char* slot = pipe_smem + s * P_SLOT_BYTES;
            const uint32_t sslot = smem0 + s * P_SLOT_BYTES;
            const BlkPackBlock* recs = reinterpret_cast<const BlkPackBlock*>(slot + P_REC_OFF);
            const int nb = recs[0].nblocks;
            // the group's warps claim the pack's blocks (widest first) one at a time: a warp that finishes early takes more
            for (;;) {
                int b = 0;
                if (lane == 0) b = atomicAdd(next_block + s, 1);
                b = __shfl_sync(0xffffffffu, b, 0);
                if (b >= nb) break;
                const BlkPackBlock r = recs[b];
                pack_block<Tag, SOFTMAX, FLIP, ATTN>(p.C, slot + r.rowA * ROWB, sslot, sslot + P_OPER_BYTES,
                                                     sslot + 2 * P_OPER_BYTES, r.rowA, r.rowB,
                                                     ATTN ? hbase + (r.offC / PK) * p.out_row_stride : hbase + r.offC,
                                                     out_pitch, r.M, r.N, sl, scratch, lane);
            }
            // this warp's reads and writes of the slot are done: order them before the next bulk copy into it
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
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
cudaError_t launch_pipe(const BlkPackParams& p_in, int sms, cudaStream_t st) {
    const int64_t total = (int64_t)p_in.num_packs * p_in.H;
    if (total == 0) return cudaSuccess;
    BlkPackParams p = p_in;
    const bool attn = p.V != nullptr;
    // the operands as (64, rows, heads) views with boxes of 64, 32 and 16 rows
    PackMaps mA, mB, mV;
    const int bf16 = std::is_same<Tag, BlkBf16Tag>::value ? 1 : 0;
    auto maps = [&](PackMaps& m, const void* base, const BlkOperandLayout& lay, int* head_first) {
        return blk_make_row_map(&m.m64, base, bf16, PK, p.H, lay, PK, 64, head_first) &&
               blk_make_row_map(&m.m32, base, bf16, PK, p.H, lay, PK, 32, head_first) &&
               blk_make_row_map(&m.m16, base, bf16, PK, p.H, lay, PK, 16, head_first);
    };
    if (!maps(mA, p.A, p.layA, &p.head_firstA) || !maps(mB, p.B, p.layB, &p.head_firstB)) return cudaErrorInvalidValue;
    if (attn) {
        if (!maps(mV, p.V, p.layV, &p.head_firstV)) return cudaErrorInvalidValue;
    } else {
        mV = mB;  // unused
    }
    const dim3 grid((unsigned)(total < sms ? total : sms)), block(P_THREADS);
    auto go = [&](auto kern, int smem) -> cudaError_t {
        cudaError_t e = blk_func_smem(reinterpret_cast<const void*>(kern), smem);
        if (e != cudaSuccess) return e;
        kern<<<grid, block, smem, st>>>(p, mA, mB, mV);
        return cudaGetLastError();
    };
    if (attn)
        return p.scale < 0.f ? go(blk_scores_pipe_kernel<Tag, true, true, true>, PL<true>::SMEM_BYTES)
                             : go(blk_scores_pipe_kernel<Tag, true, false, true>, PL<true>::SMEM_BYTES);
    if (p.epi != BLK_EPI_SOFTMAX) return go(blk_scores_pipe_kernel<Tag, false, false, false>, PL<false>::SMEM_BYTES);
    return p.scale < 0.f ? go(blk_scores_pipe_kernel<Tag, true, true, false>, PL<false>::SMEM_BYTES)
                         : go(blk_scores_pipe_kernel<Tag, true, false, false>, PL<false>::SMEM_BYTES);
}

}  // namespace

cudaError_t blk_launch_scores_pipe(const BlkPackParams& p, int dtype_in, int sms, cudaStream_t st) {
    return dtype_in == BLK_F16 ? launch_pipe<BlkHalfTag>(p, sms, st) : launch_pipe<BlkBf16Tag>(p, sms, st);
}
