// Device-side helpers shared by the kernels of libblkattn (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "blk_internal.h"

#define BLK_LOG2E 1.4426950408889634f

// 16-bit storage type used for both fp16 and bf16 buffers; the tag types pick
// the arithmetic.
struct BlkHalfTag {};
struct BlkBf16Tag {};

template <typename Tag> struct BlkCvt;
template <> struct BlkCvt<BlkHalfTag> {
    static __device__ __forceinline__ uint32_t pack2(float a, float b) {
        __half2 h = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&h);
    }
    static __device__ __forceinline__ uint16_t pack1(float a) {
        __half h = __float2half_rn(a);
        return *reinterpret_cast<uint16_t*>(&h);
    }
    static __device__ __forceinline__ float unpack1(uint16_t v) {
        return __half2float(*reinterpret_cast<__half*>(&v));
    }
};
template <> struct BlkCvt<BlkBf16Tag> {
    static __device__ __forceinline__ uint32_t pack2(float a, float b) {
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&h);
    }
    static __device__ __forceinline__ uint16_t pack1(float a) {
        __nv_bfloat16 h = __float2bfloat16_rn(a);
        return *reinterpret_cast<uint16_t*>(&h);
    }
    static __device__ __forceinline__ float unpack1(uint16_t v) {
        return __uint_as_float(((uint32_t)v) << 16);
    }
};

// D(16x8,f32) += A(16x16) * B(16x8); A row-major fragment, B column fragment.
template <typename Tag>
__device__ __forceinline__ void blk_mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void blk_mma16816<BlkHalfTag>(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                         uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void blk_mma16816<BlkBf16Tag>(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                         uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t blk_smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void blk_ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void blk_ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

__device__ __forceinline__ float blk_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// max(a, b, c) in one instruction (three-input maximum of sm_100).
__device__ __forceinline__ float blk_max3(float a, float b, float c) {
    float y;
    asm("max.f32 %0, %1, %2, %3;\n" : "=f"(y) : "f"(a), "f"(b), "f"(c));
    return y;
}
// exp2 of two values at once on packed 16-bit arguments: the pair is rounded to the Tag's 16-bit format, one
// special-function instruction evaluates both, and the result is the packed pair in that format.
template <typename Tag> __device__ __forceinline__ uint32_t blk_exp2_pair(float a, float b);
template <> __device__ __forceinline__ uint32_t blk_exp2_pair<BlkHalfTag>(float a, float b) {
    uint32_t x = BlkCvt<BlkHalfTag>::pack2(a, b), y;
    asm("ex2.approx.f16x2 %0, %1;\n" : "=r"(y) : "r"(x));
    return y;
}
template <> __device__ __forceinline__ uint32_t blk_exp2_pair<BlkBf16Tag>(float a, float b) {
    uint32_t x = BlkCvt<BlkBf16Tag>::pack2(a, b), y;
    asm("ex2.approx.ftz.bf16x2 %0, %1;\n" : "=r"(y) : "r"(x));
    return y;
}

// 16-byte global load that does not allocate in L1 (data touched once).  Not a
// read-only (.nc) load: the softmax may run in place.
__device__ __forceinline__ uint4 blk_ldg_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
// Shared-memory stores through 32-bit shared-window addresses.
__device__ __forceinline__ void blk_sts_b32(uint32_t addr, uint32_t v) {
    asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(addr), "r"(v));
}
__device__ __forceinline__ void blk_sts_b16(uint32_t addr, uint32_t v) {
    asm volatile("st.shared.b16 [%0], %1;\n" ::"r"(addr), "h"((uint16_t)v));
}
__device__ __forceinline__ void blk_sts_f32(uint32_t addr, float v) {
    asm volatile("st.shared.f32 [%0], %1;\n" ::"r"(addr), "f"(v));
}
__device__ __forceinline__ void blk_sts_f32x2(uint32_t addr, float x, float y) {
    asm volatile("st.shared.v2.f32 [%0], {%1, %2};\n" ::"r"(addr), "f"(x), "f"(y));
}

__device__ __forceinline__ uint4 blk_ldg16(const void* p) {
    return __ldg(reinterpret_cast<const uint4*>(p));
}

__device__ __forceinline__ float blk_quad_max(float v) {
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
    return v;
}
__device__ __forceinline__ float blk_quad_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    return v;
}
