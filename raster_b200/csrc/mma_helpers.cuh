// Device helpers shared by the decode kernels: streaming loads, the two
// mma.sync tiles (int8 m16n8k32, bf16 m16n8k16) and exact small conversions.
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

#include "../../include/rstq.h"

namespace rstq {

__device__ __forceinline__ uint4 ldg_stream_u4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ float4 ldg_f4(const void* p) {
    float4 v;
    asm volatile("ld.global.nc.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "l"(p));
    return v;
}

// D(16x8, s32) = A(16x32, u8, row) * B(32x8, s8, col)
__device__ __forceinline__ void imma_u8s8(int (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                          uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%11,%12,%13};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0), "r"(0), "r"(0),
          "r"(0));
}

// D(16x8, f32) += A(16x16, bf16, row) * B(16x8, bf16, col)
__device__ __forceinline__ void hmma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                          uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// exact int -> float for |v| < 2^22 on the full-rate pipes (no conversion unit)
__device__ __forceinline__ float small_int_to_float(int v) {
    return __int_as_float(0x4B400000 + v) - 12582912.0f;
}

__device__ __forceinline__ uint32_t sub_bf16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float hi, float lo) {
    uint32_t d;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}

// Term t of the bf16 expansion x = t0 + t1 + t2 (each step exact in f32).
__device__ __forceinline__ __nv_bfloat16 bf16_term(float x, int t) {
    __nv_bfloat16 h = __float2bfloat16_rn(x);
    for (int j = 0; j < t; ++j) {
        x -= __bfloat162float(h);
        h = __float2bfloat16_rn(x);
    }
    return h;
}

__device__ __forceinline__ void store_out(void* y, int out_dtype, int64_t idx, float v) {
    if (out_dtype == RSTQ_BF16)
        reinterpret_cast<__nv_bfloat16*>(y)[idx] = __float2bfloat16_rn(v);
    else
        reinterpret_cast<float*>(y)[idx] = v;
}

}  // namespace rstq
