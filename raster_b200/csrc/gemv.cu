// Decode-shape (M <= 16) dequant-fused GEMV kernels for sm_100a.
//
// Replaces, on the device, the reference's CPU stream GEMV
//   qmatmul-q4-x8! / qmatmul-q8-x8!   src/raster/quant/kernels.clj:216-247, :308-333
// (mode A8: integer block dots, zero-point fold, per-block scale) and the
// float-activation linear
//   qlinear-q8                        src/raster/quant/train.clj:77-108
// (mode F: y = dequant(W) . x).
//
// Work decomposition.  One CTA (8 warps) owns one group of 32 output rows and
// one contiguous K-slice of that group; with S slices per group the CTAs of a
// group leave their partial sums in scratch and the last one to arrive adds
// them in slice order (no spinning, result independent of arrival order).
// Inside a CTA warp w takes blocks w, w+8, ... of the slice.  A lane loads its
// 16-byte slot of each unit straight from global memory (streaming, L1
// no-allocate) -- by the mma32 layout that slot is already its share of the
// tensor-core A fragments of two 16-row tiles, so nibbles are unpacked with
// three logic ops per register and no data moves between lanes.  The token
// dimension (M <= 8 per n-tile) is the n = 8 side of mma.sync, so one
// instruction forms all M block dots of 16 rows; per-block scales are applied
// to the accumulator fragment in registers.  Activations for the slice are
// staged once per CTA in shared memory in fragment order.
#include <cuda_bf16.h>

#include "internal.h"

namespace rstq {

constexpr int kThreads = 256;
constexpr int kWarps = 8;
constexpr int kBatch = 2;                    // units in flight per lane per buffer
constexpr int kSmemCap = 64 * 1024;          // activation staging budget per CTA

// ---------------------------------------------------------------------------
// small device helpers
// ---------------------------------------------------------------------------
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

// ---------------------------------------------------------------------------
// unit registers: one lane's share of `kBatch` units
// ---------------------------------------------------------------------------
template <int BITS>
struct UnitRegs {
    uint4 c0;
    uint4 c1;   // second plane, 8-bit only
    float4 sc;  // scales of rows gid + 8i
};

template <int BITS>
__device__ __forceinline__ void load_unit(UnitRegs<BITS>& u, const uint8_t* unit, int lane,
                                          bool valid) {
    constexpr int CODES = BITS == 4 ? kUnitCodesQ4 : kUnitCodesQ8;
    if (valid) {
        u.c0 = ldg_stream_u4(unit + lane * 16);
        if (BITS == 8) u.c1 = ldg_stream_u4(unit + 512 + lane * 16);
        u.sc = ldg_f4(unit + CODES + (lane >> 2) * 16);
    } else {
        u.c0 = make_uint4(0, 0, 0, 0);
        u.c1 = make_uint4(0, 0, 0, 0);
        u.sc = make_float4(0.f, 0.f, 0.f, 0.f);
    }
}

struct SliceInfo {
    int g, s, b0, nblk;
};
__device__ __forceinline__ SliceInfo slice_of_cta(int S, int nb) {
    SliceInfo si;
    si.g = blockIdx.x / S;
    si.s = blockIdx.x - si.g * S;
    si.b0 = (int)(((int64_t)si.s * nb) / S);
    si.nblk = (int)(((int64_t)(si.s + 1) * nb) / S) - si.b0;
    return si;
}

// Sum over the 8 warps of the accumulator fragment element that holds
// (row, col) of the CTA's 32 x (NT*8) tile.  red is [warp][v][lane].
template <int NT>
__device__ __forceinline__ float reduce_rc(const float* red, int row, int col) {
    constexpr int NV = NT * 8;
    const int gid = row & 7, i = row >> 3;
    const int nt = col >> 3, within = col & 7;
    const int lane = gid * 4 + (within >> 1);
    const int v = (nt * 4 + i) * 2 + (within & 1);
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) s += red[(w * NV + v) * 32 + lane];
    return s;
}

__device__ __forceinline__ void store_out(void* y, int out_dtype, int64_t idx, float v) {
    if (out_dtype == RSTQ_BF16)
        reinterpret_cast<__nv_bfloat16*>(y)[idx] = __float2bfloat16_rn(v);
    else
        reinterpret_cast<float*>(y)[idx] = v;
}

// Shared tail of both kernels: cross-warp reduction, then either the final
// store (S == 1) or the partial store + last-arriver sum.
// T = accumulator columns per token (split terms of a float activation).
template <int NT>
__device__ __forceinline__ void finish(float (&acc)[NT][4][2], float* red, const SliceInfo& si,
                                       int S, int M, int T, int64_t out, void* y, int out_dtype,
                                       float* partials, int* counters) {
    constexpr int NV = NT * 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();  // staging area is dead from here on
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int c = 0; c < 2; ++c)
                red[(warp * NV + (nt * 4 + i) * 2 + c) * 32 + lane] = acc[nt][i][c];
    __syncthreads();
    const int64_t row0 = (int64_t)si.g * 32;
    if (S == 1) {
        for (int o = threadIdx.x; o < M * 32; o += kThreads) {
            const int m = o >> 5, row = o & 31;
            float s = 0.f;
            for (int t = 0; t < T; ++t) s += reduce_rc<NT>(red, row, m * T + t);
            if (row0 + row < out) store_out(y, out_dtype, (int64_t)m * out + row0 + row, s);
        }
        return;
    }
    float* mine = partials + (int64_t)blockIdx.x * M * 32;
    for (int o = threadIdx.x; o < M * 32; o += kThreads) {
        const int m = o >> 5, row = o & 31;
        float s = 0.f;
        for (int t = 0; t < T; ++t) s += reduce_rc<NT>(red, row, m * T + t);
        mine[o] = s;
    }
    __threadfence();
    __shared__ int s_last;
    __syncthreads();
    if (threadIdx.x == 0) {
        const int prev = atomicAdd(&counters[si.g], 1);
        s_last = (prev == S - 1);
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const float* base = partials + (int64_t)si.g * S * M * 32;
    for (int o = threadIdx.x; o < M * 32; o += kThreads) {
        const int m = o >> 5, row = o & 31;
        float s = 0.f;
        for (int k = 0; k < S; ++k) s += __ldcg(base + (int64_t)k * M * 32 + o);
        if (row0 + row < out) store_out(y, out_dtype, (int64_t)m * out + row0 + row, s);
    }
    if (threadIdx.x == 0) counters[si.g] = 0;  // ready for the next launch
}

// ---------------------------------------------------------------------------
// mode A8
// ---------------------------------------------------------------------------
struct A8Params {
    const uint8_t* w;
    const int8_t* xq;
    const float* xs;
    const int32_t* xsum;
    float* y;
    float* partials;
    int* counters;
    int64_t in, out;
    int M, nb, S, zp;
};

// smem per block of the slice: [2 planes][NC cols][4 words] int8 codes, then
// the per-column {xs, zp*xsum} pairs in a second array.
template <int BITS, int NT, bool ONECOL>
__global__ void __launch_bounds__(kThreads, (BITS == 4 && NT == 1) ? 3 : 2)
gemv_a8_kernel(const A8Params p) {
    constexpr int UNIT = BITS == 4 ? kUnitBytesQ4 : kUnitBytesQ8;
    constexpr int NC = NT * 8;
    extern __shared__ __align__(16) uint8_t smem[];
    const SliceInfo si = slice_of_cta(p.S, p.nb);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gid = lane >> 2, tig = lane & 3;
    const uint8_t* wslice = p.w + ((int64_t)si.g * p.nb + si.b0) * UNIT;

    // first batch of weight loads goes out before anything else
    UnitRegs<BITS> cur[kBatch];
    int k = warp;
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
        const int bl = k + u * kWarps;
        load_unit<BITS>(cur[u], wslice + (int64_t)bl * UNIT, lane, bl < si.nblk);
    }

    // stage this slice's quantized activations in fragment order
    uint4* sxq = reinterpret_cast<uint4*>(smem);                       // [nblk][2][NC]
    int2* sxz = reinterpret_cast<int2*>(smem + (size_t)si.nblk * 2 * NC * 16);  // [nblk][NC]
    for (int i = threadIdx.x; i < si.nblk * 2 * NC; i += kThreads) {
        const int bl = i / (2 * NC), r = i - bl * 2 * NC;
        const int pl = r / NC, c = r - pl * NC;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (c < p.M)
            v = *reinterpret_cast<const uint4*>(p.xq + (int64_t)c * p.in +
                                                (int64_t)(si.b0 + bl) * 32 + pl * 16);
        sxq[i] = v;
    }
    for (int i = threadIdx.x; i < si.nblk * NC; i += kThreads) {
        const int bl = i / NC, c = i - bl * NC;
        int2 v = make_int2(0, 0);
        if (c < p.M) {
            const int64_t idx = (int64_t)c * p.nb + si.b0 + bl;
            v.x = __float_as_int(p.xs[idx]);
            v.y = p.xsum ? p.zp * p.xsum[idx] : 0;
        }
        sxz[i] = v;
    }
    __syncthreads();

    float acc[NT][4][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nt][i][0] = acc[nt][i][1] = 0.f;

    const uint32_t* sxw = reinterpret_cast<const uint32_t*>(sxq);
    while (k < si.nblk) {
        UnitRegs<BITS> nxt[kBatch];
        const int kn = k + kBatch * kWarps;
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            const int bl = kn + u * kWarps;
            load_unit<BITS>(nxt[u], wslice + (int64_t)bl * UNIT, lane, bl < si.nblk);
        }
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            const int bl = k + u * kWarps;
            if (bl >= si.nblk) break;
            uint32_t a[2][4];
            if (BITS == 4) {
                const uint32_t w0 = cur[u].c0.x, w1 = cur[u].c0.y, w2 = cur[u].c0.z,
                               w3 = cur[u].c0.w;
                a[0][0] = w0 & 0x0F0F0F0Fu;
                a[0][1] = w1 & 0x0F0F0F0Fu;
                a[0][2] = (w0 >> 4) & 0x0F0F0F0Fu;
                a[0][3] = (w1 >> 4) & 0x0F0F0F0Fu;
                a[1][0] = w2 & 0x0F0F0F0Fu;
                a[1][1] = w3 & 0x0F0F0F0Fu;
                a[1][2] = (w2 >> 4) & 0x0F0F0F0Fu;
                a[1][3] = (w3 >> 4) & 0x0F0F0F0Fu;
            } else {
                a[0][0] = cur[u].c0.x;
                a[0][1] = cur[u].c0.y;
                a[0][2] = cur[u].c1.x;
                a[0][3] = cur[u].c1.y;
                a[1][0] = cur[u].c0.z;
                a[1][1] = cur[u].c0.w;
                a[1][2] = cur[u].c1.z;
                a[1][3] = cur[u].c1.w;
            }
            const float sc[4] = {cur[u].sc.x, cur[u].sc.y, cur[u].sc.z, cur[u].sc.w};
            const uint32_t* xw = sxw + (size_t)bl * 2 * NC * 4;
            const int2* xz = sxz + (size_t)bl * NC;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const uint32_t b0 = xw[(nt * 8 + gid) * 4 + tig];
                const uint32_t b1 = xw[(NC + nt * 8 + gid) * 4 + tig];
                const int4 z = *reinterpret_cast<const int4*>(xz + nt * 8 + 2 * tig);
                const float xs0 = __int_as_float(z.x), xs1 = __int_as_float(z.z);
#pragma unroll
                for (int mt = 0; mt < 2; ++mt) {
                    int c[4];
                    imma_u8s8(c, a[mt], b0, b1);
                    const float s0 = sc[2 * mt], s1 = sc[2 * mt + 1];
                    acc[nt][2 * mt][0] =
                        fmaf(s0 * xs0, small_int_to_float(c[0] - z.y), acc[nt][2 * mt][0]);
                    acc[nt][2 * mt + 1][0] =
                        fmaf(s1 * xs0, small_int_to_float(c[2] - z.y), acc[nt][2 * mt + 1][0]);
                    if (!ONECOL) {
                        acc[nt][2 * mt][1] =
                            fmaf(s0 * xs1, small_int_to_float(c[1] - z.w), acc[nt][2 * mt][1]);
                        acc[nt][2 * mt + 1][1] = fmaf(s1 * xs1, small_int_to_float(c[3] - z.w),
                                                      acc[nt][2 * mt + 1][1]);
                    }
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kBatch; ++u) cur[u] = nxt[u];
        k = kn;
    }
    finish<NT>(acc, reinterpret_cast<float*>(smem), si, p.S, p.M, 1, p.out, p.y, RSTQ_F32,
               p.partials, p.counters);
}

// ---------------------------------------------------------------------------
// mode F
// ---------------------------------------------------------------------------
struct FParams {
    const uint8_t* w;
    const void* x;
    void* y;
    float* partials;
    int* counters;
    int64_t in, out;
    int M, T, nb, S, act_dtype, out_dtype;
};

// Term t of the bf16 expansion x = t0 + t1 + t2 (each step exact in f32).
__device__ __forceinline__ __nv_bfloat16 bf16_term(float x, int t) {
    __nv_bfloat16 h = __float2bfloat16_rn(x);
    for (int j = 0; j < t; ++j) {
        x -= __bfloat162float(h);
        h = __float2bfloat16_rn(x);
    }
    return h;
}

// smem per block: [2 halves][NC cols][4 tig] entries of 8 bytes = bf16
// (e0, e2, e1, e3) of the four elements 16h + 4tig + 0..3 of that column.
template <int BITS, int NT>
__global__ void __launch_bounds__(kThreads, 2) gemv_f_kernel(const FParams p) {
    constexpr int UNIT = BITS == 4 ? kUnitBytesQ4 : kUnitBytesQ8;
    constexpr int NC = NT * 8;
    extern __shared__ __align__(16) uint8_t smem[];
    const SliceInfo si = slice_of_cta(p.S, p.nb);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gid = lane >> 2, tig = lane & 3;
    const uint8_t* wslice = p.w + ((int64_t)si.g * p.nb + si.b0) * UNIT;

    UnitRegs<BITS> cur[kBatch];
    int k = warp;
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
        const int bl = k + u * kWarps;
        load_unit<BITS>(cur[u], wslice + (int64_t)bl * UNIT, lane, bl < si.nblk);
    }

    uint2* sx = reinterpret_cast<uint2*>(smem);  // [nblk][2][NC][4]
    const int ncols = p.M * p.T;
    for (int i = threadIdx.x; i < si.nblk * 2 * NC * 4; i += kThreads) {
        const int tg = i & 3;
        const int c = (i >> 2) % NC;
        const int h = ((i >> 2) / NC) & 1;
        const int bl = (i >> 2) / (2 * NC);
        uint2 v = make_uint2(0, 0);
        if (c < ncols) {
            const int m = c / p.T, t = c - m * p.T;
            const int64_t e = (int64_t)m * p.in + (int64_t)(si.b0 + bl) * 32 + h * 16 + tg * 4;
            __nv_bfloat16 q[4];
            if (p.act_dtype == RSTQ_BF16) {
                const uint2 raw = *reinterpret_cast<const uint2*>(
                    reinterpret_cast<const __nv_bfloat16*>(p.x) + e);
                q[0] = __ushort_as_bfloat16((unsigned short)(raw.x & 0xFFFF));
                q[1] = __ushort_as_bfloat16((unsigned short)(raw.x >> 16));
                q[2] = __ushort_as_bfloat16((unsigned short)(raw.y & 0xFFFF));
                q[3] = __ushort_as_bfloat16((unsigned short)(raw.y >> 16));
            } else {
                const float4 f = *reinterpret_cast<const float4*>(
                    reinterpret_cast<const float*>(p.x) + e);
                q[0] = bf16_term(f.x, t);
                q[1] = bf16_term(f.y, t);
                q[2] = bf16_term(f.z, t);
                q[3] = bf16_term(f.w, t);
            }
            v.x = (uint32_t)__bfloat16_as_ushort(q[0]) | ((uint32_t)__bfloat16_as_ushort(q[2]) << 16);
            v.y = (uint32_t)__bfloat16_as_ushort(q[1]) | ((uint32_t)__bfloat16_as_ushort(q[3]) << 16);
        }
        sx[i] = v;
    }
    __syncthreads();

    float acc[NT][4][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nt][i][0] = acc[nt][i][1] = 0.f;

    while (k < si.nblk) {
        UnitRegs<BITS> nxt[kBatch];
        const int kn = k + kBatch * kWarps;
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            const int bl = kn + u * kWarps;
            load_unit<BITS>(nxt[u], wslice + (int64_t)bl * UNIT, lane, bl < si.nblk);
        }
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            const int bl = k + u * kWarps;
            if (bl >= si.nblk) break;
            // fr[h][i][j]: half h, row i, j = 0 -> elements (+0, +2), j = 1 -> (+1, +3)
            uint32_t fr[2][4][2];
            const uint32_t c0[4] = {cur[u].c0.x, cur[u].c0.y, cur[u].c0.z, cur[u].c0.w};
            const uint32_t c1[4] = {cur[u].c1.x, cur[u].c1.y, cur[u].c1.z, cur[u].c1.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (BITS == 4) {
                    // 0x4300 | n is bf16(128 + n); subtract 128 + zero point 8
                    const uint32_t w = c0[i];
                    const uint32_t m4 = 0x000F000Fu, ex = 0x43004300u, off = 0x43084308u;
                    fr[0][i][0] = sub_bf16x2((w & m4) | ex, off);
                    fr[0][i][1] = sub_bf16x2(((w >> 8) & m4) | ex, off);
                    fr[1][i][0] = sub_bf16x2(((w >> 4) & m4) | ex, off);
                    fr[1][i][1] = sub_bf16x2(((w >> 12) & m4) | ex, off);
                } else {
                    // 0x4B000000 | b is f32(2^23 + b); subtract 2^23 + zero point 128
                    const float off = 8388736.0f;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint32_t w = h ? c1[i] : c0[i];
                        const float f0 = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7440)) - off;
                        const float f1 = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7441)) - off;
                        const float f2 = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7442)) - off;
                        const float f3 = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7443)) - off;
                        fr[h][i][0] = pack_bf16x2(f2, f0);
                        fr[h][i][1] = pack_bf16x2(f3, f1);
                    }
                }
            }
            const float sc[4] = {cur[u].sc.x, cur[u].sc.y, cur[u].sc.z, cur[u].sc.w};
            const uint2* xb = sx + (size_t)bl * 2 * NC * 4;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const uint2 bx0 = xb[(nt * 8 + gid) * 4 + tig];
                const uint2 bx1 = xb[(NC + nt * 8 + gid) * 4 + tig];
#pragma unroll
                for (int mt = 0; mt < 2; ++mt) {
                    const int r0 = 2 * mt, r1 = 2 * mt + 1;
                    float c[4] = {0.f, 0.f, 0.f, 0.f};
                    const uint32_t a_lo[4] = {fr[0][r0][0], fr[0][r1][0], fr[0][r0][1], fr[0][r1][1]};
                    const uint32_t a_hi[4] = {fr[1][r0][0], fr[1][r1][0], fr[1][r0][1], fr[1][r1][1]};
                    hmma_bf16(c, a_lo, bx0.x, bx0.y);
                    hmma_bf16(c, a_hi, bx1.x, bx1.y);
                    acc[nt][r0][0] = fmaf(sc[r0], c[0], acc[nt][r0][0]);
                    acc[nt][r0][1] = fmaf(sc[r0], c[1], acc[nt][r0][1]);
                    acc[nt][r1][0] = fmaf(sc[r1], c[2], acc[nt][r1][0]);
                    acc[nt][r1][1] = fmaf(sc[r1], c[3], acc[nt][r1][1]);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kBatch; ++u) cur[u] = nxt[u];
        k = kn;
    }
    finish<NT>(acc, reinterpret_cast<float*>(smem), si, p.S, p.M, p.T, p.out, p.y, p.out_dtype,
               p.partials, p.counters);
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
static int choose_slices(const rstq_ctx* ctx, const DeviceState& ds, int64_t groups, int64_t nb,
                         int smem_per_block, int reduce_bytes) {
    // smallest S whose slice fits the staging budget
    int64_t per_cta_max = kSmemCap / smem_per_block;
    if (per_cta_max < 1) per_cta_max = 1;
    int64_t smin = (nb + per_cta_max - 1) / per_cta_max;
    if (smin < 1) smin = 1;
    int64_t smax = nb / (2 * kWarps);  // keep >= 2 blocks per warp
    if (smax < smin) smax = smin;
    int64_t S;
    if (ctx->tune_splitk > 0) {
        S = ctx->tune_splitk;
    } else {
        // aim at ~32 blocks per CTA, but do not cut large problems finer than
        // about four CTAs per resident slot
        const int64_t resident = (int64_t)ds.sm_count * ds.gemv_ctas_per_sm;
        S = (nb + 16) / 32;
        const int64_t cap = (4 * resident + groups - 1) / groups;
        if (S > cap) S = cap;
    }
    if (S < smin) S = smin;
    if (S > smax) S = smax;
    if (S > nb) S = nb;
    if (S < 1) S = 1;
    (void)reduce_bytes;
    return (int)S;
}

static size_t smem_bytes(int64_t nb, int S, int smem_per_block, int NT) {
    const int64_t nblk = (nb + S - 1) / S;  // largest slice
    size_t stage = (size_t)nblk * smem_per_block;
    size_t red = (size_t)kWarps * NT * 8 * 32 * sizeof(float);
    return stage > red ? stage : red;
}

template <typename K>
static int32_t set_smem_attr(K kernel) {
    RSTQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   kSmemCap + 8 * 1024));
    return RSTQ_OK;
}

int32_t gemv_configure(DeviceState& ds) {
    int32_t rc;
#define CFG(k) if ((rc = set_smem_attr(k)) != RSTQ_OK) return rc
    CFG((gemv_a8_kernel<4, 1, true>));
    CFG((gemv_a8_kernel<4, 1, false>));
    CFG((gemv_a8_kernel<4, 2, false>));
    CFG((gemv_a8_kernel<8, 1, true>));
    CFG((gemv_a8_kernel<8, 1, false>));
    CFG((gemv_a8_kernel<8, 2, false>));
    CFG((gemv_f_kernel<4, 1>));
    CFG((gemv_f_kernel<4, 2>));
    CFG((gemv_f_kernel<4, 4>));
    CFG((gemv_f_kernel<8, 1>));
    CFG((gemv_f_kernel<8, 2>));
    CFG((gemv_f_kernel<8, 4>));
#undef CFG
    ds.gemv_ctas_per_sm = 3;
    return RSTQ_OK;
}

static int32_t check_scratch(const DeviceState& ds, int64_t groups, int S, int64_t M) {
    if (S == 1) return RSTQ_OK;
    RSTQ_REQUIRE(groups <= ds.counters_len, RSTQ_E_LIMIT,
                 "out = %lld rows needs %lld split-K counters, limit %lld", (long long)groups * 32,
                 (long long)groups, (long long)ds.counters_len);
    const int64_t need = groups * S * M * 32 * (int64_t)sizeof(float);
    RSTQ_REQUIRE(need <= ds.partials_bytes, RSTQ_E_LIMIT,
                 "split-K partials need %lld bytes, scratch holds %lld", (long long)need,
                 (long long)ds.partials_bytes);
    return RSTQ_OK;
}

int32_t launch_gemv_a8(rstq_ctx* ctx, DeviceState& ds, const GemvA8Args& a) {
    RSTQ_REQUIRE(a.M >= 1 && a.M <= kGemvMaxM, RSTQ_E_SHAPE, "decode kernel takes 1 <= M <= %d",
                 kGemvMaxM);
    const int NT = a.M <= 8 ? 1 : 2;
    const int64_t nb = a.in / 32, groups = (a.out + 31) / 32;
    const int per_block = NT * 8 * 40;
    const int S = choose_slices(ctx, ds, groups, nb, per_block, 0);
    int32_t rc = check_scratch(ds, groups, S, a.M);
    if (rc != RSTQ_OK) return rc;
    RSTQ_REQUIRE(groups * S < (1ll << 31), RSTQ_E_LIMIT, "grid too large");
    A8Params p{a.w, a.xq, a.xs, a.xsum, a.y, ds.partials, ds.counters, a.in, a.out,
               (int)a.M, (int)nb, S, a.zp};
    const size_t smem = smem_bytes(nb, S, per_block, NT);
    const dim3 grid((unsigned)(groups * S));
#define LAUNCH(B, N, O) gemv_a8_kernel<B, N, O><<<grid, kThreads, smem, ds.stream>>>(p)
    if (a.bits == 4) {
        if (NT == 2) LAUNCH(4, 2, false);
        else if (a.M == 1) LAUNCH(4, 1, true);
        else LAUNCH(4, 1, false);
    } else {
        if (NT == 2) LAUNCH(8, 2, false);
        else if (a.M == 1) LAUNCH(8, 1, true);
        else LAUNCH(8, 1, false);
    }
#undef LAUNCH
    ctx->launches++;
    RSTQ_CUDA(cudaGetLastError());
    return RSTQ_OK;
}

int32_t launch_gemv_f(rstq_ctx* ctx, DeviceState& ds, const GemvFArgs& a) {
    RSTQ_REQUIRE(a.M >= 1 && a.M <= kGemvMaxM, RSTQ_E_SHAPE, "decode kernel takes 1 <= M <= %d",
                 kGemvMaxM);
    // f32 activations are expanded into exact bf16 terms: three while they fit
    // one 8-column tile, else two (16 significant bits).
    int T = 1;
    if (a.act_dtype == RSTQ_F32) T = (3 * a.M <= 8) ? 3 : 2;
    const int64_t cols = a.M * T;
    const int NT = cols <= 8 ? 1 : (cols <= 16 ? 2 : 4);
    const int64_t nb = a.in / 32, groups = (a.out + 31) / 32;
    const int per_block = NT * 8 * 64;
    const int S = choose_slices(ctx, ds, groups, nb, per_block, 0);
    int32_t rc = check_scratch(ds, groups, S, a.M);
    if (rc != RSTQ_OK) return rc;
    RSTQ_REQUIRE(groups * S < (1ll << 31), RSTQ_E_LIMIT, "grid too large");
    FParams p{a.w, a.x, a.y, ds.partials, ds.counters, a.in, a.out,
              (int)a.M, T, (int)nb, S, a.act_dtype, a.out_dtype};
    const size_t smem = smem_bytes(nb, S, per_block, NT);
    const dim3 grid((unsigned)(groups * S));
#define LAUNCH(B, N) gemv_f_kernel<B, N><<<grid, kThreads, smem, ds.stream>>>(p)
    if (a.bits == 4) {
        if (NT == 1) LAUNCH(4, 1);
        else if (NT == 2) LAUNCH(4, 2);
        else LAUNCH(4, 4);
    } else {
        if (NT == 1) LAUNCH(8, 1);
        else if (NT == 2) LAUNCH(8, 2);
        else LAUNCH(8, 4);
    }
#undef LAUNCH
    ctx->launches++;
    RSTQ_CUDA(cudaGetLastError());
    return RSTQ_OK;
}

}  // namespace rstq
