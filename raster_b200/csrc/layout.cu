// Load-time layout transform: reference host layouts -> the mma32 device layout.
//
// Takes the place of repack-stream (src/raster/compiler/backend/cpu/quant.clj:317-326,
// src/raster/compiler/core/layout.clj:246-286) as the one-time weight re-tiling,
// and accepts every host layout the reference's operators take:
//   row-major Q4_0 / Q8_0  {wq, ws}         quant.clj:42-70
//   8-row stream layout    {wqi, wsi}       layout.clj:246-286
//   signed row-major codes {codes, scales}  src/raster/quant/train.clj:34-58
//                          (= the int32-packed {wp, ws} of src/raster/quant/pack.clj:55-81
//                           read as little-endian bytes)
#include "internal.h"

namespace rstq {

// Source accessors return the *unsigned* stored code of (row, block b, element e).
struct SrcView {
    const uint8_t* codes;
    const float* scales;
    int64_t nb_src;   // blocks per source row
    int64_t kb0;      // first source block of this shard
    int layout;       // RSTQ_LAYOUT_*
};

__device__ __forceinline__ uint32_t src_nibble(const SrcView& s, int64_t row, int64_t b, int e) {
    const int64_t sb = b + s.kb0;
    if (s.layout == RSTQ_LAYOUT_ROWMAJOR) {
        uint32_t bv = s.codes[(row * s.nb_src + sb) * 16 + (e & 15)];
        return e < 16 ? (bv & 0xF) : (bv >> 4);
    }
    // 8-row interleave: byte ((g*nb + b)*8 + ig)*16 + j, j = (row%8 % 4)*4 + e%4,
    // low nibble for rows 0..3 of the group, high nibble for rows 4..7.
    const int64_t g = row >> 3;
    const int rr = (int)(row & 7);
    uint32_t bv = s.codes[((g * s.nb_src + sb) * 8 + (e >> 2)) * 16 + (rr & 3) * 4 + (e & 3)];
    return rr < 4 ? (bv & 0xF) : (bv >> 4);
}

__device__ __forceinline__ uint32_t src_byte(const SrcView& s, int64_t row, int64_t b, int e) {
    const int64_t sb = b + s.kb0;
    if (s.layout == RSTQ_LAYOUT_ROWMAJOR) return s.codes[(row * s.nb_src + sb) * 32 + e];
    const int64_t g = row >> 3;
    const int rr = (int)(row & 7);
    return s.codes[((g * s.nb_src + sb) * 8 + (e >> 2)) * 32 + rr * 4 + (e & 3)];
}

__device__ __forceinline__ float src_scale(const SrcView& s, int64_t row, int64_t b) {
    const int64_t sb = b + s.kb0;
    if (s.layout == RSTQ_LAYOUT_ROWMAJOR) return s.scales[row * s.nb_src + sb];
    return s.scales[((row >> 3) * s.nb_src + sb) * 8 + (row & 7)];
}

// One thread per destination 32-bit word (codes) or scale.
template <int BITS>
__global__ void repack_kernel(SrcView s, uint8_t* __restrict__ dst, int64_t out, int64_t nb,
                              int64_t groups, int flip_sign) {
    constexpr int UNIT = BITS == 4 ? kUnitBytesQ4 : kUnitBytesQ8;
    constexpr int WORDS = UNIT / 4;  // code words + 32 scale words
    const int64_t total = groups * nb * WORDS;
    for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t unit = idx / WORDS;
        const int wi = (int)(idx % WORDS);
        const int64_t g = unit / nb, b = unit % nb;
        uint32_t* dword = reinterpret_cast<uint32_t*>(dst + unit * UNIT) + wi;
        constexpr int CODE_WORDS = (UNIT - 128) / 4;
        if (wi >= CODE_WORDS) {  // scale gid*4 + i -> row 32g + gid + 8i
            const int si = wi - CODE_WORDS;
            const int64_t row = g * 32 + (si >> 2) + 8 * (si & 3);
            float v = row < out ? src_scale(s, row, b) : 0.0f;
            *reinterpret_cast<float*>(dword) = v;
            continue;
        }
        const int slot = (wi & 127) >> 2;    // lane slot
        const int gid = slot >> 2, tig = slot & 3;
        uint32_t word = 0;
        if (BITS == 4) {
            // word 2q + h: low nibbles = row gid + 16q, high nibbles = row gid + 16q + 8,
            // elements 16h + 4tig + j
            const int q = (wi & 3) >> 1, h = wi & 1;
            const int64_t r_lo = g * 32 + gid + 16 * q, r_hi = r_lo + 8;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int e = 16 * h + 4 * tig + j;
                const uint32_t lo = r_lo < out ? src_nibble(s, r_lo, b, e) : 8u;  // zero point:
                const uint32_t hi = r_hi < out ? src_nibble(s, r_hi, b, e) : 8u;  // padding -> 0
                word |= (lo | (hi << 4)) << (8 * j);
            }
        } else {
            const int plane = wi >> 7, i = wi & 3;
            const int64_t row = g * 32 + gid + 8 * i;
            if (row < out) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint32_t v = src_byte(s, row, b, 16 * plane + 4 * tig + j);
                    if (flip_sign) v ^= 0x80u;  // signed code c -> c + 128
                    word |= v << (8 * j);
                }
            } else {
                word = 0x80808080u;
            }
        }
        *dword = word;
    }
}

int32_t launch_repack(rstq_ctx* ctx, DeviceState& ds, const uint8_t* src_codes,
                      const float* src_scales, uint8_t* dst, int fmt, int layout, int64_t out,
                      int64_t in, int64_t src_in, int64_t k_block0) {
    SrcView s{src_codes, src_scales, src_in / 32, k_block0, layout};
    const int64_t nb = in / 32, groups = (out + 31) / 32;
    const int bits = fmt == RSTQ_FMT_Q4_0 ? 4 : 8;
    const int64_t total = groups * nb * (unit_bytes(bits) / 4);
    int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    if (blocks < 1) blocks = 1;
    if (bits == 4)
        repack_kernel<4><<<blocks, 256, 0, ds.stream>>>(s, dst, out, nb, groups, 0);
    else
        repack_kernel<8><<<blocks, 256, 0, ds.stream>>>(s, dst, out, nb, groups,
                                                        fmt == RSTQ_FMT_Q8_S ? 1 : 0);
    ctx->launches++;
    RSTQ_CUDA(cudaGetLastError());
    return RSTQ_OK;
}

// One thread per destination word: 160 words of codes and scales as they are, then the 32 minima.
__global__ void q4k_units_kernel(const uint8_t* __restrict__ src, const float* __restrict__ mins,
                                 uint8_t* __restrict__ dst, int64_t out, int64_t nb, int64_t groups) {
    constexpr int SW = kUnitBytesQ4 / 4, DW = kUnitBytesQ4K / 4;
    const int64_t total = groups * nb * DW;
    for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t unit = idx / DW;
        const int wi = (int)(idx % DW);
        uint32_t v;
        if (wi < SW) {
            v = reinterpret_cast<const uint32_t*>(src + unit * kUnitBytesQ4)[wi];
        } else {
            const int si = wi - SW;
            const int64_t g = unit / nb, b = unit % nb;
            const int64_t row = g * 32 + (si >> 2) + 8 * (si & 3);
            v = __float_as_uint(row < out ? mins[row * nb + b] : 0.0f);
        }
        reinterpret_cast<uint32_t*>(dst + unit * kUnitBytesQ4K)[wi] = v;
    }
}

// 1152-byte 8-bit units (their 32 scales are dropped) + row-major scales per 16 elements
// [out, in/16] -> 1280-byte Q6_K units: one thread per destination word, 256 words of codes as they
// are, then 64 scales: float (gid*4 + i)*2 + h = row gid + 8i of the group, elements 16h .. 16h + 15.
__global__ void q6k_units_kernel(const uint8_t* __restrict__ src, const float* __restrict__ scales16,
                                 uint8_t* __restrict__ dst, int64_t out, int64_t nb, int64_t groups) {
    constexpr int CW = kUnitCodesQ8 / 4, DW = kUnitBytesQ6K / 4;
    const int64_t total = groups * nb * DW;
    for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t unit = idx / DW;
        const int wi = (int)(idx % DW);
        uint32_t v;
        if (wi < CW) {
            v = reinterpret_cast<const uint32_t*>(src + unit * kUnitBytesQ8)[wi];
        } else {
            const int si = wi - CW, h = si & 1, slot = si >> 1;
            const int64_t g = unit / nb, b = unit % nb;
            const int64_t row = g * 32 + (slot >> 2) + 8 * (slot & 3);
            v = __float_as_uint(row < out ? scales16[row * (nb * 2) + b * 2 + h] : 0.0f);
        }
        reinterpret_cast<uint32_t*>(dst + unit * kUnitBytesQ6K)[wi] = v;
    }
}

int32_t launch_q6k_units(rstq_ctx* ctx, DeviceState& ds, const uint8_t* src, const float* scales16, uint8_t* dst,
                         int64_t out, int64_t nb) {
    const int64_t groups = (out + 31) / 32, total = groups * nb * (kUnitBytesQ6K / 4);
    int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    if (blocks < 1) blocks = 1;
    q6k_units_kernel<<<blocks, 256, 0, ds.stream>>>(src, scales16, dst, out, nb, groups);
    ctx->launches++;
    RSTQ_CUDA(cudaGetLastError());
    return RSTQ_OK;
}

int32_t launch_q4k_units(rstq_ctx* ctx, DeviceState& ds, const uint8_t* src, const float* mins, uint8_t* dst,
                         int64_t out, int64_t nb) {
    const int64_t groups = (out + 31) / 32, total = groups * nb * (kUnitBytesQ4K / 4);
    int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    if (blocks < 1) blocks = 1;
    q4k_units_kernel<<<blocks, 256, 0, ds.stream>>>(src, mins, dst, out, nb, groups);
    ctx->launches++;
    RSTQ_CUDA(cudaGetLastError());
    return RSTQ_OK;
}

}  // namespace rstq
