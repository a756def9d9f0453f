// Per-32-block int8 activation quantizer on the device.
//
// Arithmetic of quantize-act-blocks! / quantize-act-i8
// (src/raster/compiler/backend/cpu/quant.clj:282-305) and, without the block
// sums, of quant-act-i8-rows-gpu! (src/raster/quant/kernels_k.clj:309-342):
//   mx = max|x| over the block, d = mx / 127 (double), id = d == 0 ? 0 : 1 / d,
//   q = clamp(round_half_up((double)x * id), -127, 127), xs = (float)d, xsum = sum q.
// The scale and the rounding are carried in double so the codes are bit-exact
// with the JVM's (Java Math.round = nearest, ties toward +infinity).
#include "internal.h"

namespace rstq {

__device__ __forceinline__ int round_half_up(double v) {
    double f = floor(v);
    return (int)f + ((v - f) >= 0.5 ? 1 : 0);
}

// One warp per block; lane k owns element k.  Bytes are gathered so that each
// of eight lanes stores one 32-bit word.
// BF16IN: x holds bf16 bit patterns (uint16_t); they are widened exactly, so the codes are those
// the f32 quantizer gives for the widened values.
template <bool BF16IN>
__global__ void __launch_bounds__(256)
quant_act_i8_kernel(const void* __restrict__ xv, int8_t* __restrict__ xq, float* __restrict__ xs,
                    int32_t* __restrict__ xsum, int64_t nblocks, uint8_t* __restrict__ img, int M, int nb, int zp,
                    int four_bit) {
    // programmatic dependent launch: let the consumer kernel start its weight stream now;
    // x may come from the kernel before this one, so wait for it
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int lane = threadIdx.x & 31;
    const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t blk = warp; blk < nblocks; blk += nwarps) {
        const float v = BF16IN ? __uint_as_float((uint32_t)reinterpret_cast<const uint16_t*>(xv)[blk * 32 + lane] << 16)
                               : reinterpret_cast<const float*>(xv)[blk * 32 + lane];
        float mx = fabsf(v);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        const double d = (double)mx / 127.0;
        const double id = d == 0.0 ? 0.0 : 1.0 / d;
        int q = round_half_up((double)v * id);
        q = max(-127, min(127, q));
        int s = q;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        // pack four neighbouring codes into the word lane (lane & ~3) stores
        uint32_t b = (uint32_t)(q & 0xFF);
        uint32_t w = b << (8 * (lane & 3));
        w |= __shfl_xor_sync(0xffffffffu, w, 1);
        w |= __shfl_xor_sync(0xffffffffu, w, 2);
        if ((lane & 3) == 0) reinterpret_cast<uint32_t*>(xq)[blk * 8 + (lane >> 2)] = w;
        if (lane == 0) {
            xs[blk] = (float)d;
            if (xsum) xsum[blk] = s;
        }
        if (img) {
            // The decode kernel's staged form of the same data, for M > 1 (block-major, the eight
            // code words of a (block, token) as four (word tg, word 4 + tg) pairs; then the records of
            // put_act_record), so that it can take it with a bulk copy.
            // More than kGemvMaxM tokens: one image per decode launch of kGemvMaxM tokens, act_image_stride apart.
            const int ct = (int)(blk / nb), b = (int)(blk - (int64_t)ct * nb);   // token, block
            const int piece = ct / kGemvMaxM, c = ct - piece * kGemvMaxM;        // token inside its launch
            const int Mp = min(kGemvMaxM, M - piece * kGemvMaxM);                // tokens of that launch
            uint8_t* im = img + piece * act_image_stride(nb);
            const int j = lane >> 2;                                            // word held by lanes 0, 4, .. 28
            if ((lane & 3) == 0)
                reinterpret_cast<uint32_t*>(im)[((int64_t)(b * Mp + c) * 4 + (j & 3)) * 2 + (j >> 2)] = w;
            const int Mz = (Mp + 1) & ~1;
            uint8_t* recs = im + (((int64_t)nb * Mp * 32 + 127) & ~127ll);
            if (lane == 0) put_act_record(recs, b, Mz, c, (float)d, zp * s, four_bit);
            if (lane == 1 && c == Mp - 1 && Mz > Mp) put_act_record(recs, b, Mz, Mp, 0.f, 0, four_bit);
        }
    }
}

// The same image from activations that arrive quantized (rstq_qmatmul_prequant): codes [M][in], scales and
// code sums [M][nb].  Eight lanes per (token, block), one code word each.
__global__ void __launch_bounds__(256)
act_image_kernel(const int8_t* __restrict__ xq, const float* __restrict__ xs, const int32_t* __restrict__ xsum,
                 int64_t nblocks, uint8_t* __restrict__ img, int M, int nb, int zp, int four_bit, int uk) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int Mz = (M + 1) & ~1;
    uint8_t* recs = img + (((int64_t)nb * M * 32 + 127) & ~127ll);
    // K-quant units keep their own records: Q4_K (uk 1) {xs, xs * code sum} per (block, token), Q6_K (uk 2)
    // {xs, zp * sum of elements 0..15, zp * sum of 16..31, 0} with the sums per 16 elements in xsum
    int2* z2 = reinterpret_cast<int2*>(recs);
    int4* z4 = reinterpret_cast<int4*>(recs);
    const int64_t n = nblocks * 8, step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += step) {
        const int64_t blk = i >> 3;
        const int j = (int)(i & 7);
        const int c = (int)(blk / nb), b = (int)(blk - (int64_t)c * nb);
        reinterpret_cast<uint32_t*>(img)[((int64_t)(b * M + c) * 4 + (j & 3)) * 2 + (j >> 2)] =
            reinterpret_cast<const uint32_t*>(xq)[i];
        if (uk == 1) {
            if (j == 0) z2[(int64_t)b * Mz + c] = make_int2(__float_as_int(xs[blk]), __float_as_int(xs[blk] * (float)xsum[blk]));
            if (j == 1 && c == M - 1 && Mz > M) z2[(int64_t)b * Mz + M] = make_int2(0, 0);
        } else if (uk == 2) {
            if (j == 0) z4[(int64_t)b * Mz + c] = make_int4(__float_as_int(xs[blk]), zp * xsum[2 * blk], zp * xsum[2 * blk + 1], 0);
            if (j == 1 && c == M - 1 && Mz > M) z4[(int64_t)b * Mz + M] = make_int4(0, 0, 0, 0);
        } else {
            if (j == 0) put_act_record(recs, b, Mz, c, xs[blk], zp * xsum[blk], four_bit);
            if (j == 1 && c == M - 1 && Mz > M) put_act_record(recs, b, Mz, M, 0.f, 0, four_bit);
        }
    }
}

int32_t launch_act_image(rstq_ctx* ctx, DeviceState& ds, const int8_t* xq, const float* xs, const int32_t* xsum,
                         int64_t M, int64_t in, uint8_t* img, int zp, int bits, int uk) {
    const int64_t nblocks = M * (in / 32);
    int64_t ctas = (nblocks * 8 + 255) / 256;
    const int64_t cap = (int64_t)ds.sm_count * 8;
    if (ctas > cap) ctas = cap;
    if (ctas < 1) ctas = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ctas);
    cfg.blockDim = dim3(256);
    cfg.stream = ds.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ds.pdl ? 1 : 0;
    RSTQ_CUDA(cudaLaunchKernelEx(&cfg, act_image_kernel, xq, xs, xsum, nblocks, img, (int)M, (int)(in / 32), zp,
                                 (int)(bits == 4), uk));
    ctx->launches++;
    RSTQ_CUDA(cudaGetLastError());
    return RSTQ_OK;
}

int32_t launch_quant_act_i8(rstq_ctx* ctx, DeviceState& ds, const void* x, int8_t* xq, float* xs,
                            int32_t* xsum, int64_t M, int64_t in, int act_dtype, uint8_t* img, int zp, int bits) {
    const int64_t nblocks = M * (in / 32);
    int64_t ctas = (nblocks + 7) / 8;  // 8 warps per CTA
    const int64_t cap = (int64_t)ds.sm_count * 8;
    if (ctas > cap) ctas = cap;
    if (ctas < 1) ctas = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ctas);
    cfg.blockDim = dim3(256);
    cfg.stream = ds.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ds.pdl ? 1 : 0;
    if (act_dtype == RSTQ_BF16)
        RSTQ_CUDA(cudaLaunchKernelEx(&cfg, quant_act_i8_kernel<true>, x, xq, xs, xsum, nblocks, img, (int)M,
                                     (int)(in / 32), zp, (int)(bits == 4)));
    else
        RSTQ_CUDA(cudaLaunchKernelEx(&cfg, quant_act_i8_kernel<false>, x, xq, xs, xsum, nblocks, img, (int)M,
                                     (int)(in / 32), zp, (int)(bits == 4)));
    ctx->launches++;
    RSTQ_CUDA(cudaGetLastError());
    return RSTQ_OK;
}

}  // namespace rstq
