// Q4_K and Q6_K, the reference's super-block formats, on the decode kernel.
//
// Q6_K (symmetric, 16 sub-blocks of 16 with an integer scale each, codes 0..63 with zero point 32;
// qmatmul-q6k-composable!, src/raster/quant/kernels_k.clj:50-79): a 16-element sub-block has no
// place in a 32-element block with one scale, so a row is bound as TWO rows of 8-bit units -- twin A
// keeps the codes of the even sub-blocks and holds the zero point (32) in the odd ones, twin B the
// converse; block scales ds*sc_even and ds*sc_odd.  A zero-point code contributes (32 - 32) * x = 0,
// so each twin's integer dots are exactly dp_j - 32 * bsum_j of its own sub-blocks and
// y[o] = t[2o] + t[2o+1] (pair_sum_kernel).  Twice the code bytes of the reference's layout: a first
// correct path, not the final layout.
//
// Q4_K:
// The reference's Q4_K GEMV (qmatmul-q4k-composable! / qmatmul-q4k-gpu! / qmatmul-q4k-dp4a!,
// src/raster/quant/kernels_k.clj:15-48, :156-186, :195-237) computes, per output row o,
//   y[o] = sum over super-blocks sb of dact[sb] * sum over j < 8 of
//              (da[o,sb] * aq[o,sb*8+j]) * dp_j  +  (db[o,sb] * bq[o,sb*8+j]) * bsum_j
// dp_j = nibble x int8 dot of the 32-element sub-block, bsum_j = sum of its activation codes.
// A sub-block is exactly a 32-element block of the decode kernel with block scale
// a = da*aq, zero point 0 and the activation scale of its super-block, so the first term is the
// streaming kernel unchanged (the weight is bound as 4-bit units with scales a); the second term
// is a small f32 GEMV over the per-sub-block minima  b = db*bq  ([out, in/32] floats, a quarter
// of the code bytes), added to y by q4k_min_kernel.  The q8_K activation quantizer
// (quantize-act-q8k, src/raster/compiler/backend/cpu/quant.clj:172-193; device form
// quant-act-q8k-gpu!, kernels_k.clj:93-134) is one kernel here: a CTA per super-block.
#include "internal.h"

namespace rstq {

__device__ __forceinline__ int kq_round_half_up(double v) {
    const double f = floor(v);
    return (int)f + ((v - f) >= 0.5 ? 1 : 0);
}

// One CTA of 256 threads per (row, super-block); thread t owns element t.
// xs: [rows, nsb] (the reference's array) and / or xs32: [rows, nsb * 8], the super-block scale
// repeated for each of its 32-element blocks (what the decode kernel reads); either may be null.
// bsums: [rows, nsb * 256 / SUB].
template <int SUB>
__global__ void __launch_bounds__(256)
quant_act_q8k_kernel(const float* __restrict__ x, int8_t* __restrict__ xq, float* __restrict__ xs,
                     float* __restrict__ xs32, int32_t* __restrict__ bsums) {
    __shared__ float s_mx[8];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int64_t sb = blockIdx.x;  // row * nsb + super-block
    const float v = x[sb * 256 + t];
    float mx = fabsf(v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) s_mx[warp] = mx;
    __syncthreads();
    mx = s_mx[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) mx = fmaxf(mx, s_mx[i]);
    const double d = (double)mx / 127.0;
    const double id = d == 0.0 ? 0.0 : 1.0 / d;
    int q = kq_round_half_up((double)v * id);
    q = max(-127, min(127, q));
    uint32_t w = (uint32_t)(q & 0xFF) << (8 * (lane & 3));
    w |= __shfl_xor_sync(0xffffffffu, w, 1);
    w |= __shfl_xor_sync(0xffffffffu, w, 2);
    if ((lane & 3) == 0) reinterpret_cast<uint32_t*>(xq)[sb * 64 + (t >> 2)] = w;
    int s = q;
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (SUB == 16) {
        if ((lane & 15) == 0) bsums[sb * 16 + warp * 2 + (lane >> 4)] = s;
    } else {
        s += __shfl_xor_sync(0xffffffffu, s, 16);
        if (lane == 0) bsums[sb * 8 + warp] = s;
    }
    if (xs && t == 0) xs[sb] = (float)d;
    if (xs32 && t < 8) xs32[sb * 8 + t] = (float)d;
}

// xs32[i] = xs[i / 8]: the reference's per-super-block scales laid out per 32-element block
__global__ void __launch_bounds__(256)
expand_scales_kernel(const float* __restrict__ xs, float* __restrict__ xs32, int64_t n32) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n32; i += (int64_t)gridDim.x * blockDim.x)
        xs32[i] = xs[i >> 3];
}

// Q6_K kernel-level call (qmatmul-q6k-dp4a!, src/raster/quant/kernels_k.clj:270-300): the caller holds the
// q8_K activation scale per super-block and the code sums per 16-element sub-block; the twin-row units want
// a scale and a sum per 32-element block: xs32[i] = xs[i / 8], bsum32[i] = bsums16[2 i] + bsums16[2 i + 1].
__global__ void __launch_bounds__(256)
q6k_prep_kernel(const float* __restrict__ xs, const int32_t* __restrict__ bsums16, float* __restrict__ xs32,
                int32_t* __restrict__ bsum32, int64_t n32) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n32; i += (int64_t)gridDim.x * blockDim.x) {
        xs32[i] = xs[i >> 3];
        bsum32[i] = bsums16[2 * i] + bsums16[2 * i + 1];
    }
}

// y[m, o] += sum over b of mins[o, b] * (xs32[m, b] * bsums[m, b]).  The products t[m, b] of up to
// TT tokens are staged in shared memory once per CTA; a warp owns an output row at a time and reads
// it with 16-byte loads (nb % 8 == 0), so mins crosses the memory system once per TT tokens.
// Launched with programmatic serialization: the CTAs are resident while the decode kernel
// finishes and start adding as soon as its results are visible.
constexpr int kMinTok = 8;
__global__ void __launch_bounds__(256)
q4k_min_kernel(const float* __restrict__ mins, const float* __restrict__ xs32, const int32_t* __restrict__ bsums,
               float* __restrict__ y, int64_t M, int64_t nb, int64_t out, int TT) {
    extern __shared__ float s_t[];  // [TT][nb]
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = blockIdx.x * 8ll + (threadIdx.x >> 5), nwarps = gridDim.x * 8ll;
    const int64_t nb4 = nb >> 2;
    for (int64_t m0 = 0; m0 < M; m0 += TT) {
        const int tt = (int)min((int64_t)TT, M - m0);
        if (m0) __syncthreads();
        for (int64_t i = threadIdx.x; i < tt * nb; i += 256) s_t[i] = xs32[m0 * nb + i] * (float)bsums[m0 * nb + i];
        __syncthreads();
        for (int64_t o = warp0; o < out; o += nwarps) {
            const float4* mrow = reinterpret_cast<const float4*>(mins + o * nb);
            float acc[kMinTok];
#pragma unroll
            for (int j = 0; j < kMinTok; ++j) acc[j] = 0.f;
            for (int64_t b = lane; b < nb4; b += 32) {
                const float4 mn = __ldg(mrow + b);
#pragma unroll
                for (int j = 0; j < kMinTok; ++j) {
                    if (j < tt) {
                        const float4 t = *reinterpret_cast<const float4*>(s_t + j * nb + b * 4);
                        acc[j] = fmaf(mn.x, t.x, fmaf(mn.y, t.y, fmaf(mn.z, t.z, fmaf(mn.w, t.w, acc[j]))));
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < kMinTok; ++j) {
                if (j < tt) {
                    float a = acc[j];
#pragma unroll
                    for (int s = 16; s > 0; s >>= 1) a += __shfl_xor_sync(0xffffffffu, a, s);
                    if (lane == 0) y[(m0 + j) * out + o] += a;
                }
            }
        }
    }
}

// y[m, o] = t[m, 2o] + t[m, 2o + 1]: the two twin rows of a Q6_K row (see rstq_weight_bind_q6k)
__global__ void __launch_bounds__(256)
pair_sum_kernel(const float2* __restrict__ t, float* __restrict__ y, int64_t n) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const float2 v = t[i];
        y[i] = v.x + v.y;
    }
}

template <typename K, typename... Args>
static cudaError_t launch_pdl(K kernel, dim3 grid, const DeviceState& ds, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(256);
    cfg.stream = ds.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ds.pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

int32_t launch_quant_act_q8k(rstq_ctx* ctx, DeviceState& ds, const float* x, int8_t* xq, float* xs, float* xs32,
                             int32_t* bsums, int64_t rows, int64_t in, int sub) {
    const int64_t ctas = rows * (in / 256);
    RSTQ_REQUIRE(ctas >= 1 && ctas < (1ll << 31), RSTQ_E_LIMIT, "rows * in / 256 = %lld", (long long)ctas);
    if (sub == 16)
        RSTQ_CUDA(launch_pdl(quant_act_q8k_kernel<16>, dim3((unsigned)ctas), ds, x, xq, xs, xs32, bsums));
    else
        RSTQ_CUDA(launch_pdl(quant_act_q8k_kernel<32>, dim3((unsigned)ctas), ds, x, xq, xs, xs32, bsums));
    ctx->launches++;
    return RSTQ_OK;
}

int32_t launch_expand_scales(rstq_ctx* ctx, DeviceState& ds, const float* xs, float* xs32, int64_t n32) {
    int64_t ctas = (n32 + 255) / 256;
    if (ctas > (int64_t)ds.sm_count * 4) ctas = (int64_t)ds.sm_count * 4;
    RSTQ_CUDA(launch_pdl(expand_scales_kernel, dim3((unsigned)ctas), ds, xs, xs32, n32));
    ctx->launches++;
    return RSTQ_OK;
}

int32_t launch_q6k_prep(rstq_ctx* ctx, DeviceState& ds, const float* xs, const int32_t* bsums16, float* xs32,
                        int32_t* bsum32, int64_t n32) {
    int64_t ctas = (n32 + 255) / 256;
    if (ctas > (int64_t)ds.sm_count * 4) ctas = (int64_t)ds.sm_count * 4;
    RSTQ_CUDA(launch_pdl(q6k_prep_kernel, dim3((unsigned)ctas), ds, xs, bsums16, xs32, bsum32, n32));
    ctx->launches++;
    return RSTQ_OK;
}

int32_t launch_q4k_min(rstq_ctx* ctx, DeviceState& ds, const float* mins, const float* xs32, const int32_t* bsums,
                       float* y, int64_t M, int64_t nb, int64_t out) {
    int64_t TT = 48 * 1024 / (nb * 4);  // tokens whose products fit the default shared-memory window
    RSTQ_REQUIRE(TT >= 1, RSTQ_E_LIMIT, "in = %lld too long for the Q4_K min term", (long long)(nb * 32));
    if (TT > kMinTok) TT = kMinTok;
    if (TT > M) TT = M;
    int64_t ctas = (out + 7) / 8;
    if (ctas > (int64_t)ds.sm_count * 4) ctas = (int64_t)ds.sm_count * 4;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ctas);
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = (size_t)(TT * nb * 4);
    cfg.stream = ds.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ds.pdl ? 1 : 0;
    RSTQ_CUDA(cudaLaunchKernelEx(&cfg, q4k_min_kernel, mins, xs32, bsums, y, M, nb, out, (int)TT));
    ctx->launches++;
    return RSTQ_OK;
}

int32_t launch_pair_sum(rstq_ctx* ctx, DeviceState& ds, const float* t, float* y, int64_t M, int64_t out) {
    const int64_t n = M * out;   // twin rows are neighbours, so token m's pairs start at t + m * 2 * out
    int64_t ctas = (n + 255) / 256;
    if (ctas > (int64_t)ds.sm_count * 8) ctas = (int64_t)ds.sm_count * 8;
    RSTQ_CUDA(launch_pdl(pair_sum_kernel, dim3((unsigned)ctas), ds, reinterpret_cast<const float2*>(t), y, n));
    ctx->launches++;
    return RSTQ_OK;
}

}  // namespace rstq
