// The f32 element-wise / row-wise neighbours of the quantized matmul in a decoder layer's decode
// chain (rms-norm -> quantize -> matmul -> SwiGLU / GeGLU -> residual), so that the chain can stay
// on the device and in one CUDA graph:
//   rms_norm      y_i = x_i / sqrt(mean_j x_j^2 + eps) * (gain_offset + w_i)   src/raster/dl/nn.clj:497-513
//   silu_mul      out = g * sigmoid(g) * up                                     src/raster/dl/nn.clj:200-203
//   gelu_mul      out = 0.5 g (1 + tanh(0.7978845608028654 (g + 0.044715 g^3))) * up      nn.clj:208-214
//   residual_add  out = a + b                                                   src/raster/dl/nn.clj:217-219
// and the fusion the chain invites: rms-norm whose output is quantized to int8 blocks in the same
// kernel (the normalized row never goes to memory; codes, scales and block sums are exactly what
// quant_act_i8_kernel would produce from rms_norm's f32 output).
#include "internal.h"

namespace rstq {

constexpr int kRowThreads = 1024;

__device__ __forceinline__ int chain_round_half_up(double v) {
    const double f = floor(v);
    return (int)f + ((v - f) >= 0.5 ? 1 : 0);
}

// sum over the CTA; every thread gets the result
__device__ __forceinline__ float cta_sum(float v, float* s_red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < kRowThreads / 32; ++i) t += s_red[i];
    __syncthreads();
    return t;
}

// One CTA per row.  QUANT = false: out f32.  QUANT = true: int8 codes + per-32-block scale and sum
// (features % 32 == 0; each warp owns whole blocks so the block reductions are warp shuffles).
// RES: the row normalized is x + res (residual-add! feeding rms-norm!); the sum is stored to
// `sum` first (the residual stream the layer carries on).
// 1024 threads per row and the row kept in registers (up to kRowKeep elements per thread = 8192
// features; longer rows read the rest back): a decode step has ONE row, so the kernel's time is its
// dependent chain -- loads, a block reduction, the double-precision quantizer -- and not its bytes.
// With 256 threads and two passes over memory it took 15 us per launch on a 4096-feature row, a third
// of a whole decoder layer.
constexpr int kRowKeep = 8;

__device__ __forceinline__ void quant_block_store(float v, int lane, int64_t blk, int8_t* __restrict__ xq,
                                                  float* __restrict__ xs, int32_t* __restrict__ xsum) {
    float mx = fabsf(v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    const double d = (double)mx / 127.0;
    const double id = d == 0.0 ? 0.0 : 1.0 / d;
    int q = chain_round_half_up((double)v * id);
    q = max(-127, min(127, q));
    int s = q;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    uint32_t word = (uint32_t)(q & 0xFF) << (8 * (lane & 3));
    word |= __shfl_xor_sync(0xffffffffu, word, 1);
    word |= __shfl_xor_sync(0xffffffffu, word, 2);
    if ((lane & 3) == 0) reinterpret_cast<uint32_t*>(xq)[blk * 8 + (lane >> 2)] = word;
    if (lane == 0) {
        xs[blk] = (float)d;
        if (xsum) xsum[blk] = s;
    }
}

template <bool QUANT, bool RES = false>
__global__ void __launch_bounds__(kRowThreads)
rms_norm_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ out,
                int8_t* __restrict__ xq, float* __restrict__ xs, int32_t* __restrict__ xsum, int64_t features,
                float eps, float gain_offset, const float* __restrict__ res = nullptr, float* sum = nullptr) {
    __shared__ float s_red[kRowThreads / 32];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int64_t r = blockIdx.x;
    const float* xr = RES ? sum + r * features : x + r * features;   // where the row is read back from
    float keep[kRowKeep], gain[kRowKeep];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < kRowKeep; ++k) {
        const int64_t i = threadIdx.x + (int64_t)k * kRowThreads;
        float v = 0.f;
        if (i < features) {
            if (RES) {
                v = x[r * features + i] + res[r * features + i];
                sum[r * features + i] = v;
            } else {
                v = xr[i];
            }
        }
        keep[k] = v;
        gain[k] = i < features ? gain_offset + w[i] : 0.f;   // fetched now: its latency hides under the reduction
        ss = fmaf(v, v, ss);
    }
    for (int64_t i = threadIdx.x + (int64_t)kRowKeep * kRowThreads; i < features; i += kRowThreads) {
        float v;
        if (RES) {
            v = x[r * features + i] + res[r * features + i];
            sum[r * features + i] = v;   // read back below by this same thread
        } else {
            v = xr[i];
        }
        ss = fmaf(v, v, ss);
    }
    const float ms = cta_sum(ss, s_red) / (float)features;
    const float inv = 1.0f / sqrtf(ms + eps);
    const int lane = threadIdx.x & 31;
    const int64_t nb = features >> 5;
    // element i = threadIdx.x + k * 1024: a warp holds the 32 elements of block i / 32 (features % 32 == 0
    // when QUANT), so the block reductions are warp shuffles and a whole warp is in or out of range
#pragma unroll
    for (int k = 0; k < kRowKeep; ++k) {
        const int64_t i = threadIdx.x + (int64_t)k * kRowThreads;
        if (i < features) {
            const float v = keep[k] * inv * gain[k];
            if (QUANT) quant_block_store(v, lane, r * nb + (i >> 5), xq, xs, xsum);
            else out[r * features + i] = v;
        }
    }
    for (int64_t i = threadIdx.x + (int64_t)kRowKeep * kRowThreads; i < features; i += kRowThreads) {
        const float v = xr[i] * inv * (gain_offset + w[i]);
        if (QUANT) quant_block_store(v, lane, r * nb + (i >> 5), xq, xs, xsum);
        else out[r * features + i] = v;
    }
}

template <int OP>  // 0 silu_mul, 1 gelu_mul, 2 residual_add
__global__ void __launch_bounds__(256)
map_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out, int64_t n) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const float g = a[i], u = b[i];
        float v;
        if (OP == 0) v = g * (1.0f / (1.0f + expf(-g))) * u;
        else if (OP == 1) v = 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g))) * u;
        else v = g + u;
        out[i] = v;
    }
}

// silu-mul! / gelu-mul! whose result is quantized to int8 blocks in the same kernel (the input of
// the down projection): one warp per 32-element block, codes / scales / sums exactly those of
// quant_act_i8_kernel run on map_kernel's f32 output, which never goes to memory.
template <int OP>
__global__ void __launch_bounds__(256)
gated_quant_kernel(const float* __restrict__ gate, const float* __restrict__ up, int8_t* __restrict__ xq,
                   float* __restrict__ xs, int32_t* __restrict__ xsum, int64_t nblocks) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int lane = threadIdx.x & 31;
    const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t blk = warp; blk < nblocks; blk += nwarps) {
        const float g = gate[blk * 32 + lane], u = up[blk * 32 + lane];
        float v;
        if (OP == 0) v = g * (1.0f / (1.0f + expf(-g))) * u;
        else v = 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g))) * u;
        float mx = fabsf(v);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        const double d = (double)mx / 127.0;
        const double id = d == 0.0 ? 0.0 : 1.0 / d;
        int q = chain_round_half_up((double)v * id);
        q = max(-127, min(127, q));
        int sm = q;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sm += __shfl_xor_sync(0xffffffffu, sm, o);
        uint32_t word = (uint32_t)(q & 0xFF) << (8 * (lane & 3));
        word |= __shfl_xor_sync(0xffffffffu, word, 1);
        word |= __shfl_xor_sync(0xffffffffu, word, 2);
        if ((lane & 3) == 0) reinterpret_cast<uint32_t*>(xq)[blk * 8 + (lane >> 2)] = word;
        if (lane == 0) {
            xs[blk] = (float)d;
            if (xsum) xsum[blk] = sm;
        }
    }
}

template <typename K, typename... Args>
static cudaError_t launch_chain(K kernel, dim3 grid, dim3 block, const DeviceState& ds, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.stream = ds.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ds.pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

}  // namespace rstq

using namespace rstq;

static bool chain_buf(const rstq_buf* b, const rstq_ctx* ctx, int64_t bytes) {
    return b && b->magic == kBufMagic && b->ctx == ctx && b->bytes >= bytes;
}

extern "C" {

int32_t rstq_rms_norm(rstq_ctx* ctx, rstq_buf* x, rstq_buf* weight, rstq_buf* out, int64_t rows, int64_t features,
                      double eps, double gain_offset) {
    RSTQ_REQUIRE(ctx && ctx->magic == kCtxMagic, RSTQ_E_INVALID, "invalid context handle");
    RSTQ_REQUIRE(rows >= 1 && features >= 1 && rows < (1ll << 31), RSTQ_E_SHAPE, "rows = %lld, features = %lld",
                 (long long)rows, (long long)features);
    RSTQ_REQUIRE(chain_buf(x, ctx, rows * features * 4) && chain_buf(weight, ctx, features * 4) &&
                     chain_buf(out, ctx, rows * features * 4),
                 RSTQ_E_INVALID, "invalid or too small buffer");
    RSTQ_REQUIRE(x->dev == weight->dev && x->dev == out->dev, RSTQ_E_DEVICE, "buffers live on different devices");
    DeviceState& ds = ctx->devs[x->dev];
    int32_t rc = use_dev(ctx, x->dev);
    if (rc != RSTQ_OK) return rc;
    RSTQ_CUDA(launch_chain(rms_norm_kernel<false>, dim3((unsigned)rows), dim3(kRowThreads), ds, (const float*)x->ptr,
                           (const float*)weight->ptr, (float*)out->ptr, (int8_t*)nullptr, (float*)nullptr,
                           (int32_t*)nullptr, features, (float)eps, (float)gain_offset, (const float*)nullptr,
                           (float*)nullptr));
    ctx->launches++;
    return RSTQ_OK;
}

int32_t rstq_rms_norm_quant_act(rstq_ctx* ctx, rstq_buf* x, rstq_buf* weight, rstq_buf* xq, rstq_buf* xs,
                                rstq_buf* xsum, int64_t rows, int64_t features, double eps, double gain_offset) {
    RSTQ_REQUIRE(ctx && ctx->magic == kCtxMagic, RSTQ_E_INVALID, "invalid context handle");
    RSTQ_REQUIRE(rows >= 1 && features >= 32 && features % 32 == 0 && rows < (1ll << 31), RSTQ_E_SHAPE,
                 "features = %lld must be a positive multiple of 32 (rows = %lld)", (long long)features,
                 (long long)rows);
    const int64_t nb = features / 32;
    RSTQ_REQUIRE(chain_buf(x, ctx, rows * features * 4) && chain_buf(weight, ctx, features * 4) &&
                     chain_buf(xq, ctx, rows * features) && chain_buf(xs, ctx, rows * nb * 4) &&
                     (!xsum || chain_buf(xsum, ctx, rows * nb * 4)),
                 RSTQ_E_INVALID, "invalid or too small buffer");
    RSTQ_REQUIRE(x->dev == weight->dev && x->dev == xq->dev && x->dev == xs->dev && (!xsum || x->dev == xsum->dev),
                 RSTQ_E_DEVICE, "buffers live on different devices");
    DeviceState& ds = ctx->devs[x->dev];
    int32_t rc = use_dev(ctx, x->dev);
    if (rc != RSTQ_OK) return rc;
    RSTQ_CUDA(launch_chain(rms_norm_kernel<true>, dim3((unsigned)rows), dim3(kRowThreads), ds, (const float*)x->ptr,
                           (const float*)weight->ptr, (float*)nullptr, (int8_t*)xq->ptr, (float*)xs->ptr,
                           xsum ? (int32_t*)xsum->ptr : (int32_t*)nullptr, features, (float)eps, (float)gain_offset,
                           (const float*)nullptr, (float*)nullptr));
    ctx->launches++;
    return RSTQ_OK;
}

static int32_t chain_map(rstq_ctx* ctx, rstq_buf* a, rstq_buf* b, rstq_buf* out, int64_t n, int op) {
    RSTQ_REQUIRE(ctx && ctx->magic == kCtxMagic, RSTQ_E_INVALID, "invalid context handle");
    RSTQ_REQUIRE(n >= 1, RSTQ_E_SHAPE, "n = %lld", (long long)n);
    RSTQ_REQUIRE(chain_buf(a, ctx, n * 4) && chain_buf(b, ctx, n * 4) && chain_buf(out, ctx, n * 4), RSTQ_E_INVALID,
                 "invalid or too small buffer");
    RSTQ_REQUIRE(a->dev == b->dev && a->dev == out->dev, RSTQ_E_DEVICE, "buffers live on different devices");
    DeviceState& ds = ctx->devs[a->dev];
    int32_t rc = use_dev(ctx, a->dev);
    if (rc != RSTQ_OK) return rc;
    int64_t ctas = (n + 255) / 256;
    if (ctas > (int64_t)ds.sm_count * 8) ctas = (int64_t)ds.sm_count * 8;
    const float* pa = (const float*)a->ptr;
    const float* pb = (const float*)b->ptr;
    float* po = (float*)out->ptr;
    cudaError_t e;
    if (op == 0) e = launch_chain(map_kernel<0>, dim3((unsigned)ctas), dim3(256), ds, pa, pb, po, n);
    else if (op == 1) e = launch_chain(map_kernel<1>, dim3((unsigned)ctas), dim3(256), ds, pa, pb, po, n);
    else e = launch_chain(map_kernel<2>, dim3((unsigned)ctas), dim3(256), ds, pa, pb, po, n);
    RSTQ_CUDA(e);
    ctx->launches++;
    return RSTQ_OK;
}

int32_t rstq_silu_mul(rstq_ctx* ctx, rstq_buf* gate, rstq_buf* up, rstq_buf* out, int64_t n) {
    return chain_map(ctx, gate, up, out, n, 0);
}
int32_t rstq_gelu_mul(rstq_ctx* ctx, rstq_buf* gate, rstq_buf* up, rstq_buf* out, int64_t n) {
    return chain_map(ctx, gate, up, out, n, 1);
}
int32_t rstq_residual_add(rstq_ctx* ctx, rstq_buf* a, rstq_buf* b, rstq_buf* out, int64_t n) {
    return chain_map(ctx, a, b, out, n, 2);
}

int32_t rstq_residual_rms_norm_quant_act(rstq_ctx* ctx, rstq_buf* a, rstq_buf* b, rstq_buf* sum, rstq_buf* weight,
                                         rstq_buf* xq, rstq_buf* xs, rstq_buf* xsum, int64_t rows, int64_t features,
                                         double eps, double gain_offset) {
    RSTQ_REQUIRE(ctx && ctx->magic == kCtxMagic, RSTQ_E_INVALID, "invalid context handle");
    RSTQ_REQUIRE(rows >= 1 && features >= 32 && features % 32 == 0 && rows < (1ll << 31), RSTQ_E_SHAPE,
                 "features = %lld must be a positive multiple of 32 (rows = %lld)", (long long)features,
                 (long long)rows);
    const int64_t nb = features / 32;
    RSTQ_REQUIRE(chain_buf(a, ctx, rows * features * 4) && chain_buf(b, ctx, rows * features * 4) &&
                     chain_buf(sum, ctx, rows * features * 4) && chain_buf(weight, ctx, features * 4) &&
                     chain_buf(xq, ctx, rows * features) && chain_buf(xs, ctx, rows * nb * 4) &&
                     (!xsum || chain_buf(xsum, ctx, rows * nb * 4)),
                 RSTQ_E_INVALID, "invalid or too small buffer");
    RSTQ_REQUIRE(sum->ptr != a->ptr && sum->ptr != b->ptr, RSTQ_E_INVALID, "sum may not alias an input");
    RSTQ_REQUIRE(a->dev == b->dev && a->dev == sum->dev && a->dev == weight->dev && a->dev == xq->dev &&
                     a->dev == xs->dev && (!xsum || a->dev == xsum->dev),
                 RSTQ_E_DEVICE, "buffers live on different devices");
    DeviceState& ds = ctx->devs[a->dev];
    int32_t rc = use_dev(ctx, a->dev);
    if (rc != RSTQ_OK) return rc;
    RSTQ_CUDA(launch_chain(rms_norm_kernel<true, true>, dim3((unsigned)rows), dim3(kRowThreads), ds,
                           (const float*)a->ptr, (const float*)weight->ptr, (float*)nullptr, (int8_t*)xq->ptr,
                           (float*)xs->ptr, xsum ? (int32_t*)xsum->ptr : (int32_t*)nullptr, features, (float)eps,
                           (float)gain_offset, (const float*)b->ptr, (float*)sum->ptr));
    ctx->launches++;
    return RSTQ_OK;
}

static int32_t gated_quant(rstq_ctx* ctx, rstq_buf* gate, rstq_buf* up, rstq_buf* xq, rstq_buf* xs, rstq_buf* xsum,
                           int64_t n, int op) {
    RSTQ_REQUIRE(ctx && ctx->magic == kCtxMagic, RSTQ_E_INVALID, "invalid context handle");
    RSTQ_REQUIRE(n >= 32 && n % 32 == 0, RSTQ_E_SHAPE, "n = %lld must be a positive multiple of 32", (long long)n);
    RSTQ_REQUIRE(chain_buf(gate, ctx, n * 4) && chain_buf(up, ctx, n * 4) && chain_buf(xq, ctx, n) &&
                     chain_buf(xs, ctx, n / 32 * 4) && (!xsum || chain_buf(xsum, ctx, n / 32 * 4)),
                 RSTQ_E_INVALID, "invalid or too small buffer");
    RSTQ_REQUIRE(gate->dev == up->dev && gate->dev == xq->dev && gate->dev == xs->dev && (!xsum || gate->dev == xsum->dev),
                 RSTQ_E_DEVICE, "buffers live on different devices");
    DeviceState& ds = ctx->devs[gate->dev];
    int32_t rc = use_dev(ctx, gate->dev);
    if (rc != RSTQ_OK) return rc;
    const int64_t nblocks = n / 32;
    int64_t ctas = (nblocks + 7) / 8;
    if (ctas > (int64_t)ds.sm_count * 8) ctas = (int64_t)ds.sm_count * 8;
    int32_t* ps = xsum ? (int32_t*)xsum->ptr : (int32_t*)nullptr;
    cudaError_t e;
    if (op == 0)
        e = launch_chain(gated_quant_kernel<0>, dim3((unsigned)ctas), dim3(256), ds, (const float*)gate->ptr,
                         (const float*)up->ptr, (int8_t*)xq->ptr, (float*)xs->ptr, ps, nblocks);
    else
        e = launch_chain(gated_quant_kernel<1>, dim3((unsigned)ctas), dim3(256), ds, (const float*)gate->ptr,
                         (const float*)up->ptr, (int8_t*)xq->ptr, (float*)xs->ptr, ps, nblocks);
    RSTQ_CUDA(e);
    ctx->launches++;
    return RSTQ_OK;
}

int32_t rstq_silu_mul_quant_act(rstq_ctx* ctx, rstq_buf* gate, rstq_buf* up, rstq_buf* xq, rstq_buf* xs,
                                rstq_buf* xsum, int64_t n) {
    return gated_quant(ctx, gate, up, xq, xs, xsum, n, 0);
}
int32_t rstq_gelu_mul_quant_act(rstq_ctx* ctx, rstq_buf* gate, rstq_buf* up, rstq_buf* xq, rstq_buf* xs,
                                rstq_buf* xsum, int64_t n) {
    return gated_quant(ctx, gate, up, xq, xs, xsum, n, 1);
}

}  // extern "C"
