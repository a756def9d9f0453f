// The attention steps of the decoder layer's decode chain (one token), f32, so that the chain
// norm -> quantize -> q/k/v matmuls -> rope -> cache append -> attention -> o matmul stays on the
// device and in one CUDA graph:
//   rope      rope-pos-gpu! / rope-pos-buf!            src/raster/dl/attention.clj:386-408, :482-499
//   append    kv-append! / kv-append-buf!              attention.clj:413-416, :501-504
//   attention gqa-decode-attention-gpu! / -buf!        attention.clj:423-471, :514-575
// The position / cache length is a host scalar or, when a one-element int64 device buffer is given,
// read inside the kernel (the reference's -buf variants), so a captured graph serves every token.
//
// Attention is one kernel where the reference has three phases: a CTA owns one KV head and a slice
// of the cache positions and serves every query head of the group from the K / V rows it reads
// once (the reference reads them once per query head); warps walk the positions with an online
// softmax (running max, sum and weighted V in registers), the warps of a CTA are merged through
// shared memory and the slices through a small scratch in device memory, where the last CTA to
// arrive for a KV head writes out = sum_j p_j v_j.  The reference's score scratch `sc` is not used.
#include "internal.h"

namespace rstq {

constexpr int kAttnWarps = 8;
constexpr int kAttnGroup = 8;     // query heads of one KV head served by a CTA
constexpr int kAttnVec = 2;       // float4 per lane along head_dim: head_dim <= 256
constexpr int kAttnCounters = 1024;
constexpr float kNegInf = -1.0e38f;   // the reference's sentinel below any real score

__global__ void __launch_bounds__(256)
rope_pos_kernel(const float* __restrict__ x, float* __restrict__ out, int64_t heads, int64_t head_dim, double ln_theta,
                int64_t pos, const int64_t* __restrict__ posbuf) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int64_t h2 = head_dim >> 1;
    const int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (idx >= heads * h2) return;
    const int64_t h = idx / h2, i = idx - h * h2;
    const double p = (double)(posbuf ? posbuf[0] : pos);
    const double freq = exp((-2.0 * (double)i) / (double)head_dim * ln_theta);
    double s, c;
    sincos(p * freq, &s, &c);
    const double x0 = (double)x[h * head_dim + i], x1 = (double)x[h * head_dim + i + h2];
    out[h * head_dim + i] = (float)(x0 * c - x1 * s);
    out[h * head_dim + i + h2] = (float)(x1 * c + x0 * s);
}

__global__ void __launch_bounds__(256)
kv_append_kernel(const float* __restrict__ src, float* __restrict__ cache, int64_t kvrow, int64_t pos,
                 const int64_t* __restrict__ posbuf) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int64_t p = posbuf ? posbuf[0] : pos;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < kvrow; i += (int64_t)gridDim.x * blockDim.x)
        cache[p * kvrow + i] = src[i];
}

struct AttnParams {
    const float *q, *k, *v;
    float* out;
    float* part;     // [n_kv][gz][S][kAttnGroup][head_dim + 4]: weighted V, running max, sum, 2 pad
    int* counters;   // [n_kv * gz], zero between launches
    const int64_t* clenbuf;
    int64_t cache_len;
    int n_q, group, n_kv, head_dim, S;
    float scale;
};

// merge `n` partial states (max m, sum l, weighted V o[d]) of one query head for one d
__device__ __forceinline__ void attn_merge(const float* base, int n, int stride, int hd, int d, float* o_out,
                                           float* l_out) {
    float M = kNegInf;
    for (int w = 0; w < n; ++w) M = fmaxf(M, __ldcg(base + w * stride + hd));
    float L = 0.f, O = 0.f;
    for (int w = 0; w < n; ++w) {
        const float e = expf(__ldcg(base + w * stride + hd) - M);
        L = fmaf(__ldcg(base + w * stride + hd + 1), e, L);
        O = fmaf(__ldcg(base + w * stride + d), e, O);
    }
    *o_out = O;
    *l_out = L;
}

__global__ void __launch_bounds__(kAttnWarps * 32)
gqa_decode_kernel(const AttnParams p) {
    extern __shared__ __align__(16) float s_part[];   // [kAttnWarps][gc][hd + 4]
    __shared__ int s_last;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int hkv = blockIdx.x, split = blockIdx.y, gz = blockIdx.z;
    const int hd = p.head_dim, hd4 = hd >> 2, row = hd + 4;   // row: weighted V, max, sum, 2 pad (16-byte rows)
    const int g0 = gz * kAttnGroup;
    const int gc = min(kAttnGroup, p.group - g0);            // query heads this CTA serves
    const int64_t clen = p.clenbuf ? p.clenbuf[0] : p.cache_len;
    const int64_t chunk = (clen + p.S - 1) / p.S;
    const int64_t j0 = split * chunk, j1 = min(clen, j0 + chunk);
    const int64_t kvstride = (int64_t)p.n_kv * hd;
    const float4* kb = reinterpret_cast<const float4*>(p.k + (int64_t)hkv * hd);
    const float4* vb = reinterpret_cast<const float4*>(p.v + (int64_t)hkv * hd);

    // this lane's slice of every served query head, pre-multiplied by the score scale
    float4 qv[kAttnGroup][kAttnVec];
    float4 acc[kAttnGroup][kAttnVec];
    float m[kAttnGroup], l[kAttnGroup];
#pragma unroll
    for (int g = 0; g < kAttnGroup; ++g) {
        m[g] = kNegInf;
        l[g] = 0.f;
#pragma unroll
        for (int u = 0; u < kAttnVec; ++u) {
            acc[g][u] = make_float4(0.f, 0.f, 0.f, 0.f);
            const int c = lane + u * 32;
            qv[g][u] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (g < gc && c < hd4) {
                const float4 t = reinterpret_cast<const float4*>(p.q + (int64_t)(hkv * p.group + g0 + g) * hd)[c];
                qv[g][u] = make_float4(t.x * p.scale, t.y * p.scale, t.z * p.scale, t.w * p.scale);
            }
        }
    }
    for (int64_t j = j0 + warp; j < j1; j += kAttnWarps) {
        float4 kk[kAttnVec], vv[kAttnVec];
#pragma unroll
        for (int u = 0; u < kAttnVec; ++u) {
            const int c = lane + u * 32;
            kk[u] = vv[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c < hd4) {
                kk[u] = __ldg(kb + j * (kvstride >> 2) + c);
                vv[u] = __ldg(vb + j * (kvstride >> 2) + c);
            }
        }
#pragma unroll
        for (int g = 0; g < kAttnGroup; ++g) {
            if (g < gc) {
                float s = 0.f;
#pragma unroll
                for (int u = 0; u < kAttnVec; ++u)
                    s = fmaf(qv[g][u].x, kk[u].x, fmaf(qv[g][u].y, kk[u].y, fmaf(qv[g][u].z, kk[u].z, fmaf(qv[g][u].w, kk[u].w, s))));
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                const float mn = fmaxf(m[g], s);
                const float corr = expf(m[g] - mn), pj = expf(s - mn);
                m[g] = mn;
                l[g] = fmaf(l[g], corr, pj);
#pragma unroll
                for (int u = 0; u < kAttnVec; ++u) {
                    acc[g][u].x = fmaf(acc[g][u].x, corr, pj * vv[u].x);
                    acc[g][u].y = fmaf(acc[g][u].y, corr, pj * vv[u].y);
                    acc[g][u].z = fmaf(acc[g][u].z, corr, pj * vv[u].z);
                    acc[g][u].w = fmaf(acc[g][u].w, corr, pj * vv[u].w);
                }
            }
        }
    }
    // warps -> shared memory
#pragma unroll
    for (int g = 0; g < kAttnGroup; ++g) {
        if (g < gc) {
            float* dst = s_part + (warp * gc + g) * row;
#pragma unroll
            for (int u = 0; u < kAttnVec; ++u) {
                const int c = lane + u * 32;
                if (c < hd4) reinterpret_cast<float4*>(dst)[c] = acc[g][u];
            }
            if (lane == 0) {
                dst[hd] = m[g];
                dst[hd + 1] = l[g];
            }
        }
    }
    __syncthreads();
    // CTA state per (g, d): straight to out when there is one slice, else to the scratch
    float* mine = p.part + ((((int64_t)hkv * gridDim.z + gz) * p.S + split) * kAttnGroup) * row;
    for (int i = threadIdx.x; i < gc * row; i += blockDim.x) {
        const int g = i / row, d = i - g * row;
        if (d >= hd + 2) continue;   // padding
        const float* base = s_part + g * row;
        float M = kNegInf;
        for (int w = 0; w < kAttnWarps; ++w) M = fmaxf(M, base[w * gc * row + hd]);
        float val;
        if (d == hd) {
            val = M;
        } else {
            float acc1 = 0.f;
            const int src = d == hd + 1 ? hd + 1 : d;
            for (int w = 0; w < kAttnWarps; ++w)
                acc1 = fmaf(base[w * gc * row + src], expf(base[w * gc * row + hd] - M), acc1);
            val = acc1;
        }
        if (p.S == 1) {
            if (d < hd) {
                float L = 0.f;
                for (int w = 0; w < kAttnWarps; ++w)
                    L = fmaf(base[w * gc * row + hd + 1], expf(base[w * gc * row + hd] - M), L);
                p.out[(int64_t)(hkv * p.group + g0 + g) * hd + d] = val * (1.0f / L);
            }
        } else {
            mine[g * row + d] = val;
        }
    }
    if (p.S == 1) return;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int prev = atomicAdd(p.counters + hkv * gridDim.z + gz, 1);
        s_last = prev == p.S - 1;
        if (s_last) p.counters[hkv * gridDim.z + gz] = 0;   // ready for the next launch / graph replay
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const float* all = p.part + (((int64_t)hkv * gridDim.z + gz) * p.S * kAttnGroup) * row;
    for (int i = threadIdx.x; i < gc * hd; i += blockDim.x) {
        const int g = i / hd, d = i - g * hd;
        float O, L;
        attn_merge(all + g * row, p.S, kAttnGroup * row, hd, d, &O, &L);
        p.out[(int64_t)(hkv * p.group + g0 + g) * hd + d] = O * (1.0f / L);
    }
}

template <typename K, typename... Args>
static cudaError_t launch_attn(K kernel, dim3 grid, dim3 block, size_t smem, const DeviceState& ds, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
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

static bool attn_buf(const rstq_buf* b, const rstq_ctx* ctx, int64_t bytes) {
    return b && b->magic == kBufMagic && b->ctx == ctx && b->bytes >= bytes && ((uintptr_t)b->ptr & 15) == 0;
}

extern "C" {

int32_t rstq_rope_pos(rstq_ctx* ctx, rstq_buf* x, rstq_buf* out, int64_t heads, int64_t head_dim, double theta,
                      int64_t pos, rstq_buf* posbuf) {
    RSTQ_REQUIRE(ctx && ctx->magic == kCtxMagic, RSTQ_E_INVALID, "invalid context handle");
    RSTQ_REQUIRE(heads >= 1 && head_dim >= 2 && head_dim % 2 == 0 && theta > 0.0 && (posbuf || pos >= 0), RSTQ_E_SHAPE,
                 "heads = %lld, head_dim = %lld (even), theta = %g, pos = %lld", (long long)heads,
                 (long long)head_dim, theta, (long long)pos);
    const int64_t n = heads * head_dim;
    RSTQ_REQUIRE(attn_buf(x, ctx, n * 4) && attn_buf(out, ctx, n * 4) && (!posbuf || attn_buf(posbuf, ctx, 8)),
                 RSTQ_E_INVALID, "invalid, unaligned or too small buffer");
    RSTQ_REQUIRE(x->dev == out->dev && (!posbuf || posbuf->dev == x->dev), RSTQ_E_DEVICE,
                 "buffers live on different devices");
    DeviceState& ds = ctx->devs[x->dev];
    int32_t rc = use_dev(ctx, x->dev);
    if (rc != RSTQ_OK) return rc;
    const int64_t items = heads * (head_dim / 2);
    RSTQ_CUDA(launch_attn(rope_pos_kernel, dim3((unsigned)((items + 255) / 256)), dim3(256), 0, ds,
                          (const float*)x->ptr, (float*)out->ptr, heads, head_dim, log(theta), pos,
                          posbuf ? (const int64_t*)posbuf->ptr : (const int64_t*)nullptr));
    ctx->launches++;
    return RSTQ_OK;
}

int32_t rstq_kv_append(rstq_ctx* ctx, rstq_buf* src, rstq_buf* cache, int64_t kvrow, int64_t pos, int64_t maxpos,
                       rstq_buf* posbuf) {
    RSTQ_REQUIRE(ctx && ctx->magic == kCtxMagic, RSTQ_E_INVALID, "invalid context handle");
    RSTQ_REQUIRE(kvrow >= 1 && maxpos >= 1 && (posbuf || (pos >= 0 && pos < maxpos)), RSTQ_E_SHAPE,
                 "kvrow = %lld, pos = %lld of %lld", (long long)kvrow, (long long)pos, (long long)maxpos);
    RSTQ_REQUIRE(attn_buf(src, ctx, kvrow * 4) && attn_buf(cache, ctx, maxpos * kvrow * 4) &&
                     (!posbuf || attn_buf(posbuf, ctx, 8)),
                 RSTQ_E_INVALID, "invalid, unaligned or too small buffer (the cache holds maxpos rows)");
    RSTQ_REQUIRE(src->dev == cache->dev && (!posbuf || posbuf->dev == src->dev), RSTQ_E_DEVICE,
                 "buffers live on different devices");
    DeviceState& ds = ctx->devs[src->dev];
    int32_t rc = use_dev(ctx, src->dev);
    if (rc != RSTQ_OK) return rc;
    int64_t ctas = (kvrow + 255) / 256;
    if (ctas > ds.sm_count * 4) ctas = ds.sm_count * 4;
    RSTQ_CUDA(launch_attn(kv_append_kernel, dim3((unsigned)ctas), dim3(256), 0, ds, (const float*)src->ptr,
                          (float*)cache->ptr, kvrow, pos, posbuf ? (const int64_t*)posbuf->ptr : (const int64_t*)nullptr));
    ctx->launches++;
    return RSTQ_OK;
}

int32_t rstq_gqa_decode_attention(rstq_ctx* ctx, rstq_buf* q, rstq_buf* k, rstq_buf* v, rstq_buf* out,
                                  int64_t cache_len, rstq_buf* clenbuf, int64_t n_q, int64_t group, int64_t n_kv,
                                  int64_t head_dim, int64_t maxpos, double scale) {
    RSTQ_REQUIRE(ctx && ctx->magic == kCtxMagic, RSTQ_E_INVALID, "invalid context handle");
    RSTQ_REQUIRE(n_q >= 1 && group >= 1 && n_kv >= 1 && n_q == group * n_kv, RSTQ_E_SHAPE,
                 "n_q = %lld must be group (%lld) x n_kv (%lld)", (long long)n_q, (long long)group, (long long)n_kv);
    RSTQ_REQUIRE(head_dim >= 4 && head_dim % 4 == 0 && head_dim <= 128 * kAttnVec, RSTQ_E_SHAPE,
                 "head_dim = %lld (a multiple of 4, at most %d)", (long long)head_dim, 128 * kAttnVec);
    RSTQ_REQUIRE(maxpos >= 1 && (clenbuf || (cache_len >= 1 && cache_len <= maxpos)), RSTQ_E_SHAPE,
                 "cache_len = %lld of maxpos = %lld", (long long)cache_len, (long long)maxpos);
    const int64_t kvbytes = maxpos * n_kv * head_dim * 4;
    RSTQ_REQUIRE(attn_buf(q, ctx, n_q * head_dim * 4) && attn_buf(out, ctx, n_q * head_dim * 4) &&
                     attn_buf(k, ctx, kvbytes) && attn_buf(v, ctx, kvbytes) && (!clenbuf || attn_buf(clenbuf, ctx, 8)),
                 RSTQ_E_INVALID, "invalid, unaligned or too small buffer (the caches hold maxpos rows)");
    RSTQ_REQUIRE(q->dev == k->dev && q->dev == v->dev && q->dev == out->dev && (!clenbuf || clenbuf->dev == q->dev),
                 RSTQ_E_DEVICE, "buffers live on different devices");
    DeviceState& ds = ctx->devs[q->dev];
    int32_t rc = use_dev(ctx, q->dev);
    if (rc != RSTQ_OK) return rc;
    const int64_t gz = (group + kAttnGroup - 1) / kAttnGroup;
    RSTQ_REQUIRE(n_kv * gz <= kAttnCounters, RSTQ_E_LIMIT, "n_kv x ceil(group / %d) = %lld exceeds %d", kAttnGroup,
                 (long long)(n_kv * gz), kAttnCounters);
    // slices of the cache: enough CTAs for two per SM, at least 64 positions each; sized from the
    // capacity when the length lives on the device, so that one captured launch serves every length
    const int64_t span = clenbuf ? maxpos : cache_len;
    int64_t S = (2 * (int64_t)ds.sm_count + n_kv * gz - 1) / (n_kv * gz);
    if (S > (span + 63) / 64) S = (span + 63) / 64;
    if (S < 1) S = 1;
    if (S > 65535) S = 65535;
    const int64_t row = head_dim + 4;
    const int64_t part_bytes = n_kv * gz * S * kAttnGroup * row * 4;
    const bool fresh = ds.attn_scratch_bytes < kAttnCounters * 4 + part_bytes;
    rc = dev_reserve(ds, &ds.attn_scratch, &ds.attn_scratch_bytes, kAttnCounters * 4 + part_bytes);
    if (rc != RSTQ_OK) return rc;
    if (fresh) RSTQ_CUDA(cudaMemsetAsync(ds.attn_scratch, 0, kAttnCounters * 4, ds.stream));
    AttnParams p;
    p.q = (const float*)q->ptr;
    p.k = (const float*)k->ptr;
    p.v = (const float*)v->ptr;
    p.out = (float*)out->ptr;
    p.counters = (int*)ds.attn_scratch;
    p.part = (float*)((char*)ds.attn_scratch + kAttnCounters * 4);
    p.clenbuf = clenbuf ? (const int64_t*)clenbuf->ptr : nullptr;
    p.cache_len = cache_len;
    p.n_q = (int)n_q;
    p.group = (int)group;
    p.n_kv = (int)n_kv;
    p.head_dim = (int)head_dim;
    p.S = (int)S;
    p.scale = (float)scale;
    const int64_t gc = group < kAttnGroup ? group : kAttnGroup;
    const size_t smem = (size_t)(kAttnWarps * gc * row * 4);
    if (smem > 48 * 1024)
        RSTQ_CUDA(cudaFuncSetAttribute(gqa_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    RSTQ_CUDA(launch_attn(gqa_decode_kernel, dim3((unsigned)n_kv, (unsigned)S, (unsigned)gz), dim3(kAttnWarps * 32), smem,
                          ds, p));
    ctx->launches++;
    return RSTQ_OK;
}

}  // extern "C"
