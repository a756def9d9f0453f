// The attention steps of the decoder layer's decode chain (one token), f32, so that the chain
// norm -> quantize -> q/k/v matmuls -> rope -> cache append -> attention -> o matmul stays on the
// device and in one CUDA graph:
//   rope      rope-pos-gpu! / rope-pos-buf!            src/raster/dl/attention.clj:386-408, :482-499
//   append    kv-append! / kv-append-buf!              attention.clj:413-416, :501-504
//   attention gqa-decode-attention-gpu! / -buf!        attention.clj:423-471, :514-575
// The position / cache length is a host scalar or, when a one-element int64 device buffer is given,
// read inside the kernel (the reference's -buf variants), so a captured graph serves every token.
//
// Attention is one kernel where the reference has three phases: a CTA owns one KV head, a slice of
// the cache positions and up to two query heads of the group (eight in the general kernel), which
// it serves from the K / V rows it reads once; the group's other heads find the rows in L2 (the
// reference reads them once per query head); warps walk the positions with an online
// softmax (running max, sum and weighted V in registers), the warps of a CTA are merged through
// shared memory and the slices through a small scratch in device memory, where the last CTA to
// arrive for a KV head writes out = sum_j p_j v_j.  The reference's score scratch `sc` is not used.
// head_dim 64 and 128 take gqa_decode_fast_kernel (eight lanes per position, four positions per
// warp step); every other head_dim % 4 == 0 up to 256 takes the general gqa_decode_kernel (a
// warp per position).
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

// rope(q), rope(k), append k, append v of one token in ONE launch (four steps of the reference's
// chain): q is turned in place; k is turned, stored back and written to its cache row; v is copied
// to its cache row.  One thread per rotation pair of q and k, and per pair of v elements.
__global__ void __launch_bounds__(256)
rope_append_kernel(float* __restrict__ q, float* __restrict__ k, const float* __restrict__ v,
                   float* __restrict__ kcache, float* __restrict__ vcache, int64_t n_q, int64_t n_kv, int64_t head_dim,
                   double ln_theta, int64_t pos, const int64_t* __restrict__ posbuf) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int64_t h2 = head_dim >> 1, kvrow = n_kv * head_dim;
    const int64_t nrot = (n_q + n_kv) * h2, idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    const int64_t p = posbuf ? posbuf[0] : pos;
    if (idx < nrot) {
        const int64_t h = idx / h2, i = idx - h * h2;
        const bool isk = h >= n_q;
        float* x = isk ? k + (h - n_q) * head_dim : q + h * head_dim;
        const double freq = exp((-2.0 * (double)i) / (double)head_dim * ln_theta);
        double s, c;
        sincos((double)p * freq, &s, &c);
        const double x0 = (double)x[i], x1 = (double)x[i + h2];
        const float y0 = (float)(x0 * c - x1 * s), y1 = (float)(x1 * c + x0 * s);
        x[i] = y0;
        x[i + h2] = y1;
        if (isk) {
            float* dst = kcache + p * kvrow + (h - n_q) * head_dim;
            dst[i] = y0;
            dst[i + h2] = y1;
        }
    } else if (idx < nrot + n_kv * h2) {
        const int64_t e = (idx - nrot) * 2;
        *reinterpret_cast<float2*>(vcache + p * kvrow + e) = *reinterpret_cast<const float2*>(v + e);
    }
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
    // optional: the output quantized to int8 blocks of 32 as well (the o projection's input), by the
    // CTA that writes it; only with head_dim % 32 == 0 (a warp then owns whole blocks)
    int8_t* xq;
    float* xs;
    int32_t* xsum;
};

__device__ __forceinline__ int attn_round_half_up(double v) {
    const double f = floor(v);
    return (int)f + ((v - f) >= 0.5 ? 1 : 0);
}

// Second half of both attention kernels: the per-warp states in shared memory ([warps][gc][row]:
// weighted V, max, sum) are merged per CTA, then per KV head across the slices of the cache.
// GS = query heads per CTA (the stride of the scratch).
// one value of the output, and with it -- when asked for -- its 32-element quantizer block (the 32
// lanes of the warp hold 32 consecutive elements of one head)
__device__ __forceinline__ void attn_store(const AttnParams& p, int64_t e, float v, int lane) {
    p.out[e] = v;
    if (p.xq) {
        float mx = fabsf(v);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        const double dq = (double)mx / 127.0;
        const double id = dq == 0.0 ? 0.0 : 1.0 / dq;
        int q = attn_round_half_up((double)v * id);
        q = max(-127, min(127, q));
        int sm = q;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sm += __shfl_xor_sync(0xffffffffu, sm, o);
        uint32_t word = (uint32_t)(q & 0xFF) << (8 * (lane & 3));
        word |= __shfl_xor_sync(0xffffffffu, word, 1);
        word |= __shfl_xor_sync(0xffffffffu, word, 2);
        const int64_t blk = e >> 5;
        if ((lane & 3) == 0) reinterpret_cast<uint32_t*>(p.xq)[blk * 8 + (lane >> 2)] = word;
        if (lane == 0) {
            p.xs[blk] = (float)dq;
            if (p.xsum) p.xsum[blk] = sm;
        }
    }
}

template <int GS>
__device__ __forceinline__ void attn_finish(const AttnParams& p, float* s_part, int* s_last_p, int gc, int g0, int hkv,
                                            int split, int gz, int hd, int row) {
    __shared__ float s_cw[kAttnGroup][kAttnWarps];   // weight of each warp's state in the CTA's state
    __shared__ float s_cM[kAttnGroup], s_cL[kAttnGroup];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (warp < gc && lane < kAttnWarps) {            // warp g merges the eight (max, sum) pairs of head g
        const float* st = s_part + (lane * gc + warp) * row + hd;
        const float mw = st[0], lw = st[1];
        float M = mw;
#pragma unroll
        for (int o = kAttnWarps / 2; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xFFu, M, o));
        const float e = expf(mw - M);
        float L = lw * e;
#pragma unroll
        for (int o = kAttnWarps / 2; o > 0; o >>= 1) L += __shfl_xor_sync(0xFFu, L, o);
        s_cw[warp][lane] = e;
        if (lane == 0) {
            s_cM[warp] = M;
            s_cL[warp] = L;
        }
    }
    __syncthreads();
    // CTA state per (g, d): straight to out when there is one slice, else to the scratch
    float* mine = p.part + ((((int64_t)hkv * gridDim.z + gz) * p.S + split) * GS) * row;
    for (int i = threadIdx.x; i < gc * hd; i += blockDim.x) {
        const int g = i / hd, d = i - g * hd;
        const float* base = s_part + g * row + d;
        float O = 0.f;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) O = fmaf(base[w * gc * row], s_cw[g][w], O);
        if (p.S == 1) attn_store(p, (int64_t)(hkv * p.group + g0 + g) * hd + d, O * (1.0f / s_cL[g]), lane);
        else mine[g * row + d] = O;
    }
    if (p.S > 1 && threadIdx.x < gc) {
        mine[threadIdx.x * row + hd] = s_cM[threadIdx.x];
        mine[threadIdx.x * row + hd + 1] = s_cL[threadIdx.x];
    }
    if (p.S == 1) return;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int prev = atomicAdd(p.counters + hkv * gridDim.z + gz, 1);
        *s_last_p = prev == p.S - 1;
        if (*s_last_p) p.counters[hkv * gridDim.z + gz] = 0;   // ready for the next launch / graph replay
    }
    __syncthreads();
    if (!*s_last_p) return;
    __threadfence();
    // The last CTA of this KV head merges the S slices.  Slice weights exp(m_s - M) and the sums L go
    // through shared memory (the per-warp states are dead by now; the host keeps S + 1 <= 8 * row),
    // so that the loop over the slices below is independent loads the compiler can batch.
    const float* all = p.part + (((int64_t)hkv * gridDim.z + gz) * p.S * GS) * row;
    const int S = p.S;
    float* s_w = s_part;            // [gc][S] maxima, then weights
    float* s_L = s_part + gc * S;   // [gc]
    for (int i = threadIdx.x; i < gc * S; i += blockDim.x) {
        const int g = i / S, sl = i - g * S;
        s_w[i] = __ldcg(all + ((int64_t)sl * GS + g) * row + hd);
    }
    __syncthreads();
    if (warp < gc) {
        float M = kNegInf;
        for (int sl = lane; sl < S; sl += 32) M = fmaxf(M, s_w[warp * S + sl]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
        float Lsum = 0.f;
        for (int sl = lane; sl < S; sl += 32) {
            const float e = expf(s_w[warp * S + sl] - M);
            Lsum = fmaf(__ldcg(all + ((int64_t)sl * GS + warp) * row + hd + 1), e, Lsum);
            s_w[warp * S + sl] = e;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) Lsum += __shfl_xor_sync(0xffffffffu, Lsum, o);
        if (lane == 0) s_L[warp] = Lsum;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < gc * hd; i += blockDim.x) {
        const int g = i / hd, d = i - g * hd;
        const float* col = all + (int64_t)g * row + d;
        float O = 0.f;
#pragma unroll 8
        for (int sl = 0; sl < S; ++sl) O = fmaf(__ldcg(col + (int64_t)sl * GS * row), s_w[g * S + sl], O);
        attn_store(p, (int64_t)(hkv * p.group + g0 + g) * hd + d, O * (1.0f / s_L[g]), lane);
    }
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
    attn_finish<kAttnGroup>(p, s_part, &s_last, gc, g0, hkv, split, gz, hd, row);
}

// head_dim = 32 * VEC (64, 128): eight lanes share a cache position, so a warp works on four
// positions at once and a dot needs three shuffles; a lane owns float4 columns sub, sub + 8, ... of
// the head.  Query heads (pre-scaled) sit in shared memory; a CTA serves up to kFastGroup of them.
// GC = query heads a CTA serves at most (1 or 2): the accumulators of unused heads would only cost
// registers, and with one head per CTA four CTAs fit an SM instead of two.
constexpr int kFastGroup = 2;
template <int VEC, int GC>
__global__ void __launch_bounds__(kAttnWarps * 32, GC == 1 ? 4 : 2)
gqa_decode_fast_kernel(const AttnParams p) {
    extern __shared__ __align__(16) float s_part[];   // [kAttnWarps][gc][hd + 4], then q [gc][hd]
    __shared__ int s_last;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    constexpr int hd = 32 * VEC, hd4 = hd / 4, row = hd + 4;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, grp = lane >> 3, sub = lane & 7;
    const int hkv = blockIdx.x, split = blockIdx.y, gz = blockIdx.z;
    const int g0 = gz * GC;
    const int gc = min(GC, p.group - g0);
    float4* s_q = reinterpret_cast<float4*>(s_part + kAttnWarps * gc * row);
    for (int i = threadIdx.x; i < gc * hd4; i += blockDim.x) {
        const float4 t = reinterpret_cast<const float4*>(p.q + (int64_t)(hkv * p.group + g0) * hd)[i];
        s_q[i] = make_float4(t.x * p.scale, t.y * p.scale, t.z * p.scale, t.w * p.scale);
    }
    __syncthreads();
    const int64_t clen = p.clenbuf ? p.clenbuf[0] : p.cache_len;
    const int64_t chunk = (clen + p.S - 1) / p.S;
    const int64_t j0 = split * chunk, j1 = min(clen, j0 + chunk);
    const int64_t kv4 = ((int64_t)p.n_kv * hd) >> 2;
    const float4* kb = reinterpret_cast<const float4*>(p.k + (int64_t)hkv * hd) + sub;
    const float4* vb = reinterpret_cast<const float4*>(p.v + (int64_t)hkv * hd) + sub;
    const unsigned gmask = 0xFFu << (grp * 8);
    float4 acc[GC][VEC];
    float m[GC], l[GC];
#pragma unroll
    for (int g = 0; g < GC; ++g) {
        m[g] = kNegInf;
        l[g] = 0.f;
#pragma unroll
        for (int u = 0; u < VEC; ++u) acc[g][u] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    // the rows of the next position are requested before the current one is worked on: a CTA has only
    // a few positions per lane group, so an exposed load latency per step is most of the kernel
    // (not with one head per CTA, where four CTAs per SM hide the latency already: measured)
    constexpr bool PF = GC > 1;
    float4 kk[VEC], vv[VEC], kn[VEC], vn[VEC];
    {
        const int64_t jf = j0 + warp * 4 + grp;
        if (PF && jf < j1) {
#pragma unroll
            for (int u = 0; u < VEC; ++u) kn[u] = __ldg(kb + jf * kv4 + 8 * u);
#pragma unroll
            for (int u = 0; u < VEC; ++u) vn[u] = __ldg(vb + jf * kv4 + 8 * u);
        }
    }
    for (int64_t j = j0 + warp * 4 + grp; j < j1; j += kAttnWarps * 4) {
        if (PF) {
#pragma unroll
            for (int u = 0; u < VEC; ++u) {
                kk[u] = kn[u];
                vv[u] = vn[u];
            }
        }
        const int64_t jn = j + kAttnWarps * 4;
        if (!PF) {   // fetch this position's rows now
#pragma unroll
            for (int u = 0; u < VEC; ++u) kk[u] = __ldg(kb + j * kv4 + 8 * u);
#pragma unroll
            for (int u = 0; u < VEC; ++u) vv[u] = __ldg(vb + j * kv4 + 8 * u);
        } else if (jn < j1) {
#pragma unroll
            for (int u = 0; u < VEC; ++u) kn[u] = __ldg(kb + jn * kv4 + 8 * u);
#pragma unroll
            for (int u = 0; u < VEC; ++u) vn[u] = __ldg(vb + jn * kv4 + 8 * u);
        }
#pragma unroll
        for (int g = 0; g < GC; ++g) {
            if (g < gc) {
                float s = 0.f;
#pragma unroll
                for (int u = 0; u < VEC; ++u) {
                    const float4 qq = s_q[g * hd4 + sub + 8 * u];
                    s = fmaf(qq.x, kk[u].x, fmaf(qq.y, kk[u].y, fmaf(qq.z, kk[u].z, fmaf(qq.w, kk[u].w, s))));
                }
                s += __shfl_xor_sync(gmask, s, 1);   // the eight lanes of this position only: the other
                s += __shfl_xor_sync(gmask, s, 2);   // groups of the warp may have left the loop already
                s += __shfl_xor_sync(gmask, s, 4);
                const float mn = fmaxf(m[g], s);
                const float corr = expf(m[g] - mn), pj = expf(s - mn);
                m[g] = mn;
                l[g] = fmaf(l[g], corr, pj);
#pragma unroll
                for (int u = 0; u < VEC; ++u) {
                    acc[g][u].x = fmaf(acc[g][u].x, corr, pj * vv[u].x);
                    acc[g][u].y = fmaf(acc[g][u].y, corr, pj * vv[u].y);
                    acc[g][u].z = fmaf(acc[g][u].z, corr, pj * vv[u].z);
                    acc[g][u].w = fmaf(acc[g][u].w, corr, pj * vv[u].w);
                }
            }
        }
    }
    // the four position groups of the warp -> one state (every lane ends with the merged values)
#pragma unroll
    for (int g = 0; g < GC; ++g) {
        if (g < gc) {
#pragma unroll
            for (int o = 8; o <= 16; o <<= 1) {
                const float mo = __shfl_xor_sync(0xffffffffu, m[g], o);
                const float lo = __shfl_xor_sync(0xffffffffu, l[g], o);
                const float mn = fmaxf(m[g], mo);
                const float es = expf(m[g] - mn), eo = expf(mo - mn);
                m[g] = mn;
                l[g] = fmaf(l[g], es, lo * eo);
#pragma unroll
                for (int u = 0; u < VEC; ++u) {
                    acc[g][u].x = fmaf(acc[g][u].x, es, __shfl_xor_sync(0xffffffffu, acc[g][u].x, o) * eo);
                    acc[g][u].y = fmaf(acc[g][u].y, es, __shfl_xor_sync(0xffffffffu, acc[g][u].y, o) * eo);
                    acc[g][u].z = fmaf(acc[g][u].z, es, __shfl_xor_sync(0xffffffffu, acc[g][u].z, o) * eo);
                    acc[g][u].w = fmaf(acc[g][u].w, es, __shfl_xor_sync(0xffffffffu, acc[g][u].w, o) * eo);
                }
            }
            if (grp == 0) {
                float* dst = s_part + (warp * gc + g) * row;
#pragma unroll
                for (int u = 0; u < VEC; ++u) reinterpret_cast<float4*>(dst)[sub + 8 * u] = acc[g][u];
                if (sub == 0) {
                    dst[hd] = m[g];
                    dst[hd + 1] = l[g];
                }
            }
        }
    }
    attn_finish<GC>(p, s_part, &s_last, gc, g0, hkv, split, gz, hd, row);
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

int32_t rstq_rope_pos(rstq_ctx* ctx, rstq_buf* x, rstq_buf* out, rstq_buf* posbuf, int64_t heads,
                      int64_t head_dim, double theta, int64_t pos) {
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

int32_t rstq_kv_append(rstq_ctx* ctx, rstq_buf* src, rstq_buf* cache, rstq_buf* posbuf, int64_t kvrow,
                       int64_t pos, int64_t maxpos) {
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

int32_t rstq_rope_append(rstq_ctx* ctx, rstq_buf* q, rstq_buf* k, rstq_buf* v, rstq_buf* kcache,
                         rstq_buf* vcache, rstq_buf* posbuf, int64_t n_q, int64_t n_kv, int64_t head_dim,
                         double theta, int64_t pos, int64_t maxpos) {
    RSTQ_REQUIRE(ctx && ctx->magic == kCtxMagic, RSTQ_E_INVALID, "invalid context handle");
    RSTQ_REQUIRE(n_q >= 1 && n_kv >= 1 && head_dim >= 2 && head_dim % 2 == 0 && theta > 0.0 && maxpos >= 1 &&
                     (posbuf || (pos >= 0 && pos < maxpos)),
                 RSTQ_E_SHAPE, "n_q = %lld, n_kv = %lld, head_dim = %lld (even), pos = %lld of %lld", (long long)n_q,
                 (long long)n_kv, (long long)head_dim, (long long)pos, (long long)maxpos);
    const int64_t kvrow = n_kv * head_dim;
    RSTQ_REQUIRE(attn_buf(q, ctx, n_q * head_dim * 4) && attn_buf(k, ctx, kvrow * 4) && attn_buf(v, ctx, kvrow * 4) &&
                     attn_buf(kcache, ctx, maxpos * kvrow * 4) && attn_buf(vcache, ctx, maxpos * kvrow * 4) &&
                     (!posbuf || attn_buf(posbuf, ctx, 8)),
                 RSTQ_E_INVALID, "invalid, unaligned or too small buffer (the caches hold maxpos rows)");
    RSTQ_REQUIRE(q->dev == k->dev && q->dev == v->dev && q->dev == kcache->dev && q->dev == vcache->dev &&
                     (!posbuf || posbuf->dev == q->dev),
                 RSTQ_E_DEVICE, "buffers live on different devices");
    DeviceState& ds = ctx->devs[q->dev];
    int32_t rc = use_dev(ctx, q->dev);
    if (rc != RSTQ_OK) return rc;
    const int64_t items = (n_q + 2 * n_kv) * (head_dim / 2);
    RSTQ_CUDA(launch_attn(rope_append_kernel, dim3((unsigned)((items + 255) / 256)), dim3(256), 0, ds, (float*)q->ptr,
                          (float*)k->ptr, (const float*)v->ptr, (float*)kcache->ptr, (float*)vcache->ptr, n_q, n_kv,
                          head_dim, log(theta), pos, posbuf ? (const int64_t*)posbuf->ptr : (const int64_t*)nullptr));
    ctx->launches++;
    return RSTQ_OK;
}

static int32_t attention_impl(rstq_ctx* ctx, rstq_buf* q, rstq_buf* k, rstq_buf* v, rstq_buf* out,
                              int64_t cache_len, rstq_buf* clenbuf, int64_t n_q, int64_t group, int64_t n_kv,
                              int64_t head_dim, int64_t maxpos, double scale, rstq_buf* xq, rstq_buf* xs,
                              rstq_buf* xsum) {
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
    const bool fast = head_dim == 64 || head_dim == 128;
    // heads per CTA of the fast kernel: two (one when the group is one).  Four leave no registers for the
    // rows fetched ahead at head_dim 128 (23.2 against 16.2 us at 32 q / 8 kv x 4096, although K / V then pass
    // through L2 twice) and lose at head_dim 64 too (14.8 against 13.3 us).
    const int64_t fg = group >= 2 ? 2 : 1;
    const int64_t gs = fast ? fg : kAttnGroup;                         // query heads per CTA
    const int64_t gz = (group + gs - 1) / gs;
    RSTQ_REQUIRE(n_kv * gz <= kAttnCounters, RSTQ_E_LIMIT, "n_kv x ceil(group / %d) = %lld exceeds %d", (int)gs,
                 (long long)(n_kv * gz), kAttnCounters);
    // slices of the cache: enough CTAs for three per SM, at least 64 positions each; sized from the
    // capacity when the length lives on the device, so that one captured launch serves every length
    const int64_t span = clenbuf ? maxpos : cache_len;
    const int64_t resident = fast && fg == 1 ? 4 : 2;   // CTAs an SM holds (registers): aim at one wave
    int64_t S = resident * (int64_t)ds.sm_count / (n_kv * gz);
    if (S > (span + 63) / 64) S = (span + 63) / 64;
    const int64_t row = head_dim + 4;
    if (S > 8 * row - 1) S = 8 * row - 1;   // the final merge keeps S weights + 1 sum per head in shared memory
    if (S > 512) S = 512;
    if (S < 1) S = 1;
    if (xq) {
        RSTQ_REQUIRE(fast, RSTQ_E_SHAPE, "the quantized output needs head_dim 64 or 128, got %lld", (long long)head_dim);
        const int64_t n = n_q * head_dim;
        RSTQ_REQUIRE(attn_buf(xq, ctx, n) && attn_buf(xs, ctx, n / 32 * 4) && (!xsum || attn_buf(xsum, ctx, n / 32 * 4)),
                     RSTQ_E_INVALID, "invalid, unaligned or too small quantizer buffer");
        RSTQ_REQUIRE(xq->dev == q->dev && xs->dev == q->dev && (!xsum || xsum->dev == q->dev), RSTQ_E_DEVICE,
                     "buffers live on different devices");
    }
    const int64_t part_bytes = n_kv * gz * S * gs * row * 4;
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
    p.xq = xq ? (int8_t*)xq->ptr : nullptr;
    p.xs = xq ? (float*)xs->ptr : nullptr;
    p.xsum = xq && xsum ? (int32_t*)xsum->ptr : nullptr;
    const int64_t gc = group < gs ? group : gs;
    const dim3 grid((unsigned)n_kv, (unsigned)S, (unsigned)gz), block(kAttnWarps * 32);
    if (fast) {
        const size_t smem = (size_t)((kAttnWarps * gc * row + gc * head_dim) * 4);   // <= 17.5 KB
        cudaError_t e;
        if (head_dim == 64)
            e = fg == 1 ? launch_attn(gqa_decode_fast_kernel<2, 1>, grid, block, smem, ds, p)
                        : launch_attn(gqa_decode_fast_kernel<2, 2>, grid, block, smem, ds, p);
        else
            e = fg == 1 ? launch_attn(gqa_decode_fast_kernel<4, 1>, grid, block, smem, ds, p)
                        : launch_attn(gqa_decode_fast_kernel<4, 2>, grid, block, smem, ds, p);
        RSTQ_CUDA(e);
    } else {
        const size_t smem = (size_t)(kAttnWarps * gc * row * 4);
        if (smem > 48 * 1024)
            RSTQ_CUDA(cudaFuncSetAttribute(gqa_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        RSTQ_CUDA(launch_attn(gqa_decode_kernel, grid, block, smem, ds, p));
    }
    ctx->launches++;
    return RSTQ_OK;
}

int32_t rstq_gqa_decode_attention(rstq_ctx* ctx, rstq_buf* q, rstq_buf* k, rstq_buf* v, rstq_buf* out,
                                  rstq_buf* clenbuf, int64_t cache_len, int64_t n_q, int64_t group,
                                  int64_t n_kv, int64_t head_dim, int64_t maxpos, double scale) {
    return attention_impl(ctx, q, k, v, out, cache_len, clenbuf, n_q, group, n_kv, head_dim, maxpos, scale, nullptr,
                          nullptr, nullptr);
}

int32_t rstq_gqa_decode_attention_quant_act(rstq_ctx* ctx, rstq_buf* q, rstq_buf* k, rstq_buf* v, rstq_buf* out,
                                            rstq_buf* xq, rstq_buf* xs, rstq_buf* xsum, rstq_buf* clenbuf,
                                            int64_t cache_len, int64_t n_q, int64_t group, int64_t n_kv,
                                            int64_t head_dim, int64_t maxpos, double scale) {
    RSTQ_REQUIRE(xq && xs, RSTQ_E_INVALID, "null quantizer buffer");
    return attention_impl(ctx, q, k, v, out, cache_len, clenbuf, n_q, group, n_kv, head_dim, maxpos, scale, xq, xs, xsum);
}

}  // extern "C"
