// C ABI of librstq: contexts, buffers, weight binding, operator dispatch,
// graphs and events.  See include/rstq.h for the contract of each entry point.
#include <stdarg.h>
#include <stdio.h>
#include <math.h>
#include <string.h>

#include <new>
#include <vector>

#include "internal.h"

namespace rstq {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int32_t cuda_fail(cudaError_t e, const char* what, const char* file, int line) {
    const char* base = strrchr(file, '/');
    set_error("CUDA error %d (%s) at %s:%d in %s", (int)e, cudaGetErrorString(e),
              base ? base + 1 : file, line, what);
    return e == cudaErrorMemoryAllocation ? RSTQ_E_OOM : RSTQ_E_CUDA;
}

static bool ok_ctx(const rstq_ctx* c) { return c && c->magic == kCtxMagic; }
static bool ok_buf(const rstq_buf* b) { return b && b->magic == kBufMagic && ok_ctx(b->ctx); }
static bool ok_w(const rstq_weight* w) { return w && w->magic == kWgtMagic && ok_ctx(w->ctx); }

#define CHECK_CTX(c) RSTQ_REQUIRE(ok_ctx(c), RSTQ_E_INVALID, "invalid context handle")
#define CHECK_DEV(c, d)                                                              \
    RSTQ_REQUIRE((d) >= 0 && (d) < (int)(c)->devs.size(), RSTQ_E_NODEV,              \
                 "device index %d out of range (context has %d)", (int)(d), (int)(c)->devs.size())

int32_t use_dev(rstq_ctx* ctx, int dev) {
    RSTQ_CUDA(cudaSetDevice(ctx->devs[dev].ordinal));
    return RSTQ_OK;
}

// grow-only scratch helpers (never called while capturing)
int32_t dev_reserve(DeviceState& ds, void** p, int64_t* have, int64_t need) {
    if (need <= *have) return RSTQ_OK;
    RSTQ_REQUIRE(!ds.capturing, RSTQ_E_STATE,
                 "scratch must grow (%lld bytes) during graph capture; run the call once before "
                 "capturing", (long long)need);
    if (*p) {
        int32_t rc = dev_release_scratch(ds, *p);
        if (rc != RSTQ_OK) return rc;
        *p = nullptr;
        *have = 0;
    }
    need = (need + 0xFFFFF) & ~0xFFFFFll;
    RSTQ_CUDA(cudaMalloc(p, (size_t)need));
    *have = need;
    return RSTQ_OK;
}

int32_t dev_release_scratch(DeviceState& ds, void* p) {
    if (!p) return RSTQ_OK;
    if (ds.live_graphs > 0) {   // a recorded launch may still name this block
        ds.retired.push_back(p);
        return RSTQ_OK;
    }
    RSTQ_CUDA(cudaStreamSynchronize(ds.stream));
    RSTQ_CUDA(cudaFree(p));
    return RSTQ_OK;
}

static int32_t ensure_pinned(DeviceState& ds, int64_t need) {
    if (need <= ds.pinned_bytes) return RSTQ_OK;
    if (ds.pinned) {
        RSTQ_CUDA(cudaStreamSynchronize(ds.stream));
        RSTQ_CUDA(cudaFreeHost(ds.pinned));
        ds.pinned = nullptr;
        ds.pinned_bytes = 0;
    }
    need = (need + 0xFFFF) & ~0xFFFFll;
    RSTQ_CUDA(cudaMallocHost(&ds.pinned, (size_t)need));
    ds.pinned_bytes = need;
    return RSTQ_OK;
}

__global__ void block_sum_kernel(const int8_t* __restrict__ xq, int32_t* __restrict__ xsum,
                                 int64_t nblocks) {
    const int64_t b = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (b >= nblocks) return;
    const int4* p = reinterpret_cast<const int4*>(xq + b * 32);
    int s = 0;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int4 v = p[h];
        s = __dp4a(v.x, 0x01010101, s);
        s = __dp4a(v.y, 0x01010101, s);
        s = __dp4a(v.z, 0x01010101, s);
        s = __dp4a(v.w, 0x01010101, s);
    }
    xsum[b] = s;
}

// y[o] = (float) sum_w dp4a(wp[o*kw + w], xp[w]) : exact int32 dot, one warp per row.
__global__ void i8gemv_dp4a_kernel(const int32_t* __restrict__ wp, const int32_t* __restrict__ xp,
                                   float* __restrict__ y, int64_t kw, int64_t out) {
    const int lane = threadIdx.x & 31;
    const int64_t o = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
    if (o >= out) return;
    int acc = 0;
    for (int64_t k = lane; k < kw; k += 32) acc = __dp4a(wp[o * kw + k], xp[k], acc);
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
    if (lane == 0) y[o] = (float)acc;
}

// Activation scratch layout for MODE_A8: [xq: M*in int8][xs: M*nb f32][xsum: M*nb i32]
struct ActScratch {
    int8_t* xq;
    float* xs;
    int32_t* xsum;
    uint8_t* img;   // the decode kernel's staged form of the three (2 <= M < 64), see quant_act_i8_kernel
};
static int32_t act_scratch(DeviceState& ds, int64_t M, int64_t in, ActScratch* out) {
    const int64_t nb = in / 32;
    const int64_t xq_bytes = (M * in + 255) & ~255ll;
    const int64_t sb = (M * nb * 4 + 255) & ~255ll;
    const bool image = M >= 1 && M < 64;   // what the decode kernels serve in MODE_A8: one image per launch of kGemvMaxM tokens
    const int64_t img_bytes = image ? ((M + kGemvMaxM - 1) / kGemvMaxM) * act_image_stride(nb) : 0;
    // xsum has room for sums per 16 elements (Q6_K units): two per block
    int32_t rc = dev_reserve(ds, &ds.act_scratch, &ds.act_scratch_bytes, xq_bytes + 3 * sb + img_bytes);
    if (rc != RSTQ_OK) return rc;
    char* base = (char*)ds.act_scratch;
    out->xq = (int8_t*)base;
    out->xs = (float*)(base + xq_bytes);
    out->xsum = (int32_t*)(base + xq_bytes + sb);
    out->img = image ? (uint8_t*)(base + xq_bytes + 3 * sb) : nullptr;
    return RSTQ_OK;
}

// A decode launch of w is about to be made: remember the order of the weights on this device (the
// previous one learns that w follows it) and return what followed w last time, if it still exists.
static NextWeight note_decode_launch(rstq_ctx* ctx, DeviceState& ds, rstq_weight* w) {
    if (ds.last_decode_w && ds.last_decode_w != w && ctx->live_weights.count(ds.last_decode_w))
        ds.last_decode_w->next_hint = w;
    ds.last_decode_w = w;
    NextWeight n;
    rstq_weight* h = w->next_hint;
    if (ds.prefetch_next && h && h != w && ctx->live_weights.count(h) && h->dev == w->dev) {
        n.data = h->data;
        n.groups = h->outp / 32;
        n.nb = h->nb;
        n.bits = h->kq ? 5 : (h->k6 ? 6 : h->bits);   // the unit kind
    }
    return n;
}

// One matmul over device pointers, M split into decode-kernel chunks.
static int32_t run_a8(rstq_ctx* ctx, rstq_weight* w, const int8_t* xq, const float* xs,
                      const int32_t* xsum, float* y, int64_t M, const TpFuse* tp = nullptr,
                      const uint8_t* img = nullptr, uint8_t* img_scratch = nullptr) {
    GemvA8Args a{w->data, xq, xs, xsum, y, M, w->in, w->out, w->bits, w->zp, tp};
    a.img = img;
    a.img_scratch = img_scratch;
    a.uk = w->kq ? 1 : (w->k6 ? 2 : 0);
    a.next = note_decode_launch(ctx, ctx->devs[w->dev], w);
    return launch_gemv_a8(ctx, ctx->devs[w->dev], a);
}

static int32_t run_f(rstq_ctx* ctx, rstq_weight* w, const void* x, void* y, int64_t M,
                     int act_dtype, int out_dtype, const TpFuse* tp = nullptr) {
    GemvFArgs a{w->data, x, y, M, w->in, w->out, w->bits, w->zp, act_dtype, out_dtype, tp};
    DeviceState& ds = ctx->devs[w->dev];
    if (M > 1 || act_dtype == RSTQ_F32) {   // room for the staged activations to ride the weight ring; without it: fewer tokens per launch
        const int64_t need = gemv_f_image_bytes(w->in);
        if (ds.f_image_bytes >= need || dev_reserve(ds, &ds.f_image, &ds.f_image_bytes, need) == RSTQ_OK)
            a.img_scratch = (uint8_t*)ds.f_image;
    }
    a.next = note_decode_launch(ctx, ctx->devs[w->dev], w);
    return launch_gemv_f(ctx, ctx->devs[w->dev], a);
}

// Q4_K: decode kernel over the sub-block scales (zero point 0), then the min term added to y.
static int32_t run_q4k(rstq_ctx* ctx, rstq_weight* w, const int8_t* xq, const float* xs32, const int32_t* bsums,
                       float* y, int64_t M, uint8_t* img_scratch = nullptr) {
    int32_t rc = run_a8(ctx, w, xq, xs32, bsums, y, M, nullptr, nullptr, w->kq ? img_scratch : nullptr);
    if (rc != RSTQ_OK || w->kq) return rc;   // Q4_K units: the decode kernel added the min term itself
    return launch_q4k_min(ctx, ctx->devs[w->dev], w->mins, xs32, bsums, y, M, w->nb, w->out);
}

// scratch of the tensor-core path: [x16: M*in halves][rowscale: M floats][acc: M*out f32, only for
// calls small enough to be split along K]
static int32_t gemm_scratch(DeviceState& ds, int64_t M, int64_t in, int64_t out, void** x16, float** rowscale,
                            float** acc) {
    const int64_t xb = (M * in * 2 + 255) & ~255ll, rb = (M * 4 + 255) & ~255ll;
    // the partial tiles of a GEMM split along K (launch_gemm; gemm_tc_kernel's f32 array for M <= 256 fits too)
    const int64_t ab = M <= 256 && M * out * 4 > kPairScratchBytes ? M * out * 4 : kPairScratchBytes;
    int32_t rc = dev_reserve(ds, &ds.gemm_scratch, &ds.gemm_scratch_bytes, xb + rb + ab);
    if (rc != RSTQ_OK) return rc;
    *x16 = ds.gemm_scratch;
    *rowscale = (float*)((char*)ds.gemm_scratch + xb);
    *acc = ab ? (float*)((char*)ds.gemm_scratch + xb + rb) : nullptr;
    return RSTQ_OK;
}

int32_t matmul_device(rstq_ctx* ctx, rstq_weight* w, const void* x, void* y, int64_t M, int act_dtype,
                      int out_dtype, int mode, const TpFuse* tp) {
    DeviceState& ds = ctx->devs[w->dev];
    if (w->pair_out) {
        // Q6_K: q8_K activations (the decode kernel wants the code sums per 32 elements), the twin
        // rows through the decode kernel, then the pairs added (src/raster/quant/core.clj:68-75).
        RSTQ_REQUIRE(mode == RSTQ_MODE_A8 && act_dtype == RSTQ_F32 && out_dtype == RSTQ_F32, RSTQ_E_INVALID,
                     "a Q6_K weight takes f32 activations in MODE_A8 and writes f32");
        if (tp) return kNotFused;   // the exchange is fused into the per-32-block kernels only
        ActScratch s;
        int32_t rc = act_scratch(ds, M, w->in, &s);
        if (rc != RSTQ_OK) return rc;
        if (w->k6) {
            // units with a scale per 16 elements: code sums per 16, one decode launch, y as it is
            rc = launch_quant_act_q8k(ctx, ds, (const float*)x, s.xq, nullptr, s.xs, s.xsum, M, w->in, 16);
            if (rc != RSTQ_OK) return rc;
            return run_a8(ctx, w, s.xq, s.xs, s.xsum, (float*)y, M, nullptr, nullptr, ds.act_image ? s.img : nullptr);
        }
        if ((rc = dev_reserve(ds, &ds.kq_scratch, &ds.kq_scratch_bytes, M * w->out * 4)) != RSTQ_OK) return rc;
        rc = launch_quant_act_q8k(ctx, ds, (const float*)x, s.xq, nullptr, s.xs, s.xsum, M, w->in, 32);
        if (rc != RSTQ_OK) return rc;
        if ((rc = run_a8(ctx, w, s.xq, s.xs, s.xsum, (float*)ds.kq_scratch, M)) != RSTQ_OK) return rc;
        return launch_pair_sum(ctx, ds, (const float*)ds.kq_scratch, (float*)y, M, w->pair_out);
    }
    if (w->mins) {
        // Q4_K: the one arithmetic the reference has for it -- q8_K activations, integer sub-block
        // dots, scale / min fold (src/raster/quant/core.clj:57-66) -- at any M, on the decode kernel.
        RSTQ_REQUIRE(mode == RSTQ_MODE_A8 && act_dtype == RSTQ_F32 && out_dtype == RSTQ_F32, RSTQ_E_INVALID,
                     "a Q4_K weight takes f32 activations in MODE_A8 and writes f32");
        if (tp) return kNotFused;
        ActScratch s;
        int32_t rc = act_scratch(ds, M, w->in, &s);
        if (rc != RSTQ_OK) return rc;
        rc = launch_quant_act_q8k(ctx, ds, (const float*)x, s.xq, nullptr, s.xs, s.xsum, M, w->in, 32);
        if (rc != RSTQ_OK) return rc;
        return run_q4k(ctx, w, s.xq, s.xs, s.xsum, (float*)y, M, ds.act_image ? s.img : nullptr);
    }
    // Prefill shapes go to the tensor-core GEMM (fp16 operands, results within 1e-3 of the
    // reference).  A8 keeps its exact integer path up to M = 63: callers that chose the
    // quantized-activation arithmetic get it bit-faithfully at decode and small-batch sizes.
    bool tc = M >= (mode == RSTQ_MODE_A8 ? (ctx->tune_gemm_min_m > 64 ? ctx->tune_gemm_min_m : 64)
                                          : ctx->tune_gemm_min_m);
    // MODE_F below the threshold: the decode kernel keeps every token's activations (for f32, two or
    // three bf16 terms each) in shared memory beside the weight ring; what does not fit is cut into
    // several launches, each streaming all the weights again.  Measured at the Llama-7B shapes, M = 1 .. 16:
    // two launches of f32 (three of bf16) activations already cost more than the tensor-core path.
    // (Matrices of a few MB stay on the decode kernel and keep its f32-grade result.)
    if (mode == RSTQ_MODE_F && !tc && M >= 2 && ctx->tune_gemm_min_m == 17 && w->data_bytes >= (4ll << 20)) {
        const int pieces = gemv_f_pieces(ds, w->bits, w->out, w->in, M, act_dtype);
        if (pieces >= (act_dtype == RSTQ_F32 ? 2 : 3)) tc = true;
    }
    // The same for MODE_A8 when not even 8 tokens of codes fit (K > 16 K): the codes and scales the
    // quantizer produced feed the tensor-core path instead (<= 1e-3, no longer the exact integer dots).
    // Up to 16 tokens this does not arise: their activations ride the weight ring, whatever K is.
    const bool rides = M <= 16 && ds.act_image && ds.act_ring != 1 && ds.act_ring != 4;
    if (mode == RSTQ_MODE_A8 && !tc && M >= 9 && !rides && ctx->tune_gemm_min_m == 17 && w->in * 8 > 128 * 1024) tc = true;
    if (tp && (tc || out_dtype != RSTQ_F32)) return kNotFused;  // only the decode kernel fuses the exchange
    if (mode == RSTQ_MODE_A8) {
        RSTQ_REQUIRE(act_dtype == RSTQ_F32 || act_dtype == RSTQ_BF16, RSTQ_E_INVALID, "unknown activation type");
        RSTQ_REQUIRE(out_dtype == RSTQ_F32 || tc, RSTQ_E_INVALID, "MODE_A8 decode writes f32");
        if (M == 1 && !tc && ds.fuse_quant && !ds.x_on_host && w->in <= kFusedQuantMaxIn) {
            // one token: every CTA of the decode kernel quantizes x (16 - 112 KB, in L2) while it
            // stages it, bit for bit as the quantizer kernel would -- one launch, no scratch
            GemvA8Args a{w->data, nullptr, nullptr, nullptr, (float*)y, 1, w->in, w->out, w->bits, w->zp, tp, x, act_dtype};
            a.next = note_decode_launch(ctx, ds, w);
            return launch_gemv_a8(ctx, ds, a);
        }
        ActScratch s;
        int32_t rc = act_scratch(ds, M, w->in, &s);
        if (rc != RSTQ_OK) return rc;
        uint8_t* img = (!tc && ds.act_image) ? s.img : nullptr;
        rc = launch_quant_act_i8(ctx, ds, x, s.xq, s.xs, s.xsum, M, w->in, act_dtype, img, w->zp, w->bits);
        if (rc != RSTQ_OK) return rc;
        if (!tc) return run_a8(ctx, w, s.xq, s.xs, s.xsum, (float*)y, M, tp, img);
        void* x16;
        float* rowscale;
        float* acc;
        if ((rc = gemm_scratch(ds, M, w->in, w->out, &x16, &rowscale, &acc)) != RSTQ_OK) return rc;
        return launch_gemm(ctx, ds, w, s.xq, s.xs, 2, y, out_dtype, M, x16, rowscale, acc);
    }
    if (!tc) return run_f(ctx, w, x, y, M, act_dtype, out_dtype, tp);
    void* x16;
    float* rowscale;
    float* acc;
    int32_t rc = gemm_scratch(ds, M, w->in, w->out, &x16, &rowscale, &acc);
    if (rc != RSTQ_OK) return rc;
    return launch_gemm(ctx, ds, w, x, nullptr, act_dtype == RSTQ_F32 ? 0 : 1, y, out_dtype, M, x16, rowscale, acc);
}

static int32_t bind_impl(rstq_ctx* ctx, rstq_weight** wout, const void* codes,
                         const float* scales, int dev, int64_t out, int64_t in, int format,
                         int layout, int split, int rank, int nranks) {
    CHECK_CTX(ctx);
    RSTQ_REQUIRE(wout && codes && scales, RSTQ_E_INVALID, "null argument");
    *wout = nullptr;
    CHECK_DEV(ctx, dev);
    RSTQ_REQUIRE(format >= RSTQ_FMT_Q4_0 && format <= RSTQ_FMT_Q8_S, RSTQ_E_INVALID,
                 "unknown weight format %d", format);
    RSTQ_REQUIRE(layout == RSTQ_LAYOUT_ROWMAJOR || layout == RSTQ_LAYOUT_STREAM8, RSTQ_E_INVALID,
                 "unknown host layout %d", layout);
    RSTQ_REQUIRE(out >= 1 && in >= 32 && in % 32 == 0, RSTQ_E_SHAPE,
                 "in = %lld must be a positive multiple of 32 and out = %lld >= 1", (long long)in,
                 (long long)out);
    RSTQ_REQUIRE(layout != RSTQ_LAYOUT_STREAM8 || out % 8 == 0, RSTQ_E_SHAPE,
                 "stream layout needs out %% 8 == 0 (out = %lld)", (long long)out);
    RSTQ_REQUIRE(layout != RSTQ_LAYOUT_STREAM8 || format != RSTQ_FMT_Q8_S, RSTQ_E_INVALID,
                 "signed codes have no stream layout in the reference");
    RSTQ_REQUIRE(split >= RSTQ_SPLIT_NONE && split <= RSTQ_SPLIT_ROW, RSTQ_E_INVALID,
                 "unknown split %d", split);
    if (split == RSTQ_SPLIT_NONE) { rank = 0; nranks = 1; }
    RSTQ_REQUIRE(nranks >= 1 && rank >= 0 && rank < nranks, RSTQ_E_INVALID,
                 "rank %d of %d", rank, nranks);
    const int bits = format == RSTQ_FMT_Q4_0 ? 4 : 8;
    const int64_t nb_full = in / 32;
    int64_t sh_out = out, sh_in = in, row0 = 0, kb0 = 0;
    if (split == RSTQ_SPLIT_COLUMN) {
        const int64_t q = layout == RSTQ_LAYOUT_STREAM8 ? 8 : 1;
        RSTQ_REQUIRE(out % (nranks * q) == 0, RSTQ_E_SHAPE,
                     "column split: out = %lld not divisible by %lld", (long long)out,
                     (long long)(nranks * q));
        sh_out = out / nranks;
        row0 = rank * sh_out;
    } else if (split == RSTQ_SPLIT_ROW) {
        RSTQ_REQUIRE(nb_full % nranks == 0, RSTQ_E_SHAPE,
                     "row split: in/32 = %lld not divisible by %d", (long long)nb_full, nranks);
        sh_in = in / nranks;
        kb0 = rank * (sh_in / 32);
    }
    DeviceState& ds = ctx->devs[dev];
    RSTQ_REQUIRE(!ds.capturing, RSTQ_E_STATE, "cannot bind a weight during graph capture");
    int32_t rc = use_dev(ctx, dev);
    if (rc != RSTQ_OK) return rc;

    // Host slab holding the rows of this shard (all K; a row split selects its
    // K range inside the re-tiling kernel).
    const int64_t code_row_bytes = (int64_t)in * bits / 8;
    const uint8_t* hcodes = (const uint8_t*)codes + row0 * code_row_bytes;
    const float* hscales = scales + row0 * nb_full;
    const int64_t codes_bytes = sh_out * code_row_bytes;
    const int64_t scales_bytes = sh_out * nb_full * 4;

    rstq_weight* w = new (std::nothrow) rstq_weight();
    RSTQ_REQUIRE(w, RSTQ_E_OOM, "out of host memory");
    w->magic = kWgtMagic;
    w->ctx = ctx;
    w->dev = dev;
    w->bits = bits;
    w->zp = bits == 4 ? 8 : 128;
    w->out = sh_out;
    w->in = sh_in;
    w->outp = (sh_out + 31) / 32 * 32;
    w->nb = sh_in / 32;
    w->data_bytes = (w->outp / 32) * w->nb * unit_bytes(bits);
    w->data = nullptr;
    {
        float mxs = 0.f;
        const int64_t ns = sh_out * nb_full;
        for (int64_t i = 0; i < ns; ++i) {
            const float a = fabsf(hscales[i]);
            if (a > mxs && a < 3.0e38f) mxs = a;
        }
        int ex = 0;
        if (mxs > 0.f) frexpf(mxs, &ex);       // mxs = f * 2^ex, f in [0.5, 1)
        w->gemm_exp = mxs > 0.f ? 7 - ex : 0;  // largest scaled |weight| = 128 * f * 2^7 < 2^14
    }
    uint8_t *stage_c = nullptr;
    float* stage_s = nullptr;
    cudaError_t e = cudaMalloc((void**)&w->data, (size_t)w->data_bytes);
    if (e == cudaSuccess) e = cudaMalloc((void**)&stage_c, (size_t)codes_bytes);
    if (e == cudaSuccess) e = cudaMalloc((void**)&stage_s, (size_t)scales_bytes);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(stage_c, hcodes, (size_t)codes_bytes, cudaMemcpyHostToDevice, ds.stream);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(stage_s, hscales, (size_t)scales_bytes, cudaMemcpyHostToDevice, ds.stream);
    if (e == cudaSuccess) {
        rc = launch_repack(ctx, ds, stage_c, stage_s, w->data, format, layout, sh_out, sh_in, in, kb0);
        if (rc == RSTQ_OK) e = cudaStreamSynchronize(ds.stream);
    }
    if (stage_c) cudaFree(stage_c);
    if (stage_s) cudaFree(stage_s);
    if (e != cudaSuccess || rc != RSTQ_OK) {
        if (w->data) cudaFree(w->data);
        delete w;
        if (e != cudaSuccess) return cuda_fail(e, "weight bind", __FILE__, __LINE__);
        return rc;
    }
    ctx->live_weights.insert(w);
    *wout = w;
    return RSTQ_OK;
}

}  // namespace rstq

using namespace rstq;

extern "C" {

int32_t rstq_version(void) { return 100; }

const char* rstq_last_error(void) { return g_err; }

int32_t rstq_device_count(int32_t* count) {
    RSTQ_REQUIRE(count, RSTQ_E_INVALID, "null argument");
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) {
        *count = 0;
        cudaGetLastError();
        set_error("no CUDA device: %s", cudaGetErrorString(e));
        return RSTQ_E_NODEV;
    }
    *count = n;
    return RSTQ_OK;
}

int32_t rstq_init(const int32_t* devices, rstq_ctx** ctxp, int32_t ndev) {
    RSTQ_REQUIRE(ctxp, RSTQ_E_INVALID, "null argument");
    *ctxp = nullptr;
    RSTQ_REQUIRE(devices && ndev >= 1 && ndev <= 64, RSTQ_E_INVALID, "need 1..64 devices");
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0) {
        cudaGetLastError();
        set_error("no CUDA device visible (%s); this library has no CPU path",
                  e == cudaSuccess ? "count is 0" : cudaGetErrorString(e));
        return RSTQ_E_NODEV;
    }
    rstq_ctx* ctx = new (std::nothrow) rstq_ctx();
    RSTQ_REQUIRE(ctx, RSTQ_E_OOM, "out of host memory");
    ctx->magic = kCtxMagic;
    ctx->devs.resize(ndev);
    int32_t rc = RSTQ_OK;
    for (int i = 0; i < ndev && rc == RSTQ_OK; ++i) {
        DeviceState& ds = ctx->devs[i];
        if (devices[i] < 0 || devices[i] >= n) {
            set_error("CUDA ordinal %d not present (%d devices)", devices[i], n);
            rc = RSTQ_E_NODEV;
            break;
        }
        ds.ordinal = devices[i];
        auto step = [&]() -> int32_t {
            cudaDeviceProp prop;
            RSTQ_CUDA(cudaSetDevice(ds.ordinal));
            RSTQ_CUDA(cudaGetDeviceProperties(&prop, ds.ordinal));
            ds.cc = prop.major * 10 + prop.minor;
            RSTQ_REQUIRE(prop.major == 10, RSTQ_E_ARCH,
                         "device %d is sm_%d%d; this library holds sm_100a code only", ds.ordinal,
                         prop.major, prop.minor);
            ds.sm_count = prop.multiProcessorCount;
            ds.l2_bytes = prop.l2CacheSize;
            ds.total_mem = (int64_t)prop.totalGlobalMem;
            RSTQ_CUDA(cudaStreamCreateWithFlags(&ds.own_stream, cudaStreamNonBlocking));
            ds.stream = ds.own_stream;
            ds.partials_bytes = 32ll << 20;
            RSTQ_CUDA(cudaMalloc((void**)&ds.partials, (size_t)ds.partials_bytes));
            ds.counters_len = 1 << 18;
            RSTQ_CUDA(cudaMalloc((void**)&ds.counters, (size_t)ds.counters_len * 4));
            RSTQ_CUDA(cudaMemsetAsync(ds.counters, 0, (size_t)ds.counters_len * 4, ds.stream));
            RSTQ_CUDA(cudaMalloc((void**)&ds.dbg_store, 1024 * 8 * 8));
            RSTQ_CUDA(cudaMalloc((void**)&ds.status, 256));
            RSTQ_CUDA(cudaMemsetAsync(ds.status, 0, 256, ds.stream));
            int32_t r = gemv_configure(ds);
            if (r != RSTQ_OK) return r;
            if ((r = gemm_configure(ds)) != RSTQ_OK) return r;
            RSTQ_CUDA(cudaStreamSynchronize(ds.stream));
            return RSTQ_OK;
        };
        rc = step();
    }
    if (rc != RSTQ_OK) {
        char keep[512];
        strncpy(keep, g_err, sizeof(keep));
        keep[sizeof(keep) - 1] = 0;
        rstq_shutdown(ctx);
        set_error("%s", keep);
        return rc;
    }
    *ctxp = ctx;
    return RSTQ_OK;
}

int32_t rstq_shutdown(rstq_ctx* ctx) {
    if (!ctx) return RSTQ_OK;
    CHECK_CTX(ctx);
    for (auto& kv : ctx->wcache) {
        rstq_weight* w = kv.second;
        if (w) {
            cudaSetDevice(ctx->devs[w->dev].ordinal);
            cudaFree(w->data);
            w->magic = 0;
            delete w;
        }
    }
    ctx->wcache.clear();
    for (auto& ds : ctx->devs) {
        if (ds.ordinal < 0) continue;
        cudaSetDevice(ds.ordinal);
        if (ds.stream) cudaStreamSynchronize(ds.stream);
        for (void* r : ds.retired) cudaFree(r);
        ds.retired.clear();
        if (ds.act_scratch) cudaFree(ds.act_scratch);
        if (ds.gemm_scratch) cudaFree(ds.gemm_scratch);
        if (ds.attn_scratch) cudaFree(ds.attn_scratch);
        if (ds.kq_scratch) cudaFree(ds.kq_scratch);
        if (ds.f_image) cudaFree(ds.f_image);
        if (ds.partials) cudaFree(ds.partials);
        if (ds.counters) cudaFree(ds.counters);
        if (ds.status) cudaFree(ds.status);
        if (ds.dbg_store) cudaFree(ds.dbg_store);
        if (ds.io_dev) cudaFree(ds.io_dev);
        if (ds.pinned) cudaFreeHost(ds.pinned);
        if (ds.own_stream) cudaStreamDestroy(ds.own_stream);
    }
    cudaGetLastError();
    ctx->magic = 0;
    delete ctx;
    return RSTQ_OK;
}

int32_t rstq_gemm_plan(int32_t* plan2, int64_t out, int64_t in, int64_t m, int32_t sm_count) {
    RSTQ_REQUIRE(plan2, RSTQ_E_INVALID, "null argument");
    RSTQ_REQUIRE(out >= 1 && in >= 32 && in % 32 == 0 && m >= 1 && sm_count >= 1, RSTQ_E_SHAPE,
                 "out = %lld, in = %lld, m = %lld, sm_count = %d", (long long)out, (long long)in, (long long)m, sm_count);
    int ntok = 0;
    bool split = false;
    gemm_plan(out, in, m, sm_count, true, 0, &ntok, &split);
    plan2[0] = ntok;
    plan2[1] = split ? 2 : 1;
    return RSTQ_OK;
}

int32_t rstq_decode_plan(int32_t* plan6, int32_t mode, int32_t bits, int64_t out, int64_t in, int64_t m, int32_t act_dtype,
                         int32_t sm_count) {
    RSTQ_REQUIRE(plan6, RSTQ_E_INVALID, "null argument");
    RSTQ_REQUIRE(mode == RSTQ_MODE_A8 || mode == RSTQ_MODE_F, RSTQ_E_INVALID, "unknown mode %d", mode);
    RSTQ_REQUIRE(bits == 4 || bits == 8, RSTQ_E_INVALID, "bits = %d", bits);
    RSTQ_REQUIRE(act_dtype == RSTQ_F32 || act_dtype == RSTQ_BF16, RSTQ_E_INVALID, "unknown activation type");
    RSTQ_REQUIRE(out >= 1 && in >= 32 && in % 32 == 0 && m >= 1 && sm_count >= 1, RSTQ_E_SHAPE,
                 "out = %lld, in = %lld, m = %lld, sm_count = %d", (long long)out, (long long)in, (long long)m, sm_count);
    return decode_plan(mode == RSTQ_MODE_A8 ? 1 : 0, bits, out, in, m, act_dtype, sm_count, plan6);
}

int32_t rstq_sync(rstq_ctx* ctx, int32_t dev) {
    CHECK_CTX(ctx);
    CHECK_DEV(ctx, dev);
    RSTQ_REQUIRE(!ctx->devs[dev].capturing, RSTQ_E_STATE, "cannot synchronise during capture");
    int32_t rc = use_dev(ctx, dev);
    if (rc != RSTQ_OK) return rc;
    DeviceState& ds = ctx->devs[dev];
    int st = 0;
    RSTQ_CUDA(cudaMemcpyAsync(&st, ds.status, 4, cudaMemcpyDeviceToHost, ds.stream));
    RSTQ_CUDA(cudaStreamSynchronize(ds.stream));
    if (st != 0) {
        // the flag is sticky until read: clear it so the context stays usable
        RSTQ_CUDA(cudaMemsetAsync(ds.status, 0, 4, ds.stream));
        // a launch that gave up may have left hand-over flags set: the next launch must not take them
        RSTQ_CUDA(cudaMemsetAsync(ds.counters, 0, (size_t)ds.counters_len * 4, ds.stream));
        RSTQ_CUDA(cudaStreamSynchronize(ds.stream));
        set_error("a time-bounded wait inside a kernel ran out (status %d); results since the "
                  "last rstq_sync are invalid", st);
        return RSTQ_E_WAIT;
    }
    return RSTQ_OK;
}

int32_t rstq_tune(rstq_ctx* ctx, int32_t key, int64_t value) {
    CHECK_CTX(ctx);
    switch (key) {
        case RSTQ_TUNE_GEMM_KERNEL:
            RSTQ_REQUIRE(value == 0 || value == 1, RSTQ_E_INVALID, "GEMM kernel selector 0..1");
            ctx->tune_gemm_kernel = value;
            return RSTQ_OK;
        case RSTQ_TUNE_PDL:
            for (auto& ds : ctx->devs) ds.pdl = value != 0;
            return RSTQ_OK;
        case RSTQ_TUNE_TIMELINE:
            for (auto& ds : ctx->devs) {
                ds.dbg = value ? ds.dbg_store : nullptr;
                ds.dbg_launch = 0;
                if (value && ds.ordinal >= 0 && !ds.capturing) {   // a fresh record: unused rows read as zero
                    RSTQ_CUDA(cudaSetDevice(ds.ordinal));
                    RSTQ_CUDA(cudaMemsetAsync(ds.dbg_store, 0, 1024 * 8 * 8, ds.stream));
                }
            }
            return RSTQ_OK;
        case RSTQ_TUNE_GEMV_PLAN:
            RSTQ_REQUIRE(value >= 0 && value <= 2, RSTQ_E_INVALID, "decode plan selector 0..2");
            for (auto& ds : ctx->devs) ds.gemv_plan = (int)value;
            return RSTQ_OK;
        case RSTQ_TUNE_GEMV_PREFETCH:
            RSTQ_REQUIRE(value >= -1 && value <= (1 << 20), RSTQ_E_INVALID, "prefetch distance -1 (by size), 0..2^20 KB");
            for (auto& ds : ctx->devs) ds.gemv_prefetch_kb = value;
            return RSTQ_OK;
        case RSTQ_TUNE_PROBE:
#if defined(RSTQ_PROBES) && RSTQ_PROBES
            RSTQ_REQUIRE(value >= 0 && value <= 3, RSTQ_E_INVALID, "probe selector 0..3");
            for (auto& ds : ctx->devs) ds.gemv_probe = (int)value;
            return RSTQ_OK;
#else
            RSTQ_REQUIRE(value == 0, RSTQ_E_INVALID, "this library was built without timing probes");
            return RSTQ_OK;
#endif
        case RSTQ_TUNE_PREFETCH_NEXT:
            for (auto& ds : ctx->devs) ds.prefetch_next = value != 0;
            return RSTQ_OK;
        case RSTQ_TUNE_Q4K_UNITS:
            ctx->tune_q4k_units = value != 0;
            return RSTQ_OK;
        case RSTQ_TUNE_Q6K_UNITS:
            ctx->tune_q6k_units = value != 0;
            return RSTQ_OK;
        case RSTQ_TUNE_GEMM_WIDE:
            RSTQ_REQUIRE(value >= 0 && value <= 3, RSTQ_E_INVALID, "256-token tile selector 0..3");
            ctx->tune_gemm_wide = value;
            return RSTQ_OK;
        case RSTQ_TUNE_ACT_IMAGE:
            for (auto& ds : ctx->devs) ds.act_image = value != 0;
            return RSTQ_OK;
        case RSTQ_TUNE_TP_TAIL:
            RSTQ_REQUIRE(value >= 0 && value <= 1024, RSTQ_E_INVALID, "thread blocks for the exchange's tail: 0 (all) .. 1024");
            for (auto& ds : ctx->devs) ds.tp_tail_ctas = (int)value;
            return RSTQ_OK;
        case RSTQ_TUNE_ACT_RING:
            RSTQ_REQUIRE(value >= 0 && value <= 4, RSTQ_E_INVALID, "activation ring selector 0..4");
            for (auto& ds : ctx->devs) ds.act_ring = value;
            return RSTQ_OK;
        case RSTQ_TUNE_FUSE_QUANT:
            for (auto& ds : ctx->devs) ds.fuse_quant = value != 0;
            return RSTQ_OK;
        case RSTQ_TUNE_GEMM_MIN_M:
            RSTQ_REQUIRE(value >= 1, RSTQ_E_INVALID, "threshold must be >= 1");
            ctx->tune_gemm_min_m = value;
            return RSTQ_OK;
        default:
            set_error("unknown tuning key %d", key);
            return RSTQ_E_INVALID;
    }
}

int32_t rstq_timeline_read(rstq_ctx* ctx, int64_t* out, int32_t dev, int64_t n) {
    CHECK_CTX(ctx);
    CHECK_DEV(ctx, dev);
    RSTQ_REQUIRE(out && n >= 0 && n <= 1024 * 8, RSTQ_E_INVALID, "need 0 <= n <= 8192");
    DeviceState& ds = ctx->devs[dev];
    int32_t rc = use_dev(ctx, dev);
    if (rc != RSTQ_OK) return rc;
    RSTQ_CUDA(cudaMemcpyAsync(out, ds.dbg_store, (size_t)n * 8, cudaMemcpyDeviceToHost, ds.stream));
    RSTQ_CUDA(cudaStreamSynchronize(ds.stream));
    return RSTQ_OK;
}

int32_t rstq_device_info(rstq_ctx* ctx, int64_t* out4, int32_t dev) {
    CHECK_CTX(ctx);
    CHECK_DEV(ctx, dev);
    RSTQ_REQUIRE(out4, RSTQ_E_INVALID, "null argument");
    const DeviceState& ds = ctx->devs[dev];
    out4[0] = ds.sm_count;
    out4[1] = ds.l2_bytes;
    out4[2] = ds.total_mem;
    out4[3] = ds.cc;
    return RSTQ_OK;
}

// ---- buffers ---------------------------------------------------------------
int32_t rstq_alloc(rstq_ctx* ctx, rstq_buf** buf, int32_t dev, int64_t bytes) {
    CHECK_CTX(ctx);
    RSTQ_REQUIRE(buf, RSTQ_E_INVALID, "null argument");
    *buf = nullptr;
    CHECK_DEV(ctx, dev);
    RSTQ_REQUIRE(bytes >= 1, RSTQ_E_SHAPE, "bytes = %lld", (long long)bytes);
    RSTQ_REQUIRE(!ctx->devs[dev].capturing, RSTQ_E_STATE, "cannot allocate during graph capture");
    int32_t rc = use_dev(ctx, dev);
    if (rc != RSTQ_OK) return rc;
    void* p = nullptr;
    RSTQ_CUDA(cudaMalloc(&p, (size_t)bytes));
    rstq_buf* b = new (std::nothrow) rstq_buf{kBufMagic, ctx, dev, p, bytes, true};
    if (!b) {
        cudaFree(p);
        set_error("out of host memory");
        return RSTQ_E_OOM;
    }
    *buf = b;
    return RSTQ_OK;
}

int32_t rstq_buf_wrap(rstq_ctx* ctx, rstq_buf** buf, void* device_ptr, int32_t dev, int64_t bytes) {
    CHECK_CTX(ctx);
    RSTQ_REQUIRE(buf, RSTQ_E_INVALID, "null argument");
    *buf = nullptr;
    CHECK_DEV(ctx, dev);
    RSTQ_REQUIRE(device_ptr && bytes > 0, RSTQ_E_INVALID, "need a device address and a positive size");
    RSTQ_REQUIRE(((uintptr_t)device_ptr & 15) == 0, RSTQ_E_ALIGN, "device address must be 16-byte aligned");
    rstq_buf* b = new (std::nothrow) rstq_buf{kBufMagic, ctx, dev, device_ptr, bytes, false};
    RSTQ_REQUIRE(b, RSTQ_E_OOM, "out of host memory");
    *buf = b;
    return RSTQ_OK;
}

int32_t rstq_stream_set(rstq_ctx* ctx, void* stream, int32_t dev) {
    CHECK_CTX(ctx);
    CHECK_DEV(ctx, dev);
    DeviceState& ds = ctx->devs[dev];
    RSTQ_REQUIRE(!ds.capturing, RSTQ_E_STATE, "cannot change the stream during graph capture");
    int32_t rc = use_dev(ctx, dev);
    if (rc != RSTQ_OK) return rc;
    RSTQ_CUDA(cudaStreamSynchronize(ds.stream));
    if (stream) {
        ds.stream = (cudaStream_t)stream;
    } else {
        ds.stream = ds.own_stream;
    }
    return RSTQ_OK;
}

int32_t rstq_free(rstq_buf* buf) {
    if (!buf) return RSTQ_OK;
    RSTQ_REQUIRE(ok_buf(buf), RSTQ_E_INVALID, "invalid buffer handle");
    DeviceState& ds = buf->ctx->devs[buf->dev];
    cudaSetDevice(ds.ordinal);
    if (!ds.capturing) cudaStreamSynchronize(ds.stream);
    if (buf->owned) cudaFree(buf->ptr);
    cudaGetLastError();
    buf->magic = 0;
    delete buf;
    return RSTQ_OK;
}

static int32_t check_range(rstq_buf* buf, const void* host, int64_t offset, int64_t bytes) {
    RSTQ_REQUIRE(ok_buf(buf), RSTQ_E_INVALID, "invalid buffer handle");
    RSTQ_REQUIRE(host || bytes == 0, RSTQ_E_INVALID, "null host pointer");
    RSTQ_REQUIRE(offset >= 0 && bytes >= 0 && offset + bytes <= buf->bytes, RSTQ_E_RANGE,
                 "range [%lld, %lld) outside buffer of %lld bytes", (long long)offset,
                 (long long)(offset + bytes), (long long)buf->bytes);
    return RSTQ_OK;
}

int32_t rstq_upload(rstq_buf* buf, const void* host, int64_t offset, int64_t bytes) {
    int32_t rc = check_range(buf, host, offset, bytes);
    if (rc != RSTQ_OK) return rc;
    DeviceState& ds = buf->ctx->devs[buf->dev];
    RSTQ_REQUIRE(!ds.capturing, RSTQ_E_STATE, "upload during graph capture");
    if ((rc = use_dev(buf->ctx, buf->dev)) != RSTQ_OK) return rc;
    RSTQ_CUDA(cudaMemcpyAsync((char*)buf->ptr + offset, host, (size_t)bytes,
                              cudaMemcpyHostToDevice, ds.stream));
    RSTQ_CUDA(cudaStreamSynchronize(ds.stream));
    return RSTQ_OK;
}

int32_t rstq_download(rstq_buf* buf, void* host, int64_t offset, int64_t bytes) {
    int32_t rc = check_range(buf, host, offset, bytes);
    if (rc != RSTQ_OK) return rc;
    DeviceState& ds = buf->ctx->devs[buf->dev];
    RSTQ_REQUIRE(!ds.capturing, RSTQ_E_STATE, "download during graph capture");
    if ((rc = use_dev(buf->ctx, buf->dev)) != RSTQ_OK) return rc;
    RSTQ_CUDA(cudaMemcpyAsync(host, (const char*)buf->ptr + offset, (size_t)bytes,
                              cudaMemcpyDeviceToHost, ds.stream));
    RSTQ_CUDA(cudaStreamSynchronize(ds.stream));
    return RSTQ_OK;
}

int32_t rstq_memset(rstq_buf* buf, int32_t byte_value, int64_t offset, int64_t bytes) {
    int32_t rc = check_range(buf, buf, offset, bytes);
    if (rc != RSTQ_OK) return rc;
    DeviceState& ds = buf->ctx->devs[buf->dev];
    if ((rc = use_dev(buf->ctx, buf->dev)) != RSTQ_OK) return rc;
    RSTQ_CUDA(cudaMemsetAsync((char*)buf->ptr + offset, byte_value, (size_t)bytes, ds.stream));
    return RSTQ_OK;
}

int32_t rstq_buf_ptr(rstq_buf* buf, void** device_ptr, int64_t* bytes) {
    RSTQ_REQUIRE(ok_buf(buf), RSTQ_E_INVALID, "invalid buffer handle");
    if (device_ptr) *device_ptr = buf->ptr;
    if (bytes) *bytes = buf->bytes;
    return RSTQ_OK;
}

// ---- weights ---------------------------------------------------------------
int32_t rstq_weight_bind(rstq_ctx* ctx, rstq_weight** w, const void* codes, const float* scales,
                         int32_t dev, int64_t out, int64_t in, int32_t format, int32_t layout) {
    return bind_impl(ctx, w, codes, scales, dev, out, in, format, layout, RSTQ_SPLIT_NONE, 0, 1);
}

int32_t rstq_weight_bind_shard(rstq_ctx* ctx, rstq_weight** w, const void* codes,
                               const float* scales, int32_t dev, int64_t out, int64_t in,
                               int32_t format, int32_t layout, int32_t split, int32_t rank,
                               int32_t nranks) {
    return bind_impl(ctx, w, codes, scales, dev, out, in, format, layout, split, rank, nranks);
}

int32_t rstq_weight_bind_q4k(rstq_ctx* ctx, rstq_weight** wout, const void* wq, const float* da, const float* db,
                             const int8_t* aq, const int8_t* bq, int32_t dev, int64_t out, int64_t in) {
    CHECK_CTX(ctx);
    RSTQ_REQUIRE(wout && wq && da && db && aq && bq, RSTQ_E_INVALID, "null argument");
    *wout = nullptr;
    RSTQ_REQUIRE(out >= 1 && in >= 256 && in % 256 == 0, RSTQ_E_SHAPE,
                 "in = %lld must be a positive multiple of 256 and out = %lld >= 1", (long long)in, (long long)out);
    const int64_t nb = in / 32, n = out * nb;
    // per-sub-block scale da*aq and min db*bq: the products the reference forms (in double) before
    // it multiplies by the integer dot and the sub-block sum, rounded to f32 once
    std::vector<float> a((size_t)n), b((size_t)n);
    for (int64_t i = 0; i < n; ++i) {
        a[(size_t)i] = (float)((double)da[i >> 3] * (double)aq[i]);
        b[(size_t)i] = (float)((double)db[i >> 3] * (double)bq[i]);
    }
    rstq_weight* w = nullptr;
    int32_t rc = bind_impl(ctx, &w, wq, a.data(), dev, out, in, RSTQ_FMT_Q4_0, RSTQ_LAYOUT_ROWMAJOR,
                           RSTQ_SPLIT_NONE, 0, 1);
    if (rc != RSTQ_OK) return rc;
    w->zp = 0;  // codes are 0 .. 15 as they stand; the offset is the min term
    DeviceState& ds = ctx->devs[dev];
    cudaError_t e = cudaMalloc((void**)&w->mins, (size_t)n * 4);
    if (e == cudaSuccess) e = cudaMemcpyAsync(w->mins, b.data(), (size_t)n * 4, cudaMemcpyHostToDevice, ds.stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ds.stream);
    if (e != cudaSuccess) {
        w->mins = nullptr;
        rstq_weight_free(w);
        return cuda_fail(e, "Q4_K bind", __FILE__, __LINE__);
    }
    if (ctx->tune_q4k_units) {
        // the minima move into the units (768 B): the decode kernel folds them, no third kernel
        const int64_t kbytes = (w->outp / 32) * w->nb * kUnitBytesQ4K;
        uint8_t* kdata = nullptr;
        e = cudaMalloc((void**)&kdata, (size_t)kbytes);
        if (e == cudaSuccess) {
            rc = launch_q4k_units(ctx, ds, w->data, w->mins, kdata, w->out, w->nb);
            if (rc == RSTQ_OK) e = cudaStreamSynchronize(ds.stream);
        }
        if (e != cudaSuccess || rc != RSTQ_OK) {
            if (kdata) cudaFree(kdata);
            rstq_weight_free(w);
            return rc != RSTQ_OK ? rc : cuda_fail(e, "Q4_K units", __FILE__, __LINE__);
        }
        cudaFree(w->data);
        w->data = kdata;
        w->data_bytes = kbytes;
        w->kq = true;
    }
    *wout = w;
    return RSTQ_OK;
}

int32_t rstq_weight_bind_q6k(rstq_ctx* ctx, rstq_weight** wout, const void* wq, const int8_t* sc, const float* dsup,
                             int32_t dev, int64_t out, int64_t in) {
    CHECK_CTX(ctx);
    RSTQ_REQUIRE(wout && wq && sc && dsup, RSTQ_E_INVALID, "null argument");
    *wout = nullptr;
    RSTQ_REQUIRE(out >= 1 && in >= 256 && in % 256 == 0, RSTQ_E_SHAPE,
                 "in = %lld must be a positive multiple of 256 and out = %lld >= 1", (long long)in, (long long)out);
    const int64_t nb = in / 32, nsb = in / 256;
    const uint8_t* q = (const uint8_t*)wq;
    if (ctx->tune_q6k_units) {
        // Units with a scale per 16 elements (1280 B): the reference's code bytes, one launch.  The codes
        // go through the 8-bit repack as they are (with scales that are then dropped), the 2 * nb scales
        // per row ds * sc (the product the reference forms in double, rounded to f32 once) behind them.
        const int64_t n16 = out * (in / 16);
        std::vector<float> s16((size_t)n16), s32((size_t)(out * nb), 0.0f);
        for (int64_t o = 0; o < out; ++o)
            for (int64_t j = 0; j < in / 16; ++j)
                s16[(size_t)(o * (in / 16) + j)] = (float)((double)dsup[o * nsb + j / 16] * (double)sc[o * (in / 16) + j]);
        rstq_weight* w = nullptr;
        int32_t rc = bind_impl(ctx, &w, q, s32.data(), dev, out, in, RSTQ_FMT_Q8_0, RSTQ_LAYOUT_ROWMAJOR,
                               RSTQ_SPLIT_NONE, 0, 1);
        if (rc != RSTQ_OK) return rc;
        DeviceState& ds = ctx->devs[dev];
        const int64_t kbytes = (w->outp / 32) * w->nb * kUnitBytesQ6K;
        uint8_t* kdata = nullptr;
        float* d16 = nullptr;
        cudaError_t e = cudaMalloc((void**)&kdata, (size_t)kbytes);
        if (e == cudaSuccess) e = cudaMalloc((void**)&d16, (size_t)n16 * 4);
        if (e == cudaSuccess) e = cudaMemcpyAsync(d16, s16.data(), (size_t)n16 * 4, cudaMemcpyHostToDevice, ds.stream);
        if (e == cudaSuccess) {
            rc = launch_q6k_units(ctx, ds, w->data, d16, kdata, out, w->nb);
            if (rc == RSTQ_OK) e = cudaStreamSynchronize(ds.stream);
        }
        if (d16) cudaFree(d16);
        if (e != cudaSuccess || rc != RSTQ_OK) {
            if (kdata) cudaFree(kdata);
            rstq_weight_free(w);
            return rc != RSTQ_OK ? rc : cuda_fail(e, "Q6_K units", __FILE__, __LINE__);
        }
        cudaFree(w->data);
        w->data = kdata;
        w->data_bytes = kbytes;
        w->zp = 32;
        w->pair_out = out;   // marks the format; `out` stays the logical row count
        w->k6 = true;
        *wout = w;
        return RSTQ_OK;
    }
    std::vector<uint8_t> codes((size_t)(2 * out * in));
    std::vector<float> scales((size_t)(2 * out * nb));
    for (int64_t o = 0; o < out; ++o) {
        uint8_t* ra = codes.data() + (2 * o) * in;
        uint8_t* rb = ra + in;
        for (int64_t b = 0; b < nb; ++b) {
            const uint8_t* src = q + o * in + b * 32;
            memcpy(ra + b * 32, src, 16);            // twin A: even sub-block, zero point elsewhere
            memset(ra + b * 32 + 16, 32, 16);
            memset(rb + b * 32, 32, 16);             // twin B: odd sub-block
            memcpy(rb + b * 32 + 16, src + 16, 16);
            const double d = (double)dsup[o * nsb + b / 8];
            scales[(size_t)((2 * o) * nb + b)] = (float)(d * (double)sc[o * (in / 16) + 2 * b]);
            scales[(size_t)((2 * o + 1) * nb + b)] = (float)(d * (double)sc[o * (in / 16) + 2 * b + 1]);
        }
    }
    rstq_weight* w = nullptr;
    int32_t rc = bind_impl(ctx, &w, codes.data(), scales.data(), dev, 2 * out, in, RSTQ_FMT_Q8_0, RSTQ_LAYOUT_ROWMAJOR,
                           RSTQ_SPLIT_NONE, 0, 1);
    if (rc != RSTQ_OK) return rc;
    w->zp = 32;
    w->pair_out = out;
    *wout = w;
    return RSTQ_OK;
}

int32_t rstq_weight_clone(rstq_weight* src, rstq_weight** wout) {
    RSTQ_REQUIRE(wout, RSTQ_E_INVALID, "null argument");
    *wout = nullptr;
    RSTQ_REQUIRE(ok_w(src), RSTQ_E_INVALID, "invalid weight handle");
    rstq_ctx* ctx = src->ctx;
    DeviceState& ds = ctx->devs[src->dev];
    RSTQ_REQUIRE(!ds.capturing, RSTQ_E_STATE, "cannot clone during graph capture");
    int32_t rc = use_dev(ctx, src->dev);
    if (rc != RSTQ_OK) return rc;
    rstq_weight* w = new (std::nothrow) rstq_weight(*src);
    RSTQ_REQUIRE(w, RSTQ_E_OOM, "out of host memory");
    w->data = nullptr;
    w->raw_codes = nullptr;
    w->raw_scales = nullptr;
    w->mins = nullptr;
    const size_t min_bytes = (size_t)(src->out * src->nb * 4);
    cudaError_t e = cudaMalloc((void**)&w->data, (size_t)w->data_bytes);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(w->data, src->data, (size_t)w->data_bytes, cudaMemcpyDeviceToDevice,
                            ds.stream);
    if (e == cudaSuccess && src->mins) e = cudaMalloc((void**)&w->mins, min_bytes);
    if (e == cudaSuccess && src->mins)
        e = cudaMemcpyAsync(w->mins, src->mins, min_bytes, cudaMemcpyDeviceToDevice, ds.stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ds.stream);
    if (e != cudaSuccess) {
        if (w->data) cudaFree(w->data);
        if (w->mins) cudaFree(w->mins);
        delete w;
        return cuda_fail(e, "weight clone", __FILE__, __LINE__);
    }
    w->next_hint = nullptr;
    ctx->live_weights.insert(w);
    *wout = w;
    return RSTQ_OK;
}

int32_t rstq_weight_free(rstq_weight* w) {
    if (!w) return RSTQ_OK;
    RSTQ_REQUIRE(ok_w(w), RSTQ_E_INVALID, "invalid weight handle");
    DeviceState& ds = w->ctx->devs[w->dev];
    w->ctx->live_weights.erase(w);
    if (ds.last_decode_w == w) ds.last_decode_w = nullptr;
    cudaSetDevice(ds.ordinal);
    if (!ds.capturing) cudaStreamSynchronize(ds.stream);
    cudaFree(w->data);
    if (w->raw_codes) cudaFree(w->raw_codes);
    if (w->raw_scales) cudaFree(w->raw_scales);
    if (w->mins) cudaFree(w->mins);
    cudaGetLastError();
    w->magic = 0;
    delete w;
    return RSTQ_OK;
}

int32_t rstq_weight_info(rstq_weight* w, int64_t* out6) {
    RSTQ_REQUIRE(ok_w(w), RSTQ_E_INVALID, "invalid weight handle");
    RSTQ_REQUIRE(out6, RSTQ_E_INVALID, "null argument");
    out6[0] = w->pair_out ? w->pair_out : w->out;
    out6[1] = w->in;
    out6[2] = w->pair_out ? 6 : w->bits;
    out6[3] = w->data_bytes + (w->mins && !w->kq ? w->out * w->nb * 4 : 0);
    // Q4_K as the reference stores it: nibbles, da + db per super-block, aq + bq per sub-block
    out6[4] = w->mins ? w->out * w->in / 2 + w->out * (w->in / 256) * 8 + w->out * w->nb * 2
                      : w->out * w->in * w->bits / 8 + w->out * w->nb * 4;
    // Q6_K as the reference stores it: a byte per code, an int8 scale per 16, an f32 per 256
    if (w->pair_out) out6[4] = w->pair_out * (w->in + w->in / 16 + (w->in / 256) * 4);
    out6[5] = w->dev;
    return RSTQ_OK;
}

// ---- device-resident ops ----------------------------------------------------
static int32_t need_bytes(rstq_buf* b, int64_t bytes, const char* name) {
    RSTQ_REQUIRE(ok_buf(b), RSTQ_E_INVALID, "invalid buffer handle for %s", name);
    RSTQ_REQUIRE(b->bytes >= bytes, RSTQ_E_RANGE, "%s holds %lld bytes, call needs %lld", name,
                 (long long)b->bytes, (long long)bytes);
    RSTQ_REQUIRE(((uintptr_t)b->ptr & 15) == 0, RSTQ_E_ALIGN, "%s is not 16-byte aligned", name);
    return RSTQ_OK;
}

int32_t rstq_quant_act_i8(rstq_ctx* ctx, rstq_buf* x, rstq_buf* xq, rstq_buf* xs, rstq_buf* xsum,
                          int64_t M, int64_t in) {
    CHECK_CTX(ctx);
    RSTQ_REQUIRE(M >= 1 && in >= 32 && in % 32 == 0, RSTQ_E_SHAPE,
                 "M = %lld, in = %lld (in must be a multiple of 32)", (long long)M, (long long)in);
    const int64_t nb = in / 32;
    int32_t rc;
    if ((rc = need_bytes(x, M * in * 4, "x")) != RSTQ_OK) return rc;
    if ((rc = need_bytes(xq, M * in, "xq")) != RSTQ_OK) return rc;
    if ((rc = need_bytes(xs, M * nb * 4, "xs")) != RSTQ_OK) return rc;
    if (xsum && (rc = need_bytes(xsum, M * nb * 4, "xsum")) != RSTQ_OK) return rc;
    RSTQ_REQUIRE(x->dev == xq->dev && x->dev == xs->dev && (!xsum || xsum->dev == x->dev),
                 RSTQ_E_DEVICE, "buffers live on different devices");
    if ((rc = use_dev(ctx, x->dev)) != RSTQ_OK) return rc;
    return launch_quant_act_i8(ctx, ctx->devs[x->dev], (const float*)x->ptr, (int8_t*)xq->ptr,
                               (float*)xs->ptr, xsum ? (int32_t*)xsum->ptr : nullptr, M, in);
}

int32_t rstq_quant_act_q8k(rstq_ctx* ctx, rstq_buf* x, rstq_buf* xq, rstq_buf* xs, rstq_buf* bsums, int64_t rows,
                           int64_t in, int32_t sub) {
    CHECK_CTX(ctx);
    RSTQ_REQUIRE(rows >= 1 && in >= 256 && in % 256 == 0, RSTQ_E_SHAPE,
                 "rows = %lld, in = %lld (in must be a multiple of 256)", (long long)rows, (long long)in);
    RSTQ_REQUIRE(sub == 16 || sub == 32, RSTQ_E_INVALID, "sub-block of %d elements (16 or 32)", sub);
    int32_t rc;
    if ((rc = need_bytes(x, rows * in * 4, "x")) != RSTQ_OK) return rc;
    if ((rc = need_bytes(xq, rows * in, "xq")) != RSTQ_OK) return rc;
    if ((rc = need_bytes(xs, rows * (in / 256) * 4, "xs")) != RSTQ_OK) return rc;
    if ((rc = need_bytes(bsums, rows * (in / sub) * 4, "bsums")) != RSTQ_OK) return rc;
    RSTQ_REQUIRE(x->dev == xq->dev && x->dev == xs->dev && x->dev == bsums->dev, RSTQ_E_DEVICE,
                 "buffers live on different devices");
    if ((rc = use_dev(ctx, x->dev)) != RSTQ_OK) return rc;
    return launch_quant_act_q8k(ctx, ctx->devs[x->dev], (const float*)x->ptr, (int8_t*)xq->ptr, (float*)xs->ptr,
                                nullptr, (int32_t*)bsums->ptr, rows, in, sub);
}

int32_t rstq_qmatmul(rstq_ctx* ctx, rstq_weight* w, rstq_buf* x, rstq_buf* y, int64_t M,
                     int32_t act_dtype, int32_t out_dtype, int32_t mode) {
    CHECK_CTX(ctx);
    RSTQ_REQUIRE(ok_w(w) && w->ctx == ctx, RSTQ_E_INVALID, "invalid weight handle");
    RSTQ_REQUIRE(M >= 1, RSTQ_E_SHAPE, "M = %lld", (long long)M);
    RSTQ_REQUIRE(act_dtype == RSTQ_F32 || act_dtype == RSTQ_BF16, RSTQ_E_INVALID, "bad act dtype");
    RSTQ_REQUIRE(out_dtype == RSTQ_F32 || out_dtype == RSTQ_BF16, RSTQ_E_INVALID, "bad out dtype");
    RSTQ_REQUIRE(mode == RSTQ_MODE_F || mode == RSTQ_MODE_A8, RSTQ_E_INVALID, "bad mode");
    int32_t rc;
    if ((rc = need_bytes(x, M * w->in * (act_dtype == RSTQ_F32 ? 4 : 2), "x")) != RSTQ_OK) return rc;
    if ((rc = need_bytes(y, M * (w->pair_out ? w->pair_out : w->out) * (out_dtype == RSTQ_F32 ? 4 : 2), "y")) != RSTQ_OK)
        return rc;
    RSTQ_REQUIRE(x->dev == w->dev && y->dev == w->dev, RSTQ_E_DEVICE,
                 "weight and buffers live on different devices");
    if ((rc = use_dev(ctx, w->dev)) != RSTQ_OK) return rc;
    return matmul_device(ctx, w, x->ptr, y->ptr, M, act_dtype, out_dtype, mode);
}

int32_t rstq_qmatmul_prequant(rstq_ctx* ctx, rstq_weight* w, rstq_buf* xq, rstq_buf* xs,
                              rstq_buf* xsum, rstq_buf* y, int64_t M) {
    CHECK_CTX(ctx);
    RSTQ_REQUIRE(ok_w(w) && w->ctx == ctx, RSTQ_E_INVALID, "invalid weight handle");
    RSTQ_REQUIRE(M >= 1, RSTQ_E_SHAPE, "M = %lld", (long long)M);
    int32_t rc;
    if (w->pair_out) {
        // qmatmul-q6k-dp4a! (src/raster/quant/kernels_k.clj:270-300): q8_K activations, xs per super-block,
        // bsums per 16-element sub-block (rstq_quant_act_q8k with sub = 16 produces exactly these)
        RSTQ_REQUIRE(xsum, RSTQ_E_INVALID, "a Q6_K weight needs the sub-block sums");
        const int64_t nsb = w->in / 256;
        if ((rc = need_bytes(xq, M * w->in, "xq")) != RSTQ_OK) return rc;
        if ((rc = need_bytes(xs, M * nsb * 4, "xs")) != RSTQ_OK) return rc;
        if ((rc = need_bytes(xsum, M * (w->in / 16) * 4, "bsums")) != RSTQ_OK) return rc;
        if ((rc = need_bytes(y, M * w->pair_out * 4, "y")) != RSTQ_OK) return rc;
        RSTQ_REQUIRE(xq->dev == w->dev && xs->dev == w->dev && y->dev == w->dev && xsum->dev == w->dev,
                     RSTQ_E_DEVICE, "weight and buffers live on different devices");
        if ((rc = use_dev(ctx, w->dev)) != RSTQ_OK) return rc;
        DeviceState& dsk = ctx->devs[w->dev];
        ActScratch s;
        if ((rc = act_scratch(dsk, M, w->in, &s)) != RSTQ_OK) return rc;
        if (w->k6) {   // the sums per 16 go to the kernel as they are; the scales per super-block are spread over the blocks
            if ((rc = launch_expand_scales(ctx, dsk, (const float*)xs->ptr, s.xs, M * w->nb)) != RSTQ_OK) return rc;
            return run_a8(ctx, w, (const int8_t*)xq->ptr, s.xs, (const int32_t*)xsum->ptr, (float*)y->ptr, M, nullptr, nullptr,
                          dsk.act_image ? s.img : nullptr);
        }
        if ((rc = dev_reserve(dsk, &dsk.kq_scratch, &dsk.kq_scratch_bytes, M * w->out * 4)) != RSTQ_OK) return rc;
        if ((rc = launch_q6k_prep(ctx, dsk, (const float*)xs->ptr, (const int32_t*)xsum->ptr, s.xs, s.xsum,
                                  M * w->nb)) != RSTQ_OK)
            return rc;
        if ((rc = run_a8(ctx, w, (const int8_t*)xq->ptr, s.xs, s.xsum, (float*)dsk.kq_scratch, M)) != RSTQ_OK) return rc;
        return launch_pair_sum(ctx, dsk, (const float*)dsk.kq_scratch, (float*)y->ptr, M, w->pair_out);
    }
    if (w->mins) {
        // qmatmul-q4k-dp4a! (src/raster/quant/kernels_k.clj:195-237): q8_K activations, xs per
        // super-block, bsums per 32-element sub-block
        const int64_t nsb = w->in / 256;
        RSTQ_REQUIRE(xsum, RSTQ_E_INVALID, "a Q4_K weight needs the sub-block sums");
        if ((rc = need_bytes(xq, M * w->in, "xq")) != RSTQ_OK) return rc;
        if ((rc = need_bytes(xs, M * nsb * 4, "xs")) != RSTQ_OK) return rc;
        if ((rc = need_bytes(xsum, M * w->nb * 4, "bsums")) != RSTQ_OK) return rc;
        if ((rc = need_bytes(y, M * w->out * 4, "y")) != RSTQ_OK) return rc;
        RSTQ_REQUIRE(xq->dev == w->dev && xs->dev == w->dev && y->dev == w->dev && xsum->dev == w->dev,
                     RSTQ_E_DEVICE, "weight and buffers live on different devices");
        if ((rc = use_dev(ctx, w->dev)) != RSTQ_OK) return rc;
        DeviceState& dsk = ctx->devs[w->dev];
        ActScratch s;
        if ((rc = act_scratch(dsk, M, w->in, &s)) != RSTQ_OK) return rc;
        if ((rc = launch_expand_scales(ctx, dsk, (const float*)xs->ptr, s.xs, M * w->nb)) != RSTQ_OK) return rc;
        return run_q4k(ctx, w, (const int8_t*)xq->ptr, s.xs, (const int32_t*)xsum->ptr, (float*)y->ptr, M,
                       dsk.act_image ? s.img : nullptr);
    }
    if ((rc = need_bytes(xq, M * w->in, "xq")) != RSTQ_OK) return rc;
    if ((rc = need_bytes(xs, M * w->nb * 4, "xs")) != RSTQ_OK) return rc;
    if (xsum && (rc = need_bytes(xsum, M * w->nb * 4, "xsum")) != RSTQ_OK) return rc;
    if ((rc = need_bytes(y, M * w->out * 4, "y")) != RSTQ_OK) return rc;
    RSTQ_REQUIRE(xq->dev == w->dev && xs->dev == w->dev && y->dev == w->dev &&
                     (!xsum || xsum->dev == w->dev),
                 RSTQ_E_DEVICE, "weight and buffers live on different devices");
    if ((rc = use_dev(ctx, w->dev)) != RSTQ_OK) return rc;
    DeviceState& ds = ctx->devs[w->dev];
    const int32_t* sums = xsum ? (const int32_t*)xsum->ptr : nullptr;
    ActScratch s{};
    if (!sums) {
        if ((rc = act_scratch(ds, M, w->in, &s)) != RSTQ_OK) return rc;
    } else if (M >= 1 && M <= 16 && ds.act_image) {
        if (act_scratch(ds, M, w->in, &s) != RSTQ_OK) s = ActScratch{};   // no room to be had now (a capture in progress): without the image
    }
    if (!sums) {
        // the stored codes carry a zero point, so the block sums are needed even
        // when the caller's arithmetic (signed x signed) has none
        const int64_t nblocks = M * w->nb;
        block_sum_kernel<<<(unsigned)((nblocks + 127) / 128), 128, 0, ds.stream>>>(
            (const int8_t*)xq->ptr, s.xsum, nblocks);
        ctx->launches++;
        RSTQ_CUDA(cudaGetLastError());
        sums = s.xsum;
    }
    // (2 <= M <= 16: with room for the decode kernel's image of the activations, built when shared memory
    // cannot hold them for all of K beside a ring deep enough)
    return run_a8(ctx, w, (const int8_t*)xq->ptr, (const float*)xs->ptr, sums, (float*)y->ptr, M, nullptr, nullptr,
                  ds.act_image ? s.img : nullptr);
}

// ---- host-array operators -----------------------------------------------------
// A fingerprint of the host arrays (8 samples of 8 bytes spread over the codes, 8 over the
// scales): the cache is keyed by address, and a caller may free a matrix and get the same address
// back for another one of the same shape.  A hit whose fingerprint differs is bound again.
static uint64_t host_fingerprint(const void* codes, int64_t code_bytes, const float* scales, int64_t nscales) {
    uint64_t h = 0x9E3779B97F4A7C15ull;
    auto mix = [&](uint64_t v) { h = (h ^ v) * 0xBF58476D1CE4E5B9ull; h ^= h >> 29; };
    const uint8_t* c = (const uint8_t*)codes;
    const int64_t cw = code_bytes / 8;
    // eight samples of each: every sample is a cache miss on a matrix that was not touched since
    // the last call (about 40 ns apiece), and this runs on every host-array call
    for (int i = 0; i < 8 && cw > 0; ++i) {
        uint64_t v;
        memcpy(&v, c + (cw - 1) * i / 7 * 8, 8);
        mix(v);
    }
    for (int i = 0; i < 8 && nscales > 0; ++i) {
        uint32_t v;
        memcpy(&v, scales + (nscales - 1) * i / 7, 4);
        mix(v);
    }
    return h;
}

static int32_t cached_weight(rstq_ctx* ctx, const void* codes, const float* scales, int64_t in,
                             int64_t out, int fmt, int layout, rstq_weight** w) {
    rstq_ctx::CacheKey key{codes, scales, in, out, fmt, layout};
    const int bits = fmt == RSTQ_FMT_Q4_0 ? 4 : 8;
    const uint64_t fp = host_fingerprint(codes, out * in * bits / 8, scales, out * (in / 32));
    auto it = ctx->wcache.find(key);
    if (it != ctx->wcache.end()) {
        if (it->second->host_fp == fp) {
            *w = it->second;
            return RSTQ_OK;
        }
        rstq_weight_free(it->second);  // same address, other contents: the old matrix is gone
        ctx->wcache.erase(it);
    }
    int32_t rc = bind_impl(ctx, w, codes, scales, 0, out, in, fmt, layout, RSTQ_SPLIT_NONE, 0, 1);
    if (rc != RSTQ_OK) return rc;
    (*w)->host_fp = fp;
    ctx->wcache.emplace(key, *w);
    return RSTQ_OK;
}

// Stage x (x_bytes) to the device, run `body(dev_x, dev_y)`, bring y (y_bytes) back.
extern "C++" {
template <typename Body>
int32_t host_roundtrip(rstq_ctx* ctx, int dev, const void* x, int64_t x_bytes, void* y,
                              int64_t y_bytes, Body body, bool y_write_only = false, bool x_read_once = false) {
    DeviceState& ds = ctx->devs[dev];
    RSTQ_REQUIRE(!ds.capturing, RSTQ_E_STATE, "host-array operators cannot be captured");
    int32_t rc = use_dev(ctx, dev);
    if (rc != RSTQ_OK) return rc;
    const int64_t xa = (x_bytes + 255) & ~255ll, ya = (y_bytes + 255) & ~255ll;
    if ((rc = ensure_pinned(ds, xa + ya)) != RSTQ_OK) return rc;
    if ((rc = dev_reserve(ds, &ds.io_dev, &ds.io_dev_bytes, xa + ya)) != RSTQ_OK) return rc;
    char* hp = (char*)ds.pinned;
    char* dp = (char*)ds.io_dev;
    memcpy(hp, x, (size_t)x_bytes);
    // Small activations are read by the first kernel straight from the pinned host copy (unified
    // addressing makes it device-visible): one PCIe round trip instead of a copy engine launch.  Only
    // where that kernel reads x once (the activation quantizer): the decode kernels stage x in every
    // thread block, which would cross PCIe a hundred times over.
    const bool direct = x_read_once && x_bytes <= 256 * 1024;
    ds.x_on_host = direct;
    if (!direct) RSTQ_CUDA(cudaMemcpyAsync(dp, hp, (size_t)x_bytes, cudaMemcpyHostToDevice, ds.stream));
    // A small result the kernels only write goes straight to the pinned host copy too (posted
    // PCIe writes during the kernel instead of a copy-engine launch after it).
    const bool y_direct = y_write_only && y_bytes <= 64 * 1024;
    rc = body(direct ? (void*)hp : (void*)dp, y_direct ? (void*)(hp + xa) : (void*)(dp + xa));
    ds.x_on_host = false;
    if (rc != RSTQ_OK) return rc;
    if (!y_direct)
        RSTQ_CUDA(cudaMemcpyAsync(hp + xa, dp + xa, (size_t)y_bytes, cudaMemcpyDeviceToHost, ds.stream));
    RSTQ_CUDA(cudaStreamSynchronize(ds.stream));
    memcpy(y, hp + xa, (size_t)y_bytes);
    return RSTQ_OK;
}
}  // extern "C++"

static int32_t qlinear_i8_impl(rstq_ctx* ctx, const float* x, const void* wqi, const float* wsi,
                               float* y, int64_t in, int64_t out, int fmt) {
    CHECK_CTX(ctx);
    RSTQ_REQUIRE(x && wqi && wsi && y, RSTQ_E_INVALID, "null argument");
    RSTQ_REQUIRE(in >= 32 && in % 32 == 0 && out >= 8 && out % 8 == 0, RSTQ_E_SHAPE,
                 "qlinear-i8 contract: in %% 32 == 0 and out %% 8 == 0 (in = %lld, out = %lld)",
                 (long long)in, (long long)out);
    rstq_weight* w = nullptr;
    int32_t rc = cached_weight(ctx, wqi, wsi, in, out, fmt, RSTQ_LAYOUT_STREAM8, &w);
    if (rc != RSTQ_OK) return rc;
    return host_roundtrip(ctx, w->dev, x, in * 4, y, out * 4, [&](void* dx, void* dy) {
        return matmul_device(ctx, w, dx, dy, 1, RSTQ_F32, RSTQ_F32, RSTQ_MODE_A8);
    }, true, true);  // M = 1: the decode kernel stores each result once and never reads y; the quantizer reads x once
}

int32_t rstq_qlinear_i8(rstq_ctx* ctx, const float* x, const void* wqi, const float* wsi, float* y,
                        int64_t in, int64_t out) {
    return qlinear_i8_impl(ctx, x, wqi, wsi, y, in, out, RSTQ_FMT_Q4_0);
}

int32_t rstq_qlinear_i8_q8(rstq_ctx* ctx, const float* x, const void* wqi, const float* wsi,
                           float* y, int64_t in, int64_t out) {
    return qlinear_i8_impl(ctx, x, wqi, wsi, y, in, out, RSTQ_FMT_Q8_0);
}

int32_t rstq_qlinear_q8(rstq_ctx* ctx, const float* x, const void* codes, const float* scales,
                        float* y, int64_t m, int64_t in, int64_t out) {
    CHECK_CTX(ctx);
    RSTQ_REQUIRE(x && codes && scales && y, RSTQ_E_INVALID, "null argument");
    RSTQ_REQUIRE(m >= 1 && out >= 1 && in >= 32 && in % 32 == 0, RSTQ_E_SHAPE,
                 "in=%lld not a multiple of 32 (m = %lld, out = %lld)", (long long)in, (long long)m,
                 (long long)out);
    rstq_weight* w = nullptr;
    int32_t rc = cached_weight(ctx, codes, scales, in, out, RSTQ_FMT_Q8_S, RSTQ_LAYOUT_ROWMAJOR, &w);
    if (rc != RSTQ_OK) return rc;
    return host_roundtrip(ctx, w->dev, x, m * in * 4, y, m * out * 4, [&](void* dx, void* dy) {
        return matmul_device(ctx, w, dx, dy, m, RSTQ_F32, RSTQ_F32, RSTQ_MODE_F);
    });
}

int32_t rstq_qlinear_q8_dx(rstq_ctx* ctx, const float* dy, const void* codes, const float* scales, float* dx,
                           int64_t m, int64_t in, int64_t out) {
    CHECK_CTX(ctx);
    RSTQ_REQUIRE(dy && codes && scales && dx, RSTQ_E_INVALID, "null argument");
    RSTQ_REQUIRE(m >= 1 && out >= 1 && in >= 32 && in % 32 == 0, RSTQ_E_SHAPE,
                 "in=%lld not a multiple of 32 (m = %lld, out = %lld)", (long long)in, (long long)m,
                 (long long)out);
    rstq_weight* w = nullptr;
    int32_t rc = cached_weight(ctx, codes, scales, in, out, RSTQ_FMT_Q8_S, RSTQ_LAYOUT_ROWMAJOR, &w);
    if (rc != RSTQ_OK) return rc;
    DeviceState& ds = ctx->devs[w->dev];
    RSTQ_REQUIRE(!ds.capturing, RSTQ_E_STATE, "host-array operators cannot be captured");
    if ((rc = use_dev(ctx, w->dev)) != RSTQ_OK) return rc;
    if (!w->raw_codes) {  // the transposed product reads W as the reference stores it
        const int64_t cb = out * in, sb = out * (in / 32) * 4;
        RSTQ_CUDA(cudaMalloc((void**)&w->raw_codes, (size_t)cb));
        RSTQ_CUDA(cudaMalloc((void**)&w->raw_scales, (size_t)sb));
        RSTQ_CUDA(cudaMemcpyAsync(w->raw_codes, codes, (size_t)cb, cudaMemcpyHostToDevice, ds.stream));
        RSTQ_CUDA(cudaMemcpyAsync(w->raw_scales, scales, (size_t)sb, cudaMemcpyHostToDevice, ds.stream));
        RSTQ_CUDA(cudaStreamSynchronize(ds.stream));
    }
    return host_roundtrip(ctx, w->dev, dy, m * out * 4, dx, m * in * 4, [&](void* d_dy, void* d_dx) {
        return launch_qlinear_q8_dx(ctx, ds, (const float*)d_dy, w->raw_codes, w->raw_scales, (float*)d_dx, m, in, out);
    });
}

int32_t rstq_qlinear_q8_dx_device(rstq_ctx* ctx, rstq_buf* dy, rstq_buf* codes, rstq_buf* scales, rstq_buf* dx,
                                  int64_t m, int64_t in, int64_t out) {
    CHECK_CTX(ctx);
    RSTQ_REQUIRE(m >= 1 && out >= 1 && in >= 32 && in % 32 == 0, RSTQ_E_SHAPE,
                 "in=%lld not a multiple of 32 (m = %lld, out = %lld)", (long long)in, (long long)m, (long long)out);
    int32_t rc;
    if ((rc = need_bytes(dy, m * out * 4, "dy")) != RSTQ_OK) return rc;
    if ((rc = need_bytes(codes, out * in, "codes")) != RSTQ_OK) return rc;
    if ((rc = need_bytes(scales, out * (in / 32) * 4, "scales")) != RSTQ_OK) return rc;
    if ((rc = need_bytes(dx, m * in * 4, "dx")) != RSTQ_OK) return rc;
    RSTQ_REQUIRE(dy->dev == codes->dev && dy->dev == scales->dev && dy->dev == dx->dev, RSTQ_E_DEVICE,
                 "buffers live on different devices");
    if ((rc = use_dev(ctx, dy->dev)) != RSTQ_OK) return rc;
    return launch_qlinear_q8_dx(ctx, ctx->devs[dy->dev], (const float*)dy->ptr, (const int8_t*)codes->ptr,
                                (const float*)scales->ptr, (float*)dx->ptr, m, in, out);
}

int32_t rstq_qmatmul_i8_gemm(rstq_ctx* ctx, const int32_t* xp, const float* xs, const int32_t* wp,
                             const float* ws, float* y, int64_t in, int64_t out, int64_t nrows) {
    CHECK_CTX(ctx);
    RSTQ_REQUIRE(xp && xs && wp && ws && y, RSTQ_E_INVALID, "null argument");
    RSTQ_REQUIRE(nrows >= 1 && out >= 1 && in >= 32 && in % 32 == 0, RSTQ_E_SHAPE,
                 "in = %lld must be a multiple of 32", (long long)in);
    rstq_weight* w = nullptr;
    int32_t rc = cached_weight(ctx, wp, ws, in, out, RSTQ_FMT_Q8_S, RSTQ_LAYOUT_ROWMAJOR, &w);
    if (rc != RSTQ_OK) return rc;
    DeviceState& ds = ctx->devs[w->dev];
    RSTQ_REQUIRE(!ds.capturing, RSTQ_E_STATE, "host-array operators cannot be captured");
    if ((rc = use_dev(ctx, w->dev)) != RSTQ_OK) return rc;
    const int64_t nb = in / 32;
    const int64_t xq_b = (nrows * in + 255) & ~255ll, xs_b = (nrows * nb * 4 + 255) & ~255ll;
    const int64_t y_b = (nrows * out * 4 + 255) & ~255ll;
    if ((rc = ensure_pinned(ds, xq_b + xs_b + y_b)) != RSTQ_OK) return rc;
    if ((rc = dev_reserve(ds, &ds.io_dev, &ds.io_dev_bytes, xq_b + xs_b + y_b)) != RSTQ_OK) return rc;
    ActScratch s;
    if ((rc = act_scratch(ds, nrows, in, &s)) != RSTQ_OK) return rc;
    char* hp = (char*)ds.pinned;
    char* dp = (char*)ds.io_dev;
    memcpy(hp, xp, (size_t)(nrows * in));
    memcpy(hp + xq_b, xs, (size_t)(nrows * nb * 4));
    RSTQ_CUDA(cudaMemcpyAsync(dp, hp, (size_t)(xq_b + xs_b), cudaMemcpyHostToDevice, ds.stream));
    const int64_t nblocks = nrows * nb;
    block_sum_kernel<<<(unsigned)((nblocks + 127) / 128), 128, 0, ds.stream>>>((const int8_t*)dp,
                                                                              s.xsum, nblocks);
    ctx->launches++;
    RSTQ_CUDA(cudaGetLastError());
    rc = run_a8(ctx, w, (const int8_t*)dp, (const float*)(dp + xq_b), s.xsum,
                (float*)(dp + xq_b + xs_b), nrows);
    if (rc != RSTQ_OK) return rc;
    RSTQ_CUDA(cudaMemcpyAsync(hp + xq_b + xs_b, dp + xq_b + xs_b, (size_t)(nrows * out * 4),
                              cudaMemcpyDeviceToHost, ds.stream));
    RSTQ_CUDA(cudaStreamSynchronize(ds.stream));
    memcpy(y, hp + xq_b + xs_b, (size_t)(nrows * out * 4));
    return RSTQ_OK;
}

int32_t rstq_i8gemv_dp4a(rstq_ctx* ctx, const int32_t* wp, const int32_t* xp, float* y, int64_t kw,
                         int64_t out) {
    CHECK_CTX(ctx);
    RSTQ_REQUIRE(wp && xp && y, RSTQ_E_INVALID, "null argument");
    RSTQ_REQUIRE(kw >= 1 && out >= 1, RSTQ_E_SHAPE, "kw = %lld, out = %lld", (long long)kw,
                 (long long)out);
    DeviceState& ds = ctx->devs[0];
    RSTQ_REQUIRE(!ds.capturing, RSTQ_E_STATE, "host-array operators cannot be captured");
    int32_t rc = use_dev(ctx, 0);
    if (rc != RSTQ_OK) return rc;
    const int64_t w_b = (out * kw * 4 + 255) & ~255ll, x_b = (kw * 4 + 255) & ~255ll;
    const int64_t y_b = (out * 4 + 255) & ~255ll;
    if ((rc = ensure_pinned(ds, x_b + y_b)) != RSTQ_OK) return rc;
    if ((rc = dev_reserve(ds, &ds.io_dev, &ds.io_dev_bytes, w_b + x_b + y_b)) != RSTQ_OK) return rc;
    char* hp = (char*)ds.pinned;
    char* dp = (char*)ds.io_dev;
    memcpy(hp, xp, (size_t)(kw * 4));
    RSTQ_CUDA(cudaMemcpyAsync(dp, wp, (size_t)(out * kw * 4), cudaMemcpyHostToDevice, ds.stream));
    RSTQ_CUDA(cudaMemcpyAsync(dp + w_b, hp, (size_t)(kw * 4), cudaMemcpyHostToDevice, ds.stream));
    const int64_t threads = out * 32;
    i8gemv_dp4a_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, ds.stream>>>(
        (const int32_t*)dp, (const int32_t*)(dp + w_b), (float*)(dp + w_b + x_b), kw, out);
    ctx->launches++;
    RSTQ_CUDA(cudaGetLastError());
    RSTQ_CUDA(cudaMemcpyAsync(hp + x_b, dp + w_b + x_b, (size_t)(out * 4), cudaMemcpyDeviceToHost,
                              ds.stream));
    RSTQ_CUDA(cudaStreamSynchronize(ds.stream));
    memcpy(y, hp + x_b, (size_t)(out * 4));
    return RSTQ_OK;
}

int32_t rstq_qmatmul_host(rstq_ctx* ctx, rstq_weight* w, const void* x, float* y, int64_t M,
                          int32_t act_dtype, int32_t mode) {
    CHECK_CTX(ctx);
    RSTQ_REQUIRE(ok_w(w) && w->ctx == ctx, RSTQ_E_INVALID, "invalid weight handle");
    RSTQ_REQUIRE(x && y, RSTQ_E_INVALID, "null argument");
    RSTQ_REQUIRE(M >= 1, RSTQ_E_SHAPE, "M = %lld", (long long)M);
    RSTQ_REQUIRE(act_dtype == RSTQ_F32 || act_dtype == RSTQ_BF16, RSTQ_E_INVALID, "bad act dtype");
    RSTQ_REQUIRE(mode == RSTQ_MODE_F || mode == RSTQ_MODE_A8, RSTQ_E_INVALID, "bad mode");
    const int64_t xe = act_dtype == RSTQ_F32 ? 4 : 2;
    return host_roundtrip(ctx, w->dev, x, M * w->in * xe, y, M * (w->pair_out ? w->pair_out : w->out) * 4,
                          [&](void* dx, void* dy) {
                              return matmul_device(ctx, w, dx, dy, M, act_dtype, RSTQ_F32, mode);
                          });
}

int32_t rstq_weight_cache_clear(rstq_ctx* ctx) {
    CHECK_CTX(ctx);
    for (auto& kv : ctx->wcache) rstq_weight_free(kv.second);
    ctx->wcache.clear();
    return RSTQ_OK;
}

// ---- graphs / events ----------------------------------------------------------
int32_t rstq_graph_begin(rstq_ctx* ctx, int32_t dev) {
    CHECK_CTX(ctx);
    CHECK_DEV(ctx, dev);
    DeviceState& ds = ctx->devs[dev];
    RSTQ_REQUIRE(!ds.capturing, RSTQ_E_STATE, "capture already in progress");
    int32_t rc = use_dev(ctx, dev);
    if (rc != RSTQ_OK) return rc;
    RSTQ_CUDA(cudaStreamBeginCapture(ds.stream, cudaStreamCaptureModeThreadLocal));
    ds.capturing = true;
    return RSTQ_OK;
}

int32_t rstq_graph_end(rstq_ctx* ctx, rstq_graph** graph, int32_t dev) {
    CHECK_CTX(ctx);
    RSTQ_REQUIRE(graph, RSTQ_E_INVALID, "null argument");
    *graph = nullptr;
    CHECK_DEV(ctx, dev);
    DeviceState& ds = ctx->devs[dev];
    RSTQ_REQUIRE(ds.capturing, RSTQ_E_STATE, "no capture in progress");
    int32_t rc = use_dev(ctx, dev);
    if (rc != RSTQ_OK) return rc;
    ds.capturing = false;
    cudaGraph_t g = nullptr;
    RSTQ_CUDA(cudaStreamEndCapture(ds.stream, &g));
    cudaGraphExec_t exec = nullptr;
    cudaError_t e = cudaGraphInstantiate(&exec, g, 0);
    if (e != cudaSuccess) {
        cudaGraphDestroy(g);
        return cuda_fail(e, "cudaGraphInstantiate", __FILE__, __LINE__);
    }
    size_t nodes = 0;
    cudaGraphGetNodes(g, nullptr, &nodes);
    int64_t kernels = 0;
    if (nodes) {
        std::vector<cudaGraphNode_t> v(nodes);
        cudaGraphGetNodes(g, v.data(), &nodes);
        for (auto n : v) {
            cudaGraphNodeType t;
            if (cudaGraphNodeGetType(n, &t) == cudaSuccess && t == cudaGraphNodeTypeKernel) ++kernels;
        }
    }
    ctx->launches -= kernels;  // recorded, not run: replays count them
    rstq_graph* gr = new (std::nothrow) rstq_graph{kGrfMagic, ctx, dev, g, exec, kernels};
    if (!gr) {
        cudaGraphExecDestroy(exec);
        cudaGraphDestroy(g);
        set_error("out of host memory");
        return RSTQ_E_OOM;
    }
    ds.live_graphs++;
    *graph = gr;
    return RSTQ_OK;
}

int32_t rstq_graph_replay(rstq_graph* graph) {
    RSTQ_REQUIRE(graph && graph->magic == kGrfMagic, RSTQ_E_INVALID, "invalid graph handle");
    rstq_ctx* ctx = graph->ctx;
    int32_t rc = use_dev(ctx, graph->dev);
    if (rc != RSTQ_OK) return rc;
    RSTQ_CUDA(cudaGraphLaunch(graph->exec, ctx->devs[graph->dev].stream));
    ctx->launches += graph->kernels;
    return RSTQ_OK;
}

int32_t rstq_graph_destroy(rstq_graph* graph) {
    if (!graph) return RSTQ_OK;
    RSTQ_REQUIRE(graph->magic == kGrfMagic, RSTQ_E_INVALID, "invalid graph handle");
    DeviceState& ds = graph->ctx->devs[graph->dev];
    cudaSetDevice(ds.ordinal);
    cudaStreamSynchronize(ds.stream);
    cudaGraphExecDestroy(graph->exec);
    cudaGraphDestroy(graph->graph);
    if (--ds.live_graphs <= 0) {   // nothing recorded names the outgrown scratch any more
        ds.live_graphs = 0;
        for (void* r : ds.retired) cudaFree(r);
        ds.retired.clear();
    }
    cudaGetLastError();
    graph->magic = 0;
    delete graph;
    return RSTQ_OK;
}

int32_t rstq_event_create(rstq_ctx* ctx, rstq_event** ev, int32_t dev) {
    CHECK_CTX(ctx);
    RSTQ_REQUIRE(ev, RSTQ_E_INVALID, "null argument");
    *ev = nullptr;
    CHECK_DEV(ctx, dev);
    int32_t rc = use_dev(ctx, dev);
    if (rc != RSTQ_OK) return rc;
    cudaEvent_t e;
    RSTQ_CUDA(cudaEventCreate(&e));
    rstq_event* r = new (std::nothrow) rstq_event{kEvtMagic, ctx, dev, e};
    if (!r) {
        cudaEventDestroy(e);
        set_error("out of host memory");
        return RSTQ_E_OOM;
    }
    *ev = r;
    return RSTQ_OK;
}

int32_t rstq_event_record(rstq_event* ev) {
    RSTQ_REQUIRE(ev && ev->magic == kEvtMagic, RSTQ_E_INVALID, "invalid event handle");
    int32_t rc = use_dev(ev->ctx, ev->dev);
    if (rc != RSTQ_OK) return rc;
    RSTQ_CUDA(cudaEventRecord(ev->ev, ev->ctx->devs[ev->dev].stream));
    return RSTQ_OK;
}

int32_t rstq_event_elapsed_ms(rstq_event* start, rstq_event* stop, float* ms) {
    RSTQ_REQUIRE(start && start->magic == kEvtMagic && stop && stop->magic == kEvtMagic && ms,
                 RSTQ_E_INVALID, "invalid event handle");
    RSTQ_REQUIRE(start->dev == stop->dev, RSTQ_E_DEVICE, "events live on different devices");
    int32_t rc = use_dev(start->ctx, start->dev);
    if (rc != RSTQ_OK) return rc;
    RSTQ_CUDA(cudaEventSynchronize(stop->ev));
    RSTQ_CUDA(cudaEventElapsedTime(ms, start->ev, stop->ev));
    return RSTQ_OK;
}

int32_t rstq_event_destroy(rstq_event* ev) {
    if (!ev) return RSTQ_OK;
    RSTQ_REQUIRE(ev->magic == kEvtMagic, RSTQ_E_INVALID, "invalid event handle");
    cudaSetDevice(ev->ctx->devs[ev->dev].ordinal);
    cudaEventDestroy(ev->ev);
    cudaGetLastError();
    ev->magic = 0;
    delete ev;
    return RSTQ_OK;
}

int32_t rstq_launch_count(rstq_ctx* ctx, int64_t* count) {
    CHECK_CTX(ctx);
    RSTQ_REQUIRE(count, RSTQ_E_INVALID, "null argument");
    *count = ctx->launches;
    return RSTQ_OK;
}

}  // extern "C"
