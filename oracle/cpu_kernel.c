/*
 * TEST / BENCHMARK INFRASTRUCTURE -- NOT PART OF THE PRODUCT.
 *
 * Vectorised, threaded CPU restatement of the reference's production CPU path
 * for the quantized linear operator, used only as the timed CPU baseline and
 * as a second check of the scalar oracle:
 *
 *   operator            src/raster/quant/op.clj:43-51, :81-90
 *   activation quant    src/raster/compiler/backend/cpu/quant.clj:282-305, :399-415
 *   8-row tile          src/raster/quant/kernels.clj:63-90 (Q4), :258-278 (Q8)
 *                       (the reference lowers the tile to an unsigned x signed
 *                        byte multiply-accumulate over the interleaved layout)
 *   per-block fold      src/raster/quant/kernels.clj:216-247, :308-333
 *   slicing over a pool src/raster/quant/kernels.clj:375-393,
 *                       src/raster/compiler/backend/cpu/quant.clj:328-397
 *
 * The reference compiles this path to C at -O3 -march=native and drives it
 * from the JVM; there is no JVM on this machine, so the same arithmetic is
 * compiled directly.  Groups of 8 output rows are split into contiguous chunks
 * of ceil(ng / T) per worker exactly as the reference's pool driver does.
 */
#define _GNU_SOURCE
#include <immintrin.h>
#include <math.h>
#include <pthread.h>
#include <sched.h>
#include <stdatomic.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define CPK_API __attribute__((visibility("default")))

/* ---- u8 x s8 -> s32 four-way multiply-accumulate, best form the host has ---- */
static inline __m256i mac_u8s8(__m256i acc, __m256i u, __m256i s) {
#if defined(__AVX512VNNI__) && defined(__AVX512VL__)
    return _mm256_dpbusd_epi32(acc, u, s);
#elif defined(__AVXVNNI__)
    return _mm256_dpbusd_avx_epi32(acc, u, s);
#else
    __m256i p16 = _mm256_maddubs_epi16(u, s);
    return _mm256_add_epi32(acc, _mm256_madd_epi16(p16, _mm256_set1_epi16(1)));
#endif
}

CPK_API int cpk_isa(void) {
#if defined(__AVX512VNNI__) && defined(__AVX512VL__)
    return 3;
#elif defined(__AVXVNNI__)
    return 2;
#else
    return 1;
#endif
}

/* Eight raw integer column dots of one block, rows of the group in the lanes. */
static inline __m256i tile_q4(const uint8_t* wb, const int8_t* xb) {
    const __m256i nib = _mm256_set1_epi8(0x0F);
    __m256i acc = _mm256_setzero_si256();
    for (int ig = 0; ig < 8; ++ig) {
        __m128i packed = _mm_loadu_si128((const __m128i*)(wb + 16 * ig));
        __m256i both = _mm256_inserti128_si256(_mm256_castsi128_si256(packed),
                                               _mm_srli_epi16(packed, 4), 1);
        int32_t a4;
        memcpy(&a4, xb + 4 * ig, 4);
        acc = mac_u8s8(acc, _mm256_and_si256(both, nib), _mm256_set1_epi32(a4));
    }
    return acc;
}

static inline __m256i tile_q8(const uint8_t* wb, const int8_t* xb) {
    __m256i acc = _mm256_setzero_si256();
    for (int ig = 0; ig < 8; ++ig) {
        __m256i wv = _mm256_loadu_si256((const __m256i*)(wb + 32 * ig));
        int32_t a4;
        memcpy(&a4, xb + 4 * ig, 4);
        acc = mac_u8s8(acc, wv, _mm256_set1_epi32(a4));
    }
    return acc;
}

/* Groups [g0, g0+cnt): acc8 += (xs[b] * wsi[..L]) * (float)(dot[L] - zp * xsum[b]).
 * The reference's compiled fold widens the int lanes to f32 and accumulates in
 * an f32 vector register (its C is built with -ffast-math). */
static void gemv_groups(const int8_t* xq, const float* xs, const int32_t* xsum,
                        const uint8_t* wqi, const float* wsi, float* y, int64_t nb, int bits,
                        int64_t g0, int64_t cnt) {
    const int zp = bits == 4 ? 8 : 128;
    const int64_t gbytes = bits == 4 ? 128 : 256;
    for (int64_t g = g0; g < g0 + cnt; ++g) {
        __m256 acc = _mm256_setzero_ps();
        const uint8_t* wg = wqi + g * nb * gbytes;
        const float* sg = wsi + g * nb * 8;
        for (int64_t b = 0; b < nb; ++b) {
            __m256i dots = bits == 4 ? tile_q4(wg + b * gbytes, xq + b * 32)
                                     : tile_q8(wg + b * gbytes, xq + b * 32);
            __m256i folded = _mm256_sub_epi32(dots, _mm256_set1_epi32(zp * xsum[b]));
            __m256 scale = _mm256_mul_ps(_mm256_set1_ps(xs[b]), _mm256_loadu_ps(sg + b * 8));
#if defined(__FMA__)
            acc = _mm256_fmadd_ps(scale, _mm256_cvtepi32_ps(folded), acc);
#else
            acc = _mm256_add_ps(acc, _mm256_mul_ps(scale, _mm256_cvtepi32_ps(folded)));
#endif
        }
        _mm256_storeu_ps(y + g * 8, acc);
    }
}

static inline int64_t jround(double v) {
    double f = floor(v);
    return (int64_t)f + ((v - f) >= 0.5 ? 1 : 0);
}

static void quant_blocks(const float* x, int8_t* xq, float* xs, int32_t* xsum, int64_t r0,
                         int64_t cnt) {
    for (int64_t r = r0; r < r0 + cnt; ++r) {
        const float* blk = x + r * 32;
        double mx = 0.0;
        for (int j = 0; j < 32; ++j) {
            double a = fabs((double)blk[j]);
            if (a > mx) mx = a;
        }
        double d = mx / 127.0, id = d == 0.0 ? 0.0 : 1.0 / d;
        xs[r] = (float)d;
        int32_t s = 0;
        for (int k = 0; k < 32; ++k) {
            int64_t q = jround((double)blk[k] * id);
            q = q < -127 ? -127 : (q > 127 ? 127 : q);
            xq[r * 32 + k] = (int8_t)q;
            s += (int32_t)q;
        }
        xsum[r] = s;
    }
}

/* ---- persistent pool: caller is worker 0, spin barrier, bounded spin then yield ---- */
typedef struct {
    int nthreads;
    pthread_t* th;
    atomic_long gen;
    atomic_long arrived;
    atomic_int stop;
    /* current task */
    int phase; /* 0 = quantize activation blocks, 1 = gemv groups */
    const float* x;
    int8_t* xq;
    float* xs;
    int32_t* xsum;
    const uint8_t* wqi;
    const float* wsi;
    float* y;
    int64_t in, out;
    int bits;
} cpk_pool;

typedef struct {
    cpk_pool* p;
    int wid;
} worker_arg;

static void run_slice(cpk_pool* p, int wid) {
    int64_t n = p->nthreads;
    if (p->phase == 0) {
        int64_t nb = p->in / 32, chunk = (nb + n - 1) / n, r0 = wid * chunk;
        int64_t cnt = nb - r0 < chunk ? nb - r0 : chunk;
        if (cnt > 0) quant_blocks(p->x, p->xq, p->xs, p->xsum, r0, cnt);
    } else {
        int64_t ng = p->out / 8, chunk = (ng + n - 1) / n, g0 = wid * chunk;
        int64_t cnt = ng - g0 < chunk ? ng - g0 : chunk;
        if (cnt > 0)
            gemv_groups(p->xq, p->xs, p->xsum, p->wqi, p->wsi, p->y, p->in / 32, p->bits, g0,
                        cnt);
    }
}

static void* worker_main(void* argp) {
    worker_arg* a = (worker_arg*)argp;
    cpk_pool* p = a->p;
    int wid = a->wid;
    free(a);
    long seen = 0;
    for (;;) {
        long spins = 0;
        while (atomic_load_explicit(&p->gen, memory_order_acquire) == seen) {
            if (atomic_load(&p->stop)) return NULL;
            if (++spins > 100000) sched_yield();
            else _mm_pause();
        }
        seen = atomic_load_explicit(&p->gen, memory_order_acquire);
        run_slice(p, wid);
        atomic_fetch_add_explicit(&p->arrived, 1, memory_order_release);
    }
}

static void run_phase(cpk_pool* p, int phase) {
    p->phase = phase;
    if (p->nthreads == 1) { run_slice(p, 0); return; }
    atomic_store(&p->arrived, 0);
    atomic_fetch_add_explicit(&p->gen, 1, memory_order_release);
    run_slice(p, 0);
    while (atomic_load_explicit(&p->arrived, memory_order_acquire) < p->nthreads - 1) _mm_pause();
}

CPK_API void* cpk_pool_create(int nthreads) {
    if (nthreads < 1) nthreads = 1;
    cpk_pool* p = (cpk_pool*)calloc(1, sizeof(cpk_pool));
    if (!p) return NULL;
    p->nthreads = nthreads;
    p->th = (pthread_t*)calloc((size_t)nthreads, sizeof(pthread_t));
    for (int w = 1; w < nthreads; ++w) {
        worker_arg* a = (worker_arg*)malloc(sizeof(worker_arg));
        a->p = p;
        a->wid = w;
        pthread_create(&p->th[w], NULL, worker_main, a);
    }
    return p;
}

CPK_API void cpk_pool_destroy(void* pool) {
    cpk_pool* p = (cpk_pool*)pool;
    if (!p) return;
    atomic_store(&p->stop, 1);
    for (int w = 1; w < p->nthreads; ++w) pthread_join(p->th[w], NULL);
    free(p->th);
    free(p);
}

/* y = qlinear_i8(x) over an interleaved (8-row) weight; scratch holds
 * in + 8*(in/32) bytes and is supplied by the caller so the timed region
 * allocates nothing beyond what the reference's op allocates per call. */
CPK_API int cpk_qlinear_i8(void* pool, const float* x, const uint8_t* wqi, const float* wsi,
                           float* y, int64_t in, int64_t out, int bits, void* scratch) {
    cpk_pool* p = (cpk_pool*)pool;
    if (!p || in % 32 || out % 8) return -1;
    int64_t nb = in / 32;
    p->x = x;
    p->xs = (float*)scratch;
    p->xsum = (int32_t*)((char*)scratch + nb * 4);
    p->xq = (int8_t*)((char*)scratch + nb * 8);
    p->wqi = wqi;
    p->wsi = wsi;
    p->y = y;
    p->in = in;
    p->out = out;
    p->bits = bits;
    run_phase(p, 0);
    run_phase(p, 1);
    return 0;
}
