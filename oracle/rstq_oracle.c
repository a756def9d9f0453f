/*
 * TEST INFRASTRUCTURE -- NOT PART OF THE PRODUCT.
 *
 * CPU restatement, in plain scalar C, of the quantized-matmul arithmetic of
 * replikativ/raster.  Only tests, the smoke check and the CPU-baseline leg of
 * the benchmark may load this file's shared object; the CUDA library never does.
 *
 * Every function follows one reference function and names it (paths are
 * relative to the reference project root).  The reference ships no binary
 * fixtures for this path; its own tests are seeded generators plus properties
 * (known dp4a answers, layout sizes, tile == single-column dot, codec
 * invariants, rounding rule).  tests/test_oracle_pins.py re-creates each of
 * those against this file, so parity is pinned by the reference's own tests
 * restated, not by outputs of the reference run here (no JVM on this machine).
 *
 * Conventions: W is row-major [out, in]; a block is 32 consecutive K elements
 * of one row; nb = in / 32; all packing is little-endian.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

/* Java Math.round(double): nearest integer, ties toward +infinity, computed on
 * the exact value (test/raster/compiler/backend/cpu/aot_test.clj:119-128 pins
 * the half-up rule).  v - floor(v) is exact for |v| < 2^52. */
ORC_API int64_t orc_jround(double v) {
    double f = floor(v);
    double r = v - f;
    return (int64_t)f + (r >= 0.5 ? 1 : 0);
}

static inline int64_t clampi(int64_t v, int64_t lo, int64_t hi) {
    return v < lo ? lo : (v > hi ? hi : v);
}

/* ------------------------------------------------------------------------
 * Weight codec: src/raster/compiler/backend/cpu/quant.clj:42-70
 * (format rows q4-0 :27-31 = bits 4 / zp 8 / nibble pack, q8-0 :33-39 =
 * bits 8 / zp 128 / byte-direct).  Flat array, len % 32 == 0.
 * Per block: v = signed element of largest magnitude (first on ties),
 * d = v / (-zp), id = d == 0 ? 0 : 1/d,
 * q(x) = clamp(jround(x*id) + zp, 0, 2^bits - 1), ws = (float)d.
 * nibble pack: byte k = q(w[k]) | q(w[k+16]) << 4.
 * ---------------------------------------------------------------------- */
ORC_API void orc_quantize_weight(const float* w, int64_t len, int bits, int zp,
                                 uint8_t* wq, float* ws) {
    const int64_t nb = len / 32;
    const int64_t qmax = (1 << bits) - 1;
    for (int64_t b = 0; b < nb; ++b) {
        const float* blk = w + b * 32;
        double amax = 0.0, v = 0.0;
        for (int j = 0; j < 32; ++j) {
            double ax = (double)fabsf(blk[j]);
            if (ax > amax) { amax = ax; v = (double)blk[j]; }
        }
        double d = v / (double)(-zp);
        double id = (d == 0.0) ? 0.0 : 1.0 / d;
        ws[b] = (float)d;
        if (bits == 4) {
            for (int k = 0; k < 16; ++k) {
                int64_t lo = clampi(orc_jround((double)blk[k] * id) + zp, 0, qmax);
                int64_t hi = clampi(orc_jround((double)blk[k + 16] * id) + zp, 0, qmax);
                wq[b * 16 + k] = (uint8_t)(lo | (hi << 4));
            }
        } else {
            for (int k = 0; k < 32; ++k)
                wq[b * 32 + k] =
                    (uint8_t)clampi(orc_jround((double)blk[k] * id) + zp, 0, qmax);
        }
    }
}

/* Inverse used by the reference's codec test:
 * test/raster/compiler/backend/cpu/quant_encode_test.clj:9-24
 * w ~= d * (q - zp); low nibble = element k, high nibble = element k + 16. */
ORC_API void orc_dequant_weight(const uint8_t* wq, const float* ws, int64_t len,
                                int bits, int zp, float* out) {
    const int64_t nb = len / 32;
    for (int64_t b = 0; b < nb; ++b) {
        float d = ws[b];
        if (bits == 4) {
            for (int k = 0; k < 16; ++k) {
                int bv = wq[b * 16 + k];
                out[b * 32 + k] = (float)((double)d * (double)((bv & 0xF) - zp));
                out[b * 32 + k + 16] = (float)((double)d * (double)((bv >> 4) - zp));
            }
        } else {
            for (int k = 0; k < 32; ++k)
                out[b * 32 + k] = (float)((double)d * (double)((int)wq[b * 32 + k] - zp));
        }
    }
}

/* ------------------------------------------------------------------------
 * Activation quantizer: src/raster/compiler/backend/cpu/quant.clj:282-305
 * (quantize-act-blocks! / quantize-act-i8; the pooled variant :399-415 slices
 * the same blocks over threads and is bit-identical).
 * Per block: mx = max|x|, d = mx/127 (double), id = d == 0 ? 0 : 1/d,
 * xq = clamp(jround((double)x * id), -127, 127), xs = (float)d, xsum = sum xq.
 * ---------------------------------------------------------------------- */
ORC_API void orc_quantize_act_i8(const float* x, int64_t M, int64_t in, int8_t* xq,
                                 float* xs, int32_t* xsum) {
    const int64_t nblk = M * (in / 32);
    for (int64_t r = 0; r < nblk; ++r) {
        const float* blk = x + r * 32;
        double mx = 0.0;
        for (int j = 0; j < 32; ++j) {
            double a = (double)fabsf(blk[j]);
            if (a > mx) mx = a;
        }
        double d = mx / 127.0;
        double id = (d == 0.0) ? 0.0 : 1.0 / d;
        xs[r] = (float)d;
        int32_t s = 0;
        for (int k = 0; k < 32; ++k) {
            int64_t q = clampi(orc_jround((double)blk[k] * id), -127, 127);
            xq[r * 32 + k] = (int8_t)q;
            s += (int32_t)q;
        }
        xsum[r] = s;
    }
}

/* ------------------------------------------------------------------------
 * Stream layout sizes and repack: src/raster/compiler/core/layout.clj:33-70
 * (descriptor), :246-286 (repack); src/raster/compiler/backend/cpu/quant.clj
 * :317-326 (repack-stream, tile 8).  `tile` = NC output rows interleaved per
 * group; k-group 4; igroups 8; nibble formats pack rows [0,NC/2) in the low
 * nibble and rows [NC/2,NC) in the high nibble.
 * ---------------------------------------------------------------------- */
ORC_API int64_t orc_wqi_len(int tile, int bits, int64_t out, int64_t in) {
    int64_t bpig = (bits == 4) ? (tile / 2) * 4 : tile * 4;
    return (out / tile) * (in / 32) * 8 * bpig;
}
ORC_API int64_t orc_wsi_len(int tile, int64_t out, int64_t in) {
    return (out / tile) * (in / 32) * tile;
}

static inline int src_nibble(const uint8_t* wq, int64_t in, int64_t row, int64_t b, int e) {
    int bv = wq[row * (in / 2) + b * 16 + (e < 16 ? e : e - 16)];
    return e < 16 ? (bv & 0xF) : (bv >> 4);
}

ORC_API void orc_repack_stream(const uint8_t* wq, const float* ws, int64_t out, int64_t in,
                               int bits, int tile, uint8_t* wqi, float* wsi) {
    const int64_t nb = in / 32, ng = out / tile;
    const int half = tile / 2;
    const int bpig = (bits == 4) ? half * 4 : tile * 4;
    for (int64_t g = 0; g < ng; ++g)
        for (int64_t b = 0; b < nb; ++b) {
            for (int ig = 0; ig < 8; ++ig)
                for (int j = 0; j < bpig; ++j) {
                    int64_t idx = ((g * nb + b) * 8 + ig) * bpig + j;
                    int e = ig * 4 + (j % 4);
                    int64_t row = g * tile + j / 4;
                    if (bits == 4) {
                        int lo = src_nibble(wq, in, row, b, e);
                        int hi = src_nibble(wq, in, row + half, b, e);
                        wqi[idx] = (uint8_t)(lo | (hi << 4));
                    } else {
                        wqi[idx] = wq[row * in + b * 32 + e];
                    }
                }
            for (int r = 0; r < tile; ++r)
                wsi[(g * nb + b) * tile + r] = ws[(g * tile + r) * nb + b];
        }
}

/* ------------------------------------------------------------------------
 * Integer dot seams: src/raster/quant/kernels.clj
 *   wi8-dot-q4      :33-46   one Q4_0 block, unsigned nibble x signed int8
 *   wi8-dot         :48-61   unsigned byte x signed int8, `len` elements
 *   wi8-dot-q4-x8   :63-90   8-row tile over the interleaved layout
 *   wi8-dot-q8-x8   :258-278 byte-direct twin
 * ---------------------------------------------------------------------- */
ORC_API int64_t orc_wi8_dot_q4(const uint8_t* wq, int64_t woff, const int8_t* xq, int64_t xoff) {
    int64_t s = 0;
    for (int k = 0; k < 16; ++k) {
        int bv = wq[woff + k];
        s += (int64_t)xq[xoff + k] * (bv & 0xF) + (int64_t)xq[xoff + k + 16] * (bv >> 4);
    }
    return s;
}

ORC_API int64_t orc_wi8_dot(const uint8_t* wq, int64_t woff, const int8_t* xq, int64_t xoff,
                            int64_t len) {
    int64_t s = 0;
    for (int64_t k = 0; k < len; ++k) s += (int64_t)wq[woff + k] * (int64_t)xq[xoff + k];
    return s;
}

ORC_API void orc_wi8_dot_q4_x8(const uint8_t* wqi, int64_t woff, const int8_t* xq, int64_t xoff,
                               int32_t* out8) {
    for (int L = 0; L < 8; ++L) {
        int64_t acc = 0;
        for (int ig = 0; ig < 8; ++ig)
            for (int k = 0; k < 4; ++k) {
                int ni = L * 4 + k; /* position inside the 32 nibbles of this igroup */
                int bv = wqi[woff + ig * 16 + (ni < 16 ? ni : ni - 16)];
                int nib = ni < 16 ? (bv & 0xF) : (bv >> 4);
                acc += (int64_t)xq[xoff + ig * 4 + k] * nib;
            }
        out8[L] = (int32_t)acc;
    }
}

ORC_API void orc_wi8_dot_q8_x8(const uint8_t* wqi, int64_t woff, const int8_t* xq, int64_t xoff,
                               int32_t* out8) {
    for (int L = 0; L < 8; ++L) {
        int64_t acc = 0;
        for (int ig = 0; ig < 8; ++ig)
            for (int k = 0; k < 4; ++k)
                acc += (int64_t)xq[xoff + ig * 4 + k] * (int64_t)wqi[woff + ig * 32 + L * 4 + k];
        out8[L] = (int32_t)acc;
    }
}

/* ------------------------------------------------------------------------
 * Row-major composable GEMV (scalar reference):
 * src/raster/quant/kernels.clj:140-184.  `bits` 4 -> zero point 8 (the
 * reference body); bits 8 uses wi8-dot with zero point 128, the same formula
 * the byte-direct x8 kernel folds.  Double accumulation across blocks, one
 * cast at the end.  Writes rows [o_start, o_start + o_count).
 * ---------------------------------------------------------------------- */
ORC_API void orc_qmatmul_composable(const int8_t* xq, const float* xs, const int32_t* xsum,
                                    const uint8_t* wq, const float* ws, float* y, int64_t in,
                                    int64_t out, int bits, int64_t o_start, int64_t o_count) {
    (void)out;
    const int64_t nb = in / 32;
    const int zp = bits == 4 ? 8 : 128;
    for (int64_t oi = 0; oi < o_count; ++oi) {
        int64_t o = o_start + oi;
        double a = 0.0;
        for (int64_t b = 0; b < nb; ++b) {
            int64_t dot = bits == 4 ? orc_wi8_dot_q4(wq, o * (in / 2) + b * 16, xq, b * 32)
                                    : orc_wi8_dot(wq, o * in + b * 32, xq, b * 32, 32);
            int64_t folded = dot - (int64_t)zp * xsum[b];
            double scale = (double)xs[b] * (double)ws[o * nb + b];
            a += scale * (double)folded;
        }
        y[o] = (float)a;
    }
}

/* ------------------------------------------------------------------------
 * Production CPU GEMV over the 8-row interleaved layout:
 * src/raster/quant/kernels.clj:216-247 (Q4_0, zero point 8) and :308-333
 * (Q8_0, zero point 128).  Accumulator is f32 and is rounded after every
 * block: acc = (float)((double)acc + (xs*ws) * (double)(dot - zp*xsum)).
 * ---------------------------------------------------------------------- */
ORC_API void orc_qmatmul_x8(const int8_t* xq, const float* xs, const int32_t* xsum,
                            const uint8_t* wqi, const float* wsi, float* y, int64_t in,
                            int64_t out, int bits, int64_t g_start, int64_t g_count) {
    (void)out;
    const int64_t nb = in / 32;
    const int zp = bits == 4 ? 8 : 128;
    const int64_t gbytes = bits == 4 ? 128 : 256;
    int32_t out8[8];
    float acc8[8];
    for (int64_t gi = 0; gi < g_count; ++gi) {
        int64_t g = g_start + gi;
        for (int L = 0; L < 8; ++L) acc8[L] = 0.0f;
        for (int64_t b = 0; b < nb; ++b) {
            int64_t woff = (g * nb + b) * gbytes;
            if (bits == 4) orc_wi8_dot_q4_x8(wqi, woff, xq, b * 32, out8);
            else orc_wi8_dot_q8_x8(wqi, woff, xq, b * 32, out8);
            double xsb = (double)xs[b];
            int64_t fold = (int64_t)zp * xsum[b];
            for (int L = 0; L < 8; ++L) {
                double scale = xsb * (double)wsi[(g * nb + b) * 8 + L];
                acc8[L] = (float)((double)acc8[L] + scale * (double)((int64_t)out8[L] - fold));
            }
        }
        for (int L = 0; L < 8; ++L) y[g * 8 + L] = acc8[L];
    }
}

/* The operator: src/raster/quant/op.clj:43-51 (qlinear-i8!, Q4_0 weight) and
 * :81-90 (qlinear-i8-q8!, Q8_0 weight): quantize the activation, then the x8
 * GEMV over all out/8 groups.  y is fully overwritten.  Returns 0, or -1 when
 * the contract (in % 32, out % 8) is broken or memory is short. */
ORC_API int orc_qlinear_i8(const float* x, const uint8_t* wqi, const float* wsi, float* y,
                           int64_t in, int64_t out, int bits) {
    if (in % 32 || out % 8) return -1;
    int64_t nb = in / 32;
    int8_t* xq = (int8_t*)malloc((size_t)in);
    float* xs = (float*)malloc((size_t)nb * sizeof(float));
    int32_t* xsum = (int32_t*)malloc((size_t)nb * sizeof(int32_t));
    if (!xq || !xs || !xsum) { free(xq); free(xs); free(xsum); return -1; }
    orc_quantize_act_i8(x, 1, in, xq, xs, xsum);
    orc_qmatmul_x8(xq, xs, xsum, wqi, wsi, y, in, out, bits, 0, out / 8);
    free(xq); free(xs); free(xsum);
    return 0;
}

/* The reference's own independent scalar oracle:
 * bench/raster/quant_faithfulness.clj:55-73.
 * y[o] = sum_b xs[b]*ws[o,b] * sum_i xq_i * (nibble_i - 8), in double, first
 * `rows` rows of a row-major Q4_0 weight. */
ORC_API void orc_scalar_ref_q4(const uint8_t* wq, const float* ws, const int8_t* xq,
                               const float* xs, int64_t in, int64_t rows, double* y) {
    const int64_t nb = in / 32;
    for (int64_t o = 0; o < rows; ++o) {
        double acc = 0.0;
        for (int64_t b = 0; b < nb; ++b) {
            int64_t ss = 0;
            for (int k = 0; k < 16; ++k) {
                int bv = wq[o * (in / 2) + b * 16 + k];
                ss += (int64_t)xq[b * 32 + k] * ((bv & 0xF) - 8) +
                      (int64_t)xq[b * 32 + k + 16] * ((bv >> 4) - 8);
            }
            acc += ((double)xs[b] * (double)ws[o * nb + b]) * (double)ss;
        }
        y[o] = acc;
    }
}

/* ------------------------------------------------------------------------
 * Signed row-major Q8_0 and the W8A32 linear: src/raster/quant/train.clj
 *   q8-quantize       :34-58   d = max|w|/127, code = clamp(jround(w/d))
 *   dequant-q8-dense  :60-71
 *   qlinear-q8        :77-108  y[m,o] = sum_i (scales*code)*x, products in
 *                              f32, accumulated in double (the JVM literal
 *                              0.0), one cast to f32
 *   qlinear-q8-dx     :110-137 dx[m,i] = sum_o (scales*code)*dy[m,o]
 * ---------------------------------------------------------------------- */
ORC_API void orc_q8_quantize(const float* W, int64_t out, int64_t in, int8_t* codes,
                             float* scales) {
    const int64_t nb = in / 32;
    for (int64_t o = 0; o < out; ++o)
        for (int64_t b = 0; b < nb; ++b) {
            const float* blk = W + o * in + b * 32;
            double mx = 0.0;
            for (int k = 0; k < 32; ++k) {
                double a = fabs((double)blk[k]);
                if (a > mx) mx = a;
            }
            double d = mx / 127.0;
            double id = d > 0.0 ? 1.0 / d : 0.0;
            scales[o * nb + b] = (float)d;
            for (int k = 0; k < 32; ++k)
                codes[o * in + b * 32 + k] =
                    (int8_t)clampi(orc_jround((double)blk[k] * id), -127, 127);
        }
}

ORC_API void orc_dequant_q8_dense(const int8_t* codes, const float* scales, int64_t in,
                                  int64_t out, float* W) {
    const int64_t nb = in / 32;
    for (int64_t o = 0; o < out; ++o)
        for (int64_t i = 0; i < in; ++i)
            W[o * in + i] = (float)((double)scales[o * nb + i / 32] * (double)codes[o * in + i]);
}

ORC_API void orc_qlinear_q8(const float* x, const int8_t* codes, const float* scales, float* y,
                            int64_t m, int64_t in, int64_t out) {
    const int64_t nb = in / 32;
    for (int64_t mi = 0; mi < m; ++mi)
        for (int64_t o = 0; o < out; ++o) {
            double acc = 0.0;
            for (int64_t i = 0; i < in; ++i) {
                float wv = scales[o * nb + i / 32] * (float)codes[o * in + i];
                float p = wv * x[mi * in + i];
                acc += (double)p;
            }
            y[mi * out + o] = (float)acc;
        }
}

ORC_API void orc_qlinear_q8_dx(const float* dy, const int8_t* codes, const float* scales,
                               float* dx, int64_t m, int64_t in, int64_t out) {
    const int64_t nb = in / 32;
    for (int64_t mi = 0; mi < m; ++mi)
        for (int64_t i = 0; i < in; ++i) {
            double acc = 0.0;
            for (int64_t o = 0; o < out; ++o) {
                float wv = scales[o * nb + i / 32] * (float)codes[o * in + i];
                float p = wv * dy[mi * out + o];
                acc += (double)p;
            }
            dx[mi * in + i] = (float)acc;
        }
}

/* ------------------------------------------------------------------------
 * Signed q8_0 packed four codes per little-endian int32:
 * src/raster/quant/pack.clj:55-81 (quantize-one-q8) and :30-33 (nextpad).
 * ---------------------------------------------------------------------- */
ORC_API int64_t orc_nextpad(int64_t in) { return 256 * (int64_t)ceil((double)in / 256.0); }

ORC_API void orc_quantize_one_q8(const float* W, int64_t in, int64_t out, int32_t* wp, float* ws) {
    const int64_t nb = in / 32;
    for (int64_t o = 0; o < out; ++o)
        for (int64_t b = 0; b < nb; ++b) {
            const float* blk = W + o * in + b * 32;
            double mx = 0.0;
            for (int k = 0; k < 32; ++k) {
                double a = fabs((double)blk[k]);
                if (a > mx) mx = a;
            }
            double d = mx / 127.0;
            double id = d > 0.0 ? 1.0 / d : 0.0;
            ws[o * nb + b] = (float)d;
            for (int w = 0; w < 8; ++w) {
                uint32_t word = 0;
                for (int i = 0; i < 4; ++i) {
                    int64_t q = orc_jround((double)blk[w * 4 + i] * id);
                    word |= ((uint32_t)(q & 0xFF)) << (8 * i);
                }
                wp[o * (in / 4) + b * 8 + w] = (int32_t)word;
            }
        }
}

/* ------------------------------------------------------------------------
 * dp4a and the int32-packed kernels: src/raster/par.clj:421-440 (dp4a);
 * src/raster/quant/kernels_k.clj:141-150 (i8gemv-dp4a!), :309-342
 * (quant-act-i8-rows-gpu!), :344-370 (qmatmul-i8-gemm!).
 * ---------------------------------------------------------------------- */
ORC_API int64_t orc_dp4a(int32_t a, int32_t b, int64_t acc) {
    for (int lane = 0; lane < 4; ++lane) {
        int va = (int8_t)((uint32_t)a >> (8 * lane));
        int vb = (int8_t)((uint32_t)b >> (8 * lane));
        acc += (int64_t)va * vb;
    }
    return acc;
}

ORC_API void orc_i8gemv_dp4a(const int32_t* wp, const int32_t* xp, float* y, int64_t kw,
                             int64_t out) {
    for (int64_t o = 0; o < out; ++o) {
        int64_t a = 0;
        for (int64_t k = 0; k < kw; ++k) a = orc_dp4a(wp[o * kw + k], xp[k], a);
        y[o] = (float)a;
    }
}

ORC_API void orc_quant_act_i8_rows(const float* x, int32_t* xp, float* xs, int64_t in,
                                   int64_t nrows) {
    const int64_t nb = in / 32;
    for (int64_t rb = 0; rb < nrows * nb; ++rb) {
        int64_t b = rb % nb, r = rb / nb;
        const float* blk = x + r * in + b * 32;
        float mx = 0.0f; /* the loop maximum stays in the element type */
        for (int k = 0; k < 32; ++k) {
            float v = blk[k], nv = -v;
            float a = v > nv ? v : nv;
            if (a > mx) mx = a;
        }
        double d = (double)mx / 127.0;
        double id = d > 0.0 ? 1.0 / d : 0.0;
        xs[rb] = (float)d;
        for (int w = 0; w < 8; ++w) {
            uint32_t word = 0;
            for (int i = 0; i < 4; ++i) {
                int64_t q = orc_jround((double)blk[w * 4 + i] * id);
                word |= ((uint32_t)(q & 0xFF)) << (8 * i);
            }
            xp[rb * 8 + w] = (int32_t)word;
        }
    }
}

ORC_API void orc_qmatmul_i8_gemm(const int32_t* xp, const float* xs, const int32_t* wp,
                                 const float* ws, float* y, int64_t in, int64_t out,
                                 int64_t nrows) {
    const int64_t nb = in / 32, ni4 = in / 4;
    for (int64_t t = 0; t < nrows; ++t)
        for (int64_t o = 0; o < out; ++o) {
            double a = 0.0;
            for (int64_t b = 0; b < nb; ++b) {
                int64_t dp = 0;
                for (int k = 0; k < 8; ++k)
                    dp = orc_dp4a(wp[o * ni4 + b * 8 + k], xp[t * ni4 + b * 8 + k], dp);
                a += ((double)ws[o * nb + b] * (double)xs[t * nb + b]) * (double)dp;
            }
            y[t * out + o] = (float)a;
        }
}

/* ------------------------------------------------------------------------
 * Float-activation reference ("weights x f32/bf16 activations"):
 * y[m,o] = sum_i dq(W)[o,i] * x[m,i] accumulated in double, with dq per the
 * codec above.  fmt 0: Q4_0 zero point 8 (row-major nibble pack); fmt 1: Q8_0
 * zero point 128 (unsigned byte); fmt 2: signed int8 codes
 * (src/raster/quant/train.clj:60-71).  The staged form sum_b d_b * (sum_t ..)
 * equals the flat one in exact arithmetic
 * (src/raster/compiler/ir/contract_stages.clj:7-24).
 * ---------------------------------------------------------------------- */
ORC_API void orc_matmul_dq_f64(const uint8_t* codes, const float* scales, int fmt, const float* x,
                               int64_t m, int64_t in, int64_t out, double* y) {
    const int64_t nb = in / 32;
    for (int64_t mi = 0; mi < m; ++mi)
        for (int64_t o = 0; o < out; ++o) {
            double acc = 0.0;
            for (int64_t b = 0; b < nb; ++b) {
                double blk = 0.0;
                const float* xb = x + mi * in + b * 32;
                if (fmt == 0) {
                    const uint8_t* c = codes + o * (in / 2) + b * 16;
                    for (int k = 0; k < 16; ++k) {
                        blk += (double)((c[k] & 0xF) - 8) * (double)xb[k];
                        blk += (double)((c[k] >> 4) - 8) * (double)xb[k + 16];
                    }
                } else if (fmt == 1) {
                    const uint8_t* c = codes + o * in + b * 32;
                    for (int k = 0; k < 32; ++k) blk += (double)((int)c[k] - 128) * (double)xb[k];
                } else {
                    const int8_t* c = (const int8_t*)codes + o * in + b * 32;
                    for (int k = 0; k < 32; ++k) blk += (double)c[k] * (double)xb[k];
                }
                acc += (double)scales[o * nb + b] * blk;
            }
            y[mi * out + o] = acc;
        }
}

/* A8 reference for M rows in double (the composable formula applied per
 * activation row); zero point 0 serves the signed x signed prefill kernel. */
ORC_API void orc_matmul_a8_f64(const uint8_t* codes, const float* scales, int fmt,
                               const int8_t* xq, const float* xs, const int32_t* xsum, int64_t m,
                               int64_t in, int64_t out, double* y) {
    const int64_t nb = in / 32;
    const int zp = fmt == 0 ? 8 : (fmt == 1 ? 128 : 0);
    for (int64_t mi = 0; mi < m; ++mi)
        for (int64_t o = 0; o < out; ++o) {
            double acc = 0.0;
            for (int64_t b = 0; b < nb; ++b) {
                const int8_t* xb = xq + mi * in + b * 32;
                int64_t dot;
                if (fmt == 0) dot = orc_wi8_dot_q4(codes, o * (in / 2) + b * 16, xb, 0);
                else if (fmt == 1) dot = orc_wi8_dot(codes, o * in + b * 32, xb, 0, 32);
                else {
                    dot = 0;
                    const int8_t* c = (const int8_t*)codes + o * in + b * 32;
                    for (int k = 0; k < 32; ++k) dot += (int64_t)c[k] * xb[k];
                }
                int64_t folded = dot - (int64_t)zp * xsum[mi * nb + b];
                acc += ((double)xs[mi * nb + b] * (double)scales[o * nb + b]) * (double)folded;
            }
            y[mi * out + o] = acc;
        }
}

/* ---- decode-chain neighbours of the matmul (src/raster/dl/nn.clj) ------------------------------
 * The reference writes these as generic par/map-void! bodies whose literals (0.0, 1.0, 0.5, ...) are
 * doubles, so the element arithmetic is carried in double and stored as float.  Parity for these is
 * unpinned against reference outputs (its tests compare variants of the same op with one another,
 * test/raster/dl/nn_test.clj:659-680, and report ~5e-7 between its own CPU and GPU lowerings). */

/* rms-norm!  nn.clj:497-513: ms = (sum x^2) / features (double accumulator), inv = 1 / sqrt(ms + eps),
 * out = x * inv * (gain_offset + weight). */
ORC_API void orc_rms_norm(const float* x, const float* weight, float* out, int64_t rows, int64_t features,
                          double eps, double gain_offset) {
    for (int64_t r = 0; r < rows; ++r) {
        const float* xr = x + r * features;
        double s = 0.0;
        for (int64_t i = 0; i < features; ++i) s += (double)xr[i] * (double)xr[i];
        const double ms = s / (double)features;
        const double inv = 1.0 / sqrt(ms + eps);
        for (int64_t i = 0; i < features; ++i)
            out[r * features + i] = (float)((double)xr[i] * inv * (gain_offset + (double)weight[i]));
    }
}

/* silu-mul!  nn.clj:200-203: out = g * (1 / (1 + exp(-g))) * up */
ORC_API void orc_silu_mul(const float* gate, const float* up, float* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) {
        const double g = gate[i];
        out[i] = (float)(g * (1.0 / (1.0 + exp(-g))) * (double)up[i]);
    }
}

/* gelu-mul!  nn.clj:208-214: out = 0.5 g (1 + tanh(0.7978845608028654 (g + 0.044715 g g g))) * up */
ORC_API void orc_gelu_mul(const float* gate, const float* up, float* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) {
        const double g = gate[i];
        out[i] = (float)(0.5 * g * (1.0 + tanh(0.7978845608028654 * (g + 0.044715 * g * g * g))) * (double)up[i]);
    }
}

/* residual-add!  nn.clj:217-219: out = a + b (float + float) */
ORC_API void orc_residual_add(const float* a, const float* b, float* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = a[i] + b[i];
}

/* ------------------------------------------------------------------------
 * K-quant super-block formats (the reference's own layout, not GGUF bytes).
 *
 * Q4_K weight codec: src/raster/compiler/backend/cpu/quant.clj:85-150.
 * Super-block = 256 elements = 8 sub-blocks of 32.  Per sub-block a = (max-min)/15
 * and b = min; per super-block dav = max(a)/63, dbv = max|b|/31 (doubles; the stored
 * da, db are their float roundings); aq = clamp(jround(a/dav), 0, 63),
 * bq = clamp(jround(b/dbv), -32, 31); weights are quantized against the QUANTIZED
 * sub scale a' = dav*aq and min b' = dbv*bq: q = clamp(jround((w - b')/a'), 0, 15);
 * byte k of a sub-block = q(w[k]) | q(w[k+16]) << 4.
 * ---------------------------------------------------------------------- */
ORC_API void orc_quantize_weight_q4k(const float* w, int64_t len, uint8_t* wq, float* da, float* db,
                                     int8_t* aq, int8_t* bq) {
    const int64_t nsb = len / 256;
    for (int64_t sb = 0; sb < nsb; ++sb) {
        const float* s = w + sb * 256;
        double as[8], bs[8];
        for (int j = 0; j < 8; ++j) {
            double lo = (double)s[j * 32], hi = lo;
            for (int i = 1; i < 32; ++i) {
                double v = (double)s[j * 32 + i];
                if (v < lo) lo = v;
                if (v > hi) hi = v;
            }
            as[j] = (hi - lo) / 15.0;
            bs[j] = lo;
        }
        double amax = 0.0, bmax = 0.0;
        for (int j = 0; j < 8; ++j) {
            if (as[j] > amax) amax = as[j];
            if (fabs(bs[j]) > bmax) bmax = fabs(bs[j]);
        }
        const double dav = amax / 63.0, dbv = bmax / 31.0;
        const double ida = dav == 0.0 ? 0.0 : 1.0 / dav, idb = dbv == 0.0 ? 0.0 : 1.0 / dbv;
        da[sb] = (float)dav;
        db[sb] = (float)dbv;
        for (int j = 0; j < 8; ++j) {
            const int64_t aqj = clampi(orc_jround(as[j] * ida), 0, 63);
            const int64_t bqj = clampi(orc_jround(bs[j] * idb), -32, 31);
            const double a1 = dav * (double)aqj, b1 = dbv * (double)bqj;
            const double ia1 = a1 == 0.0 ? 0.0 : 1.0 / a1;
            aq[sb * 8 + j] = (int8_t)aqj;
            bq[sb * 8 + j] = (int8_t)bqj;
            for (int k = 0; k < 16; ++k) {
                const int64_t q0 = clampi(orc_jround(((double)s[j * 32 + k] - b1) * ia1), 0, 15);
                const int64_t q1 = clampi(orc_jround(((double)s[j * 32 + k + 16] - b1) * ia1), 0, 15);
                wq[(sb * 256 + j * 32) / 2 + k] = (uint8_t)(q0 | (q1 << 4));
            }
        }
    }
}

/* dequant-q4k, quant.clj:152-170: x = (da*aq)*q + (db*bq), products and sum in double from the
 * stored floats, rounded to float once. */
ORC_API void orc_dequant_q4k(const uint8_t* wq, const float* da, const float* db, const int8_t* aq,
                             const int8_t* bq, int64_t len, float* out) {
    for (int64_t sub = 0; sub < len / 32; ++sub) {
        const double a1 = (double)da[sub / 8] * (double)aq[sub], b1 = (double)db[sub / 8] * (double)bq[sub];
        for (int k = 0; k < 16; ++k) {
            const uint8_t bv = wq[sub * 16 + k];
            out[sub * 32 + k] = (float)(a1 * (double)(bv & 0xF) + b1);
            out[sub * 32 + k + 16] = (float)(a1 * (double)(bv >> 4) + b1);
        }
    }
}

/* quantize-act-q8k, quant.clj:172-193 (and its two-phase device form quant-act-q8k-gpu!,
 * src/raster/quant/kernels_k.clj:93-134, which yields the same codes): one row of `in` floats,
 * per 256 super-block d = max|x|/127, xq = clamp(jround(x/d), -127, 127), xs = (float)d, and
 * bsums = the sum of the codes per sub-block of `sub` elements (32 for Q4_K, 16 for Q6_K). */
ORC_API void orc_quantize_act_q8k(const float* x, int64_t in, int sub, int8_t* xq, float* xs, int32_t* bsums) {
    const int per = 256 / sub;
    for (int64_t sb = 0; sb < in / 256; ++sb) {
        const float* s = x + sb * 256;
        double mx = 0.0;
        for (int i = 0; i < 256; ++i) {
            const double a = (double)fabsf(s[i]);
            if (a > mx) mx = a;
        }
        const double d = mx / 127.0, id = d == 0.0 ? 0.0 : 1.0 / d;
        xs[sb] = (float)d;
        for (int j = 0; j < per; ++j) {
            int32_t t = 0;
            for (int k = 0; k < sub; ++k) {
                const int64_t q = clampi(orc_jround((double)s[j * sub + k] * id), -127, 127);
                xq[sb * 256 + j * sub + k] = (int8_t)q;
                t += (int32_t)q;
            }
            bsums[sb * per + j] = t;
        }
    }
}

/* qmatmul-q4k-composable!, src/raster/quant/kernels_k.clj:15-48 (row dot = q4k-q8k-dot,
 * quant.clj:195-220): y[o] = sum_sb dact[sb] * sum_j ((da*aq_j) * dp_j + (db*bq_j) * bsum_j), dp_j the
 * nibble x int8 dot of one 32-element sub-block, everything after the integer dot in double;
 * y rounded to float once.  y64 (may be null) receives the unrounded sums. */
ORC_API void orc_qmatmul_q4k(const int8_t* xq, const float* xs, const int32_t* bsums, const uint8_t* wq,
                             const float* da, const float* db, const int8_t* aq, const int8_t* bq, float* y,
                             double* y64, int64_t in, int64_t out, int64_t o_start, int64_t o_count) {
    (void)out;
    const int64_t nsb = in / 256, nsub = in / 32, wrow = in / 2;
    for (int64_t oi = 0; oi < o_count; ++oi) {
        const int64_t o = o_start + oi;
        double acc = 0.0;
        for (int64_t sb = 0; sb < nsb; ++sb) {
            const double dav = (double)da[o * nsb + sb], dbv = (double)db[o * nsb + sb], dact = (double)xs[sb];
            double ssum = 0.0;
            for (int j = 0; j < 8; ++j) {
                const int64_t sidx = sb * 8 + j, base = sb * 256 + j * 32;
                const double aj = dav * (double)aq[o * nsub + sidx], bj = dbv * (double)bq[o * nsub + sidx];
                const int64_t dp = orc_wi8_dot_q4(wq, o * wrow + base / 2, xq, base);
                ssum = ssum + aj * (double)dp + bj * (double)bsums[sidx];
            }
            acc += dact * ssum;
        }
        if (y) y[o] = (float)acc;
        if (y64) y64[o] = acc;
    }
}

/* Q6_K weight codec: quant.clj:222-262.  256 = 16 sub-blocks of 16; per sub-block a = max|w|/32,
 * per super-block dv = max(a)/127 (stored as float), sc = clamp(jround(a/dv), 0, 127),
 * q = clamp(jround(w/(dv*sc)) + 32, 0, 63), one unsigned 6-bit code per byte. */
ORC_API void orc_quantize_weight_q6k(const float* w, int64_t len, uint8_t* wq, int8_t* sc, float* ds) {
    for (int64_t sb = 0; sb < len / 256; ++sb) {
        const float* s = w + sb * 256;
        double as[16], amax = 0.0;
        for (int j = 0; j < 16; ++j) {
            double mx = 0.0;
            for (int i = 0; i < 16; ++i) {
                const double a = (double)fabsf(s[j * 16 + i]);
                if (a > mx) mx = a;
            }
            as[j] = mx / 32.0;
            if (as[j] > amax) amax = as[j];
        }
        const double dv = amax / 127.0, idv = dv == 0.0 ? 0.0 : 1.0 / dv;
        ds[sb] = (float)dv;
        for (int j = 0; j < 16; ++j) {
            const int64_t scj = clampi(orc_jround(as[j] * idv), 0, 127);
            const double a1 = dv * (double)scj, ia1 = a1 == 0.0 ? 0.0 : 1.0 / a1;
            sc[sb * 16 + j] = (int8_t)scj;
            for (int k = 0; k < 16; ++k)
                wq[sb * 256 + j * 16 + k] = (uint8_t)clampi(orc_jround((double)s[j * 16 + k] * ia1) + 32, 0, 63);
        }
    }
}

/* dequant-q6k, quant.clj:264-278: x = (ds*sc)*(q - 32). */
ORC_API void orc_dequant_q6k(const uint8_t* wq, const int8_t* sc, const float* ds, int64_t len, float* out) {
    for (int64_t sub = 0; sub < len / 16; ++sub) {
        const double a1 = (double)ds[sub / 16] * (double)sc[sub];
        for (int k = 0; k < 16; ++k) out[sub * 16 + k] = (float)(a1 * (double)((int)wq[sub * 16 + k] - 32));
    }
}

/* qmatmul-q6k-composable!, kernels_k.clj:50-79 (row dot = q6k-q8k-dot, quant.clj:280-304):
 * y[o] = sum_sb ds*dact * sum_j sc_j * (dp_j - 32*bsum_j), 16-element sub-blocks. */
ORC_API void orc_qmatmul_q6k(const int8_t* xq, const float* xs, const int32_t* bsums, const uint8_t* wq,
                             const int8_t* sc, const float* ds, float* y, double* y64, int64_t in, int64_t out,
                             int64_t o_start, int64_t o_count) {
    (void)out;
    const int64_t nsb = in / 256, nsub = in / 16;
    for (int64_t oi = 0; oi < o_count; ++oi) {
        const int64_t o = o_start + oi;
        double acc = 0.0;
        for (int64_t sb = 0; sb < nsb; ++sb) {
            const double dv = (double)ds[o * nsb + sb], dact = (double)xs[sb];
            double ssum = 0.0;
            for (int j = 0; j < 16; ++j) {
                const int64_t sidx = sb * 16 + j, base = sb * 256 + j * 16;
                const int64_t dp = orc_wi8_dot(wq, o * in + base, xq, base, 16);
                ssum += (double)sc[o * nsub + sidx] * (double)(dp - 32 * (int64_t)bsums[sidx]);
            }
            acc += dv * dact * ssum;
        }
        if (y) y[o] = (float)acc;
        if (y64) y64[o] = acc;
    }
}

/* ------------------------------------------------------------------------
 * The attention steps of the decoder layer's decode chain (one token), carried in double and
 * rounded to float once per stored value.
 *
 * rope-pos-gpu! / rope-pos-buf!, src/raster/dl/attention.clj:386-408, :482-499: NeoX rotate-half at
 * absolute position pos; pair (i, i + head_dim/2) of every head turns by pos * exp(-2i/head_dim * ln theta).
 * ---------------------------------------------------------------------- */
ORC_API void orc_rope_pos(const float* x, float* out, int64_t heads, int64_t head_dim, double theta, int64_t pos) {
    const int64_t h2 = head_dim / 2;
    const double ln_theta = log(theta);
    for (int64_t h = 0; h < heads; ++h)
        for (int64_t i = 0; i < h2; ++i) {
            const double freq = exp((-2.0 * (double)i) / (double)head_dim * ln_theta);
            const double ang = (double)pos * freq, c = cos(ang), s = sin(ang);
            const double x0 = (double)x[h * head_dim + i], x1 = (double)x[h * head_dim + i + h2];
            out[h * head_dim + i] = (float)(x0 * c - x1 * s);
            out[h * head_dim + i + h2] = (float)(x1 * c + x0 * s);
        }
}

/* kv-append! / kv-append-buf!, attention.clj:413-416, :501-504: cache[pos*kvrow + i] = src[i]. */
ORC_API void orc_kv_append(const float* src, float* cache, int64_t kvrow, int64_t pos) {
    memcpy(cache + pos * kvrow, src, (size_t)kvrow * sizeof(float));
}

/* gqa-decode-attention-gpu! / -buf!, attention.clj:423-471, :514-575: per query head hq (kv head
 * hq / group): scores = scale * q.k_j over the cache positions, max-subtracted softmax, out = sum_j
 * p_j * v_j.  K / V cache layout [pos][n_kv][head_dim]. */
ORC_API void orc_gqa_decode_attention(const float* q, const float* k, const float* v, float* out, int64_t cache_len,
                                      int64_t n_q, int64_t group, int64_t n_kv, int64_t head_dim, double scale) {
    const int64_t kvstride = n_kv * head_dim;
    double* sc = (double*)malloc((size_t)cache_len * sizeof(double));
    for (int64_t hq = 0; hq < n_q; ++hq) {
        const int64_t hkvb = (hq / group) * head_dim;
        double mx = -1.0e38;
        for (int64_t j = 0; j < cache_len; ++j) {
            double dot = 0.0;
            for (int64_t d = 0; d < head_dim; ++d) dot += (double)q[hq * head_dim + d] * (double)k[j * kvstride + hkvb + d];
            sc[j] = dot * scale;
            if (sc[j] > mx) mx = sc[j];
        }
        double sum = 0.0;
        for (int64_t j = 0; j < cache_len; ++j) {
            sc[j] = exp(sc[j] - mx);
            sum += sc[j];
        }
        const double inv = 1.0 / sum;
        for (int64_t d = 0; d < head_dim; ++d) {
            double a = 0.0;
            for (int64_t j = 0; j < cache_len; ++j) a += sc[j] * inv * (double)v[j * kvstride + hkvb + d];
            out[hq * head_dim + d] = (float)a;
        }
    }
    free(sc);
}
