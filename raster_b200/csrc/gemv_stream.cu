// Streaming decode GEMV for sm_100a (M <= 16 per launch).
//
// Arithmetic: mode A8 = qmatmul-q4-x8! / qmatmul-q8-x8!
// (src/raster/quant/kernels.clj:216-247, :308-333: integer block dots,
// zero-point fold, per-block scale), mode F = qlinear-q8
// (src/raster/quant/train.clj:77-108: y = dequant(W) . x).
//
// Work decomposition, built for HBM bandwidth:
//  * The weight is a sequence of U = groups * nb units (mma32 layout) stored in
//    exactly the order they are consumed.  G persistent CTAs (one per SM) each
//    own ONE contiguous range of units, i.e. one contiguous byte range.
//  * A producer warp copies that range into a shared-memory ring with bulk
//    async copies (cp.async.bulk, up to 64 units per copy) that complete on
//    mbarriers; 16 consumer warps each take up to four units of a chunk, read
//    their 16-byte A-fragment slot from shared memory, run the tensor-core
//    block dot (mma.sync) against activations staged once per CTA, and apply
//    the per-block scale to the accumulator fragment in registers.  Bytes in
//    flight per SM are set by the ring depth, not by registers or occupancy.
//  * int4 unpacking is two AND masks per 32-bit word (no shifts): the layout
//    pairs rows r / r+8 in the low / high nibble, the high-nibble rows come out
//    of the tile multiplied by 16 and the factor is undone in the scale.  The
//    zero-point term and the int->float bias ride in the accumulator input of
//    the int8 tile, so the fold is one FADD + one FMUL + one FFMA per value.
//  * Chunks never straddle a 32-row group, so all consumer warps reach a group
//    boundary together: they reduce across warps and store y directly when the
//    CTA covered the whole K range of the group; otherwise the group is cut
//    between neighbouring CTAs: the one holding its head finishes it (its last
//    segment), the ones behind hand their partial sums over as soon as their
//    first segment is done (see hand_over in the kernel).  All CTAs of a launch
//    are resident together (one per SM, G <= #SM); every wait -- mbarrier or
//    hand-over flag -- is time-bounded and reports through a status word
//    instead of hanging.
#include "internal.h"
#include "mma_helpers.cuh"
#include "sync_helpers.cuh"

// Timing probes and the per-chunk stamps of CTA 0 exist only in builds made with -DRSTQ_PROBES=1
// (python -m raster_b200.build --probes); the shipped library carries neither.
#ifndef RSTQ_PROBES
#define RSTQ_PROBES 0
#endif
#if RSTQ_PROBES
#define PROBE(bit) (p.probe & (bit))
#else
#define PROBE(bit) false
#endif

namespace rstq {

#ifndef RSTQ_CW
#define RSTQ_CW 16
#endif
constexpr int kCW = RSTQ_CW;                     // consumer warps (16, 24 or 32: the cross-warp sums fold warps 16.. onto 0..15)
static_assert(kCW >= 16 && kCW <= 32, "the M = 1 reduction reads two partial sums per thread");
constexpr int kConsumers = kCW * 32;
constexpr int kStreamThreads = kConsumers + 32;  // + producer warp
// units per consumer warp per chunk: 4 (40 KB chunks) for 4-bit, 2 (36 KB chunks) for 8-bit
#ifndef RSTQ_UPW4
#define RSTQ_UPW4 4
#endif
#ifndef RSTQ_NSMAX
#define RSTQ_NSMAX 6
#endif
// `bits` of the host-side helpers is the unit kind: 4, 8, or 5 = 4-bit codes with the 32 Q4_K minima behind the scales
//   and 6 = 8-bit codes with a scale per 16 elements (Q6_K: 64 scales behind the codes)
__host__ __device__ constexpr int upw_of(int bits) { return (bits == 8 || bits == 6) ? 2 : RSTQ_UPW4; }
__host__ __device__ constexpr int chunk_units_of(int bits) { return upw_of(bits) * kCW; }
constexpr int kMaxDynSmem = 232448 - 1024;       // 227 KB opt-in limit less the static part
// the in-kernel quantizer holds all of a thread's activations in registers: in <= 3 * 512 * 8
constexpr int kQuantPasses = 3;
constexpr int kQuantMaxIn = kQuantPasses * kConsumers * 8;
static_assert(kGemvMaxM * 32 <= kConsumers, "one output per consumer thread in the hand-over");
static_assert(kQuantMaxIn >= kFusedQuantMaxIn, "the host routes by kFusedQuantMaxIn");
// M = 1: the per-warp partial sums of whole groups are parked in shared memory (kParkStride floats per
// group: [warp][33]) and reduced across warps once per kParkGroups groups, not once per group
constexpr int kParkGroups = 8;
constexpr int kParkStride = kCW * 33;
constexpr int kMagicInt = kActMagicInt;          // bits of 12582912.0f = 2^23 + 2^22
constexpr float kMagicFlt = 12582912.0f;

enum { MODE_F = 0, MODE_A8 = 1 };

struct StreamParams {
    const uint8_t* w;
    const int8_t* xq;     // A8
    const float* xs;
    const int32_t* xsum;
    const void* x;        // F
    void* y;
    float* partials;      // [G][M*32]: slot c = what CTA c hands over (the partial sums of its first segment)
    int* flags;           // [G]: 1 while slot c holds a partial nobody has taken yet; zero between launches
    int* status;          // device status word (0 = ok)
    unsigned long long* dbg;  // optional per-CTA phase timestamps (8 per CTA), or null
    unsigned long long* dbg_fine;  // with dbg: 512 values behind the slots, CTA 0's stamp per wait / chunk / flush
    int64_t in, out;
    int64_t uq, ur;       // units per CTA: CTA c owns uq (+1 if c < ur) units
    int64_t U;            // all units (the last CTA's range is clipped to it)
    int M, nb, G, zp, NS, T, act_dtype, out_dtype;
    int64_t pf_ahead;     // bytes of the CTA's range requested into L2 ahead of the ring (0: none)
    // the weight expected to be streamed by the NEXT launch of this stream (null: unknown): its
    // thread block j will own units [range_begin(j), range_begin(j + 1)) of nx_U, of nx_unit bytes each
    const uint8_t* nx_w;
    int64_t nx_uq, nx_ur, nx_U, nx_pf_units;
    int nx_G, nx_unit;
    int probe;            // timing probes (results invalid): 1 = the producer signals without copying, 2 = the consumers skip the arithmetic
    uint32_t act_off, act2_off, red_off, bar_off;  // byte offsets into dynamic smem (ring at 0)
    // MODE_A8, M > 1: the staged activations as the quantizer wrote them out, an image of what
    // stage_a8 would build (fragments at act_off, scale / sum records at act2_off); the producer
    // thread copies it in with two bulk copies under a barrier of its own.  Null: stage in the kernel.
    const uint8_t* img;
    uint32_t img_b_bytes, img_z_bytes, img_z_off;
    // M > 1 (in mode F also one token of f32), `ring` set: nothing of the image is kept for the whole launch; every ring stage holds,
    // behind its weight chunk, the image's slice for the chunk's K blocks (fragments at act_off, records at
    // act2_off, both counted from the stage), copied by the producer with the chunk.  Shared memory then
    // does not grow with K, at the price of reading the image (from L2) once per 32-row group.
    int ring;
    uint32_t slice1, slice2;   // ring: bytes per K block of the image's two arrays (mode F: one array)
    int cu;                 // units per chunk (M > 1: a multiple of the consumer warps, <= chunk_units_of)
    uint32_t stage_bytes;   // distance between ring stages
    int kq;   // Q4_K units (zero point 0): the staged constant of a block is t = xs * code sum, which the minima multiply
    int k6;   // Q6_K units: xsum holds the code sums per 16 elements (2 per block), a record two constants
    int tp_tail;          // fused exchange: thread blocks that wait for the peers' results and write y (0 = all)
    TpFuse tp;            // tp.nranks == 0: no exchange, results go to y
};

__device__ __forceinline__ void consumer_bar() {
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumers) : "memory");
}

// CTA c owns units [range_begin(c), range_begin(c + 1)): the first ur CTAs get uq + 1.
__host__ __device__ __forceinline__ int64_t range_begin(int64_t c, int64_t uq, int64_t ur) {
    return c * uq + (c < ur ? c : ur);
}
__device__ __forceinline__ int cta_of_unit(int64_t u, int64_t uq, int64_t ur) {
    const int64_t big = ur * (uq + 1);
    return u < big ? (int)(u / (uq + 1)) : (int)(ur + (u - big) / uq);
}

// D(16x8, s32) = A(16x32, u8) * B(32x8, s8) + C
__device__ __forceinline__ void imma_acc(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1,
                                         int c0, int c1, int c2, int c3) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%11,%12,%13};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(c0), "r"(c1), "r"(c2),
          "r"(c3));
}

// ---- activation staging (once per CTA, all of K) ---------------------------------------------
// A8, M == 1: srec [nb][4 tig] uint4 {xq word tig, xq word 4+tig, xs_t bits, c_t}: lane tig
//            folds row gid + 8*tig only (all eight tile columns are the same token), so the
//            record carries that row's constants: for 4-bit codes the rows of odd tig sit in
//            the high nibbles (tile value x16): xs_t = xs/16 and c_t = bias - 16*zp*xsum;
//            otherwise xs_t = xs and c_t = bias - zp*xsum (bias = bits of 2^23 + 2^22).
// A8, M > 1 : sB [nb][M][4 tig] uint2 {xq word tig, xq word 4+tig};
//             plain units: [nb][Mz / 2] records of a token pair (put_act_record), Mz = M rounded up to even;
//             Q4_K units: sxz [nb][Mz] int2 {xs bits, bits of xs * code sum}.
//             (For 2 <= M <= 16 the activation quantizer can write both arrays in this order itself:
//             StreamParams::img, copied in by the producer thread instead of staged here.)
// K-quant units: Q4_K (zero point 0): the constant of a record is t = xs * code sum, which the unit's
//             minima multiply (c_t at M = 1, the second word of sxz otherwise).  Q6_K: xsum holds the
//             code sums per 16 elements; M = 1 records are 32 bytes {.., c of elements 0..15 | c of
//             16..31, 0, 0, 0}, sxz entries int4 {xs bits, zp*sum of 0..15, zp*sum of 16..31, 0}.
template <bool ONECOL, int BITS>
__device__ __forceinline__ void stage_a8(const StreamParams& p, uint8_t* smem, int tid) {
    const int nb = p.nb, M = p.M;
    const uint32_t* xqw = reinterpret_cast<const uint32_t*>(p.xq);
    if (ONECOL) {
        uint4* srec = reinterpret_cast<uint4*>(smem + p.act_off);
        for (int i0 = tid; i0 < nb * 4; i0 += 4 * kConsumers) {
            uint32_t wa[4], wb[4];
            float xs[4];
            int zs[4], zs2[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int i = i0 + j * kConsumers;
                if (i < nb * 4) {
                    const int b = i >> 2, tg = i & 3;
                    wa[j] = xqw[b * 8 + tg];
                    wb[j] = xqw[b * 8 + 4 + tg];
                    xs[j] = p.xs[b];
                    zs[j] = p.k6 ? p.xsum[2 * b] : p.xsum[b];
                    zs2[j] = p.k6 ? p.xsum[2 * b + 1] : 0;
                }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int i = i0 + j * kConsumers;
                if (i < nb * 4) {
                    const bool hi = BITS == 4 && (i & 1);
                    uint4 r;
                    r.x = wa[j];
                    r.y = wb[j];
                    r.z = __float_as_uint(hi ? xs[j] * 0.0625f : xs[j]);
                    r.w = p.kq ? __float_as_uint(xs[j] * (float)zs[j]) : (uint32_t)(kMagicInt - (p.zp * zs[j]) * (hi ? 16 : 1));
                    if (p.k6) {   // 32-byte records: the second half's constant behind the first 16 bytes
                        srec[2 * i] = r;
                        srec[2 * i + 1] = make_uint4((uint32_t)(kMagicInt - p.zp * zs2[j]), 0u, 0u, 0u);
                    } else {
                        srec[i] = r;
                    }
                }
            }
        }
        return;
    }
    uint2* sB = reinterpret_cast<uint2*>(smem + p.act_off);
    int2* sxz = reinterpret_cast<int2*>(smem + p.act2_off);
    const int Mz = (M + 1) & ~1;
    const int64_t row_words = p.in >> 2;
    // The (token, word pair) space is walked flat, four global loads in flight per thread before
    // the first store: the loads of different tokens do not wait for one another.
    constexpr int U = 4;
    const int per = nb * 4, tot = M * per;
    for (int o0 = tid; o0 < tot; o0 += U * kConsumers) {
        uint32_t wa[U], wb[U];
        int dst[U];
#pragma unroll
        for (int j = 0; j < U; ++j) {
            const int o = o0 + j * kConsumers;
            dst[j] = -1;
            if (o < tot) {
                const int c = o / per, i = o - c * per, b = i >> 2, tg = i & 3;
                const uint32_t* xr = xqw + c * row_words;
                wa[j] = xr[b * 8 + tg];
                wb[j] = xr[b * 8 + 4 + tg];
                dst[j] = (b * M + c) * 4 + tg;
            }
        }
#pragma unroll
        for (int j = 0; j < U; ++j)
            if (dst[j] >= 0) sB[dst[j]] = make_uint2(wa[j], wb[j]);
    }
    const int tot2 = nb * Mz;
    if (p.k6) {   // Q6_K: {xs bits, zp * code sum of elements 0..15, of 16..31, 0} per (block, token)
        int4* sxz4 = reinterpret_cast<int4*>(smem + p.act2_off);
        for (int o = tid; o < tot2; o += kConsumers) {
            const int b = o / Mz, c = o - b * Mz;
            int4 v = make_int4(0, 0, 0, 0);
            if (c < M) {
                v.x = __float_as_int(p.xs[(int64_t)c * nb + b]);
                v.y = p.zp * p.xsum[((int64_t)c * nb + b) * 2];
                v.z = p.zp * p.xsum[((int64_t)c * nb + b) * 2 + 1];
            }
            sxz4[o] = v;
        }
        return;
    }
    if (!p.kq) {   // plain units: the pair records
        uint8_t* recs = smem + p.act2_off;
        for (int o = tid; o < tot2; o += kConsumers) {
            const int b = o / Mz, c = o - b * Mz;
            float xs = 0.f;
            int zs = 0;
            if (c < M) {
                xs = p.xs[(int64_t)c * nb + b];
                zs = p.zp * p.xsum[(int64_t)c * nb + b];
            }
            put_act_record(recs, b, Mz, c, xs, zs, BITS == 4);
        }
        return;
    }
    for (int o0 = tid; o0 < tot2; o0 += U * kConsumers) {
        int2 v[U];
#pragma unroll
        for (int j = 0; j < U; ++j) {
            const int o = o0 + j * kConsumers;
            v[j] = make_int2(0, 0);
            if (o < tot2) {
                const int b = o / Mz, c = o - b * Mz;
                if (c < M) {
                    v[j].x = __float_as_int(p.xs[(int64_t)c * nb + b]);
                    const int cs = p.xsum[(int64_t)c * nb + b];
                    v[j].y = __float_as_int(__int_as_float(v[j].x) * (float)cs);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < U; ++j) {
            const int o = o0 + j * kConsumers;
            if (o < tot2) sxz[o] = v[j];
        }
    }
}

// A8, M == 1, the activation quantizer inside the staging pass (quantize-act-blocks!,
// src/raster/compiler/backend/cpu/quant.clj:282-305): per 32-element block d = max|x| / 127 in double,
// id = 1 / d, q = clamp(round_half_up((double)x * id), -127, 127), xs = (float)d, xsum = sum q.
// Thread (b, tig) holds the eight elements its record needs; the four threads of a block are
// neighbouring lanes (two shuffles for the maximum, two for the sum).  The codes come from f32
// arithmetic whenever that provably gives the double result: t = x * fl32(127 / max) is within
// 127 * 2^-22 of the double product, so a t further than 1e-3 from every k + 0.5 rounds the same way;
// anything closer, and blocks whose maximum is zero, tiny, huge or not finite, take the double path.
// xs: fl32(max / 127) equals (float)((double)max / 127.0) for every f32 max -- the quotient of a
// 24-bit integer by 127 cannot sit on a 25-bit midpoint, so rounding through double changes nothing.
__device__ __forceinline__ int quant_exact(float x, double id) {
    const double v = (double)x * id, f = floor(v);
    const int q = (int)f + ((v - f) >= 0.5 ? 1 : 0);
    return max(-127, min(127, q));
}
template <int BITS>
__device__ __forceinline__ void stage_a8_quant(const StreamParams& p, uint8_t* smem, int tid) {
    uint4* srec = reinterpret_cast<uint4*>(smem + p.act_off);
    const int items = p.nb * 4;   // a multiple of 4: the lanes of a block are active together
    const bool bf = p.act_dtype == RSTQ_BF16;
    // every load of the thread is issued before the first use (one trip to L2, not one per pass):
    // kQuantPasses passes of kConsumers items cover in <= kQuantMaxIn
    uint4 raw[kQuantPasses][2];
#pragma unroll
    for (int it = 0; it < kQuantPasses; ++it) {
        const int i = it * kConsumers + tid;
        raw[it][0] = raw[it][1] = make_uint4(0, 0, 0, 0);
        if (i < items) {
            const int b = i >> 2, tg = i & 3;
            if (bf) {
                const uint16_t* xb = reinterpret_cast<const uint16_t*>(p.x) + b * 32 + tg * 4;
                const uint2 lo = *reinterpret_cast<const uint2*>(xb), hi = *reinterpret_cast<const uint2*>(xb + 16);
                raw[it][0] = make_uint4(lo.x << 16, lo.x & 0xFFFF0000u, lo.y << 16, lo.y & 0xFFFF0000u);
                raw[it][1] = make_uint4(hi.x << 16, hi.x & 0xFFFF0000u, hi.y << 16, hi.y & 0xFFFF0000u);
            } else {
                const uint4* xf = reinterpret_cast<const uint4*>(reinterpret_cast<const float*>(p.x) + b * 32 + tg * 4);
                raw[it][0] = xf[0];
                raw[it][1] = xf[4];
            }
        }
    }
#pragma unroll
    for (int it = 0; it < kQuantPasses; ++it) {
        const int i = it * kConsumers + tid;
        if (it * kConsumers + (tid & ~31) >= items) break;   // warp-uniform: the shuffles below need whole warps
        const bool act = i < items;
        const float f[8] = {__uint_as_float(raw[it][0].x), __uint_as_float(raw[it][0].y), __uint_as_float(raw[it][0].z),
                            __uint_as_float(raw[it][0].w), __uint_as_float(raw[it][1].x), __uint_as_float(raw[it][1].y),
                            __uint_as_float(raw[it][1].z), __uint_as_float(raw[it][1].w)};
        float mx = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) mx = fmaxf(mx, fabsf(f[k]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        // f32 shortcut: u = fma(x, 127 / max, 1.5 * 2^23) holds round-to-nearest(x * 127 / max) in its low
        // mantissa bits (two's complement in the low byte); the quotient is 2 ulp accurate, so the
        // product is within 4e-5 of the double one and every element whose remainder is further than
        // 2e-4 from a tie rounds exactly as round_half_up of the double product does.
        uint32_t wa, wb;
        int sum;
        float xs = 0.f;
        bool exact = !(mx >= 1e-30f && mx <= 1e37f);
        if (!exact) {
            const float idf = __fdividef(127.f, mx);
            xs = __fdiv_rn(mx, 127.f);
            uint32_t ub[8];
            float amb = 0.f;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const float u = fmaf(f[k], idf, kMagicFlt);
                const float frac = fmaf(f[k], idf, kMagicFlt - u);   // x * idf - n, n = u - magic exactly
                amb = fmaxf(amb, fabsf(frac));
                ub[k] = __float_as_uint(u);
            }
            exact = amb > 0.5f - 2e-4f;
            wa = __byte_perm(__byte_perm(ub[0], ub[1], 0x0040), __byte_perm(ub[2], ub[3], 0x0040), 0x5410);
            wb = __byte_perm(__byte_perm(ub[4], ub[5], 0x0040), __byte_perm(ub[6], ub[7], 0x0040), 0x5410);
        }
        if (exact) {
            const double d = (double)mx / 127.0;
            const double id = d == 0.0 ? 0.0 : 1.0 / d;
            xs = (float)d;
            int q[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) q[k] = quant_exact(f[k], id);
            wa = (uint32_t)(q[0] & 0xFF) | ((uint32_t)(q[1] & 0xFF) << 8) | ((uint32_t)(q[2] & 0xFF) << 16) |
                 ((uint32_t)(q[3] & 0xFF) << 24);
            wb = (uint32_t)(q[4] & 0xFF) | ((uint32_t)(q[5] & 0xFF) << 8) | ((uint32_t)(q[6] & 0xFF) << 16) |
                 ((uint32_t)(q[7] & 0xFF) << 24);
        }
        sum = __dp4a((int)wa, 0x01010101, __dp4a((int)wb, 0x01010101, 0));
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if (act) {
            const bool hi = BITS == 4 && (i & 1);
            uint4 r;
            r.x = wa;
            r.y = wb;
            r.z = __float_as_uint(hi ? xs * 0.0625f : xs);
            r.w = (uint32_t)(kMagicInt - (p.zp * sum) * (hi ? 16 : 1));
            srec[i] = r;
        }
    }
}

// F: sx [nb][2 halves][C][4 tig] entries of 8 bytes = bf16 (e0, e2, e1, e3) of the four
// elements 16h + 4tig + 0..3 of column c = m*T + t (term t of token m), C = M*T.
// the entry of elements e .. e + 3 of x (f32 or bf16), term t
__device__ __forceinline__ uint2 f_entry(const void* x, int act_dtype, int64_t e, int t) {
    __nv_bfloat16 q[4];
    if (act_dtype == RSTQ_BF16) {
        const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(x) + e);
        q[0] = __ushort_as_bfloat16((unsigned short)(raw.x & 0xFFFF));
        q[1] = __ushort_as_bfloat16((unsigned short)(raw.x >> 16));
        q[2] = __ushort_as_bfloat16((unsigned short)(raw.y & 0xFFFF));
        q[3] = __ushort_as_bfloat16((unsigned short)(raw.y >> 16));
    } else {
        const float4 f = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + e);
        q[0] = bf16_term(f.x, t);
        q[1] = bf16_term(f.y, t);
        q[2] = bf16_term(f.z, t);
        q[3] = bf16_term(f.w, t);
    }
    uint2 v;
    v.x = (uint32_t)__bfloat16_as_ushort(q[0]) | ((uint32_t)__bfloat16_as_ushort(q[2]) << 16);
    v.y = (uint32_t)__bfloat16_as_ushort(q[1]) | ((uint32_t)__bfloat16_as_ushort(q[3]) << 16);
    return v;
}
__device__ __forceinline__ void stage_f(const StreamParams& p, uint8_t* smem, int tid) {
    uint2* sx = reinterpret_cast<uint2*>(smem + p.act_off);
    const int C = p.M * p.T, nb = p.nb;
    int m = 0, t = 0;
    for (int c = 0; c < C; ++c) {
        for (int i = tid; i < nb * 8; i += kConsumers) {
            const int tg = i & 3, h = (i >> 2) & 1, b = i >> 3;
            const int64_t e = (int64_t)m * p.in + b * 32 + h * 16 + tg * 4;
            sx[((b * 2 + h) * C + c) * 4 + tg] = f_entry(p.x, p.act_dtype, e, t);
        }
        if (++t == p.T) { t = 0; ++m; }
    }
}
// The same array in global memory, for launches whose activations ride the weight ring (StreamParams::ring):
// block-major, so the entries of a chunk's K blocks are one contiguous slice.
__global__ void __launch_bounds__(256)
act_image_f_kernel(const void* __restrict__ x, uint2* __restrict__ img, int M, int T, int nb, int64_t in, int act_dtype) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int C = M * T;
    const int64_t n = (int64_t)nb * 8 * C, step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < n; o += step) {
        const int tg = (int)(o & 3);
        const int64_t r = o >> 2;                 // (b * 2 + h) * C + c
        const int c = (int)(r % C);
        const int64_t bh = r / C;
        const int h = (int)(bh & 1);
        const int64_t b = bh >> 1;
        const int m = c / T, t = c - m * T;
        img[o] = f_entry(x, act_dtype, (int64_t)m * in + b * 32 + h * 16 + tg * 4, t);
    }
}

// ---- one unit (32 rows x one 32-element block) from the ring ------------------------
// UK: unit kind beyond the plain one: 1 = Q4_K (32 minima behind the scales), 2 = Q6_K (8-bit codes, 64
// scales: for row gid + 8i of the group the scales of elements 0..15 and 16..31 at floats (gid*4 + i)*2 + h)
// Shared-memory loads by 32-bit shared address: a pointer derived from the dynamic array through offsets that
// live in the kernel parameters is a generic 64-bit pointer to the compiler (two-instruction additions, generic
// loads).  Measured: mode F above one token 10 % faster with these, mode A8 unchanged.
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ ulonglong2 lds128q(uint32_t a) {
    ulonglong2 v;
    asm volatile("ld.shared.v2.u64 {%0,%1}, [%2];" : "=l"(v.x), "=l"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ float4 lds128f(uint32_t a) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ float lds32f(uint32_t a) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
    return v;
}

template <int BITS>
struct SUnit {
    uint4 c0, c1;
    float4 sc, mn;   // Q6_K: sc = {row i=0 h=0, i=0 h=1, i=1 h=0, i=1 h=1}, mn = the same of i = 2, 3
};
template <int BITS, int UK = 0>
__device__ __forceinline__ void lds_unit(SUnit<BITS>& u, uint32_t unit, int lane) {
    constexpr int CODES = BITS == 4 ? kUnitCodesQ4 : kUnitCodesQ8;
    u.c0 = lds128(unit + lane * 16);
    if (BITS == 8) u.c1 = lds128(unit + 512 + lane * 16);
    if (UK == 2) {
        u.sc = lds128f(unit + CODES + (lane >> 2) * 32);
        u.mn = lds128f(unit + CODES + (lane >> 2) * 32 + 16);
        return;
    }
    u.sc = lds128f(unit + CODES + (lane >> 2) * 16);
    if (UK == 1) u.mn = lds128f(unit + CODES + 128 + (lane >> 2) * 16);
}

// A-fragment registers of the two 16-row tiles (q = 0: rows gid, gid+8; q = 1: rows
// gid+16, gid+24).  For 4-bit codes the rows gid+8 / gid+24 come out multiplied by 16.
template <int BITS>
__device__ __forceinline__ void a_frags(const SUnit<BITS>& u, uint32_t (&a)[2][4]) {
    if (BITS == 4) {
        const uint32_t lo = 0x0F0F0F0Fu, hi = 0xF0F0F0F0u;
        a[0][0] = u.c0.x & lo;
        a[0][1] = u.c0.x & hi;
        a[0][2] = u.c0.y & lo;
        a[0][3] = u.c0.y & hi;
        a[1][0] = u.c0.z & lo;
        a[1][1] = u.c0.z & hi;
        a[1][2] = u.c0.w & lo;
        a[1][3] = u.c0.w & hi;
    } else {
        a[0][0] = u.c0.x;
        a[0][1] = u.c0.y;
        a[0][2] = u.c1.x;
        a[0][3] = u.c1.y;
        a[1][0] = u.c0.z;
        a[1][1] = u.c0.w;
        a[1][2] = u.c1.z;
        a[1][3] = u.c1.w;
    }
}

// ---- M == 1 -------------------------------------------------------------------------------
// Lane (gid, tig) owns output row gid + 8*tig of the group.  Everything is addressed by 32-bit
// shared-memory addresses: `codes` = the lane's 16-byte slot of a unit, `scale` = the f32 scale of
// its row, `rec` = its staged record {xq word tig, xq word 4 + tig, xs_t, c_t}.
//
// 4-bit codes: two masks per word give the low-nibble rows (gid, gid + 16) and the high-nibble rows
// (gid + 8, gid + 24), the latter multiplied by 16 (undone in the staged scale and constant).
template <int BITS>
struct RowUnit {
    uint4 c0, c1, r;
    float sc, mn;    // Q6_K: the row's scales of elements 0..15 and 16..31
    uint32_t c2;     // Q6_K: the constant of the second half (the first half's is r.w)
};
// `scale` = address of the lane's first scale: unit + CODES + lane * 4 (Q6_K: + lane * 8)
template <int BITS, int UK = 0>
__device__ __forceinline__ void row_load(RowUnit<BITS>& u, uint32_t codes, uint32_t scale, uint32_t rec) {
    u.c0 = lds128(codes);
    if (BITS == 8) u.c1 = lds128(codes + 512);
    u.sc = lds32f(scale);
    if (UK == 1) u.mn = lds32f(scale + 128);   // the row's minimum db * bq: 32 floats behind the 32 scales
    if (UK == 2) u.mn = lds32f(scale + 4);
    u.r = lds128(rec);
    if (UK == 2) u.c2 = __float_as_uint(lds32f(rec + 16));
}
template <int BITS, int UK = 0>
__device__ __forceinline__ float row_fold(const RowUnit<BITS>& u, uint32_t m, bool upper, float acc) {
    constexpr bool KQ = UK == 1;
    uint32_t a[2][4];
    if (BITS == 4) {
        const uint32_t lo = 0x0F0F0F0Fu, hi = 0xF0F0F0F0u;
        a[0][0] = u.c0.x & lo; a[0][1] = u.c0.x & hi; a[0][2] = u.c0.y & lo; a[0][3] = u.c0.y & hi;
        a[1][0] = u.c0.z & lo; a[1][1] = u.c0.z & hi; a[1][2] = u.c0.w & lo; a[1][3] = u.c0.w & hi;
    } else {
        a[0][0] = u.c0.x; a[0][1] = u.c0.y; a[0][2] = u.c1.x; a[0][3] = u.c1.y;
        a[1][0] = u.c0.z; a[1][1] = u.c0.w; a[1][2] = u.c1.z; a[1][3] = u.c1.w;
    }
    if (UK == 2) {
        // Q6_K: a scale per 16 elements, so the two halves of the block are two tiles each: the
        // same A registers against {b0, 0} and {0, b1}
        int e0[4], e1[4], f0[4], f1[4];
        imma_u8s8(e0, a[0], u.r.x, 0u);
        imma_u8s8(f0, a[0], 0u, u.r.y);
        imma_u8s8(e1, a[1], u.r.x, 0u);
        imma_u8s8(f1, a[1], 0u, u.r.y);
        const uint32_t lo_e = (uint32_t)(upper ? e1[0] : e0[0]), hi_e = (uint32_t)(upper ? e1[2] : e0[2]);
        const uint32_t lo_f = (uint32_t)(upper ? f1[0] : f0[0]), hi_f = (uint32_t)(upper ? f1[2] : f0[2]);
        const float ve = __uint_as_float((m ? hi_e : lo_e) + u.r.w) - kMagicFlt;
        const float vf = __uint_as_float((m ? hi_f : lo_f) + u.c2) - kMagicFlt;
        const float xs = __uint_as_float(u.r.z);
        return fmaf(u.mn * xs, vf, fmaf(u.sc * xs, ve, acc));
    }
    int d0[4], d1[4];
    imma_u8s8(d0, a[0], u.r.x, u.r.y);
    imma_u8s8(d1, a[1], u.r.x, u.r.y);
    // tig 0 -> d0[0] (row gid), 1 -> d0[2] (gid+8), 2 -> d1[0] (gid+16), 3 -> d1[2] (gid+24)
    const uint32_t lo = (uint32_t)(upper ? d1[0] : d0[0]), hi = (uint32_t)(upper ? d1[2] : d0[2]);
    if (KQ) {   // zero point 0: the record's last word is t = xs * code sum of the block, for the minimum term
        const uint32_t iv = (m ? hi : lo) + (uint32_t)kMagicInt;
        const float f = __uint_as_float(iv) - kMagicFlt;
        return fmaf(u.mn, __uint_as_float(u.r.w), fmaf(u.sc * __uint_as_float(u.r.z), f, acc));
    }
    const uint32_t iv = (m ? hi : lo) + u.r.w;
    const float f = __uint_as_float(iv) - kMagicFlt;
    return fmaf(u.sc * __uint_as_float(u.r.z), f, acc);
}

// Two f32 in one 64-bit register (element 0 in the low half) and the packed arithmetic of sm_100 on them.
__device__ __forceinline__ uint64_t pack_b32x2(uint32_t lo, uint32_t hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
    return r;
}
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
    return pack_b32x2(__float_as_uint(lo), __float_as_uint(hi));
}
__device__ __forceinline__ float lo_f32x2(uint64_t v) {
    uint32_t lo, hi;
    asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(v));
    return __uint_as_float(lo);
}
__device__ __forceinline__ float hi_f32x2(uint64_t v) {
    uint32_t lo, hi;
    asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(v));
    return __uint_as_float(hi);
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t mul_f32x2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}

template <int BITS, int NT, int UK = 0>
__device__ __forceinline__ void unit_a8(const SUnit<BITS>& u, uint32_t actB, uint32_t actZ,
                                        const StreamParams& p, int b, int gid, int tig,
                                        float (&acc)[NT][4][2]) {
    constexpr bool KQ = UK == 1;
    uint32_t a[2][4];
    a_frags<BITS>(u, a);
    if (UK == 2) {
        // Q6_K: per (block, token) {xs, zp * sum of 0..15, zp * sum of 16..31}; two tiles per 16 rows
        const int M = p.M, Mz = (M + 1) & ~1;
        const uint32_t xB = actB + b * M * 32, xz = actZ + b * Mz * 16;
        const float se[4] = {u.sc.x, u.sc.z, u.mn.x, u.mn.z};   // rows gid + 8i, elements 0..15
        const float sf[4] = {u.sc.y, u.sc.w, u.mn.y, u.mn.w};   // elements 16..31
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            int col = nt * 8 + gid;
            col = col < M ? col : M - 1;
            const uint2 bb = lds64(xB + (col * 4 + tig) * 8);
            int c0 = nt * 8 + 2 * tig;
            c0 = c0 < Mz ? c0 : 0;
            const uint4 z0u = lds128(xz + c0 * 16), z1u = lds128(xz + c0 * 16 + 16);
            const int4 z0 = make_int4((int)z0u.x, (int)z0u.y, (int)z0u.z, (int)z0u.w);
            const int4 z1 = make_int4((int)z1u.x, (int)z1u.y, (int)z1u.z, (int)z1u.w);
            const float xs0 = __int_as_float(z0.x), xs1 = __int_as_float(z1.x);
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                int de[4], df[4];
                imma_acc(de, a[q], bb.x, 0u, kMagicInt - z0.y, kMagicInt - z1.y, kMagicInt - z0.y, kMagicInt - z1.y);
                imma_acc(df, a[q], 0u, bb.y, kMagicInt - z0.z, kMagicInt - z1.z, kMagicInt - z0.z, kMagicInt - z1.z);
#pragma unroll
                for (int i = 0; i < 2; ++i) {   // row gid + 8 (2q + i)
                    const float s_e = se[2 * q + i], s_f = sf[2 * q + i];
                    acc[nt][2 * q + i][0] = fmaf(s_f * xs0, __int_as_float(df[2 * i]) - kMagicFlt,
                                                 fmaf(s_e * xs0, __int_as_float(de[2 * i]) - kMagicFlt, acc[nt][2 * q + i][0]));
                    acc[nt][2 * q + i][1] = fmaf(s_f * xs1, __int_as_float(df[2 * i + 1]) - kMagicFlt,
                                                 fmaf(s_e * xs1, __int_as_float(de[2 * i + 1]) - kMagicFlt, acc[nt][2 * q + i][1]));
                }
            }
        }
        return;
    }
    if (UK == 0) {
        // Plain units: everything that depends on the (block, token) alone comes ready-made in the pair record
        // (put_act_record); the fold of a row's two values is two packed f32 operations and two fmas:
        // t = (float(d) - bias) * xs for both tokens at once, acc += s * t each.
        const float sc[4] = {u.sc.x, u.sc.y, u.sc.z, u.sc.w};
        const int M = p.M, Mh = (M + 1) >> 1;
        const uint32_t xB = actB + b * M * 32, rec = actZ + b * Mh * 32;
        const uint64_t nbias = pack_f32x2(-kMagicFlt, -kMagicFlt);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            // columns beyond M are never stored, so any valid address will do for them
            int col = nt * 8 + gid;
            col = col < M ? col : M - 1;
            const uint2 bb = lds64(xB + (col * 4 + tig) * 8);
            int pr = nt * 4 + tig;
            pr = pr < Mh ? pr : 0;
            const ulonglong2 xv = lds128q(rec + pr * 32);         // {xs_a, xs_b}, {xs_a h, xs_b h}
            const uint4 cv = lds128(rec + pr * 32 + 16);          // ca_a, ca_b, cb_a, cb_b
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                int d[4];
                imma_acc(d, a[q], bb.x, bb.y, (int)cv.x, (int)cv.y, (int)cv.z, (int)cv.w);
                const uint64_t tl = mul_f32x2(add_f32x2(pack_b32x2((uint32_t)d[0], (uint32_t)d[1]), nbias), xv.x);
                const uint64_t th = mul_f32x2(add_f32x2(pack_b32x2((uint32_t)d[2], (uint32_t)d[3]), nbias), xv.y);
                const float s0 = sc[2 * q], s1 = sc[2 * q + 1];
                acc[nt][2 * q][0] = fmaf(s0, lo_f32x2(tl), acc[nt][2 * q][0]);
                acc[nt][2 * q][1] = fmaf(s0, hi_f32x2(tl), acc[nt][2 * q][1]);
                acc[nt][2 * q + 1][0] = fmaf(s1, lo_f32x2(th), acc[nt][2 * q + 1][0]);
                acc[nt][2 * q + 1][1] = fmaf(s1, hi_f32x2(th), acc[nt][2 * q + 1][1]);
            }
        }
        return;
    }
    const float sc[4] = {u.sc.x, u.sc.y, u.sc.z, u.sc.w};
    const float mn[4] = {u.mn.x, u.mn.y, u.mn.z, u.mn.w};
    // value of the high-nibble rows is 16x: scale by xs/16 and shift their zero-point term
    constexpr float HI = BITS == 4 ? 0.0625f : 1.0f;
    constexpr int ZSH = BITS == 4 ? 4 : 0;
    const int M = p.M, Mz = (M + 1) & ~1;
    const uint32_t xB = actB + b * M * 32, xz = actZ + b * Mz * 8;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        // columns beyond M are never stored, so any valid address will do for them
        int col = nt * 8 + gid;
        col = col < M ? col : M - 1;
        const uint2 bb = lds64(xB + (col * 4 + tig) * 8);
        int c0 = nt * 8 + 2 * tig;
        c0 = c0 < Mz ? c0 : 0;
        const uint4 zu = lds128(xz + c0 * 8);
        const int4 z = make_int4((int)zu.x, (int)zu.y, (int)zu.z, (int)zu.w);
        const float xs0 = __int_as_float(z.x), xs1 = __int_as_float(z.z);
        const float xs0h = xs0 * HI, xs1h = xs1 * HI;
        // Q4_K (zero point 0): the second word of a record is t = xs * code sum, which the minima multiply
        const int ca0 = KQ ? kMagicInt : kMagicInt - z.y, ca1 = KQ ? kMagicInt : kMagicInt - z.w;
        const int cb0 = KQ ? kMagicInt : kMagicInt - (z.y << ZSH), cb1 = KQ ? kMagicInt : kMagicInt - (z.w << ZSH);
        const float t0 = __int_as_float(z.y), t1 = __int_as_float(z.w);
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            int d[4];
            imma_acc(d, a[q], bb.x, bb.y, ca0, ca1, cb0, cb1);
            const float s0 = sc[2 * q], s1 = sc[2 * q + 1];
            acc[nt][2 * q][0] = fmaf(s0 * xs0, __int_as_float(d[0]) - kMagicFlt, acc[nt][2 * q][0]);
            acc[nt][2 * q][1] = fmaf(s0 * xs1, __int_as_float(d[1]) - kMagicFlt, acc[nt][2 * q][1]);
            acc[nt][2 * q + 1][0] =
                fmaf(s1 * xs0h, __int_as_float(d[2]) - kMagicFlt, acc[nt][2 * q + 1][0]);
            acc[nt][2 * q + 1][1] =
                fmaf(s1 * xs1h, __int_as_float(d[3]) - kMagicFlt, acc[nt][2 * q + 1][1]);
            if (KQ) {
                acc[nt][2 * q][0] = fmaf(mn[2 * q], t0, acc[nt][2 * q][0]);
                acc[nt][2 * q][1] = fmaf(mn[2 * q], t1, acc[nt][2 * q][1]);
                acc[nt][2 * q + 1][0] = fmaf(mn[2 * q + 1], t0, acc[nt][2 * q + 1][0]);
                acc[nt][2 * q + 1][1] = fmaf(mn[2 * q + 1], t1, acc[nt][2 * q + 1][1]);
            }
        }
    }
}

// Two 4-bit codes (bits S .. S+3 of each half of w) -> bf16x2 of (code - 8): a shift, one three-input logic
// operation ((t & mask) | 0x4300 = bf16 of 128 + code) and one packed subtract, spelled out: left to the
// compiler the same expression took 16 more instructions per unit (ncu: 63 -> 47 on the integer pipe).
template <int S>
__device__ __forceinline__ uint32_t dq4_bf16x2(uint32_t w, uint32_t m4, uint32_t ex, uint32_t off) {
    uint32_t d;
    if (S == 0) {
        asm("{ .reg .b32 t; lop3.b32 t, %1, %2, %3, 0xEA; sub.bf16x2 %0, t, %4; }" : "=r"(d) : "r"(w), "r"(m4), "r"(ex), "r"(off));
    } else {
        asm("{ .reg .b32 t; shr.b32 t, %1, %5; lop3.b32 t, t, %2, %3, 0xEA; sub.bf16x2 %0, t, %4; }"
            : "=r"(d)
            : "r"(w), "r"(m4), "r"(ex), "r"(off), "n"(S));
    }
    return d;
}

template <int BITS, int NT>
__device__ __forceinline__ void unit_f(const SUnit<BITS>& u, uint32_t actB,
                                       const StreamParams& p, int b, int gid, int tig,
                                       float (&acc)[NT][4][2]) {
    // fr[h][i][j]: half h, row gid + 8i, j = 0 -> elements (+0, +2), j = 1 -> (+1, +3)
    uint32_t fr[2][4][2];
    const uint32_t c0[4] = {u.c0.x, u.c0.y, u.c0.z, u.c0.w};
    const uint32_t c1[4] = {u.c1.x, u.c1.y, u.c1.z, u.c1.w};
    if (BITS == 4) {
        // word 2q + h: low nibbles = row i = 2q, high nibbles = row i = 2q + 1.
        // 0x4300 | n is bf16(128 + n); subtract 128 + zero point 8.
        const uint32_t m4 = 0x000F000Fu, ex = 0x43004300u, off = 0x43084308u;
#pragma unroll
        for (int q = 0; q < 2; ++q)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t w = c0[2 * q + h];
                fr[h][2 * q][0] = dq4_bf16x2<0>(w, m4, ex, off);
                fr[h][2 * q][1] = dq4_bf16x2<8>(w, m4, ex, off);
                fr[h][2 * q + 1][0] = dq4_bf16x2<4>(w, m4, ex, off);
                fr[h][2 * q + 1][1] = dq4_bf16x2<12>(w, m4, ex, off);
            }
    } else {
        // 0x4B000000 | b is f32(2^23 + b); subtract 2^23 + zero point 128
        const float off = 8388736.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i)
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
    const float sc[4] = {u.sc.x, u.sc.y, u.sc.z, u.sc.w};
    const int C = p.M * p.T;
    const uint32_t xb = actB + b * C * 64;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        int col = nt * 8 + gid;
        col = col < C ? col : C - 1;
        const uint2 bx0 = lds64(xb + (col * 4 + tig) * 8);
        const uint2 bx1 = lds64(xb + ((C + col) * 4 + tig) * 8);
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

// Sum over the consumer warps of the fragment element holding (row, col); red is [warp][v][lane].
template <int NT>
__device__ __forceinline__ float stream_reduce_rc(const float* red, int row, int col) {
    constexpr int NV = NT * 8;
    const int gid = row & 7, i = row >> 3;
    const int nt = col >> 3, within = col & 7;
    const int lane = gid * 4 + (within >> 1);
    const int v = (nt * 4 + i) * 2 + (within & 1);
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < kCW; ++w) s += red[(w * NV + v) * 32 + lane];
    return s;
}

// ---- the kernel ---------------------------------------------------------------------
// QF: M == 1 only, the kernel quantizes the raw activations p.x itself while staging.
template <int BITS, int NT, int MODE, bool ONECOL, bool TP, bool QF = false, int UK = 0>
__global__ void __launch_bounds__(kStreamThreads, 1) gemv_stream_kernel(const StreamParams p) {
    constexpr int UNIT = BITS == 4 ? (UK == 1 ? kUnitBytesQ4K : kUnitBytesQ4) : (UK == 2 ? kUnitBytesQ6K : kUnitBytesQ8);
    constexpr int REC = UK == 2 ? 32 : 16;   // bytes of a staged (block, tig) record at M = 1
    constexpr int kUPW = upw_of(BITS), kChunkUnits = chunk_units_of(BITS);
    constexpr int CHUNK_BYTES = kChunkUnits * UNIT;
    constexpr int NV = NT * 8;
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int s_abort;
    __shared__ int s_cn;
    __shared__ long long s_g0;
    __shared__ int s_bstart, s_total;
    __shared__ int s_tp_ok;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int gid = lane >> 2, tig = lane & 3;
    const int NS = p.NS, nb = p.nb;
    unsigned long long* dbg = p.dbg ? p.dbg + (size_t)blockIdx.x * 8 : nullptr;
    if (dbg && tid == 0) {
        dbg[0] = gtime_ns();
        uint32_t smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        dbg[6] = smid;
    }
    const uint32_t full0 = smem_u32(smem + p.bar_off), empty0 = full0 + NS * 8;
    const uint32_t act_bar = empty0 + NS * 8;
    if (tid < NS) mbar_init(full0 + 8 * tid, 1);
    else if (tid < 2 * NS) mbar_init(empty0 + 8 * (tid - NS), kCW);
    else if (tid == 2 * NS + 1) mbar_init(act_bar, 1);
    if (tid == 2 * NS) {
        // this CTA's unit range, as (first group, first block in it, unit count)
        const int64_t u0 = range_begin(blockIdx.x, p.uq, p.ur);
        const int64_t g0 = u0 / nb;
        s_g0 = g0;
        s_bstart = (int)(u0 - g0 * nb);
        const int64_t u1 = range_begin(blockIdx.x + 1, p.uq, p.ur);
        s_total = (int)((u1 < p.U ? u1 : p.U) - u0);
        s_abort = 0;
    }
    if (tid < 2 * NS || tid == 2 * NS + 1) asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    // Programmatic dependent launch: the next kernel in the stream may be scheduled onto
    // SMs as this grid's CTAs retire (a no-op for a plain launch).
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    __syncthreads();
    volatile int* abort_flag = &s_abort;
    const int64_t g0 = s_g0;
    const int b_start = s_bstart, total = s_total;

    // Both roles walk the same chunk schedule with incremental indices: g = group,
    // b = block inside the group, left = units still to do, (s, ph) = ring slot and
    // its phase.  A chunk is n = min(32, nb - b, left) units: it never straddles a group.
    if (warp == kCW) {
        // ---------------- producer: one lane streams the CTA's byte range ----------------
        if (lane == 0) {
            const uint8_t* src = p.w + (g0 * nb + b_start) * UNIT;
            const uint64_t pol = l2_evict_first_policy();  // the weights pass through L2 once
            int b = b_start, left = total, s = 0, issued = 0;
            uint32_t ph = 0;
            bool ok = true;
            // HBM requests beyond what the ring holds: the range is requested into L2 up to `pf_ahead`
            // bytes ahead of the copy position, so the bytes in flight from HBM are not bounded by
            // shared memory and the ring only has to cover the L2 round trip.
            // Once this CTA's own range is requested in full, ask for the head of the next launch's weights to be
            // brought into L2: by the time this launch's consumers have drained their rings -- HBM would
            // idle meanwhile, the next launch's CTAs cannot be resident before these leave -- the next
            // launch finds its first chunks in L2 and fills its rings at L2 speed.
            auto prefetch_next = [&]() {
                if (!p.nx_w) return;
                for (int j = blockIdx.x; j < p.nx_G; j += gridDim.x) {
                    const int64_t u0 = range_begin(j, p.nx_uq, p.nx_ur);
                    int64_t u1 = range_begin(j + 1, p.nx_uq, p.nx_ur);
                    u1 = u1 < p.nx_U ? u1 : p.nx_U;
                    int64_t n = u1 - u0 < p.nx_pf_units ? u1 - u0 : p.nx_pf_units;
                    const uint8_t* q = p.nx_w + u0 * p.nx_unit;
                    for (int64_t rest = n * p.nx_unit; rest > 0; rest -= 32768, q += 32768) {
                        const uint32_t nbytes = (uint32_t)(rest < 32768 ? rest : 32768);
                        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(q), "r"(nbytes) : "memory");
                    }
                }
            };
            bool nx_done = false;
            const uint8_t* const end = src + (int64_t)total * UNIT;
            const uint8_t* pf = src;
#if RSTQ_PROBES
            unsigned long long* pfine = (p.dbg && blockIdx.x == 0) ? p.dbg_fine + 256 : nullptr;  // producer stamps
            int npf = 0;
#endif
            const int64_t pf_ahead = p.pf_ahead;
            // The activation image is the quantizer's output: it is copied once the ring has its first
            // NS chunks on the way (the weights do not depend on the kernel before this one, the image
            // does), as bulk copies that run beside the weight stream instead of 16 warps of loads
            // and stores in front of it.
            bool img_done = p.img == nullptr;
            auto copy_image = [&]() {
                asm volatile("griddepcontrol.wait;" ::: "memory");
                mbar_expect_tx(act_bar, p.img_b_bytes + p.img_z_bytes);
                for (uint32_t o = 0; o < p.img_b_bytes; o += 32768) {
                    const uint32_t n = p.img_b_bytes - o < 32768 ? p.img_b_bytes - o : 32768;
                    bulk_copy_g2s(smem_u32(smem + p.act_off) + o, p.img + o, n, act_bar);
                }
                bulk_copy_g2s(smem_u32(smem + p.act2_off), p.img + p.img_z_off, p.img_z_bytes, act_bar);
                img_done = true;
            };
            // Ring of activations: a stage's slice of the image depends on the kernel before this one, its
            // weights do not.  The first NS chunks of weights leave at once, registered on their barriers
            // without an arrival; their slices follow after the wait, with the arrival.
            const bool ring = !ONECOL && p.ring;
            const int Mz8 = (int)p.slice2, M32 = (int)p.slice1;   // bytes of a block's records / fragments (entries in mode F, no records)
            const int cu = ONECOL ? kChunkUnits : p.cu;
            const uint32_t stage_bytes = ONECOL ? (uint32_t)CHUNK_BYTES : p.stage_bytes;
            int pend_b[RSTQ_NSMAX], pend_n[RSTQ_NSMAX], npend = 0;
            bool dep_waited = !ring;
            if (ring) img_done = true;   // nothing is copied for the whole launch
            auto copy_slice = [&](int slot, int bb, int nn, uint32_t more) {
                const uint32_t nb1 = (uint32_t)(nn * M32), nb2 = (uint32_t)(nn * Mz8);
                const uint32_t dst = smem_u32(smem) + (uint32_t)slot * stage_bytes;
                mbar_expect_tx(full0 + 8 * slot, more + nb1 + nb2);
                bulk_copy_g2s(dst + p.act_off, p.img + (int64_t)bb * M32, nb1, full0 + 8 * slot);
                if (nb2) bulk_copy_g2s(dst + p.act2_off, p.img + p.img_z_off + (int64_t)bb * Mz8, nb2, full0 + 8 * slot);
            };
            auto slices_of_first = [&]() {
                asm volatile("griddepcontrol.wait;" ::: "memory");
                for (int k = 0; k < npend; ++k) copy_slice(k, pend_b[k], pend_n[k], 0u);
                npend = 0;
                dep_waited = true;
            };
            while (left > 0) {
                if (!img_done && issued >= NS) copy_image();
                if (!dep_waited && issued >= NS) slices_of_first();
                if (pf_ahead > 0) {
                    const uint8_t* lim = src + pf_ahead < end ? src + pf_ahead : end;
                    while (pf < lim) {
                        const int64_t rest = end - pf;
                        const uint32_t nbytes = (uint32_t)(rest < 32768 ? rest : 32768);
                        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(pf), "r"(nbytes) : "memory");
                        pf += nbytes;
                    }
                }
                int n = nb - b < left ? nb - b : left;
                n = n < cu ? n : cu;
                ok = mbar_try(empty0 + 8 * s, ph ^ 1u) || mbar_wait(empty0 + 8 * s, ph ^ 1u, abort_flag);
                if (!ok) break;
#if RSTQ_PROBES
                if (pfine && npf < 250) pfine[1 + npf++] = gtime_ns();
#endif
                const uint32_t bytes = (uint32_t)(n * UNIT);
                if (PROBE(1)) {
                    mbar_arrive(full0 + 8 * s);
                } else if (ring) {
                    if (dep_waited) {
                        copy_slice(s, b, n, bytes);
                    } else {
                        mbar_expect_only(full0 + 8 * s, bytes);
                        pend_b[npend] = b;
                        pend_n[npend++] = n;
                    }
                    bulk_copy_g2s_hint(smem_u32(smem) + (uint32_t)s * stage_bytes, src, bytes, full0 + 8 * s, pol);
                } else {
                    mbar_expect_tx(full0 + 8 * s, bytes);
                    bulk_copy_g2s_hint(smem_u32(smem) + (uint32_t)s * stage_bytes, src, bytes, full0 + 8 * s, pol);
                }
#if RSTQ_PROBES
                if (pfine && npf < 250) pfine[1 + npf++] = gtime_ns();
#endif
                src += bytes;
                b += n;
                if (b == nb) b = 0;
                left -= n;
                ++issued;
                if (++s == NS) { s = 0; ph ^= 1u; }
                if (!nx_done && left == 0) {   // behind the last request of this launch's own stream
                    prefetch_next();
                    nx_done = true;
                }
            }
#if RSTQ_PROBES
            if (pfine) pfine[0] = (unsigned long long)npf;
#endif
            if (!img_done && ok) copy_image();
            if (!dep_waited && ok) slices_of_first();
            if (!ok && p.img && img_done) {  // gave up with the image copy in flight: let it land (bounded)
                const unsigned long long t0 = gtime_ns();
                while (!mbar_try(act_bar, 0) && gtime_ns() - t0 < kWaitLimitNs) {
                }
            }
            if (!ok) {
                // gave up: still wait (bounded) for the copies already issued to land,
                // so no copy is in flight into this CTA's shared memory when it exits
                for (int k = issued > NS ? issued - NS : 0; k < issued; ++k) {
                    const uint32_t bar = full0 + 8 * (k % NS), kph = (uint32_t)(k / NS) & 1u;
                    const unsigned long long t0 = gtime_ns();
                    while (!mbar_try(bar, kph) && gtime_ns() - t0 < kWaitLimitNs) {
                    }
                }
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    // Everything above (barriers, the weight stream) is independent of earlier kernels;
    // activations, y and the scratch are not: wait for the preceding grid to finish.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (dbg && tid == 0) dbg[1] = gtime_ns();
    // Fused exchange: results go to slot `rank` of every rank's stage (epoch parity picks the
    // half; the epoch is written by the previous exchange of this stream, hence read after the wait)
    const int tpn = TP ? p.tp.nranks : 0;  // (a separate instantiation: the plain kernel keeps its registers)
    uint32_t tp_e = 0;
    int64_t tp_off = 0, tp_slot = 0;
    uint8_t* tp_mine = nullptr;
    if (TP) {
#pragma unroll
        for (int r = 0; r < kTpMaxRanks; ++r)
            if (r == p.tp.rank) tp_mine = p.tp.region[r];
        tp_e = *reinterpret_cast<volatile uint32_t*>(tp_mine + 256) + 1u;
        tp_off = p.tp.ll_off + ((int64_t)(tp_e & 1u) * tpn) * p.tp.slot_bytes;
        tp_slot = tp_off + (int64_t)p.tp.rank * p.tp.slot_bytes;
    }
    auto emit = [&](int64_t idx, float v) {
        if (!TP) {
            store_out(p.y, p.out_dtype, idx, v);
        } else {
            // value and epoch travel in ONE 8-byte store: whoever reads the epoch has the value,
            // so no fence and no separate flag stand between this store and the reader
#pragma unroll
            for (int r = 0; r < kTpMaxRanks; ++r)  // static indices keep the pointer table in the parameter bank
                if (r < tpn)
                    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p.tp.region[r] + tp_slot + idx * 8),
                                 "r"(__float_as_uint(v)), "r"(tp_e)
                                 : "memory");
        }
    };
    if (QF) {
        stage_a8_quant<BITS>(p, smem, tid);
    } else if (MODE == MODE_A8) {
        if (!ONECOL && p.ring) {
            // the slices arrive with the weight chunks
        } else if (!ONECOL && p.img) {
            int got = 1;
            if (lane == 0) got = mbar_spin(act_bar, 0, abort_flag);   // on expiry the abort flag ends the loops below
            (void)__shfl_sync(0xffffffffu, got, 0);
        } else {
            stage_a8<ONECOL, BITS>(p, smem, tid);
        }
    } else if (!p.ring) {
        stage_f(p, smem, tid);
    }
    consumer_bar();
    if (dbg && tid == 0) dbg[2] = gtime_ns();

    float acc[NT][4][2];
    float* red = reinterpret_cast<float*>(smem + p.red_off);
    const int M = p.M, T = p.T;
    // fine record of CTA 0 (thread 0): a stamp after every wait, chunk and flush step, behind the slots
#if RSTQ_PROBES
    unsigned long long* fine = (p.dbg && blockIdx.x == 0 && tid == 0) ? p.dbg_fine : nullptr;
    int nfine = 0;
#endif
    auto stamp = [&]() {
#if RSTQ_PROBES
        if (fine && nfine < 250) fine[1 + nfine++] = gtime_ns();
#endif
    };

    auto zero_acc = [&]() {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[nt][i][0] = acc[nt][i][1] = 0.f;
    };
    // A group whose K range is cut between CTAs (the equal-range split) is finished by the CTA that
    // holds its head, for which it is the LAST segment; every CTA behind it holds a later part as its
    // FIRST segment (or only one) and hands the partial sums over through its slot as soon as that
    // segment is done -- early in its loop, so the finisher normally finds them waiting and the
    // hand-over costs one read from L2 at the end instead of a chain of dependent trips.  Sums are
    // added in CTA order.  The wait for a slot is time-bounded; the finisher clears the flags it took.
    auto hand_over = [&](int64_t g, float sum, int64_t o, bool owner) {
        // called by all consumer threads; `owner` threads hold `sum` for output index o of group g
        const int c = blockIdx.x;
        if (tid == 0) {
            const int cl = cta_of_unit((g + 1) * nb - 1, p.uq, p.ur);
            int cn = cl - c;
            const unsigned long long t0 = gtime_ns();
            for (int k = 1; k <= cn; ++k) {
                const volatile int* f = p.flags + c + k;
                uint32_t spins = 0;
                while (*f == 0) {
                    if ((++spins & 255u) == 0 && (*abort_flag || gtime_ns() - t0 > kWaitLimitNs)) {
                        *abort_flag = 1;   // a contributor never delivered: report, do not hang
                        cn = 0;
                        break;
                    }
                }
            }
            __threadfence();
            s_cn = cn;
        }
        consumer_bar();
        const int cn = s_cn;
        if (owner && cn > 0) {
            const int64_t row = o & 31, m = o >> 5;
            for (int k = 1; k <= cn; ++k) sum += __ldcg(p.partials + (int64_t)(c + k) * M * 32 + o);
            if (g * 32 + row < p.out) emit(m * p.out + g * 32 + row, sum);
        }
        consumer_bar();   // every slot has been read
        if (tid == 0)
            for (int k = 1; k <= cn; ++k) p.flags[c + k] = 0;
    };
    auto publish = [&]() {   // after every partial store of this CTA's slot
        consumer_bar();
        if (tid == 0) {
            __threadfence();
            *reinterpret_cast<volatile int*>(p.flags + blockIdx.x) = 1;
        }
    };
    // Cross-warp reduction of the segment [b_from, b_to) of group g, then store / hand over.  With one
    // tile of tokens two reduction buffers alternate, so one barrier per flush is enough.
    int flush_no = 0;
    auto flush = [&](int64_t g, int b_from, int b_to) {
        const bool head = b_from == 0, whole = head && (b_to == nb);
        const int64_t row0 = g * 32;
        float* part = p.partials + (int64_t)blockIdx.x * M * 32;
        // (two tiles of tokens and more: one buffer and a barrier before it is written again -- the second
        // buffer would take 32 KB and more from the ring)
        float* rbuf = ONECOL ? red + kParkGroups * kParkStride : red + (NT == 1 ? (flush_no & 1) * (kCW * NV * 32) : 0);
        if (!ONECOL && NT > 1 && flush_no > 0) consumer_bar();
        ++flush_no;
        if (ONECOL) {
            // (whole groups are parked by the loop and reduced in batches; this serves the cut ones)
            rbuf[warp * 33 + lane] = acc[0][0][0];  // row gid + 8*tig of this lane (33: the 16 readers of a row hit 16 banks)
            consumer_bar();
            // thread t < 512: row t >> 4, warps t & 15 (and 16 + that); 16 neighbouring lanes add up one row
            const int row = (tid >> 4) & 31, wsrc = tid & 15;
            float sum = rbuf[wsrc * 33 + (row & 7) * 4 + (row >> 3)];
            if (wsrc + 16 < kCW) sum += rbuf[(wsrc + 16) * 33 + (row & 7) * 4 + (row >> 3)];
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            const bool owner = (tid & 15) == 0 && tid < 512;
            if (whole) {
                if (owner && row0 + row < p.out) emit(row0 + row, sum);
            } else if (!head) {
                if (owner) part[row] = sum;
                publish();
            } else {
                hand_over(g, sum, row, owner);
            }
        } else {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int c = 0; c < 2; ++c)
                        rbuf[(warp * NV + (nt * 4 + i) * 2 + c) * 32 + lane] = acc[nt][i][c];
            consumer_bar();
            const int o = tid;   // M <= 16: at most one output per consumer thread
            const bool owner = o < M * 32;
            const int m = o >> 5, row = o & 31;
            float sum = 0.f;
            if (owner)
                for (int t = 0; t < T; ++t) sum += stream_reduce_rc<NT>(rbuf, row, m * T + t);
            if (whole) {
                if (owner && row0 + row < p.out) emit((int64_t)m * p.out + row0 + row, sum);
            } else if (!head) {
                if (owner) part[o] = sum;
                publish();
            } else {
                hand_over(g, sum, o, owner);
            }
        }
    };

    // M = 1: reduce the parked groups [g_first, g_first + count) across the warps and store them
    auto flush_parked = [&](int64_t g_first, int count, bool more) {
        consumer_bar();
        const int row = (tid >> 4) & 31, wsrc = tid & 15;
        const int src = wsrc * 33 + (row & 7) * 4 + (row >> 3);
        float* sres = red + kParkGroups * kParkStride;   // (TP) the finished sums, [group][32 rows]
        for (int i = 0; i < count; ++i) {
            float sum = red[i * kParkStride + src];
            if (wsrc + 16 < kCW) sum += red[i * kParkStride + src + 16 * 33];
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            const int64_t r = (g_first + i) * 32 + row;
            if ((tid & 15) == 0 && tid < 512) {
                if (TP) sres[i * 32 + row] = sum;
                else if (r < p.out) store_out(p.y, p.out_dtype, r, sum);
            }
        }
        if (TP) {
            // Fused exchange: the 32 (value, epoch) pairs of a group are neighbours in every rank's
            // stage, so one warp writes them to one peer as one 256-byte row (two full NVLink
            // packets) instead of 32 separate 8-byte stores from 32 threads.
            consumer_bar();
            for (int job = warp; job < count * tpn; job += kCW) {
                const int i = job / tpn, peer = job - i * tpn;
                const int64_t r = (g_first + i) * 32 + lane;
                uint8_t* dst = nullptr;
#pragma unroll
                for (int q = 0; q < kTpMaxRanks; ++q)   // static indices keep the pointer table in the parameter bank
                    if (q == peer) dst = p.tp.region[q];
                if (r < p.out)
                    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(dst + tp_slot + r * 8),
                                 "r"(__float_as_uint(sres[i * 32 + lane])), "r"(tp_e)
                                 : "memory");
            }
        }
        if (more) consumer_bar();   // the slots are written again
    };

    if (ONECOL) {
        // ---- M == 1: the loop is bound by instruction issue, so it is kept lean: 32-bit shared-memory
        // addresses that run along, segments cut into full chunks (four units per warp, fully unrolled,
        // every load issued before the first tensor-core tile) and one ragged chunk, whole groups
        // parked without a barrier.
        constexpr int CODES = BITS == 4 ? kUnitCodesQ4 : kUnitCodesQ8;
        constexpr uint32_t USTEP = kCW * UNIT, RSTEP = kCW * 4 * REC;   // next unit / record of this warp in a chunk
        const uint32_t ring = smem_u32(smem), act = smem_u32(smem + p.act_off);
        const uint32_t m = (tig & 1) ? 0xFFFFFFFFu : 0u;
        const bool upper = tig & 2;
        uint32_t codes = ring + warp * UNIT + lane * 16;            // this lane's slot of the warp's first unit
        uint32_t scale = ring + warp * UNIT + CODES + lane * (UK == 2 ? 8 : 4);
        uint32_t rec = act + ((b_start + warp) * 4 + tig) * REC;
        int s = 0, left = total, b = b_start;
        uint32_t ph = 0;
        bool alive = true;
        int64_t g = g0, g_parked = g0;
        int parked = 0;
#if RSTQ_PROBES
        long long waited = 0, ck[5] = {0, 0, 0, 0, 0}, ckt = 0;
        const long long loop0 = clock64();
#define CK_START() ckt = clock64()
#define CK_ADD(i) do { const long long t__ = clock64(); ck[i] += t__ - ckt; ckt = t__; } while (0)
#else
#define CK_START()
#define CK_ADD(i)
#endif
        if (dbg) {  // timestamp of the first weights; the loop's own wait then passes at once
            if (!mbar_try(full0, 0)) alive = mbar_wait(full0, 0, abort_flag);
            if (tid == 0) dbg[3] = gtime_ns();
        }
        // the answer of a barrier test takes a while: the test of the next chunk is issued before
        // the arithmetic of this one
        bool ready = mbar_test(full0, 0);
        while (left > 0) {
            const int seg = nb - b < left ? nb - b : left;   // this segment: blocks [b, b + seg) of group g
            float v = 0.f;
            for (int done = 0; done < seg;) {
                const int n = seg - done < kChunkUnits ? seg - done : kChunkUnits;
                const uint32_t bar = full0 + 8 * s;
#if RSTQ_PROBES
                const long long w0 = clock64();
#endif
                if (alive && !ready && !mbar_try(bar, ph)) alive = mbar_wait(bar, ph, abort_flag);
#if RSTQ_PROBES
                waited += clock64() - w0;
#endif
                stamp();
                CK_START();
                const int sn = s + 1 == NS ? 0 : s + 1;
                ready = mbar_test(full0 + 8 * sn, sn ? ph : ph ^ 1u);
                CK_ADD(0);
                if (alive && !PROBE(2)) {
                    if (n == kChunkUnits) {
                        RowUnit<BITS> u[kUPW];
#pragma unroll
                        for (int j = 0; j < kUPW; ++j) row_load<BITS, UK>(u[j], codes + j * USTEP, scale + j * USTEP, rec + j * RSTEP);
#pragma unroll
                        for (int j = 0; j < kUPW; ++j) v = row_fold<BITS, UK>(u[j], m, upper, v);
                    } else {
                        for (int j = 0; warp + j * kCW < n; ++j) {
                            RowUnit<BITS> u;
                            row_load<BITS, UK>(u, codes + j * USTEP, scale + j * USTEP, rec + j * RSTEP);
                            v = row_fold<BITS, UK>(u, m, upper, v);
                        }
                    }
                }
                CK_ADD(1);
                __syncwarp();
                stamp();
                if (lane == 0) mbar_arrive(empty0 + 8 * s);  // also when not alive: never block the producer
                stamp();
                CK_ADD(2);
                done += n;
                rec += n * 4 * REC;
                if (sn) {
                    codes += CHUNK_BYTES;
                    scale += CHUNK_BYTES;
                } else {
                    codes -= (NS - 1) * CHUNK_BYTES;
                    scale -= (NS - 1) * CHUNK_BYTES;
                    ph ^= 1u;
                }
                s = sn;
                CK_ADD(3);
            }
            left -= seg;
            CK_START();
            if (b == 0 && seg == nb) {
                // a whole group: park this warp's sums, no barrier
                if (parked == 0) g_parked = g;
                red[parked * kParkStride + warp * 33 + lane] = v;
                if (++parked == kParkGroups || left == 0) {
                    flush_parked(g_parked, parked, left > 0);
                    parked = 0;
                }
            } else {
                acc[0][0][0] = v;
                flush(g, b, b + seg);
                if (left == 0 && parked > 0) {
                    flush_parked(g_parked, parked, false);
                    parked = 0;
                }
            }
            stamp();
            CK_ADD(4);
            rec -= (b + seg) * 4 * REC;   // back to block 0 of the next group
            b = 0;
            ++g;
        }
#if RSTQ_PROBES
        if (dbg && tid == 0) dbg[7] = ((unsigned long long)(clock64() - loop0) << 32) | (unsigned long long)(waited & 0xFFFFFFFF);
        if (p.dbg && blockIdx.x == 0 && tid == 0)
            for (int i = 0; i < 5; ++i) p.dbg_fine[300 + i] = (unsigned long long)ck[i];
#endif
    } else {
        int64_t g = g0;
        int b = b_start, seg_from = b_start, left = total, s = 0;
        uint32_t ph = 0;
        bool alive = true;
        uint32_t unit0 = smem_u32(smem) + warp * UNIT;   // this warp's first unit in ring slot s (32-bit shared addresses throughout)
        const int cu = p.cu;
        const uint32_t stage_bytes = p.stage_bytes;
        // activations: staged for all of K (block index = the block in the group), or the stage's own slice
        // (block index = the unit's place in the chunk)
        const bool ring = p.ring;
        uint32_t actB = smem_u32(smem) + p.act_off;
        uint32_t actZ = smem_u32(smem) + p.act2_off;
        zero_acc();
        if (dbg) {  // timestamp of the first weights; the loop's own wait then passes at once
            if (!mbar_try(full0, 0)) alive = mbar_wait(full0, 0, abort_flag);
            if (tid == 0) dbg[3] = gtime_ns();
        }
        while (left > 0) {
            int n = nb - b < left ? nb - b : left;
            n = n < cu ? n : cu;
            if (alive && !mbar_test(full0 + 8 * s, ph) && !mbar_try(full0 + 8 * s, ph))
                alive = mbar_wait(full0 + 8 * s, ph, abort_flag);
            if (alive && !PROBE(2)) {
                const int b0 = ring ? warp : b + warp;   // block index of this warp's first unit
                if (n == kChunkUnits && NT == 1) {
                    // a full chunk: this warp's units are all loaded before the first tile, so that
                    // the shared-memory round trips of one unit run under the arithmetic of another
                    SUnit<BITS> un[kUPW];
#pragma unroll
                    for (int j = 0; j < kUPW; ++j) lds_unit<BITS, UK>(un[j], unit0 + j * kCW * UNIT, lane);
#pragma unroll
                    for (int j = 0; j < kUPW; ++j) {
                        if (MODE == MODE_A8) unit_a8<BITS, NT, UK>(un[j], actB, actZ, p, b0 + j * kCW, gid, tig, acc);
                        else unit_f<BITS, NT>(un[j], actB, p, b0 + j * kCW, gid, tig, acc);
                    }
                } else if (kUPW == 4 && n == kChunkUnits / 2 && NT == 1 && MODE == MODE_A8) {
                    SUnit<BITS> un[2];   // a full chunk of the half-size ring
#pragma unroll
                    for (int j = 0; j < 2; ++j) lds_unit<BITS, UK>(un[j], unit0 + j * kCW * UNIT, lane);
#pragma unroll
                    for (int j = 0; j < 2; ++j) unit_a8<BITS, NT, UK>(un[j], actB, actZ, p, b0 + j * kCW, gid, tig, acc);
                } else {
                    for (int j = 0; warp + j * kCW < n; ++j) {
                        SUnit<BITS> un;
                        lds_unit<BITS, UK>(un, unit0 + j * kCW * UNIT, lane);
                        if (MODE == MODE_A8) unit_a8<BITS, NT, UK>(un, actB, actZ, p, b0 + j * kCW, gid, tig, acc);
                        else unit_f<BITS, NT>(un, actB, p, b0 + j * kCW, gid, tig, acc);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + 8 * s);  // also when not alive: never block the producer
            b += n;
            left -= n;
            unit0 += stage_bytes;
            if (ring) { actB += stage_bytes; actZ += stage_bytes; }
            if (++s == NS) {
                s = 0;
                ph ^= 1u;
                unit0 -= (uint32_t)NS * stage_bytes;
                if (ring) { actB -= (uint32_t)NS * stage_bytes; actZ -= (uint32_t)NS * stage_bytes; }
            }
            if (b == nb || left == 0) {
                flush(g, seg_from, b);
                ++g;
                b = 0;
                seg_from = 0;
                zero_acc();
            }
        }
    }
#if RSTQ_PROBES
    if (fine) fine[0] = (unsigned long long)nfine;
#endif

    if (dbg && tid == 0) dbg[4] = gtime_ns();
    if (tid == 0 && s_abort) atomicExch(p.status, 1);
    if (dbg && tid == 0) dbg[5] = gtime_ns();

    // ---- fused exchange: wait for the other ranks' results, combine ----
    if (TP) {
        uint32_t* ctl = reinterpret_cast<uint32_t*>(tp_mine + 256);
        if (tid == 0) {
            s_tp_ok = 1;
            // every CTA read the epoch when it started; the last one to get here closes it
            if (atomicAdd(ctl + 1, 1u) == gridDim.x - 1) {
                ctl[1] = 0u;
                *reinterpret_cast<volatile uint32_t*>(ctl) = tp_e;
            }
        }
        consumer_bar();
        // this CTA's share of the result, two elements (one 16-byte load of two value/epoch
        // pairs) per thread and step; a pair is polled until it carries this exchange's epoch
        const int64_t row_pairs = p.out >> 1, pairs = (int64_t)M * row_pairs;
        // Only the first few thread blocks stay for it (p.tp_tail; 0 = all): the others leave their SMs to the
        // next launch, whose thread blocks fill their weight rings while this exchange is still under way.
        // (at least p.tp_tail of them, and enough for one pair per thread: measured on two GPUs, Llama-7B shapes,
        // all 115 blocks 5624 GB/s, 32 blocks 5859, 16 blocks 5817, 4 blocks 5348)
        int64_t tail = (pairs + kConsumers - 1) / kConsumers;
        tail = tail < p.tp_tail ? p.tp_tail : tail;
        if (p.tp_tail <= 0 || tail > (int64_t)gridDim.x) tail = gridDim.x;
        const int64_t per = (pairs + tail - 1) / tail;
        const int64_t q0 = min(pairs, per * blockIdx.x), q1 = blockIdx.x < tail ? min(pairs, q0 + per) : q0;
        const uint8_t* stage = tp_mine + tp_off;
        float2* dst = reinterpret_cast<float2*>(p.tp.y);
        const unsigned long long t0 = gtime_ns();
        bool ok = true;
        for (int64_t q = q0 + tid; q < q1 && ok; q += kConsumers) {
            const int64_t row = q / row_pairs, col = q - row * row_pairs;
            // All ranks' slots of this pair are read at once and only those that do not carry this
            // exchange's epoch yet are read again: one L2 round trip when everything has arrived,
            // instead of one per rank in a row.
            uint32_t v[kTpMaxRanks][4];
            uint32_t pend = (1u << tpn) - 1u;
            for (uint32_t spins = 1; pend; ++spins) {
#pragma unroll
                for (int r = 0; r < kTpMaxRanks; ++r)
                    if ((pend >> r) & 1u)
                        asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                                     : "=r"(v[r][0]), "=r"(v[r][1]), "=r"(v[r][2]), "=r"(v[r][3])
                                     : "l"(stage + (int64_t)r * p.tp.slot_bytes + q * 16)
                                     : "memory");
#pragma unroll
                for (int r = 0; r < kTpMaxRanks; ++r)
                    if (((pend >> r) & 1u) && v[r][1] == tp_e && v[r][3] == tp_e) pend &= ~(1u << r);
                if (pend && (spins & 63u) == 0 && (s_tp_ok == 0 || gtime_ns() - t0 > kWaitLimitNs)) {
                    ok = false;  // a rank never delivered: report, do not hang
                    s_tp_ok = 0;
                    atomicExch(p.status, 2);
                    break;
                }
            }
            if (!ok) break;
            if (p.tp.sum) {
                float2 acc = make_float2(__uint_as_float(v[0][0]), __uint_as_float(v[0][2]));
#pragma unroll
                for (int r = 1; r < kTpMaxRanks; ++r)   // rank order: the same sum on every rank
                    if (r < tpn) { acc.x += __uint_as_float(v[r][0]); acc.y += __uint_as_float(v[r][2]); }
                dst[q] = acc;
            } else {
#pragma unroll
                for (int r = 0; r < kTpMaxRanks; ++r)
                    if (r < tpn)
                        dst[(row * tpn + r) * row_pairs + col] = make_float2(__uint_as_float(v[r][0]), __uint_as_float(v[r][2]));
            }
        }
        if (dbg && tid == 0) dbg[7] = gtime_ns();
    }
}

// ---- host side --------------------------------------------------------------------------
struct StreamPlan {
    bool fits;
    int NS, G;
    int64_t uq, ur;
    uint32_t act_off, act2_off, red_off, bar_off;
    size_t smem;
    int cu, ring;           // units per chunk; the activations travel with the chunks (StreamParams::ring)
    uint32_t stage_bytes;
    int64_t in_flight() const { return (int64_t)(NS - 1) * cu; }   // units on their way while one chunk is consumed
};

// Measured on B200 at 14 shapes from 512x4096 to 28672x8192 (int4 and int8, M = 1..8): whole
// groups were faster every time, by 3 % (64 groups) to 37 % (Llama-7B shapes), even with only 32 of
// 148 SMs holding a CTA.  The equal-range split is kept for matrices so flat that a handful of
// CTAs would each have to stream many megabytes.
// Two token tiles (9 .. 16 tokens): the loop is bound by the consumers, so SMs left without a thread block cost
// their share: 70B-class matrices (7 groups per block, 128 of 148 SMs busy) gain 3 - 6 % from the equal-range
// split, the 7B shapes (3 groups per block) still lose 7 - 15 % to its hand-overs.
static bool whole_groups_pay(int64_t groups, int64_t nb, int64_t k, int64_t Gw, int sm_count, int unit, int nt) {
    (void)groups;
    const int64_t bytes_per_cta = k * nb * unit;
    if (nt >= 2 && Gw * 8 < sm_count * 7 && bytes_per_cta >= (1ll << 20)) return false;
    return !(Gw * 2 < sm_count && bytes_per_cta > (4ll << 20));
}

// How the units of a weight are cut over the CTAs of a launch: G ranges, CTA c owns uq (+1 if c < ur).
static void split_units(const DeviceState& ds, int bits, int64_t groups, int64_t nb, int* Gout, int64_t* uq,
                        int64_t* ur, int nt = 1) {
    const int kChunkUnits = chunk_units_of(bits);
    const int64_t U = groups * nb;
    int64_t G = (U + kChunkUnits - 1) / kChunkUnits;  // at least one chunk of work per CTA
    if (G > ds.sm_count) G = ds.sm_count;
    if (G < 1) G = 1;
    *Gout = (int)G;
    *uq = U / G;
    *ur = U % G;
    // Whole 32-row groups per CTA: no group is shared, nothing is handed over between CTAs.  Fewer
    // CTAs then stream more each; HBM stays the limit as long as enough SMs pull.
    const int64_t k = (groups + ds.sm_count - 1) / ds.sm_count;   // groups per CTA
    const int64_t Gw = (groups + k - 1) / k;
    bool whole = ds.gemv_plan == 2;
    if (ds.gemv_plan == 0) whole = whole_groups_pay(groups, nb, k, Gw, ds.sm_count, unit_bytes(bits), nt);
    if (whole && groups >= 1) {
        *Gout = (int)Gw;
        *uq = k * nb;
        *ur = 0;
    }
}

// cu: units per chunk (0: the full chunk of the unit kind).  ring: act_bytes / act2_bytes are the bytes PER UNIT
// of a chunk's slice of the activation image, which rides in the ring stage behind the weights.
static StreamPlan plan_stream(const DeviceState& ds, int bits, int NT, int64_t groups, int64_t nb,
                              int64_t act_bytes, int64_t act2_bytes, bool onecol = false, int cu = 0,
                              bool ring = false) {
    StreamPlan pl{};
    if (cu <= 0) cu = chunk_units_of(bits);
    const int chunk = cu * unit_bytes(bits);
    // reduction buffers ([warp][lane] at M = 1; [warp][value][lane] otherwise, two that alternate for one tile of tokens)
    const int64_t red = onecol ? (int64_t)(kParkGroups + 1) * kParkStride * 4 : (NT == 1 ? 2 : 1) * (int64_t)kCW * NT * 8 * 32 * 4;
    int64_t a1 = (act_bytes + 127) & ~127ll, a2 = (act2_bytes + 127) & ~127ll;
    int64_t stage = chunk, room;
    if (ring) {
        a1 = (act_bytes * cu + 127) & ~127ll;
        a2 = (act2_bytes * cu + 127) & ~127ll;
        stage = chunk + a1 + a2;
        room = kMaxDynSmem - (red + 512);
    } else {
        room = kMaxDynSmem - (a1 + a2 + red + 512);
    }
    int64_t ns = room / stage;
    if (ns > RSTQ_NSMAX) ns = RSTQ_NSMAX;
    pl.fits = ns >= 2;
    if (!pl.fits) return pl;
    split_units(ds, bits, groups, nb, &pl.G, &pl.uq, &pl.ur, onecol ? 1 : NT);
    pl.NS = (int)ns;
    pl.cu = cu;
    pl.ring = ring;
    pl.stage_bytes = (uint32_t)stage;
    if (ring) {
        pl.act_off = (uint32_t)chunk;            // inside every stage
        pl.act2_off = (uint32_t)(chunk + a1);
        pl.red_off = (uint32_t)(ns * stage);
    } else {
        pl.act_off = (uint32_t)(ns * chunk);
        pl.act2_off = pl.act_off + (uint32_t)a1;
        pl.red_off = pl.act2_off + (uint32_t)a2;
    }
    pl.bar_off = pl.red_off + (uint32_t)red;
    pl.smem = pl.bar_off + 2 * ns * 8 + 16;  // ring barriers + the activation image's
    return pl;
}

template <typename K>
static int32_t set_stream_attr(K kernel) {
    RSTQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynSmem));
    return RSTQ_OK;
}

int32_t gemv_configure(DeviceState& ds) {
    (void)ds;
    int32_t rc;
#define CFG(...) if ((rc = set_stream_attr(gemv_stream_kernel<__VA_ARGS__>)) != RSTQ_OK) return rc
    CFG(4, 1, MODE_A8, true, false);
    CFG(4, 1, MODE_A8, true, true);
    CFG(4, 1, MODE_A8, false, false);
    CFG(4, 1, MODE_A8, false, true);
    CFG(4, 2, MODE_A8, false, false);
    CFG(4, 2, MODE_A8, false, true);
    CFG(8, 1, MODE_A8, true, false);
    CFG(8, 1, MODE_A8, true, true);
    CFG(8, 1, MODE_A8, false, false);
    CFG(8, 1, MODE_A8, false, true);
    CFG(8, 2, MODE_A8, false, false);
    CFG(8, 2, MODE_A8, false, true);
    CFG(4, 1, MODE_F, false, false);
    CFG(4, 1, MODE_F, false, true);
    CFG(4, 2, MODE_F, false, false);
    CFG(4, 2, MODE_F, false, true);
    CFG(4, 4, MODE_F, false, false);
    CFG(4, 4, MODE_F, false, true);
    CFG(8, 1, MODE_F, false, false);
    CFG(8, 1, MODE_F, false, true);
    CFG(8, 2, MODE_F, false, false);
    CFG(8, 2, MODE_F, false, true);
    CFG(8, 4, MODE_F, false, false);
    CFG(8, 4, MODE_F, false, true);
#undef CFG
    // the M = 1 kernel with the activation quantizer inside
    if ((rc = set_stream_attr(gemv_stream_kernel<4, 1, MODE_A8, true, false, true>)) != RSTQ_OK) return rc;
    if ((rc = set_stream_attr(gemv_stream_kernel<4, 1, MODE_A8, true, true, true>)) != RSTQ_OK) return rc;
    if ((rc = set_stream_attr(gemv_stream_kernel<8, 1, MODE_A8, true, false, true>)) != RSTQ_OK) return rc;
    if ((rc = set_stream_attr(gemv_stream_kernel<8, 1, MODE_A8, true, true, true>)) != RSTQ_OK) return rc;
    // Q4_K units (minima inside)
    if ((rc = set_stream_attr(gemv_stream_kernel<4, 1, MODE_A8, true, false, false, 1>)) != RSTQ_OK) return rc;
    if ((rc = set_stream_attr(gemv_stream_kernel<4, 1, MODE_A8, false, false, false, 1>)) != RSTQ_OK) return rc;
    if ((rc = set_stream_attr(gemv_stream_kernel<4, 2, MODE_A8, false, false, false, 1>)) != RSTQ_OK) return rc;
    // Q6_K units (8-bit codes, a scale per 16 elements)
    if ((rc = set_stream_attr(gemv_stream_kernel<8, 1, MODE_A8, true, false, false, 2>)) != RSTQ_OK) return rc;
    if ((rc = set_stream_attr(gemv_stream_kernel<8, 1, MODE_A8, false, false, false, 2>)) != RSTQ_OK) return rc;
    if ((rc = set_stream_attr(gemv_stream_kernel<8, 2, MODE_A8, false, false, false, 2>)) != RSTQ_OK) return rc;
    return RSTQ_OK;
}

static int32_t stream_scratch_ok(const DeviceState& ds, int64_t groups, int G, int64_t M) {
    (void)groups;
    RSTQ_REQUIRE(G <= ds.counters_len - kPairTiles, RSTQ_E_LIMIT, "%d thread blocks exceed the %lld hand-over flags", G,
                 (long long)ds.counters_len);
    RSTQ_REQUIRE((int64_t)G * M * 32 * 4 <= ds.partials_bytes, RSTQ_E_LIMIT, "partials scratch too small");
    return RSTQ_OK;
}

static void fill_common(StreamParams& p, const DeviceState& ds, const StreamPlan& pl, int64_t in,
                        int64_t out, int M, int64_t nb, int zp, int bits_of_unit) {
    p.partials = ds.partials; p.flags = ds.counters; p.status = ds.status;
    // timeline: six launch slots of 160 CTA rows each, used in turn
    p.dbg = ds.dbg ? ds.dbg + (size_t)(ds.dbg_launch++ % 6) * 160 * 8 : nullptr;
    p.dbg_fine = ds.dbg ? ds.dbg + 6 * 160 * 8 : nullptr;
    p.in = in; p.out = out; p.uq = pl.uq; p.ur = pl.ur; p.U = ((out + 31) / 32) * nb;
    p.M = M; p.nb = (int)nb; p.G = pl.G; p.zp = zp; p.NS = pl.NS;
    // L2 requests ahead of the ring: by default 64 KB for matrices of 16 .. 64 MB (a CTA's range is then a
    // little longer than its ring: the chunks behind the ring would otherwise be requested only when the
    // consumers free slots); measured: smaller and, at one token, much larger matrices lose a little with any
    // distance; above one token (a shallower ring beside the activations) 64 KB gains 1 - 5 % at 147 MB too
    const int64_t wbytes = p.U * unit_bytes(bits_of_unit);
    p.pf_ahead = ds.gemv_prefetch_kb >= 0 ? ds.gemv_prefetch_kb << 10
                                          : (wbytes >= (16ll << 20) && (M > 1 || wbytes <= (64ll << 20)) ? 64ll << 10 : 0);
    p.probe = ds.gemv_probe;
    p.act_off = pl.act_off; p.act2_off = pl.act2_off; p.red_off = pl.red_off; p.bar_off = pl.bar_off;
    p.cu = pl.cu; p.ring = pl.ring; p.stage_bytes = pl.stage_bytes;
    p.tp_tail = ds.tp_tail_ctas;
}

// At most this much of the next launch's weight is requested into L2 ahead of time (the head of
// every thread block's range); larger matrices are HBM-bound anyway and must not flood the L2.
constexpr int64_t kNextPrefetchBytes = 48ll << 20;

static void fill_next(StreamParams& p, const DeviceState& ds, const NextWeight& n) {
    p.nx_w = nullptr;
    if (!n.data || n.groups < 1 || n.nb < 1) return;
    p.nx_w = n.data;
    p.nx_unit = unit_bytes(n.bits);
    p.nx_U = n.groups * n.nb;
    // (the next launch is taken to have this one's token tiles: a decode loop runs its matrices with one M)
    split_units(ds, n.bits, n.groups, n.nb, &p.nx_G, &p.nx_uq, &p.nx_ur, p.M * (p.T > 0 ? p.T : 1) <= 8 ? 1 : 2);
    const int64_t per_cta = kNextPrefetchBytes / p.nx_G / p.nx_unit;
    p.nx_pf_units = per_cta < 1 ? 1 : per_cta;
}

template <typename K>
static cudaError_t launch_stream(K kernel, const DeviceState& ds, const StreamPlan& pl,
                                 const StreamParams& p) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)pl.G);
    cfg.blockDim = dim3(kStreamThreads);
    cfg.dynamicSmemBytes = pl.smem;
    cfg.stream = ds.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ds.pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, p);
}

// Largest token count <= want whose staged activations fit next to a ring of >= 2 chunks.
template <typename BytesFn>
static int fit_tokens(const DeviceState& ds, int bits, int64_t groups, int64_t nb, int want, BytesFn f,
                      StreamPlan* out, bool a8 = false) {
    for (int m = want; m >= 1; --m) {
        int NT;
        int64_t a1, a2;
        f(m, &NT, &a1, &a2);
        StreamPlan pl = plan_stream(ds, bits, NT, groups, nb, a1, a2, a8 && m == 1);
        if (pl.fits) {
            *out = pl;
            return m;
        }
    }
    return 0;
}

// Mode A8, one launch: how many of `want` tokens it takes and with which plan.  uk = unit kind of the weight
// (GemvA8Args::uk); have_img: the quantizer's image of exactly these tokens exists; can_make: it can be built by
// act_image_kernel (one more small launch).  *make: the chosen plan needs that kernel.
// With the image at hand, the activations can travel with the weight chunks instead of staying in shared
// memory for all of K (StreamParams::ring).  Measured on B200, int4, 4096 <= K <= 28672: the ring is as fast as
// resident activations where those fit at the same depth and up to 3x faster where they do not; 32-unit chunks
// lose 10 - 30 % in either form and 48-unit ones 3 - 6 %, whatever depth they buy: above one token the loop is
// bound by the consumers, not by the bytes in flight.
static int plan_a8_piece(const DeviceState& ds, int uk, int bits, int64_t groups, int64_t nb, int want, bool have_img,
                         bool can_make, StreamPlan* pl, bool* make) {
    const bool k6 = uk == 2;
    const int ukind = uk == 1 ? 5 : (k6 ? 6 : bits);
    const int rec_bytes = uk == 1 ? 8 : kActRecBytes;   // of a (block, token) record: Q4_K units keep {xs, xs * code sum}
    auto bytes = [&](int m, int* NT, int64_t* a1, int64_t* a2) {
        *NT = m <= 8 ? 1 : 2;
        if (m == 1) { *a1 = nb * (k6 ? 128 : 64); *a2 = 0; }
        else { *a1 = nb * m * 32; *a2 = nb * ((m + 1) & ~1) * rec_bytes; }
    };
    *make = false;
    int M = fit_tokens(ds, ukind, groups, nb, want, bytes, pl, true);
    if (want <= 1) {
        // one token of a row so long that its staged record leaves no room for two ring stages (4-bit units:
        // K > ~57 K): the general kernel with the image riding the ring serves it
        if (M < 1 && (have_img || can_make) && ds.act_ring != 1 && ds.act_ring != 4) {
            const StreamPlan r = plan_stream(ds, ukind, 1, groups, nb, 32, 2 * rec_bytes, false, chunk_units_of(ukind), true);
            if (r.fits) {
                *pl = r;
                M = 1;
                *make = !have_img;
            }
        }
        return M;
    }
    const int full = chunk_units_of(ukind), half = full / 2, NTw = want <= 8 ? 1 : 2;
    const int64_t b1 = (int64_t)want * 32, b2 = (int64_t)((want + 1) & ~1) * rec_bytes;
    const bool imgs = have_img || can_make;
    const StreamPlan res_h = plan_stream(ds, ukind, NTw, groups, nb, nb * b1, nb * b2, false, half);
    const StreamPlan ring_f = imgs ? plan_stream(ds, ukind, NTw, groups, nb, b1, b2, false, full, true) : StreamPlan{};
    const StreamPlan ring_h = imgs ? plan_stream(ds, ukind, NTw, groups, nb, b1, b2, false, half, true) : StreamPlan{};
    const StreamPlan* pick = nullptr;
    switch (ds.act_ring) {
        case 1: break;
        case 2: if (ring_f.fits) pick = &ring_f; break;
        case 3: if (ring_h.fits) pick = &ring_h; break;
        case 4: if (res_h.fits) pick = &res_h; break;
        default:
            if (ring_f.fits && (have_img || M < want || ring_f.NS > pl->NS)) pick = &ring_f;
    }
    if (pick) {
        *pl = *pick;
        M = want;
        *make = pl->ring && !have_img;
    }
    return M;
}

static int plan_f_piece(const DeviceState& ds, int bits, int64_t groups, int64_t nb, int want, int act_dtype,
                        int* max_terms, bool ring_ok, StreamPlan* pl);

// What the decode kernel's launcher would do with the first launch of a call, as host arithmetic (rstq_decode_plan).
int32_t decode_plan(int mode, int bits, int64_t out, int64_t in, int64_t M, int act_dtype, int sm_count, int32_t* res) {
    DeviceState ds;
    ds.sm_count = sm_count;
    const int64_t nb = in / 32, groups = (out + 31) / 32;
    const int want = (int)(M < kGemvMaxM ? M : kGemvMaxM);
    StreamPlan pl{};
    int m;
    if (mode == MODE_A8) {
        bool make = false;
        // (the operator's quantizer lays the image out whenever it runs as a kernel of its own: above one token,
        // and at one token of a row longer than the in-kernel quantizer takes)
        m = plan_a8_piece(ds, 0, bits, groups, nb, want, want > 1 || in > kFusedQuantMaxIn, false, &pl, &make);
    } else {
        int max_terms = 3;
        m = plan_f_piece(ds, bits, groups, nb, want, act_dtype, &max_terms, true, &pl);
    }
    res[0] = m;
    res[1] = m >= 1 ? pl.NS : 0;
    res[2] = m >= 1 ? pl.cu : 0;
    res[3] = m >= 1 ? pl.ring : 0;
    res[4] = m >= 1 ? (int32_t)pl.smem : 0;
    res[5] = m >= 1 ? pl.G : 0;
    return RSTQ_OK;
}

int32_t launch_gemv_a8(rstq_ctx* ctx, DeviceState& ds, const GemvA8Args& a) {
    RSTQ_REQUIRE(a.M >= 1, RSTQ_E_SHAPE, "M = %lld", (long long)a.M);
    const int64_t nb = a.in / 32, groups = (a.out + 31) / 32;
    RSTQ_REQUIRE(nb < (1 << 24) && groups * nb < (1ll << 40), RSTQ_E_LIMIT, "matrix too large");
    const bool k6 = a.uk == 2;
    // unit kind for the size helpers: Q4_K units carry 128 more bytes than 4-bit ones, Q6_K units 128 more than 8-bit ones
    const int ukind = a.uk == 1 ? 5 : (k6 ? 6 : a.bits);
    RSTQ_REQUIRE(a.uk == 0 || (a.bits == (k6 ? 8 : 4) && !a.tp && !a.x), RSTQ_E_INVALID,
                 "K-quant units: one device, pre-quantized activations");
    for (int64_t m0 = 0; m0 < a.M;) {
        const int want = (int)(a.M - m0 < kGemvMaxM ? a.M - m0 : kGemvMaxM);
        StreamPlan pl;
        // the quantizer's image of this launch's tokens: laid out per kGemvMaxM tokens, so it serves a launch
        // that starts at such a boundary and takes all that is left up to the next
        const bool at_piece = a.img && a.uk == 0 && m0 % kGemvMaxM == 0 && (want > 1 || a.M == 1);
        const uint8_t* img = at_piece ? a.img + (m0 / kGemvMaxM) * act_image_stride(nb) : nullptr;
        const int rec_bytes = a.uk == 1 ? 8 : kActRecBytes;
        bool make = false;
        const bool can_make = !img && a.img_scratch && want == a.M;   // pre-quantized: one more small kernel
        int M = plan_a8_piece(ds, a.uk, a.bits, groups, nb, want, img != nullptr, can_make, &pl, &make);
        if (make) {
            int32_t rc = launch_act_image(ctx, ds, a.xq, a.xs, a.xsum, a.M, a.in, a.img_scratch, a.zp, a.bits, a.uk);
            if (rc != RSTQ_OK) return rc;
            img = a.img_scratch;
        }
        RSTQ_REQUIRE(M >= 1, RSTQ_E_LIMIT, "in = %lld: one row of activations exceeds shared memory",
                     (long long)a.in);
        if (a.tp && (M < a.M || a.out % 4 != 0)) return kNotFused;  // the exchange fuses into ONE launch
        const bool qf = a.x != nullptr;
        RSTQ_REQUIRE(!qf || (a.M == 1 && a.in <= kQuantMaxIn), RSTQ_E_INVALID,
                     "the in-kernel quantizer serves M = 1 and in <= %d", kQuantMaxIn);
        int32_t rc = stream_scratch_ok(ds, groups, pl.G, M);
        if (rc != RSTQ_OK) return rc;
        const int NT = M <= 8 ? 1 : 2;
        StreamParams p{};
        fill_common(p, ds, pl, a.in, a.out, M, nb, a.zp, ukind);
        p.w = a.w;
        p.kq = a.uk == 1;
        p.k6 = k6;
        if (qf) {
            p.x = a.x;
        } else {
            p.xq = a.xq + m0 * a.in;
            p.xs = a.xs + m0 * nb;
            p.xsum = a.xsum + m0 * nb * (k6 ? 2 : 1);   // Q6_K: sums per 16 elements
        }
        p.y = a.y + m0 * a.out;
        p.T = 1; p.act_dtype = qf ? a.act_dtype : RSTQ_F32; p.out_dtype = RSTQ_F32;
        if (M != want || (M == 1 && !pl.ring)) img = nullptr;   // fewer tokens than the image was laid out for; one token keeps its own record
        RSTQ_REQUIRE(!pl.ring || img, RSTQ_E_STATE, "a ring of activations without their image");
        if (img) {
            p.slice1 = (uint32_t)M * 32u;
            p.slice2 = (uint32_t)((M + 1) & ~1) * rec_bytes;
            p.img = img;
            p.img_b_bytes = (uint32_t)(nb * M * 32);
            p.img_z_bytes = (uint32_t)(nb * ((M + 1) & ~1) * rec_bytes);
            p.img_z_off = (p.img_b_bytes + 127u) & ~127u;
        }
        if (a.tp) p.tp = *a.tp;
        if (m0 + M >= a.M) fill_next(p, ds, a.next);   // the last piece of this call: what comes next is another weight
        cudaError_t le = cudaSuccess;
#define LAUNCH(...)                                                                  \
    le = a.tp ? launch_stream(gemv_stream_kernel<__VA_ARGS__, true>, ds, pl, p)      \
              : launch_stream(gemv_stream_kernel<__VA_ARGS__, false>, ds, pl, p)
#define LAUNCH1(B)                                                                                       \
    do {                                                                                                 \
        if (a.tp) le = qf ? launch_stream(gemv_stream_kernel<B, 1, MODE_A8, true, true, true>, ds, pl, p)  \
                          : launch_stream(gemv_stream_kernel<B, 1, MODE_A8, true, true, false>, ds, pl, p);\
        else le = qf ? launch_stream(gemv_stream_kernel<B, 1, MODE_A8, true, false, true>, ds, pl, p)      \
                     : launch_stream(gemv_stream_kernel<B, 1, MODE_A8, true, false, false>, ds, pl, p);    \
    } while (0)
        if (k6) {
            if (NT == 2) le = launch_stream(gemv_stream_kernel<8, 2, MODE_A8, false, false, false, 2>, ds, pl, p);
            else if (M == 1 && !pl.ring) le = launch_stream(gemv_stream_kernel<8, 1, MODE_A8, true, false, false, 2>, ds, pl, p);
            else le = launch_stream(gemv_stream_kernel<8, 1, MODE_A8, false, false, false, 2>, ds, pl, p);
        } else if (a.uk == 1) {
            if (NT == 2) le = launch_stream(gemv_stream_kernel<4, 2, MODE_A8, false, false, false, 1>, ds, pl, p);
            else if (M == 1 && !pl.ring) le = launch_stream(gemv_stream_kernel<4, 1, MODE_A8, true, false, false, 1>, ds, pl, p);
            else le = launch_stream(gemv_stream_kernel<4, 1, MODE_A8, false, false, false, 1>, ds, pl, p);
        } else if (a.bits == 4) {
            if (NT == 2) LAUNCH(4, 2, MODE_A8, false);
            else if (M == 1 && !pl.ring) LAUNCH1(4);
            else LAUNCH(4, 1, MODE_A8, false);
        } else {
            if (NT == 2) LAUNCH(8, 2, MODE_A8, false);
            else if (M == 1 && !pl.ring) LAUNCH1(8);
            else LAUNCH(8, 1, MODE_A8, false);
        }
#undef LAUNCH1
        ctx->launches++;
        RSTQ_CUDA(le);
        RSTQ_CUDA(cudaGetLastError());
        m0 += M;
    }
    return RSTQ_OK;
}

// Mode F, one launch: how many of `want` tokens it takes and with which plan.  f32 activations are expanded
// into exact bf16 terms: three while they fit one 8-column tile, else two (16 significant bits); a very long
// row may force two.  When shared memory cannot keep all of K for `want` tokens beside the ring, the staged
// array is built in global memory by a kernel of its own and rides the ring in slices (up to two column
// tiles: the slice of a chunk grows with the columns); `ring` off: fewer tokens per launch instead.
static int plan_f_piece(const DeviceState& ds, int bits, int64_t groups, int64_t nb, int want, int act_dtype,
                        int* max_terms, bool ring_ok, StreamPlan* pl) {
    auto terms = [&](int m) { return act_dtype == RSTQ_F32 ? ((3 * m <= 8 && *max_terms == 3) ? 3 : 2) : 1; };
    auto bytes = [&](int m, int* NT, int64_t* a1, int64_t* a2) {
        const int C = m * terms(m);
        *NT = C <= 8 ? 1 : (C <= 16 ? 2 : 4);
        *a1 = nb * 2 * C * 32;
        *a2 = 0;
    };
    int m = fit_tokens(ds, bits, groups, nb, want, bytes, pl);
    if (m < 1 && *max_terms == 3) {
        *max_terms = 2;  // a very long row: two bf16 terms (16 significant bits) per element
        m = fit_tokens(ds, bits, groups, nb, want, bytes, pl);
    }
    if (m < want && ring_ok && ds.act_ring != 1 && ds.act_ring != 4) {
        for (int mm = want; mm > m; --mm) {   // the most tokens whose columns of terms ride the ring
            const int C = mm * terms(mm);
            if (C > 16) continue;
            const int NT = C <= 8 ? 1 : 2, full = chunk_units_of(bits);
            StreamPlan r = plan_stream(ds, bits, NT, groups, nb, 2 * C * 32, 0, false, full, true);
            if (!r.fits || ds.act_ring == 3) r = plan_stream(ds, bits, NT, groups, nb, 2 * C * 32, 0, false, full / 2, true);
            if (r.fits) {
                *pl = r;
                m = mm;
                break;
            }
        }
    }
    return m;
}

// How many launches launch_gemv_f would make for M tokens (each streams all the weights again).
int gemv_f_pieces(const DeviceState& ds, int bits, int64_t out, int64_t in, int64_t M, int act_dtype) {
    const int64_t nb = in / 32, groups = (out + 31) / 32;
    int max_terms = 3;
    int pieces = 0;
    for (int64_t m0 = 0; m0 < M;) {
        const int want = (int)(M - m0 < kGemvMaxM ? M - m0 : kGemvMaxM);
        StreamPlan pl;
        const int m = plan_f_piece(ds, bits, groups, nb, want, act_dtype, &max_terms, true, &pl);
        if (m < 1) return 1 << 20;
        m0 += m;
        ++pieces;
    }
    return pieces;
}

// bytes of the staged array of mode F for one launch of up to kGemvMaxM tokens riding the ring (two column tiles)
int64_t gemv_f_image_bytes(int64_t in) { return (in / 32) * 2 * 16 * 32; }

int32_t launch_gemv_f(rstq_ctx* ctx, DeviceState& ds, const GemvFArgs& a) {
    RSTQ_REQUIRE(a.M >= 1, RSTQ_E_SHAPE, "M = %lld", (long long)a.M);
    const int64_t nb = a.in / 32, groups = (a.out + 31) / 32;
    RSTQ_REQUIRE(nb < (1 << 24) && groups * nb < (1ll << 40), RSTQ_E_LIMIT, "matrix too large");
    int max_terms = 3;
    const int64_t xe = a.act_dtype == RSTQ_F32 ? 4 : 2, ye = a.out_dtype == RSTQ_F32 ? 4 : 2;
    for (int64_t m0 = 0; m0 < a.M;) {
        const int want = (int)(a.M - m0 < kGemvMaxM ? a.M - m0 : kGemvMaxM);
        StreamPlan pl;
        const int M = plan_f_piece(ds, a.bits, groups, nb, want, a.act_dtype, &max_terms, a.img_scratch != nullptr, &pl);
        RSTQ_REQUIRE(M >= 1, RSTQ_E_LIMIT, "in = %lld: one row of activations exceeds shared memory",
                     (long long)a.in);
        if (a.tp && (M < a.M || a.out % 4 != 0 || a.out_dtype != RSTQ_F32)) return kNotFused;
        int32_t rc = stream_scratch_ok(ds, groups, pl.G, M);
        if (rc != RSTQ_OK) return rc;
        const int T = a.act_dtype == RSTQ_F32 ? ((3 * M <= 8 && max_terms == 3) ? 3 : 2) : 1, C = M * T;
        const int NT = C <= 8 ? 1 : (C <= 16 ? 2 : 4);
        StreamParams p{};
        fill_common(p, ds, pl, a.in, a.out, M, nb, a.zp, a.bits);
        p.w = a.w;
        p.x = (const char*)a.x + m0 * a.in * xe;
        p.y = (char*)a.y + m0 * a.out * ye;
        p.T = T; p.act_dtype = a.act_dtype; p.out_dtype = a.out_dtype;
        if (pl.ring) {
            // the staged array of this launch's tokens, built by a kernel of its own; the decode kernel's copy
            // thread waits for that grid before the first slice, as it does for the quantizer in mode A8
            const int64_t n = nb * 8 * C;
            int64_t ctas = (n + 255) / 256;
            if (ctas > (int64_t)ds.sm_count * 8) ctas = (int64_t)ds.sm_count * 8;
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3((unsigned)ctas);
            cfg.blockDim = dim3(256);
            cfg.stream = ds.stream;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[0].val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs = attr;
            cfg.numAttrs = ds.pdl ? 1 : 0;
            RSTQ_CUDA(cudaLaunchKernelEx(&cfg, act_image_f_kernel, p.x, reinterpret_cast<uint2*>(a.img_scratch), M, T,
                                         (int)nb, a.in, a.act_dtype));
            ctx->launches++;
            p.img = a.img_scratch;
            p.slice1 = (uint32_t)(2 * C * 32);
            p.slice2 = 0;
        }
        if (a.tp) p.tp = *a.tp;
        if (m0 + M >= a.M) fill_next(p, ds, a.next);   // the last piece of this call: what comes next is another weight
        cudaError_t le = cudaSuccess;
        if (a.bits == 4) {
            if (NT == 1) LAUNCH(4, 1, MODE_F, false);
            else if (NT == 2) LAUNCH(4, 2, MODE_F, false);
            else LAUNCH(4, 4, MODE_F, false);
        } else {
            if (NT == 1) LAUNCH(8, 1, MODE_F, false);
            else if (NT == 2) LAUNCH(8, 2, MODE_F, false);
            else LAUNCH(8, 4, MODE_F, false);
        }
#undef LAUNCH
        ctx->launches++;
        RSTQ_CUDA(le);
        RSTQ_CUDA(cudaGetLastError());
        m0 += M;
    }
    return RSTQ_OK;
}

}  // namespace rstq
