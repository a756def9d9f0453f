// Prefill-shape (M > 16) dequant-fused GEMM on the 5th-generation tensor cores.
//
// Replaces qmatmul-i8-gemm! (src/raster/quant/kernels_k.clj:344-370) and
// qlinear-q8 at large M (src/raster/quant/train.clj:77-108): where the
// reference runs one work-item per (token, output) with a serial K loop, this
// is a tiled tcgen05 GEMM:
//
//   D[128 features, NTOK tokens] (f32, in tensor memory)
//       += A[128, 128] (fp16, dequantized weights) * B[NTOK, 128]^T (fp16 activations)
//
//  * A is produced on the fly: 16 warps read the packed 4/8-bit codes and f32
//    block scales of the mma32 layout straight from global memory (register
//    prefetch four K-steps ahead, behind requests into L2 eight more ahead),
//    turn code and block scale into fp16 (exact integers times the rounded
//    scale) and hand them to the tensor core: gemm_tmem_kernel, the default,
//    stores them into a ring in tensor memory; gemm_tc_kernel stores 16-byte
//    rows into shared memory in the K-major 128-byte-swizzled layout.  fp16
//    (11-bit significand) rather than bf16 keeps the result within 1e-3 of the
//    f32 reference; a per-matrix power of two keeps scaled weights in fp16 range.
//  * B comes from a small pre-pass that rewrites the activations as fp16 with
//    one power-of-two exponent per token row (exact for bf16 inputs), loaded by
//    TMA (cp.async.bulk.tensor, 128-byte swizzle) by one producer thread.
//  * One thread (gemm_tmem_kernel: one of two, on alternate K-steps) issues
//    tcgen05.mma (cta_group::1, kind::f16, M = 128, N = NTOK, K = 16 per
//    instruction); tcgen05.commit releases a stage to the producers.
//  * The 16 dequant warps then read the accumulator with tcgen05.ld, undo the two
//    exponents and store y (f32 or bf16) row-major [token, feature].
// Every mbarrier wait is time-bounded; on expiry the CTA reports through the
// status word, drains and still frees its tensor memory.
#include <cuda.h>
#include <cuda_fp16.h>

#include "internal.h"
#include "mma_helpers.cuh"
#include "sync_helpers.cuh"

namespace rstq {

constexpr int kDqWarps = 16;
constexpr int kGemmThreads = (2 + kDqWarps) * 32;  // TMA warp, MMA warp, 16 dequant/epilogue warps
constexpr int kKStep = 128;                        // K elements per pipeline stage (4 blocks)
constexpr int kAStage = 128 * kKStep * 2;          // 32 KB of fp16 weights per stage
constexpr int kPrefetch = 4;                       // K-steps of packed weights held in registers

// ---- tcgen05 / TMA wrappers -------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{ .reg .pred p; setp.ne.b32 p, %4, 0; "
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// mbarrier arrives once all tcgen05.mma issued so far by this thread have completed
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
                   "=r"(r[7])
                 : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, "
        "%3}], [%4];" ::"r"(dst),
        "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void fence_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of 128 bytes
// (64 fp16), 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);  // start address
    d |= (uint64_t)1 << 16;                   // leading byte offset (unused with swizzle): 16 B
    d |= (uint64_t)(1024 >> 4) << 32;         // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                   // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                   // SWIZZLE_128B
    return d;
}
// Instruction descriptor of kind::f16: fp16 A and B (both K-major), f32 accumulate, M = 128.
__host__ __device__ constexpr uint32_t idesc_f16(int n) {
    return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

// ---- activation pre-pass: x (f32 / bf16 / int8 codes + block scales) -> fp16 * 2^-e(row) ---
// One CTA per token row.  rowscale[m] = 2^e so that max|x| * 2^-e lies in [2^13, 2^14).
template <int SRC>  // 0 = f32, 1 = bf16, 2 = int8 codes with per-32-block f32 scales
__global__ void __launch_bounds__(256)
act_to_f16_kernel(const void* __restrict__ x, const float* __restrict__ xs, __half* __restrict__ x16,
                  float* __restrict__ rowscale, int64_t in) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int64_t m = blockIdx.x;
    // eight consecutive elements (one 16-byte fp16 store) per thread and step
    auto load8 = [&](int64_t k, float (&v)[8]) {
        if (SRC == 0) {
            const float4* q = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + m * in + k);
            const float4 a = __ldg(q), b = __ldg(q + 1);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        } else if (SRC == 1) {
            const uint4 a = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(x) + m * in + k));
            const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                v[2 * j] = __uint_as_float(w[j] << 16);
                v[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
            }
        } else {
            const uint2 a = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const int8_t*>(x) + m * in + k));
            const float sc = __ldg(xs + m * (in >> 5) + (k >> 5));
            const uint32_t w[2] = {a.x, a.y};
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = (float)(int8_t)(w[j >> 2] >> (8 * (j & 3))) * sc;
        }
    };
    // Rows of up to 8192 elements stay in registers between the two passes (max, convert);
    // longer rows are read twice.
    constexpr int kKeep = 4;  // x 256 threads x 8 elements
    const bool keep = in <= (int64_t)kKeep * 256 * 8;
    float held[kKeep][8];
    float mx = 0.f;
    if (keep) {
#pragma unroll
        for (int i = 0; i < kKeep; ++i) {
            const int64_t k = (int64_t)(i * 256 + threadIdx.x) * 8;
            if (k < in) {
                load8(k, held[i]);
#pragma unroll
                for (int j = 0; j < 8; ++j) mx = fmaxf(mx, fabsf(held[i][j]));
            }
        }
    } else {
        for (int64_t k = threadIdx.x * 8; k < in; k += 256 * 8) {
            float v[8];
            load8(k, v);
#pragma unroll
            for (int j = 0; j < 8; ++j) mx = fmaxf(mx, fabsf(v[j]));
        }
    }
    __shared__ float s_mx[8];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if ((threadIdx.x & 31) == 0) s_mx[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = s_mx[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) mx = fmaxf(mx, s_mx[i]);
    int e = 0;
    if (mx > 0.f && mx < 3.0e38f) {
        int ex;
        frexpf(mx, &ex);  // mx = f * 2^ex, f in [0.5, 1)
        e = ex - 14;
    }
    const float down = ldexpf(1.0f, -e);
    auto store8 = [&](int64_t k, const float (&v)[8]) {
        uint32_t h[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const __half2 t = __floats2half2_rn(v[2 * j] * down, v[2 * j + 1] * down);
            h[j] = *reinterpret_cast<const uint32_t*>(&t);
        }
        *reinterpret_cast<uint4*>(x16 + m * in + k) = make_uint4(h[0], h[1], h[2], h[3]);
    };
    if (keep) {
#pragma unroll
        for (int i = 0; i < kKeep; ++i) {
            const int64_t k = (int64_t)(i * 256 + threadIdx.x) * 8;
            if (k < in) store8(k, held[i]);
        }
    } else {
        for (int64_t k = threadIdx.x * 8; k < in; k += 256 * 8) {
            float v[8];
            load8(k, v);
            store8(k, v);
        }
    }
    if (threadIdx.x == 0) rowscale[m] = ldexpf(1.0f, e);
}

// ---- the GEMM kernel ---------------------------------------------------------------------
constexpr int kNST = 3;  // pipeline stages

struct GemmParams {
    const uint8_t* w;       // mma32 units
    void* y;                // [M, out] f32 or bf16
    const float* rowscale;  // 2^e per token row (activation pre-pass)
    int* status;
    int64_t out;            // output features
    int nb, ngroups;        // K blocks per row, 32-row groups stored
    int M, ksteps, ttiles;
    int tiles, ksplit;      // feature x token tiles; K is cut into ksplit ranges of ksteps steps (last may be shorter)
    int ksteps_total;
    float* part;            // ksplit > 1 (gemm_tmem_kernel): the K range 1 CTA of a tile leaves its f32 accumulator
                            // here ([tile][warp][column][lane]), the K range 0 CTA adds it to its own and stores y
    int* pair_flags;        // one word per tile, zero between launches: set when `part` of the tile is complete
    float wmul, wdiv;       // 2^ew applied to the block scales, 2^-ew applied to the result
    int out_dtype;
    unsigned long long* dbg;  // optional timeline of CTA 0 (see RSTQ_TUNE_TIMELINE), or null
};

// packed weights of one dequant task, as loaded from global memory
template <int BITS>
struct RawW;
template <>
struct RawW<4> {
    uint2 a, b;  // slot 2t', 2t'+1: words (2q, 2q+1)
    float2 s;    // scales of rows gid + 16q, gid + 16q + 8
};
template <>
struct RawW<8> {
    uint4 a, b;  // plane p, slot 2t', 2t'+1: rows gid + 8i
    float4 s;
};

__device__ __forceinline__ uint32_t hsub_hmul(uint32_t v, uint32_t off, uint32_t scale2) {
    __half2 h = *reinterpret_cast<__half2*>(&v);
    h = __hmul2(__hsub2(h, *reinterpret_cast<__half2*>(&off)), *reinterpret_cast<__half2*>(&scale2));
    return *reinterpret_cast<uint32_t*>(&h);
}
// four unsigned bytes (each < 256) -> four fp16 (value - zero) * scale, in byte order
__device__ __forceinline__ uint2 bytes_to_h4(uint32_t bytes, uint32_t off, uint32_t scale2) {
    uint2 r;
    r.x = hsub_hmul(__byte_perm(bytes, 0x64646464u, 0x4140), off, scale2);
    r.y = hsub_hmul(__byte_perm(bytes, 0x64646464u, 0x4342), off, scale2);
    return r;
}
__device__ __forceinline__ uint32_t scale_h2(float s) {
    __half2 h = __half2half2(__float2half_rn(s));
    return *reinterpret_cast<uint32_t*>(&h);
}

// The conversion of gemm_tmem_kernel: one fused multiply-add per pair of weights.  A byte b placed
// in the low byte of a half (0x00bb) IS the fp16 subnormal b * 2^-24, so
//     fma(0x00bb, s, -zero * 2^-24 * s) = (b - zero) * s * 2^-24, rounded once:
// the product is exact inside the fma and the addend, a power of two times the already rounded
// scale s, is exact as well, which makes the result the same bits as subtracting the zero point
// first (exact integers) and multiplying by s afterwards, in half the instructions.  The caller
// folds the 2^-24 into the scale.
__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
// bytes 0..3 of `bytes` (other bits of each byte pair must be zero) -> four halves v * scale + add
__device__ __forceinline__ uint2 bytes_fma_h4(uint32_t bytes, uint32_t scale2, uint32_t add2) {
    uint2 r;
    r.x = hfma2_u32(__byte_perm(bytes, 0u, 0x4140), scale2, add2);
    r.y = hfma2_u32(__byte_perm(bytes, 0u, 0x4342), scale2, add2);
    return r;
}
constexpr int kSubnormalShift = 8;  // block scales carry 2^8 more: code * 2^-24 * (s * 2^8) stays in fp16 range

template <int BITS, int NTOK>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tc_kernel(const GemmParams p, const __grid_constant__ CUtensorMap tmap) {
    constexpr int UNIT = BITS == 4 ? kUnitBytesQ4 : kUnitBytesQ8;
    constexpr int CODES = BITS == 4 ? kUnitCodesQ4 : kUnitCodesQ8;
    constexpr int BSTAGE = NTOK * kKStep * 2;
    constexpr int STAGE = kAStage + BSTAGE;
    constexpr uint32_t TMEM_COLS = NTOK < 32 ? 32 : NTOK;
    extern __shared__ uint8_t smem_raw[];
    __shared__ int s_abort;
    __shared__ uint32_t s_tmem;
    __shared__ __align__(8) uint64_t s_bar[3 * kNST + 1];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // 128-byte swizzle atoms need 1024-byte alignment
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar0 = smem_u32(s_bar);
    const uint32_t full_a = bar0, full_b = bar0 + 8 * kNST, empty = bar0 + 16 * kNST, acc_full = bar0 + 24 * kNST;
    const int ft = blockIdx.x / p.ttiles, tt = blockIdx.x - ft * p.ttiles;
    const int tok0 = tt * NTOK;
    volatile int* abort_flag = &s_abort;

    if (tid < kNST) {
        mbar_init(full_a + 8 * tid, kDqWarps);
        mbar_init(full_b + 8 * tid, 1);
        mbar_init(empty + 8 * tid, 1);
    }
    if (tid == kNST) {
        mbar_init(acc_full, 1);
        s_abort = 0;
    }
    if (tid <= kNST) asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (warp == 1) {
        tmem_alloc(smem_u32(&s_tmem), TMEM_COLS);
        tmem_relinquish();
    }
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;
    const int ksteps = p.ksteps;

    if (warp == 0) {
        // ---------------- TMA producer of the activation tiles ----------------
        if (lane == 0) {
            asm volatile("griddepcontrol.wait;" ::: "memory");  // activations come from the pre-pass
            int s = 0, issued = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int ks = 0; ks < ksteps; ++ks) {
                ok = mbar_spin(empty + 8 * s, ph ^ 1u, abort_flag);
                if (!ok) break;
                const uint32_t dst = sbase + s * STAGE + kAStage;
                mbar_expect_tx(full_b + 8 * s, BSTAGE);
                tma_load_2d(dst, &tmap, ks * kKStep, tok0, full_b + 8 * s);
                tma_load_2d(dst + NTOK * 128, &tmap, ks * kKStep + 64, tok0, full_b + 8 * s);
                ++issued;
                if (++s == kNST) { s = 0; ph ^= 1u; }
            }
            if (!ok) {  // let the copies already issued land before this CTA's shared memory goes away
                for (int k = issued > kNST ? issued - kNST : 0; k < issued; ++k) {
                    const unsigned long long t0 = gtime_ns();
                    while (!mbar_try(full_b + 8 * (k % kNST), (uint32_t)(k / kNST) & 1u) &&
                           gtime_ns() - t0 < kWaitLimitNs) {
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = idesc_f16(NTOK);
            int s = 0;
            uint32_t ph = 0;
            bool ok = true, any = false;
            for (int ks = 0; ks < ksteps; ++ks) {
                ok = mbar_spin(full_a + 8 * s, ph, abort_flag) && mbar_spin(full_b + 8 * s, ph, abort_flag);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a0 = sbase + s * STAGE, b0 = a0 + kAStage;
#pragma unroll
                for (int kk = 0; kk < kKStep / 16; ++kk) {
                    const uint32_t aa = a0 + (kk >> 2) * (128 * 128) + (kk & 3) * 32;
                    const uint32_t bb = b0 + (kk >> 2) * (NTOK * 128) + (kk & 3) * 32;
                    umma_f16(tmem, smem_desc_sw128(aa), smem_desc_sw128(bb), idesc, (ks | kk) != 0);
                }
                any = true;
                umma_commit(empty + 8 * s);  // stage free once these MMAs have read it
                if (++s == kNST) { s = 0; ph ^= 1u; }
            }
            if (ok || any) {
                umma_commit(acc_full);
                if (!ok) {  // gave up: tensor core must be idle before tensor memory is freed
                    const unsigned long long t0 = gtime_ns();
                    while (!mbar_try(acc_full, 0) && gtime_ns() - t0 < kWaitLimitNs) {
                    }
                }
            }
        }
    } else {
        // ---------------- dequant warps: group = dq >> 2, block of the K-step = dq & 3 ----------------
        const int dq = warp - 2, grp = dq >> 2, sub = dq & 3;
        const int sel = (lane >> 4) & 1;  // 4-bit: row pair q; 8-bit: plane p
        const int tp = (lane >> 3) & 1, gid = lane & 7;
        const int64_t g_glob = (int64_t)ft * 4 + grp;
        const bool g_valid = g_glob < p.ngroups;
        // running pointer to this task's unit of the current prefetch K-step
        const uint8_t* wptr = p.w + (g_glob * p.nb + sub) * UNIT + (gid * 4 + 2 * tp) * 16 +
                              (BITS == 4 ? sel * 8 : sel * 512);
        const uint8_t* sptr = p.w + (g_glob * p.nb + sub) * UNIT + CODES + gid * 16 + (BITS == 4 ? sel * 8 : 0);
        int bk_next = sub;  // block index the next load refers to

        auto load = [&](RawW<BITS>& r) {
            if (g_valid && bk_next < p.nb) {
                if constexpr (BITS == 4) {
                    r.a = __ldg(reinterpret_cast<const uint2*>(wptr));
                    r.b = __ldg(reinterpret_cast<const uint2*>(wptr + 16));
                    r.s = __ldg(reinterpret_cast<const float2*>(sptr));
                } else {
                    r.a = __ldg(reinterpret_cast<const uint4*>(wptr));
                    r.b = __ldg(reinterpret_cast<const uint4*>(wptr + 16));
                    r.s = __ldg(reinterpret_cast<const float4*>(sptr));
                }
            } else {
                r = RawW<BITS>{};  // zero scale: rows / blocks beyond the matrix contribute 0
            }
            wptr += 4 * UNIT;
            sptr += 4 * UNIT;
            bk_next += 4;
        };
        // Shared-memory byte offsets of this task's 16-byte chunks inside a stage (K-major,
        // 128-byte swizzle: chunk c of row r sits at (r/8)*1024 + (r%8)*128 + ((c ^ r%8) * 16)).
        // Rows of one task differ by multiples of 8, so they share the xor and sit 1024 B apart.
        const uint32_t katom_off = (sub >> 1) * (128 * 128);
        uint32_t soff0, soff1;
        if (BITS == 4) {
            const uint32_t rbase = katom_off + (grp * 4 + 2 * sel) * 1024 + gid * 128;
            soff0 = rbase + (((4 * (sub & 1) + tp) ^ gid) << 4);      // h = 0
            soff1 = rbase + (((4 * (sub & 1) + 2 + tp) ^ gid) << 4);  // h = 1
        } else {
            soff0 = katom_off + (grp * 4) * 1024 + gid * 128 + (((4 * (sub & 1) + 2 * sel + tp) ^ gid) << 4);
            soff1 = 0;
        }
        const float wmul = p.wmul;
        auto convert = [&](const RawW<BITS>& r, uint32_t stage) {
            if constexpr (BITS == 4) {
                const uint32_t off = 0x64086408u;  // 1024 + zero point 8
                const uint32_t s_lo = scale_h2(r.s.x * wmul), s_hi = scale_h2(r.s.y * wmul);
                const uint32_t wa[2] = {r.a.x, r.a.y}, wb[2] = {r.b.x, r.b.y};
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint32_t dst = stage + (h ? soff1 : soff0);
                    const uint2 l0 = bytes_to_h4(wa[h] & 0x0F0F0F0Fu, off, s_lo);
                    const uint2 l1 = bytes_to_h4(wb[h] & 0x0F0F0F0Fu, off, s_lo);
                    sts128(dst, l0.x, l0.y, l1.x, l1.y);            // row gid + 16q
                    const uint2 h0 = bytes_to_h4((wa[h] >> 4) & 0x0F0F0F0Fu, off, s_hi);
                    const uint2 h1 = bytes_to_h4((wb[h] >> 4) & 0x0F0F0F0Fu, off, s_hi);
                    sts128(dst + 1024, h0.x, h0.y, h1.x, h1.y);     // row gid + 16q + 8
                }
            } else {
                const uint32_t off = 0x64806480u;  // 1024 + zero point 128
                const uint32_t wa[4] = {r.a.x, r.a.y, r.a.z, r.a.w}, wb[4] = {r.b.x, r.b.y, r.b.z, r.b.w};
                const float sc[4] = {r.s.x, r.s.y, r.s.z, r.s.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint32_t s2 = scale_h2(sc[i] * wmul);
                    const uint2 l0 = bytes_to_h4(wa[i], off, s2);
                    const uint2 l1 = bytes_to_h4(wb[i], off, s2);
                    sts128(stage + soff0 + i * 1024, l0.x, l0.y, l1.x, l1.y);  // row gid + 8i
                }
            }
        };

        RawW<BITS> raw[kPrefetch];
#pragma unroll
        for (int j = 0; j < kPrefetch; ++j) load(raw[j]);
        int s = 0;
        uint32_t ph = 0;
        bool ok = true;
        for (int ks0 = 0; ks0 < ksteps && ok; ks0 += kPrefetch) {
#pragma unroll
            for (int j = 0; j < kPrefetch; ++j) {
                const int ks = ks0 + j;
                if (ks < ksteps && ok) {
                    const bool got = mbar_spin(empty + 8 * s, ph ^ 1u, abort_flag);
                    ok = __all_sync(0xffffffffu, got);
                    if (ok) {
                        convert(raw[j], sbase + s * STAGE);
                        fence_async_smem();  // generic-proxy stores -> visible to the tensor core
                        __syncwarp();
                        if (lane == 0) mbar_arrive(full_a + 8 * s);
                        load(raw[j]);
                        if (++s == kNST) { s = 0; ph ^= 1u; }
                    }
                }
            }
        }

        // ---------------- epilogue: tensor memory -> y ----------------
        if (ok) {
            const bool got = mbar_spin(acc_full, 0, abort_flag);
            ok = __all_sync(0xffffffffu, got);
        }
        if (ok) {
            asm volatile("griddepcontrol.wait;" ::: "memory");  // y may still be read by the grid before us
            tc_fence_after();
            const int sp = warp & 3;          // tensor-memory lanes 32*sp .. 32*sp + 31
            const int cq = dq >> 2;           // column quarter
            const int64_t f = (int64_t)ft * 128 + sp * 32 + lane;
            constexpr int CPW = NTOK / 4;     // columns per warp
#pragma unroll
            for (int c0 = 0; c0 < CPW; c0 += 8) {
                uint32_t v[8];
                const int col = cq * CPW + c0;
                tmem_ld8(tmem + ((uint32_t)(sp * 32) << 16) + (uint32_t)col, v);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int tok = tok0 + col + j;
                    if (tok < p.M && f < p.out) {
                        const float val = __uint_as_float(v[j]) * p.wdiv * __ldg(p.rowscale + tok);
                        store_out(p.y, p.out_dtype, (int64_t)tok * p.out + f, val);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, TMEM_COLS);
    if (tid == 0 && s_abort) atomicExch(p.status, 2);
}

// ---- GEMM with the dequantized weights kept in tensor memory ------------------------------------
// Same tile and pipeline as gemm_tc_kernel, but A never touches shared memory: the
// tcgen05.st.16x256b fragment layout (lane = 4*gid + tig writes rows gid and gid + 8,
// 32-bit columns 2*tig and 2*tig + 1) is exactly how the mma32 layout hands a lane its 16-byte
// slot, so every lane converts its slot in registers and stores it to the A ring in tensor
// memory (64 columns per 128-element K-step); tcgen05.mma reads A from tensor memory and only B
// from shared memory, which halves the shared-memory traffic of the K loop.
// Warp roles: 0 = TMA (activations) and the L2 requests for the weights, 1 and 18 = MMA (even / odd
// K-steps), 2..17 = dequant, then epilogue: warp & 3 = 32-row group (= its tensor-memory
// sub-partition); t = (warp - 2) >> 2 picks, on whole K-steps, the set (t & 1: even / odd K-steps) and
// the pair of blocks (2 (t >> 1), + 1) of a K-step, otherwise the one block t of every K-step.
constexpr int kGemmThreadsT = (3 + kDqWarps) * 32;  // TMA warp, MMA warp (even K-steps), 16 dequant / epilogue warps, MMA warp (odd K-steps)
// pipeline stages (B in shared memory, A in tensor memory): what is left of the 512 columns after two
// accumulators, at most 4: with exactly four the dequant warps run their two-set schedule, which
// measured faster than six stages on the one-set schedule where six would fit (M <= 64: 76 -> 68 us
// at M = 16 on 28672 x 8192)
__host__ __device__ constexpr int gemm_stages(int ntok) { return ntok > 128 ? 3 : ((512 - 2 * ntok) / 64 > 4 ? 4 : (512 - 2 * ntok) / 64); }
// A 256-token tile has one accumulator (256 columns) and one issuing thread: an MMA then takes the
// tensor core 128 cycles, more than its issue costs; its activation stage is 64 KB, so three stages.
__host__ __device__ constexpr int gemm_issuers(int ntok) { return ntok > 128 ? 1 : 2; }
constexpr int kAColsPerStage = kKStep / 2;
constexpr int kWeightPfSteps = 8;  // K-steps of packed weights requested into L2 ahead of the loads

__device__ __forceinline__ void tmem_st_16x256b_x2(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.16x256b.x2.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr),
                 "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc], issued by the lanes whose `leader` is non-zero (one lane).
// The descriptor comes as two words so that stepping through a stage is one 32-bit add.
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t bdesc_lo, uint32_t bdesc_hi,
                                            uint32_t idesc, uint32_t accumulate, uint32_t leader) {
    asm volatile(
        "{ .reg .pred p, q; .reg .b64 bd; setp.ne.b32 p, %5, 0; setp.ne.b32 q, %6, 0; mov.b64 bd, {%2, %3}; "
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], bd, %4, p; }" ::"r"(d_tmem),
        "r"(a_tmem), "r"(bdesc_lo), "r"(bdesc_hi), "r"(idesc), "r"(accumulate), "r"(leader)
        : "memory");
}
// One 128-element K-step as a single block of instructions, so that nothing but a branch sits
// between the last MMA of a step and the first of the next: eight MMAs (A columns a0 + 8 kk, B
// descriptor b_lo + 2 (kk & 3) + BHALF (kk >> 2) in 16-byte units, BHALF = second 64-element half
// of the stage), with the two barrier operations of the pipeline tucked in between them where the
// issuing lane is waiting for the tensor core anyway: the commit that frees the PREVIOUS stage
// (it then also covers the first MMAs of this one, so that stage is released a little later,
// which the ring absorbs) and a non-blocking test of the NEXT stage's barrier, whose answer is
// read at the end.  first = 0 makes MMA 0 overwrite the accumulator; lanes with leader = 0
// issue no tensor-core instruction.
template <int BHALF>
__device__ __forceinline__ uint32_t umma_f16_ts_step(uint32_t d_tmem, uint32_t a0, uint32_t b_lo, uint32_t b_hi,
                                                     uint32_t idesc, uint32_t first, uint32_t leader,
                                                     uint32_t prev_empty, uint32_t commit_prev,
                                                     uint32_t next_full, uint32_t next_parity) {
    uint32_t next_ready;
    asm volatile(
        "{\n"
        ".reg .pred p, q, t, r, c;\n"
        ".reg .b64 bd0, bd1, bd2, bd3, bd4, bd5, bd6, bd7;\n"
        ".reg .b32 a1, a2, a3, a4, a5, a6, a7, b;\n"
        "setp.ne.b32 p, %6, 0;\n"
        "setp.ne.b32 q, %7, 0;\n"
        "setp.ne.b32 c, %13, 0;\n"
        "and.pred c, c, q;\n"
        "setp.eq.b32 t, 0, 0;\n"
        "mov.b64 bd0, {%3, %4};\n"
        "add.u32 a1, %2, 8;  add.u32 b, %3, 2;   mov.b64 bd1, {b, %4};\n"
        "add.u32 a2, %2, 16; add.u32 b, %3, 4;   mov.b64 bd2, {b, %4};\n"
        "add.u32 a3, %2, 24; add.u32 b, %3, 6;   mov.b64 bd3, {b, %4};\n"
        "add.u32 a4, %2, 32; add.u32 b, %3, %8;  mov.b64 bd4, {b, %4};\n"
        "add.u32 a5, %2, 40; add.u32 b, %3, %9;  mov.b64 bd5, {b, %4};\n"
        "add.u32 a6, %2, 48; add.u32 b, %3, %10; mov.b64 bd6, {b, %4};\n"
        "add.u32 a7, %2, 56; add.u32 b, %3, %11; mov.b64 bd7, {b, %4};\n"
        "tcgen05.fence::after_thread_sync;\n"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%1], [%2], bd0, %5, p;\n"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%1], [a1], bd1, %5, t;\n"
        "mbarrier.test_wait.parity.shared::cta.b64 r, [%14], %15;\n"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%1], [a2], bd2, %5, t;\n"
        "@c tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%12];\n"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%1], [a3], bd3, %5, t;\n"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%1], [a4], bd4, %5, t;\n"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%1], [a5], bd5, %5, t;\n"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%1], [a6], bd6, %5, t;\n"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%1], [a7], bd7, %5, t;\n"
        "selp.u32 %0, 1, 0, r;\n"
        "}"
        : "=r"(next_ready)
        : "r"(d_tmem), "r"(a0), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(first), "r"(leader), "n"(BHALF),
          "n"(BHALF + 2), "n"(BHALF + 4), "n"(BHALF + 6), "r"(prev_empty), "r"(commit_prev), "r"(next_full),
          "r"(next_parity)
        : "memory");
    return next_ready;
}
__device__ __forceinline__ void umma_commit_if(uint32_t bar, uint32_t leader) {
    asm volatile(
        "{ .reg .pred q; setp.ne.b32 q, %1, 0; "
        "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0]; }" ::"r"(bar),
        "r"(leader)
        : "memory");
}

template <int BITS>
struct RawT;
template <>
struct RawT<4> {
    uint4 c;    // the lane's slot: words 2q + h
    float4 s;   // scales of rows gid + 8i
};
template <>
struct RawT<8> {
    uint4 c0, c1;  // plane 0 / 1 slot: word i = row gid + 8i
    float4 s;
};

template <int BITS, int NTOK>
__global__ void __launch_bounds__(kGemmThreadsT, 1)
gemm_tmem_kernel(const GemmParams p, const __grid_constant__ CUtensorMap tmap) {
    constexpr int UNIT = BITS == 4 ? kUnitBytesQ4 : kUnitBytesQ8;
    constexpr int CODES = BITS == 4 ? kUnitCodesQ4 : kUnitCodesQ8;
    constexpr int BSTAGE = NTOK * kKStep * 2;
    constexpr int kNSTT = gemm_stages(NTOK);
    constexpr int ISS = gemm_issuers(NTOK);
    constexpr uint32_t TMEM_COLS = 512;                       // ISS accumulators (NTOK columns each) + A ring, power of two
    constexpr uint32_t A_COL0 = ISS * NTOK;                   // A ring starts after the accumulators
    static_assert(ISS * NTOK + kNSTT * kAColsPerStage <= 512 && kNSTT >= 3,
                  "tensor memory holds the accumulators and the A ring");
    extern __shared__ uint8_t smem_raw[];
    if (p.dbg && blockIdx.x == 0 && threadIdx.x == 64) { p.dbg[300] = (unsigned long long)clock64(); p.dbg[304] = gtime_ns(); }
    __shared__ int s_abort;
    __shared__ uint32_t s_tmem;
    __shared__ __align__(8) uint64_t s_bar[2 * 6 + 1];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar0 = smem_u32(s_bar);
    // full[s]: 16 dequant warps have stored A of the stage and the TMA bytes of B have landed;
    // empty[s]: the MMAs that read the stage have completed (tcgen05.commit)
    const uint32_t full = bar0, empty = bar0 + 8 * kNSTT, acc_full = bar0 + 16 * kNSTT;
    const int kz = blockIdx.x / p.tiles, tile = blockIdx.x - kz * p.tiles;  // K range, output tile
    const int ft = tile / p.ttiles, tt = tile - ft * p.ttiles;
    const int ks_begin = kz * p.ksteps;
    const int tok0 = tt * NTOK;
    volatile int* abort_flag = &s_abort;
    const int ksteps = min(p.ksteps, p.ksteps_total - ks_begin);

    // four-stage ring and whole K-steps: the dequant warps work as two sets of eight on alternate
    // K-steps (see there), so a stage collects eight arrivals instead of sixteen
    const bool paired = (p.nb & 3) == 0;
    if (tid == 0) asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap)) : "memory");
    if (paired && warp >= 2 && warp < 2 + kDqWarps) {
        // the first weights this warp will load: ask for them now, so that the HBM round trip
        // runs while the CTA sets itself up (barriers, tensor memory, the CTA-wide sync)
        const int t = (warp - 2) >> 2, pset = t & 1, blk0 = 2 * (t >> 1);
        int64_t g = (int64_t)ft * 4 + (warp & 3);
        g = g < p.ngroups ? g : (int64_t)p.ngroups - 1;
        const uint8_t* q = p.w + (g * p.nb + 4 * (ks_begin + pset) + blk0) * UNIT + lane * 128;
        if (lane * 128 < 2 * UNIT) {
#pragma unroll
            for (int d = 0; d < 2; ++d)
                if (pset + 2 * d < ksteps) asm volatile("prefetch.global.L2 [%0];" ::"l"(q + (size_t)d * 8 * UNIT));
        }
    }
    if (tid < kNSTT) {
        mbar_init(full + 8 * tid, (paired ? kDqWarps / 2 : kDqWarps) + 1);
        mbar_init(empty + 8 * tid, 1);
    } else if (tid == kNSTT) {
        mbar_init(acc_full, (ISS == 2 && ksteps >= 2) ? 2 : 1);  // one arrival per MMA issuer that has steps
        s_abort = 0;
    }
    if (tid <= kNSTT) asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (warp == 1) {
        tmem_alloc(smem_u32(&s_tmem), TMEM_COLS);
        tmem_relinquish();
    }
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;
    unsigned long long* dbg = (p.dbg && blockIdx.x == 0) ? p.dbg : nullptr;
    if (dbg && tid == 64) dbg[301] = (unsigned long long)clock64();

    if (warp == 0) {
        // ---------------- TMA producer of the activation tiles ----------------
        if (lane == 0) {
            // The dequant warps read the packed weights with plain loads a few K-steps ahead, which
            // covers an L2 round trip but not one to HBM.  This thread therefore asks for the
            // weights to be brought into L2 kPfSteps K-steps ahead of those loads, four K-steps (16
            // units, one contiguous run per row group) per request.
            constexpr int kPfSteps = kWeightPfSteps;
            const int nb_end = min(p.nb, 4 * (ks_begin + ksteps));
            auto request = [&](int ks) {  // K-steps ks .. ks + 3 of this CTA's range
                const int b0 = 4 * (ks_begin + ks);
                const int nblk = min(16, nb_end - b0);
                if (nblk <= 0) return;
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const int64_t gg = (int64_t)ft * 4 + g;
                    if (gg < p.ngroups) {
                        const uint8_t* q = p.w + (gg * p.nb + b0) * UNIT;
                        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(q), "r"((uint32_t)(nblk * UNIT))
                                     : "memory");
                    }
                }
            };
            asm volatile("griddepcontrol.wait;" ::: "memory");  // activations come from the pre-pass
            int s = 0, issued = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int ks = 0; ks < ksteps; ++ks) {
                // weight requests: none before the wait above (they would compete for HBM with the
                // pre-pass this kernel waits for) nor before the first activation tiles are on their
                // way; the dequant warps load K-steps 0 .. 3 themselves
                if (kPfSteps > 0 && ks == kNSTT)
                    for (int k2 = 4; k2 < 8 + kPfSteps; k2 += 4) request(k2);
                if (kPfSteps > 0 && (ks & 3) == 0 && ks >= 4) request(ks + 4 + kPfSteps);
                ok = mbar_block(empty + 8 * s, ph ^ 1u, abort_flag);
                if (!ok) break;
                const uint32_t dst = sbase + s * BSTAGE;
                mbar_expect_tx(full + 8 * s, BSTAGE);
                tma_load_2d(dst, &tmap, (ks_begin + ks) * kKStep, tok0, full + 8 * s);
                tma_load_2d(dst + NTOK * 128, &tmap, (ks_begin + ks) * kKStep + 64, tok0, full + 8 * s);
                ++issued;
                if (++s == kNSTT) { s = 0; ph ^= 1u; }
            }
            if (!ok) {  // let the copies already issued land before this CTA's shared memory goes away
                for (int k = issued > kNSTT ? issued - kNSTT : 0; k < issued; ++k) {
                    const unsigned long long t0 = gtime_ns();
                    while (!mbar_try(full + 8 * (k % kNSTT), (uint32_t)(k / kNSTT) & 1u) &&
                           gtime_ns() - t0 < kWaitLimitNs) {
                    }
                }
            }
        }
    } else if (warp == 1 || (ISS == 2 && warp == 2 + kDqWarps)) {
        // ---------------- MMA issuers ----------------
        // Issuing is what limits the tensor core here: a tcgen05 instruction costs the issuing
        // thread 50 - 60 cycles (measured: an MMA, a commit and a barrier test alike, whatever N
        // is), so the eight MMAs of a step plus its barrier work take one thread about 900 cycles
        // while the tensor core needs 512 for them.  Two warps on different schedulers therefore
        // take alternate K-steps, each into an accumulator of its own (the epilogue adds them);
        // each commits its own stages, so the rest of the pipeline does not notice.
        // The whole warp runs the loop with identical values (the address arithmetic stays
        // warp-uniform) and lane 0 alone issues the tensor-core instructions.
        const int m = warp == 1 ? 0 : 1;
        constexpr uint32_t idesc = idesc_f16(NTOK);
        const uint32_t leader = lane == 0;
        const uint64_t d0 = smem_desc_sw128(sbase);
        const uint32_t d_lo = (uint32_t)d0, d_hi = (uint32_t)(d0 >> 32);
        const uint32_t dcol = tmem + (uint32_t)(m * NTOK);
        static_assert(kKStep == 128, "eight MMAs per step");
        if (m < ksteps) {
            int s = m;
            uint32_t ph = 0;
            bool any = false;
            bool ok = mbar_spin(full + 8 * s, 0, abort_flag);
            if (dbg && lane == 0) dbg[306 + 2 * m] = (unsigned long long)clock64();
            for (int ks = m; ks < ksteps && ok; ks += ISS) {
                int s2 = s + ISS;
                uint32_t ph2 = ph;
                if (s2 >= kNSTT) { s2 -= kNSTT; ph2 ^= 1u; }
                const uint32_t a0 = tmem + A_COL0 + s * kAColsPerStage, b_lo = d_lo + (uint32_t)s * (BSTAGE >> 4);
                // the block also tests the barrier of this issuer's next step (ks + 2) early
                const uint32_t n2 = umma_f16_ts_step<NTOK * 8>(dcol, a0, b_lo, d_hi, idesc, ks != m, leader, empty, 0u,
                                                               full + 8 * s2, ph2);
                umma_commit_if(empty + 8 * s, leader);  // the stage is free once these MMAs have read it
                any = true;
                if (ks + ISS < ksteps && !n2) ok = mbar_spin(full + 8 * s2, ph2, abort_flag);
                    s = s2;
                ph = ph2;
            }
            if (dbg && lane == 0) dbg[307 + 2 * m] = (unsigned long long)clock64();
            if (any) {
                umma_commit_if(acc_full, leader);
                if (!ok) {  // gave up: the tensor core must be idle before tensor memory is freed
                    const unsigned long long t0 = gtime_ns();
                    while (!mbar_try(acc_full, 0) && gtime_ns() - t0 < kWaitLimitNs) {
                    }
                }
            }
        }
    } else if (warp == 2 + kDqWarps) {
        // the second issuer warp of the two-accumulator tiles: nothing to do on a 256-token tile
    } else {
        // ---------------- dequant warps ----------------
        const int dq = warp - 2, grp = warp & 3, sub = dq >> 2;
        const int gid = lane >> 2;
        const int64_t g_glob = (int64_t)ft * 4 + grp;
        const bool g_valid = g_glob < p.ngroups;
        const uint8_t* wptr = p.w + (g_glob * p.nb + sub + 4 * ks_begin) * UNIT + lane * 16;
        const uint8_t* sptr = p.w + (g_glob * p.nb + sub + 4 * ks_begin) * UNIT + CODES + gid * 16;
        int bk_next = sub + 4 * ks_begin;
        auto load = [&](RawT<BITS>& r) {
            if (g_valid && bk_next < p.nb) {
                if constexpr (BITS == 4) {
                    r.c = __ldg(reinterpret_cast<const uint4*>(wptr));
                } else {
                    r.c0 = __ldg(reinterpret_cast<const uint4*>(wptr));
                    r.c1 = __ldg(reinterpret_cast<const uint4*>(wptr + 512));
                }
                r.s = __ldg(reinterpret_cast<const float4*>(sptr));
            } else {
                r = RawT<BITS>{};  // zero scale: rows / blocks beyond the matrix contribute 0
            }
            wptr += 4 * UNIT;
            sptr += 4 * UNIT;
            bk_next += 4;
        };
        const float wmul = p.wmul;
        // this warp's rows are tensor-memory lanes 32*grp .. 32*grp + 31; its block is 16 columns wide
        const uint32_t t_lane = (uint32_t)(grp * 32) << 16;
        auto convert_store = [&](const RawT<BITS>& r, uint32_t a_stage, int blk) {
            const uint32_t dst = a_stage + t_lane + blk * 16;
            const float sc[4] = {r.s.x, r.s.y, r.s.z, r.s.w};
            if constexpr (BITS == 4) {
                constexpr uint32_t kZero = 0x80088008u;   // -8 * 2^-24 twice
                constexpr uint32_t kSixteenth = 0x2C002C00u;
                const uint32_t w[4] = {r.c.x, r.c.y, r.c.z, r.c.w};
#pragma unroll
                for (int q = 0; q < 2; ++q) {  // rows gid + 16q (low nibbles) and gid + 16q + 8 (high)
                    const uint32_t s_lo = scale_h2(sc[2 * q] * wmul), s_hi = scale_h2(sc[2 * q + 1] * wmul);
                    const uint32_t z_lo = hmul2_u32(s_lo, kZero), z_hi = hmul2_u32(s_hi, kZero);
                    const uint32_t s_hi16 = hmul2_u32(s_hi, kSixteenth);  // high nibbles stay where they are: 16 n
                    uint32_t v[8];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {  // columns 8h .. 8h + 7: elements 16h + 4tig ..
                        const uint2 lo = bytes_fma_h4(w[2 * q + h] & 0x0F0F0F0Fu, s_lo, z_lo);
                        const uint2 hi = bytes_fma_h4(w[2 * q + h] & 0xF0F0F0F0u, s_hi16, z_hi);
                        v[4 * h + 0] = lo.x;
                        v[4 * h + 1] = lo.y;
                        v[4 * h + 2] = hi.x;
                        v[4 * h + 3] = hi.y;
                    }
                    tmem_st_16x256b_x2(dst + ((uint32_t)(16 * q) << 16), v);
                }
            } else {
                constexpr uint32_t kZero = 0x80808080u;  // -128 * 2^-24 twice
                const uint32_t w0[4] = {r.c0.x, r.c0.y, r.c0.z, r.c0.w}, w1[4] = {r.c1.x, r.c1.y, r.c1.z, r.c1.w};
#pragma unroll
                for (int q = 0; q < 2; ++q) {  // rows gid + 16q (i = 2q) and gid + 16q + 8 (i = 2q + 1)
                    const uint32_t s_a = scale_h2(sc[2 * q] * wmul), s_b = scale_h2(sc[2 * q + 1] * wmul);
                    const uint32_t z_a = hmul2_u32(s_a, kZero), z_b = hmul2_u32(s_b, kZero);
                    uint32_t v[8];
                    const uint2 a0 = bytes_fma_h4(w0[2 * q], s_a, z_a), b0 = bytes_fma_h4(w0[2 * q + 1], s_b, z_b);
                    const uint2 a1 = bytes_fma_h4(w1[2 * q], s_a, z_a), b1 = bytes_fma_h4(w1[2 * q + 1], s_b, z_b);
                    v[0] = a0.x; v[1] = a0.y; v[2] = b0.x; v[3] = b0.y;   // plane 0: columns 0..7
                    v[4] = a1.x; v[5] = a1.y; v[6] = b1.x; v[7] = b1.y;   // plane 1: columns 8..15
                    tmem_st_16x256b_x2(dst + ((uint32_t)(16 * q) << 16), v);
                }
            }
        };
        // one K-step of this warp: wait for the stage, convert, store, hand over
        auto step = [&](const RawT<BITS>& r, int st, uint32_t parity) -> bool {
            if (!__all_sync(0xffffffffu, mbar_block(empty + 8 * st, parity, abort_flag))) return false;
            tc_fence_after();
            convert_store(r, tmem + A_COL0 + st * kAColsPerStage, sub);
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(full + 8 * st);
            return true;
        };

        bool ok = true;
        if (paired) {
            // Two sets of eight warps take alternate K-steps, a warp converting two adjacent
            // blocks of its row group per step: while one set converts, the other waits for its
            // stage or stores, so the issue slots do not idle between bursts, and the fixed cost
            // of a step (barrier test, store wait, arrival) is paid once per two units.
            // Own step i of set `pset` is K-step pset + 2i, stage pset + 2 (i & 1), ring pass i / 2.
            const int t = dq >> 2, pset = t & 1, blk0 = 2 * (t >> 1);
            const int n_own = (ksteps - pset + 1) >> 1;
            const int64_t g_ld = g_valid ? g_glob : (int64_t)p.ngroups - 1;
            const uint8_t* wl = p.w + (g_ld * p.nb + 4 * (ks_begin + pset) + blk0) * UNIT + lane * 16;
            const uint32_t s_delta = (uint32_t)(CODES + gid * 16 - lane * 16);
            auto fetch2 = [&](RawT<BITS> (&r)[2], int own_off) {
                const uint8_t* q = wl + (size_t)own_off * (8 * UNIT);
#pragma unroll
                for (int u = 0; u < 2; ++u, q += UNIT) {
                    if constexpr (BITS == 4) {
                        r[u].c = __ldg(reinterpret_cast<const uint4*>(q));
                    } else {
                        r[u].c0 = __ldg(reinterpret_cast<const uint4*>(q));
                        r[u].c1 = __ldg(reinterpret_cast<const uint4*>(q + 512));
                    }
                    r[u].s = __ldg(reinterpret_cast<const float4*>(q + s_delta));
                }
            };
            auto step2 = [&](const RawT<BITS> (&r)[2], int st, uint32_t parity) -> bool {
                if (!__all_sync(0xffffffffu, mbar_block(empty + 8 * st, parity, abort_flag))) return false;
                tc_fence_after();
                    const uint32_t a_stage = tmem + A_COL0 + st * kAColsPerStage;
                convert_store(r[0], a_stage, blk0);
                convert_store(r[1], a_stage, blk0 + 1);
                    tmem_st_wait();
                    tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(full + 8 * st);
                    return true;
            };
            RawT<BITS> raw[2][2];
#pragma unroll
            for (int d = 0; d < 2; ++d) {
                raw[d][0] = RawT<BITS>{};
                raw[d][1] = RawT<BITS>{};
                if (d < n_own) fetch2(raw[d], d);
            }
            // stage and "stage free" parity of K-step ks: ring position ks % stages, pass ks / stages
            // (the first pass finds every stage free: parity 1)
            auto stage_of = [&](int ks) { return ks % kNSTT; };
            auto parity_of = [&](int ks) { return (uint32_t)(((ks / kNSTT) & 1) ^ 1); };
            int i = 0;
            for (; i + 2 <= n_own && ok; i += 2) {
                const int ks = pset + 2 * i;
                ok = step2(raw[0], stage_of(ks), parity_of(ks));
                if (i + 2 < n_own) fetch2(raw[0], 2);
                if (ok) {
                    ok = step2(raw[1], stage_of(ks + 2), parity_of(ks + 2));
                    if (i + 3 < n_own) fetch2(raw[1], 3);
                }
                wl += (size_t)16 * UNIT;
            }
            if (ok && i < n_own) ok = step2(raw[0], stage_of(pset + 2 * i), parity_of(pset + 2 * i));
        } else {
            RawT<BITS> raw[kPrefetch];
#pragma unroll
            for (int j = 0; j < kPrefetch; ++j) load(raw[j]);
            int s = 0;
            uint32_t ph = 0;
            for (int ks0 = 0; ks0 < ksteps && ok; ks0 += kPrefetch) {
#pragma unroll
                for (int j = 0; j < kPrefetch; ++j) {
                    const int ks = ks0 + j;
                    if (ks < ksteps && ok) {
                        ok = step(raw[j], s, ph ^ 1u);
                        if (ok) {
                            load(raw[j]);
                            if (++s == kNSTT) { s = 0; ph ^= 1u; }
                        }
                    }
                }
            }
        }

        // ---------------- epilogue: tensor memory -> y ----------------
        // A warp owns 32 features (its tensor-memory lanes) x CPW tokens, handled CH <= 32 tokens at a
        // time.  Its token scales, one per lane and chunk, are fetched while the last MMAs run (the
        // pre-pass that wrote them completed before any activation tile was loaded).
        constexpr int CPW = NTOK / 4;                 // columns per warp
        constexpr int CH = CPW < 32 ? CPW : 32;       // columns per chunk
        constexpr int NCH = CPW / CH;
        const int cq = dq >> 2;                       // column quarter
        float rs_lane[NCH];
#pragma unroll
        for (int h = 0; h < NCH; ++h) rs_lane[h] = 0.f;
        if (ok) {
            asm volatile("griddepcontrol.wait;" ::: "memory");
#pragma unroll
            for (int h = 0; h < NCH; ++h) {
                const int tl = tok0 + cq * CPW + h * CH + lane;
                if (lane < CH && tl < p.M) rs_lane[h] = __ldg(p.rowscale + tl);
            }
        }
        if (ok) {
            const bool got = mbar_block(acc_full, 0, abort_flag);
            ok = __all_sync(0xffffffffu, got);
        }
        if (dbg && tid == 64) dbg[302] = (unsigned long long)clock64();
        // Two CTAs on one tile (each half of K): the K range 1 CTA hands its accumulator over through
        // L2, the K range 0 CTA adds it to its own (always a + b in this order) and writes y.
        const bool pair = p.ksplit > 1;
        const bool giver = pair && kz == 1, taker = pair && kz == 0;
        float* part = pair ? p.part + ((size_t)tile * kDqWarps + dq) * (CPW * 32) : nullptr;
        if (ok && taker) {
            int got = 1;
            if (lane == 0) {
                const unsigned long long t0 = gtime_ns();
                for (;;) {
                    int v;
                    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p.pair_flags + tile) : "memory");
                    if (v != 0) break;
                    if (*abort_flag || gtime_ns() - t0 > kWaitLimitNs) {
                        *abort_flag = 1;
                        got = 0;
                        break;
                    }
                    __nanosleep(64);
                }
            }
            ok = __shfl_sync(0xffffffffu, got, 0) != 0;
        }
        if (ok) {
            tc_fence_after();
            const int sp = warp & 3;          // tensor-memory lanes 32*sp .. 32*sp + 31
            const int64_t f = (int64_t)ft * 128 + sp * 32 + lane;
            const float wdiv = p.wdiv;
            constexpr int LD = 36;  // floats per token row of the staging tile (16-byte aligned rows)
            float* tile_s = reinterpret_cast<float*>(smem) + dq * (CH * LD);
#pragma unroll
            for (int h = 0; h < NCH; ++h) {
                // all loads of the chunk first, one wait, then the stores with the output type decided
                // once (a lane owns one feature: consecutive lanes write consecutive elements of a row)
                uint32_t v[CH];
                const uint32_t t0 = tmem + ((uint32_t)(sp * 32) << 16) + (uint32_t)(cq * CPW + h * CH);
#pragma unroll
                for (int c0 = 0; c0 < CH; c0 += 8) tmem_ld8(t0 + c0, *reinterpret_cast<uint32_t(*)[8]>(&v[c0]));
                tmem_ld_wait();
                if (ISS == 2 && ksteps >= 2) {  // the odd K-steps went into the second accumulator
                    uint32_t v2[CH];
#pragma unroll
                    for (int c0 = 0; c0 < CH; c0 += 8) tmem_ld8(t0 + NTOK + c0, *reinterpret_cast<uint32_t(*)[8]>(&v2[c0]));
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < CH; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(v2[j]));
                }
                const int tokb = tok0 + cq * CPW + h * CH;
                if (giver) {   // raw sums, 128 bytes per column and warp
#pragma unroll
                    for (int j = 0; j < CH; ++j) part[(h * CH + j) * 32 + lane] = __uint_as_float(v[j]);
                    continue;
                }
                if (taker) {
#pragma unroll
                    for (int j = 0; j < CH; ++j)
                        v[j] = __float_as_uint(__uint_as_float(v[j]) + __ldcg(part + (h * CH + j) * 32 + lane));
                }
                if ((p.out & 7) == 0) {
                    // Fast path: transpose the warp's 32-feature x CH-token tile through shared memory
                    // (the B ring is idle: every MMA has completed) so that a lane stores eight
                    // consecutive features of one token with one 16-byte (bf16) or two (f32) stores,
                    // instead of one element per store.
                    if (h) __syncwarp();   // the tile of the previous chunk has been read
#pragma unroll
                    for (int j = 0; j < CH; ++j) tile_s[j * LD + lane] = __uint_as_float(v[j]);
                    __syncwarp();
                    const int fg = (lane & 3) * 8;
                    const int64_t f0 = (int64_t)ft * 128 + sp * 32 + fg;
#pragma unroll
                    for (int t0c = 0; t0c < CH; t0c += 8) {
                        const int t = t0c + (lane >> 2), tok = tokb + t;
                        const float sc = wdiv * __shfl_sync(0xffffffffu, rs_lane[h], t);
                        if (tok < p.M && f0 < p.out) {
                            const float4 a = *reinterpret_cast<const float4*>(tile_s + t * LD + fg);
                            const float4 c = *reinterpret_cast<const float4*>(tile_s + t * LD + fg + 4);
                            if (p.out_dtype == RSTQ_BF16) {
                                uint4 o;
                                o.x = pack_bf16x2(a.y * sc, a.x * sc);
                                o.y = pack_bf16x2(a.w * sc, a.z * sc);
                                o.z = pack_bf16x2(c.y * sc, c.x * sc);
                                o.w = pack_bf16x2(c.w * sc, c.z * sc);
                                *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.y) + (int64_t)tok * p.out + f0) = o;
                            } else {
                                float* y = reinterpret_cast<float*>(p.y) + (int64_t)tok * p.out + f0;
                                *reinterpret_cast<float4*>(y) = make_float4(a.x * sc, a.y * sc, a.z * sc, a.w * sc);
                                *reinterpret_cast<float4*>(y + 4) = make_float4(c.x * sc, c.y * sc, c.z * sc, c.w * sc);
                            }
                        }
                    }
                } else {
                    // one element per store (a lane owns one feature)
                    const bool f_ok = f < p.out;
#pragma unroll
                    for (int j = 0; j < CH; ++j) {
                        const float val = __uint_as_float(v[j]) * wdiv * __shfl_sync(0xffffffffu, rs_lane[h], j);
                        if (f_ok && tokb + j < p.M) {
                            store_out(p.y, p.out_dtype, (int64_t)(tokb + j) * p.out + f, val);
                        }
                    }
                }
            }
        }
        if (pair) {
            // giver: every warp's part is out before the flag goes up; taker: every warp has read its
            // part before the flag goes down again (the next launch's giver writes only after this
            // grid has completed).  All sixteen warps meet here whether or not a wait ran out.
            if (giver && ok) __threadfence();
            asm volatile("bar.sync 6, %0;" ::"r"(kDqWarps * 32) : "memory");
            if (dq == 0 && lane == 0) {
                if (taker) p.pair_flags[tile] = 0;
                else if (ok) asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p.pair_flags + tile), "r"(1) : "memory");
            }
        }
    }
    if (dbg && tid == 64) { dbg[303] = (unsigned long long)clock64(); dbg[305] = gtime_ns(); }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, TMEM_COLS);
    if (tid == 0 && s_abort) atomicExch(p.status, 2);
}

// ---- host side --------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

template <int BITS, int NTOK>
static int32_t gemm_attr() {
    if constexpr (NTOK <= 128)
        RSTQ_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<BITS, NTOK>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       kNST * (kAStage + NTOK * kKStep * 2) + 1024));
    RSTQ_CUDA(cudaFuncSetAttribute(gemm_tmem_kernel<BITS, NTOK>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   gemm_stages(NTOK) * (NTOK * kKStep * 2) + 1024));
    return RSTQ_OK;
}

int32_t gemm_configure(DeviceState& ds) {
    (void)ds;
    int32_t rc;
    if ((rc = gemm_attr<4, 32>()) != RSTQ_OK) return rc;
    if ((rc = gemm_attr<4, 64>()) != RSTQ_OK) return rc;
    if ((rc = gemm_attr<4, 128>()) != RSTQ_OK) return rc;
    if ((rc = gemm_attr<8, 32>()) != RSTQ_OK) return rc;
    if ((rc = gemm_attr<8, 64>()) != RSTQ_OK) return rc;
    if ((rc = gemm_attr<8, 128>()) != RSTQ_OK) return rc;
    if ((rc = gemm_attr<4, 256>()) != RSTQ_OK) return rc;
    if ((rc = gemm_attr<8, 256>()) != RSTQ_OK) return rc;
    return RSTQ_OK;
}

template <typename K, typename... Args>
static cudaError_t launch_pdl(K kernel, dim3 grid, dim3 block, size_t smem, const DeviceState& ds,
                              Args... args) {
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

// x (src 0 = f32, 1 = bf16, 2 = int8 codes with per-block scales xs) -> fp16 rows x16 and 2^e per row
static int32_t launch_act_to_f16(rstq_ctx* ctx, DeviceState& ds, const void* x, const float* xs, int src, void* x16,
                                 float* rowscale, int64_t M, int64_t in) {
    cudaError_t le;
    const dim3 grid((unsigned)M), block(256);
    if (src == 0)
        le = launch_pdl(act_to_f16_kernel<0>, grid, block, 0, ds, x, xs, (__half*)x16, rowscale, in);
    else if (src == 1)
        le = launch_pdl(act_to_f16_kernel<1>, grid, block, 0, ds, x, xs, (__half*)x16, rowscale, in);
    else
        le = launch_pdl(act_to_f16_kernel<2>, grid, block, 0, ds, x, xs, (__half*)x16, rowscale, in);
    ctx->launches++;
    RSTQ_CUDA(le);
    return RSTQ_OK;
}

// Token-tile width and split along K of a prefill GEMM on a device of `sm_count` SMs: whichever of
// 128- / 256-wide tiles, one or two CTAs per tile, needs the fewest cycles over the waves of CTAs
// the grid makes.  `tmem_kernel`: the call runs gemm_tmem_kernel with a pair scratch (wide tiles and
// the split exist only there); `wide`: RSTQ_TUNE_GEMM_WIDE.
// (measured: a 128-wide K-step 690 cycles; a 256-wide one 1140 with 64 CTAs running, 1240 with 96,
// 1400 with all 148 -- their activation tiles are twice as large and all come from L2; set-up, first
// loads and epilogue of a CTA about 8000 resp. 9000 cycles; the hand-over of a pair about 1500)
void gemm_plan(int64_t out, int64_t in, int64_t M, int sm_count, bool tmem_kernel, int wide, int* ntok_out,
               bool* split_out) {
    const int64_t ftiles = (out + 127) / 128, sm = sm_count > 0 ? sm_count : 1;
    const int64_t ksteps_total = (in / 32 + 3) / 4;
    auto cycles = [&](int nt, bool* split) {
        const int64_t tiles = ftiles * ((M + nt - 1) / nt);
        *split = tmem_kernel && tiles * 2 <= sm && tiles <= kPairTiles && ksteps_total >= 16 && wide != 3;
        const int64_t ctas = *split ? tiles * 2 : tiles, active = ctas < sm ? ctas : sm;
        const int64_t c = nt == 256 ? 1140 + (active > 64 ? (active - 64) * 31 / 10 : 0) : 690;
        const int64_t fixed = nt == 256 ? 9000 : 8000;
        return *split ? (ksteps_total + 1) / 2 * c + 1500 + fixed : (tiles + sm - 1) / sm * (ksteps_total * c + fixed);
    };
    int ntok = M <= 32 ? 32 : (M <= 64 ? 64 : 128);
    bool split = false;
    const int64_t c_narrow = cycles(ntok, &split);
    if (M > 128 && tmem_kernel && wide != 1) {
        bool split_w = false;
        const int64_t c_wide = cycles(256, &split_w);
        if (wide == 2 || c_wide < c_narrow) {
            ntok = 256;
            split = split_w;
        }
    }
    *ntok_out = ntok;
    *split_out = split;
}

// y[M, out] = x[M, in] . dequant(W)^T on the tensor cores.  src: 0 = f32 x, 1 = bf16 x,
// 2 = int8 codes x with per-block scales xs.  x16 / rowscale are caller-provided scratch
// (M*in fp16, M floats).
int32_t launch_gemm(rstq_ctx* ctx, DeviceState& ds, const rstq_weight* w, const void* x, const float* xs,
                    int src, void* y, int out_dtype, int64_t M, void* x16, float* rowscale, float* acc32) {
    RSTQ_REQUIRE(M >= 1 && M < (1ll << 30), RSTQ_E_SHAPE, "M = %lld", (long long)M);
    RSTQ_REQUIRE(((uintptr_t)x16 & 15) == 0 && (w->in * 2) % 16 == 0, RSTQ_E_ALIGN,
                 "activation scratch must be 16-byte aligned");
    EncodeTiledFn enc = encode_tiled_fn();
    RSTQ_REQUIRE(enc, RSTQ_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const bool a_in_tmem = ctx->tune_gemm_kernel != 1;
    // Token-tile width and the split along K.  Above 128 tokens a tile may be 256 wide (gemm_tmem_kernel
    // only): the K loop is bound by the issue of the tensor-core instructions, and an instruction of
    // twice the width does twice the work -- a K-step of a 256-wide tile takes 1140 cycles against
    // 690 of a 128-wide one (measured) -- but halves the number of tiles.  When a grid would fill at
    // most half the SMs and K is long, two CTAs share a tile, each taking half of K; the second hands
    // its accumulator to the first through L2 (about 1500 cycles).  Whichever combination needs the
    // fewest cycles over the waves of CTAs it makes on this device is taken (4096 features: M <= 256: 128
    // wide, split; M = 512: 128 wide, one wave of 128 tiles; M = 768: 256 wide, one wave of 96 tiles
    // instead of two of 192; M >= 1024: 256 wide).
    const int64_t ftiles = (w->out + 127) / 128;
    int ntok = 128;
    bool split = false;
    gemm_plan(w->out, w->in, M, ds.sm_count, a_in_tmem && acc32 != nullptr, (int)ctx->tune_gemm_wide, &ntok, &split);
    // pre-pass: activations -> fp16 with one exponent per token row.  kind::f16 wants A and B of
    // one type (fp16 weights against bf16 activations raise "illegal instruction"), and fp16 on
    // both sides keeps three more mantissa bits of the weights than bf16 would.
    int32_t rc = launch_act_to_f16(ctx, ds, x, xs, src, x16, rowscale, M, w->in);
    if (rc != RSTQ_OK) return rc;
    cudaError_t le;

    CUtensorMap tmap;
    const cuuint64_t dims[2] = {(cuuint64_t)w->in, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)w->in * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)ntok};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult cr = enc(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, x16, dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    RSTQ_REQUIRE(cr == CUDA_SUCCESS, RSTQ_E_CUDA, "cuTensorMapEncodeTiled failed with %d", (int)cr);

    GemmParams p{};
    p.w = w->data;
    p.y = y;
    p.rowscale = rowscale;
    p.status = ds.status;
    p.out = w->out;
    p.nb = (int)w->nb;
    p.ngroups = (int)(w->outp / 32);
    p.M = (int)M;
    p.ksteps_total = (int)((w->nb + 3) / 4);
    p.ttiles = (int)((M + ntok - 1) / ntok);
    // gemm_tmem_kernel converts codes as fp16 subnormals (code * 2^-24): its block scales carry
    // 2^kSubnormalShift more and the result the remaining 2^(24 - kSubnormalShift)
    p.wmul = ldexpf(1.0f, w->gemm_exp + (a_in_tmem ? kSubnormalShift : 0));
    p.wdiv = ldexpf(1.0f, -w->gemm_exp + (a_in_tmem ? 24 - kSubnormalShift : 0));
    p.out_dtype = out_dtype;
    p.dbg = ds.dbg;
    RSTQ_REQUIRE(ftiles * p.ttiles < (1ll << 30), RSTQ_E_LIMIT, "grid too large");
    p.tiles = (int)(ftiles * p.ttiles);
    p.ksplit = split ? 2 : 1;
    p.ksteps = (p.ksteps_total + p.ksplit - 1) / p.ksplit;
    p.part = split ? acc32 : nullptr;   // [tile][16 warps][columns per warp][32 lanes] f32: tiles * 128 * ntok floats
    p.pair_flags = ds.counters + ds.counters_len - kPairTiles;
    const dim3 grid((unsigned)(p.tiles * p.ksplit));
    const size_t smem = a_in_tmem ? gemm_stages(ntok) * ((size_t)ntok * kKStep * 2) + 1024
                                  : kNST * (kAStage + (size_t)ntok * kKStep * 2) + 1024;
#define GL(B, N)                                                                                     \
    le = a_in_tmem ? launch_pdl(gemm_tmem_kernel<B, N>, grid, dim3(kGemmThreadsT), smem, ds, p, tmap) \
                   : launch_pdl(gemm_tc_kernel<B, N>, grid, dim3(kGemmThreads), smem, ds, p, tmap)
    if (w->bits == 4) {
        if (ntok == 32) GL(4, 32);
        else if (ntok == 64) GL(4, 64);
        else if (ntok == 128) GL(4, 128);
        else le = launch_pdl(gemm_tmem_kernel<4, 256>, grid, dim3(kGemmThreadsT), smem, ds, p, tmap);
    } else {
        if (ntok == 32) GL(8, 32);
        else if (ntok == 64) GL(8, 64);
        else if (ntok == 128) GL(8, 128);
        else le = launch_pdl(gemm_tmem_kernel<8, 256>, grid, dim3(kGemmThreadsT), smem, ds, p, tmap);
    }
#undef GL
    ctx->launches++;
    RSTQ_CUDA(le);
    RSTQ_CUDA(cudaGetLastError());
    return RSTQ_OK;
}

}  // namespace rstq
