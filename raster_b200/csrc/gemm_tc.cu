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
//    prefetch three K-steps ahead), convert code -> fp16 with the 0x6400 magic
//    (exact integers), multiply by the block scale and store 16-byte rows into
//    shared memory in the K-major 128-byte-swizzled layout the tensor core
//    reads.  fp16 (11-bit significand) rather than bf16 keeps the result within
//    1e-3 of the f32 reference; a per-matrix power of two keeps scaled weights
//    in fp16 range.
//  * B comes from a small pre-pass that rewrites the activations as fp16 with
//    one power-of-two exponent per token row (exact for bf16 inputs), loaded by
//    TMA (cp.async.bulk.tensor, 128-byte swizzle) by one producer thread.
//  * One thread issues tcgen05.mma (cta_group::1, kind::f16, M = 128, N = NTOK,
//    K = 16 per instruction); tcgen05.commit releases a stage to the producers.
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
constexpr int kPrefetch = 3;                       // K-steps of packed weights held in registers

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
    auto value = [&](int64_t k) -> float {
        if (SRC == 0) return reinterpret_cast<const float*>(x)[m * in + k];
        if (SRC == 1) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(x)[m * in + k]);
        return (float)reinterpret_cast<const int8_t*>(x)[m * in + k] * xs[m * (in >> 5) + (k >> 5)];
    };
    float mx = 0.f;
    for (int64_t k = threadIdx.x; k < in; k += 256) mx = fmaxf(mx, fabsf(value(k)));
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
    for (int64_t k = threadIdx.x; k < in; k += 256) x16[m * in + k] = __float2half_rn(value(k) * down);
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
    float wmul, wdiv;       // 2^ew applied to the block scales, 2^-ew applied to the result
    int out_dtype;
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
                ok = mbar_try(empty + 8 * s, ph ^ 1u) || mbar_wait(empty + 8 * s, ph ^ 1u, abort_flag);
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
                ok = mbar_try(full_a + 8 * s, ph) || mbar_wait(full_a + 8 * s, ph, abort_flag);
                if (ok) ok = mbar_try(full_b + 8 * s, ph) || mbar_wait(full_b + 8 * s, ph, abort_flag);
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
        const uint8_t* wg = p.w + g_glob * p.nb * UNIT;
        const int slot_off = (gid * 4 + 2 * tp) * 16;

        auto load = [&](RawW<BITS>& r, int ks) {
            const int bk = ks * 4 + sub;
            if (g_valid && bk < p.nb && ks < ksteps) {
                const uint8_t* u = wg + (int64_t)bk * UNIT;
                if constexpr (BITS == 4) {
                    RawW<4>& q = r;
                    q.a = __ldg(reinterpret_cast<const uint2*>(u + slot_off + sel * 8));
                    q.b = __ldg(reinterpret_cast<const uint2*>(u + slot_off + 16 + sel * 8));
                    q.s = __ldg(reinterpret_cast<const float2*>(u + CODES + gid * 16 + sel * 8));
                } else {
                    RawW<8>& q = r;
                    q.a = __ldg(reinterpret_cast<const uint4*>(u + sel * 512 + slot_off));
                    q.b = __ldg(reinterpret_cast<const uint4*>(u + sel * 512 + slot_off + 16));
                    q.s = __ldg(reinterpret_cast<const float4*>(u + CODES + gid * 16));
                }
            } else {
                r = RawW<BITS>{};  // zero scale: rows / blocks beyond the matrix contribute 0
            }
        };
        // address of chunk c (16 bytes = 8 fp16) of tile row r inside a stage's A region
        const uint32_t katom_off = (sub >> 1) * (128 * 128);
        auto chunk_addr = [&](uint8_t* stage, int row, int c) -> uint4* {
            return reinterpret_cast<uint4*>(stage + katom_off + (row >> 3) * 1024 + (row & 7) * 128 +
                                            ((c ^ (row & 7)) << 4));
        };
        auto convert = [&](const RawW<BITS>& r, uint8_t* stage) {
            if constexpr (BITS == 4) {
                const RawW<4>& q = r;
                const uint32_t off = 0x64086408u;  // 1024 + zero point 8
                const uint32_t s_lo = scale_h2(q.s.x * p.wmul), s_hi = scale_h2(q.s.y * p.wmul);
                const int row_lo = grp * 32 + gid + 16 * sel, row_hi = row_lo + 8;
                const uint32_t wa[2] = {q.a.x, q.a.y}, wb[2] = {q.b.x, q.b.y};
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int c = 4 * (sub & 1) + 2 * h + tp;
                    const uint2 l0 = bytes_to_h4(wa[h] & 0x0F0F0F0Fu, off, s_lo);
                    const uint2 l1 = bytes_to_h4(wb[h] & 0x0F0F0F0Fu, off, s_lo);
                    *chunk_addr(stage, row_lo, c) = make_uint4(l0.x, l0.y, l1.x, l1.y);
                    const uint2 h0 = bytes_to_h4((wa[h] >> 4) & 0x0F0F0F0Fu, off, s_hi);
                    const uint2 h1 = bytes_to_h4((wb[h] >> 4) & 0x0F0F0F0Fu, off, s_hi);
                    *chunk_addr(stage, row_hi, c) = make_uint4(h0.x, h0.y, h1.x, h1.y);
                }
            } else {
                const RawW<8>& q = r;
                const uint32_t off = 0x64806480u;  // 1024 + zero point 128
                const uint32_t wa[4] = {q.a.x, q.a.y, q.a.z, q.a.w}, wb[4] = {q.b.x, q.b.y, q.b.z, q.b.w};
                const float sc[4] = {q.s.x, q.s.y, q.s.z, q.s.w};
                const int c = 4 * (sub & 1) + 2 * sel + tp;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint32_t s2 = scale_h2(sc[i] * p.wmul);
                    const uint2 l0 = bytes_to_h4(wa[i], off, s2);
                    const uint2 l1 = bytes_to_h4(wb[i], off, s2);
                    *chunk_addr(stage, grp * 32 + gid + 8 * i, c) = make_uint4(l0.x, l0.y, l1.x, l1.y);
                }
            }
        };

        RawW<BITS> raw[kPrefetch];
#pragma unroll
        for (int j = 0; j < kPrefetch; ++j) load(raw[j], j);
        int s = 0;
        uint32_t ph = 0;
        bool ok = true;
        for (int ks0 = 0; ks0 < ksteps && ok; ks0 += kPrefetch) {
#pragma unroll
            for (int j = 0; j < kPrefetch; ++j) {
                const int ks = ks0 + j;
                if (ks < ksteps && ok) {
                    bool got = mbar_try(empty + 8 * s, ph ^ 1u) || mbar_wait(empty + 8 * s, ph ^ 1u, abort_flag);
                    ok = __all_sync(0xffffffffu, got);
                    if (ok) {
                        convert(raw[j], smem + s * STAGE);
                        fence_async_smem();  // generic-proxy stores -> visible to the tensor core
                        __syncwarp();
                        if (lane == 0) mbar_arrive(full_a + 8 * s);
                        load(raw[j], ks + kPrefetch);
                        if (++s == kNST) { s = 0; ph ^= 1u; }
                    }
                }
            }
        }

        // ---------------- epilogue: tensor memory -> y ----------------
        if (ok) {
            bool got = mbar_try(acc_full, 0) || mbar_wait(acc_full, 0, abort_flag);
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
    RSTQ_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<BITS, NTOK>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   kNST * (kAStage + NTOK * kKStep * 2) + 1024));
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

// y[M, out] = x[M, in] . dequant(W)^T on the tensor cores.  src: 0 = f32 x, 1 = bf16 x,
// 2 = int8 codes x with per-block scales xs.  x16 / rowscale are caller-provided scratch
// (M*in fp16, M floats).
int32_t launch_gemm(rstq_ctx* ctx, DeviceState& ds, const rstq_weight* w, const void* x, const float* xs,
                    int src, void* y, int out_dtype, int64_t M, void* x16, float* rowscale) {
    RSTQ_REQUIRE(M >= 1 && M < (1ll << 30), RSTQ_E_SHAPE, "M = %lld", (long long)M);
    RSTQ_REQUIRE(((uintptr_t)x16 & 15) == 0 && (w->in * 2) % 16 == 0, RSTQ_E_ALIGN,
                 "activation scratch must be 16-byte aligned");
    EncodeTiledFn enc = encode_tiled_fn();
    RSTQ_REQUIRE(enc, RSTQ_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    // pre-pass: activations -> fp16 with one exponent per token row
    cudaError_t le;
    if (src == 0)
        le = launch_pdl(act_to_f16_kernel<0>, dim3((unsigned)M), dim3(256), 0, ds, x, xs, (__half*)x16,
                        rowscale, w->in);
    else if (src == 1)
        le = launch_pdl(act_to_f16_kernel<1>, dim3((unsigned)M), dim3(256), 0, ds, x, xs, (__half*)x16,
                        rowscale, w->in);
    else
        le = launch_pdl(act_to_f16_kernel<2>, dim3((unsigned)M), dim3(256), 0, ds, x, xs, (__half*)x16,
                        rowscale, w->in);
    ctx->launches++;
    RSTQ_CUDA(le);

    const int ntok = M <= 32 ? 32 : (M <= 64 ? 64 : 128);
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
    p.ksteps = (int)((w->nb + 3) / 4);
    p.ttiles = (int)((M + ntok - 1) / ntok);
    p.wmul = ldexpf(1.0f, w->gemm_exp);
    p.wdiv = ldexpf(1.0f, -w->gemm_exp);
    p.out_dtype = out_dtype;
    const int64_t ftiles = (w->out + 127) / 128;
    RSTQ_REQUIRE(ftiles * p.ttiles < (1ll << 31), RSTQ_E_LIMIT, "grid too large");
    const dim3 grid((unsigned)(ftiles * p.ttiles));
    const size_t smem = kNST * (kAStage + (size_t)ntok * kKStep * 2) + 1024;
#define GL(B, N) le = launch_pdl(gemm_tc_kernel<B, N>, grid, dim3(kGemmThreads), smem, ds, p, tmap)
    if (w->bits == 4) {
        if (ntok == 32) GL(4, 32);
        else if (ntok == 64) GL(4, 64);
        else GL(4, 128);
    } else {
        if (ntok == 32) GL(8, 32);
        else if (ntok == 64) GL(8, 64);
        else GL(8, 128);
    }
#undef GL
    ctx->launches++;
    RSTQ_CUDA(le);
    RSTQ_CUDA(cudaGetLastError());
    return RSTQ_OK;
}

}  // namespace rstq
