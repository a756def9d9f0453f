// Backward-data of the frozen-weight linear, qlinear-q8-dx (src/raster/quant/train.clj:110-142):
//   dx[m, i] = sum over o of scales[o, i / 32] * codes[o, i] * dy[m, o]
// the dequant-transpose GEMM dX = dY . dequant(W), W = [out, in] signed 8-bit codes in the
// reference's row-major layout with one f32 scale per 32 columns.
//
// Two kernels: the tensor-core one below (m >= 16 and out % 8 == 0) and a tiled f32 kernel on the
// CUDA cores for everything else.  In the f32 kernel a CTA owns a
// 32-token x 128-column tile of dx and walks `out` in chunks of 32 rows: the chunk of W is
// dequantized once into shared memory (code * scale in f32, the product the reference forms
// first), the chunk of dy is stored transposed, and every thread keeps a 4 x 4 micro-tile in
// registers.  Products are f32, sums are f32 in o order per thread.
#include "internal.h"
#include "mma_helpers.cuh"

namespace rstq {

constexpr int kDxTok = 32, kDxCols = 128, kDxChunk = 32, kDxThreads = 256;

__global__ void __launch_bounds__(kDxThreads)
qlinear_q8_dx_kernel(const float* __restrict__ dy, const int8_t* __restrict__ codes,
                     const float* __restrict__ scales, float* __restrict__ dx, int64_t m, int64_t in, int64_t out) {
    __shared__ __align__(16) float s_w[kDxChunk][kDxCols];   // dequantized W chunk
    __shared__ __align__(16) float s_dy[kDxChunk][kDxTok];   // dy chunk, [o][token]
    const int tid = threadIdx.x;
    const int64_t col0 = (int64_t)blockIdx.x * kDxCols, tok0 = (int64_t)blockIdx.y * kDxTok;
    const int64_t nb = in >> 5;
    const int tc = (tid & 31) * 4, tt = (tid >> 5) * 4;       // this thread's 4 columns / 4 tokens
    float acc[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;
    // loader roles: W chunk = 32 rows x 128 codes: thread -> (row, 16 consecutive columns);
    // dy chunk = 32 tokens x 32 o: thread -> (token, 4 consecutive o)
    const int wr = tid >> 3, wc = (tid & 7) * 16;
    const int dt = tid >> 3, dq = (tid & 7) * 4;
    for (int64_t o0 = 0; o0 < out; o0 += kDxChunk) {
        {
            const int64_t o = o0 + wr, c = col0 + wc;
            float v[16];
            if (o < out && c < in) {   // in % 32 == 0 and wc % 16 == 0: the 16 columns share a block
                const int4 raw = *reinterpret_cast<const int4*>(codes + o * in + c);
                const float s = scales[o * nb + (c >> 5)];
                const int w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = s * (float)(int8_t)(w[j >> 2] >> (8 * (j & 3)));
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = 0.f;
            }
#pragma unroll
            for (int j = 0; j < 16; j += 4)
                *reinterpret_cast<float4*>(&s_w[wr][wc + j]) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        }
        {
            const int64_t t = tok0 + dt, o = o0 + dq;
#pragma unroll
            for (int j = 0; j < 4; ++j) s_dy[dq + j][dt] = (t < m && o + j < out) ? dy[t * out + o + j] : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int o = 0; o < kDxChunk; ++o) {
            const float4 w4 = *reinterpret_cast<const float4*>(&s_w[o][tc]);
            const float4 d4 = *reinterpret_cast<const float4*>(&s_dy[o][tt]);
            const float wv[4] = {w4.x, w4.y, w4.z, w4.w}, dv[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(wv[b], dv[a], acc[a][b]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int a = 0; a < 4; ++a) {
        const int64_t t = tok0 + tt + a, c = col0 + tc;
        if (t < m && c < in)   // in % 4 == 0: the four columns are in range together
            *reinterpret_cast<float4*>(dx + t * in + c) = make_float4(acc[a][0], acc[a][1], acc[a][2], acc[a][3]);
    }
}

// ---- the same product on the tensor cores (m >= 16, out % 8 == 0) --------------------------------
// mma roles: M = 16 tokens, N = 8 columns i, K = 16 rows o of W.  For the 32 columns of one scale
// block b,  dx[m, i] = sum_o (dy[m, o] * s[o, b]) * c[o, i]:  the codes c are exact in bf16, the f32
// factor dy * s is split into three bf16 terms (each step of the expansion exact in f32), so three
// bf16 m16n8k16 MMAs per tile give the f32 product to about 2^-24 -- the arithmetic of the decode
// kernel's float-activation mode.  A CTA owns 64 tokens x 128 columns and walks `out` in chunks of 32
// rows: dy chunk (f32), the four scale columns and the codes come in by asynchronous copies, two
// chunks in flight; the codes are then transposed to bf16 [column][o] so a B fragment is one 32-bit load; warp w holds tokens 16 * (w & 3) and the
// two column blocks 2 * (w >> 2), 2 * (w >> 2) + 1 (eight accumulator tiles).
constexpr int kMmaTok = 64, kMmaCols = 128, kMmaChunk = 32;
constexpr int kDyStride = 40;   // floats per token row of the dy chunk: conflict-free 8-byte fragment loads
constexpr int kBStride = 20;    // 32-bit words per column row of the bf16 codes: conflict-free fragment loads

__device__ __forceinline__ void split3_bf16x2(float hi, float lo, uint32_t (&t)[3]) {
    // terms of hi (upper half) and lo (lower half) side by side; bf16 -> f32 is a 16-bit shift
#pragma unroll
    for (int k = 0; k < 3; ++k) {
        t[k] = pack_bf16x2(hi, lo);
        hi -= __uint_as_float(t[k] & 0xFFFF0000u);
        lo -= __uint_as_float(t[k] << 16);
    }
}

// 16-byte / 4-byte asynchronous copies global -> shared; `ok` false copies nothing and fills zeros
// (the source address is then only required to be a valid one).
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool ok) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(ok ? 16 : 0) : "memory");
}
__device__ __forceinline__ void cp_async4(void* dst, const void* src, bool ok) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(d), "l"(src), "r"(ok ? 4 : 0) : "memory");
}

struct DxStage {   // one chunk of 32 rows o as it comes from memory
    float dy[kMmaTok][kDyStride];
    int8_t codes[kMmaChunk][kMmaCols];
    float s[kMmaChunk][4];
};

__global__ void __launch_bounds__(256)
qlinear_q8_dx_mma_kernel(const float* __restrict__ dy, const int8_t* __restrict__ codes,
                         const float* __restrict__ scales, float* __restrict__ dx, int64_t m, int64_t in, int64_t out) {
    // two stages in flight: while the MMAs of chunk c run, the copies of chunk c + 1 land
    __shared__ __align__(16) DxStage stage[2];
    __shared__ __align__(16) uint32_t s_b[kMmaCols][kBStride];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int64_t col0 = (int64_t)blockIdx.x * kMmaCols, tok0 = (int64_t)blockIdx.y * kMmaTok;
    const int64_t nb = in >> 5;
    const int wm = warp & 3, wb = (warp >> 2) * 2;
    float acc[8][4];
#pragma unroll
    for (int a = 0; a < 8; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;
    const int f_tok = tid >> 2, f_o = (tid & 3) * 8;   // dy copies: a token, eight consecutive o (two 16-byte copies)
    const int k_o = tid >> 3, k_i = (tid & 7) * 16;    // code copies: a row o, 16 consecutive columns
    const int c_i = tid & 127, c_p = tid >> 7;         // conversion: a column, o pairs c_p, c_p + 2, ...

    auto issue = [&](int64_t o0, DxStage& st) {
        {
            const int64_t tk = tok0 + f_tok, o = o0 + f_o;
            const bool ok = tk < m && o < out;           // out % 8 == 0: the eight are in range together
            const float* src = ok ? dy + tk * out + o : dy;
            cp_async16(&st.dy[f_tok][f_o], src, ok);
            cp_async16(&st.dy[f_tok][f_o + 4], src + (ok ? 4 : 0), ok);
        }
        {
            const int64_t o = o0 + k_o, i = col0 + k_i;
            const bool ok = o < out && i < in;           // in % 32 == 0: the sixteen are in range together
            cp_async16(&st.codes[k_o][k_i], ok ? codes + o * in + i : codes, ok);
        }
        if (tid < 128) {
            const int64_t o = o0 + (tid >> 2), b = (col0 >> 5) + (tid & 3);
            const bool ok = o < out && b < nb;
            cp_async4(&st.s[tid >> 2][tid & 3], ok ? scales + o * nb + b : scales, ok);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    issue(0, stage[0]);
    int cur = 0;
    for (int64_t o0 = 0; o0 < out; o0 += kMmaChunk, cur ^= 1) {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();   // chunk `cur` has landed for everyone; the MMAs of the chunk before are done
        if (o0 + kMmaChunk < out) issue(o0 + kMmaChunk, stage[cur ^ 1]);
        const DxStage& st = stage[cur];
        // codes -> bf16, transposed to [column][o] so that a B fragment is one 32-bit load
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const int op = c_p + 2 * q;                  // rows 2 op, 2 op + 1 of the chunk
            s_b[c_i][op] = pack_bf16x2((float)st.codes[2 * op + 1][c_i], (float)st.codes[2 * op][c_i]);
        }
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
            const int kb = ks * 16;
            const float2 d00 = *reinterpret_cast<const float2*>(&st.dy[wm * 16 + g][kb + 2 * t]);
            const float2 d10 = *reinterpret_cast<const float2*>(&st.dy[wm * 16 + g + 8][kb + 2 * t]);
            const float2 d01 = *reinterpret_cast<const float2*>(&st.dy[wm * 16 + g][kb + 2 * t + 8]);
            const float2 d11 = *reinterpret_cast<const float2*>(&st.dy[wm * 16 + g + 8][kb + 2 * t + 8]);
#pragma unroll
            for (int blk = 0; blk < 2; ++blk) {
                const int bc = wb + blk;
                const float s0 = st.s[kb + 2 * t][bc], s1 = st.s[kb + 2 * t + 1][bc];
                const float s8 = st.s[kb + 2 * t + 8][bc], s9 = st.s[kb + 2 * t + 9][bc];
                uint32_t a0[3], a1[3], a2[3], a3[3];
                split3_bf16x2(d00.y * s1, d00.x * s0, a0);   // row g,     k 2t, 2t+1
                split3_bf16x2(d10.y * s1, d10.x * s0, a1);   // row g + 8, k 2t, 2t+1
                split3_bf16x2(d01.y * s9, d01.x * s8, a2);   // row g,     k 2t+8, 2t+9
                split3_bf16x2(d11.y * s9, d11.x * s8, a3);   // row g + 8, k 2t+8, 2t+9
                uint32_t b0[4], b1[4];
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) {
                    const int ci = bc * 32 + nt * 8 + g;
                    b0[nt] = s_b[ci][ks * 8 + t];
                    b1[nt] = s_b[ci][ks * 8 + t + 4];
                }
                // smallest term first; the four column tiles of a term are independent MMAs
#pragma unroll
                for (int k = 2; k >= 0; --k) {
                    const uint32_t af[4] = {a0[k], a1[k], a2[k], a3[k]};
#pragma unroll
                    for (int nt = 0; nt < 4; ++nt) hmma_bf16(acc[blk * 4 + nt], af, b0[nt], b1[nt]);
                }
            }
        }
    }
#pragma unroll
    for (int blk = 0; blk < 2; ++blk)
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            const int64_t c = col0 + (wb + blk) * 32 + nt * 8 + 2 * t;
            const int64_t r0 = tok0 + wm * 16 + g;
            if (c < in) {   // in % 2 == 0: the pair is in range together
                if (r0 < m) *reinterpret_cast<float2*>(dx + r0 * in + c) = make_float2(acc[blk * 4 + nt][0], acc[blk * 4 + nt][1]);
                if (r0 + 8 < m)
                    *reinterpret_cast<float2*>(dx + (r0 + 8) * in + c) = make_float2(acc[blk * 4 + nt][2], acc[blk * 4 + nt][3]);
            }
        }
}

int32_t launch_qlinear_q8_dx(rstq_ctx* ctx, DeviceState& ds, const float* dy, const int8_t* codes,
                             const float* scales, float* dx, int64_t m, int64_t in, int64_t out) {
    if (m >= 16 && out % 8 == 0) {
        const dim3 gm((unsigned)((in + kMmaCols - 1) / kMmaCols), (unsigned)((m + kMmaTok - 1) / kMmaTok));
        RSTQ_REQUIRE(gm.y < 65536, RSTQ_E_LIMIT, "m = %lld too large for one launch", (long long)m);
        qlinear_q8_dx_mma_kernel<<<gm, 256, 0, ds.stream>>>(dy, codes, scales, dx, m, in, out);
        ctx->launches++;
        RSTQ_CUDA(cudaGetLastError());
        return RSTQ_OK;
    }
    const dim3 grid((unsigned)((in + kDxCols - 1) / kDxCols), (unsigned)((m + kDxTok - 1) / kDxTok));
    RSTQ_REQUIRE(grid.y < 65536, RSTQ_E_LIMIT, "m = %lld too large for one launch", (long long)m);
    qlinear_q8_dx_kernel<<<grid, kDxThreads, 0, ds.stream>>>(dy, codes, scales, dx, m, in, out);
    ctx->launches++;
    RSTQ_CUDA(cudaGetLastError());
    return RSTQ_OK;
}

}  // namespace rstq
