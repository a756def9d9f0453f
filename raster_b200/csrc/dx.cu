// Backward-data of the frozen-weight linear, qlinear-q8-dx (src/raster/quant/train.clj:110-142):
//   dx[m, i] = sum over o of scales[o, i / 32] * codes[o, i] * dy[m, o]
// the dequant-transpose GEMM dX = dY . dequant(W), W = [out, in] signed 8-bit codes in the
// reference's row-major layout with one f32 scale per 32 columns.
//
// First correct path: a tiled f32 kernel on the CUDA cores (no tensor cores yet).  A CTA owns a
// 32-token x 128-column tile of dx and walks `out` in chunks of 32 rows: the chunk of W is
// dequantized once into shared memory (code * scale in f32, the product the reference forms
// first), the chunk of dy is stored transposed, and every thread keeps a 4 x 4 micro-tile in
// registers.  Products are f32, sums are f32 in o order per thread.
#include "internal.h"

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

int32_t launch_qlinear_q8_dx(rstq_ctx* ctx, DeviceState& ds, const float* dy, const int8_t* codes,
                             const float* scales, float* dx, int64_t m, int64_t in, int64_t out) {
    const dim3 grid((unsigned)((in + kDxCols - 1) / kDxCols), (unsigned)((m + kDxTok - 1) / kDxTok));
    RSTQ_REQUIRE(grid.y < 65536, RSTQ_E_LIMIT, "m = %lld too large for one launch", (long long)m);
    qlinear_q8_dx_kernel<<<grid, kDxThreads, 0, ds.stream>>>(dy, codes, scales, dx, m, in, out);
    ctx->launches++;
    RSTQ_CUDA(cudaGetLastError());
    return RSTQ_OK;
}

}  // namespace rstq
