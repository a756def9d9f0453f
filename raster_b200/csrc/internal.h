// Internal declarations shared by the translation units of librstq.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "../../include/rstq.h"

namespace rstq {

// ---- error plumbing --------------------------------------------------------
void set_error(const char* fmt, ...);
int32_t cuda_fail(cudaError_t e, const char* what, const char* file, int line);

#define RSTQ_CUDA(call)                                                      \
    do {                                                                     \
        cudaError_t e__ = (call);                                            \
        if (e__ != cudaSuccess) return ::rstq::cuda_fail(e__, #call, __FILE__, __LINE__); \
    } while (0)

#define RSTQ_REQUIRE(cond, code, ...)     \
    do {                                  \
        if (!(cond)) {                    \
            ::rstq::set_error(__VA_ARGS__); \
            return (code);                \
        }                                 \
    } while (0)

// ---- device weight layout ("mma32") -----------------------------------------
// Rows are padded to a multiple of 32.  A unit (g, b) holds block b (32 K
// elements) of the 32 rows of group g.  Units are stored b-fastest, so the
// K-slice of one group is one contiguous byte range.
//
//   4-bit unit, 640 B : [32 slots x 16 B codes][32 x f32 scales]
//   8-bit unit, 1152 B: [plane 0: 32 slots x 16 B][plane 1: 32 x 16 B][32 x f32 scales]
//
// Slot `lane` = gid*4 + tig (gid = lane >> 2, tig = lane & 3) holds four 32-bit
// words.
//   4-bit: word 2q + h (q = 0,1; h = 0,1), byte j: low nibble = code of row
//          32g + gid + 16q, high nibble = code of row 32g + gid + 16q + 8, both at
//          element 16h + 4tig + j of the block.  Masking a word with 0x0F0F0F0F /
//          0xF0F0F0F0 therefore yields two int8 A-fragment registers of
//          mma.sync m16n8k32 with no shift: the high-nibble rows come out
//          multiplied by 16, which the kernels undo in the per-block scale.
//   8-bit: plane p (p = 0,1), word i (i = 0..3) = elements 4tig + 16p .. +3 of
//          row 32g + gid + 8i, unsigned with zero point 128.
// Scale index gid*4 + i is the (true) scale of row 32g + gid + 8i.
// One 16-byte load per lane thus feeds two 16-row tensor-core tiles with no
// data movement between lanes.
constexpr int kUnitBytesQ4 = 640;
// prefill GEMM, two CTAs per tile: at most this many tiles (their flags are the last words of
// DeviceState::counters, their partial tiles of up to 128 x 256 floats live in the GEMM scratch)
constexpr int kPairTiles = 128;
constexpr int64_t kPairScratchBytes = (int64_t)kPairTiles * 128 * 256 * 4;
constexpr int kUnitBytesQ6K = 1280;  // 1024 bytes of 8-bit codes as in the 8-bit unit, then 64 scales (one per row and 16 elements)
constexpr int kUnitBytesQ4K = 768;  // a 4-bit unit with the 32 Q4_K minima (db * bq, added as they are) behind the 32 scales
constexpr int kUnitBytesQ8 = 1152;
constexpr int kUnitCodesQ4 = 512;
constexpr int kUnitCodesQ8 = 1024;
// `bits` here is the unit kind: 4, 8, or 5 = the Q4_K unit
inline int unit_bytes(int bits) {
    return bits == 4 ? kUnitBytesQ4 : (bits == 5 ? kUnitBytesQ4K : (bits == 6 ? kUnitBytesQ6K : kUnitBytesQ8));
}

struct DeviceState {
    int ordinal = -1;
    int sm_count = 0;
    int64_t l2_bytes = 0;
    int64_t total_mem = 0;
    int cc = 0;
    cudaStream_t stream = nullptr;      // where everything launches: own_stream or one the caller lent
    cudaStream_t own_stream = nullptr;
    bool capturing = false;
    bool pdl = true;               // launch the hot kernels with programmatic stream serialization
    int gemv_plan = 0;             // decode work split: 0 = per shape, 1 = equal unit ranges, 2 = whole groups
    int64_t gemv_prefetch_kb = -1; // decode kernels: KB of a CTA's weight range requested into L2 ahead of its ring (-1: by size)
    int gemv_probe = 0;            // timing probes of the decode kernel (RSTQ_TUNE_PROBE); results are invalid while set
    bool prefetch_next = true;     // decode launches request the weight that followed this one last time into L2
    rstq_weight* last_decode_w = nullptr;   // the weight of the most recent decode launch on this device
    int tp_tail_ctas = 32;         // fused exchange: fewest thread blocks of the decode kernel that stay for the exchange's tail (0 = all)
    int act_ring = 0;              // MODE_A8, M > 1: 0 = the plan with most weight bytes in flight, 1 = activations resident + full chunks, 2 / 3 = activations ride the ring (full / half chunks), 4 = resident + half chunks
    bool act_image = true;         // MODE_A8, 2 <= M <= 16: the quantizer also writes the decode kernel's staged form, taken by bulk copy
    bool x_on_host = false;        // the current host-array call lets its first kernel read x from pinned host memory
    bool fuse_quant = true;        // M = 1 operator: quantize the activations inside the decode kernel
    // scratch owned by the context
    void* act_scratch = nullptr;   // quantized / converted activations
    int64_t act_scratch_bytes = 0;
    float* partials = nullptr;     // decode kernel: partial sums handed between CTAs that share a 32-row group
    int64_t partials_bytes = 0;
    int* counters = nullptr;       // decode kernel: one hand-over flag per CTA (zero between calls)
    int64_t counters_len = 0;
    void* gemm_scratch = nullptr;  // fp16 activations + row exponents of the GEMM path
    int64_t gemm_scratch_bytes = 0;
    void* kq_scratch = nullptr;    // Q6_K: the twin-row results before they are added in pairs
    int64_t kq_scratch_bytes = 0;
    void* f_image = nullptr;       // mode F: the staged activations of a decode launch that ride the weight ring
    int64_t f_image_bytes = 0;
    void* attn_scratch = nullptr;  // decode attention: arrival counters + per-slice softmax states
    int64_t attn_scratch_bytes = 0;
    void* pinned = nullptr;        // host staging for the host-array entry points
    int64_t pinned_bytes = 0;
    void* io_dev = nullptr;        // device staging for the host-array entry points
    int64_t io_dev_bytes = 0;
    int* status = nullptr;         // device status word: nonzero after a bounded wait ran out
    // Instantiated graphs hold the scratch addresses of the launches they recorded.  While any is
    // alive, scratch that has to grow is parked here instead of freed, so a replay never touches
    // memory that went back to the allocator; the blocks are released when the last graph is gone.
    int live_graphs = 0;
    std::vector<void*> retired;
    unsigned long long* dbg = nullptr;      // phase timestamps of the last streaming launch, when enabled
    unsigned long long* dbg_store = nullptr;
    mutable uint64_t dbg_launch = 0;        // decode launches recorded so far (picks the timeline slot)
};

}  // namespace rstq

struct rstq_ctx {
    uint32_t magic;
    std::vector<rstq::DeviceState> devs;
    int64_t tune_gemm_min_m = 17;
    bool tune_q4k_units = true;     // Q4_K weights bound from now on keep their minima inside the units
    bool tune_q6k_units = true;     // Q6_K weights bound from now on are 1280-byte units (a scale per 16 elements), not twin rows
    int64_t tune_gemm_wide = 0;        // 256-token tiles of the prefill GEMM above 128 tokens: 0 = where they need fewer cycles, 1 = never, 2 = always, 3 = as 0 but no split along K
    int64_t tune_gemm_kernel = 0;   // 0 = weights in tensor memory, 1 = weights through shared memory
    int64_t launches = 0;
    struct CacheKey {
        const void* codes;
        const void* scales;
        int64_t in, out;
        int fmt, layout;
        bool operator==(const CacheKey& o) const {
            return codes == o.codes && scales == o.scales && in == o.in && out == o.out &&
                   fmt == o.fmt && layout == o.layout;
        }
    };
    struct CacheHash {
        size_t operator()(const CacheKey& k) const {
            size_t h = (size_t)k.codes * 1315423911u ^ (size_t)k.scales;
            return h ^ (size_t)(k.in * 31 + k.out) ^ (size_t)(k.fmt * 7 + k.layout);
        }
    };
    std::unordered_map<CacheKey, rstq_weight*, CacheHash> wcache;
    std::unordered_set<const rstq_weight*> live_weights;   // handles that may be named as a prefetch target
};

struct rstq_buf {
    uint32_t magic;
    rstq_ctx* ctx;
    int dev;
    void* ptr;
    int64_t bytes;
    bool owned;  // false: wraps memory the caller allocated (rstq_buf_wrap)
};

struct rstq_weight {
    uint32_t magic;
    rstq_ctx* ctx;
    int dev;
    int bits;          // 4 or 8
    int zp;            // 8 or 128 (signed codes are stored offset by 128)
    int64_t out, in;   // logical shape of this (possibly sharded) matrix
    int64_t outp;      // rows padded to a multiple of 32
    int64_t nb;        // in / 32
    uint8_t* data;     // mma32 units, (outp/32) * nb of them
    int64_t data_bytes;
    int gemm_exp;      // power of two applied to the block scales in the fp16 GEMM path
    uint64_t host_fp = 0;          // fingerprint of the host arrays (host-array operators' cache)
    int8_t* raw_codes = nullptr;   // row-major signed codes / scales as the reference holds them:
    float* raw_scales = nullptr;   // made on first use by the backward-data operator
    // The weight a decode launch of THIS one was followed by last time on the same device.  A decode
    // loop walks its matrices in the same order for every token, so the next launch of this weight
    // asks for that one's first bytes to be brought into L2 while its own consumers still work
    // (a hint: a wrong guess costs bandwidth, not correctness).  Checked against live_weights.
    rstq_weight* next_hint = nullptr;
    float* mins = nullptr;         // Q4_K only: per-sub-block minima db*bq, [out, nb]; zp is 0 then
    bool kq = false;               // Q4_K only: `data` holds 768-byte units with the minima inside (default)
    bool k6 = false;               // Q6_K only: `data` holds 1280-byte units with a scale per 16 elements (default);
                                   // `out` is then the logical row count (= pair_out), not twice it
    int64_t pair_out = 0;          // Q6_K only: logical rows; `out` = 2 * pair_out twin rows, y[o] = t[2o] + t[2o+1]
};

struct rstq_graph {
    uint32_t magic;
    rstq_ctx* ctx;
    int dev;
    cudaGraph_t graph;
    cudaGraphExec_t exec;
    int64_t kernels;  // kernel nodes per replay
};

struct rstq_event {
    uint32_t magic;
    rstq_ctx* ctx;
    int dev;
    cudaEvent_t ev;
};

namespace rstq {

constexpr uint32_t kCtxMagic = 0x52535143;   // 'RSQC'
constexpr uint32_t kBufMagic = 0x52535142;
constexpr uint32_t kWgtMagic = 0x52535157;
constexpr uint32_t kGrfMagic = 0x52535147;
constexpr uint32_t kEvtMagic = 0x52535145;

// ---- kernel launchers (each returns a status; all launch on ds.stream) -------
// layout.cu
int32_t launch_repack(rstq_ctx* ctx, DeviceState& ds, const uint8_t* src_codes,
                      const float* src_scales, uint8_t* dst, int fmt, int layout, int64_t out,
                      int64_t in, int64_t src_in, int64_t k_block0);
// 640-byte 4-bit units + row-major minima [out, nb] -> 768-byte Q4_K units (the minimum db * bq of
// row gid + 8i of the group at float gid*4 + i behind the scales, the order the scales have)
int32_t launch_q4k_units(rstq_ctx* ctx, DeviceState& ds, const uint8_t* src, const float* mins, uint8_t* dst,
                         int64_t out, int64_t nb);
// 1152-byte 8-bit units + row-major scales per 16 elements [out, in/16] -> 1280-byte Q6_K units
int32_t launch_q6k_units(rstq_ctx* ctx, DeviceState& ds, const uint8_t* src, const float* scales16, uint8_t* dst,
                         int64_t out, int64_t nb);
// kquant.cu (Q4_K: q8_K activation quantizer, scale expansion, the min-term GEMV)
int32_t launch_quant_act_q8k(rstq_ctx* ctx, DeviceState& ds, const float* x, int8_t* xq, float* xs, float* xs32,
                             int32_t* bsums, int64_t rows, int64_t in, int sub);
int32_t launch_expand_scales(rstq_ctx* ctx, DeviceState& ds, const float* xs, float* xs32, int64_t n32);
int32_t launch_q6k_prep(rstq_ctx* ctx, DeviceState& ds, const float* xs, const int32_t* bsums16, float* xs32,
                        int32_t* bsum32, int64_t n32);
int32_t launch_pair_sum(rstq_ctx* ctx, DeviceState& ds, const float* t, float* y, int64_t M, int64_t out);
int32_t launch_q4k_min(rstq_ctx* ctx, DeviceState& ds, const float* mins, const float* xs32, const int32_t* bsums,
                       float* y, int64_t M, int64_t nb, int64_t out);
// actquant.cu
constexpr int kGemvMaxM = 16;             // widest token tile of the decode kernels
// bytes of the decode kernel's image of kGemvMaxM tokens' quantized activations (fragments, then the records)
constexpr int kActRecBytes = 16;   // per (block, token), plain units
__host__ __device__ constexpr int64_t act_image_stride(int64_t nb) {
    return ((nb * kGemvMaxM * 32 + 127) & ~127ll) + ((nb * kGemvMaxM * kActRecBytes + 255) & ~255ll);
}
constexpr int kActMagicInt = 0x4B400000;   // bits of 12582912.0f = 2^23 + 2^22: int -> float through the tile's accumulator input
#ifdef __CUDACC__
// The record of a (block, token) for the decode kernel above one token, plain units: the tokens of a block go
// in pairs (a, b) of 32 bytes {xs_a, xs_b, xs_a*h, xs_b*h | ca_a, ca_b, cb_a, cb_b}: the scale as the rows in
// the low nibbles want it and as those in the high nibbles do (their tile values are 16 times the codes:
// h = 1/16 for 4-bit units, else 1), and the accumulator inputs of the two kinds of rows (the int -> float
// bias less the zero-point term zs = zp * code sum, times 16 for the high-nibble rows).  A lane holds two
// neighbouring tokens' results, so it reads one pair: two 16-byte loads, nothing to compute.  (Measured:
// records of half the size, the high-nibble variants derived in the loop, were 2 - 8 % slower: the loop is
// bound by instruction issue before shared-memory bandwidth.)
__device__ __forceinline__ void put_act_record(uint8_t* recs, int64_t b, int Mz, int c, float xs, int zs, bool four_bit) {
    uint32_t* r = reinterpret_cast<uint32_t*>(recs + (b * (Mz >> 1) + (c >> 1)) * 32) + (c & 1);
    r[0] = __float_as_uint(xs);
    r[2] = __float_as_uint(four_bit ? xs * 0.0625f : xs);
    r[4] = (uint32_t)(kActMagicInt - zs);
    r[6] = (uint32_t)(kActMagicInt - (four_bit ? zs * 16 : zs));
}
#endif
int32_t launch_act_image(rstq_ctx* ctx, DeviceState& ds, const int8_t* xq, const float* xs, const int32_t* xsum,
                         int64_t M, int64_t in, uint8_t* img, int zp, int bits, int uk);
int32_t launch_quant_act_i8(rstq_ctx* ctx, DeviceState& ds, const void* x, int8_t* xq, float* xs,
                            int32_t* xsum, int64_t M, int64_t in, int act_dtype = RSTQ_F32, uint8_t* img = nullptr, int zp = 0,
                            int bits = 8);
// Exchange fused into the tail of the decode kernel (layout of a region: see tp.cu).  The
// kernel writes its results into slot `rank` of every rank's stage instead of y, signals, waits
// (time-bounded) for the other ranks and lays the slots side by side (sum = 0) or adds them in
// rank order (sum = 1) into y.
constexpr int kTpMaxRanks = 8;
constexpr int64_t kTpHeader = 512;
struct TpFuse {
    uint8_t* region[kTpMaxRanks];
    int rank, nranks, sum;
    int64_t ll_off;      // byte offset of the value/epoch pair stage inside a region
    int64_t slot_bytes;  // bytes of one slot of that stage (8 per result)
    float* y;  // [M, nranks * out] (gather) or [M, out] (sum), f32
};
constexpr int32_t kNotFused = 1;  // a launcher declined the fused exchange before launching anything

// gemv.cu
struct NextWeight {      // what a decode launch may prefetch for the launch expected after it
    const uint8_t* data = nullptr;
    int64_t groups = 0, nb = 0;
    int bits = 0;
};
struct GemvA8Args {
    const uint8_t* w;
    const int8_t* xq;
    const float* xs;
    const int32_t* xsum;  // may be null (treated as zero-point-free: signed x signed)
    float* y;
    int64_t M, in, out;   // y is [M, out] f32
    int bits, zp;
    const TpFuse* tp = nullptr;
    const void* x = nullptr;     // M == 1 only: raw activations (f32 or bf16), quantized by the kernel
    int act_dtype = RSTQ_F32;    // itself while staging; xq / xs / xsum are then not read
    NextWeight next;
    const uint8_t* img = nullptr;  // M > 1: the quantizer's image of the staged activations (see StreamParams::img)
    uint8_t* img_scratch = nullptr;  // pre-quantized activations, 2 <= M <= 16: room for that image, built by a kernel of its own when the ring of activations pays
    int uk = 0;                    // unit kind of w: 0 = plain, 1 = Q4_K units (768 B, minima inside; xs / xsum are the
                                   // q8_K scales per block and sums per 32), 2 = Q6_K units (1280 B, a scale per 16
                                   // elements; xsum holds the sums per 16, two per block)
};
struct GemvFArgs {
    const uint8_t* w;
    const void* x;        // f32 or bf16 [M, in]
    void* y;              // f32 or bf16 [M, out]
    int64_t M, in, out;
    int bits, zp;
    int act_dtype, out_dtype;
    const TpFuse* tp = nullptr;
    NextWeight next;
    uint8_t* img_scratch = nullptr;   // gemv_f_image_bytes(in) of room for the staged activations of a launch whose
                                      // tokens do not fit in shared memory for all of K (they then ride the weight ring)
};
// gemv_stream.cu.  Any M >= 1: the launchers cut M into pieces the kernel takes.
int32_t launch_gemv_a8(rstq_ctx* ctx, DeviceState& ds, const GemvA8Args& a);
int32_t launch_gemv_f(rstq_ctx* ctx, DeviceState& ds, const GemvFArgs& a);
int gemv_f_pieces(const DeviceState& ds, int bits, int64_t out, int64_t in, int64_t M, int act_dtype);
int64_t gemv_f_image_bytes(int64_t in);
int32_t decode_plan(int mode, int bits, int64_t out, int64_t in, int64_t M, int act_dtype, int sm_count, int32_t* res);
int32_t gemv_configure(DeviceState& ds);  // shared-memory attributes, once per device
// gemm_tc.cu
// gemm_tc.cu: token-tile width (32 / 64 / 128 / 256) and whether two CTAs share a tile, for a device of sm_count SMs
void gemm_plan(int64_t out, int64_t in, int64_t M, int sm_count, bool tmem_kernel, int wide, int* ntok_out,
               bool* split_out);
int32_t launch_gemm(rstq_ctx* ctx, DeviceState& ds, const rstq_weight* w, const void* x, const float* xs,
                    int src, void* y, int out_dtype, int64_t M, void* x16, float* rowscale,
                    float* acc32 = nullptr);
int32_t gemm_configure(DeviceState& ds);
// dx.cu
int32_t launch_qlinear_q8_dx(rstq_ctx* ctx, DeviceState& ds, const float* dy, const int8_t* codes,
                             const float* scales, float* dx, int64_t m, int64_t in, int64_t out);
// capi.cu
int32_t use_dev(rstq_ctx* ctx, int dev);
int32_t matmul_device(rstq_ctx* ctx, rstq_weight* w, const void* x, void* y, int64_t M, int act_dtype,
                      int out_dtype, int mode, const TpFuse* tp = nullptr);
// capi.cu: grow-only device scratch (refuses to grow during graph capture; the outgrown block is
// freed at once, or parked until the last live graph of the device is destroyed)
int32_t dev_reserve(DeviceState& ds, void** p, int64_t* have, int64_t need);
int32_t dev_release_scratch(DeviceState& ds, void* p);
constexpr int64_t kFusedQuantMaxIn = 12288; // longest row the decode kernel quantizes itself (3 passes of 512 threads x 8)

}  // namespace rstq
