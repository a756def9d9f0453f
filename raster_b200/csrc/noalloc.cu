// An entry point of the decode GEMV that allocates nothing.
//
// Who needs it: hosts that are not allowed to allocate device memory at the
// moment they call -- a runtime that hands out all device memory from its own
// arena at session start and forbids later growth, a caller in the middle of a
// stream capture (allocation is illegal there), or a real-time decode loop that
// must never reach the driver's allocator.  The regular entry points draw their
// split-group scratch (the partial sums thread blocks hand to one another and
// one hand-over flag per block) from buffers the context allocated; this one
// keeps the same scratch in fixed
// arrays that live in the library's device image, so every GPU that loads the
// library carries them (about 1.3 MB) until the process exits.
//
// Limits that follow from the fixed size: out <= 2 097 152 rows, at most 256
// thread blocks (more than any sm_100 part has SMs), M <= 16 per launch (larger
// M is cut into launches of <= 16, as everywhere else).
//
// The arrays are shared by every call on the device.  They keep the last call's
// contents; the only part that must start at zero -- the hand-over flags -- is
// cleared once at set-up and put back to zero by each launch before it ends.
// Two calls that overlap on the GPU (different streams, no dependency) would
// race on the arrays: serialise them.
//
// A time-bounded wait that runs out inside such a launch is reported like
// everywhere else: the kernel sets the context's own status word (allocated
// when the context was made, so nothing is allocated here) and the next
// rstq_sync returns RSTQ_E_WAIT.
#include "internal.h"

namespace rstq {

constexpr int kNaMaxCtas = 256;
constexpr int kNaMaxGroups = 65536;
constexpr int kNaMaxM = 16;

// Scratch of the allocation-free entry point (device image, not the heap).
static __device__ __align__(256) float g_na_partials[kNaMaxCtas * 2 * kNaMaxM * 32];
static __device__ __align__(256) int g_na_counters[kNaMaxGroups];

struct NaDevice {
    bool ready = false;
    float* partials = nullptr;
    int* counters = nullptr;
};
static NaDevice g_na_dev[64];

// Once per device, with that device current: turn the host-side stand-ins of
// the arrays into device addresses (a kernel must never be handed the symbol
// itself) and clear the flags.
static int32_t na_setup(int ordinal, cudaStream_t stream) {
    NaDevice& d = g_na_dev[ordinal];
    if (d.ready) return RSTQ_OK;
    RSTQ_CUDA(cudaGetSymbolAddress((void**)&d.partials, g_na_partials));
    RSTQ_CUDA(cudaGetSymbolAddress((void**)&d.counters, g_na_counters));
    RSTQ_CUDA(cudaMemsetAsync(d.counters, 0, sizeof(int) * kNaMaxGroups, stream));
    d.ready = true;
    return RSTQ_OK;
}

}  // namespace rstq

using namespace rstq;

extern "C" int32_t rstq_qmatmul_prequant_noalloc(rstq_weight* w, const void* xq, const void* xs,
                                                 const void* xsum, void* y, void* stream,
                                                 int64_t M) {
    RSTQ_REQUIRE(w && w->magic == kWgtMagic && w->ctx && w->ctx->magic == kCtxMagic, RSTQ_E_INVALID,
                 "invalid weight handle");
    RSTQ_REQUIRE(xq && xs && xsum && y, RSTQ_E_INVALID, "null argument");
    RSTQ_REQUIRE(!w->mins && !w->pair_out, RSTQ_E_INVALID, "K-quant weights go through rstq_qmatmul / rstq_qmatmul_prequant");
    RSTQ_REQUIRE(M >= 1, RSTQ_E_SHAPE, "M = %lld", (long long)M);
    RSTQ_REQUIRE((((uintptr_t)xq | (uintptr_t)xs | (uintptr_t)xsum | (uintptr_t)y) & 15) == 0,
                 RSTQ_E_ALIGN, "device pointers must be 16-byte aligned");
    const int64_t groups = (w->out + 31) / 32;
    RSTQ_REQUIRE(groups <= kNaMaxGroups, RSTQ_E_LIMIT,
                 "out = %lld rows exceeds the fixed scratch of this entry point (%d rows)",
                 (long long)w->out, kNaMaxGroups * 32);
    rstq_ctx* ctx = w->ctx;
    const DeviceState& real = ctx->devs[w->dev];
    RSTQ_REQUIRE(real.ordinal >= 0 && real.ordinal < 64 && real.sm_count <= kNaMaxCtas, RSTQ_E_LIMIT,
                 "device outside the fixed limits of this entry point");
    RSTQ_CUDA(cudaSetDevice(real.ordinal));
    const cudaStream_t st = stream ? (cudaStream_t)stream : real.stream;
    int32_t rc = na_setup(real.ordinal, st);
    if (rc != RSTQ_OK) return rc;
    // Same launcher, same kernel; only the scratch and the stream differ.
    DeviceState ds = real;
    const NaDevice& d = g_na_dev[real.ordinal];
    ds.partials = d.partials;
    ds.partials_bytes = (int64_t)sizeof(float) * kNaMaxCtas * 2 * kNaMaxM * 32;
    ds.counters = d.counters;
    ds.counters_len = kNaMaxGroups;
    ds.dbg = nullptr;
    ds.stream = st;
    GemvA8Args a{w->data, (const int8_t*)xq, (const float*)xs, (const int32_t*)xsum, (float*)y,
                 M, w->in, w->out, w->bits, w->zp};
    return launch_gemv_a8(ctx, ds, a);
}
