// Tensor-parallel exchange of the sharded operator: all-gather (column split) and
// all-reduce (row split) of the per-rank results, written as one kernel over peer memory.
//
// Every rank owns a "region" that all ranks can address (peer access in one process, or a
// symmetric / IPC mapping across processes):
//
//   [0, 256)    flags    uint32 flag[src]: last epoch whose data rank `src` has delivered here
//   [256, 512)  control  uint32 epoch (exchanges completed by the owner), uint32 done (CTA counter)
//   [512, ...)  stage    [2 parities][nranks slots][slot_bytes]            plain results
//   then        pairs    [2 parities][nranks slots][2 * slot_bytes]        (value, epoch) pairs
//
// One exchange = one launch on every rank:
//   push     every CTA copies its chunk of the local result into slot `rank` (parity e & 1) of
//            every rank's stage with plain 16-byte peer stores, fences at system scope and
//            counts itself in; the last CTA to arrive releases flag[rank] = e on every rank.
//   combine  every CTA waits (time-bounded) until all flags of its own region have reached e,
//            then reads the slots back (L2, not L1: they were written by other GPUs) and either
//            lays them side by side (gather) or adds them in rank order (sum: every rank adds
//            the same numbers in the same order, so all ranks hold bit-identical results).
// Two parities make the slots of exchange e + 1 distinct from those of e: a fast rank may
// already push its next result while a slow one still reads the current one; it cannot get two
// ahead because its next combine needs the slow rank's next flag.  The flags only grow, so a
// launch captured in a CUDA graph replays correctly: the epoch lives in device memory.
//
// Decode shapes skip this kernel: the matmul kernel itself stores each result as a (value,
// epoch) pair into the `pairs` stage of every rank with one 8-byte store and, in its tail, polls
// the pairs of the other ranks until they carry the current epoch (gemv_stream.cu).  A pair
// needs no fence and no flag, which makes that exchange one NVLink crossing long.
//
// No collective library is involved and nothing here multicasts: peers are reached by ordinary
// stores, local data by ordinary loads.
#include <string.h>

#include <new>

#include "internal.h"
#include "sync_helpers.cuh"

namespace rstq {

constexpr int kTpThreads = 512;
constexpr uint32_t kTpMagic = 0x52535154;

struct TpParams {
    uint8_t* region[kTpMaxRanks];  // region[r] as seen from this device
    int rank, nranks;
    int64_t slot_bytes;
    const uint8_t* src;  // local result: rows x row_bytes, dense
    uint8_t* dst;        // gather: rows x (nranks * row_bytes); sum: rows x row_bytes
    int64_t rows, row_bytes;
    int* status;
    unsigned long long* dbg;  // optional phase timestamps (RSTQ_TUNE_TIMELINE), or null
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

template <int SUM>
__global__ void __launch_bounds__(kTpThreads) tp_exchange_kernel(const TpParams p) {
    __shared__ int s_last, s_ok;
    // let the next kernel of the stream start its prologue; wait for the one that produced src
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    uint8_t* mine = p.region[p.rank];
    uint32_t* ctl = reinterpret_cast<uint32_t*>(mine + 256);
    if (threadIdx.x == 0) s_ok = 1;
    // (the epoch is written by the previous exchange of this stream: read it after the wait)
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t e = *reinterpret_cast<volatile uint32_t*>(ctl) + 1u;  // this exchange's epoch
    unsigned long long* dbg = (p.dbg && blockIdx.x == 0 && threadIdx.x == 0) ? p.dbg : nullptr;
    if (dbg) dbg[2000] = gtime_ns();  // producer kernel finished, push starts
    const int64_t total = p.rows * p.row_bytes;
    const int64_t vecs = total >> 4;
    const int64_t per = (vecs + gridDim.x - 1) / gridDim.x;
    const int64_t v0 = per * blockIdx.x, v1 = min(vecs, v0 + per);
    const int64_t slot_off = kTpHeader + ((int64_t)(e & 1u) * p.nranks) * p.slot_bytes;

    // ---- push ----
    const uint4* src = reinterpret_cast<const uint4*>(p.src);
    for (int64_t v = v0 + threadIdx.x; v < v1; v += kTpThreads) {
        const uint4 val = __ldcg(src + v);
        for (int r = 0; r < p.nranks; ++r)
            reinterpret_cast<uint4*>(p.region[r] + slot_off + (int64_t)p.rank * p.slot_bytes)[v] = val;
    }
    __syncthreads();  // the CTA's stores happen before thread 0's release below (cumulative)
    if (threadIdx.x == 0) {
        __threadfence_system();
        s_last = gridDim.x == 1 ? 1 : (atomicAdd(ctl + 1, 1u) == gridDim.x - 1);
    }
    __syncthreads();
    if (s_last) {
        // every CTA of this rank has pushed and fenced: tell all ranks, then close the epoch
        if (threadIdx.x < p.nranks) {
            if (gridDim.x > 1) __threadfence_system();
            st_release_sys(reinterpret_cast<uint32_t*>(p.region[threadIdx.x]) + p.rank, e);
        }
        if (threadIdx.x == 0) {
            ctl[1] = 0u;
            *reinterpret_cast<volatile uint32_t*>(ctl) = e;  // all CTAs have read the old value by now
        }
    }

    if (dbg) dbg[2001] = gtime_ns();  // pushed and signalled

    // ---- combine ----
    if (threadIdx.x < p.nranks) {
        const uint32_t* flag = reinterpret_cast<const uint32_t*>(mine) + threadIdx.x;
        const unsigned long long t0 = gtime_ns();
        for (uint32_t spins = 1; (int32_t)(ld_acquire_sys(flag) - e) < 0; ++spins) {
            if ((spins & 63u) == 0 && gtime_ns() - t0 > kWaitLimitNs) {  // a rank never delivered:
                s_ok = 0;                                               // report, do not hang
                atomicExch(p.status, 2);
                break;
            }
        }
    }
    __syncthreads();
    if (dbg) dbg[2002] = gtime_ns();  // all ranks' data has arrived
    if (!s_ok) return;
    const uint8_t* stage = mine + slot_off;
    if (SUM) {
        float4* dst = reinterpret_cast<float4*>(p.dst);
        for (int64_t v = v0 + threadIdx.x; v < v1; v += kTpThreads) {
            float4 acc = __ldcg(reinterpret_cast<const float4*>(stage) + v);
            for (int r = 1; r < p.nranks; ++r) {
                const float4 t = __ldcg(reinterpret_cast<const float4*>(stage + (int64_t)r * p.slot_bytes) + v);
                acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
            }
            dst[v] = acc;
        }
    } else {
        const int64_t row_vecs = p.row_bytes >> 4;
        uint4* dst = reinterpret_cast<uint4*>(p.dst);
        for (int64_t v = v0 + threadIdx.x; v < v1; v += kTpThreads) {
            const int64_t row = v / row_vecs, col = v - row * row_vecs;
            for (int r = 0; r < p.nranks; ++r)
                dst[(row * p.nranks + r) * row_vecs + col] =
                    __ldcg(reinterpret_cast<const uint4*>(stage + (int64_t)r * p.slot_bytes) + v);
        }
    }
    if (dbg) dbg[2003] = gtime_ns();  // combined
}

}  // namespace rstq

using namespace rstq;

struct rstq_tp {
    uint32_t magic;
    rstq_ctx* ctx;
    int dev, rank, nranks;
    uint8_t* region[kTpMaxRanks];
    int64_t region_bytes, slot_bytes;
    bool owns_region;   // single-process set-up: this endpoint allocated region[rank]
    void* tmp;          // local result of rstq_tp_qmatmul before the exchange
    int64_t tmp_bytes;
};

static bool ok_tp(const rstq_tp* t) { return t && t->magic == kTpMagic && t->ctx && t->ctx->magic == kCtxMagic; }

static int32_t tp_exchange(rstq_tp* tp, const void* src, void* dst, int64_t rows, int64_t row_bytes, bool sum) {
    RSTQ_REQUIRE(rows >= 1 && row_bytes >= 16 && row_bytes % 16 == 0, RSTQ_E_SHAPE,
                 "an exchanged row must be a positive multiple of 16 bytes (got %lld)", (long long)row_bytes);
    RSTQ_REQUIRE(rows * row_bytes <= tp->slot_bytes, RSTQ_E_LIMIT,
                 "payload of %lld bytes exceeds the slot of %lld bytes this endpoint was created with",
                 (long long)(rows * row_bytes), (long long)tp->slot_bytes);
    RSTQ_REQUIRE((((uintptr_t)src | (uintptr_t)dst) & 15) == 0, RSTQ_E_ALIGN, "buffers must be 16-byte aligned");
    DeviceState& ds = tp->ctx->devs[tp->dev];
    int32_t rc = use_dev(tp->ctx, tp->dev);
    if (rc != RSTQ_OK) return rc;
    TpParams p{};
    for (int r = 0; r < tp->nranks; ++r) p.region[r] = tp->region[r];
    p.rank = tp->rank;
    p.nranks = tp->nranks;
    p.slot_bytes = tp->slot_bytes;
    p.src = (const uint8_t*)src;
    p.dst = (uint8_t*)dst;
    p.rows = rows;
    p.row_bytes = row_bytes;
    p.status = ds.status;
    p.dbg = ds.dbg;
    // one CTA per 8 KB (one 16-byte vector per thread: the copy loops are latency-bound), at most one per SM: all CTAs of a launch must be resident together
    // because each of them waits for the peers' flags
    const int64_t total = rows * row_bytes;
    int grid = (int)((total + 8191) / 8192);
    if (grid > ds.sm_count) grid = ds.sm_count;
    if (grid < 1) grid = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kTpThreads);
    cfg.stream = ds.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ds.pdl ? 1 : 0;
    RSTQ_CUDA(sum ? cudaLaunchKernelEx(&cfg, tp_exchange_kernel<1>, p) : cudaLaunchKernelEx(&cfg, tp_exchange_kernel<0>, p));
    tp->ctx->launches++;
    RSTQ_CUDA(cudaGetLastError());
    return RSTQ_OK;
}

extern "C" {

int64_t rstq_tp_region_bytes(int32_t nranks, int64_t max_payload_bytes) {
    if (nranks < 1 || nranks > kTpMaxRanks || max_payload_bytes < 16) return 0;
    const int64_t slot = (max_payload_bytes + 255) / 256 * 256;
    return kTpHeader + 6 * (int64_t)nranks * slot;
}

int32_t rstq_tp_attach(rstq_ctx* ctx, void* const* regions, rstq_tp** out, int32_t dev, int32_t rank,
                       int32_t nranks, int64_t region_bytes) {
    RSTQ_REQUIRE(ctx && ctx->magic == kCtxMagic, RSTQ_E_INVALID, "invalid context handle");
    RSTQ_REQUIRE(dev >= 0 && dev < (int)ctx->devs.size(), RSTQ_E_INVALID, "device index %d out of range", dev);
    RSTQ_REQUIRE(out && regions, RSTQ_E_INVALID, "null argument");
    RSTQ_REQUIRE(nranks >= 1 && nranks <= kTpMaxRanks && rank >= 0 && rank < nranks, RSTQ_E_INVALID,
                 "rank %d of %d (at most %d ranks)", rank, nranks, kTpMaxRanks);
    const int64_t slot = (region_bytes - kTpHeader) / (6 * (int64_t)nranks) / 256 * 256;
    RSTQ_REQUIRE(region_bytes > kTpHeader && slot >= 256, RSTQ_E_LIMIT, "region of %lld bytes is too small",
                 (long long)region_bytes);
    for (int r = 0; r < nranks; ++r)
        RSTQ_REQUIRE(regions[r] && ((uintptr_t)regions[r] & 255) == 0, RSTQ_E_ALIGN,
                     "region %d must be a 256-byte aligned device address", r);
    rstq_tp* tp = new (std::nothrow) rstq_tp{};
    RSTQ_REQUIRE(tp, RSTQ_E_OOM, "out of host memory");
    tp->magic = kTpMagic;
    tp->ctx = ctx;
    tp->dev = dev;
    tp->rank = rank;
    tp->nranks = nranks;
    for (int r = 0; r < nranks; ++r) tp->region[r] = (uint8_t*)regions[r];
    tp->region_bytes = region_bytes;
    tp->slot_bytes = slot;
    tp->owns_region = false;
    *out = tp;
    return RSTQ_OK;
}

int32_t rstq_tp_create_local(rstq_ctx* ctx, const int32_t* devs, rstq_tp** tps, int32_t nranks,
                             int64_t max_payload_bytes) {
    RSTQ_REQUIRE(ctx && ctx->magic == kCtxMagic, RSTQ_E_INVALID, "invalid context handle");
    RSTQ_REQUIRE(devs && tps, RSTQ_E_INVALID, "null argument");
    const int64_t bytes = rstq_tp_region_bytes(nranks, max_payload_bytes);
    RSTQ_REQUIRE(bytes > 0, RSTQ_E_INVALID, "need 1..%d ranks and a payload of at least 16 bytes", kTpMaxRanks);
    for (int r = 0; r < nranks; ++r) {
        RSTQ_REQUIRE(devs[r] >= 0 && devs[r] < (int)ctx->devs.size(), RSTQ_E_INVALID, "device index %d out of range",
                     devs[r]);
        for (int q = 0; q < r; ++q)
            RSTQ_REQUIRE(devs[q] != devs[r], RSTQ_E_INVALID, "ranks must sit on distinct devices");
    }
    // peer access both ways between every pair, then one zeroed region per rank
    for (int r = 0; r < nranks; ++r) {
        RSTQ_CUDA(cudaSetDevice(ctx->devs[devs[r]].ordinal));
        for (int q = 0; q < nranks; ++q) {
            if (q == r) continue;
            int can = 0;
            RSTQ_CUDA(cudaDeviceCanAccessPeer(&can, ctx->devs[devs[r]].ordinal, ctx->devs[devs[q]].ordinal));
            RSTQ_REQUIRE(can, RSTQ_E_NODEV, "device %d cannot address device %d", ctx->devs[devs[r]].ordinal,
                         ctx->devs[devs[q]].ordinal);
            const cudaError_t e = cudaDeviceEnablePeerAccess(ctx->devs[devs[q]].ordinal, 0);
            if (e == cudaErrorPeerAccessAlreadyEnabled)
                (void)cudaGetLastError();
            else
                RSTQ_CUDA(e);
        }
    }
    void* regions[kTpMaxRanks] = {};
    for (int r = 0; r < nranks; ++r) tps[r] = nullptr;
    auto undo = [&]() {   // a failure half-way: give back what was made so far
        for (int r = 0; r < nranks; ++r) {
            if (tps[r]) { tps[r]->magic = 0; delete tps[r]; tps[r] = nullptr; }
            if (regions[r]) { cudaSetDevice(ctx->devs[devs[r]].ordinal); cudaFree(regions[r]); }
        }
        cudaGetLastError();
    };
    for (int r = 0; r < nranks; ++r) {
        cudaError_t e = cudaSetDevice(ctx->devs[devs[r]].ordinal);
        if (e == cudaSuccess) e = cudaMalloc(&regions[r], (size_t)bytes);
        if (e == cudaSuccess) e = cudaMemset(regions[r], 0, (size_t)bytes);
        if (e == cudaSuccess) e = cudaDeviceSynchronize();
        if (e != cudaSuccess) {
            undo();
            return cuda_fail(e, "region allocation", __FILE__, __LINE__);
        }
    }
    for (int r = 0; r < nranks; ++r) {
        const int32_t rc = rstq_tp_attach(ctx, regions, &tps[r], devs[r], r, nranks, bytes);
        if (rc != RSTQ_OK) {
            undo();
            return rc;
        }
        tps[r]->owns_region = true;
    }
    return RSTQ_OK;
}

int32_t rstq_tp_allgather(rstq_tp* tp, rstq_buf* src, rstq_buf* dst, int64_t rows, int64_t row_bytes) {
    RSTQ_REQUIRE(ok_tp(tp), RSTQ_E_INVALID, "invalid endpoint handle");
    RSTQ_REQUIRE(src && dst && src->magic == kBufMagic && dst->magic == kBufMagic, RSTQ_E_INVALID, "invalid buffer");
    RSTQ_REQUIRE(src->dev == tp->dev && dst->dev == tp->dev, RSTQ_E_INVALID, "buffers live on another device");
    RSTQ_REQUIRE(rows >= 1 && row_bytes >= 1 && src->bytes >= rows * row_bytes &&
                     dst->bytes >= rows * row_bytes * tp->nranks,
                 RSTQ_E_SHAPE, "buffers too small for %lld rows of %lld bytes", (long long)rows, (long long)row_bytes);
    return tp_exchange(tp, src->ptr, dst->ptr, rows, row_bytes, false);
}

int32_t rstq_tp_allreduce_f32(rstq_tp* tp, rstq_buf* src, rstq_buf* dst, int64_t count) {
    RSTQ_REQUIRE(ok_tp(tp), RSTQ_E_INVALID, "invalid endpoint handle");
    RSTQ_REQUIRE(src && dst && src->magic == kBufMagic && dst->magic == kBufMagic, RSTQ_E_INVALID, "invalid buffer");
    RSTQ_REQUIRE(src->dev == tp->dev && dst->dev == tp->dev, RSTQ_E_INVALID, "buffers live on another device");
    RSTQ_REQUIRE(count >= 4 && count % 4 == 0 && src->bytes >= count * 4 && dst->bytes >= count * 4, RSTQ_E_SHAPE,
                 "count must be a positive multiple of 4 that fits both buffers (got %lld)", (long long)count);
    return tp_exchange(tp, src->ptr, dst->ptr, 1, count * 4, true);
}

int32_t rstq_tp_qmatmul(rstq_tp* tp, rstq_weight* w, rstq_buf* x, rstq_buf* y, int64_t M, int32_t act_dtype,
                        int32_t mode, int32_t split) {
    RSTQ_REQUIRE(ok_tp(tp), RSTQ_E_INVALID, "invalid endpoint handle");
    RSTQ_REQUIRE(w && w->magic == kWgtMagic && w->ctx == tp->ctx && w->dev == tp->dev, RSTQ_E_INVALID,
                 "weight shard belongs to another context or device");
    RSTQ_REQUIRE(x && y && x->magic == kBufMagic && y->magic == kBufMagic && x->dev == tp->dev && y->dev == tp->dev,
                 RSTQ_E_INVALID, "invalid buffer");
    RSTQ_REQUIRE(split == RSTQ_SPLIT_COLUMN || split == RSTQ_SPLIT_ROW, RSTQ_E_INVALID, "split must be column or row");
    // K-quant shards (the rows, or the K range in whole super-blocks, of the arrays a rank bound) take the
    // unfused route: quantizer, decode kernel, exchange kernel
    RSTQ_REQUIRE((!w->mins || w->kq) && (!w->pair_out || w->k6), RSTQ_E_INVALID,
                 "K-quant weights are sharded in their unit layouts only (RSTQ_TUNE_Q4K_UNITS / _Q6K_UNITS = 1)");
    RSTQ_REQUIRE(M >= 1, RSTQ_E_SHAPE, "M = %lld", (long long)M);
    RSTQ_REQUIRE(w->out % 4 == 0, RSTQ_E_SHAPE, "out of a shard must be a multiple of 4 (16-byte rows), got %lld",
                 (long long)w->out);
    const int64_t esz = act_dtype == RSTQ_BF16 ? 2 : 4;
    const int64_t full_out = split == RSTQ_SPLIT_COLUMN ? w->out * tp->nranks : w->out;
    RSTQ_REQUIRE(x->bytes >= M * w->in * esz && y->bytes >= M * full_out * 4, RSTQ_E_SHAPE,
                 "x or y too small for M = %lld", (long long)M);
    DeviceState& ds = tp->ctx->devs[tp->dev];
    int32_t rc = use_dev(tp->ctx, tp->dev);
    if (rc != RSTQ_OK) return rc;
    const int64_t need = M * w->out * 4;
    if (need > tp->tmp_bytes) {
        RSTQ_REQUIRE(!ds.capturing, RSTQ_E_INVALID, "first call of this size must happen outside graph capture");
        if ((rc = dev_release_scratch(ds, tp->tmp)) != RSTQ_OK) return rc;  // parked while a graph may name it
        tp->tmp = nullptr;
        tp->tmp_bytes = 0;
        RSTQ_CUDA(cudaMalloc(&tp->tmp, (size_t)need));
        tp->tmp_bytes = need;
    }
    // Decode shapes: the exchange runs in the tail of the matmul kernel itself (one launch).
    if (M * w->out * 4 <= tp->slot_bytes && w->out % 4 == 0 && ((uintptr_t)y->ptr & 15) == 0) {
        TpFuse f{};
        for (int r = 0; r < tp->nranks; ++r) f.region[r] = tp->region[r];
        f.rank = tp->rank;
        f.nranks = tp->nranks;
        f.sum = split == RSTQ_SPLIT_ROW;
        f.ll_off = kTpHeader + 2 * (int64_t)tp->nranks * tp->slot_bytes;
        f.slot_bytes = 2 * tp->slot_bytes;
        f.y = (float*)y->ptr;
        rc = matmul_device(tp->ctx, w, x->ptr, tp->tmp, M, act_dtype, RSTQ_F32, mode, &f);
        if (rc != kNotFused) return rc;
    }
    // Otherwise (prefill shapes, M cut into several launches): matmul, then the exchange kernel.
    rc = matmul_device(tp->ctx, w, x->ptr, tp->tmp, M, act_dtype, RSTQ_F32, mode);
    if (rc != RSTQ_OK) return rc;
    if (split == RSTQ_SPLIT_COLUMN) return tp_exchange(tp, tp->tmp, y->ptr, M, w->out * 4, false);
    return tp_exchange(tp, tp->tmp, y->ptr, 1, M * w->out * 4, true);
}

// ---- regions shared between processes: one process per GPU, the other ranks' regions are
// mapped through CUDA IPC handles that the host side passes around (any channel will do) ----
int32_t rstq_ipc_export(rstq_buf* buf, void* handle64) {
    RSTQ_REQUIRE(buf && buf->magic == kBufMagic && handle64, RSTQ_E_INVALID, "invalid buffer or null handle");
    RSTQ_REQUIRE(buf->owned, RSTQ_E_INVALID, "only buffers this library allocated can be exported");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle travels as 64 opaque bytes");
    int32_t rc = use_dev(buf->ctx, buf->dev);
    if (rc != RSTQ_OK) return rc;
    cudaIpcMemHandle_t h;
    RSTQ_CUDA(cudaIpcGetMemHandle(&h, buf->ptr));
    memcpy(handle64, &h, 64);
    return RSTQ_OK;
}

int32_t rstq_ipc_open(rstq_ctx* ctx, const void* handle64, void** device_ptr, int32_t dev) {
    RSTQ_REQUIRE(ctx && ctx->magic == kCtxMagic, RSTQ_E_INVALID, "invalid context handle");
    RSTQ_REQUIRE(dev >= 0 && dev < (int)ctx->devs.size(), RSTQ_E_NODEV, "device index %d out of range", dev);
    RSTQ_REQUIRE(handle64 && device_ptr, RSTQ_E_INVALID, "null argument");
    int32_t rc = use_dev(ctx, dev);
    if (rc != RSTQ_OK) return rc;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    RSTQ_CUDA(cudaIpcOpenMemHandle(device_ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return RSTQ_OK;
}

int32_t rstq_ipc_close(rstq_ctx* ctx, void* device_ptr, int32_t dev) {
    RSTQ_REQUIRE(ctx && ctx->magic == kCtxMagic, RSTQ_E_INVALID, "invalid context handle");
    RSTQ_REQUIRE(dev >= 0 && dev < (int)ctx->devs.size(), RSTQ_E_NODEV, "device index %d out of range", dev);
    RSTQ_REQUIRE(device_ptr, RSTQ_E_INVALID, "null argument");
    int32_t rc = use_dev(ctx, dev);
    if (rc != RSTQ_OK) return rc;
    RSTQ_CUDA(cudaStreamSynchronize(ctx->devs[dev].stream));
    RSTQ_CUDA(cudaIpcCloseMemHandle(device_ptr));
    return RSTQ_OK;
}

int32_t rstq_tp_free(rstq_tp* tp) {
    RSTQ_REQUIRE(ok_tp(tp), RSTQ_E_INVALID, "invalid endpoint handle");
    int32_t rc = use_dev(tp->ctx, tp->dev);
    if (rc != RSTQ_OK) return rc;
    // peers store into this rank's region: when this process drives them too (one process, several
    // devices), their streams must be idle before the region goes away
    if (tp->owns_region)
        for (auto& other : tp->ctx->devs) {
            if (other.ordinal < 0 || !other.stream) continue;
            cudaSetDevice(other.ordinal);
            cudaStreamSynchronize(other.stream);
        }
    if ((rc = use_dev(tp->ctx, tp->dev)) != RSTQ_OK) return rc;
    RSTQ_CUDA(cudaStreamSynchronize(tp->ctx->devs[tp->dev].stream));
    if (tp->tmp) cudaFree(tp->tmp);
    if (tp->owns_region) cudaFree(tp->region[tp->rank]);
    tp->magic = 0;
    delete tp;
    return RSTQ_OK;
}

}  // extern "C"
