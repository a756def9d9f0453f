/*
 * rstq -- Blackwell (sm_100a) quantized matmul for Raster: C ABI.
 *
 * This is the boundary Raster's Clojure host code binds through Panama FFM
 * (java.lang.foreign), the way it already binds its generated CPU kernels
 * (src/raster/compiler/backend/cpu/codegen.clj:100-125) and its OpenCL driver
 * (src/raster/gpu/ocl_runtime.clj:59-76, :192-199).  Conventions kept from
 * there:
 *   - pointers first, then scalars, in every signature;
 *   - only int32_t / int64_t / float / double / pointers cross the boundary;
 *   - every function returns an int32_t status (0 = ok, < 0 = error code) and
 *     hands results back through out-pointers; rstq_last_error() returns the
 *     text of the calling thread's most recent failure;
 *   - no C++ exception and no abort() crosses this boundary;
 *   - every create has a destroy; destroying NULL is a no-op returning 0.
 *
 * Shapes use the reference's names: `in` = K (reduction length), `out` = N
 * (rows of W; W is row-major [out, in]); a block is 32 consecutive K elements
 * of one row; nb = in / 32.  Activations are row-major [M, in], results
 * row-major [M, out].
 *
 * Threading: a context is thread-compatible -- calls on one context must be
 * serialised by the caller.  Work on one device of a context runs in order on
 * that device's stream and is asynchronous to the host unless stated.
 */
#ifndef RSTQ_H
#define RSTQ_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RSTQ_API __attribute__((visibility("default")))

typedef struct rstq_ctx rstq_ctx;
typedef struct rstq_buf rstq_buf;
typedef struct rstq_weight rstq_weight;
typedef struct rstq_graph rstq_graph;
typedef struct rstq_event rstq_event;

/* status codes */
#define RSTQ_OK 0
#define RSTQ_E_INVALID (-1)  /* null pointer, bad enum, bad handle            */
#define RSTQ_E_SHAPE (-2)    /* in % 32 != 0, out % 8 != 0 (stream layout), M < 1, size overflow */
#define RSTQ_E_ALIGN (-3)    /* device pointer / offset not 16-byte aligned   */
#define RSTQ_E_CUDA (-4)     /* a CUDA runtime call failed                    */
#define RSTQ_E_OOM (-5)      /* device or pinned-host allocation failed       */
#define RSTQ_E_NODEV (-6)    /* no CUDA device, or device index out of range  */
#define RSTQ_E_ARCH (-7)     /* device is not compute capability 10.x         */
#define RSTQ_E_DEVICE (-8)   /* handles live on different devices             */
#define RSTQ_E_STATE (-9)    /* call not legal now (e.g. sync during capture) */
#define RSTQ_E_LIMIT (-10)   /* problem exceeds a stated fixed limit          */
#define RSTQ_E_RANGE (-11)   /* offset + bytes beyond the buffer              */
#define RSTQ_E_WAIT (-12)    /* a time-bounded wait inside a kernel ran out; results of that
                                launch are invalid (reported by rstq_sync)     */

/* weight formats (the `format` argument of rstq_weight_bind) */
#define RSTQ_FMT_Q4_0 0 /* unsigned nibble, zero point 8, two per byte (lo = elem k, hi = elem k+16);
                           src/raster/compiler/backend/cpu/quant.clj:27-31 */
#define RSTQ_FMT_Q8_0 1 /* unsigned byte, zero point 128; src/raster/compiler/backend/cpu/quant.clj:33-39 */
#define RSTQ_FMT_Q8_S 2 /* signed int8 codes, W = scale * code; src/raster/quant/train.clj:34-71,
                           and, read as bytes, the int32-packed rows of src/raster/quant/pack.clj:55-81 */

/* host layouts accepted at bind time */
#define RSTQ_LAYOUT_ROWMAJOR 0 /* codes row-major by output row, scales [out, nb] */
#define RSTQ_LAYOUT_STREAM8 1  /* 8-row interleaved stream layout (wqi / wsi);
                                  src/raster/compiler/core/layout.clj:246-286; needs out % 8 == 0 */

/* element types of activations / results */
#define RSTQ_F32 0
#define RSTQ_BF16 1 /* raw bits in uint16_t, as the reference carries f16 in short[] */

/* arithmetic modes */
#define RSTQ_MODE_F 0  /* y = dequant(W) . x on the float activations (f32 accumulate) */
#define RSTQ_MODE_A8 1 /* activations quantized per 32-block to int8 inside the op, integer block
                          dots, per-block scale fold: the arithmetic of qlinear-i8 */

/* shard kinds (rstq_weight_bind_shard) */
#define RSTQ_SPLIT_NONE 0
#define RSTQ_SPLIT_COLUMN 1 /* rank owns output rows [rank*out/P, (rank+1)*out/P) */
#define RSTQ_SPLIT_ROW 2    /* rank owns K range   [rank*in/P,  (rank+1)*in/P) of every row */

/* tuning keys (rstq_tune) */
#define RSTQ_TUNE_GEMM_MIN_M 1  /* smallest M routed to the tensor-core GEMM (default 17; at the
                                   default, MODE_F also takes it from M = 9 when the rows are too long
                                   for the decode kernel to hold M tokens in shared memory) */
#define RSTQ_TUNE_GEMM_KERNEL 0  /* prefill GEMM: 0 (default) = dequantized weights kept in tensor
                                     memory, 1 = staged through shared memory */
#define RSTQ_TUNE_PDL 2           /* 1 (default) = launch the decode kernels with programmatic
                                     dependent launch so consecutive launches overlap; 0 = plain */
#define RSTQ_TUNE_TIMELINE 3      /* 1 = streaming kernel records per-CTA phase timestamps */
#define RSTQ_TUNE_GEMV_PLAN 4     /* decode kernel work split: 0 (default) = choose per shape, 1 = equal
                                     unit ranges (32-row groups may be shared by neighbouring thread
                                     blocks), 2 = whole 32-row groups per thread block */
#define RSTQ_TUNE_GEMV_PREFETCH 7  /* decode kernels: KB of a thread block's weight range requested into L2
                                     ahead of its shared-memory ring; -1 (default) = 64 KB for matrices of
                                     16 .. 64 MB, none otherwise; 0 = none */
#define RSTQ_TUNE_PROBE 8         /* only in a library built with -DRSTQ_PROBES=1 (otherwise any value but 0 is
                                     refused): timing probes of the decode kernel, RESULTS ARE INVALID while
                                     set: 1 = the weight stream is not copied (consumer rate alone), 2 = the
                                     arithmetic is skipped (copy rate alone) */
#define RSTQ_TUNE_PREFETCH_NEXT 9  /* 1 (default) = a decode launch asks for the head of the weight that followed
                                     it last time on this device to be brought into L2 (up to 48 MB) while its own
                                     consumers drain: a decode loop walks its matrices in the same order for
                                     every token, so consecutive launches overlap at the memory system.  A hint
                                     only: results never depend on it.  A launch recorded in a graph keeps
                                     naming that weight: destroy graphs before freeing weights they ran beside.
                                     0 = off */
#define RSTQ_TUNE_Q4K_UNITS 11   /* 1 (default) = Q4_K weights bound from now on are stored as 768-byte units with the
                                     sub-block minima behind the scales and the decode kernel adds the min term
                                     itself (quantizer + one kernel); 0 = 640-byte units and a third kernel for it */
#define RSTQ_TUNE_Q6K_UNITS 12   /* 1 (default) = Q6_K weights bound from now on are stored as 1280-byte units (8-bit
                                     codes, one scale per row and 16 elements: the reference's code bytes) and
                                     take quantizer + one decode launch; 0 = two twin rows of 8-bit units per
                                     row (twice the code bytes) and a third kernel that adds the pairs */
#define RSTQ_TUNE_GEMM_WIDE 13    /* prefill GEMM above 128 tokens, 256-token tiles (one accumulator, one issuing
                                     thread) instead of 128-token ones: 0 (default) = where the grid then needs
                                     fewer cycles over its waves of thread blocks, 1 = never, 2 = always,
                                     3 = as 0 but never two thread blocks per tile (each half of K) */
#define RSTQ_TUNE_TP_TAIL 15      /* fused decode + exchange (rstq_tp_qmatmul): how many thread blocks of the decode kernel
                                     stay for the exchange's tail (wait for the peers' results, write y); the others
                                     leave their SMs to the next launch, which fills its weight rings meanwhile.
                                     0 = all of them; default 32, and never fewer than one thread per pair of results */
#define RSTQ_TUNE_ACT_RING 14     /* MODE_A8 decode launches of 2 .. 16 tokens, how the activations share shared memory
                                     with the weight ring: 0 (default) = every ring stage carries its own slice of
                                     the activation image wherever that image exists (always in rstq_qmatmul; in
                                     rstq_qmatmul_prequant and for Q4_K / Q6_K weights it is built when the
                                     resident form would need more launches or leave a shallower ring), so shared memory does not grow with K and
                                     the image is read from L2 once per 32-row group; 1 = all of K resident beside
                                     the ring (tokens that do not fit go to further launches, each streaming the
                                     weights again); 2 = as 0, also where the resident form fits; 3 = the slices
                                     ride 32-unit chunks; 4 = resident, 32-unit chunks (3, 4: measured slower).
                                     Every token's result is the same bit for bit in every setting, except that a
                                     last launch of ONE token (setting 1 or 4) adds a row's blocks up in the M = 1
                                     kernel's order.  MODE_F decode launches follow the same key: 0 = staged
                                     activations that do not fit in shared memory for all of K ride the ring (up
                                     to 16 columns: bf16 tokens, or two bf16 terms per f32 token), 1 / 4 = further
                                     launches (or the tensor-core route) instead */
#define RSTQ_TUNE_ACT_IMAGE 10    /* 1 (default) = rstq_qmatmul in MODE_A8 at 2 <= M < 64: the activation quantizer
                                     also writes the codes, scales and sums in the order the decode kernel
                                     keeps them in shared memory, and that kernel's copy thread brings them
                                     in with bulk copies beside the weight stream; 0 = the kernel's warps
                                     gather them from the quantizer's row-major output first */
#define RSTQ_TUNE_FUSE_QUANT 6    /* 1 (default) = rstq_qmatmul in MODE_A8 at M = 1 quantizes the
                                     activations inside the decode kernel; 0 = separate quantizer launch */

/* ---- library / errors -------------------------------------------------- */
RSTQ_API int32_t rstq_version(void);
RSTQ_API const char* rstq_last_error(void);
RSTQ_API int32_t rstq_device_count(int32_t* count);

/* ---- context: replaces the session / runtime init of
 *      src/raster/gpu/core.clj:243-293 and src/raster/gpu/ocl_runtime.clj:205-215.
 * `devices` lists CUDA ordinals; later calls name a device by its index in
 * that list (device index 0 = devices[0]). ------------------------------- */
RSTQ_API int32_t rstq_init(const int32_t* devices, rstq_ctx** ctx, int32_t ndev);
RSTQ_API int32_t rstq_shutdown(rstq_ctx* ctx);
/* How the prefill GEMM (M above the decode kernel's range) would tile a call on a device of sm_count SMs
 * at the default settings: plan2[0] = tokens per tile (32, 64, 128 or 256), plan2[1] = thread blocks per
 * tile (2 = each takes half of K; the second hands its sums to the first).  Pure host arithmetic: no
 * device, no context.  No counterpart in the reference (its GEMM is one work-item per output). */
RSTQ_API int32_t rstq_gemm_plan(int32_t* plan2, int64_t out, int64_t in, int64_t m, int32_t sm_count);
/* What the FIRST decode launch of rstq_qmatmul (mode, bits 4 / 8, act_dtype) on an out x in weight with m tokens
 * would be at the default settings on a device of sm_count SMs: plan6[0] = tokens it takes (up to 16; 0 = a
 * row of activations does not fit at all), [1] = ring stages, [2] = units per chunk, [3] = 1 when the
 * activations ride the ring (RSTQ_TUNE_ACT_RING), [4] = dynamic shared memory in bytes (<= 231424),
 * [5] = thread blocks.  Pure host arithmetic: no device, no context.  No counterpart in the reference. */
RSTQ_API int32_t rstq_decode_plan(int32_t* plan6, int32_t mode, int32_t bits, int64_t out, int64_t in, int64_t m,
                                  int32_t act_dtype, int32_t sm_count);
RSTQ_API int32_t rstq_sync(rstq_ctx* ctx, int32_t dev);
RSTQ_API int32_t rstq_tune(rstq_ctx* ctx, int32_t key, int64_t value);
/* out[0] = SM count, out[1] = L2 bytes, out[2] = total device memory, out[3] = cc major*10+minor */
RSTQ_API int32_t rstq_device_info(rstq_ctx* ctx, int64_t* out4, int32_t dev);
/* Phase timestamps (ns, device global timer) of the streaming decode launches made since
 * RSTQ_TUNE_TIMELINE was set to 1: six slots of 160 rows used in turn (launch k writes slot k % 6),
 * a row of 8 values per CTA: [0] entry, [1] consumers start (the preceding kernel has finished),
 * [2] activations staged, [3] first weights landed, [4] main loop done, [5] exit, [6] SM id.
 * Rows of CTAs a launch did not have read as zero. */
RSTQ_API int32_t rstq_timeline_read(rstq_ctx* ctx, int64_t* out, int32_t dev, int64_t n);

/* ---- device buffers: make-buffer / array->buffer! / buffer->array /
 *      free-buffer! of src/raster/gpu/ocl_runtime.clj:405-499. ----------- */
RSTQ_API int32_t rstq_alloc(rstq_ctx* ctx, rstq_buf** buf, int32_t dev, int64_t bytes);
RSTQ_API int32_t rstq_free(rstq_buf* buf);
RSTQ_API int32_t rstq_upload(rstq_buf* buf, const void* host, int64_t offset, int64_t bytes);
RSTQ_API int32_t rstq_download(rstq_buf* buf, void* host, int64_t offset, int64_t bytes);
RSTQ_API int32_t rstq_memset(rstq_buf* buf, int32_t byte_value, int64_t offset, int64_t bytes);
RSTQ_API int32_t rstq_buf_ptr(rstq_buf* buf, void** device_ptr, int64_t* bytes);
/* A buffer handle over device memory the caller allocated (a runtime's own arena, a tensor of
 * another library); rstq_free releases the handle only.  The reference's counterpart is
 * buffer-of-array (src/raster/gpu/ocl_runtime.clj:452-499), which wraps an existing segment. */
RSTQ_API int32_t rstq_buf_wrap(rstq_ctx* ctx, rstq_buf** buf, void* device_ptr, int32_t dev, int64_t bytes);
/* Launch on a CUDA stream of the caller (cudaStream_t) instead of the context's own, so that the
 * operators order with the caller's other work without events; NULL returns to the own stream.
 * Plays the part of *current-arena* (src/raster/gpu/ocl_runtime.clj:222-224): the queue every
 * launch of the session goes to. */
RSTQ_API int32_t rstq_stream_set(rstq_ctx* ctx, void* stream, int32_t dev);

/* ---- weights: the one-time host->device bind.  Replaces repack-stream
 *      (src/raster/compiler/backend/cpu/quant.clj:317-326) as the load-time
 *      layout transform: the host arrays keep the reference's layouts, the
 *      device copy is re-tiled for the sm_100a kernels. ------------------- */
RSTQ_API int32_t rstq_weight_bind(rstq_ctx* ctx, rstq_weight** w, const void* codes,
                                  const float* scales, int32_t dev, int64_t out, int64_t in,
                                  int32_t format, int32_t layout);
/* Bind rank `rank` of `nranks`'s shard of a full host matrix (column or row split). */
RSTQ_API int32_t rstq_weight_bind_shard(rstq_ctx* ctx, rstq_weight** w, const void* codes,
                                        const float* scales, int32_t dev, int64_t out, int64_t in,
                                        int32_t format, int32_t layout, int32_t split,
                                        int32_t rank, int32_t nranks);
/* Q4_K, the reference's asymmetric 4-bit super-block format, from the arrays quantize-weight-q4k
 * makes (src/raster/compiler/backend/cpu/quant.clj:85-150): wq nibbles [out, in/2] (element k low,
 * k+16 high per 32-element sub-block), da / db f32 [out, in/256], aq (0..63) / bq (-32..31) int8
 * [out, in/32]; in % 256 == 0.  On the device the sub-block scales da*aq ride the 4-bit units of
 * the decode kernel, and so do the minima db*bq (768-byte units; RSTQ_TUNE_Q4K_UNITS = 0 keeps them
 * as a separate f32 [out, in/32] array folded by a second kernel).  Such a weight is
 * used with rstq_qmatmul (f32 activations, MODE_A8: q8_K quantizer + qmatmul-q4k, the `:apply` of
 * the registered :q4_K format, src/raster/quant/core.clj:57-66) and rstq_qmatmul_prequant (xs per
 * super-block [M, in/256], xsum = bsums [M, in/32]: qmatmul-q4k-dp4a!,
 * src/raster/quant/kernels_k.clj:195-237).  Sharded by binding a rank's rows (column split) or its
 * super-blocks of K (row split) and calling rstq_tp_qmatmul, which then runs the exchange as a launch
 * of its own.  No tensor-core route, no MODE_F. */
RSTQ_API int32_t rstq_weight_bind_q4k(rstq_ctx* ctx, rstq_weight** w, const void* wq, const float* da,
                                      const float* db, const int8_t* aq, const int8_t* bq, int32_t dev,
                                      int64_t out, int64_t in);
/* Q6_K from the arrays quantize-weight-q6k makes (src/raster/compiler/backend/cpu/quant.clj:222-262):
 * wq one unsigned 6-bit code per byte [out, in] (zero point 32), sc int8 [out, in/16], ds f32
 * [out, in/256]; in % 256 == 0.  Used with rstq_qmatmul / rstq_qmatmul_host (f32 activations,
 * MODE_A8: q8_K quantizer + qmatmul-q6k, the `:apply` of :q6_K, src/raster/quant/core.clj:68-75).
 * Held on the device as two 8-bit rows per matrix row (twice the reference's code bytes). */
RSTQ_API int32_t rstq_weight_bind_q6k(rstq_ctx* ctx, rstq_weight** w, const void* wq, const int8_t* sc,
                                      const float* ds, int32_t dev, int64_t out, int64_t in);
/* Second device copy of a bound weight at a distinct address (cold-cache measurement). */
RSTQ_API int32_t rstq_weight_clone(rstq_weight* src, rstq_weight** w);
RSTQ_API int32_t rstq_weight_free(rstq_weight* w);
/* out[0]=out rows, out[1]=in, out[2]=bits, out[3]=device bytes (codes+scales as stored),
 * out[4]=algorithmic stream bytes out*in*bits/8 + out*nb*4, out[5]=device index */
RSTQ_API int32_t rstq_weight_info(rstq_weight* w, int64_t* out6);

/* ---- activation quantizer on the device: quantize-act-i8 of
 *      src/raster/compiler/backend/cpu/quant.clj:282-305 (xsum != NULL) and
 *      quant-act-i8-rows-gpu! of src/raster/quant/kernels_k.clj:309-342
 *      (xsum == NULL; xq read as int32 words is its `xp`).
 *      x: f32 [M, in]; xq: int8 [M, in]; xs: f32 [M, nb]; xsum: int32 [M, nb].
 *      Bit-exact with the reference (double-precision scale and rounding). */
RSTQ_API int32_t rstq_quant_act_i8(rstq_ctx* ctx, rstq_buf* x, rstq_buf* xq, rstq_buf* xs,
                                   rstq_buf* xsum, int64_t M, int64_t in);

/* q8_K activation quantizer, quant-act-q8k-gpu! (src/raster/quant/kernels_k.clj:93-134; CPU form
 * quantize-act-q8k, src/raster/compiler/backend/cpu/quant.clj:172-193): per 256-element
 * super-block d = max|x|/127, codes = round-half-up(x/d); x f32 [rows, in], xq int8 [rows, in]
 * (read as int32 words it is the reference's `xp`), xs f32 [rows, in/256], bsums int32
 * [rows, in/sub] = code sums per sub-block of `sub` = 32 (Q4_K) or 16 (Q6_K) elements.
 * Bit-exact with the reference.  One launch, no `submax` scratch. */
RSTQ_API int32_t rstq_quant_act_q8k(rstq_ctx* ctx, rstq_buf* x, rstq_buf* xq, rstq_buf* xs, rstq_buf* bsums,
                                    int64_t rows, int64_t in, int32_t sub);

/* ---- the matmul on device-resident data.
 * rstq_qmatmul: y[M, out] = W . x[M, in]; x is act_dtype, y is out_dtype.
 *   MODE_A8 quantizes x inside the call -- the arithmetic of qlinear-i8! / qlinear-i8-q8!
 *   (src/raster/quant/op.clj:43-51, :81-90); bf16 activations are widened exactly first, so they
 *   give the result of the same values passed as f32.  At M = 1 (in <= 12288) the quantizer runs
 *   inside the decode kernel (same codes, scales and sums, bit for bit).  Up to M = 63 the block dots
 *   are exact integers and the result agrees with the reference formula to <= 2e-6 of max|y|; from
 *   M = 64 -- and from M = 17 when in > 16384, where the decode kernel would need a launch per 16
 *   tokens of rows that long -- the exact codes and scales feed the fp16 tensor-core path instead: <= 1e-3 of
 *   max|y| (measured ~4e-5), no longer the exact integer dots.  RSTQ_TUNE_GEMM_MIN_M raised above
 *   M keeps the exact path at any size.
 *   MODE_F multiplies the float activations directly -- qlinear-q8
 *   (src/raster/quant/train.clj:77-108) and the prefill GEMM: decode kernel (f32-grade, <= 2e-5)
 *   up to M = 16, tensor-core path (<= 1e-3) from M = 17, and already from M = 9 (f32 activations;
 *   from M = 2 with RSTQ_TUNE_ACT_RING = 1) when the matrix is larger than 4 MB and the decode kernel
 *   would have to stream it twice or more: activations that do not fit in shared memory for all of K
 *   ride the weight ring, up to 16 columns (bf16 tokens, or two exact bf16 terms per f32 token).
 * rstq_qmatmul_prequant: the kernel-level call of the reference,
 *   (xq xs xsum wqi wsi y in out ...) of qmatmul-q4-x8! / qmatmul-q8-x8!
 *   (src/raster/quant/kernels.clj:216-247, :308-333), and with xsum == NULL and a
 *   Q8_S weight the signed x signed qmatmul-i8-gemm!
 *   (src/raster/quant/kernels_k.clj:344-370). y is f32. */
RSTQ_API int32_t rstq_qmatmul(rstq_ctx* ctx, rstq_weight* w, rstq_buf* x, rstq_buf* y, int64_t M,
                              int32_t act_dtype, int32_t out_dtype, int32_t mode);
RSTQ_API int32_t rstq_qmatmul_prequant(rstq_ctx* ctx, rstq_weight* w, rstq_buf* xq, rstq_buf* xs,
                                       rstq_buf* xsum, rstq_buf* y, int64_t M);

/* Allocation-free form of rstq_qmatmul_prequant: same arithmetic and the same kernel, for
 * hosts that may not allocate device memory when they call -- a runtime that owns all
 * device memory through its own arena, a caller inside a stream capture, a decode loop that
 * must stay clear of the driver's allocator.  Has no counterpart in the reference.
 * xq / xs / xsum / y are plain 16-byte-aligned device pointers (int8 [M, in], f32 [M, nb],
 * int32 [M, nb], f32 [M, out]) on the weight's device; `stream` is a cudaStream_t, or NULL for
 * the context's own stream.  The split-group scratch lives in fixed arrays inside the
 * library's device image (about 1.3 MB held by every GPU that loads the library, until
 * exit), hence the limits: out <= 2 097 152 rows (RSTQ_E_LIMIT beyond), M cut into launches of
 * <= 16.  The first call on a device resolves the arrays' addresses and clears the counters:
 * make that call before any stream capture.  Every call shares the arrays: calls that could
 * overlap on the GPU must be serialised by the caller.  No cudaMalloc / cudaFree is reached. */
RSTQ_API int32_t rstq_qmatmul_prequant_noalloc(rstq_weight* w, const void* xq, const void* xs,
                                               const void* xsum, void* y, void* stream, int64_t M);

/* ---- the operators on HOST arrays, same argument order as the reference's
 *      CPU operators, so the Clojure method bodies change one call.  x and y
 *      cross PCIe on every call; the weight is uploaded and re-tiled on first
 *      sight of its (codes pointer, scales pointer, in, out) and kept resident
 *      (weights are immutable after load); rstq_weight_cache_clear drops it.
 *      These calls block until y is on the host.
 *   rstq_qlinear_i8      qlinear-i8!       src/raster/quant/op.clj:43-51   (Q4_0 wqi/wsi)
 *   rstq_qlinear_i8_q8   qlinear-i8-q8!    src/raster/quant/op.clj:81-90   (Q8_0 wqi/wsi)
 *   rstq_qlinear_q8      qlinear-q8        src/raster/quant/train.clj:77-108
 *   rstq_qmatmul_i8_gemm qmatmul-i8-gemm!  src/raster/quant/kernels_k.clj:344-370
 *   rstq_i8gemv_dp4a     i8gemv-dp4a!      src/raster/quant/kernels_k.clj:141-150 */
RSTQ_API int32_t rstq_qlinear_i8(rstq_ctx* ctx, const float* x, const void* wqi, const float* wsi,
                                 float* y, int64_t in, int64_t out);
RSTQ_API int32_t rstq_qlinear_i8_q8(rstq_ctx* ctx, const float* x, const void* wqi,
                                    const float* wsi, float* y, int64_t in, int64_t out);
RSTQ_API int32_t rstq_qlinear_q8(rstq_ctx* ctx, const float* x, const void* codes,
                                 const float* scales, float* y, int64_t m, int64_t in,
                                 int64_t out);
/* qlinear-q8-dx (src/raster/quant/train.clj:110-142), the backward-data of qlinear-q8:
 * dx[m, in] = dy[m, out] . dequant(codes, scales), W frozen.  Host arrays, same argument order. */
RSTQ_API int32_t rstq_qlinear_q8_dx(rstq_ctx* ctx, const float* dy, const void* codes,
                                    const float* scales, float* dx, int64_t m, int64_t in,
                                    int64_t out);
/* qlinear-q8-dx on device-resident arrays: dy f32 [m, out], codes int8 [out, in] and scales f32
 * [out, in/32] row-major as the reference holds them, dx f32 [m, in]. */
RSTQ_API int32_t rstq_qlinear_q8_dx_device(rstq_ctx* ctx, rstq_buf* dy, rstq_buf* codes, rstq_buf* scales,
                                           rstq_buf* dx, int64_t m, int64_t in, int64_t out);
RSTQ_API int32_t rstq_qmatmul_i8_gemm(rstq_ctx* ctx, const int32_t* xp, const float* xs,
                                      const int32_t* wp, const float* ws, float* y, int64_t in,
                                      int64_t out, int64_t nrows);
RSTQ_API int32_t rstq_i8gemv_dp4a(rstq_ctx* ctx, const int32_t* wp, const int32_t* xp, float* y,
                                  int64_t kw, int64_t out);
/* Host x / y against an already bound weight (the resident path for callers whose
 * arrays move, e.g. JVM heap arrays): x is act_dtype [M, in], y is f32 [M, out]. */
RSTQ_API int32_t rstq_qmatmul_host(rstq_ctx* ctx, rstq_weight* w, const void* x, float* y,
                                   int64_t M, int32_t act_dtype, int32_t mode);
RSTQ_API int32_t rstq_weight_cache_clear(rstq_ctx* ctx);

/* ---- graphs and events: record-graph! / replay-graph! / destroy-graph! of
 *      src/raster/gpu/ocl_runtime.clj:1051-1084 and the per-kernel device
 *      timestamps of src/raster/gpu/core.clj:1343-1388. -------------------- */
RSTQ_API int32_t rstq_graph_begin(rstq_ctx* ctx, int32_t dev);
RSTQ_API int32_t rstq_graph_end(rstq_ctx* ctx, rstq_graph** graph, int32_t dev);
RSTQ_API int32_t rstq_graph_replay(rstq_graph* graph);
RSTQ_API int32_t rstq_graph_destroy(rstq_graph* graph);
RSTQ_API int32_t rstq_event_create(rstq_ctx* ctx, rstq_event** ev, int32_t dev);
RSTQ_API int32_t rstq_event_record(rstq_event* ev);
RSTQ_API int32_t rstq_event_elapsed_ms(rstq_event* start, rstq_event* stop, float* ms);
RSTQ_API int32_t rstq_event_destroy(rstq_event* ev);
/* Number of kernels this library has launched on the context since init. */
RSTQ_API int32_t rstq_launch_count(rstq_ctx* ctx, int64_t* count);

/* ---- decode-chain neighbours of the matmul (f32, device buffers), so a decoder layer's chain
 *      rms-norm -> quantize -> matmul -> SwiGLU / GeGLU -> residual stays on the device and in one
 *      graph.  rms-norm!  src/raster/dl/nn.clj:497-513 (per row: x / sqrt(mean x^2 + eps) *
 *      (gain_offset + weight)); silu-mul! :200-203; gelu-mul! :208-214 (tanh form); residual-add!
 *      :217-219.  rstq_rms_norm_quant_act = rms-norm! followed by quantize-act-i8 in one kernel:
 *      the codes, scales and block sums are bit-identical to rstq_quant_act_i8 run on
 *      rstq_rms_norm's output (features % 32 == 0; xsum may be NULL). ----------------------- */
RSTQ_API int32_t rstq_rms_norm(rstq_ctx* ctx, rstq_buf* x, rstq_buf* weight, rstq_buf* out,
                               int64_t rows, int64_t features, double eps, double gain_offset);
RSTQ_API int32_t rstq_rms_norm_quant_act(rstq_ctx* ctx, rstq_buf* x, rstq_buf* weight, rstq_buf* xq,
                                         rstq_buf* xs, rstq_buf* xsum, int64_t rows,
                                         int64_t features, double eps, double gain_offset);
RSTQ_API int32_t rstq_silu_mul(rstq_ctx* ctx, rstq_buf* gate, rstq_buf* up, rstq_buf* out, int64_t n);
RSTQ_API int32_t rstq_gelu_mul(rstq_ctx* ctx, rstq_buf* gate, rstq_buf* up, rstq_buf* out, int64_t n);
RSTQ_API int32_t rstq_residual_add(rstq_ctx* ctx, rstq_buf* a, rstq_buf* b, rstq_buf* out, int64_t n);

/* The attention steps of the same chain, one token (src/raster/dl/attention.clj):
 *   rstq_rope_pos      rope-pos-gpu! :386-408 / rope-pos-buf! :482-499 -- NeoX rotate-half of x
 *                      [heads, head_dim] at absolute position pos (out may be x);
 *   rstq_kv_append     kv-append! :413-416 / kv-append-buf! :501-504 -- cache[pos*kvrow + i] = src[i];
 *                      the cache buffer holds maxpos rows (checked against pos when it is a host scalar);
 *   rstq_gqa_decode_attention  gqa-decode-attention-gpu! :423-471 / -buf! :514-575 -- per query head
 *                      softmax(scale * q.K^T) V over cache positions [0, cache_len), K / V caches
 *                      [maxpos][n_kv][head_dim], n_q = group * n_kv, head_dim % 4 == 0 and <= 256.
 * posbuf / clenbuf: NULL, or a device buffer holding one int64 that the kernel reads (the -buf
 * variants: a captured graph then serves every token; call once before capturing).  The
 * reference's score scratch `sc` has no counterpart (scores stay in registers).  All f32. */
RSTQ_API int32_t rstq_rope_pos(rstq_ctx* ctx, rstq_buf* x, rstq_buf* out, rstq_buf* posbuf, int64_t heads,
                               int64_t head_dim, double theta, int64_t pos);
RSTQ_API int32_t rstq_kv_append(rstq_ctx* ctx, rstq_buf* src, rstq_buf* cache, rstq_buf* posbuf, int64_t kvrow,
                                int64_t pos, int64_t maxpos);
/* Fusions the chain invites (no counterpart in the reference; each equals its steps run one by one,
 * bit for bit):
 *   rstq_rope_append                  rope of q and k in place + append of the turned k and of v to
 *                                     their caches: four steps, one launch;
 *   rstq_residual_rms_norm_quant_act  sum = a + b (stored: the residual stream), then rms-norm of
 *                                     sum quantized to int8 blocks; sum may not alias a or b;
 *   rstq_silu_mul_quant_act / rstq_gelu_mul_quant_act   the gated activation quantized to int8
 *                                     blocks (the input of the down projection), n % 32 == 0. */
/* rstq_gqa_decode_attention whose output is also quantized to int8 blocks of 32 (codes, scales, sums as
 * rstq_quant_act_i8 gives them for `out`) by the CTA that writes it: the o projection then starts from
 * rstq_qmatmul_prequant.  head_dim 64 or 128; xsum may be NULL. */
RSTQ_API int32_t rstq_gqa_decode_attention_quant_act(rstq_ctx* ctx, rstq_buf* q, rstq_buf* k, rstq_buf* v,
                                                     rstq_buf* out, rstq_buf* xq, rstq_buf* xs, rstq_buf* xsum,
                                                     rstq_buf* clenbuf, int64_t cache_len, int64_t n_q,
                                                     int64_t group, int64_t n_kv, int64_t head_dim,
                                                     int64_t maxpos, double scale);
RSTQ_API int32_t rstq_rope_append(rstq_ctx* ctx, rstq_buf* q, rstq_buf* k, rstq_buf* v, rstq_buf* kcache,
                                  rstq_buf* vcache, rstq_buf* posbuf, int64_t n_q, int64_t n_kv,
                                  int64_t head_dim, double theta, int64_t pos, int64_t maxpos);
RSTQ_API int32_t rstq_residual_rms_norm_quant_act(rstq_ctx* ctx, rstq_buf* a, rstq_buf* b, rstq_buf* sum,
                                                  rstq_buf* weight, rstq_buf* xq, rstq_buf* xs, rstq_buf* xsum,
                                                  int64_t rows, int64_t features, double eps, double gain_offset);
RSTQ_API int32_t rstq_silu_mul_quant_act(rstq_ctx* ctx, rstq_buf* gate, rstq_buf* up, rstq_buf* xq, rstq_buf* xs,
                                         rstq_buf* xsum, int64_t n);
RSTQ_API int32_t rstq_gelu_mul_quant_act(rstq_ctx* ctx, rstq_buf* gate, rstq_buf* up, rstq_buf* xq, rstq_buf* xs,
                                         rstq_buf* xsum, int64_t n);
RSTQ_API int32_t rstq_gqa_decode_attention(rstq_ctx* ctx, rstq_buf* q, rstq_buf* k, rstq_buf* v, rstq_buf* out,
                                           rstq_buf* clenbuf, int64_t cache_len, int64_t n_q, int64_t group,
                                           int64_t n_kv, int64_t head_dim, int64_t maxpos, double scale);

/* ---- tensor-parallel exchange of the sharded operator.  No counterpart in the reference: it
 *      extends the placement / plan vocabulary (src/raster/compiler/passes/placement.clj:21-89)
 *      with a weight split over the GPUs of one box.  One endpoint per rank.  Every rank owns a
 *      zero-filled "region" of rstq_tp_region_bytes() bytes that all ranks can address: peer
 *      access inside one process (rstq_tp_create_local sets that up), or a symmetric / IPC
 *      mapping between processes (rstq_tp_attach takes the addresses as this device sees them).
 *      The exchange is one kernel per rank over that memory (peer stores, a flag per rank,
 *      time-bounded waits: a rank that never arrives yields RSTQ_E_WAIT from rstq_sync, not a
 *      hang); all ranks must issue the same sequence of exchanges. ------------------------- */
typedef struct rstq_tp rstq_tp;
#define RSTQ_TP_MAX_RANKS 8
RSTQ_API int64_t rstq_tp_region_bytes(int32_t nranks, int64_t max_payload_bytes); /* 0 = bad arguments */
RSTQ_API int32_t rstq_tp_attach(rstq_ctx* ctx, void* const* regions, rstq_tp** tp, int32_t dev, int32_t rank,
                                int32_t nranks, int64_t region_bytes);
/* one process, nranks devices of ctx (devs = device indexes of the context): tps[nranks] */
RSTQ_API int32_t rstq_tp_create_local(rstq_ctx* ctx, const int32_t* devs, rstq_tp** tps, int32_t nranks,
                                      int64_t max_payload_bytes);
/* dst[row][rank][row_bytes] = src of rank `rank` [row][row_bytes]; row_bytes % 16 == 0 */
RSTQ_API int32_t rstq_tp_allgather(rstq_tp* tp, rstq_buf* src, rstq_buf* dst, int64_t rows,
                                   int64_t row_bytes);
/* dst[i] = sum over ranks (in rank order, the same on every rank) of src[i]; count % 4 == 0 */
RSTQ_API int32_t rstq_tp_allreduce_f32(rstq_tp* tp, rstq_buf* src, rstq_buf* dst, int64_t count);
/* The sharded operator: w is this rank's shard (rstq_weight_bind_shard).  Column split: x is
 * the full activation, y [M, nranks * w.out] f32 gathers every rank's columns.  Row split: x is
 * this rank's K slice [M, w.in], y [M, w.out] f32 is the sum of the partial products. */
RSTQ_API int32_t rstq_tp_qmatmul(rstq_tp* tp, rstq_weight* w, rstq_buf* x, rstq_buf* y, int64_t M,
                                 int32_t act_dtype, int32_t mode, int32_t split);
RSTQ_API int32_t rstq_tp_free(rstq_tp* tp);
/* One process per GPU: export the region (a buffer of rstq_alloc) as 64 opaque bytes, hand them
 * to the other processes of the box by any channel, and map theirs.  The mapped address goes
 * into the `regions` array of rstq_tp_attach. */
RSTQ_API int32_t rstq_ipc_export(rstq_buf* buf, void* handle64);
RSTQ_API int32_t rstq_ipc_open(rstq_ctx* ctx, const void* handle64, void** device_ptr, int32_t dev);
RSTQ_API int32_t rstq_ipc_close(rstq_ctx* ctx, void* device_ptr, int32_t dev);

#ifdef __cplusplus
}
#endif
#endif /* RSTQ_H */
