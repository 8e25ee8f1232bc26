/*
 * shrewq.h — C ABI of libshrewq, the B200 (sm_100a) implementation of Shrew's INT8
 * symmetric quantization path: quantize / dequantize of f32 weights and the forward of
 * a quantized Linear.
 *
 * The reference has no C ABI: its boundary is the Rust API of the facade crate's
 * `quantize` module (crates/shrew/src/quantize.rs; re-exported at
 * crates/shrew/src/lib.rs:120-124).  Each entry point below names the Rust item whose
 * work it performs on the device; a Rust shim binds them with `extern "C"` and keeps the
 * `Tensor<B>` / `Module::forward` surface unchanged.
 *
 * Conventions
 *  - Every function returns an int status (SHREWQ_OK == 0, negative on error), never
 *    throws or aborts.  `shrewq_last_error` returns the message of the last failure on
 *    the given context (or of the last failed create call on this thread when ctx is NULL).
 *  - Pointers named *_dev are device pointers owned by the caller, valid on the context's
 *    device; pointers named *_host are ordinary host memory.  The library allocates only
 *    its own workspaces, inside contexts and handles.  A workspace grows (synchronize + cudaMalloc)
 *    the first time a call needs more than it holds; a call that would have to grow one while its
 *    stream is being captured fails with SHREWQ_ERR_UNSUPPORTED instead of breaking the capture —
 *    make the same call once outside the capture first.
 *    A workspace that is outgrown is kept until the context is destroyed (a graph captured earlier still launches
 *    kernels with its address), so graphs stay valid when a later call needs a larger workspace.
 *  - Device entry points enqueue work on the context's stream and return without
 *    synchronising.  Host entry points (suffix _host) copy in, run, copy out and
 *    synchronise the stream before returning.
 *  - A context belongs to one host thread at a time: its stream, workspaces and error text are not
 *    locked.  A shrewq_linear is immutable after creation (a forward reads it and writes nothing to
 *    it) but is bound to the context it was created on, so threads that share a handle share that
 *    context and must serialise their calls.  The reference's `Module: Send + Sync` bound
 *    (distributed.rs:175-179) is met by a shim that keeps the context behind a mutex, or by one
 *    context and one set of handles per thread over the same device buffers (handles are cheap: a
 *    copy of the scales and two tensor maps).
 *  - There is no CPU fallback: without a CUDA device every compute call fails with
 *    SHREWQ_ERR_NO_DEVICE.
 */
#ifndef SHREWQ_H
#define SHREWQ_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define SHREWQ_API __attribute__((visibility("default")))
#else
#define SHREWQ_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------------------ */
#define SHREWQ_OK 0
#define SHREWQ_ERR_INVALID_ARG (-1) /* null pointer, bad enum, misaligned or mismatched shape */
#define SHREWQ_ERR_CUDA (-2)        /* a CUDA runtime / driver call failed                     */
#define SHREWQ_ERR_UNSUPPORTED (-3) /* valid request this build has no kernel for             */
#define SHREWQ_ERR_NO_DEVICE (-4)   /* no CUDA device / wrong architecture                    */
#define SHREWQ_ERR_TIMEOUT (-5)     /* a bounded device-side wait ran out (kernel gave up)    */
#define SHREWQ_ERR_ALLOC (-6)       /* out of device or host memory                           */

/* ---- enums (ints in the ABI) -------------------------------------------------------- */
/* QuantGranularity — quantize.rs:55-61 */
#define SHREWQ_PER_TENSOR 0
#define SHREWQ_PER_CHANNEL 1
/* element types of activations / outputs (shrew_core DType F32 and BF16) */
#define SHREWQ_F32 0
#define SHREWQ_BF16 1
/* storage types accepted only by shrewq_quantize_any / shrewq_dequantize_ex */
#define SHREWQ_F16 2
#define SHREWQ_F64 3
/* elementwise op fused after the bias add (the tensor op a caller applies next) */
/* QuantMode (quantize.rs:51-58) */
#define SHREWQ_SYMMETRIC 0
#define SHREWQ_ASYMMETRIC 1

#define SHREWQ_EPILOGUE_NONE 0
#define SHREWQ_EPILOGUE_RELU 1

typedef struct shrewq_ctx shrewq_ctx;
typedef struct shrewq_linear shrewq_linear;

/* ---- context ------------------------------------------------------------------------ */
/* Plays the role of the reference's `B::Device` (QuantizedLinear::device,
 * quantize.rs:389-390): which GPU, and here also which stream.  `stream` is a
 * cudaStream_t (NULL = the default stream). */
SHREWQ_API int shrewq_ctx_create(int device, void *stream, shrewq_ctx **out);
SHREWQ_API int shrewq_ctx_set_stream(shrewq_ctx *ctx, void *stream);
/* Launch options of a context (no counterpart in the reference); the defaults are the measured choices and
 * need no setting.  name / value:
 *   "tc_groups"    1..3   converter groups of the tensor-core kernel (default 3)
 *   "tc_splitk"    0/1    split K when the tile grid leaves SMs idle (default 1)
 *   "tc_tok"       0, 16, 32, 64, 128, 256   force the token tile (default 0 = choose)
 *   "tc_tok_gated" the same for gate/up launches only
 *   "tc_tailsplit" 0..2   a short last wave of tiles as a second launch split along K: 0 (default) = the CTA-pair
 *                         kernel does so for tails of up to a quarter wave, 1 = whenever a tail exists, 2 = never
 *   "tc_pair"      0..2   CTA pairs (tcgen05.mma.cta_group::2) for batches above 128 tokens: 0 never, 1 where
 *                         they win by measurement (default), 2 always
 *   "ring_stages"  0, 2, 3  stages of the ring kernel's shared-memory ring (default 0 = three while all its CTAs are
 *                         resident at once, two for larger grids)
 *   "pdl"          0/1    programmatic dependent launch of the forward kernels (default 1): from a handle's second
 *                         forward on, a forward kernel may start while the previous kernel of the stream still runs
 *                         and request its WEIGHTS; it reads activations and writes outputs, partial sums and
 *                         counters only after that kernel has completed (griddepcontrol.wait).  The first forward
 *                         of a handle is always fully ordered behind the stream, so weights quantized on the same
 *                         stream just before are complete; a caller that rewrites a handle's weights in place
 *                         LATER must set 0.  ("gemv_pdl" is accepted as an older name of the same option.)
 * Unknown names and values out of range return SHREWQ_ERR_INVALID_ARG. */
SHREWQ_API int shrewq_ctx_set_option(shrewq_ctx *ctx, const char *name, int value);
SHREWQ_API int shrewq_ctx_synchronize(shrewq_ctx *ctx);
SHREWQ_API void shrewq_ctx_destroy(shrewq_ctx *ctx);
SHREWQ_API const char *shrewq_last_error(const shrewq_ctx *ctx);
/* Library version and the architecture it was compiled for, e.g. "shrewq 0.1 sm_100a". */
SHREWQ_API const char *shrewq_version(void);

/* ---- quantize / dequantize ---------------------------------------------------------- */
/*
 * quantize_tensor for an F32 tensor — quantize.rs:194-205 (with quantize_per_tensor
 * :229-260, quantize_per_channel :270-318, compute_scale_zp :339-352).
 * rows = shape[0], cols = product(shape[1..]).  Writes rows*cols INT8 codes in the
 * source order and 1 (per-tensor) or `rows` (per-channel) f64 scales; zero points are
 * all 0.0 in symmetric mode and are not materialised.  Codes and scales are bit-exact
 * with the reference's f64 host arithmetic.
 */
SHREWQ_API int shrewq_quantize_f32(shrewq_ctx *ctx, const float *w_dev, size_t rows, size_t cols,
                        int granularity, int8_t *q_dev, double *scales_dev);
/*
 * quantize_named_parameters (quantize.rs:500-516: every parameter of rank >= 2, one after the other) as
 * ONE call for many F32 tensors: `items` is a HOST array of n_items descriptors with the arguments of
 * shrewq_quantize_f32; all tensors take the same granularity.  The tensors are covered by a few launches
 * in all (one per 64 tensors per-channel, three per-tensor) instead of one to three each, which is what
 * a model of many small matrices needs; results are the same bits as shrewq_quantize_f32 gives.  Tuned
 * for small tensors (a warp per row): tensors of many MB are better quantized one by one.  No device
 * memory is allocated beyond the context's scratch.
 */
typedef struct shrewq_quant_item {
    const float *w_dev;
    size_t rows, cols;
    int8_t *q_dev;
    double *scales_dev;
} shrewq_quant_item;
SHREWQ_API int shrewq_quantize_f32_batch(shrewq_ctx *ctx, const shrewq_quant_item *items, size_t n_items,
                              int granularity);
/* Same with host buffers: what `quantize_tensor(&tensor, &cfg)` does for a caller whose
 * tensor lives on the host (upload, quantize on the GPU, download codes and scales). */
SHREWQ_API int shrewq_quantize_f32_host(shrewq_ctx *ctx, const float *w_host, size_t rows, size_t cols,
                             int granularity, int8_t *q_host, double *scales_host);

/*
 * dequantize_tensor — quantize.rs:210-225 (dequantize_per_tensor :262-266,
 * dequantize_per_channel :320-335): out = narrow((q as f64 - 0.0) * scale) to
 * out_dtype (SHREWQ_F32 or SHREWQ_BF16), bit-exact with the reference.
 */
SHREWQ_API int shrewq_dequantize(shrewq_ctx *ctx, const int8_t *q_dev, const double *scales_dev,
                      size_t rows, size_t cols, int granularity, int out_dtype, void *out_dev);

/*
 * Per-tensor quantization of a ROW SHARD of a tensor that is split over several GPUs.  The one
 * per-tensor scale is amax / 127 of the WHOLE tensor (quantize.rs:349-351), so: every rank calls
 * shrewq_absmax_f32 on its shard (max |w|, NaN ignored, +0.0 for n = 0, written as one f32), the
 * ranks reduce those with MAX (one float through ncclAllReduce / torch.distributed, the caller's
 * job), then every rank calls shrewq_quantize_f32_given_amax with the reduced value.  Codes and
 * scale are then bit-identical to quantizing the unsplit tensor.  Per-channel shards need none of
 * this: shrewq_quantize_f32 on the shard is already identical.  No counterpart in the reference
 * (which is single-device).
 */
SHREWQ_API int shrewq_absmax_f32(shrewq_ctx *ctx, const float *w_dev, size_t n, float *amax_dev);
SHREWQ_API int shrewq_quantize_f32_given_amax(shrewq_ctx *ctx, const float *w_dev, size_t n,
                                   const float *amax_dev, int8_t *q_dev, double *scale_dev);

/*
 * The same two calls for every mode of QuantConfig (quantize.rs:64-139): bits = 8 or 4 (INT4
 * codes are stored one per byte, as the reference's Vec<i8> does, within [-8, 7]), mode =
 * SHREWQ_SYMMETRIC or SHREWQ_ASYMMETRIC (compute_scale_zp, :353-364: scale from max - min, zero
 * point round(qmin - min / scale)).  zero_points_dev receives 1 or `rows` f64 values (0.0 in
 * symmetric mode).  bits = 8 with SHREWQ_SYMMETRIC runs the kernels of shrewq_quantize_f32; the other
 * modes replay the reference's f64 operations one for one (correct first, not tuned).
 * shrewq_dequantize_ex with zero_points_dev = NULL is shrewq_dequantize.
 */
SHREWQ_API int shrewq_quantize_f32_ex(shrewq_ctx *ctx, const float *w_dev, size_t rows, size_t cols,
                           int granularity, int bits, int mode, int8_t *q_dev, double *scales_dev,
                           double *zero_points_dev);
/* quantize_tensor for a tensor of any float storage type (quantize.rs:194-205 widens every dtype with
 * to_f64_vec): w_dtype = SHREWQ_F32, SHREWQ_BF16, SHREWQ_F16 or SHREWQ_F64, any bits / mode.  All
 * arithmetic in f64 as in the reference (f32 INT8 symmetric input should use shrewq_quantize_f32, the
 * tuned path).  shrewq_dequantize_ex likewise narrows to any of the
 * four types when given SHREWQ_F16 / SHREWQ_F64 (dequantize_tensor, quantize.rs:210-225). */
SHREWQ_API int shrewq_quantize_any(shrewq_ctx *ctx, const void *w_dev, int w_dtype, size_t rows, size_t cols,
                        int granularity, int bits, int mode, int8_t *q_dev, double *scales_dev,
                        double *zero_points_dev);
SHREWQ_API int shrewq_dequantize_ex(shrewq_ctx *ctx, const int8_t *q_dev, const double *scales_dev,
                         const double *zero_points_dev, size_t rows, size_t cols, int granularity,
                         int out_dtype, void *out_dev);

/* ---- quantized Linear --------------------------------------------------------------- */
/*
 * QuantizedLinear::new — quantize.rs:437-447 (from_linear, :413-434, is
 * shrewq_quantize_f32 followed by this).  q_dev is [out_features, in_features] row-major,
 * scales_dev holds 1 or out_features f64 values, bias_dev is NULL or out_features f32
 * values (the reference's [1,out] bias, kept in float: quantize.rs:387-388).
 * The handle keeps the caller's q_dev and bias_dev pointers (they must outlive it) and
 * owns a small f32 copy of the scales.
 * A row shard of a larger layer is simply a Linear over rows [n0,n1): pass the shard's
 * pointers and out_features = n1-n0.
 */
SHREWQ_API int shrewq_linear_create(shrewq_ctx *ctx, const int8_t *q_dev, const double *scales_dev,
                         const float *bias_dev, size_t out_features, size_t in_features,
                         int granularity, shrewq_linear **out);
/* QuantizedLinear::new for a weight quantized with zero points (asymmetric mode): the forward
 * computes scale * sum(q x) + bias - (scale * zero_point) * sum(x), which equals the reference's
 * x . dequant(W)^T + bias up to f32 rounding.  zero_points_dev = NULL is shrewq_linear_create.
 * Such a handle is not accepted by the gate/up, peer-destination and no-allocation forwards. */
SHREWQ_API int shrewq_linear_create_ex(shrewq_ctx *ctx, const int8_t *q_dev, const double *scales_dev,
                            const double *zero_points_dev, const float *bias_dev, size_t out_features,
                            size_t in_features, int granularity, shrewq_linear **out);
/*
 * INT4 codes two per byte, beyond the reference (whose INT4 tensors keep one code per i8 and only
 * report the packed size, quantize.rs:176): shrewq_pack_int4 turns rows*cols INT4 codes (from
 * shrewq_quantize_f32_ex with bits = 4, values in [-8, 7]) into rows*cols/2 bytes, byte j of a row =
 * code 2j + 8 in the low and code 2j+1 + 8 in the high nibble; shrewq_linear_create_int4 builds a
 * QuantizedLinear over such rows (symmetric scales).  Its forward streams half the bytes of INT8; it
 * is served by the warp-MMA kernel only: bf16 activations, M <= 32, in_features a multiple of 128.
 */
SHREWQ_API int shrewq_pack_int4(shrewq_ctx *ctx, const int8_t *q_dev, size_t rows, size_t cols, uint8_t *packed_dev);
SHREWQ_API int shrewq_linear_create_int4(shrewq_ctx *ctx, const uint8_t *packed_dev, const double *scales_dev,
                              const float *bias_dev, size_t out_features, size_t in_features,
                              int granularity, shrewq_linear **out);
SHREWQ_API void shrewq_linear_destroy(shrewq_linear *lin);

/*
 * <QuantizedLinear as Module>::forward — quantize.rs:463-476:
 *   y[m, n] = sum_k x[m,k] * dequant(W)[n,k] + bias[n],   then the optional epilogue.
 * x_dev is [M, in_features] row-major of x_dtype; y_dev has M rows of out_features
 * values of y_dtype with a row stride of ldy elements (ldy >= out_features; pass
 * out_features for a dense output, or the full layer width when a shard writes its
 * column slice of a wider buffer).  The weight is never expanded in memory: the INT8
 * codes are streamed and the per-channel scale is applied to the f32 accumulator.
 * Accumulation is f32; with bf16 activations products are exact bf16 x int8 products.
 */
SHREWQ_API int shrewq_linear_forward(shrewq_linear *lin, const void *x_dev, int x_dtype, size_t M,
                          void *y_dev, int y_dtype, size_t ldy, int epilogue);
/* Same with host activations and host output (dense, ldy = out_features): the call a
 * host-tensor caller of `qlinear.forward(&x)` makes. */
SHREWQ_API int shrewq_linear_forward_host(shrewq_linear *lin, const void *x_host, int x_dtype, size_t M,
                               void *y_host, int y_dtype, int epilogue);

/*
 * The same forward for callers that must not allocate device memory.  (No counterpart in
 * the reference.)  Who that is: a serving process that reserved all of HBM for its own
 * pools at start-up, so any later cudaMalloc simply fails; a latency-critical loop that
 * cannot afford the device-wide synchronisation a cudaMalloc / cudaFree implies; a host
 * that runs under an allocator it must account every byte to.  shrewq_linear_forward may
 * grow the context's scratch buffer (cudaMalloc) the first time a small batch makes it
 * split the K dimension; this entry point instead keeps the split-K partial sums in a
 * 4 MiB array that is part of the library image, and calls no cudaMalloc, cudaFree or
 * allocating library routine.
 *  - bf16 activations only (x_dev is [M, in_features] bf16), tensor-core kernel only; the
 *    same requirements as that kernel: in_features a multiple of 16, 16-byte aligned x_dev
 *    and weights.  Anything else returns SHREWQ_ERR_UNSUPPORTED.
 *  - Limit: a shape whose split-K scratch (4096 B + tiles * splits * TOK * 128 * 4 B, with
 *    TOK the token tile of 16, 32 or 64) exceeds 4 MiB is refused with
 *    SHREWQ_ERR_UNSUPPORTED and a message giving both sizes.  This entry point splits K for
 *    token tiles of up to 64 tokens only (with the default options: batches above 64 tokens
 *    are not split and do not touch the array; option "tc_tok" can force a small tile for a
 *    larger batch, which the size check then covers like any other shape).
 *  - Every GPU that loads the library holds the 4 MiB until the process exits.
 *  - The first call on each device looks up the array's device address (a host-side
 *    query, done once and cached; safe from several threads) and, like the first use of any
 *    kernel, may make the CUDA runtime load the library's device code, which can allocate:
 *    make that first call at start-up, before memory is tight and before any stream capture.
 *  - All calls on a device share the one array, which keeps the previous call's contents
 *    (the tile counters are cleared at the start of every call).  Two calls that overlap
 *    on the GPU — different streams, or different contexts on one device — race on it;
 *    keep them on one stream or order them yourself.
 * Results are identical to shrewq_linear_forward on the same inputs.
 */
SHREWQ_API int shrewq_linear_forward_noalloc(shrewq_linear *lin, const void *x_dev, size_t M, void *y_dev,
                                             int y_dtype, size_t ldy, int epilogue);

/*
 * Two forwards sharing one activation read, for a gated MLP block:
 *   h[m,n] = silu(gate.forward(x)[m,n]) * up.forward(x)[m,n]
 * (the reference composes this from two QuantizedLinear::forward calls and the tensor ops
 * silu and mul).  gate and up must have identical shapes and the same context.
 */
SHREWQ_API int shrewq_linear_forward_gate_up_silu(shrewq_linear *gate, shrewq_linear *up, const void *x_dev,
                                       int x_dtype, size_t M, void *h_dev, int h_dtype, size_t ldh);

/*
 * The gated MLP block for a caller whose activations live in HOST memory: y = down( silu(gate(x)) * up(x) ), i.e.
 * three <QuantizedLinear as Module>::forward calls (quantize.rs:463-476) with the tensor ops silu and mul between
 * them, as a Llama-style block composes them.  x_host is [M, in_features] bf16, y_host [M, down.out_features] of
 * y_dtype; the hidden activation stays on the device.  The call copies x in, runs the two kernels on the context's
 * stream and copies y out, using two staging slots and two internal copy streams: with synchronize = 0 it returns as
 * soon as the work is enqueued, and the copies of one call overlap the kernels of the next.  The caller then keeps
 * x_host and y_host untouched (pinned memory, a y_host of its own per call in flight) until shrewq_ctx_synchronize,
 * which also waits for the results of such calls.  With synchronize = 1 the result is in y_host on return.
 */
SHREWQ_API int shrewq_mlp_forward_host(shrewq_linear *gate, shrewq_linear *up, shrewq_linear *down, const void *x_host,
                                       size_t M, void *y_host, int y_dtype, int synchronize);

/*
 * Forward of a row shard with the all-gather fused into the epilogue (no counterpart in the
 * reference, whose `distributed.rs` is single-process).  The slice y[:, n0:n1] this shard
 * computes is stored into y_dev and, with the same element offsets, into each of the
 * n_peers (<= 7) buffers peer_y_dev[i]: the other GPUs' copies of the full [M, N] output,
 * mapped into this process (CUDA peer access / IPC / symmetric memory), each pointer already
 * advanced to column n0.  Plain stores over NVLink; the caller synchronises the GPUs
 * afterwards (a cross-device barrier) before anyone reads.  `up` != NULL selects the gated
 * form silu(lin(x)) * up(x) (epilogue is then ignored).  Only the gemv and tcgen05 kernels
 * take peer destinations.
 */
SHREWQ_API int shrewq_linear_forward_peers(shrewq_linear *lin, shrewq_linear *up, const void *x_dev, int x_dtype,
                                           size_t M, void *y_dev, void *const *peer_y_dev, int n_peers, int y_dtype,
                                           size_t ldy, int epilogue);

/*
 * Barrier between the GPUs of a sharded layer, on the device (no counterpart in the reference:
 * DataParallel::forward, distributed.rs:188-201, is a sequential loop in one process).
 * shrewq_linear_forward_peers writes into other GPUs' buffers; before a rank reads its copy of the
 * output every rank's stores must have landed, and before a rank overwrites a peer's copy again that
 * peer must be done with it.  shrewq_exchange_barrier enqueues one small kernel on the context's
 * stream: it tells every peer "all work enqueued on my stream before this point is complete and
 * visible" and waits until every peer has said the same.
 *
 * flag_blocks_dev[r] (r < world <= 8) is rank r's flag block as mapped into THIS process
 * (flag_blocks_dev[rank] is this GPU's own memory): SHREWQ_EXCHANGE_FLAG_BYTES bytes each, 4-byte
 * aligned, zeroed once by its owner before any rank's first barrier (with a host-side barrier between
 * the zeroing and the first use).  Every rank must enqueue the same sequence of barriers.  The barrier
 * count lives in device memory, so a barrier captured in a CUDA graph stays correct when replayed.
 *
 * The wait is bounded (about a second): a rank whose peer never arrives gives up, the kernel ends and
 * the next shrewq_ctx_synchronize returns SHREWQ_ERR_TIMEOUT naming the missing rank.  After a timeout
 * the ranks' counts no longer agree: zero the flag blocks (all ranks, host barrier) and create a new
 * exchange before using the buffers again.
 */
#define SHREWQ_EXCHANGE_FLAG_BYTES 256
typedef struct shrewq_exchange shrewq_exchange;
SHREWQ_API int shrewq_exchange_create(shrewq_ctx *ctx, int rank, int world, void *const *flag_blocks_dev,
                                      shrewq_exchange **out);
SHREWQ_API int shrewq_exchange_barrier(shrewq_exchange *ex);
SHREWQ_API void shrewq_exchange_destroy(shrewq_exchange *ex);

/* Accessors mirroring QuantizedLinear's public fields / methods (quantize.rs:392-394,
 * :455-459). */
SHREWQ_API size_t shrewq_linear_in_features(const shrewq_linear *lin);
SHREWQ_API size_t shrewq_linear_out_features(const shrewq_linear *lin);
SHREWQ_API size_t shrewq_linear_memory_savings_bytes(const shrewq_linear *lin);

/* Name of the kernel family the calling thread's latest forward dispatched to ("gemv", "mma", "mma-ring",
 * "tcgen05", "tcgen05-2cta", "tcgen05-f32", "simt", "mma-w4"); for tests and benchmarks.  Kept per thread, not
 * in the handle: the one thing a forward writes to the handle it reads is an atomic flag saying that a
 * forward has been enqueued. */
SHREWQ_API const char *shrewq_linear_last_kernel(const shrewq_linear *lin);
/* Forces the kernel family used by forwards issued from the calling thread: "gemv" (CUDA cores, M <= 16; up to 128 in
 * slices of 16 tokens),
 * "mma" (warp-level MMA, weights streamed through registers, M <= 64), "mma-ring" (warp-level MMA, weights
 * streamed through a shared-memory ring by bulk copies, M <= 32), "tcgen05" (single-CTA tensor-core kernel), "tcgen05-2cta" (CTA pairs,
 * tcgen05.mma.cta_group::2), "tcgen05-f32" (f32 activations as a bf16 hi/lo pair on the tensor cores),
 * "simt" (general f32 kernel), or "auto"/NULL to restore the built-in choice.  A forced kernel that
 * cannot take a shape makes the forward fail with SHREWQ_ERR_UNSUPPORTED (it never falls
 * back silently).  For tests and benchmarks; no counterpart in the reference. */
SHREWQ_API int shrewq_force_kernel(const char *name);
/* Which kernel family and launch plan a forward of this shape would get on a GPU with `sm_count` SMs
 * (16-byte aligned buffers, no forced kernel): writes the family name into `kernel` (at least 16 bytes)
 * and, for "tcgen05", the token tile, the tile grid, the K splits and the pipeline rounds per split
 * (zeros otherwise).  Pure host arithmetic: needs no GPU and no context.  For tests, benchmarks and
 * capacity planning; no counterpart in the reference. */
SHREWQ_API int shrewq_plan_forward(size_t M, size_t N, size_t K, int x_is_bf16, int gated, int sm_count, char *kernel,
                        size_t kernel_len, int *tok, int *n_tiles, int *m_tiles, int *splits,
                        int *rounds_per_split);
/* Number of kernels this context has launched since creation (for benchmark accounting). */
SHREWQ_API uint64_t shrewq_ctx_launch_count(const shrewq_ctx *ctx);

#ifdef __cplusplus
}
#endif
#endif /* SHREWQ_H */
