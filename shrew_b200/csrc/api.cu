// C ABI of libshrewq: contexts, argument validation, kernel dispatch, host-buffer
// entry points.  See include/shrewq.h for the contract of each function.
#include <new>

#include "common.cuh"

namespace shrewq {

static thread_local char g_create_err[kErrLen] = {0};

int set_err(shrewq_ctx *ctx, int code, const char *fmt, ...) {
    char *dst = ctx ? ctx->err : g_create_err;
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(dst, kErrLen, fmt, ap);
    va_end(ap);
    return code;
}

static int grow(shrewq_ctx *ctx, void **p, size_t *have, size_t want, bool pinned) {
    if (*have >= want) return SHREWQ_OK;
    // Growing means a synchronize and an allocation, neither of which a stream capture survives: say so
    // instead of invalidating the caller's capture (one call of the same shape outside the capture sizes
    // the buffer for good).
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(ctx->stream, &cap) != cudaSuccess) cudaGetLastError();
    else if (cap != cudaStreamCaptureStatusNone)
        return set_err(ctx, SHREWQ_ERR_UNSUPPORTED,
                       "this call needs %zu bytes of library workspace (have %zu) and cannot allocate while its stream is "
                       "being captured: make the same call once outside the capture first", want, *have);
    // Work already enqueued, and graphs captured earlier, may still use the old buffer: it is retired, not freed
    // (sizes grow geometrically, so the retired buffers together stay below the live one).
    if (*p) {
        ctx->retired.emplace_back(*p, pinned);
        *p = nullptr;
        *have = 0;
    }
    size_t sz = want + want / 2 + 4096;
    cudaError_t e = pinned ? cudaMallocHost(p, sz) : cudaMalloc(p, sz);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return set_err(ctx, SHREWQ_ERR_ALLOC, "allocation of %zu bytes failed: %s", sz, cudaGetErrorString(e));
    }
    *have = sz;
    return SHREWQ_OK;
}

int ensure_scratch(shrewq_ctx *ctx, size_t bytes) {
    const void *before = ctx->scratch;
    // never smaller than the fixed head (quantizer words + split-K tile counters)
    int rc = grow(ctx, &ctx->scratch, &ctx->scratch_bytes, bytes < 8192 ? 8192 : bytes, false);
    if (ctx->scratch != before) ctx->counters_zeroed = false;  // new memory: counters are garbage
    return rc;
}

int ensure_xsplit(shrewq_ctx *ctx, size_t bytes) { return grow(ctx, &ctx->xsplit, &ctx->xsplit_bytes, bytes, false); }

int ensure_stage(shrewq_ctx *ctx, size_t dev_bytes, size_t pinned_bytes) {
    int rc = grow(ctx, &ctx->stage_dev, &ctx->stage_dev_bytes, dev_bytes, false);
    if (rc != SHREWQ_OK) return rc;
    if (pinned_bytes) rc = grow(ctx, &ctx->stage_pinned, &ctx->stage_pinned_bytes, pinned_bytes, true);
    return rc;
}

static int bind(shrewq_ctx *ctx) {
    SHREWQ_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    return SHREWQ_OK;
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

enum ForcedKernel { kAuto = 0, kForceGemv, kForceTc, kForceSimt, kForceMma, kForceTcF32, kForceTc2Cta, kForceRing };

}  // namespace shrewq

using namespace shrewq;

// kernel family forced by shrewq_force_kernel for this thread (tests and benchmarks)
static thread_local int g_forced_kernel = kAuto;
// kernel family of this thread's latest forward (shrewq_linear_last_kernel): per thread, so that
// forwards issued from several threads on handles they share do not write to the handle
static thread_local const char *g_last_kernel = "none";

extern "C" {

const char *shrewq_version(void) { return "shrewq 0.1 sm_100a"; }

int shrewq_ctx_create(int device, void *stream, shrewq_ctx **out) {
    if (!out) return set_err(nullptr, SHREWQ_ERR_INVALID_ARG, "ctx_create: out is NULL");
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        cudaGetLastError();
        return set_err(nullptr, SHREWQ_ERR_NO_DEVICE, "no CUDA device available (%s); this library has no CPU path",
                       e != cudaSuccess ? cudaGetErrorString(e) : "device count is 0");
    }
    if (device < 0 || device >= count)
        return set_err(nullptr, SHREWQ_ERR_INVALID_ARG, "ctx_create: device %d out of range [0,%d)", device, count);
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess)
        return set_err(nullptr, SHREWQ_ERR_CUDA, "cudaGetDeviceProperties failed");
    if (prop.major != 10)
        return set_err(nullptr, SHREWQ_ERR_NO_DEVICE, "device %d is sm_%d%d; this library is built for sm_100a only",
                       device, prop.major, prop.minor);
    shrewq_ctx *ctx = new (std::nothrow) shrewq_ctx();
    if (!ctx) return set_err(nullptr, SHREWQ_ERR_ALLOC, "out of host memory");
    ctx->device = device;
    ctx->stream = static_cast<cudaStream_t>(stream);
    ctx->sm_count = prop.multiProcessorCount;
    if (cudaSetDevice(device) != cudaSuccess || cudaMalloc(&ctx->dev_status, sizeof(DeviceStatus)) != cudaSuccess ||
        cudaMemset(ctx->dev_status, 0, sizeof(DeviceStatus)) != cudaSuccess) {
        int rc = set_err(nullptr, SHREWQ_ERR_CUDA, "ctx_create: device setup failed: %s",
                         cudaGetErrorString(cudaGetLastError()));
        delete ctx;
        return rc;
    }
    *out = ctx;
    return SHREWQ_OK;
}

int shrewq_ctx_set_stream(shrewq_ctx *ctx, void *stream) {
    if (!ctx) return set_err(nullptr, SHREWQ_ERR_INVALID_ARG, "set_stream: ctx is NULL");
    ctx->stream = static_cast<cudaStream_t>(stream);
    return SHREWQ_OK;
}

int shrewq_ctx_set_option(shrewq_ctx *ctx, const char *name, int value) {
    if (!ctx) return set_err(nullptr, SHREWQ_ERR_INVALID_ARG, "set_option: ctx is NULL");
    if (!name) return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "set_option: name is NULL");
    Tuning &t = ctx->tuning;
    if (!strcmp(name, "tc_groups")) {
        if (value < 1 || value > 3) return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "set_option: tc_groups is 1, 2 or 3");
        t.tc_groups = value;
    } else if (!strcmp(name, "tc_splitk")) t.tc_splitk = value != 0;
    else if (!strcmp(name, "tc_tok") || !strcmp(name, "tc_tok_gated")) {
        if (value != 0 && value != 16 && value != 32 && value != 64 && value != 128 && value != 256)
            return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "set_option: %s is 0 (choose), 16, 32, 64, 128 or 256", name);
        (name[6] == '_' ? t.tc_tok_gated : t.tc_tok) = value;
    } else if (!strcmp(name, "tc_tailsplit")) t.tc_tailsplit = value >= 0 && value <= 2 ? value : 0;
    else if (!strcmp(name, "tc_pair")) {
        if (value < 0 || value > 2) return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "set_option: tc_pair is 0 (never), 1 (where pairs win) or 2 (always above 128 tokens)");
        t.tc_pair = value;
    }
    else if (!strcmp(name, "pdl") || !strcmp(name, "gemv_pdl")) t.pdl = value != 0;
    else if (!strcmp(name, "ring_stages")) t.ring_stages = value == 2 || value == 3 ? value : 0;
    else return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "set_option: unknown option '%s'", name);
    return SHREWQ_OK;
}

int shrewq_ctx_synchronize(shrewq_ctx *ctx) {
    if (!ctx) return set_err(nullptr, SHREWQ_ERR_INVALID_ARG, "synchronize: ctx is NULL");
    int rc = bind(ctx);
    if (rc != SHREWQ_OK) return rc;
    SHREWQ_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    if (ctx->copy_out) SHREWQ_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->copy_out));  // results of *_host calls in flight
    DeviceStatus st;
    SHREWQ_CUDA_TRY(ctx, cudaMemcpy(&st, ctx->dev_status, sizeof(st), cudaMemcpyDeviceToHost));
    if (st.timeout_flag) {
        cudaMemset(ctx->dev_status, 0, sizeof(DeviceStatus));
        return set_err(ctx, SHREWQ_ERR_TIMEOUT,
                       "a kernel gave up a bounded wait: block %u role %u stage %u parity %u (results are invalid)",
                       st.where >> 8, st.where & 0xFF, st.stage, st.parity);
    }
    return SHREWQ_OK;
}

void shrewq_ctx_destroy(shrewq_ctx *ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->scratch) cudaFree(ctx->scratch);
    if (ctx->stage_dev) cudaFree(ctx->stage_dev);
    if (ctx->xsplit) cudaFree(ctx->xsplit);
    if (ctx->ytmp) cudaFree(ctx->ytmp);
    if (ctx->stage_pinned) cudaFreeHost(ctx->stage_pinned);
    if (ctx->mlp_stage) cudaFree(ctx->mlp_stage);
    for (auto &r : ctx->retired) {
        if (r.second) cudaFreeHost(r.first); else cudaFree(r.first);
    }
    for (int i = 0; i < 2; ++i) {
        if (ctx->ev_in[i]) cudaEventDestroy(ctx->ev_in[i]);
        if (ctx->ev_cmp[i]) cudaEventDestroy(ctx->ev_cmp[i]);
        if (ctx->ev_out[i]) cudaEventDestroy(ctx->ev_out[i]);
    }
    if (ctx->copy_in) cudaStreamDestroy(ctx->copy_in);
    if (ctx->copy_out) cudaStreamDestroy(ctx->copy_out);
    if (ctx->dev_status) cudaFree(ctx->dev_status);
    delete ctx;
}

const char *shrewq_last_error(const shrewq_ctx *ctx) { return ctx ? ctx->err : g_create_err; }

uint64_t shrewq_ctx_launch_count(const shrewq_ctx *ctx) { return ctx ? ctx->launches.load() : 0; }

// The default kernel family of a forward with bf16 activations: the one rule, shared by forward_impl and
// shrewq_plan_forward.  Measured on 4096 x 4096, 11008 x 4096, 4096 x 11008, 1376 x 4096 and 32000 x 4096: the
// CUDA-core GEMV wins up to 2 tokens, a warp-MMA kernel from 3 to 32, the tcgen05 kernel above.  Of the two warp-MMA
// kernels the ring kernel (bulk copies into shared memory) wins up to 16 tokens on grids of up to five CTAs per SM
// (three stages while all CTAs are resident at once, two stages beyond: see launch_ring_one), the register-streaming
// one on larger grids (32000 x 4096: 37 against 41 us) and above 16 tokens.
// f32 activations on SMALL layers (config 1: 784 -> 256 -> 10 at 64 tokens): the whole forward is a few MFLOP and
// what counts is the number and latency of launches; the CUDA-core GEMV in slices of 16 tokens is one short launch
// where the tensor-core route is a split pass plus a pipelined kernel that never fills.
constexpr size_t kGemvSlicedMaxTokens = 128;
static bool gemv_slices_win(size_t M, size_t N, size_t K) {
    return M > 16 && M <= kGemvSlicedMaxTokens && M * N * K <= ((size_t)1 << 26);
}
static bool ring_kernel_wins(size_t M, size_t N, bool gated, int sm_count) {
    const size_t ctas = (N + (gated ? 7 : 15)) / (gated ? 8 : 16);
    return M >= 3 && M <= 16 && ctas <= (size_t)5 * sm_count;
}
static int default_family(size_t M, size_t N, bool gated, int sm_count, bool gemv_ok, bool mma_ok, bool tc_ok) {
    if (gemv_ok && (M <= 2 || (!mma_ok && (M <= 4 || !tc_ok)))) return kForceGemv;
    if (mma_ok && M <= 32) return ring_kernel_wins(M, N, gated, sm_count) ? kForceRing : kForceMma;
    return tc_ok ? kForceTc : (gemv_ok ? kForceGemv : kForceSimt);
}

// CTA pairs against the single-CTA kernel, from measurements on 148 SMs (Llama-MLP block and 4096 x 4096 layers,
// batches 256..4096): a pair tile is 256 channels (128 gated) x 256 tokens and does twice the work per issued MMA,
// but a grid that leaves many SMs idle, or needs a deep K split to fill them, is better served by the smaller
// tiles of the single-CTA kernel.  Pairs win from one full wave of pair tiles (64) up, and from a quarter of a wave
// when the reduction is long enough (K >= 8192) for a K split to keep every pair busy (16 pair tiles, K = 11008:
// 33.4 against 36.5 us; 8 pair tiles: 37 against 27 us).
static bool pair_kernel_wins(size_t M, size_t N, size_t K, bool gated) {
    const size_t pair_tiles = ((N + (gated ? 127 : 255)) / (gated ? 128 : 256)) * ((M + 255) / 256);
    return pair_tiles >= 64 || (pair_tiles >= 16 && K >= 8192);
}

int shrewq_plan_forward(size_t M, size_t N, size_t K, int x_is_bf16, int gated, int sm_count, char *kernel, size_t kernel_len,
                        int *tok, int *n_tiles, int *m_tiles, int *splits, int *rounds_per_split) {
    if (!kernel || kernel_len < 16 || !tok || !n_tiles || !m_tiles || !splits || !rounds_per_split || sm_count < 1 || N == 0 ||
        K == 0)
        return set_err(nullptr, SHREWQ_ERR_INVALID_ARG, "plan_forward: bad argument");
    *tok = *n_tiles = *m_tiles = *splits = *rounds_per_split = 0;
    // the rule of forward_impl for aligned buffers and no forced kernel
    const bool vec16 = (K % 16) == 0;
    const bool small = M < (1u << 31) && N < (1u << 31) && K < (1u << 31);
    const bool tc_ok = x_is_bf16 && vec16 && M >= 1 && small;
    const bool mma_ok = x_is_bf16 && (K % 64) == 0 && M <= 64 && small;
    int fam = default_family(M, N, gated != 0, sm_count, vec16 && M <= 16, mma_ok, tc_ok);
    if (!x_is_bf16 && vec16 && small && M > 16 && !gated) fam = kForceTcF32;   // f32 activations: the hi/lo tensor-core pass
    if (!x_is_bf16 && vec16 && small && gemv_slices_win(M, N, K)) fam = kForceGemv;
    if (fam == kForceTc && M > 128 && pair_kernel_wins(M, N, K, gated != 0)) fam = kForceTc2Cta;
    const char *name = fam == kForceGemv ? "gemv" : fam == kForceMma ? "mma" : fam == kForceRing ? "mma-ring" : fam == kForceTc ? "tcgen05"
                       : fam == kForceTc2Cta ? "tcgen05-2cta" : fam == kForceTcF32 ? "tcgen05-f32" : "simt";
    snprintf(kernel, kernel_len, "%s", name);
    if (!strcmp(name, "tcgen05"))
        return plan_gemm_tcgen05(M, N, K, gated != 0, sm_count, tok, n_tiles, m_tiles, splits, rounds_per_split);
    return SHREWQ_OK;
}

int shrewq_force_kernel(const char *name) {
    if (!name || !*name || !strcmp(name, "auto")) g_forced_kernel = kAuto;
    else if (!strcmp(name, "gemv")) g_forced_kernel = kForceGemv;
    else if (!strcmp(name, "tcgen05")) g_forced_kernel = kForceTc;
    else if (!strcmp(name, "simt")) g_forced_kernel = kForceSimt;
    else if (!strcmp(name, "mma")) g_forced_kernel = kForceMma;
    else if (!strcmp(name, "mma-ring")) g_forced_kernel = kForceRing;
    else if (!strcmp(name, "tcgen05-f32")) g_forced_kernel = kForceTcF32;
    else if (!strcmp(name, "tcgen05-2cta")) g_forced_kernel = kForceTc2Cta;
    else return set_err(nullptr, SHREWQ_ERR_INVALID_ARG, "force_kernel: unknown kernel '%s'", name);
    return SHREWQ_OK;
}

// ---- quantize / dequantize --------------------------------------------------------------
static int check_gran(shrewq_ctx *ctx, int g, const char *who) {
    if (g != SHREWQ_PER_TENSOR && g != SHREWQ_PER_CHANNEL)
        return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "%s: granularity must be SHREWQ_PER_TENSOR or SHREWQ_PER_CHANNEL", who);
    return SHREWQ_OK;
}

int shrewq_quantize_f32(shrewq_ctx *ctx, const float *w_dev, size_t rows, size_t cols, int granularity,
                        int8_t *q_dev, double *scales_dev) {
    if (!ctx) return set_err(nullptr, SHREWQ_ERR_INVALID_ARG, "quantize: ctx is NULL");
    int rc = check_gran(ctx, granularity, "quantize");
    if (rc != SHREWQ_OK) return rc;
    const size_t n = rows * cols;
    if (cols != 0 && n / cols != rows) return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "quantize: rows*cols overflows");
    if (!scales_dev && (granularity == SHREWQ_PER_TENSOR || rows > 0))
        return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "quantize: scales_dev is NULL");
    if (n > 0 && (!w_dev || !q_dev)) return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "quantize: w_dev / q_dev is NULL");
    if ((reinterpret_cast<uintptr_t>(w_dev) & 3) || (reinterpret_cast<uintptr_t>(scales_dev) & 7))
        return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "quantize: w_dev must be 4-byte and scales_dev 8-byte aligned");
    if ((rc = bind(ctx)) != SHREWQ_OK) return rc;
    return launch_quantize(ctx, w_dev, rows, cols, granularity, q_dev, scales_dev);
}

int shrewq_quantize_f32_batch(shrewq_ctx *ctx, const shrewq_quant_item *items, size_t n_items, int granularity) {
    if (!ctx) return set_err(nullptr, SHREWQ_ERR_INVALID_ARG, "quantize_batch: ctx is NULL");
    int rc = check_gran(ctx, granularity, "quantize_batch");
    if (rc != SHREWQ_OK) return rc;
    if (n_items == 0) return SHREWQ_OK;
    if (!items) return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "quantize_batch: items is NULL");
    for (size_t i = 0; i < n_items; ++i) {
        const shrewq_quant_item &t = items[i];
        const size_t n = t.rows * t.cols;
        if (t.cols != 0 && n / t.cols != t.rows)
            return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "quantize_batch: item %zu: rows*cols overflows", i);
        if (!t.scales_dev && (granularity == SHREWQ_PER_TENSOR || t.rows > 0))
            return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "quantize_batch: item %zu: scales_dev is NULL", i);
        if (n > 0 && (!t.w_dev || !t.q_dev))
            return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "quantize_batch: item %zu: w_dev / q_dev is NULL", i);
        if ((reinterpret_cast<uintptr_t>(t.w_dev) & 3) || (reinterpret_cast<uintptr_t>(t.scales_dev) & 7))
            return set_err(ctx, SHREWQ_ERR_INVALID_ARG,
                           "quantize_batch: item %zu: w_dev must be 4-byte and scales_dev 8-byte aligned", i);
    }
    if ((rc = bind(ctx)) != SHREWQ_OK) return rc;
    return launch_quantize_batch(ctx, items, n_items, granularity);
}

int shrewq_quantize_f32_host(shrewq_ctx *ctx, const float *w_host, size_t rows, size_t cols, int granularity,
                             int8_t *q_host, double *scales_host) {
    if (!ctx) return set_err(nullptr, SHREWQ_ERR_INVALID_ARG, "quantize_host: ctx is NULL");
    int rc = check_gran(ctx, granularity, "quantize_host");
    if (rc != SHREWQ_OK) return rc;
    const size_t n = rows * cols;
    if (cols != 0 && n / cols != rows) return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "quantize_host: rows*cols overflows");
    const size_t ns = granularity == SHREWQ_PER_CHANNEL ? rows : 1;
    if ((n > 0 && (!w_host || !q_host)) || (ns > 0 && !scales_host))
        return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "quantize_host: NULL buffer");
    if ((rc = bind(ctx)) != SHREWQ_OK) return rc;
    const size_t off_q = align_up(n * 4, 256), off_s = off_q + align_up(n, 256);
    if ((rc = ensure_stage(ctx, off_s + ns * 8 + 256, 0)) != SHREWQ_OK) return rc;
    char *base = static_cast<char *>(ctx->stage_dev);
    float *w_dev = reinterpret_cast<float *>(base);
    int8_t *q_dev = reinterpret_cast<int8_t *>(base + off_q);
    double *s_dev = reinterpret_cast<double *>(base + off_s);
    if (n) SHREWQ_CUDA_TRY(ctx, cudaMemcpyAsync(w_dev, w_host, n * 4, cudaMemcpyHostToDevice, ctx->stream));
    if ((rc = launch_quantize(ctx, w_dev, rows, cols, granularity, q_dev, s_dev)) != SHREWQ_OK) return rc;
    if (n) SHREWQ_CUDA_TRY(ctx, cudaMemcpyAsync(q_host, q_dev, n, cudaMemcpyDeviceToHost, ctx->stream));
    if (ns) SHREWQ_CUDA_TRY(ctx, cudaMemcpyAsync(scales_host, s_dev, ns * 8, cudaMemcpyDeviceToHost, ctx->stream));
    SHREWQ_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    return SHREWQ_OK;
}

int shrewq_dequantize(shrewq_ctx *ctx, const int8_t *q_dev, const double *scales_dev, size_t rows, size_t cols,
                      int granularity, int out_dtype, void *out_dev) {
    if (!ctx) return set_err(nullptr, SHREWQ_ERR_INVALID_ARG, "dequantize: ctx is NULL");
    int rc = check_gran(ctx, granularity, "dequantize");
    if (rc != SHREWQ_OK) return rc;
    if (out_dtype != SHREWQ_F32 && out_dtype != SHREWQ_BF16)
        return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "dequantize: out_dtype must be SHREWQ_F32 or SHREWQ_BF16");
    const size_t n = rows * cols;
    if (cols != 0 && n / cols != rows) return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "dequantize: rows*cols overflows");
    if (n > 0 && (!q_dev || !scales_dev || !out_dev)) return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "dequantize: NULL buffer");
    if ((rc = bind(ctx)) != SHREWQ_OK) return rc;
    return launch_dequantize(ctx, q_dev, scales_dev, rows, cols, granularity, out_dtype, out_dev);
}

// ---- per-tensor quantization of a shard: amax, (caller's all-reduce), quantize -------------------
int shrewq_absmax_f32(shrewq_ctx *ctx, const float *w_dev, size_t n, float *amax_dev) {
    if (!ctx) return set_err(nullptr, SHREWQ_ERR_INVALID_ARG, "absmax: ctx is NULL");
    if (!amax_dev || (n > 0 && !w_dev)) return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "absmax: NULL buffer");
    if ((reinterpret_cast<uintptr_t>(w_dev) & 3) || (reinterpret_cast<uintptr_t>(amax_dev) & 3))
        return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "absmax: buffers must be 4-byte aligned");
    int rc = bind(ctx);
    if (rc != SHREWQ_OK) return rc;
    return launch_absmax(ctx, w_dev, n, amax_dev);
}

int shrewq_quantize_f32_given_amax(shrewq_ctx *ctx, const float *w_dev, size_t n, const float *amax_dev, int8_t *q_dev,
                                   double *scale_dev) {
    if (!ctx) return set_err(nullptr, SHREWQ_ERR_INVALID_ARG, "quantize_given_amax: ctx is NULL");
    if (!amax_dev || !scale_dev || (n > 0 && (!w_dev || !q_dev)))
        return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "quantize_given_amax: NULL buffer");
    if ((reinterpret_cast<uintptr_t>(w_dev) & 3) || (reinterpret_cast<uintptr_t>(amax_dev) & 3) ||
        (reinterpret_cast<uintptr_t>(scale_dev) & 7))
        return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "quantize_given_amax: w / amax must be 4-byte, scale 8-byte aligned");
    int rc = bind(ctx);
    if (rc != SHREWQ_OK) return rc;
    return launch_quantize_given_amax(ctx, w_dev, n, amax_dev, q_dev, scale_dev);
}

// ---- the reference's other modes (asymmetric INT8, INT4: quantize.rs:99-139,353-364) -----------------
static int check_mode(shrewq_ctx *ctx, int bits, int mode, const char *who) {
    if ((bits != 8 && bits != 4) || (mode != SHREWQ_SYMMETRIC && mode != SHREWQ_ASYMMETRIC))
        return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "%s: bits must be 8 or 4, mode SHREWQ_SYMMETRIC or SHREWQ_ASYMMETRIC", who);
    return SHREWQ_OK;
}

int shrewq_quantize_f32_ex(shrewq_ctx *ctx, const float *w_dev, size_t rows, size_t cols, int granularity, int bits,
                           int mode, int8_t *q_dev, double *scales_dev, double *zero_points_dev) {
    if (!ctx) return set_err(nullptr, SHREWQ_ERR_INVALID_ARG, "quantize_ex: ctx is NULL");
    int rc = check_gran(ctx, granularity, "quantize_ex");
    if (rc != SHREWQ_OK) return rc;
    if ((rc = check_mode(ctx, bits, mode, "quantize_ex")) != SHREWQ_OK) return rc;
    const size_t n = rows * cols;
    if (cols != 0 && n / cols != rows) return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "quantize_ex: rows*cols overflows");
    const size_t ns = granularity == SHREWQ_PER_CHANNEL ? rows : 1;
    if (ns > 0 && (!scales_dev || !zero_points_dev))
        return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "quantize_ex: scales_dev / zero_points_dev is NULL");
    if (n > 0 && (!w_dev || !q_dev)) return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "quantize_ex: w_dev / q_dev is NULL");
    if ((reinterpret_cast<uintptr_t>(w_dev) & 3) || (reinterpret_cast<uintptr_t>(scales_dev) & 7) ||
        (reinterpret_cast<uintptr_t>(zero_points_dev) & 7))
        return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "quantize_ex: w_dev must be 4-byte, scales / zero points 8-byte aligned");
    if ((rc = bind(ctx)) != SHREWQ_OK) return rc;
    if (bits == 8 && mode == SHREWQ_SYMMETRIC) {
        if ((rc = launch_quantize(ctx, w_dev, rows, cols, granularity, q_dev, scales_dev)) != SHREWQ_OK) return rc;
        if (ns) SHREWQ_CUDA_TRY(ctx, cudaMemsetAsync(zero_points_dev, 0, ns * sizeof(double), ctx->stream));  // 0.0
        return SHREWQ_OK;
    }
    return launch_quantize_ex(ctx, w_dev, rows, cols, granularity, bits, mode, q_dev, scales_dev, zero_points_dev);
}

int shrewq_quantize_any(shrewq_ctx *ctx, const void *w_dev, int w_dtype, size_t rows, size_t cols, int granularity, int bits,
                        int mode, int8_t *q_dev, double *scales_dev, double *zero_points_dev) {
    if (!ctx) return set_err(nullptr, SHREWQ_ERR_INVALID_ARG, "quantize_any: ctx is NULL");
    int rc = check_gran(ctx, granularity, "quantize_any");
    if (rc != SHREWQ_OK) return rc;
    if (w_dtype != SHREWQ_F32 && w_dtype != SHREWQ_BF16 && w_dtype != SHREWQ_F16 && w_dtype != SHREWQ_F64)
        return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "quantize_any: w_dtype must be SHREWQ_F32, _BF16, _F16 or _F64");
    if ((bits != 8 && bits != 4) || (mode != SHREWQ_SYMMETRIC && mode != SHREWQ_ASYMMETRIC))
        return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "quantize_any: bits must be 8 or 4, mode SHREWQ_SYMMETRIC or SHREWQ_ASYMMETRIC");
    const size_t n = rows * cols;
    if (cols != 0 && n / cols != rows) return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "quantize_any: rows*cols overflows");
    const size_t ns = granularity == SHREWQ_PER_CHANNEL ? rows : 1;
    if ((ns > 0 && (!scales_dev || !zero_points_dev)) || (n > 0 && (!w_dev || !q_dev)))
        return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "quantize_any: NULL buffer");
    const size_t wal = w_dtype == SHREWQ_F64 ? 8 : (w_dtype == SHREWQ_F32 ? 4 : 2);
    if ((reinterpret_cast<uintptr_t>(w_dev) % wal) || (reinterpret_cast<uintptr_t>(scales_dev) & 7) ||
        (reinterpret_cast<uintptr_t>(zero_points_dev) & 7))
        return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "quantize_any: buffers not aligned to their element size");
    if ((rc = bind(ctx)) != SHREWQ_OK) return rc;
    return launch_quantize_any(ctx, w_dev, w_dtype, rows, cols, granularity, bits, mode, q_dev, scales_dev, zero_points_dev);
}

int shrewq_dequantize_ex(shrewq_ctx *ctx, const int8_t *q_dev, const double *scales_dev, const double *zero_points_dev,
                         size_t rows, size_t cols, int granularity, int out_dtype, void *out_dev) {
    if (!zero_points_dev && (out_dtype == SHREWQ_F32 || out_dtype == SHREWQ_BF16))
        return shrewq_dequantize(ctx, q_dev, scales_dev, rows, cols, granularity, out_dtype, out_dev);
    if (!ctx) return set_err(nullptr, SHREWQ_ERR_INVALID_ARG, "dequantize_ex: ctx is NULL");
    int rc = check_gran(ctx, granularity, "dequantize_ex");
    if (rc != SHREWQ_OK) return rc;
    if (out_dtype != SHREWQ_F32 && out_dtype != SHREWQ_BF16 && out_dtype != SHREWQ_F16 && out_dtype != SHREWQ_F64)
        return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "dequantize_ex: out_dtype must be SHREWQ_F32, _BF16, _F16 or _F64");
    const size_t n = rows * cols;
    if (cols != 0 && n / cols != rows) return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "dequantize_ex: rows*cols overflows");
    if (n > 0 && (!q_dev || !scales_dev || !out_dev)) return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "dequantize_ex: NULL buffer");
    if ((rc = bind(ctx)) != SHREWQ_OK) return rc;
    return launch_dequantize_ex(ctx, q_dev, scales_dev, zero_points_dev, rows, cols, granularity, out_dtype, out_dev);
}

int shrewq_pack_int4(shrewq_ctx *ctx, const int8_t *q_dev, size_t rows, size_t cols, uint8_t *packed_dev) {
    if (!ctx) return set_err(nullptr, SHREWQ_ERR_INVALID_ARG, "pack_int4: ctx is NULL");
    if (cols % 2 != 0) return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "pack_int4: cols must be even (two codes per byte)");
    const size_t n = rows * cols;
    if (cols != 0 && n / cols != rows) return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "pack_int4: rows*cols overflows");
    if (n > 0 && (!q_dev || !packed_dev)) return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "pack_int4: NULL buffer");
    int rc = bind(ctx);
    if (rc != SHREWQ_OK) return rc;
    return launch_pack_int4(ctx, q_dev, n / 2, packed_dev);
}

// ---- quantized Linear ---------------------------------------------------------------------
int shrewq_linear_create(shrewq_ctx *ctx, const int8_t *q_dev, const double *scales_dev, const float *bias_dev,
                         size_t out_features, size_t in_features, int granularity, shrewq_linear **out) {
    if (!ctx) return set_err(nullptr, SHREWQ_ERR_INVALID_ARG, "linear_create: ctx is NULL");
    if (!out) return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "linear_create: out is NULL");
    *out = nullptr;
    int rc = check_gran(ctx, granularity, "linear_create");
    if (rc != SHREWQ_OK) return rc;
    if (out_features == 0 || in_features == 0)
        return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "linear_create: out_features and in_features must be positive");
    if (!q_dev || !scales_dev) return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "linear_create: q_dev / scales_dev is NULL");
    if (out_features > 0x7FFFFFFFull || in_features > 0x7FFFFFFFull)
        return set_err(ctx, SHREWQ_ERR_UNSUPPORTED, "linear_create: dimensions above 2^31-1");
    if ((rc = bind(ctx)) != SHREWQ_OK) return rc;
    shrewq_linear *lin = new (std::nothrow) shrewq_linear();
    if (!lin) return set_err(ctx, SHREWQ_ERR_ALLOC, "out of host memory");
    lin->ctx = ctx;
    lin->q = q_dev;
    lin->bias = bias_dev;
    lin->n = out_features;
    lin->k = in_features;
    lin->granularity = granularity;
    cudaError_t e = cudaMalloc(&lin->scales_f32, out_features * sizeof(float));
    if (e != cudaSuccess) {
        cudaGetLastError();
        delete lin;
        return set_err(ctx, SHREWQ_ERR_ALLOC, "linear_create: cudaMalloc of scales failed: %s", cudaGetErrorString(e));
    }
    rc = launch_scales_to_f32(ctx, scales_dev, granularity, out_features, lin->scales_f32);
    if (rc == SHREWQ_OK && (in_features % 16) == 0 && (reinterpret_cast<uintptr_t>(q_dev) & 15) == 0) {
        if (encode_weight_tmap(ctx, q_dev, out_features, in_features, 128, lin->w_tmap) == SHREWQ_OK &&
            encode_weight_tmap(ctx, q_dev, out_features, in_features, 64, lin->w_tmap64) == SHREWQ_OK)
            lin->tmap_ok = true;
    }
    if (rc != SHREWQ_OK) {
        cudaFree(lin->scales_f32);
        delete lin;
        return rc;
    }
    *out = lin;
    return SHREWQ_OK;
}

int shrewq_linear_create_ex(shrewq_ctx *ctx, const int8_t *q_dev, const double *scales_dev,
                            const double *zero_points_dev, const float *bias_dev, size_t out_features,
                            size_t in_features, int granularity, shrewq_linear **out) {
    if (!zero_points_dev)
        return shrewq_linear_create(ctx, q_dev, scales_dev, bias_dev, out_features, in_features, granularity, out);
    if (!ctx) return set_err(nullptr, SHREWQ_ERR_INVALID_ARG, "linear_create_ex: ctx is NULL");
    int rc = shrewq_linear_create(ctx, q_dev, scales_dev, bias_dev, out_features, in_features, granularity, out);
    if (rc != SHREWQ_OK) return rc;
    shrewq_linear *lin = *out;
    cudaError_t e = cudaMalloc(&lin->czp, out_features * sizeof(float));
    if (e != cudaSuccess) {
        cudaGetLastError();
        shrewq_linear_destroy(lin);
        *out = nullptr;
        return set_err(ctx, SHREWQ_ERR_ALLOC, "linear_create_ex: cudaMalloc failed: %s", cudaGetErrorString(e));
    }
    rc = launch_scale_zp_to_f32(ctx, scales_dev, zero_points_dev, granularity, out_features, lin->czp);
    if (rc != SHREWQ_OK) {
        shrewq_linear_destroy(lin);
        *out = nullptr;
    }
    return rc;
}

int shrewq_linear_create_int4(shrewq_ctx *ctx, const uint8_t *packed_dev, const double *scales_dev, const float *bias_dev,
                              size_t out_features, size_t in_features, int granularity, shrewq_linear **out) {
    if (!ctx) return set_err(nullptr, SHREWQ_ERR_INVALID_ARG, "linear_create_int4: ctx is NULL");
    if (!out) return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "linear_create_int4: out is NULL");
    *out = nullptr;
    if (in_features % 2 != 0) return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "linear_create_int4: in_features must be even");
    // the plain constructor does everything but the TMA descriptors, which describe an INT8 [N,K] matrix
    // and must not be used with packed rows: build the handle, then mark it
    int rc = shrewq_linear_create(ctx, reinterpret_cast<const int8_t *>(packed_dev), scales_dev, bias_dev, out_features,
                                  in_features, granularity, out);
    if (rc != SHREWQ_OK) return rc;
    (*out)->int4_packed = true;
    (*out)->tmap_ok = false;
    return SHREWQ_OK;
}

void shrewq_linear_destroy(shrewq_linear *lin) {
    if (!lin) return;
    cudaSetDevice(lin->ctx->device);
    cudaStreamSynchronize(lin->ctx->stream);
    if (lin->scales_f32) cudaFree(lin->scales_f32);
    if (lin->czp) cudaFree(lin->czp);
    delete lin;
}

size_t shrewq_linear_in_features(const shrewq_linear *lin) { return lin ? lin->k : 0; }
size_t shrewq_linear_out_features(const shrewq_linear *lin) { return lin ? lin->n : 0; }
/* fp32 size minus INT8 size — quantize.rs:455-459 */
size_t shrewq_linear_memory_savings_bytes(const shrewq_linear *lin) {
    if (!lin) return 0;
    return lin->n * lin->k * 4 - (lin->int4_packed ? lin->n * lin->k / 2 : lin->n * lin->k);
}
const char *shrewq_linear_last_kernel(const shrewq_linear *lin) { return lin ? g_last_kernel : "none"; }

// f32 activations on the tensor cores: x is split into bf16 hi + lo (exact to ~2^-17 of each value), the
// two matrices are stacked in one workspace and the kernel issues two MMAs per k-step into the same
// accumulator, so the codes are read and converted once and the result keeps the f32 path's 1e-4 tolerance.
static int forward_f32_on_tensor_cores(shrewq_linear *lin, const ForwardArgs &orig, const char *who) {
    shrewq_ctx *ctx = lin->ctx;
    const size_t n = orig.M * orig.K;
    int rc = ensure_xsplit(ctx, 2 * n * 2);
    if (rc != SHREWQ_OK) return rc;
    char *hi = static_cast<char *>(ctx->xsplit), *lo = hi + n * 2;
    if ((rc = launch_split_f32(ctx, static_cast<const float *>(orig.x), n, hi, lo)) != SHREWQ_OK) return rc;
    ForwardArgs a = orig;
    a.x_dtype = SHREWQ_BF16;
    a.x = hi;
    if (!tcgen05_supported(a)) return set_err(ctx, SHREWQ_ERR_UNSUPPORTED, "%s: the tensor-core kernel cannot take this shape", who);
    return launch_gemm_tcgen05_xsplit(ctx, a, lin->w_tmap);
}

static int forward_impl(shrewq_linear *lin, shrewq_linear *up, const void *x_dev, int x_dtype, size_t M, void *y_dev,
                        int y_dtype, size_t ldy, int epilogue, const char *who, void *const *peers = nullptr,
                        int n_peers = 0) {
    if (!lin) return set_err(nullptr, SHREWQ_ERR_INVALID_ARG, "%s: handle is NULL", who);
    shrewq_ctx *ctx = lin->ctx;
    if (up && (up->ctx != ctx || up->n != lin->n || up->k != lin->k))
        return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "%s: gate and up must share context and shape", who);
    if ((x_dtype != SHREWQ_F32 && x_dtype != SHREWQ_BF16) || (y_dtype != SHREWQ_F32 && y_dtype != SHREWQ_BF16))
        return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "%s: dtype must be SHREWQ_F32 or SHREWQ_BF16", who);
    if (epilogue != SHREWQ_EPILOGUE_NONE && epilogue != SHREWQ_EPILOGUE_RELU)
        return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "%s: unknown epilogue %d", who, epilogue);
    if (M == 0) return SHREWQ_OK;
    if (!x_dev || !y_dev) return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "%s: x / y is NULL", who);
    if (ldy < lin->n) return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "%s: ldy (%zu) smaller than out_features (%zu)", who, ldy, lin->n);
    const size_t xal = x_dtype == SHREWQ_BF16 ? 2 : 4, yal = y_dtype == SHREWQ_BF16 ? 2 : 4;
    if ((reinterpret_cast<uintptr_t>(x_dev) % xal) || (reinterpret_cast<uintptr_t>(y_dev) % yal))
        return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "%s: x / y not aligned to their element size", who);
    if (M > 0x7FFFFFFFull) return set_err(ctx, SHREWQ_ERR_UNSUPPORTED, "%s: M above 2^31-1", who);
    int rc = bind(ctx);
    if (rc != SHREWQ_OK) return rc;

    ForwardArgs a;
    a.q = lin->q; a.scales = lin->scales_f32; a.bias = lin->bias;
    a.x = x_dev; a.x_dtype = x_dtype; a.y = y_dev; a.y_dtype = y_dtype;
    a.M = M; a.N = lin->n; a.K = lin->k; a.ldy = ldy; a.epilogue = epilogue;
    if (up) { a.q_up = up->q; a.scales_up = up->scales_f32; a.bias_up = up->bias; }
    if (n_peers < 0 || n_peers > kMaxPeers || (n_peers > 0 && !peers))
        return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "%s: between 0 and %d peer destinations", who, kMaxPeers);
    for (int i = 0; i < n_peers; ++i) {
        if (!peers[i] || (reinterpret_cast<uintptr_t>(peers[i]) % yal))
            return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "%s: peer destination %d is NULL or misaligned", who, i);
        a.extra.p[i] = peers[i];
    }
    a.extra.n = n_peers;
    a.pdl = ctx->tuning.pdl != 0 && lin->forwarded.load(std::memory_order_relaxed) &&
            (!up || up->forwarded.load(std::memory_order_relaxed));

    // Packed INT4 rows: only the warp-MMA forward reads them (batch <= 32 for now)
    if (lin->int4_packed || (up && up->int4_packed)) {
        if (up && !(lin->int4_packed && up->int4_packed))
            return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "%s: gate and up must both be packed INT4 or both INT8", who);
        if (lin->czp || (up && up->czp))
            return set_err(ctx, SHREWQ_ERR_UNSUPPORTED, "%s: packed INT4 with zero points is not built", who);
        if (!gemv_mma_w4_supported(a))
            return set_err(ctx, SHREWQ_ERR_UNSUPPORTED,
                           "%s: packed INT4 weights need bf16 activations, M <= 32, in_features a multiple of 128", who);
        rc = launch_gemv_mma_w4(ctx, a);
        g_last_kernel = "mma-w4";
        return rc;
    }

    // Zero points: y = scale * (sum_k q x) + bias - (scale * zp) * sum_k x.  The kernels below
    // compute the first part into an f32 buffer; a last pass subtracts the second, applies the
    // elementwise op and narrows to the caller's type.
    const bool zp_route = lin->czp != nullptr || (up && up->czp != nullptr);
    float *zp_acc = nullptr, *zp_xsum = nullptr;
    if (zp_route) {
        if (up || n_peers > 0)
            return set_err(ctx, SHREWQ_ERR_UNSUPPORTED, "%s: zero points are not supported with a gate/up pair or peer destinations", who);
        const size_t acc_bytes = align_up(M * lin->n * sizeof(float), 256);
        if ((rc = grow(ctx, &ctx->ytmp, &ctx->ytmp_bytes, acc_bytes + M * sizeof(float), false)) != SHREWQ_OK) return rc;
        zp_acc = static_cast<float *>(ctx->ytmp);
        zp_xsum = reinterpret_cast<float *>(static_cast<char *>(ctx->ytmp) + acc_bytes);
        if ((rc = launch_row_sums(ctx, x_dev, x_dtype, M, lin->k, zp_xsum)) != SHREWQ_OK) return rc;
        a.y = zp_acc; a.y_dtype = SHREWQ_F32; a.ldy = lin->n; a.epilogue = SHREWQ_EPILOGUE_NONE;
    }

    const bool vec16 = (lin->k % 16) == 0 && (reinterpret_cast<uintptr_t>(lin->q) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(x_dev) & 15) == 0 &&
                       (!up || (reinterpret_cast<uintptr_t>(up->q) & 15) == 0);
    const bool gemv_ok = vec16 && M <= 16;
    const bool gemv_sliced_ok = vec16 && gemv_slices_win(M, lin->n, lin->k);
    const bool tc_ok = tcgen05_supported(a) && lin->tmap_ok && (!up || up->tmap_ok);
    const bool mma_ok = gemv_mma_supported(a);
    // f32 activations as bf16 hi + lo on the tensor cores (plain layers only)
    const bool f32_tc_ok = x_dtype == SHREWQ_F32 && !up && lin->tmap_ok && vec16 && n_peers == 0;
    int choice;
    switch (g_forced_kernel) {
        case kForceGemv:
            if (!gemv_ok && !(vec16 && M <= kGemvSlicedMaxTokens))
                return set_err(ctx, SHREWQ_ERR_UNSUPPORTED, "%s: forced gemv cannot take this shape", who);
            choice = kForceGemv; break;
        case kForceTc2Cta:
            if (!tc_ok) return set_err(ctx, SHREWQ_ERR_UNSUPPORTED, "%s: forced tcgen05-2cta cannot take this shape/dtype", who);
            choice = kForceTc2Cta; break;
        case kForceTcF32:
            if (!f32_tc_ok)
                return set_err(ctx, SHREWQ_ERR_UNSUPPORTED, "%s: forced tcgen05-f32 needs f32 activations, 16-byte aligned buffers, no gate/up pair", who);
            choice = kForceTcF32; break;
        case kForceTc:
            if (!tc_ok) return set_err(ctx, SHREWQ_ERR_UNSUPPORTED, "%s: forced tcgen05 cannot take this shape/dtype", who);
            choice = kForceTc; break;
        case kForceSimt: choice = kForceSimt; break;
        case kForceRing:
            if (!gemv_ring_supported(a)) return set_err(ctx, SHREWQ_ERR_UNSUPPORTED, "%s: forced mma-ring kernel cannot take this shape/dtype", who);
            choice = kForceRing; break;
        case kForceMma:
            if (!mma_ok) return set_err(ctx, SHREWQ_ERR_UNSUPPORTED, "%s: forced mma kernel cannot take this shape/dtype", who);
            choice = kForceMma; break;
        default:
            if (x_dtype == SHREWQ_F32) {
                // a few tokens: the GEMV reads f32 activations directly; beyond, the tensor cores on the
                // bf16 hi/lo pair; the general f32 kernel takes what neither can (misaligned, odd widths)
                choice = (gemv_ok || gemv_sliced_ok) ? kForceGemv : f32_tc_ok ? kForceTcF32 : kForceSimt;
            } else if (M > 128 && tc_ok && (ctx->tuning.tc_pair == 2 || (ctx->tuning.tc_pair == 1 && pair_kernel_wins(M, lin->n, lin->k, up != nullptr)))) {
                choice = kForceTc2Cta;
            } else {
                choice = default_family(M, lin->n, up != nullptr, ctx->sm_count, gemv_ok, mma_ok, tc_ok);
            }
    }
    const char *name;
    if (choice == kForceGemv) { rc = launch_gemv(ctx, a); name = "gemv"; }
    else if (choice == kForceMma) { rc = launch_gemv_mma(ctx, a); name = "mma"; }
    else if (choice == kForceRing) { rc = launch_gemv_ring(ctx, a); name = "mma-ring"; }
    else if (choice == kForceTc) {
        rc = up ? launch_gemm_tcgen05(ctx, a, lin->w_tmap64, up->w_tmap64) : launch_gemm_tcgen05(ctx, a, lin->w_tmap, nullptr);
        name = "tcgen05";
    } else if (choice == kForceTc2Cta) {
        rc = up ? launch_gemm_tcgen05_2cta(ctx, a, lin->w_tmap64, up->w_tmap64) : launch_gemm_tcgen05_2cta(ctx, a, lin->w_tmap, nullptr);
        name = "tcgen05-2cta";
    } else if (choice == kForceTcF32) {
        rc = forward_f32_on_tensor_cores(lin, a, who);
        name = "tcgen05-f32";
    } else {
        if (n_peers > 0) return set_err(ctx, SHREWQ_ERR_UNSUPPORTED, "%s: peer destinations need the gemv, mma or tcgen05 kernel", who);
        rc = launch_gemm_simt(ctx, a); name = "simt";
    }
    g_last_kernel = name;
    if (rc == SHREWQ_OK) {
        lin->forwarded.store(true, std::memory_order_relaxed);
        if (up) up->forwarded.store(true, std::memory_order_relaxed);
    }
    if (zp_route && rc == SHREWQ_OK)
        rc = launch_zero_point_fix(ctx, zp_acc, lin->czp, zp_xsum, M, lin->n, ldy, epilogue == SHREWQ_EPILOGUE_RELU, y_dtype, y_dev);
    return rc;
}

int shrewq_linear_forward(shrewq_linear *lin, const void *x_dev, int x_dtype, size_t M, void *y_dev, int y_dtype,
                          size_t ldy, int epilogue) {
    return forward_impl(lin, nullptr, x_dev, x_dtype, M, y_dev, y_dtype, ldy, epilogue, "linear_forward");
}

int shrewq_linear_forward_noalloc(shrewq_linear *lin, const void *x_dev, size_t M, void *y_dev, int y_dtype,
                                  size_t ldy, int epilogue) {
    if (!lin) return set_err(nullptr, SHREWQ_ERR_INVALID_ARG, "forward_noalloc: handle is NULL");
    shrewq_ctx *ctx = lin->ctx;
    if (y_dtype != SHREWQ_F32 && y_dtype != SHREWQ_BF16)
        return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "forward_noalloc: y_dtype must be SHREWQ_F32 or SHREWQ_BF16");
    if (epilogue != SHREWQ_EPILOGUE_NONE && epilogue != SHREWQ_EPILOGUE_RELU)
        return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "forward_noalloc: unknown epilogue %d", epilogue);
    if (lin->czp || lin->int4_packed)
        return set_err(ctx, SHREWQ_ERR_UNSUPPORTED, "forward_noalloc: handles with zero points or packed INT4 rows need shrewq_linear_forward");
    if (M == 0) return SHREWQ_OK;
    if (!x_dev || !y_dev) return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "forward_noalloc: x / y is NULL");
    if (ldy < lin->n) return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "forward_noalloc: ldy smaller than out_features");
    if ((reinterpret_cast<uintptr_t>(y_dev) % (y_dtype == SHREWQ_BF16 ? 2 : 4)))
        return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "forward_noalloc: y not aligned to its element size");
    int rc = bind(ctx);
    if (rc != SHREWQ_OK) return rc;
    ForwardArgs a;
    a.q = lin->q; a.scales = lin->scales_f32; a.bias = lin->bias;
    a.x = x_dev; a.x_dtype = SHREWQ_BF16; a.y = y_dev; a.y_dtype = y_dtype;
    a.M = M; a.N = lin->n; a.K = lin->k; a.ldy = ldy; a.epilogue = epilogue;
    if (!tcgen05_supported(a) || !lin->tmap_ok)
        return set_err(ctx, SHREWQ_ERR_UNSUPPORTED,
                       "forward_noalloc: needs bf16 activations, 16-byte aligned x and weights, in_features a multiple of 16");
    rc = launch_gemm_tcgen05_noalloc(ctx, a, lin->w_tmap);
    g_last_kernel = "tcgen05";
    return rc;
}

int shrewq_linear_forward_gate_up_silu(shrewq_linear *gate, shrewq_linear *up, const void *x_dev, int x_dtype,
                                       size_t M, void *h_dev, int h_dtype, size_t ldh) {
    if (!up) return set_err(gate ? gate->ctx : nullptr, SHREWQ_ERR_INVALID_ARG, "gate_up_silu: up handle is NULL");
    return forward_impl(gate, up, x_dev, x_dtype, M, h_dev, h_dtype, ldh, SHREWQ_EPILOGUE_NONE, "gate_up_silu");
}

int shrewq_linear_forward_peers(shrewq_linear *lin, shrewq_linear *up, const void *x_dev, int x_dtype, size_t M,
                                void *y_dev, void *const *peer_y_dev, int n_peers, int y_dtype, size_t ldy,
                                int epilogue) {
    return forward_impl(lin, up, x_dev, x_dtype, M, y_dev, y_dtype, ldy, up ? SHREWQ_EPILOGUE_NONE : epilogue,
                        "linear_forward_peers", peer_y_dev, n_peers);
}

int shrewq_linear_forward_host(shrewq_linear *lin, const void *x_host, int x_dtype, size_t M, void *y_host,
                               int y_dtype, int epilogue) {
    if (!lin) return set_err(nullptr, SHREWQ_ERR_INVALID_ARG, "linear_forward_host: handle is NULL");
    shrewq_ctx *ctx = lin->ctx;
    if ((x_dtype != SHREWQ_F32 && x_dtype != SHREWQ_BF16) || (y_dtype != SHREWQ_F32 && y_dtype != SHREWQ_BF16))
        return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "linear_forward_host: dtype must be SHREWQ_F32 or SHREWQ_BF16");
    if (M == 0) return SHREWQ_OK;
    if (!x_host || !y_host) return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "linear_forward_host: x / y is NULL");
    int rc = bind(ctx);
    if (rc != SHREWQ_OK) return rc;
    const size_t xb = M * lin->k * (x_dtype == SHREWQ_BF16 ? 2 : 4), yb = M * lin->n * (y_dtype == SHREWQ_BF16 ? 2 : 4);
    const size_t off_y = align_up(xb, 256);
    if ((rc = ensure_stage(ctx, off_y + yb + 256, 0)) != SHREWQ_OK) return rc;
    char *base = static_cast<char *>(ctx->stage_dev);
    SHREWQ_CUDA_TRY(ctx, cudaMemcpyAsync(base, x_host, xb, cudaMemcpyHostToDevice, ctx->stream));
    rc = forward_impl(lin, nullptr, base, x_dtype, M, base + off_y, y_dtype, lin->n, epilogue, "linear_forward_host");
    if (rc != SHREWQ_OK) return rc;
    SHREWQ_CUDA_TRY(ctx, cudaMemcpyAsync(y_host, base + off_y, yb, cudaMemcpyDeviceToHost, ctx->stream));
    return shrewq_ctx_synchronize(ctx);
}

int shrewq_mlp_forward_host(shrewq_linear *gate, shrewq_linear *up, shrewq_linear *down, const void *x_host, size_t M,
                            void *y_host, int y_dtype, int synchronize) {
    if (!gate || !up || !down) return set_err(nullptr, SHREWQ_ERR_INVALID_ARG, "mlp_forward_host: a handle is NULL");
    shrewq_ctx *ctx = gate->ctx;
    if (up->ctx != ctx || down->ctx != ctx || up->n != gate->n || up->k != gate->k || down->k != gate->n)
        return set_err(ctx, SHREWQ_ERR_INVALID_ARG,
                       "mlp_forward_host: gate and up must have one shape, down must take their width, all on one context");
    if (y_dtype != SHREWQ_F32 && y_dtype != SHREWQ_BF16)
        return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "mlp_forward_host: y_dtype must be SHREWQ_F32 or SHREWQ_BF16");
    if (M == 0) return SHREWQ_OK;
    if (!x_host || !y_host) return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "mlp_forward_host: x / y is NULL");
    int rc = bind(ctx);
    if (rc != SHREWQ_OK) return rc;
    if (!ctx->copy_in) {
        SHREWQ_CUDA_TRY(ctx, cudaStreamCreateWithFlags(&ctx->copy_in, cudaStreamNonBlocking));
        SHREWQ_CUDA_TRY(ctx, cudaStreamCreateWithFlags(&ctx->copy_out, cudaStreamNonBlocking));
        for (int i = 0; i < 2; ++i) {
            SHREWQ_CUDA_TRY(ctx, cudaEventCreateWithFlags(&ctx->ev_in[i], cudaEventDisableTiming));
            SHREWQ_CUDA_TRY(ctx, cudaEventCreateWithFlags(&ctx->ev_cmp[i], cudaEventDisableTiming));
            SHREWQ_CUDA_TRY(ctx, cudaEventCreateWithFlags(&ctx->ev_out[i], cudaEventDisableTiming));
        }
    }
    const size_t xb = align_up(M * gate->k * 2, 256), hb = align_up(M * gate->n * 2, 256);
    const size_t yb = align_up(M * down->n * (y_dtype == SHREWQ_BF16 ? 2 : 4), 256), slot_bytes = xb + hb + yb;
    if (ctx->mlp_stage_bytes < 2 * slot_bytes) {
        // (growing synchronises everything that may still use the old slots)
        if (ctx->copy_out) SHREWQ_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->copy_out));
        if ((rc = grow(ctx, &ctx->mlp_stage, &ctx->mlp_stage_bytes, 2 * slot_bytes, false)) != SHREWQ_OK) return rc;
        ctx->mlp_calls = 0;
    }
    const int slot = (int)(ctx->mlp_calls & 1);
    const bool reused = ctx->mlp_calls >= 2;
    ctx->mlp_calls += 1;
    char *base = static_cast<char *>(ctx->mlp_stage) + (size_t)slot * (ctx->mlp_stage_bytes / 2 / 256 * 256);
    char *x_dev = base, *h_dev = base + xb, *y_dev = base + xb + hb;
    // copy-in: after the kernels of the call two back have read this slot's x
    if (reused) SHREWQ_CUDA_TRY(ctx, cudaStreamWaitEvent(ctx->copy_in, ctx->ev_cmp[slot], 0));
    SHREWQ_CUDA_TRY(ctx, cudaMemcpyAsync(x_dev, x_host, M * gate->k * 2, cudaMemcpyHostToDevice, ctx->copy_in));
    SHREWQ_CUDA_TRY(ctx, cudaEventRecord(ctx->ev_in[slot], ctx->copy_in));
    // kernels on the context's stream: after this call's x has landed and the slot's previous y has left
    SHREWQ_CUDA_TRY(ctx, cudaStreamWaitEvent(ctx->stream, ctx->ev_in[slot], 0));
    if (reused) SHREWQ_CUDA_TRY(ctx, cudaStreamWaitEvent(ctx->stream, ctx->ev_out[slot], 0));
    rc = forward_impl(gate, up, x_dev, SHREWQ_BF16, M, h_dev, SHREWQ_BF16, gate->n, SHREWQ_EPILOGUE_NONE, "mlp_forward_host");
    if (rc != SHREWQ_OK) return rc;
    rc = forward_impl(down, nullptr, h_dev, SHREWQ_BF16, M, y_dev, y_dtype, down->n, SHREWQ_EPILOGUE_NONE, "mlp_forward_host");
    if (rc != SHREWQ_OK) return rc;
    SHREWQ_CUDA_TRY(ctx, cudaEventRecord(ctx->ev_cmp[slot], ctx->stream));
    // copy-out
    SHREWQ_CUDA_TRY(ctx, cudaStreamWaitEvent(ctx->copy_out, ctx->ev_cmp[slot], 0));
    SHREWQ_CUDA_TRY(ctx, cudaMemcpyAsync(y_host, y_dev, M * down->n * (y_dtype == SHREWQ_BF16 ? 2 : 4), cudaMemcpyDeviceToHost,
                                         ctx->copy_out));
    SHREWQ_CUDA_TRY(ctx, cudaEventRecord(ctx->ev_out[slot], ctx->copy_out));
    return synchronize ? shrewq_ctx_synchronize(ctx) : SHREWQ_OK;
}

}  // extern "C"
