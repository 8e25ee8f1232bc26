// Launchers of the INT8 symmetric quantize / dequantize kernels (device code and its description:
// quantize_kernels.cuh).
#include "common.cuh"
#include "quantize_kernels.cuh"

namespace shrewq {

namespace {

template <int GROUP, int NV>
void launch_rows_reg(shrewq_ctx *ctx, const float *w, size_t rows, size_t cols, int8_t *q, double *scales) {
    constexpr int THREADS = GROUP >= 256 ? GROUP : 256;
    constexpr int ROWS_PER_CTA = THREADS / GROUP;
    const unsigned grid = (unsigned)((rows + ROWS_PER_CTA - 1) / ROWS_PER_CTA);
    quantize_rows_reg_kernel<GROUP, NV><<<grid, THREADS, 0, ctx->stream>>>(w, rows, cols, q, scales);
}

}  // namespace

int launch_quantize(shrewq_ctx *ctx, const float *w, size_t rows, size_t cols, int granularity,
                    int8_t *q, double *scales) {
    const size_t n = rows * cols;
    if (granularity == SHREWQ_PER_CHANNEL) {
        if (rows == 0) return SHREWQ_OK;
        if (rows > 0x7FFFFFFFull) return set_err(ctx, SHREWQ_ERR_UNSUPPORTED, "quantize: more than 2^31-1 channels");
        const bool vec = (cols % 4 == 0) && ((reinterpret_cast<uintptr_t>(w) & 15) == 0) &&
                         ((reinterpret_cast<uintptr_t>(q) & 3) == 0) && cols >= 32;
        if (vec && cols <= 128) launch_rows_reg<32, 1>(ctx, w, rows, cols, q, scales);
        else if (vec && cols <= 256) launch_rows_reg<32, 2>(ctx, w, rows, cols, q, scales);
        else if (vec && cols <= 512) launch_rows_reg<32, 4>(ctx, w, rows, cols, q, scales);
        else if (vec && cols <= 1024) launch_rows_reg<32, 8>(ctx, w, rows, cols, q, scales);
        else if (vec && cols <= 2048) launch_rows_reg<256, 2>(ctx, w, rows, cols, q, scales);
        else if (vec && cols <= 4096) launch_rows_reg<256, 4>(ctx, w, rows, cols, q, scales);
        else if (vec && cols <= 8192) launch_rows_reg<256, 8>(ctx, w, rows, cols, q, scales);
        // 512 threads x 8 float4 rather than 256 x 16: 48 registers per thread instead of 80 keeps
        // more rows resident per SM (the 256 x 16 tile measured 4.4 TB/s against 5.1-5.5 TB/s for
        // the 8-float4 tiles)
        else if (vec && cols <= 16384) launch_rows_reg<512, 8>(ctx, w, rows, cols, q, scales);
        else if (vec && cols <= 32768) launch_rows_reg<1024, 8>(ctx, w, rows, cols, q, scales);
        else {
            const unsigned grid = (unsigned)(rows < (size_t)ctx->sm_count * 32 ? rows : (size_t)ctx->sm_count * 32);
            quantize_rows_generic_kernel<<<grid, 256, 0, ctx->stream>>>(w, rows, cols, q, scales);
        }
        ctx->launches += 1;
    } else {
        // scratch layout: [0] amax bits, [64..] TensorParams
        int rc = ensure_scratch(ctx, 256);
        if (rc != SHREWQ_OK) return rc;
        unsigned int *amax_bits = reinterpret_cast<unsigned int *>(ctx->scratch);
        TensorParams *tp = reinterpret_cast<TensorParams *>(reinterpret_cast<char *>(ctx->scratch) + 64);
        SHREWQ_CUDA_TRY(ctx, cudaMemsetAsync(amax_bits, 0, 4, ctx->stream));
        size_t want = (n / 4 + 255) / 256;
        const size_t cap = (size_t)ctx->sm_count * 16;
        unsigned grid = (unsigned)(want < 1 ? 1 : (want > cap ? cap : want));
        if (n > 0) {
            absmax_flat_kernel<<<grid, 256, 0, ctx->stream>>>(w, n, amax_bits);
            ctx->launches += 1;
        }
        finalize_tensor_scale_kernel<<<1, 1, 0, ctx->stream>>>(amax_bits, n, scales, tp);
        ctx->launches += 1;
        if (n > 0) {
            quantize_flat_kernel<<<grid, 256, 0, ctx->stream>>>(w, n, tp, q);
            ctx->launches += 1;
        }
    }
    SHREWQ_CUDA_TRY(ctx, cudaGetLastError());
    return SHREWQ_OK;
}

// ---- per-tensor quantization of a row shard ---------------------------------------------------
// A tensor split over several GPUs has ONE per-tensor scale, defined by the amax of the whole
// tensor (quantize.rs:349-351).  Each rank takes the amax of its shard, the ranks take the max of
// those (one float through an all-reduce, done by the caller), and every rank quantizes its shard
// with the global value.  Same kernels as the single-GPU per-tensor path.
int launch_absmax(shrewq_ctx *ctx, const float *w, size_t n, float *amax_dev) {
    SHREWQ_CUDA_TRY(ctx, cudaMemsetAsync(amax_dev, 0, sizeof(float), ctx->stream));  // +0.0f
    if (n > 0) {
        size_t want = (n / 4 + 255) / 256;
        const size_t cap = (size_t)ctx->sm_count * 16;
        const unsigned grid = (unsigned)(want < 1 ? 1 : (want > cap ? cap : want));
        absmax_flat_kernel<<<grid, 256, 0, ctx->stream>>>(w, n, reinterpret_cast<unsigned int *>(amax_dev));
        ctx->launches += 1;
    }
    SHREWQ_CUDA_TRY(ctx, cudaGetLastError());
    return SHREWQ_OK;
}

int launch_quantize_given_amax(shrewq_ctx *ctx, const float *w, size_t n, const float *amax_dev, int8_t *q,
                               double *scale) {
    int rc = ensure_scratch(ctx, 256);
    if (rc != SHREWQ_OK) return rc;
    TensorParams *tp = reinterpret_cast<TensorParams *>(reinterpret_cast<char *>(ctx->scratch) + 64);
    // n = 1 here: the scale always derives from the supplied amax, also for an empty shard (an
    // all-empty tensor has amax 0, which gives the same scale 1.0 as the reference's empty case)
    finalize_tensor_scale_kernel<<<1, 1, 0, ctx->stream>>>(reinterpret_cast<const unsigned int *>(amax_dev), 1, scale, tp);
    ctx->launches += 1;
    if (n > 0) {
        size_t want = (n / 4 + 255) / 256;
        const size_t cap = (size_t)ctx->sm_count * 16;
        const unsigned grid = (unsigned)(want < 1 ? 1 : (want > cap ? cap : want));
        quantize_flat_kernel<<<grid, 256, 0, ctx->stream>>>(w, n, tp, q);
        ctx->launches += 1;
    }
    SHREWQ_CUDA_TRY(ctx, cudaGetLastError());
    return SHREWQ_OK;
}

int launch_dequantize(shrewq_ctx *ctx, const int8_t *q, const double *scales, size_t rows,
                      size_t cols, int granularity, int out_dtype, void *out) {
    const size_t n = rows * cols;
    if (n == 0) return SHREWQ_OK;
    const int per_channel = granularity == SHREWQ_PER_CHANNEL;
    const int vec_ok = (cols % 4 == 0) && ((reinterpret_cast<uintptr_t>(q) & 3) == 0) &&
                       ((reinterpret_cast<uintptr_t>(out) & 15) == 0);
    size_t want = ((vec_ok ? n / 4 : n) + 255) / 256;
    const size_t cap = (size_t)ctx->sm_count * 32;
    unsigned grid = (unsigned)(want < 1 ? 1 : (want > cap ? cap : want));
    if (out_dtype == SHREWQ_F32)
        dequantize_kernel<float><<<grid, 256, 0, ctx->stream>>>(q, scales, rows, cols, per_channel,
                                                                 static_cast<float *>(out), vec_ok);
    else
        dequantize_kernel<uint16_t><<<grid, 256, 0, ctx->stream>>>(q, scales, rows, cols, per_channel,
                                                                    static_cast<uint16_t *>(out), vec_ok);
    ctx->launches += 1;
    SHREWQ_CUDA_TRY(ctx, cudaGetLastError());
    return SHREWQ_OK;
}

int launch_split_f32(shrewq_ctx *ctx, const float *x, size_t n, void *hi_bf16, void *lo_bf16) {
    if (n == 0) return SHREWQ_OK;
    size_t want = (n + 255) / 256;
    const size_t cap = (size_t)ctx->sm_count * 32;
    split_f32_kernel<<<(unsigned)(want > cap ? cap : want), 256, 0, ctx->stream>>>(
        x, n, static_cast<__nv_bfloat16 *>(hi_bf16), static_cast<__nv_bfloat16 *>(lo_bf16));
    ctx->launches += 1;
    SHREWQ_CUDA_TRY(ctx, cudaGetLastError());
    return SHREWQ_OK;
}

int launch_scales_to_f32(shrewq_ctx *ctx, const double *scales, int granularity, size_t n, float *out) {
    if (n == 0) return SHREWQ_OK;
    scales_to_f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(
        scales, granularity == SHREWQ_PER_CHANNEL, n, out);
    ctx->launches += 1;
    SHREWQ_CUDA_TRY(ctx, cudaGetLastError());
    return SHREWQ_OK;
}

}  // namespace shrewq
