// Launchers of the kernels for the reference's other quantization modes (device code, status and
// description: quantize_modes_kernels.cuh).
#include "common.cuh"
#include <cuda_fp16.h>

#include "quantize_modes_kernels.cuh"

namespace shrewq {
namespace {

unsigned grid_for(const shrewq_ctx *ctx, size_t items) {
    size_t want = (items + 255) / 256;
    const size_t cap = (size_t)ctx->sm_count * 32;
    return (unsigned)(want < 1 ? 1 : (want > cap ? cap : want));
}

}  // namespace

namespace {
template <typename T>
int quantize_any_t(shrewq_ctx *ctx, const T *w, size_t rows, size_t cols, int granularity, int bits, int mode, int8_t *q,
                   double *scales, double *zps) {
    const size_t n = rows * cols;
    if (granularity == SHREWQ_PER_CHANNEL) {
        if (rows == 0) return SHREWQ_OK;
        const unsigned grid = (unsigned)(rows < (size_t)ctx->sm_count * 32 ? rows : (size_t)ctx->sm_count * 32);
        quantize_rows_ex_kernel<T><<<grid, 256, 0, ctx->stream>>>(w, rows, cols, bits, mode, q, scales, zps);
        ctx->launches += 1;
    } else {
        // scratch: [1024, 1024 + sizeof(TensorWords)) of the quantizer's 4 KiB
        int rc = ensure_scratch(ctx, 4096);
        if (rc != SHREWQ_OK) return rc;
        TensorWords *t = reinterpret_cast<TensorWords *>(static_cast<char *>(ctx->scratch) + 1024);
        init_words_kernel<<<1, 1, 0, ctx->stream>>>(t);
        if (n > 0) extrema_flat_kernel<T><<<grid_for(ctx, n), 256, 0, ctx->stream>>>(w, n, t);
        finalize_ex_kernel<<<1, 1, 0, ctx->stream>>>(t, n, bits, mode, scales, zps);
        if (n > 0) quantize_flat_ex_kernel<T><<<grid_for(ctx, n), 256, 0, ctx->stream>>>(w, n, t, q);
        ctx->launches += n > 0 ? 4 : 2;
    }
    SHREWQ_CUDA_TRY(ctx, cudaGetLastError());
    return SHREWQ_OK;
}
}  // namespace

// w_dtype: SHREWQ_F32, SHREWQ_BF16, SHREWQ_F16 or SHREWQ_F64 (the storage type of the tensor)
int launch_quantize_any(shrewq_ctx *ctx, const void *w, int w_dtype, size_t rows, size_t cols, int granularity, int bits,
                        int mode, int8_t *q, double *scales, double *zps) {
    switch (w_dtype) {
        case SHREWQ_F32: return quantize_any_t(ctx, static_cast<const float *>(w), rows, cols, granularity, bits, mode, q, scales, zps);
        case SHREWQ_BF16: return quantize_any_t(ctx, static_cast<const __nv_bfloat16 *>(w), rows, cols, granularity, bits, mode, q, scales, zps);
        case SHREWQ_F16: return quantize_any_t(ctx, static_cast<const __half *>(w), rows, cols, granularity, bits, mode, q, scales, zps);
        case SHREWQ_F64: return quantize_any_t(ctx, static_cast<const double *>(w), rows, cols, granularity, bits, mode, q, scales, zps);
        default: return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "quantize: unknown storage type %d", w_dtype);
    }
}

int launch_quantize_ex(shrewq_ctx *ctx, const float *w, size_t rows, size_t cols, int granularity, int bits, int mode,
                       int8_t *q, double *scales, double *zps) {
    return quantize_any_t(ctx, w, rows, cols, granularity, bits, mode, q, scales, zps);
}

// zps may be null (zero points of 0.0); out_dtype: SHREWQ_F32, SHREWQ_BF16, SHREWQ_F16 or SHREWQ_F64
int launch_dequantize_ex(shrewq_ctx *ctx, const int8_t *q, const double *scales, const double *zps, size_t rows,
                         size_t cols, int granularity, int out_dtype, void *out) {
    const size_t n = rows * cols;
    if (n == 0) return SHREWQ_OK;
    const int pc = granularity == SHREWQ_PER_CHANNEL;
    const unsigned grid = grid_for(ctx, n);
    switch (out_dtype) {
        case SHREWQ_F32: dequantize_ex_kernel<float><<<grid, 256, 0, ctx->stream>>>(q, scales, zps, rows, cols, pc, static_cast<float *>(out)); break;
        case SHREWQ_BF16: dequantize_ex_kernel<uint16_t><<<grid, 256, 0, ctx->stream>>>(q, scales, zps, rows, cols, pc, static_cast<uint16_t *>(out)); break;
        case SHREWQ_F16: dequantize_ex_kernel<__half><<<grid, 256, 0, ctx->stream>>>(q, scales, zps, rows, cols, pc, static_cast<__half *>(out)); break;
        case SHREWQ_F64: dequantize_ex_kernel<double><<<grid, 256, 0, ctx->stream>>>(q, scales, zps, rows, cols, pc, static_cast<double *>(out)); break;
        default: return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "dequantize: unknown output type %d", out_dtype);
    }
    ctx->launches += 1;
    SHREWQ_CUDA_TRY(ctx, cudaGetLastError());
    return SHREWQ_OK;
}

int launch_pack_int4(shrewq_ctx *ctx, const int8_t *q, size_t n_pairs, uint8_t *packed) {
    if (n_pairs == 0) return SHREWQ_OK;
    pack_int4_kernel<<<grid_for(ctx, n_pairs), 256, 0, ctx->stream>>>(q, n_pairs, packed);
    ctx->launches += 1;
    SHREWQ_CUDA_TRY(ctx, cudaGetLastError());
    return SHREWQ_OK;
}

int launch_scale_zp_to_f32(shrewq_ctx *ctx, const double *scales, const double *zps, int granularity, size_t n, float *out) {
    if (n == 0) return SHREWQ_OK;
    scale_zp_to_f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(scales, zps, granularity == SHREWQ_PER_CHANNEL,
                                                                                 n, out);
    ctx->launches += 1;
    SHREWQ_CUDA_TRY(ctx, cudaGetLastError());
    return SHREWQ_OK;
}

int launch_row_sums(shrewq_ctx *ctx, const void *x, int x_dtype, size_t M, size_t K, float *sums) {
    if (M == 0) return SHREWQ_OK;
    if (x_dtype == SHREWQ_F32)
        row_sums_kernel<float><<<(unsigned)M, 256, 0, ctx->stream>>>(static_cast<const float *>(x), K, sums);
    else
        row_sums_kernel<__nv_bfloat16><<<(unsigned)M, 256, 0, ctx->stream>>>(static_cast<const __nv_bfloat16 *>(x), K, sums);
    ctx->launches += 1;
    SHREWQ_CUDA_TRY(ctx, cudaGetLastError());
    return SHREWQ_OK;
}

int launch_zero_point_fix(shrewq_ctx *ctx, const float *acc, const float *czp, const float *xsum, size_t M, size_t N,
                          size_t ldy, int relu, int y_dtype, void *y) {
    if (M * N == 0) return SHREWQ_OK;
    if (y_dtype == SHREWQ_F32)
        zero_point_fix_kernel<float><<<grid_for(ctx, M * N), 256, 0, ctx->stream>>>(acc, czp, xsum, M, N, ldy, relu,
                                                                                  static_cast<float *>(y));
    else
        zero_point_fix_kernel<__nv_bfloat16><<<grid_for(ctx, M * N), 256, 0, ctx->stream>>>(
            acc, czp, xsum, M, N, ldy, relu, static_cast<__nv_bfloat16 *>(y));
    ctx->launches += 1;
    SHREWQ_CUDA_TRY(ctx, cudaGetLastError());
    return SHREWQ_OK;
}

}  // namespace shrewq
