// CPU run of the kernels for the other quantization modes (shrew_b200/csrc/quantize_modes_kernels.cuh)
// and of the activation rescale kernel (activation_f16.cuh) under the CUDA stand-in.
// TEST INFRASTRUCTURE ONLY; see cuda_shim.h.
#include "cuda_shim.h"
#include "../../shrew_b200/csrc/quantize_modes_kernels.cuh"
#include "../../shrew_b200/csrc/activation_f16.cuh"

using namespace shrewq;

namespace {
template <typename T>
int quantize_any_t(const T *w, size_t rows, size_t cols, int per_channel, int bits, int mode, unsigned grid, int8_t *q,
                   double *scales, double *zps) {
    const size_t n = rows * cols;
    if (per_channel) {
        if (rows == 0) return 0;
        emu::launch(std::min<unsigned>(grid, (unsigned)rows), 256,
                    [&] { quantize_rows_ex_kernel<T>(w, rows, cols, bits, mode, q, scales, zps); });
        return 0;
    }
    alignas(16) unsigned char scratch[256] = {0};
    TensorWords *t = reinterpret_cast<TensorWords *>(scratch);
    emu::launch(1, 1, [&] { init_words_kernel(t); });
    if (n > 0) emu::launch(grid, 256, [&] { extrema_flat_kernel<T>(w, n, t); });
    emu::launch(1, 1, [&] { finalize_ex_kernel(t, n, bits, mode, scales, zps); });
    if (n > 0) emu::launch(grid, 256, [&] { quantize_flat_ex_kernel<T>(w, n, t, q); });
    return 0;
}
}  // namespace

// w_dtype: 0 f32, 1 bf16 bits, 2 f16 bits, 3 f64 (the codes of include/shrewq.h)
extern "C" int emu_quantize_any(const void *w, int w_dtype, size_t rows, size_t cols, int per_channel, int bits, int mode,
                                unsigned grid, int8_t *q, double *scales, double *zps) {
    switch (w_dtype) {
        case SHREWQ_F32: return quantize_any_t(static_cast<const float *>(w), rows, cols, per_channel, bits, mode, grid, q, scales, zps);
        case SHREWQ_BF16: return quantize_any_t(static_cast<const __nv_bfloat16 *>(w), rows, cols, per_channel, bits, mode, grid, q, scales, zps);
        case SHREWQ_F16: return quantize_any_t(static_cast<const __half *>(w), rows, cols, per_channel, bits, mode, grid, q, scales, zps);
        case SHREWQ_F64: return quantize_any_t(static_cast<const double *>(w), rows, cols, per_channel, bits, mode, grid, q, scales, zps);
        default: return -1;
    }
}

extern "C" int emu_quantize_ex(const float *w, size_t rows, size_t cols, int per_channel, int bits, int mode, unsigned grid,
                               int8_t *q, double *scales, double *zps) {
    return quantize_any_t(w, rows, cols, per_channel, bits, mode, grid, q, scales, zps);
}

// out_dtype: 0 f32, 1 bf16 bits, 2 f16 bits, 3 f64; zps may be null
extern "C" int emu_dequantize_any(const int8_t *q, const double *scales, const double *zps, size_t rows, size_t cols,
                                  int per_channel, int out_dtype, unsigned grid, void *out) {
    if (rows * cols == 0) return 0;
    switch (out_dtype) {
        case SHREWQ_F32: emu::launch(grid, 256, [&] { dequantize_ex_kernel<float>(q, scales, zps, rows, cols, per_channel, static_cast<float *>(out)); }); break;
        case SHREWQ_BF16: emu::launch(grid, 256, [&] { dequantize_ex_kernel<uint16_t>(q, scales, zps, rows, cols, per_channel, static_cast<uint16_t *>(out)); }); break;
        case SHREWQ_F16: emu::launch(grid, 256, [&] { dequantize_ex_kernel<__half>(q, scales, zps, rows, cols, per_channel, static_cast<__half *>(out)); }); break;
        case SHREWQ_F64: emu::launch(grid, 256, [&] { dequantize_ex_kernel<double>(q, scales, zps, rows, cols, per_channel, static_cast<double *>(out)); }); break;
        default: return -1;
    }
    return 0;
}

extern "C" int emu_dequantize_ex(const int8_t *q, const double *scales, const double *zps, size_t rows, size_t cols,
                                 int per_channel, int bf16, unsigned grid, void *out) {
    return emu_dequantize_any(q, scales, zps, rows, cols, per_channel, bf16 ? SHREWQ_BF16 : SHREWQ_F32, grid, out);
}

extern "C" int emu_scale_zp_to_f32(const double *scales, const double *zps, int per_channel, size_t n, float *out) {
    if (n) emu::launch((unsigned)((n + 255) / 256), 256, [&] { scale_zp_to_f32_kernel(scales, zps, per_channel, n, out); });
    return 0;
}

extern "C" int emu_row_sums(const void *x, int bf16, size_t M, size_t K, float *sums) {
    if (M == 0) return 0;
    if (bf16)
        emu::launch((unsigned)M, 256, [&] { row_sums_kernel<__nv_bfloat16>(static_cast<const __nv_bfloat16 *>(x), K, sums); });
    else
        emu::launch((unsigned)M, 256, [&] { row_sums_kernel<float>(static_cast<const float *>(x), K, sums); });
    return 0;
}

extern "C" int emu_zero_point_fix(const float *acc, const float *czp, const float *xsum, size_t M, size_t N, size_t ldy,
                                  int relu, int bf16, unsigned grid, void *y) {
    if (M * N == 0) return 0;
    if (bf16)
        emu::launch(grid, 256, [&] { zero_point_fix_kernel<__nv_bfloat16>(acc, czp, xsum, M, N, ldy, relu, static_cast<__nv_bfloat16 *>(y)); });
    else
        emu::launch(grid, 256, [&] { zero_point_fix_kernel<float>(acc, czp, xsum, M, N, ldy, relu, static_cast<float *>(y)); });
    return 0;
}

extern "C" int emu_x_to_f16(const void *x_bf16, size_t M, int K, void *x16, int *shift) {
    if (M) emu::launch((unsigned)M, 256, [&] {
        x_to_f16_kernel(static_cast<const __nv_bfloat16 *>(x_bf16), static_cast<__half *>(x16), shift, K);
    });
    return 0;
}

extern "C" int emu_pack_int4(const int8_t *q, size_t n_pairs, unsigned grid, uint8_t *out) {
    if (n_pairs) emu::launch(grid, 256, [&] { pack_int4_kernel(q, n_pairs, out); });
    return 0;
}

