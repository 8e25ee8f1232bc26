// CPU run of the INT8 symmetric quantize / dequantize kernels (shrew_b200/csrc/quantize_kernels.cuh)
// under the CUDA stand-in.  TEST INFRASTRUCTURE ONLY; see cuda_shim.h.
#include "cuda_shim.h"
struct uint2 { unsigned x, y; };
#include "../../shrew_b200/csrc/quantize_kernels.cuh"
#include "../../shrew_b200/csrc/quantize_batch_kernels.cuh"

using namespace shrewq;

namespace {
template <int GROUP, int NV>
void rows_reg(const float *w, size_t rows, size_t cols, int8_t *q, double *scales) {
    constexpr int THREADS = GROUP >= 256 ? GROUP : 256;
    constexpr int ROWS_PER_CTA = THREADS / GROUP;
    const unsigned grid = (unsigned)((rows + ROWS_PER_CTA - 1) / ROWS_PER_CTA);
    emu::launch(grid, THREADS, [&] { quantize_rows_reg_kernel<GROUP, NV>(w, rows, cols, q, scales); });
}
}  // namespace

// variant: 0 = two-pass generic kernel; 1..9 = register-tile kernels in the order of the launcher's
// table (32x1, 32x2, 32x4, 32x8, 256x2, 256x4, 256x8, 512x8, 1024x8).  Returns -1 when the variant
// cannot take the shape (the launcher would not choose it either).
extern "C" int emu_quantize_rows(const float *w, size_t rows, size_t cols, int variant, int8_t *q, double *scales) {
    if (rows == 0) return 0;
    static const int cap[10] = {0, 128, 256, 512, 1024, 2048, 4096, 8192, 16384, 32768};
    if (variant == 0) {
        const unsigned grid = (unsigned)std::min<size_t>(rows, 5);  // fewer blocks than rows: the row loop runs
        emu::launch(grid, 256, [&] { quantize_rows_generic_kernel(w, rows, cols, q, scales); });
        return 0;
    }
    const bool vec = (cols % 4 == 0) && ((reinterpret_cast<uintptr_t>(w) & 15) == 0) && ((reinterpret_cast<uintptr_t>(q) & 3) == 0) && cols >= 32;
    if (variant < 1 || variant > 9 || !vec || cols > (size_t)cap[variant]) return -1;
    switch (variant) {
        case 1: rows_reg<32, 1>(w, rows, cols, q, scales); break;
        case 2: rows_reg<32, 2>(w, rows, cols, q, scales); break;
        case 3: rows_reg<32, 4>(w, rows, cols, q, scales); break;
        case 4: rows_reg<32, 8>(w, rows, cols, q, scales); break;
        case 5: rows_reg<256, 2>(w, rows, cols, q, scales); break;
        case 6: rows_reg<256, 4>(w, rows, cols, q, scales); break;
        case 7: rows_reg<256, 8>(w, rows, cols, q, scales); break;
        case 8: rows_reg<512, 8>(w, rows, cols, q, scales); break;
        default: rows_reg<1024, 8>(w, rows, cols, q, scales); break;
    }
    return 0;
}

// the per-tensor chain of launch_quantize: amax with atomics, parameters, element map
extern "C" int emu_quantize_tensor(const float *w, size_t n, unsigned grid, int8_t *q, double *scale) {
    alignas(16) unsigned char scratch[256] = {0};
    unsigned int *amax_bits = reinterpret_cast<unsigned int *>(scratch);
    TensorParams *tp = reinterpret_cast<TensorParams *>(scratch + 64);
    if (n > 0) emu::launch(grid, 256, [&] { absmax_flat_kernel(w, n, amax_bits); });
    emu::launch(1, 1, [&] { finalize_tensor_scale_kernel(amax_bits, n, scale, tp); });
    if (n > 0) emu::launch(grid, 256, [&] { quantize_flat_kernel(w, n, tp, q); });
    return 0;
}

// a shard quantized with a supplied amax (launch_quantize_given_amax)
extern "C" int emu_quantize_given_amax(const float *w, size_t n, const float *amax, unsigned grid, int8_t *q, double *scale) {
    alignas(16) unsigned char scratch[256] = {0};
    TensorParams *tp = reinterpret_cast<TensorParams *>(scratch + 64);
    emu::launch(1, 1, [&] { finalize_tensor_scale_kernel(reinterpret_cast<const unsigned int *>(amax), 1, scale, tp); });
    if (n > 0) emu::launch(grid, 256, [&] { quantize_flat_kernel(w, n, tp, q); });
    return 0;
}

extern "C" int emu_absmax(const float *w, size_t n, unsigned grid, float *amax) {
    *amax = 0.0f;
    if (n > 0) emu::launch(grid, 256, [&] { absmax_flat_kernel(w, n, reinterpret_cast<unsigned int *>(amax)); });
    return 0;
}

extern "C" int emu_dequantize(const int8_t *q, const double *scales, size_t rows, size_t cols, int per_channel, int bf16,
                              int vec_ok, unsigned grid, void *out) {
    if (rows * cols == 0) return 0;
    if (vec_ok && (cols % 4 != 0 || (reinterpret_cast<uintptr_t>(q) & 3) || (reinterpret_cast<uintptr_t>(out) & 15))) return -1;
    if (bf16)
        emu::launch(grid, 256, [&] { dequantize_kernel<uint16_t>(q, scales, rows, cols, per_channel, static_cast<uint16_t *>(out), vec_ok); });
    else
        emu::launch(grid, 256, [&] { dequantize_kernel<float>(q, scales, rows, cols, per_channel, static_cast<float *>(out), vec_ok); });
    return 0;
}

// f32 activations -> bf16 hi + bf16 lo (the tensor-core route for f32 inputs)
extern "C" int emu_split_f32(const float *x, size_t n, unsigned grid, void *hi, void *lo) {
    if (n) emu::launch(grid, 256, [&] { split_f32_kernel(x, n, static_cast<__nv_bfloat16 *>(hi), static_cast<__nv_bfloat16 *>(lo)); });
    return 0;
}

// Many tensors per launch (launch_quantize_batch in shrew_b200/csrc/quantize_batch.cu): the same table,
// chunking and kernel sequence; `grid` stands for the launcher's block count (fewer blocks than work
// units makes the unit loop run).  items: n x {w, rows, cols, q, scales} as the C ABI's shrewq_quant_item.
struct EmuQuantItem {
    const float *w;
    size_t rows, cols;
    int8_t *q;
    double *scales;
};
extern "C" int emu_quantize_batch(const EmuQuantItem *items, size_t n_items, int per_channel, unsigned grid) {
    for (size_t first = 0; first < n_items; first += kBatchMax) {
        BatchTable t{};
        t.n = (int)std::min<size_t>(n_items - first, kBatchMax);
        unsigned long long units = 0;
        for (int i = 0; i < t.n; ++i) {
            const EmuQuantItem &s = items[first + i];
            t.it[i] = BatchItem{s.w, s.q, s.scales, s.rows, s.cols, (unsigned int)units, 0};
            const unsigned long long n = (unsigned long long)s.rows * s.cols;
            units += per_channel ? (unsigned long long)s.rows : (n + kBatchSegment - 1) / kBatchSegment;
        }
        t.total_units = (unsigned int)units;
        if (per_channel) {
            if (units > 0) emu::launch(grid, kBatchWarps * 32, [&] { quantize_batch_rows_kernel(t); });
        } else {
            alignas(16) unsigned char scratch[4096] = {0};
            unsigned int *amax_bits = reinterpret_cast<unsigned int *>(scratch);
            TensorParams *tp = reinterpret_cast<TensorParams *>(scratch + 256);
            if (units > 0) emu::launch(grid, kBatchWarps * 32, [&] { absmax_batch_kernel(t, amax_bits); });
            emu::launch(1, kBatchMax, [&] { finalize_batch_kernel(t, amax_bits, tp); });
            if (units > 0) emu::launch(grid, kBatchWarps * 32, [&] { quantize_batch_flat_kernel(t, tp); });
        }
    }
    return 0;
}
