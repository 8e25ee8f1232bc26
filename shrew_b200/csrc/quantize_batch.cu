// Launcher of the many-tensors-per-launch quantizer (device code and its description:
// quantize_batch_kernels.cuh).
#include "common.cuh"
#include "quantize_batch_kernels.cuh"

namespace shrewq {

int launch_quantize_batch(shrewq_ctx *ctx, const shrewq_quant_item *items, size_t n_items, int granularity) {
    const bool per_channel = granularity == SHREWQ_PER_CHANNEL;
    for (size_t first = 0; first < n_items; first += kBatchMax) {
        BatchTable t{};
        t.n = (int)(n_items - first < (size_t)kBatchMax ? n_items - first : (size_t)kBatchMax);
        unsigned long long units = 0;
        for (int i = 0; i < t.n; ++i) {
            const shrewq_quant_item &s = items[first + i];
            BatchItem &d = t.it[i];
            d.w = s.w_dev;
            d.q = s.q_dev;
            d.scales = s.scales_dev;
            d.rows = s.rows;
            d.cols = s.cols;
            d.unit_begin = (unsigned int)units;
            const unsigned long long n = (unsigned long long)s.rows * s.cols;
            units += per_channel ? (unsigned long long)s.rows : (n + kBatchSegment - 1) / kBatchSegment;
            if (units > 0xFFFFFFFFull || s.rows > 0x7FFFFFFFull)
                return set_err(ctx, SHREWQ_ERR_UNSUPPORTED, "quantize_batch: too many rows or elements for one table; "
                                                            "quantize the large tensors one by one");
        }
        t.total_units = (unsigned int)units;
        const unsigned long long want = (units + kBatchWarps - 1) / kBatchWarps;
        const unsigned long long cap = (unsigned long long)ctx->sm_count * 16;
        const unsigned grid = (unsigned)(want < 1 ? 1 : (want > cap ? cap : want));
        if (per_channel) {
            if (units > 0) {
                quantize_batch_rows_kernel<<<grid, kBatchWarps * 32, 0, ctx->stream>>>(t);
                ctx->launches += 1;
            }
        } else {
            // scratch: one amax word per tensor at [0, 256), one TensorParams per tensor from 256
            static_assert(kBatchMax * sizeof(unsigned int) <= 256 && 256 + kBatchMax * sizeof(TensorParams) <= 4096,
                          "the quantizer's part of the context scratch is its first 4096 bytes");
            int rc = ensure_scratch(ctx, 4096);
            if (rc != SHREWQ_OK) return rc;
            unsigned int *amax_bits = reinterpret_cast<unsigned int *>(ctx->scratch);
            TensorParams *tp = reinterpret_cast<TensorParams *>(static_cast<char *>(ctx->scratch) + 256);
            SHREWQ_CUDA_TRY(ctx, cudaMemsetAsync(amax_bits, 0, 256, ctx->stream));
            if (units > 0) {
                absmax_batch_kernel<<<grid, kBatchWarps * 32, 0, ctx->stream>>>(t, amax_bits);
                ctx->launches += 1;
            }
            finalize_batch_kernel<<<1, kBatchMax, 0, ctx->stream>>>(t, amax_bits, tp);
            ctx->launches += 1;
            if (units > 0) {
                quantize_batch_flat_kernel<<<grid, kBatchWarps * 32, 0, ctx->stream>>>(t, tp);
                ctx->launches += 1;
            }
        }
        SHREWQ_CUDA_TRY(ctx, cudaGetLastError());
    }
    return SHREWQ_OK;
}

}  // namespace shrewq
