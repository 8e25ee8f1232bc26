// INT8 symmetric quantization of MANY tensors per launch (sm_100a).
//
// quantize_named_parameters (crates/shrew/src/quantize.rs:500-516) walks a module and quantizes every
// parameter of rank >= 2, one tensor after the other.  A small model is dozens of small tensors (a
// 4-block GPT with 256-wide layers: 25 tensors, 16 MB in all), for which one launch per tensor costs
// more than the data: ~5 us of launch against well under 1 us of HBM time for a 256 x 256 matrix.
// Here the tensors of a model travel as a table in the kernel's parameters (no device-side table, no
// copy, so the call can sit in a CUDA graph) and one grid covers all of them.
//
// Work unit, per-channel: one row of one tensor, owned by one warp (two passes over the row: amax, then
// the element map; the second read hits L1 / L2).  Per-tensor: one 2048-element segment of the flattened
// tensor, in three kernels (segment amax -> atomic max per tensor; scale per tensor; element map).
// A unit index is mapped to its tensor by binary search over the table's prefix sums.
//
// The arithmetic is that of quantize_kernels.cuh (make_params, quant_one), so codes and scales are the
// same bits as the one-tensor kernels produce, which are the reference's.
//
// Device code only (no launch syntax, no runtime calls): it also compiles as plain C++ against the CUDA
// stand-in of the CPU tests (tests/cpu_emu/).
#pragma once

#include "quantize_kernels.cuh"

namespace shrewq {
namespace {

constexpr int kBatchMax = 64;          // tensors per launch (the table must fit the 4 KB of kernel parameters)
constexpr int kBatchSegment = 2048;    // elements per per-tensor work unit
constexpr int kBatchWarps = 8;         // warps per CTA

struct BatchItem {
    const float *w;
    int8_t *q;
    double *scales;
    unsigned long long rows, cols;
    unsigned int unit_begin;  // first work unit of this tensor
    unsigned int pad;
};

struct BatchTable {
    int n;
    unsigned int total_units;
    BatchItem it[kBatchMax];
};
static_assert(sizeof(BatchTable) <= 4000, "the table travels as a kernel parameter");

// index of the tensor that owns work unit u (the last item with unit_begin <= u; items without units are
// skipped because a later item then has the same unit_begin)
__device__ __forceinline__ int batch_find(const BatchTable &t, unsigned int u) {
    int lo = 0, hi = t.n - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (t.it[mid].unit_begin <= u) lo = mid;
        else hi = mid - 1;
    }
    return lo;
}

// max |v| over n consecutive floats, by one warp (every lane returns the result)
__device__ __forceinline__ float warp_absmax(const float *src, size_t n, int lane) {
    float amax = 0.0f;
    const bool aligned = (reinterpret_cast<uintptr_t>(src) & 15) == 0;
    const size_t nvec = aligned ? (n >> 2) : 0;
    const float4 *s4 = reinterpret_cast<const float4 *>(src);
    for (size_t i = lane; i < nvec; i += 32) amax = fmaxf(amax, abs4max(__ldg(s4 + i)));
    for (size_t i = (nvec << 2) + lane; i < n; i += 32) amax = fmaxf(amax, fabsf(src[i]));
    return warp_max(amax);
}

// the element map over n consecutive floats, by one warp
__device__ __forceinline__ void warp_quantize(const float *src, int8_t *dst, size_t n, const RowParams &p, int lane) {
    const bool aligned = ((reinterpret_cast<uintptr_t>(src) & 15) == 0) && ((reinterpret_cast<uintptr_t>(dst) & 3) == 0);
    const size_t nvec = aligned ? (n >> 2) : 0;
    const float4 *s4 = reinterpret_cast<const float4 *>(src);
    uint32_t *d4 = reinterpret_cast<uint32_t *>(dst);
    for (size_t i = lane; i < nvec; i += 32) {
        const float4 v = __ldg(s4 + i);
        d4[i] = pack4(quant_one(v.x, p), quant_one(v.y, p), quant_one(v.z, p), quant_one(v.w, p));
    }
    for (size_t i = (nvec << 2) + lane; i < n; i += 32) dst[i] = (int8_t)quant_one(src[i], p);
}

// ---- per-channel: one warp per (tensor, row) ----------------------------------------------------------
__global__ void __launch_bounds__(kBatchWarps * 32)
quantize_batch_rows_kernel(const BatchTable t) {
    const int lane = threadIdx.x & 31;
    const unsigned int stride = gridDim.x * kBatchWarps;
    for (unsigned int u = blockIdx.x * kBatchWarps + (threadIdx.x >> 5); u < t.total_units; u += stride) {
        const BatchItem &it = t.it[batch_find(t, u)];
        const size_t row = u - it.unit_begin, cols = (size_t)it.cols;
        const float *src = it.w + row * cols;
        const float amax = warp_absmax(src, cols, lane);
        double scale;
        RowParams p;
        make_params(amax, &scale, &p);
        if (lane == 0) it.scales[row] = scale;
        warp_quantize(src, it.q + row * cols, cols, p, lane);
    }
}

// ---- per-tensor: segment amax, scale per tensor, element map --------------------------------------------
// amax_bits: one zero-initialised word per tensor (non-negative floats order like their bit patterns)
__global__ void __launch_bounds__(kBatchWarps * 32)
absmax_batch_kernel(const BatchTable t, unsigned int *amax_bits) {
    const int lane = threadIdx.x & 31;
    const unsigned int stride = gridDim.x * kBatchWarps;
    for (unsigned int u = blockIdx.x * kBatchWarps + (threadIdx.x >> 5); u < t.total_units; u += stride) {
        const int i = batch_find(t, u);
        const BatchItem &it = t.it[i];
        const size_t n = (size_t)it.rows * (size_t)it.cols, begin = (size_t)(u - it.unit_begin) * kBatchSegment;
        const size_t len = n - begin < (size_t)kBatchSegment ? n - begin : (size_t)kBatchSegment;
        const float m = warp_absmax(it.w + begin, len, lane);
        if (lane == 0) atomicMax(amax_bits + i, __float_as_uint(m));  // m is never NaN: fmaxf dropped them
    }
}

__global__ void finalize_batch_kernel(const BatchTable t, const unsigned int *amax_bits, TensorParams *tp) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= t.n) return;
    double scale;
    RowParams p;
    if (t.it[i].rows * t.it[i].cols == 0) {  // empty slice: (1.0, 0.0), quantize.rs:340-342
        scale = 1.0;
        p.inv64 = 1.0;
        p.inv32 = 1.0f;
        p.exact_only = 0;
    } else {
        make_params(__uint_as_float(amax_bits[i]), &scale, &p);
    }
    t.it[i].scales[0] = scale;
    tp[i].p = p;
}

__global__ void __launch_bounds__(kBatchWarps * 32)
quantize_batch_flat_kernel(const BatchTable t, const TensorParams *__restrict__ tp) {
    const int lane = threadIdx.x & 31;
    const unsigned int stride = gridDim.x * kBatchWarps;
    for (unsigned int u = blockIdx.x * kBatchWarps + (threadIdx.x >> 5); u < t.total_units; u += stride) {
        const int i = batch_find(t, u);
        const BatchItem &it = t.it[i];
        const size_t n = (size_t)it.rows * (size_t)it.cols, begin = (size_t)(u - it.unit_begin) * kBatchSegment;
        const size_t len = n - begin < (size_t)kBatchSegment ? n - begin : (size_t)kBatchSegment;
        const RowParams p = tp[i].p;
        warp_quantize(it.w + begin, it.q + begin, len, p, lane);
    }
}

}  // namespace
}  // namespace shrewq
