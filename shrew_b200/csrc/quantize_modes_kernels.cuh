// Quantize / dequantize in the reference's other modes: asymmetric INT8, INT4 symmetric and
// asymmetric (one code per byte, as the reference stores them), sm_100a.
//
// STATUS: compiled, checked against the CPU restatement only by reading; NOT yet run on a GPU.
// Reachable only when the environment sets SHREWQ_EXPERIMENTAL_MODES=1; otherwise the entry
// points answer SHREWQ_ERR_UNSUPPORTED for anything but INT8 symmetric.
//
// Reference semantics (crates/shrew/src/quantize.rs), all in f64 on a widened copy:
//   qmax = 127 | 7;  qmin = -127 | -7 (symmetric), -128 | -8 (asymmetric)          (:124-139)
//   symmetric : scale = amax < 1e-30 ? 1 : amax / qmax,  zp = 0                     (:349-352)
//   asymmetric: range = max - min;  scale = range < 1e-30 ? 1 : range / (qmax - qmin);
//               zp = round(qmin - min / scale)                                      (:353-364)
//   inv  = |scale| < 1e-30 ? 0 : 1 / scale                                          (:236-240)
//   code = clamp(round_half_away(v * inv + zp), qmin, qmax) as i8   (NaN -> 0)      (:244-250)
//   back = (code - zp) * scale                                                      (:262-266)
// Correctness first: the element map runs the reference's f64 operations one for one (no f32
// shortcut as in the INT8 symmetric kernels); min, max and amax of f32 values are exact in f32.
// Per-channel rows are read twice (the second pass normally from L2); per-tensor takes three
// launches (min/max with atomics on order-preserving integer keys, parameters, element map).
//
// This header holds the device code only (no launch syntax, no runtime calls), so that it also
// compiles as plain C++ against a small CUDA stand-in: the CPU tests run these kernels thread by
// thread and compare them with the golden vectors (tests/cpu_emu/).
#pragma once

#include "../../include/shrewq.h"
#ifndef SHREWQ_CPU_EMU
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#endif

namespace shrewq {
namespace {

struct GroupParams {
    double scale, zp, inv, qmin, qmax;
};

__device__ __forceinline__ double qmax_of(int bits) { return bits == 4 ? 7.0 : 127.0; }
__device__ __forceinline__ double qmin_of(int bits, int mode) {
    if (bits == 4) return mode == SHREWQ_ASYMMETRIC ? -8.0 : -7.0;
    return mode == SHREWQ_ASYMMETRIC ? -128.0 : -127.0;
}

__device__ __forceinline__ double round_half_away(double t) {
    if (t != t) return t;
    double r = trunc(t);
    if (fabs(t - r) >= 0.5) r += copysign(1.0, t);  // t - r is exact; false for +-Inf (NaN compare)
    return copysign(r, t);                          // round(-0.3) is -0.0, as f64::round
}

// compute_scale_zp for a group of n elements whose extrema are lo / hi / amax
__device__ __forceinline__ GroupParams make_group(float lo, float hi, float amax, size_t n, int bits, int mode) {
    GroupParams p;
    p.qmin = qmin_of(bits, mode);
    p.qmax = qmax_of(bits);
    if (n == 0) {
        p.scale = 1.0;
        p.zp = 0.0;
    } else if (mode != SHREWQ_ASYMMETRIC) {
        const double a = (double)amax;
        p.scale = a < 1e-30 ? 1.0 : a / p.qmax;
        p.zp = 0.0;
    } else {
        const double mn = (double)lo, mx = (double)hi;
        const double range = mx - mn;
        p.scale = range < 1e-30 ? 1.0 : range / (p.qmax - p.qmin);
        p.zp = round_half_away(p.qmin - mn / p.scale);
    }
    p.inv = fabs(p.scale) < 1e-30 ? 0.0 : 1.0 / p.scale;
    return p;
}

__device__ __forceinline__ int quant_ex(float v, const GroupParams &p) {
    const double t = round_half_away(__dadd_rn(__dmul_rn((double)v, p.inv), p.zp));
    if (t != t) return 0;  // NaN as i8 == 0
    return (int)fmin(fmax(t, p.qmin), p.qmax);
}

__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}

// Block-wide extrema of (lo, hi, amax); every thread of the 256-thread CTA gets the result.
__device__ __forceinline__ void block_extrema(float &lo, float &hi, float &amax) {
    __shared__ float s_lo[8], s_hi[8], s_am[8];
    lo = warp_min(lo);
    hi = warp_max(hi);
    amax = warp_max(amax);
    __syncthreads();  // the arrays may still be read from a previous call
    if ((threadIdx.x & 31) == 0) {
        s_lo[threadIdx.x >> 5] = lo;
        s_hi[threadIdx.x >> 5] = hi;
        s_am[threadIdx.x >> 5] = amax;
    }
    __syncthreads();
    lo = s_lo[0];
    hi = s_hi[0];
    amax = s_am[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) {
        lo = fminf(lo, s_lo[i]);      // fminf / fmaxf drop a NaN operand, as f64::min / f64::max do
        hi = fmaxf(hi, s_hi[i]);
        amax = fmaxf(amax, s_am[i]);
    }
}

// ---- per-channel: one CTA per row, two passes ---------------------------------------------------
__global__ void __launch_bounds__(256)
quantize_rows_ex_kernel(const float *__restrict__ w, size_t rows, size_t cols, int bits, int mode,
                        int8_t *__restrict__ q, double *__restrict__ scales, double *__restrict__ zps) {
    for (size_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const float *src = w + row * cols;
        float lo = INFINITY, hi = -INFINITY, amax = 0.0f;
        for (size_t c = threadIdx.x; c < cols; c += 256) {
            const float v = src[c];
            lo = fminf(lo, v);
            hi = fmaxf(hi, v);
            amax = fmaxf(amax, fabsf(v));
        }
        block_extrema(lo, hi, amax);
        const GroupParams p = make_group(lo, hi, amax, cols, bits, mode);  // every thread: same inputs, same result
        if (threadIdx.x == 0) {
            scales[row] = p.scale;
            zps[row] = p.zp;
        }
        int8_t *dst = q + row * cols;
        for (size_t c = threadIdx.x; c < cols; c += 256) dst[c] = (int8_t)quant_ex(src[c], p);
    }
}

// ---- per-tensor ---------------------------------------------------------------------------------
// Floats order like these integer keys (negative floats reversed below the positive ones), so
// atomicMin / atomicMax on the keys are a float min / max.  NaN never reaches a key.
__device__ __forceinline__ unsigned int key_of(float f) {
    const unsigned int b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float float_of(unsigned int k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k);
}

struct TensorWords {
    unsigned int lo_key, hi_key, amax_bits, pad;
    GroupParams p;
};

__global__ void init_words_kernel(TensorWords *t) {
    t->lo_key = key_of(INFINITY);
    t->hi_key = key_of(-INFINITY);
    t->amax_bits = 0u;
}

__global__ void __launch_bounds__(256)
extrema_flat_kernel(const float *__restrict__ w, size_t n, TensorWords *t) {
    float lo = INFINITY, hi = -INFINITY, amax = 0.0f;
    const size_t stride = (size_t)gridDim.x * 256;
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += stride) {
        const float v = w[i];
        lo = fminf(lo, v);
        hi = fmaxf(hi, v);
        amax = fmaxf(amax, fabsf(v));
    }
    block_extrema(lo, hi, amax);
    if (threadIdx.x == 0) {
        atomicMin(&t->lo_key, key_of(lo));
        atomicMax(&t->hi_key, key_of(hi));
        atomicMax(&t->amax_bits, __float_as_uint(amax));  // non-negative floats order like their bits
    }
}

__global__ void finalize_ex_kernel(TensorWords *t, size_t n, int bits, int mode, double *scales, double *zps) {
    const GroupParams p = make_group(float_of(t->lo_key), float_of(t->hi_key), __uint_as_float(t->amax_bits), n, bits, mode);
    t->p = p;
    scales[0] = p.scale;
    zps[0] = p.zp;
}

__global__ void __launch_bounds__(256)
quantize_flat_ex_kernel(const float *__restrict__ w, size_t n, const TensorWords *__restrict__ t, int8_t *__restrict__ q) {
    const GroupParams p = t->p;
    const size_t stride = (size_t)gridDim.x * 256;
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += stride) q[i] = (int8_t)quant_ex(w[i], p);
}

// ---- dequantize with zero points ------------------------------------------------------------------
__device__ __forceinline__ uint16_t f64_to_bf16_rne(double v) {
    if (v != v) return 0x7FC0;
    float f = __double2float_rz(v);
    uint32_t b = __float_as_uint(f);
    if ((double)f != v && !isinf(f)) b |= 1u;  // sticky bit below bf16's ulp: a single rounding overall
    if (isinf(v)) return (uint16_t)(b >> 16);
    return (uint16_t)((b + 0x7FFFu + ((b >> 16) & 1u)) >> 16);
}

template <typename OutT>
__global__ void __launch_bounds__(256)
dequantize_ex_kernel(const int8_t *__restrict__ q, const double *__restrict__ scales, const double *__restrict__ zps,
                     size_t rows, size_t cols, int per_channel, OutT *__restrict__ out) {
    const size_t n = rows * cols;
    const size_t stride = (size_t)gridDim.x * 256;
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += stride) {
        const size_t g = per_channel ? i / cols : 0;
        const double v = __dmul_rn(__dsub_rn((double)q[i], zps[g]), scales[g]);
        if constexpr (sizeof(OutT) == 4) out[i] = (float)v;
        else out[i] = f64_to_bf16_rne(v);
    }
}

// ---- forward support: y -= (scale * zp)[n] * sum_k x[m,k] ----------------------------------------
__global__ void scale_zp_to_f32_kernel(const double *__restrict__ scales, const double *__restrict__ zps,
                                       int per_channel, size_t n, float *__restrict__ out) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = (float)(per_channel ? scales[i] * zps[i] : scales[0] * zps[0]);
}

template <typename XT>
__global__ void __launch_bounds__(256)
row_sums_kernel(const XT *__restrict__ x, size_t K, float *__restrict__ sums) {
    const XT *row = x + (size_t)blockIdx.x * K;
    double acc = 0.0;  // f64 partial sums: the correction term must not add error of its own
    for (size_t k = threadIdx.x; k < K; k += 256) {
        if constexpr (sizeof(XT) == 4) acc += (double)row[k];
        else acc += (double)__bfloat162float(row[k]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
    __shared__ double s_part[8];
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        double s = 0.0;
        for (int i = 0; i < 8; ++i) s += s_part[i];
        sums[blockIdx.x] = (float)s;
    }
}

template <typename YT>
__global__ void __launch_bounds__(256)
zero_point_fix_kernel(const float *__restrict__ acc, const float *__restrict__ czp, const float *__restrict__ xsum,
                      size_t M, size_t N, size_t ldy, int relu, YT *__restrict__ y) {
    const size_t total = M * N;
    const size_t stride = (size_t)gridDim.x * 256;
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < total; i += stride) {
        const size_t m = i / N, n = i % N;
        float o = acc[i] - czp[n] * xsum[m];
        if (relu) o = fmaxf(o, 0.0f);
        if constexpr (sizeof(YT) == 4) y[m * ldy + n] = o;
        else y[m * ldy + n] = __float2bfloat16_rn(o);
    }
}

}  // namespace
}  // namespace shrewq
