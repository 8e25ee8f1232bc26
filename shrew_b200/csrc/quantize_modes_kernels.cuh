// Quantize / dequantize in the reference's other modes: asymmetric INT8, INT4 symmetric and
// asymmetric (one code per byte, as the reference stores them), sm_100a.
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
#include <cuda_fp16.h>
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

// Tensor element -> f64, exactly (Tensor::to_f64_vec, quantize.rs:198): f32, f64, bf16 or f16 storage.
__device__ __forceinline__ double widen(float v) { return (double)v; }
__device__ __forceinline__ double widen(double v) { return v; }
__device__ __forceinline__ double widen(__nv_bfloat16 v) { return (double)__bfloat162float(v); }
__device__ __forceinline__ double widen(__half v) { return (double)__half2float(v); }

// compute_scale_zp for a group of n elements whose extrema are lo / hi / amax (f64: exact for every
// storage type)
__device__ __forceinline__ GroupParams make_group(double lo, double hi, double amax, size_t n, int bits, int mode) {
    GroupParams p;
    p.qmin = qmin_of(bits, mode);
    p.qmax = qmax_of(bits);
    if (n == 0) {
        p.scale = 1.0;
        p.zp = 0.0;
    } else if (mode != SHREWQ_ASYMMETRIC) {
        p.scale = amax < 1e-30 ? 1.0 : amax / p.qmax;
        p.zp = 0.0;
    } else {
        const double range = hi - lo;
        p.scale = range < 1e-30 ? 1.0 : range / (p.qmax - p.qmin);
        p.zp = round_half_away(p.qmin - lo / p.scale);
    }
    p.inv = fabs(p.scale) < 1e-30 ? 0.0 : 1.0 / p.scale;
    return p;
}

__device__ __forceinline__ int quant_ex(double v, const GroupParams &p) {
    const double t = round_half_away(__dadd_rn(__dmul_rn(v, p.inv), p.zp));
    if (t != t) return 0;  // NaN as i8 == 0
    return (int)fmin(fmax(t, p.qmin), p.qmax);
}

__device__ __forceinline__ double warp_min(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmin(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}
__device__ __forceinline__ double warp_max(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmax(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}

// Block-wide extrema of (lo, hi, amax); every thread of the 256-thread CTA gets the result.
__device__ __forceinline__ void block_extrema(double &lo, double &hi, double &amax) {
    __shared__ double s_lo[8], s_hi[8], s_am[8];
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
        lo = fmin(lo, s_lo[i]);      // fmin / fmax drop a NaN operand, as f64::min / f64::max do
        hi = fmax(hi, s_hi[i]);
        amax = fmax(amax, s_am[i]);
    }
}

// ---- per-channel: one CTA per row, two passes ---------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
quantize_rows_ex_kernel(const T *__restrict__ w, size_t rows, size_t cols, int bits, int mode,
                        int8_t *__restrict__ q, double *__restrict__ scales, double *__restrict__ zps) {
    for (size_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const T *src = w + row * cols;
        double lo = INFINITY, hi = -INFINITY, amax = 0.0;
        for (size_t c = threadIdx.x; c < cols; c += 256) {
            const double v = widen(src[c]);
            lo = fmin(lo, v);
            hi = fmax(hi, v);
            amax = fmax(amax, fabs(v));
        }
        block_extrema(lo, hi, amax);
        const GroupParams p = make_group(lo, hi, amax, cols, bits, mode);  // every thread: same inputs, same result
        if (threadIdx.x == 0) {
            scales[row] = p.scale;
            zps[row] = p.zp;
        }
        int8_t *dst = q + row * cols;
        for (size_t c = threadIdx.x; c < cols; c += 256) dst[c] = (int8_t)quant_ex(widen(src[c]), p);
    }
}

// ---- per-tensor ---------------------------------------------------------------------------------
// Doubles order like these integer keys (negative values reversed below the positive ones), so
// atomicMin / atomicMax on the keys are a min / max of the values.  NaN never reaches a key.
__device__ __forceinline__ unsigned long long key_of(double f) {
    const unsigned long long b = (unsigned long long)__double_as_longlong(f);
    return (b >> 63) ? ~b : (b | 0x8000000000000000ull);
}
__device__ __forceinline__ double double_of(unsigned long long k) {
    return __longlong_as_double((long long)((k >> 63) ? (k & 0x7FFFFFFFFFFFFFFFull) : ~k));
}

struct TensorWords {
    unsigned long long lo_key, hi_key, amax_key;
    GroupParams p;
};

__global__ void init_words_kernel(TensorWords *t) {
    t->lo_key = key_of(INFINITY);
    t->hi_key = key_of(-INFINITY);
    t->amax_key = key_of(0.0);
}

template <typename T>
__global__ void __launch_bounds__(256)
extrema_flat_kernel(const T *__restrict__ w, size_t n, TensorWords *t) {
    double lo = INFINITY, hi = -INFINITY, amax = 0.0;
    const size_t stride = (size_t)gridDim.x * 256;
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += stride) {
        const double v = widen(w[i]);
        lo = fmin(lo, v);
        hi = fmax(hi, v);
        amax = fmax(amax, fabs(v));
    }
    block_extrema(lo, hi, amax);
    if (threadIdx.x == 0) {
        atomicMin(&t->lo_key, key_of(lo));
        atomicMax(&t->hi_key, key_of(hi));
        atomicMax(&t->amax_key, key_of(amax));
    }
}

__global__ void finalize_ex_kernel(TensorWords *t, size_t n, int bits, int mode, double *scales, double *zps) {
    const GroupParams p = make_group(double_of(t->lo_key), double_of(t->hi_key), double_of(t->amax_key), n, bits, mode);
    t->p = p;
    scales[0] = p.scale;
    zps[0] = p.zp;
}

template <typename T>
__global__ void __launch_bounds__(256)
quantize_flat_ex_kernel(const T *__restrict__ w, size_t n, const TensorWords *__restrict__ t, int8_t *__restrict__ q) {
    const GroupParams p = t->p;
    const size_t stride = (size_t)gridDim.x * 256;
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += stride) q[i] = (int8_t)quant_ex(widen(w[i]), p);
}

// ---- dequantize with zero points ------------------------------------------------------------------
// f64 -> the tensor's storage type with one rounding (Tensor::from_f64_slice, quantize.rs:219-224)
__device__ __forceinline__ uint16_t f64_to_bf16_rne(double v) {
    if (v != v) return 0x7FC0;
    float f = __double2float_rz(v);
    uint32_t b = __float_as_uint(f);
    if ((double)f != v && !isinf(f)) b |= 1u;  // sticky bit below bf16's ulp: a single rounding overall
    if (isinf(v)) return (uint16_t)(b >> 16);
    return (uint16_t)((b + 0x7FFFu + ((b >> 16) & 1u)) >> 16);
}
__device__ __forceinline__ void narrow(double v, float *o) { *o = (float)v; }
__device__ __forceinline__ void narrow(double v, double *o) { *o = v; }
__device__ __forceinline__ void narrow(double v, uint16_t *o) { *o = f64_to_bf16_rne(v); }
__device__ __forceinline__ void narrow(double v, __half *o) { *o = __double2half(v); }

// OutT: float, double, uint16_t (bf16 bits) or __half; zps == nullptr means zero points of 0.0
template <typename OutT>
__global__ void __launch_bounds__(256)
dequantize_ex_kernel(const int8_t *__restrict__ q, const double *__restrict__ scales, const double *__restrict__ zps,
                     size_t rows, size_t cols, int per_channel, OutT *__restrict__ out) {
    const size_t n = rows * cols;
    const size_t stride = (size_t)gridDim.x * 256;
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += stride) {
        const size_t g = per_channel ? i / cols : 0;
        const double v = __dmul_rn(__dsub_rn((double)q[i], zps ? zps[g] : 0.0), scales[g]);
        narrow(v, out + i);
    }
}

// ---- INT4 codes, two per byte --------------------------------------------------------------------
// The reference keeps INT4 codes one per i8 (its size_bytes only pretends to pack, quantize.rs:176).
// Packed form used by the small-batch forward: byte j of a row = codes 2j (low nibble) and 2j+1 (high
// nibble), each stored as code + 8 (0..15), so unpacking needs no sign extension.
__global__ void __launch_bounds__(256)
pack_int4_kernel(const int8_t *__restrict__ q, size_t n_pairs, uint8_t *__restrict__ out) {
    const size_t stride = (size_t)gridDim.x * 256;
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n_pairs; i += stride) {
        const unsigned lo = (unsigned)(q[2 * i] + 8) & 0xFu, hi = (unsigned)(q[2 * i + 1] + 8) & 0xFu;
        out[i] = (uint8_t)(lo | (hi << 4));
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
