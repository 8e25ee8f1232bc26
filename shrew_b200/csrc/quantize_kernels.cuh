// INT8 symmetric quantize / dequantize kernels (sm_100a).
//
// Reference semantics (crates/shrew/src/quantize.rs):
//   scale     = amax < 1e-30 ? 1.0 : amax / 127.0                (f64, :349-351)
//   inv_scale = |scale| < 1e-30 ? 0.0 : 1.0 / scale              (f64, :236-240, :295-299)
//   code      = clamp(round_half_away(v * inv_scale + 0.0), -127, 127) as i8   (:244-250)
// all in f64 on a widened copy of the f32 tensor.  The kernels below produce the same
// bits.  amax of f32 values is exact in f32.  The element map runs in f32 and is trusted
// only when the product lies far from a rounding boundary; the few elements near a
// boundary (and every element of a row whose inv_scale is not an ordinary f32 number) are
// recomputed with the reference's exact f64 operations.  Why that is safe: for |t| <= 127
// the f32 product differs from the f64 one by at most 127 * 2^-23 ~ 1.5e-5, and the
// recompute window is 1e-4 on either side of x.5.
//
// Memory plan (HBM-bound, 5 B/element algorithmic): a row is read ONCE into registers,
// reduced (warp shuffles, then shared memory across warps), and quantized from registers;
// codes are written as packed 32-bit words.  Rows too long for registers take a two-pass
// kernel whose second read normally hits L2.
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

struct RowParams {
    double inv64;
    float inv32;
    int exact_only;  // 1: every element must take the f64 path
};

__device__ __forceinline__ void make_params(float amax, double *scale_out, RowParams *p) {
    double a = (double)amax;
    double scale = a < 1e-30 ? 1.0 : a / 127.0;
    double inv = fabs(scale) < 1e-30 ? 0.0 : 1.0 / scale;
    *scale_out = scale;
    p->inv64 = inv;
    p->inv32 = (float)inv;
    // f32 fast path needs an ordinary reciprocal: finite, normal in f32, not zero
    p->exact_only = !(inv > 1e-30 && inv < 1e30);
}

// The reference's element map, operation for operation, in f64.
__device__ __forceinline__ int quant_exact(float v, double inv64) {
    double t = __dadd_rn(__dmul_rn((double)v, inv64), 0.0);
    if (t != t) return 0;  // NaN as i8 == 0
    double r = trunc(t);
    if (fabs(t - r) >= 0.5) r += copysign(1.0, t);  // round half away from zero
    r = fmin(fmax(r, -127.0), 127.0);
    return (int)r;
}

__device__ __forceinline__ int quant_one(float v, const RowParams &p) {
    if (!p.exact_only) {
        float t = v * p.inv32;
        float a = fabsf(t);
        float frac = a - truncf(a);  // exact
        if (fabsf(frac - 0.5f) > 1e-4f && a < 1000.0f) {  // false for NaN
            int m = min((int)(a + 0.5f), 127);
            return t < 0.0f ? -m : m;
        }
    }
    return quant_exact(v, p.inv64);
}

__device__ __forceinline__ uint32_t pack4(int a, int b, int c, int d) {
    return (uint32_t)(a & 0xFF) | ((uint32_t)(b & 0xFF) << 8) | ((uint32_t)(c & 0xFF) << 16) |
           ((uint32_t)(d & 0xFF) << 24);
}

__device__ __forceinline__ float abs4max(float4 v) {
    // fmaxf drops a NaN operand, as f64::max does in the reference's fold
    return fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}

// ---- per-channel, row held in registers ---------------------------------------------
// GROUP threads own one row; each keeps NV float4.  cols % 4 == 0, pointers 16 B / 4 B
// aligned (checked by the launcher).
template <int GROUP, int NV>
__global__ void __launch_bounds__(GROUP >= 256 ? GROUP : 256)
quantize_rows_reg_kernel(const float *__restrict__ w, size_t rows, size_t cols,
                         int8_t *__restrict__ q, double *__restrict__ scales) {
    constexpr int THREADS = GROUP >= 256 ? GROUP : 256;
    constexpr int ROWS_PER_CTA = THREADS / GROUP;
    constexpr int WARPS_PER_GROUP = GROUP / 32;
    const int g = threadIdx.x / GROUP;
    const int t = threadIdx.x % GROUP;
    const size_t row = (size_t)blockIdx.x * ROWS_PER_CTA + g;
    const bool active = row < rows;
    const int nvec = (int)(cols >> 2);
    const float4 *src = reinterpret_cast<const float4 *>(w + (active ? row : 0) * cols);

    float4 v[NV];
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = t + i * GROUP;
        v[i] = (active && c < nvec) ? __ldcs(src + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) amax = fmaxf(amax, abs4max(v[i]));
    amax = warp_max(amax);

    RowParams p;
    if constexpr (WARPS_PER_GROUP == 1) {
        double scale;
        make_params(amax, &scale, &p);  // every lane: 2 f64 divisions, rows here are short
        if (active && t == 0) scales[row] = scale;
    } else {
        __shared__ float s_part[THREADS / 32];
        __shared__ RowParams s_p[ROWS_PER_CTA];
        const int wig = t >> 5;  // warp in group
        if ((t & 31) == 0) s_part[g * WARPS_PER_GROUP + wig] = amax;
        __syncthreads();
        if (t < 32) {
            float m = 0.0f;
            for (int i = t; i < WARPS_PER_GROUP; i += 32) m = fmaxf(m, s_part[g * WARPS_PER_GROUP + i]);
            m = warp_max(m);
            if (t == 0) {
                double scale;
                RowParams pp;
                make_params(m, &scale, &pp);
                s_p[g] = pp;
                if (active) scales[row] = scale;
            }
        }
        __syncthreads();
        p = s_p[g];
    }

    if (!active) return;
    uint32_t *dst = reinterpret_cast<uint32_t *>(q + row * cols);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = t + i * GROUP;
        if (c < nvec)
            __stcs(dst + c, pack4(quant_one(v[i].x, p), quant_one(v[i].y, p), quant_one(v[i].z, p),
                                  quant_one(v[i].w, p)));
    }
}

// ---- per-channel, any shape (two passes, scalar accesses) ----------------------------
__global__ void __launch_bounds__(256)
quantize_rows_generic_kernel(const float *__restrict__ w, size_t rows, size_t cols,
                             int8_t *__restrict__ q, double *__restrict__ scales) {
    __shared__ float s_part[8];
    __shared__ RowParams s_p;
    for (size_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const float *src = w + row * cols;
        float amax = 0.0f;
        for (size_t c = threadIdx.x; c < cols; c += blockDim.x) amax = fmaxf(amax, fabsf(src[c]));
        amax = warp_max(amax);
        if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = amax;
        __syncthreads();
        if (threadIdx.x == 0) {
            float m = 0.0f;
            for (int i = 0; i < 8; ++i) m = fmaxf(m, s_part[i]);
            double scale;
            RowParams pp;
            make_params(m, &scale, &pp);
            s_p = pp;
            scales[row] = scale;
        }
        __syncthreads();
        const RowParams p = s_p;
        int8_t *dst = q + row * cols;
        for (size_t c = threadIdx.x; c < cols; c += blockDim.x) dst[c] = (int8_t)quant_one(src[c], p);
        __syncthreads();  // s_part / s_p are reused by the next row
    }
}

// ---- per-tensor: amax over everything, then the element map --------------------------
// `amax_bits` is a zero-initialised word of scratch; non-negative floats order like their
// bit patterns, so atomicMax on the bits is a float max.
__global__ void __launch_bounds__(256)
absmax_flat_kernel(const float *__restrict__ w, size_t n, unsigned int *amax_bits) {
    float amax = 0.0f;
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t nthreads = (size_t)gridDim.x * blockDim.x;
    const bool aligned = (reinterpret_cast<uintptr_t>(w) & 15) == 0;
    const size_t nvec = aligned ? (n >> 2) : 0;
    const float4 *w4 = reinterpret_cast<const float4 *>(w);
    for (size_t i = tid; i < nvec; i += nthreads) amax = fmaxf(amax, abs4max(__ldg(w4 + i)));
    for (size_t i = (nvec << 2) + tid; i < n; i += nthreads) amax = fmaxf(amax, fabsf(w[i]));
    amax = warp_max(amax);
    __shared__ float s_part[8];
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = amax;
    __syncthreads();
    if (threadIdx.x == 0) {
        float m = 0.0f;
        for (int i = 0; i < 8; ++i) m = fmaxf(m, s_part[i]);
        atomicMax(amax_bits, __float_as_uint(m));  // m is never NaN: fmaxf dropped them
    }
}

struct TensorParams {
    RowParams p;
};

__global__ void finalize_tensor_scale_kernel(const unsigned int *amax_bits, size_t n,
                                             double *scales, TensorParams *out) {
    double scale;
    RowParams p;
    if (n == 0) {  // empty slice: (1.0, 0.0), quantize.rs:340-342
        scale = 1.0;
        p.inv64 = 1.0;
        p.inv32 = 1.0f;
        p.exact_only = 0;
    } else {
        make_params(__uint_as_float(*amax_bits), &scale, &p);
    }
    scales[0] = scale;
    out->p = p;
}

__global__ void __launch_bounds__(256)
quantize_flat_kernel(const float *__restrict__ w, size_t n, const TensorParams *__restrict__ tp,
                     int8_t *__restrict__ q) {
    const RowParams p = tp->p;
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t nthreads = (size_t)gridDim.x * blockDim.x;
    const bool aligned =
        ((reinterpret_cast<uintptr_t>(w) & 15) == 0) && ((reinterpret_cast<uintptr_t>(q) & 3) == 0);
    const size_t nvec = aligned ? (n >> 2) : 0;
    const float4 *w4 = reinterpret_cast<const float4 *>(w);
    uint32_t *q4 = reinterpret_cast<uint32_t *>(q);
    for (size_t i = tid; i < nvec; i += nthreads) {
        const float4 v = __ldcs(w4 + i);
        __stcs(q4 + i, pack4(quant_one(v.x, p), quant_one(v.y, p), quant_one(v.z, p), quant_one(v.w, p)));
    }
    for (size_t i = (nvec << 2) + tid; i < n; i += nthreads) q[i] = (int8_t)quant_one(w[i], p);
}

// ---- dequantize -----------------------------------------------------------------------
// out = narrow((q as f64 - 0.0) * scale): one f64 multiply per element, then a single
// rounding to the output type (quantize.rs:262-266, :320-335, :219-224).
__device__ __forceinline__ float dq_f32(int q, double s) { return (float)(((double)q - 0.0) * s); }

// f64 -> bf16 with one rounding: narrow to f32 toward zero, make it sticky (round to odd),
// then round the f32 to bf16 to nearest even.
__device__ __forceinline__ uint16_t f64_to_bf16_rne(double v) {
    if (v != v) return 0x7FC0;
    float f = __double2float_rz(v);
    uint32_t b = __float_as_uint(f);
    if ((double)f != v && !isinf(f)) b |= 1u;  // inexact: keep a sticky bit below bf16's ulp
    if (isinf(v)) return (uint16_t)(b >> 16);
    uint32_t rounded = b + 0x7FFFu + ((b >> 16) & 1u);
    return (uint16_t)(rounded >> 16);
}

template <typename OutT>
__global__ void __launch_bounds__(256)
dequantize_kernel(const int8_t *__restrict__ q, const double *__restrict__ scales, size_t rows,
                  size_t cols, int per_channel, OutT *__restrict__ out, int vec_ok) {
    const size_t n = rows * cols;
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t nthreads = (size_t)gridDim.x * blockDim.x;
    if (vec_ok) {  // cols % 4 == 0 and aligned pointers: a 4-code word never straddles a row
        const size_t nvec = n >> 2;
        const uint32_t *q4 = reinterpret_cast<const uint32_t *>(q);
        for (size_t i = tid; i < nvec; i += nthreads) {
            const uint32_t wd = __ldcs(q4 + i);
            const double s = per_channel ? __ldg(scales + (i << 2) / cols) : __ldg(scales);
            const int a = (int)(int8_t)(wd & 0xFF), b = (int)(int8_t)((wd >> 8) & 0xFF),
                      c = (int)(int8_t)((wd >> 16) & 0xFF), d = (int)(int8_t)(wd >> 24);
            if constexpr (sizeof(OutT) == 4) {
                __stcs(reinterpret_cast<float4 *>(out) + i,
                       make_float4(dq_f32(a, s), dq_f32(b, s), dq_f32(c, s), dq_f32(d, s)));
            } else {
                uint2 o;
                o.x = (uint32_t)f64_to_bf16_rne((double)a * s) | ((uint32_t)f64_to_bf16_rne((double)b * s) << 16);
                o.y = (uint32_t)f64_to_bf16_rne((double)c * s) | ((uint32_t)f64_to_bf16_rne((double)d * s) << 16);
                __stcs(reinterpret_cast<uint2 *>(out) + i, o);
            }
        }
    } else {
        for (size_t i = tid; i < n; i += nthreads) {
            const double s = per_channel ? scales[i / cols] : scales[0];
            const int v = (int)q[i];
            if constexpr (sizeof(OutT) == 4)
                out[i] = dq_f32(v, s);
            else
                out[i] = f64_to_bf16_rne((double)v * s);
        }
    }
}

// f64 scales -> f32 per-row scales used by the forward kernels (per-tensor is broadcast).
__global__ void scales_to_f32_kernel(const double *__restrict__ scales, int per_channel, size_t n,
                                     float *__restrict__ out) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = (float)(per_channel ? scales[i] : scales[0]);
}

// x = hi + lo with hi = bf16(x), lo = bf16(x - hi): two bf16 matrices whose sum carries ~16
// significand bits of the f32 activations (relative error ~2^-17), so two tensor-core passes
// over exact bf16 x int8 products stay inside the 1e-4 tolerance of the f32 path.
__global__ void __launch_bounds__(256)
split_f32_kernel(const float *__restrict__ x, size_t n, __nv_bfloat16 *__restrict__ hi, __nv_bfloat16 *__restrict__ lo) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float v = x[i];
        const __nv_bfloat16 h = __float2bfloat16_rn(v);
        hi[i] = h;
        lo[i] = __float2bfloat16_rn(v - __bfloat162float(h));
    }
}

}  // namespace
}  // namespace shrewq
