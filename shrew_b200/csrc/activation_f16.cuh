// Per-token power-of-two rescale of bf16 activations into f16 (used by the f16 warp-MMA forward,
// gemv_mma.cu): shift[m] = 14 - floor(log2(amax of row m)), x16 = f16(x * 2^shift[m]).
//
// Device code only (no launch syntax, no runtime calls): it also compiles as plain C++ against the
// CUDA stand-in of the CPU tests (tests/cpu_emu/).
#pragma once

#ifndef SHREWQ_CPU_EMU
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#endif

namespace shrewq {
namespace {

// amax exponent -> shift, the one rule of the staging kernel and of the in-CTA staging
__device__ __forceinline__ int shift_of_amax(float a) {
    int e = 0;
    if (a > 0.0f) e = isinf(a) ? 127 : ilogbf(a);
    return 14 - e;
}

// Token row m of bf16 activations -> f16 of x * 2^shift[m], shift[m] = 14 - floor(log2(amax of
// the row)) (0 for an all-zero row; a row holding Inf uses the largest finite exponent; NaN
// elements stay NaN and do not take part in amax).  One CTA per token row.
__global__ void __launch_bounds__(256)
x_to_f16_kernel(const __nv_bfloat16 *__restrict__ x, __half *__restrict__ x16, int *__restrict__ shift, int K,
                int perm = 0) {
    const __nv_bfloat16 *row = x + (size_t)blockIdx.x * K;
    __half *out = x16 + (size_t)blockIdx.x * K;
    float amax = 0.0f;
    for (int k = threadIdx.x; k < K; k += 256) amax = fmaxf(amax, fabsf(__bfloat162float(row[k])));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    __shared__ float s_max[8];
    __shared__ int s_shift;
    if ((threadIdx.x & 31) == 0) s_max[threadIdx.x >> 5] = amax;
    __syncthreads();
    if (threadIdx.x == 0) {
        float a = s_max[0];
#pragma unroll
        for (int w = 1; w < 8; ++w) a = fmaxf(a, s_max[w]);
        s_shift = shift_of_amax(a);
        shift[blockIdx.x] = s_shift;
    }
    __syncthreads();
    const int sh = s_shift;
    // perm: within every group of 8 the values are stored in the order 0 4 1 5 2 6 3 7 (what the
    // packed-INT4 forward pairs its codes with)
    for (int k = threadIdx.x; k < K; k += 256) {
        const int pos = perm ? ((k & ~7) | (((k & 3) << 1) | ((k >> 2) & 1))) : k;
        out[pos] = __float2half_rn(ldexpf(__bfloat162float(row[k]), sh));
    }
}

}  // namespace
}  // namespace shrewq
