// General-shape quantized Linear forward on CUDA cores (f32 FMA), sm_100a.
//
// This is the "f32 accumulate" path: activations stay f32 (or bf16 widened exactly), the
// INT8 codes are widened exactly, every product and sum is an f32 FMA, and the per-channel
// scale and bias are applied to the accumulator.  It accepts any M, N, K and any
// alignment, so it also serves shapes the TMA/tcgen05 kernel cannot take (K not a
// multiple of 16, unaligned pointers).  Tiling: 128 tokens x 64 channels x 16 k per CTA,
// 256 threads, 8x4 outputs per thread, operands staged in shared memory as f32.
//
// Device code only (no launch syntax, no runtime calls): it also compiles as plain C++ against the CUDA
// stand-in of the CPU tests (tests/cpu_emu/).
#pragma once

#include "../../include/shrewq.h"
#include "dests.cuh"
#ifndef SHREWQ_CPU_EMU
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#endif

namespace shrewq {
namespace {

constexpr int BM = 128, BN = 64, BK = 16, TM = 8, TN = 4;

template <typename XT>
__device__ __forceinline__ float to_f32(XT v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename YT>
__device__ __forceinline__ void put(YT *p, float v);
template <>
__device__ __forceinline__ void put<float>(float *p, float v) { *p = v; }
template <>
__device__ __forceinline__ void put<__nv_bfloat16>(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float silu_f(float g) { return g / (1.0f + __expf(-g)); }

template <typename XT, typename YT, bool GATED>
__global__ void __launch_bounds__(256)
gemm_i8_simt_kernel(const int8_t *__restrict__ q, const float *__restrict__ scales,
                    const float *__restrict__ bias, const int8_t *__restrict__ q_up,
                    const float *__restrict__ scales_up, const float *__restrict__ bias_up,
                    const XT *__restrict__ x, YT *__restrict__ y, size_t M, size_t N, size_t K,
                    size_t ldy, int epilogue) {
    __shared__ float xs[BK][BM + 4];
    __shared__ float ws[GATED ? 2 : 1][BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;  // tx -> channels, ty -> tokens
    const size_t m0 = (size_t)blockIdx.y * BM, n0 = (size_t)blockIdx.x * BN;

    float acc[GATED ? 2 : 1][TM][TN];
#pragma unroll
    for (int g = 0; g < (GATED ? 2 : 1); ++g)
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
            for (int j = 0; j < TN; ++j) acc[g][i][j] = 0.0f;

    for (size_t k0 = 0; k0 < K; k0 += BK) {
        // x tile: 128 x 16 values, 8 per thread; consecutive threads walk k (contiguous)
#pragma unroll
        for (int i = 0; i < (BM * BK) / 256; ++i) {
            const int e = tid + i * 256;
            const int kk = e % BK, mm = e / BK;
            const size_t m = m0 + mm, k = k0 + kk;
            xs[kk][mm] = (m < M && k < K) ? to_f32<XT>(x[m * K + k]) : 0.0f;
        }
#pragma unroll
        for (int i = 0; i < (BN * BK) / 256; ++i) {
            const int e = tid + i * 256;
            const int kk = e % BK, nn = e / BK;
            const size_t n = n0 + nn, k = k0 + kk;
            const bool ok = n < N && k < K;
            ws[0][kk][nn] = ok ? (float)q[n * K + k] : 0.0f;
            if constexpr (GATED) ws[1][kk][nn] = ok ? (float)q_up[n * K + k] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float xr[TM], wr[GATED ? 2 : 1][TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) xr[i] = xs[kk][ty * TM + i];
#pragma unroll
            for (int g = 0; g < (GATED ? 2 : 1); ++g)
#pragma unroll
                for (int j = 0; j < TN; ++j) wr[g][j] = ws[g][kk][tx * TN + j];
#pragma unroll
            for (int g = 0; g < (GATED ? 2 : 1); ++g)
#pragma unroll
                for (int i = 0; i < TM; ++i)
#pragma unroll
                    for (int j = 0; j < TN; ++j) acc[g][i][j] = fmaf(xr[i], wr[g][j], acc[g][i][j]);
        }
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const size_t m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const size_t n = n0 + tx * TN + j;
            if (n >= N) continue;
            float o = acc[0][i][j] * scales[n] + (bias ? bias[n] : 0.0f);
            if constexpr (GATED) {
                const float u = acc[1][i][j] * scales_up[n] + (bias_up ? bias_up[n] : 0.0f);
                o = silu_f(o) * u;
            } else if (epilogue == SHREWQ_EPILOGUE_RELU) {
                o = fmaxf(o, 0.0f);
            }
            put<YT>(y + m * ldy + n, o);
        }
    }
}

}  // namespace
}  // namespace shrewq
