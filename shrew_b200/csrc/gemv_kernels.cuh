// Weight-only INT8 GEMV for small batches (M <= 16), sm_100a.
//
//   y[m,n] = scale[n] * sum_k q[n,k] * x[m,k] + bias[n]        (quantize.rs:463-476 with
// the per-channel scale moved behind the dot product: codes are exact small integers, so
// the f32 accumulator holds sum_k q*x and one multiply applies the scale).
//
// HBM-bound: the only large stream is the INT8 matrix, N*K bytes, read exactly once.
// A CTA of 4 warps owns R consecutive output rows; the K range is dealt to the 4 warps in
// 512-byte pieces (32 lanes x 16 B), so every warp-level load is one fully used 512 B
// segment and each lane keeps R independent 16 B loads in flight per step.  Weights bypass
// L1 (read once); the activations are tiny, read through L1 and reused by every row.
// Codes are widened to f32 in registers and fed to FFMA; partial sums are combined with
// warp shuffles, then across the 4 warps through shared memory.
//
// Device code only (no launch syntax, no runtime calls, PTX behind ptx_small.cuh): it also compiles as
// plain C++ against the CUDA stand-in of the CPU tests (tests/cpu_emu/).
#pragma once

#include "../../include/shrewq.h"
#include "dests.cuh"
#include "ptx_small.cuh"

namespace shrewq {
namespace {

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;

// 4 INT8 codes (one word) -> 4 floats, exactly.  Two forms, chosen by the token count of the instantiation:
//  - integer-to-float conversions: they run on the quarter-rate conversion pipe, which is otherwise idle, so with two
//    or more tokens per code (where the FMA pipe is the busy one) they cost nothing: 6.3 against 8.6 us at 4096 x 4096,
//    batch 2;
//  - MAGIC (one token): at batch 1 that pipe is the bottleneck (3.6 us of conversions for 16.8 M codes against 2.6 us
//    of HBM stream), so the bytes are permuted into the mantissa of 2^23 (byte ^ 0x80 = q + 128 as an unsigned byte u;
//    0x4B0000uu is the float 2^23 + u) and 2^23 + 128 is subtracted: 5.3 against 5.9 us.
template <bool MAGIC>
__device__ __forceinline__ void i8x4_to_f32(uint32_t w, float *o) {
    if constexpr (MAGIC) {
        const uint32_t u = w ^ 0x80808080u;
        float f0 = __uint_as_float((u & 0xFFu) | 0x4B000000u);
        float f1 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7441));
        float f2 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7442));
        float f3 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7443));
        add_f32x2(f0, f1, -8388736.0f, -8388736.0f);
        add_f32x2(f2, f3, -8388736.0f, -8388736.0f);
        o[0] = f0; o[1] = f1; o[2] = f2; o[3] = f3;
    } else {
        o[0] = (float)(int)(int8_t)(w & 0xFF);
        o[1] = (float)(int)(int8_t)((w >> 8) & 0xFF);
        o[2] = (float)(int)(int8_t)((w >> 16) & 0xFF);
        o[3] = (float)(int)(int8_t)(w >> 24);
    }
}

// 16 consecutive activations of one token as f32
template <typename XT>
__device__ __forceinline__ void load_x16(const XT *p, float *o);

template <>
__device__ __forceinline__ void load_x16<float>(const float *p, float *o) {
    const float4 *p4 = reinterpret_cast<const float4 *>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float4 v = __ldg(p4 + i);
        o[4 * i] = v.x; o[4 * i + 1] = v.y; o[4 * i + 2] = v.z; o[4 * i + 3] = v.w;
    }
}

template <>
__device__ __forceinline__ void load_x16<__nv_bfloat16>(const __nv_bfloat16 *p, float *o) {
    const uint4 *p4 = reinterpret_cast<const uint4 *>(p);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const uint4 v = __ldg(p4 + i);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            o[8 * i + 2 * j] = __uint_as_float(w[j] << 16);
            o[8 * i + 2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
        }
    }
}

template <typename YT>
__device__ __forceinline__ void store_y(YT *p, float v);
template <>
__device__ __forceinline__ void store_y<float>(float *p, float v) { *p = v; }
template <>
__device__ __forceinline__ void store_y<__nv_bfloat16>(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float silu(float g) { return g / (1.0f + __expf(-g)); }

// MT: tokens handled (M padded up to MT, extra tokens masked); R: output rows per CTA.
// GATED: rows come in pairs (gate row n from q, up row n from q_up); R counts pairs * 2.
// PDL (programmatic dependent launch, opt-in): the kernel lets the next kernel of the stream start at
// once, fetches its first weights, and only then waits for the previous kernel, whose output its
// activations may be; the weights never depend on an earlier kernel.  Back-to-back GEMVs thus keep
// the weight stream going across the kernel boundary.
// SLICED: the grid's y dimension walks over slices of MT tokens (batches above MT on small layers); a separate
// instantiation, so that the unsliced kernels keep their code (the slice arithmetic cost them 15-25 % when it was
// unconditional).
template <int MT, int R, typename XT, typename YT, bool GATED, bool PDL = false, bool SLICED = false>
__global__ void __launch_bounds__(kThreads)
gemv_i8_kernel(const int8_t *__restrict__ q, const float *__restrict__ scales,
               const float *__restrict__ bias, const int8_t *__restrict__ q_up,
               const float *__restrict__ scales_up, const float *__restrict__ bias_up,
               const XT *__restrict__ x, YT *__restrict__ y, Dests extra, int M, int N, int K,
               size_t ldy, int epilogue) {
    constexpr int NR = GATED ? R / 2 : R;  // distinct output columns per CTA
    if constexpr (PDL) pdl_launch_dependents();
    int mb = 0;
    if constexpr (SLICED) {
        mb = (int)blockIdx.y * MT;
        x += (size_t)mb * K;
        M = M - mb < MT ? M - mb : MT;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * NR;
    const int chunks = K >> 4;

    const int8_t *rowp[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        int n = n0 + (GATED ? (r >> 1) : r);
        n = n < N ? n : N - 1;  // clamp: duplicates are computed and dropped
        const int8_t *base = (GATED && (r & 1)) ? q_up : q;
        rowp[r] = base + (size_t)n * K;
    }

    float acc[R][MT];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[r][m] = 0.0f;

    int c = warp * 32 + lane;
    uint4 wv[R];
    bool have = false;  // wv already holds the weights of chunk c
    if constexpr (PDL) {
        have = c < chunks;
        if (have) {
#pragma unroll
            for (int r = 0; r < R; ++r) wv[r] = ld_stream_16(rowp[r] + ((size_t)c << 4));
        }
        // neither read the activations nor write the output before the previous kernel of the
        // stream, which may have produced or may still read them, has completed
        pdl_wait();
    }

    for (; c < chunks; c += kWarps * 32) {
        if (!have) {
#pragma unroll
            for (int r = 0; r < R; ++r) wv[r] = ld_stream_16(rowp[r] + ((size_t)c << 4));
        }
        have = false;
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            float xf[16];
            if (m < M) {
                load_x16<XT>(x + (size_t)m * K + ((size_t)c << 4), xf);
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) xf[i] = 0.0f;
            }
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const uint32_t w4[4] = {wv[r].x, wv[r].y, wv[r].z, wv[r].w};
                float s = acc[r][m];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float wf[4];
                    i8x4_to_f32<MT == 1>(w4[j], wf);
                    s = fmaf(wf[0], xf[4 * j], s);
                    s = fmaf(wf[1], xf[4 * j + 1], s);
                    s = fmaf(wf[2], xf[4 * j + 2], s);
                    s = fmaf(wf[3], xf[4 * j + 3], s);
                }
                acc[r][m] = s;
            }
        }
    }

    __shared__ float s_red[kWarps][R][MT];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            float v = acc[r][m];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
            if (lane == 0) s_red[warp][r][m] = v;
        }
    __syncthreads();

    for (int i = threadIdx.x; i < NR * MT; i += kThreads) {
        const int nr = i / MT, m = i % MT;
        const int n = n0 + nr;
        if (n >= N || m >= M) continue;
        float out;
        if constexpr (GATED) {
            float g = 0.0f, u = 0.0f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                g += s_red[w][2 * nr][m];
                u += s_red[w][2 * nr + 1][m];
            }
            g = g * scales[n] + (bias ? bias[n] : 0.0f);
            u = u * scales_up[n] + (bias_up ? bias_up[n] : 0.0f);
            out = silu(g) * u;
        } else {
            float s = 0.0f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) s += s_red[w][nr][m];
            out = s * scales[n] + (bias ? bias[n] : 0.0f);
            if (epilogue == SHREWQ_EPILOGUE_RELU) out = fmaxf(out, 0.0f);
        }
        store_y<YT>(y + (size_t)(mb + m) * ldy + n, out);
        for (int d = 0; d < extra.n; ++d) store_y<YT>(static_cast<YT *>(extra.p[d]) + (size_t)(mb + m) * ldy + n, out);
    }
}

}  // namespace
}  // namespace shrewq
