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
#include <cstdlib>

#include "common.cuh"

namespace shrewq {
namespace {

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;

__device__ __forceinline__ uint4 ld_stream_16(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ void i8x4_to_f32(uint32_t w, float *o) {
    o[0] = (float)(int)(int8_t)(w & 0xFF);
    o[1] = (float)(int)(int8_t)((w >> 8) & 0xFF);
    o[2] = (float)(int)(int8_t)((w >> 16) & 0xFF);
    o[3] = (float)(int)(int8_t)(w >> 24);
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
template <int MT, int R, typename XT, typename YT, bool GATED>
__global__ void __launch_bounds__(kThreads)
gemv_i8_kernel(const int8_t *__restrict__ q, const float *__restrict__ scales,
               const float *__restrict__ bias, const int8_t *__restrict__ q_up,
               const float *__restrict__ scales_up, const float *__restrict__ bias_up,
               const XT *__restrict__ x, YT *__restrict__ y, Dests extra, int M, int N, int K,
               size_t ldy, int epilogue, int pdl) {
    constexpr int NR = GATED ? R / 2 : R;  // distinct output columns per CTA
    // Programmatic dependent launch (opt-in): let the next kernel of the stream start its
    // prologue while this one runs ...
    if (pdl) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
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

    // ... and do not touch the activations (or write the output) before the previous kernel
    // of the stream, which may have produced them, has completed
    if (pdl) asm volatile("griddepcontrol.wait;" ::: "memory");

    for (int c = warp * 32 + lane; c < chunks; c += kWarps * 32) {
        uint4 wv[R];
#pragma unroll
        for (int r = 0; r < R; ++r) wv[r] = ld_stream_16(rowp[r] + ((size_t)c << 4));
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
                    i8x4_to_f32(w4[j], wf);
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
        store_y<YT>(y + (size_t)m * ldy + n, out);
        for (int d = 0; d < extra.n; ++d) store_y<YT>(static_cast<YT *>(extra.p[d]) + (size_t)m * ldy + n, out);
    }
}

template <int MT, int R, typename XT, typename YT, bool GATED>
void launch_one(shrewq_ctx *ctx, const ForwardArgs &a) {
    constexpr int NR = GATED ? R / 2 : R;
    const unsigned grid = (unsigned)((a.N + NR - 1) / NR);
    // SHREWQ_GEMV_PDL=1 launches with programmatic stream serialization so that back-to-back
    // GEMVs overlap launch latency and prologue.  Built, compiled, NOT yet run on a GPU: off
    // unless the variable is set.
    static const bool pdl = getenv("SHREWQ_GEMV_PDL") && atoi(getenv("SHREWQ_GEMV_PDL")) != 0;
    if (pdl) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(grid);
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = 0;
        cfg.stream = ctx->stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        cudaLaunchKernelEx(&cfg, gemv_i8_kernel<MT, R, XT, YT, GATED>, a.q, a.scales, a.bias, a.q_up, a.scales_up,
                           a.bias_up, static_cast<const XT *>(a.x), static_cast<YT *>(a.y), a.extra, (int)a.M, (int)a.N,
                           (int)a.K, a.ldy, a.epilogue, 1);
        return;
    }
    gemv_i8_kernel<MT, R, XT, YT, GATED><<<grid, kThreads, 0, ctx->stream>>>(
        a.q, a.scales, a.bias, a.q_up, a.scales_up, a.bias_up, static_cast<const XT *>(a.x),
        static_cast<YT *>(a.y), a.extra, (int)a.M, (int)a.N, (int)a.K, a.ldy, a.epilogue, 0);
}

template <typename XT, typename YT, bool GATED>
void dispatch_m(shrewq_ctx *ctx, const ForwardArgs &a) {
    if (a.M <= 1) launch_one<1, 4, XT, YT, GATED>(ctx, a);
    else if (a.M <= 2) launch_one<2, 4, XT, YT, GATED>(ctx, a);
    else if (a.M <= 4) launch_one<4, 4, XT, YT, GATED>(ctx, a);
    else if (a.M <= 8) launch_one<8, 2, XT, YT, GATED>(ctx, a);
    else launch_one<16, 2, XT, YT, GATED>(ctx, a);
}

}  // namespace

int launch_gemv(shrewq_ctx *ctx, const ForwardArgs &a) {
    if (a.M == 0 || a.N == 0) return SHREWQ_OK;
    if (a.M > 16 || (a.K % 16) != 0 || a.K == 0 || a.N > 0x7FFFFFFF || a.K > 0x7FFFFFFF)
        return set_err(ctx, SHREWQ_ERR_UNSUPPORTED, "gemv: needs M<=16 and K a positive multiple of 16");
    const bool gated = a.q_up != nullptr;
    const bool xb = a.x_dtype == SHREWQ_BF16, yb = a.y_dtype == SHREWQ_BF16;
#define SHREWQ_GEMV_CASE(XT, YT)                       \
    do {                                               \
        if (gated) dispatch_m<XT, YT, true>(ctx, a);   \
        else dispatch_m<XT, YT, false>(ctx, a);        \
    } while (0)
    if (xb && yb) SHREWQ_GEMV_CASE(__nv_bfloat16, __nv_bfloat16);
    else if (xb && !yb) SHREWQ_GEMV_CASE(__nv_bfloat16, float);
    else if (!xb && !yb) SHREWQ_GEMV_CASE(float, float);
    else SHREWQ_GEMV_CASE(float, __nv_bfloat16);
#undef SHREWQ_GEMV_CASE
    ctx->launches += 1;
    SHREWQ_CUDA_TRY(ctx, cudaGetLastError());
    return SHREWQ_OK;
}

}  // namespace shrewq
