// Weight-only INT8 forward for 1..32 tokens: the weights streamed through a shared-memory ring by bulk copies
// (TMA, 1-D) and multiplied on warp-level MMA, sm_100a.
//
//   y[m,n] = scale[n] * sum_k q[n,k] * x[m,k] + bias[n]        (quantize.rs:463-476; the codes are exact in bf16,
// the products exact in the f32 accumulator, and one multiply applies the scale)
//
// HBM-bound: the INT8 matrix, N*K bytes, is read exactly once and a 4096 x 4096 layer is 2.6 us of stream, so
// what matters is that bytes are requested early, that many are in flight, and that the arithmetic per byte is
// small and independent of the batch.
//
//  - A CTA owns 16 rows of W (gated: the gate rows and the up rows of 8 channels).  A producer warp asks the copy
//    engine for them in stages of 16 rows x 512 bytes, one bulk copy per row and stage, into a ring of S stages
//    (full / empty mbarriers).  With S = 8 a whole K = 4096 row block is requested in the kernel's first hundred
//    cycles; no load instruction waits in a register scoreboard and the bytes in flight per SM (S * 8 KB per
//    CTA) do not depend on how many warps are resident.
//  - Four consumer warps split every stage by k (two 64-wide k-blocks each).  The weights are the A operand of
//    mma.sync.m16n8k16 (16 rows x 16 k), the activations the B operand (16 k x 8 tokens): widening a code to
//    bf16 costs 2.5 instructions whatever the batch, and one to four MMAs per step cover 8 to 32 tokens with
//    the same converted fragment.  Lane (g = lane / 4, t = lane % 4) reads the 16 codes [16t, 16t + 16) of
//    rows g and g + 8 of the k-block and the 16 activations of the same k for tokens g (+ 8, 16, 24); MMA
//    step j uses codes and activations 4j .. 4j+3 of those runs for A and B alike (a dot product does not care
//    about the order of k).  Rows are 576 bytes apart in shared memory, so the 16-byte reads of a quarter warp
//    fall into distinct banks.  Activations come straight from global memory (L1 keeps them: every CTA of
//    an SM reads the same few KB), requested before the wait for the stage.
//  - The four warps' accumulators meet in shared memory; 128 (gated: 64) x NT threads apply scale, bias and
//    the epilogue and store to the local and the peer destinations.
//
// Programmatic dependent launch: the kernel lets its successor start at once, and its producer requests WEIGHTS
// without waiting for the predecessor (weights never depend on an earlier kernel); the consumers wait for it
// before they read activations or write outputs.  A chain of small-batch forwards thus keeps the weight stream
// going across kernel boundaries.  Launched without the attribute the two instructions do nothing.
//
// Every wait is bounded: a wait that runs out records itself in DeviceStatus (timeout code 4) and the CTA
// leaves without writing.
//
// Device code only (PTX behind ptx_small.cuh / ptx_tcgen05.cuh): also compiles against the CUDA stand-in of the
// CPU tests (tests/cpu_emu/).
#pragma once

#include "../../include/shrewq.h"
#include "dests.cuh"
#include "ptx_small.cuh"
#include "ptx_tcgen05.cuh"

namespace shrewq {
namespace {

// W consumer warps (8 or 16) + one producer warp (warp W)
constexpr int kRingRows = 16;                          // rows of W per CTA
constexpr uint32_t kRingSpinLimit = 1u << 22;          // bounded wait: a few tenths of a second with the pauses
constexpr unsigned int kTimeoutRing = 4;               // DeviceStatus::timeout_flag of this kernel

// KC: bytes (= codes) of k per row and stage, i.e. the size of one bulk copy.  The copy engine's cost is per copy:
// measured on a B200 at 4096 x 4096, batch 1, the kernel takes 9.0 us with 512-byte, 7.3 us with 1 KB and 6.8 us
// with 2 KB copies.  Rows are KC + 64 bytes apart in shared memory, so the 16-byte reads of a quarter warp (rows
// g, g + 1; four 16-byte columns) fall into distinct banks.  Three stages of 2 KB rows are 99 KB: two CTAs per SM
// with ~200 KB of weights in flight, the choice for grids of up to two CTAs per SM; grids of several waves take two
// stages (66 KB, three CTAs per SM: the same bytes in flight, half as many more warps to widen codes).
constexpr int kRingMaxStages = 8;
template <int KC, int STAGES = (KC >= 2048 ? 3 : KC >= 1024 ? 5 : 8)>
struct RingCfg {
    static constexpr int kPitch = KC + 64;
    static constexpr int kStageBytes = kRingRows * kPitch;
    static constexpr int kStages = STAGES;
    static constexpr size_t kSmemBytes = (size_t)kStages * kStageBytes + 2 * kRingMaxStages * 8;
};
constexpr int kRingKC = 2048;     // what the launcher instantiates
constexpr int kRingConsumers = 8;

// 4 INT8 codes (one word) -> two packed bf16x2 words, exactly: byte ^ 0x80 = q + 128 as an unsigned byte u;
// 0x4B0000uu is the float 2^23 + u; subtracting 2^23 + 128 leaves q; the pack is exact for |q| <= 128
__device__ __forceinline__ void ring_cvt_i8x4(uint32_t w, uint32_t &lo, uint32_t &hi) {
    const uint32_t u = w ^ 0x80808080u;
    float f0 = __uint_as_float((u & 0xFFu) | 0x4B000000u);                 // one logic op; the others a byte permute
    float f1 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7441));
    float f2 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7442));
    float f3 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7443));
    add_f32x2(f0, f1, -8388736.0f, -8388736.0f);
    add_f32x2(f2, f3, -8388736.0f, -8388736.0f);
    lo = pack_bf16x2_rn(f1, f0);
    hi = pack_bf16x2_rn(f3, f2);
}

template <typename YT>
__device__ __forceinline__ void ring_store(YT *p, float v);
template <>
__device__ __forceinline__ void ring_store<float>(float *p, float v) { *p = v; }
template <>
__device__ __forceinline__ void ring_store<__nv_bfloat16>(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ bool ring_wait(uint32_t bar, uint32_t parity, DeviceStatus *st, uint32_t role, uint32_t stage) {
    for (uint32_t i = 0; i < kRingSpinLimit; ++i) {
        if (mbar_try(bar, parity)) return true;
        if (i > 256) __nanosleep(64);
    }
    if (atomicCAS(&st->timeout_flag, 0u, kTimeoutRing) == 0u) {
        st->where = (blockIdx.x << 8) | role;
        st->stage = stage;
        st->parity = parity;
    }
    return false;
}

// NT: token blocks of 8 (M <= 8 * NT).  K a multiple of 64; q, q_up and x 16-byte aligned.
// GATED: rows 0..7 of the CTA are gate rows, rows 8..15 the up rows of the same 8 channels.
template <int NT, int KC, int W, typename YT, bool GATED, int STAGES = RingCfg<KC>::kStages>
__global__ void __launch_bounds__((W + 1) * 32)
gemv_i8_ring_kernel(const int8_t *__restrict__ q, const float *__restrict__ scales, const float *__restrict__ bias,
                    const int8_t *__restrict__ q_up, const float *__restrict__ scales_up,
                    const float *__restrict__ bias_up, const uint16_t *__restrict__ x, YT *__restrict__ y, Dests extra,
                    int M, int N, int K, size_t ldy, int epilogue, DeviceStatus *status) {
    using C = RingCfg<KC, STAGES>;
    static_assert(KC / 64 >= W, "every consumer warp needs a k-block in every full stage");
    constexpr int kRingWarps = W, kRingThreads = (W + 1) * 32;
    constexpr int NCH = GATED ? kRingRows / 2 : kRingRows;  // output channels per CTA
    SHREWQ_DYNAMIC_SMEM(uint8_t, smem);
    __shared__ float s_red[kRingWarps][NT][4][32];
    __shared__ int s_bad;
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * NCH;
    constexpr int S = C::kStages;
    constexpr uint32_t stage_bytes = C::kStageBytes;
    const uint32_t ring_u32 = smem_u32(smem);
    const uint32_t full_u32 = ring_u32 + S * stage_bytes;
    const uint32_t empty_u32 = full_u32 + kRingMaxStages * 8;
    const int nstages = (K + KC - 1) / KC;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(full_u32 + s * 8, 1);
            mbar_init(empty_u32 + s * 8, kRingWarps);
        }
        mbar_fence_init();
        s_bad = 0;
    }
    __syncthreads();

    bool ok = true;
    if (warp == kRingWarps) {
        // ---- producer: lane r brings row r of every stage ----
        const int8_t *src = nullptr;
        if (lane < kRingRows) {
            int n = n0 + (GATED ? (lane & 7) : lane);
            n = n < N ? n : N - 1;  // clamp: duplicates are computed and dropped
            src = ((GATED && lane >= 8) ? q_up : q) + (size_t)n * K;
        }
        for (int s = 0; s < nstages; ++s) {
            const int slot = s % S;
            if (s >= S) {
                int good = 1;
                if (lane == 0) good = ring_wait(empty_u32 + slot * 8, ((s / S) - 1) & 1, status, 1, s) ? 1 : 0;
                ok = __shfl_sync(0xFFFFFFFFu, good, 0) != 0;
                if (!ok) break;
            }
            const int k0 = s * KC;
            const uint32_t bytes = (uint32_t)(K - k0 < KC ? K - k0 : KC);
            if (lane == 0) mbar_expect_tx(full_u32 + slot * 8, bytes * kRingRows);
            __syncwarp();
            if (lane < kRingRows) bulk_load_1d(ring_u32 + slot * stage_bytes + lane * C::kPitch, src + k0, bytes, full_u32 + slot * 8);
        }
        pdl_wait();  // this warp's threads also write outputs below
    } else {
        // ---- consumers: warp w takes the k-blocks w, w + W, ... ----
        const int g = lane >> 2, t = lane & 3;
        // two accumulator sets, alternating by MMA step: halves the chain of dependent MMAs
        float acc[2][NT][4];
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int r = 0; r < 4; ++r) acc[h][nt][r] = 0.0f;
        // the activations may be the previous kernel's output, which may also still read our output buffer
        pdl_wait();
        const uint16_t *xrow[NT];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) xrow[nt] = (8 * nt + g) < M ? x + (size_t)(8 * nt + g) * K + 16 * t : nullptr;

        uint4 xc[NT][2], xn[NT][2];
#define SHREWQ_RING_LOAD_X(koff, xv)                                                              \
    _Pragma("unroll") for (int nt = 0; nt < NT; ++nt) {                                           \
        xv[nt][0] = make_uint4(0, 0, 0, 0);                                                       \
        xv[nt][1] = make_uint4(0, 0, 0, 0);                                                       \
        if (xrow[nt] && (koff) < K) {                                                             \
            xv[nt][0] = __ldg(reinterpret_cast<const uint4 *>(xrow[nt] + (koff)));                \
            xv[nt][1] = __ldg(reinterpret_cast<const uint4 *>(xrow[nt] + (koff)) + 1);            \
        }                                                                                         \
    }
        SHREWQ_RING_LOAD_X(warp * 64, xc);
        const int nkb = K >> 6;
        int cur = -1;
        for (int kb = warp; kb < nkb; kb += kRingWarps) {
            const int koff = kb << 6, s = koff / KC;
            if (s != cur) {
                if (cur >= 0) {
                    __syncwarp();
                    if (lane == 0) mbar_arrive(empty_u32 + (cur % S) * 8);  // this warp is done with the stage
                }
                cur = s;
                int good = 1;
                if (lane == 0) good = ring_wait(full_u32 + (s % S) * 8, (s / S) & 1, status, 2 + warp, s) ? 1 : 0;
                ok = __shfl_sync(0xFFFFFFFFu, good, 0) != 0;
                // every lane observes the completed phase itself: its own acquire on the bytes the copies wrote
                if (ok) ok = __all_sync(0xFFFFFFFFu, mbar_try(full_u32 + (s % S) * 8, (s / S) & 1) ? 1 : 0) != 0;
                if (!ok) break;
            }
            const uint8_t *stage = smem + (size_t)(s % S) * stage_bytes;
            SHREWQ_RING_LOAD_X(koff + kRingWarps * 64, xn);  // this warp's next k-block, while this one is multiplied
            const uint8_t *wp = stage + (size_t)g * C::kPitch + (koff - s * KC) + 16 * t;
            const uint4 wlo = *reinterpret_cast<const uint4 *>(wp);
            const uint4 whi = *reinterpret_cast<const uint4 *>(wp + 8 * C::kPitch);
            const uint32_t wl[4] = {wlo.x, wlo.y, wlo.z, wlo.w}, wh[4] = {whi.x, whi.y, whi.z, whi.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint32_t a0, a1, a2, a3;
                ring_cvt_i8x4(wl[j], a0, a2);  // row g:     codes (4j, 4j+1) | (4j+2, 4j+3)
                ring_cvt_i8x4(wh[j], a1, a3);  // row g + 8
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const uint4 &xa = xc[nt][j >> 1];
                    const uint32_t b0 = (j & 1) ? xa.z : xa.x, b1 = (j & 1) ? xa.w : xa.y;
                    mma_bf16_16816(acc[j & 1][nt], a0, a1, a2, a3, b0, b1);
                }
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                xc[nt][0] = xn[nt][0];
                xc[nt][1] = xn[nt][1];
            }
        }
#undef SHREWQ_RING_LOAD_X
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int r = 0; r < 4; ++r) s_red[warp][nt][r][lane] = acc[0][nt][r] + acc[1][nt][r];
    }
    // (a CTA with a wait that ran out still meets at the barrier below; it writes nothing)
    if (!ok) s_bad = 1;
    __syncthreads();
    if (s_bad) return;

    // accumulator element (lane, r) of block nt: row (lane / 4) + (r >= 2 ? 8 : 0), token 8 * nt + 2 * (lane % 4) + (r & 1)
    for (int i = threadIdx.x; i < NCH * 8 * NT; i += kRingThreads) {
        const int c = i % NCH, m = i / NCH;
        const int n = n0 + c;
        if (m >= M || n >= N) continue;
        const int nt = m >> 3, mm = m & 7;
        const int ln = (c & 7) * 4 + (mm >> 1);
        float out;
        if constexpr (GATED) {
            float gs = 0.0f, us = 0.0f;
#pragma unroll
            for (int w = 0; w < kRingWarps; ++w) {
                gs += s_red[w][nt][mm & 1][ln];
                us += s_red[w][nt][2 + (mm & 1)][ln];
            }
            gs = gs * scales[n] + (bias ? bias[n] : 0.0f);
            us = us * scales_up[n] + (bias_up ? bias_up[n] : 0.0f);
            out = gs / (1.0f + __expf(-gs)) * us;
        } else {
            float sum = 0.0f;
            const int r = (mm & 1) + ((c & 8) ? 2 : 0);
#pragma unroll
            for (int w = 0; w < kRingWarps; ++w) sum += s_red[w][nt][r][ln];
            out = sum * scales[n] + (bias ? bias[n] : 0.0f);
            if (epilogue == SHREWQ_EPILOGUE_RELU) out = fmaxf(out, 0.0f);
        }
        const size_t off = (size_t)m * ldy + n;
        ring_store<YT>(y + off, out);
        for (int d = 0; d < extra.n; ++d) ring_store<YT>(static_cast<YT *>(extra.p[d]) + off, out);
    }
}

}  // namespace
}  // namespace shrewq
