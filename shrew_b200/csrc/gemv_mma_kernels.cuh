// Weight-only INT8 forward for small batches (M <= 64) on warp-level MMA, sm_100a.
//
// The default for 3..32 tokens where the ring kernel (gemv_ring_kernels.cuh) does not win; also the forward of
// packed INT4 weights.  Its index arithmetic is also checked on the CPU (tests/test_mma_layout.py).
//
// Why it exists: for 4 < M <= 64 the layer is HBM-bound, but the tcgen05 kernel feeds the
// tensor core from ONE issuing thread per CTA (about 80 cycles per instruction, each covering
// 2 KB of codes), which caps an SM's stream rate below what HBM delivers, and the CUDA-core
// GEMV needs M FMAs per code.  Here every warp loads its own codes straight from global
// memory into registers (no shared-memory staging, no barrier hand-offs), widens them, and
// issues mma.sync.m16n8k16 (bf16): 64 warps per SM issue in parallel and an MMA costs the
// same for 1 or 16 tokens.
//
// Mapping (per warp, per 64-wide k-block): lane (g = lane/4, t = lane%4) loads the 16 codes
// W[n0 + 8*nb + g][kb*64 + 16t .. +15] for each of its NB channel blocks, and the 16
// activations x[m][kb*64 + 16t .. +15] for token rows m = 16*mt + g and m + 8.  MMA step j
// (0..3) uses codes 4j..4j+3 and activations 4j..4j+3 of those runs: operand slot 2t+e holds
// k = 16t + 4j + e and slot 2t+8+e holds k = 16t + 4j + 2 + e, for A and B alike, so the 16
// slots of one instruction cover 16 distinct k of the block and four instructions cover all
// 64 (a dot product does not care about the order of k).
// A CTA of 8 warps owns 16 channels (8 when gated: a gate block and an up block); the warps
// split K in 64-wide blocks and their accumulators are summed through shared memory.
//
// F16 variant ("mma-f16").  Widening a code to bf16 costs 2.5 instructions (byte-permute into
// an f32 magic number, subtract, pack two f32 into bf16x2), which at batch 1-4 makes the
// kernel issue-bound like the CUDA-core GEMV.  To f16 it costs 1: a byte-permute builds the
// halves 0x6400 | u (= 1024 + u exactly, u = code + 128), one packed subtract of 1152 leaves
// the code.  The MMA then needs f16 activations, and f16 has 5 exponent bits where bf16 has
// 8, so a small kernel first rescales each token row by a power of two chosen from the row's
// largest magnitude (2^14 <= amax * 2^s < 2^15) and converts it to f16.  A bf16 value has 8
// significant bits and f16 keeps 11 down to 2^-14 (fewer below, none under 2^-24), so every
// element within 2^-31 of the row's amax converts exactly; a smaller one is rounded with an
// error of at most amax * 2^-39 (half an f16 subnormal step), so a dot product over K codes is
// off by at most K * 127 * amax * 2^-39 in the rescaled row's units: for K = 16384 that is
// 2^-18 * amax, below the f32 rounding of a sum whose terms reach 127 * amax.  The epilogue
// multiplies the sum by 2^-s (ldexp).
//
// Device code only (no launch syntax, no runtime calls, PTX behind ptx_small.cuh): it also compiles
// as plain C++ against the CUDA stand-in of the CPU tests (tests/cpu_emu/), which run these
// kernels with an emulated mma.sync and compare their results with the reference arithmetic.
#pragma once

#include "../../include/shrewq.h"
#include "dests.cuh"
#include "ptx_small.cuh"
#include "activation_f16.cuh"

namespace shrewq {
namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int NB = 2;  // channel blocks of 8 per warp

// 4 INT8 codes -> two packed bf16x2 words, exactly (see gemm_tcgen05.cu for the trick)
__device__ __forceinline__ void cvt_i8x4_bf16(uint32_t w, uint32_t &lo, uint32_t &hi) {
    const uint32_t u = w ^ 0x80808080u;
    const float f0 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7440)) - 8388736.0f;
    const float f1 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7441)) - 8388736.0f;
    const float f2 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7442)) - 8388736.0f;
    const float f3 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7443)) - 8388736.0f;
    lo = pack_bf16x2_rn(f1, f0);
    hi = pack_bf16x2_rn(f3, f2);
}

// 4 INT8 codes -> two packed f16x2 words, exactly: (1024 + (code + 128)) - 1152
__device__ __forceinline__ void cvt_i8x4_f16(uint32_t w, uint32_t &lo, uint32_t &hi) {
    const uint32_t u = w ^ 0x80808080u;
    const uint32_t h01 = __byte_perm(u, 0x64646464u, 0x4140);  // halves 0x64:u0, 0x64:u1
    const uint32_t h23 = __byte_perm(u, 0x64646464u, 0x4342);
    lo = sub_f16x2(h01, 0x64806480u);
    hi = sub_f16x2(h23, 0x64806480u);
}

// 8 packed INT4 codes (one 32-bit word; nibble i = code i + 8) -> four f16x2 words, exactly:
// (1024 + nibble) - 1032.  Word j of the result holds codes (j, j + 4): a mask and an OR place two
// nibbles that sit 16 bits apart into the two halves at once.
__device__ __forceinline__ void cvt_i4x8_f16(uint32_t w, uint32_t *p) {
    p[0] = sub_f16x2((w & 0x000F000Fu) | 0x64006400u, 0x64086408u);
    p[1] = sub_f16x2(((w >> 4) & 0x000F000Fu) | 0x64006400u, 0x64086408u);
    p[2] = sub_f16x2(((w >> 8) & 0x000F000Fu) | 0x64006400u, 0x64086408u);
    p[3] = sub_f16x2(((w >> 12) & 0x000F000Fu) | 0x64006400u, 0x64086408u);
}

// The unpacking above pairs codes (j, j + 4), so with packed INT4 weights the activations are stored in
// the order 0 4 1 5 2 6 3 7 inside every group of 8 and a contiguous load yields the matching pairs.

__device__ __forceinline__ float silu(float g) { return g / (1.0f + __expf(-g)); }

template <typename YT>
__device__ __forceinline__ void put(YT *p, float v);
template <>
__device__ __forceinline__ void put<float>(float *p, float v) { *p = v; }
template <>
__device__ __forceinline__ void put<__nv_bfloat16>(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }

constexpr int kStageMaxTokens = 4;            // in-CTA staging (XS) covers M <= 4 ...
// ... when the f16 copy of x fits this much dynamic shared memory: with the kernel's ~8.2 KB of static shared
// memory (the cross-warp reduction) the CTA stays below the 48 KB that need no opt-in attribute
constexpr int kStageMaxBytes = 36 * 1024;

// MT16: token tiles of 16 (M <= 16*MT16).  K must be a multiple of 64.
// F16: the activations are f16, rescaled per token row by 2^shift[m]; else bf16 as given.
// XS (with F16, MT16 == 1, M <= 4): x is the caller's bf16 tensor and every CTA converts it into its
// own shared memory first (x_to_f16_kernel's arithmetic), so that a batch-1..4 forward is one launch
// with no kernel-to-kernel dependency; otherwise x / xshift come from x_to_f16_kernel.
// W4 (with F16): q / q_up hold packed INT4 codes, K/2 bytes per row (byte j = codes 2j in the low and
// 2j+1 in the high nibble, each stored as code + 8); a lane then reads 32 codes per 16-byte load, a
// k-block is 128 wide, and x must be in that permuted order (x_to_f16_kernel with perm = 1, or staged here).
template <int MT16, typename YT, bool GATED, bool F16, bool XS, bool W4 = false>
__global__ void __launch_bounds__(kThreads)
gemv_mma_kernel(const int8_t *__restrict__ q, const float *__restrict__ scales, const float *__restrict__ bias,
                const int8_t *__restrict__ q_up, const float *__restrict__ scales_up,
                const float *__restrict__ bias_up, const uint16_t *__restrict__ x, const int *__restrict__ xshift,
                YT *__restrict__ y, Dests extra, int M, int N, int K, size_t ldy, int epilogue) {
    constexpr int kChan = GATED ? 8 : 8 * NB;  // output channels per CTA
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    static_assert(!W4 || F16, "packed INT4 weights go with f16 operands");
    constexpr int kRun = W4 ? 32 : 16;        // codes (and activations) per lane per k-block
    constexpr int kXWords = kRun / 2;         // 32-bit words of activations per lane, row and k-block
    const int n0 = blockIdx.x * kChan;
    const int kblocks = K / (4 * kRun);
    const size_t wrow_bytes = W4 ? (size_t)K / 2 : (size_t)K;

    // the row of codes this lane reads for each channel block
    const int8_t *wrow[NB];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
        int n = n0 + (GATED ? 0 : nb * 8) + g;
        n = n < N ? n : N - 1;  // clamp: duplicates are computed and dropped
        wrow[nb] = ((GATED && nb == 1) ? q_up : q) + (size_t)n * wrow_bytes + 16 * t;
    }
    // XS: the first kPrefetch k-blocks of this warp's codes are requested BEFORE the activations are
    // staged: the weights do not depend on them, and the staging (two dependent passes over x with
    // block-wide barriers, ~2 us) would otherwise delay the start of the weight stream, which is the
    // whole kernel at batch 1-4.
    constexpr int kPrefetch = XS ? 4 : 0;
    uint4 pre[kPrefetch > 0 ? kPrefetch : 1][NB];
    if constexpr (XS) {
        // (both calls do nothing unless the launch asked for programmatic stream serialization)
        pdl_launch_dependents();  // the next kernel of the stream may start its own prologue
#pragma unroll
        for (int p = 0; p < kPrefetch; ++p) {
            const int kb = warp + p * kWarps;
            if (kb < kblocks) {
#pragma unroll
                for (int nb = 0; nb < NB; ++nb) pre[p][nb] = ld_stream_16(wrow[nb] + ((size_t)kb << 6));
            }
        }
        // the activations may be the previous kernel's output, and the output buffer may still be
        // read by it: wait for it here, with this kernel's first weights already on their way
        pdl_wait();
    }
    // the activation rows this lane reads for each token tile (null = padding row)
    const uint16_t *xlo[MT16], *xhi[MT16];
    __shared__ int s_shift[kStageMaxTokens];
    if constexpr (XS) {
        static_assert(F16 && MT16 == 1, "in-CTA staging is the f16, single token tile case");
        SHREWQ_DYNAMIC_SMEM(uint16_t, xs);  // [M][K] f16 bits
        __shared__ float s_amax[kStageMaxTokens][kWarps];
        const int chunks = K >> 3;  // 8 values = 16 bytes
        for (int m = 0; m < M; ++m) {
            float a = 0.0f;
            for (int c = threadIdx.x; c < chunks; c += kThreads) {
                const uint4 v = __ldg(reinterpret_cast<const uint4 *>(x + (size_t)m * K) + c);
                const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    a = fmaxf(a, fabsf(__uint_as_float(w4[i] << 16)));          // fmaxf drops NaN
                    a = fmaxf(a, fabsf(__uint_as_float(w4[i] & 0xFFFF0000u)));
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xFFFFFFFFu, a, o));
            if (lane == 0) s_amax[m][warp] = a;
        }
        __syncthreads();
        if ((int)threadIdx.x < M) {
            float a = s_amax[threadIdx.x][0];
#pragma unroll
            for (int w = 1; w < kWarps; ++w) a = fmaxf(a, s_amax[threadIdx.x][w]);
            s_shift[threadIdx.x] = shift_of_amax(a);
        }
        __syncthreads();
        for (int m = 0; m < M; ++m) {
            const int sh = s_shift[m];
            for (int c = threadIdx.x; c < chunks; c += kThreads) {
                const uint4 v = __ldg(reinterpret_cast<const uint4 *>(x + (size_t)m * K) + c);
                const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
                uint32_t o4[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const __half lo = __float2half_rn(ldexpf(__uint_as_float(w4[i] << 16), sh));
                    const __half hi = __float2half_rn(ldexpf(__uint_as_float(w4[i] & 0xFFFF0000u), sh));
                    o4[i] = (uint32_t)__half_as_ushort(lo) | ((uint32_t)__half_as_ushort(hi) << 16);
                }
                if constexpr (W4) {  // the chunk is one group of 8: store it as 0 4 1 5 2 6 3 7
                    const uint32_t e[8] = {o4[0] & 0xFFFF, o4[0] >> 16, o4[1] & 0xFFFF, o4[1] >> 16,
                                           o4[2] & 0xFFFF, o4[2] >> 16, o4[3] & 0xFFFF, o4[3] >> 16};
                    o4[0] = e[0] | (e[4] << 16);
                    o4[1] = e[1] | (e[5] << 16);
                    o4[2] = e[2] | (e[6] << 16);
                    o4[3] = e[3] | (e[7] << 16);
                }
                reinterpret_cast<uint4 *>(xs + (size_t)m * K)[c] = make_uint4(o4[0], o4[1], o4[2], o4[3]);
            }
        }
        __syncthreads();
        xlo[0] = g < M ? xs + (size_t)g * K + kRun * t : nullptr;
        xhi[0] = nullptr;
    } else {
#pragma unroll
        for (int mt = 0; mt < MT16; ++mt) {
            const int m = mt * 16 + g;
            xlo[mt] = m < M ? x + (size_t)m * K + kRun * t : nullptr;
            xhi[mt] = m + 8 < M ? x + (size_t)(m + 8) * K + kRun * t : nullptr;
        }
    }

    float acc[MT16][NB][4];
#pragma unroll
    for (int mt = 0; mt < MT16; ++mt)
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
#pragma unroll
            for (int r = 0; r < 4; ++r) acc[mt][nb][r] = 0.0f;

    // one k-block: wv = this lane's 16 bytes of codes per channel block (64 bytes per row and k-block,
    // INT8 or packed INT4 alike)
    auto k_block = [&](int kb, const uint4 (&wv)[NB]) {
        const size_t koff = (size_t)kb * (4 * kRun);              // activations: elements
        // kRun activations = kXWords packed words per row
        uint32_t al[MT16][kXWords], ah[MT16][kXWords];
#pragma unroll
        for (int mt = 0; mt < MT16; ++mt) {
#pragma unroll
            for (int v4 = 0; v4 < kXWords / 4; ++v4) {
                const uint4 z = make_uint4(0, 0, 0, 0);
                uint4 l = z, h = z;
                if constexpr (XS) {  // shared memory: plain loads (the read-only global path does not apply)
                    if (xlo[mt]) l = *(reinterpret_cast<const uint4 *>(xlo[mt] + koff) + v4);
                } else {
                    if (xlo[mt]) l = __ldg(reinterpret_cast<const uint4 *>(xlo[mt] + koff) + v4);
                    if (xhi[mt]) h = __ldg(reinterpret_cast<const uint4 *>(xhi[mt] + koff) + v4);
                }
                al[mt][4 * v4 + 0] = l.x; al[mt][4 * v4 + 1] = l.y; al[mt][4 * v4 + 2] = l.z; al[mt][4 * v4 + 3] = l.w;
                ah[mt][4 * v4 + 0] = h.x; ah[mt][4 * v4 + 1] = h.y; ah[mt][4 * v4 + 2] = h.z; ah[mt][4 * v4 + 3] = h.w;
            }
        }
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
            const uint32_t w4[4] = {wv[nb].x, wv[nb].y, wv[nb].z, wv[nb].w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if constexpr (W4) {
                    uint32_t p[4];  // codes (0,4) (1,5) (2,6) (3,7) of word j; activation words 4j..4j+3 pair the same k
                    cvt_i4x8_f16(w4[j], p);
#pragma unroll
                    for (int mt = 0; mt < MT16; ++mt) {
                        mma_f16_16816(acc[mt][nb], al[mt][4 * j], ah[mt][4 * j], al[mt][4 * j + 1], ah[mt][4 * j + 1], p[0], p[1]);
                        mma_f16_16816(acc[mt][nb], al[mt][4 * j + 2], ah[mt][4 * j + 2], al[mt][4 * j + 3], ah[mt][4 * j + 3], p[2], p[3]);
                    }
                } else {
                    uint32_t b0, b1;  // codes 4j,4j+1 | 4j+2,4j+3 of this lane's run
                    if constexpr (F16) cvt_i8x4_f16(w4[j], b0, b1);
                    else cvt_i8x4_bf16(w4[j], b0, b1);
#pragma unroll
                    for (int mt = 0; mt < MT16; ++mt) {
                        if constexpr (F16)
                            mma_f16_16816(acc[mt][nb], al[mt][2 * j], ah[mt][2 * j], al[mt][2 * j + 1], ah[mt][2 * j + 1], b0, b1);
                        else
                            mma_bf16_16816(acc[mt][nb], al[mt][2 * j], ah[mt][2 * j], al[mt][2 * j + 1], ah[mt][2 * j + 1], b0, b1);
                    }
                }
            }
        }
    };

    if constexpr (XS) {
#pragma unroll
        for (int p = 0; p < kPrefetch; ++p) {
            const int kb = warp + p * kWarps;
            if (kb < kblocks) k_block(kb, pre[p]);
        }
    }
#pragma unroll 2
    for (int kb = warp + kPrefetch * kWarps; kb < kblocks; kb += kWarps) {
        uint4 wv[NB];
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) wv[nb] = ld_stream_16(wrow[nb] + ((size_t)kb << 6));
        k_block(kb, wv);
    }

    // sum the 8 warps' accumulators through shared memory
    __shared__ float s_red[kWarps][MT16 * NB * 4][32];
#pragma unroll
    for (int mt = 0; mt < MT16; ++mt)
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
#pragma unroll
            for (int r = 0; r < 4; ++r) s_red[warp][(mt * NB + nb) * 4 + r][lane] = acc[mt][nb][r];
    __syncthreads();

    // accumulator element (mt, nb, lane, r) is token 16*mt + lane/4 + (r >= 2 ? 8 : 0),
    // channel 8*nb + 2*(lane%4) + (r & 1) of the block
    constexpr int kOutBlocks = GATED ? 1 : NB;
    for (int i = threadIdx.x; i < MT16 * kOutBlocks * 4 * 32; i += kThreads) {
        const int ln = i & 31, r = (i >> 5) & 3, rest = i >> 7;
        const int nb = rest % kOutBlocks, mt = rest / kOutBlocks;
        const int m = mt * 16 + (ln >> 2) + ((r & 2) ? 8 : 0);
        const int n = n0 + nb * 8 + 2 * (ln & 3) + (r & 1);
        if (m >= M || n >= N) continue;
        float out;
        const int back = F16 ? -(XS ? s_shift[m] : xshift[m]) : 0;  // undo the row's power-of-two rescale
        if constexpr (GATED) {
            float gs = 0.0f, us = 0.0f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                gs += s_red[w][(mt * NB + 0) * 4 + r][ln];
                us += s_red[w][(mt * NB + 1) * 4 + r][ln];
            }
            // scale first, then undo the row's rescale: the raw sum times 2^-s alone could overflow
            gs = gs * scales[n];
            us = us * scales_up[n];
            if constexpr (F16) { gs = ldexpf(gs, back); us = ldexpf(us, back); }
            gs += bias ? bias[n] : 0.0f;
            us += bias_up ? bias_up[n] : 0.0f;
            out = silu(gs) * us;
        } else {
            float s = 0.0f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) s += s_red[w][(mt * NB + nb) * 4 + r][ln];
            s = s * scales[n];
            if constexpr (F16) s = ldexpf(s, back);
            out = s + (bias ? bias[n] : 0.0f);
            if (epilogue == SHREWQ_EPILOGUE_RELU) out = fmaxf(out, 0.0f);
        }
        const size_t off = (size_t)m * ldy + n;
        put<YT>(y + off, out);
        for (int d = 0; d < extra.n; ++d) put<YT>(static_cast<YT *>(extra.p[d]) + off, out);
    }
}

}  // namespace
}  // namespace shrewq
