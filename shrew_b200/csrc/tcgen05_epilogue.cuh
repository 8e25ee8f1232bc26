// Epilogue shared by the tcgen05 forward kernels: accumulators -> scale / bias / elementwise op -> output.
//
// The accumulators of a CTA sit in tensor memory as 128 lanes (weight rows) x NCOLS columns (tokens); a
// warp can only read the 32 lanes of its quadrant (warp % 4), one lane per thread.  The output is
// row-major [token][channel], so what a thread holds after tcgen05.ld (one channel, many tokens) is the
// transpose of what a wide store needs (one token, many channels).  Each converter group (4 warps, one per
// quadrant) therefore works on chunks of CW tokens: the warps write their scaled values into a
// [CW tokens][channels] staging tile in shared memory (the pipeline stages are idle by then), and the
// group's 128 threads read the tile back as 16-byte pieces and store every token row with full-width,
// contiguous stores: to the local output and, with peer destinations (the fused all-gather), to every
// other GPU's copy at the same offset.  Rows whose base is not 16-byte aligned, and the last channels of
// a ragged edge, take element-wise stores from the same staging tile.
//
// GATED: lanes 0..63 hold the gate rows and lanes 64..127 the up rows of the same 64 channels; the up
// half parks scale * acc + bias as f32 beside the staging tile, the gate half reads it back and writes
// silu(gate) * up for 64 channels.
//
// Split-K: the values of a chunk come from the partial sums in global scratch (summed in split order)
// instead of tensor memory; everything after that is the same code.
#pragma once

#include "../../include/shrewq.h"
#include "dests.cuh"
#include "ptx_small.cuh"
#include "ptx_tcgen05.cuh"

namespace shrewq {
namespace {

struct Operands {
    const float *scales;   // per output channel
    const float *bias;     // or null
    const float *scales2;  // up matrix (GATED)
    const float *bias2;
};

constexpr int kEpiLanes = 128;           // tensor-memory lanes of a CTA
constexpr int kEpiGroupBytes = 16384;    // staging per converter group: CW x 128 channels x 4 bytes at most

template <typename YT>
__device__ __forceinline__ YT to_out(float v);
template <>
__device__ __forceinline__ float to_out<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 to_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float silu_f(float g) { return g / (1.0f + __expf(-g)); }

template <int CW>
__device__ __forceinline__ void tmem_ld_chunk(uint32_t taddr, uint32_t *r);
template <>
__device__ __forceinline__ void tmem_ld_chunk<16>(uint32_t taddr, uint32_t *r) { tc_ld16(taddr, r); }
template <>
__device__ __forceinline__ void tmem_ld_chunk<32>(uint32_t taddr, uint32_t *r) { tc_ld32(taddr, r); }

// Where a chunk's raw accumulators come from when the tile was split along K: `base` points at the
// tile's partial sums [split][NCOLS tokens][128 lanes] f32.
struct PartialSums {
    const float *base;  // null: read tensor memory
    int splits;
};

// One call per converter thread (warps of all G groups); group = converter group, quad = warp % 4.
// tmem_d: tensor-memory address of accumulator column 0 (lane field 0).  stage_base: 16-byte aligned shared
// memory, G * kEpiGroupBytes bytes, not in use by anything else.  n0 / m0: first output channel / first token
// of the tile.  `ok` false (a bounded wait gave up earlier): nothing is read from tensor memory or stored,
// but every barrier below is still reached.
template <int NCOLS, int G, bool GATED, typename YT>
__device__ __forceinline__ void epilogue_tile(uint32_t tmem_d, uint8_t *stage_base, int group, int quad, int lane, bool ok,
                                              const Operands &ops, YT *__restrict__ y, const Dests &extra, int M, int N,
                                              size_t ldy, int epilogue, int n0, int m0, PartialSums ps) {
    constexpr int CW = NCOLS >= 32 ? 32 : 16;            // tokens per chunk
    constexpr int CH = GATED ? kEpiLanes / 2 : kEpiLanes;  // output channels of the tile
    constexpr int RB = CH * (int)sizeof(YT);              // bytes of a token row in the staging tile
    constexpr int EPV = 16 / (int)sizeof(YT);             // elements per 16-byte piece
    constexpr int PPR = RB / 16;                          // pieces per token row
    constexpr int PIECES = CW * PPR;
    static_assert(NCOLS % CW == 0, "token tile is a whole number of chunks");
    static_assert(CW * RB + (GATED ? CW * CH * 4 : 0) <= kEpiGroupBytes, "staging tile fits the group's share");

    const int row = quad * 32 + lane;  // tensor-memory lane of this thread
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    const bool is_up = GATED && row >= CH;
    const int ch = GATED ? (row & (CH - 1)) : row;  // channel inside the tile
    const int n = n0 + ch;
    const bool n_ok = n < N;
    const float *sc_p = is_up ? ops.scales2 : ops.scales;
    const float *bs_p = is_up ? ops.bias2 : ops.bias;
    const float sc = n_ok ? sc_p[n] : 0.0f;
    const float bs = (n_ok && bs_p) ? bs_p[n] : 0.0f;
    const bool relu = (epilogue & 0xFF) == SHREWQ_EPILOGUE_RELU;

    uint8_t *stage = stage_base + group * kEpiGroupBytes;
    YT *out_st = reinterpret_cast<YT *>(stage);                // [CW][CH]
    float *u_st = reinterpret_cast<float *>(stage + CW * RB);  // GATED: [CW][CH] f32
    // wide stores need every destination row to start on a 16-byte boundary
    uintptr_t align_bits = reinterpret_cast<uintptr_t>(y) | (uintptr_t)(ldy * sizeof(YT));
    for (int d = 0; d < extra.n; ++d) align_bits |= reinterpret_cast<uintptr_t>(extra.p[d]);
    const bool vec_ok = (align_bits & 15) == 0;
    const int t = row;  // index inside the group, 0..127

#pragma unroll 1
    for (int c = group; c < NCOLS / CW; c += G) {
        uint32_t r[CW];
        if (ok) {
            if (ps.base) {
#pragma unroll
                for (int i = 0; i < CW; ++i) {
                    const float *p = ps.base + (size_t)(c * CW + i) * kEpiLanes + row;
                    float acc = 0.0f;
                    for (int z = 0; z < ps.splits; ++z) acc += __ldcg(p + (size_t)z * (NCOLS * kEpiLanes));
                    r[i] = __float_as_uint(acc);
                }
            } else {
                tmem_ld_chunk<CW>(tmem_d + lane_addr + c * CW, r);
                tc_wait_ld();
            }
        }
        if constexpr (GATED) {
            if (is_up && ok) {
#pragma unroll
                for (int i = 0; i < CW; ++i) u_st[i * CH + ch] = __uint_as_float(r[i]) * sc + bs;
            }
            named_bar_sync(2 + group, 128);
            if (!is_up && ok) {
#pragma unroll
                for (int i = 0; i < CW; ++i) {
                    const float g = __uint_as_float(r[i]) * sc + bs;
                    out_st[i * CH + ch] = to_out<YT>(silu_f(g) * u_st[i * CH + ch]);
                }
            }
        } else if (ok) {
#pragma unroll
            for (int i = 0; i < CW; ++i) {
                float o = __uint_as_float(r[i]) * sc + bs;
                if (relu) o = fmaxf(o, 0.0f);
                out_st[i * CH + ch] = to_out<YT>(o);
            }
        }
        named_bar_sync(2 + group, 128);  // the staging tile is complete
        if (ok) {
#pragma unroll
            for (int p = t; p < PIECES; p += 128) {
                const int tr = p / PPR, seg = p % PPR;
                const int m = m0 + c * CW + tr, nn = n0 + seg * EPV;
                if (m < M && nn < N) {
                    const size_t off = (size_t)m * ldy + nn;
                    if (vec_ok && nn + EPV <= N) {
                        const uint4 v = *reinterpret_cast<const uint4 *>(stage + tr * RB + seg * 16);
                        *reinterpret_cast<uint4 *>(y + off) = v;
                        for (int d = 0; d < extra.n; ++d) *reinterpret_cast<uint4 *>(static_cast<YT *>(extra.p[d]) + off) = v;
                    } else {
                        for (int e = 0; e < EPV && nn + e < N; ++e) {
                            const YT v = out_st[tr * CH + seg * EPV + e];
                            y[off + e] = v;
                            for (int d = 0; d < extra.n; ++d) static_cast<YT *>(extra.p[d])[off + e] = v;
                        }
                    }
                }
            }
        }
        named_bar_sync(2 + group, 128);  // the next chunk rewrites the staging tile
    }
}

}  // namespace
}  // namespace shrewq
