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
// GATED: even lanes hold the gate rows and odd lanes the up rows of the same 64 channels (the converter
// warps interleave the two 64-row boxes when they fill tensor memory), so a channel's two values meet
// with one shuffle between neighbouring lanes: no shared-memory exchange, no extra barrier.
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
constexpr int kEpiGroupBytes = 16384;    // staging per converter group: 32 tokens x 128 channels x 4 bytes at most

template <typename YT>
__device__ __forceinline__ YT to_out(float v);
template <>
__device__ __forceinline__ float to_out<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 to_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// silu(g) = g / (1 + e^-g); the fast division is good to ~2 ulp, far inside every tolerance of this path
__device__ __forceinline__ float silu_f(float g) { return __fdividef(g, 1.0f + __expf(-g)); }

template <int CW>
__device__ __forceinline__ void tmem_ld_chunk(uint32_t taddr, uint32_t *r);
template <>
__device__ __forceinline__ void tmem_ld_chunk<16>(uint32_t taddr, uint32_t *r) { tc_ld16(taddr, r); }
template <>
__device__ __forceinline__ void tmem_ld_chunk<32>(uint32_t taddr, uint32_t *r) { tc_ld32(taddr, r); }

// Where a chunk's raw accumulators come from when the tile was split along K: null base = tensor memory;
// otherwise `pieces` slices of [NCOLS tokens][128 lanes] f32, `stride` floats apart, added in piece order.
struct PartialSums {
    const float *base;
    int pieces;
    size_t stride;
};

template <int NCOLS>
__device__ __forceinline__ const float *partial_piece(const PartialSums &ps, int z) {
    return ps.base + (size_t)z * ps.stride;
}

// Raw accumulators of a CTA -> scratch [NCOLS tokens][128 lanes] f32 (a piece of a tile that was split along K).
// One call per converter thread; the next chunk's tensor-memory load is in flight while this one is stored.
template <int NCOLS, int G>
__device__ __forceinline__ void dump_partials(uint32_t tmem_d, float *dst, int group, int quad, int lane) {
    constexpr int NCH = NCOLS / 16;
    const int row = quad * 32 + lane;
    const uint32_t taddr = tmem_d + ((uint32_t)(quad * 32) << 16);
    if (group >= NCH) return;
    uint32_t r[16];
    tc_ld16(taddr + group * 16, r);
    tc_wait_ld();
#pragma unroll 1
    for (int c = group; c < NCH; c += G) {
        float v[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
        const bool more = c + G < NCH;
        if (more) tc_ld16(taddr + (c + G) * 16, r);
#pragma unroll
        for (int i = 0; i < 16; ++i) __stcg(dst + (c * 16 + i) * kEpiLanes + row, v[i]);
        if (more) tc_wait_ld();
    }
}

// One call per converter thread (warps of all G groups); group = converter group, quad = warp % 4.
// tmem_d: tensor-memory address of accumulator column 0 (lane field 0).  stage_base: 16-byte aligned shared
// memory, G * GROUP_BYTES bytes, not in use by anything else.  n0 / m0: first output channel / first token
// of the tile.  `ok` false (a bounded wait gave up earlier): nothing is read from tensor memory or stored,
// but every barrier below is still reached.
// GROUP_BYTES: the staging share of a group; chunks are 32 tokens where 32 token rows fit it, else 16.
//
// Per chunk: the raw values of the NEXT chunk are requested (tcgen05.ld, or the loads of the first two partial
// pieces) before this chunk is processed, so their latency hides behind the arithmetic, the staging and the stores.
// GATED tiles split the SiLU work evenly: the gate lane (even) keeps the first half of the chunk's tokens and
// hands its values of the second half to the up lane (odd) of the same channel, the up lane hands over its first
// half, and each computes silu(gate) * up for its half.
template <int NCOLS, int G, bool GATED, typename YT, int GROUP_BYTES = kEpiGroupBytes>
__device__ __forceinline__ void epilogue_tile(uint32_t tmem_d, uint8_t *stage_base, int group, int quad, int lane, bool ok,
                                              const Operands &ops, YT *__restrict__ y, const Dests &extra, int M, int N,
                                              size_t ldy, int epilogue, int n0, int m0, PartialSums ps) {
    constexpr int CH = GATED ? kEpiLanes / 2 : kEpiLanes;  // output channels of the tile
    constexpr int RB = CH * (int)sizeof(YT);              // bytes of a token row in the staging tile
    constexpr int kPerToken = RB;                         // staging bytes per token
    constexpr int CW = (NCOLS >= 32 && 32 * kPerToken <= GROUP_BYTES) ? 32 : 16;  // tokens per chunk
    constexpr int EPV = 16 / (int)sizeof(YT);             // elements per 16-byte piece
    constexpr int PPR = RB / 16;                          // pieces per token row
    constexpr int PIECES = CW * PPR;
    constexpr int NCH = NCOLS / CW;
    constexpr bool kPrefetchPieces = CW == 16;            // two raw partial pieces held in registers across a chunk
    static_assert(NCOLS % CW == 0, "token tile is a whole number of chunks");
    static_assert(CW * kPerToken <= GROUP_BYTES, "staging tile fits the group's share");

    const int row = quad * 32 + lane;  // tensor-memory lane of this thread
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    const bool is_up = GATED && (row & 1);
    const int ch = GATED ? (row >> 1) : row;  // channel inside the tile
    const int n = n0 + ch;
    const bool n_ok = n < N;
    const float *sc_p = is_up ? ops.scales2 : ops.scales;
    const float *bs_p = is_up ? ops.bias2 : ops.bias;
    const float sc = n_ok ? sc_p[n] : 0.0f;
    const float bs = (n_ok && bs_p) ? bs_p[n] : 0.0f;
    const bool relu = (epilogue & 0xFF) == SHREWQ_EPILOGUE_RELU;

    uint8_t *stage = stage_base + group * GROUP_BYTES;
    YT *out_st = reinterpret_cast<YT *>(stage);                // [CW][CH]
    // wide stores need every destination row to start on a 16-byte boundary
    uintptr_t align_bits = reinterpret_cast<uintptr_t>(y) | (uintptr_t)(ldy * sizeof(YT));
    for (int d = 0; d < extra.n; ++d) align_bits |= reinterpret_cast<uintptr_t>(extra.p[d]);
    const bool vec_ok = (align_bits & 15) == 0;
    const int t = row;  // index inside the group, 0..127
    const bool from_tmem = ps.base == nullptr;
    const float *piece0 = nullptr, *piece1 = nullptr;
    if (!from_tmem) {
        piece0 = partial_piece<NCOLS>(ps, 0) + row;
        piece1 = ps.pieces > 1 ? partial_piece<NCOLS>(ps, 1) + row : nullptr;
    }

    // Request the raw values of chunk c_: ra, and rb when two pieces are prefetched.  (A macro, not a lambda: the
    // register arrays must not have their address taken.)
    uint32_t ra[CW];
    float rb[kPrefetchPieces ? CW : 1];
#define SHREWQ_EPI_REQUEST(c_)                                                                                        \
    do {                                                                                                              \
        if (from_tmem) {                                                                                              \
            tmem_ld_chunk<CW>(tmem_d + lane_addr + (c_) * CW, ra);                                                    \
        } else {                                                                                                      \
            _Pragma("unroll") for (int i_ = 0; i_ < CW; ++i_)                                                         \
                ra[i_] = __float_as_uint(ld_cg_ordered(piece0 + (size_t)((c_) * CW + i_) * kEpiLanes));                      \
            if constexpr (kPrefetchPieces) {                                                                          \
                _Pragma("unroll") for (int i_ = 0; i_ < CW; ++i_)                                                     \
                    rb[i_] = piece1 ? ld_cg_ordered(piece1 + (size_t)((c_) * CW + i_) * kEpiLanes) : 0.0f;                   \
            }                                                                                                         \
        }                                                                                                             \
    } while (0)
    if (ok && group < NCH) SHREWQ_EPI_REQUEST(group);

#pragma unroll 1
    for (int c = group; c < NCH; c += G) {
        float v[CW];  // scale * acc + bias of this thread's lane, CW tokens
        if (ok) {
            if (from_tmem) {
                tc_wait_ld();
#pragma unroll
                for (int i = 0; i < CW; ++i) v[i] = __uint_as_float(ra[i]);
            } else {
                // the pieces are added in piece order, whatever was prefetched
#pragma unroll
                for (int i = 0; i < CW; ++i) v[i] = __uint_as_float(ra[i]);
                int z = 1;
                if constexpr (kPrefetchPieces) {
                    if (piece1) {
#pragma unroll
                        for (int i = 0; i < CW; ++i) v[i] += rb[i];
                    }
                    z = 2;
                }
                for (; z < ps.pieces; ++z) {
                    const float *p = partial_piece<NCOLS>(ps, z) + (size_t)(c * CW) * kEpiLanes + row;
                    float piece[CW];  // all loads of the piece first, then the additions
#pragma unroll
                    for (int i = 0; i < CW; ++i) piece[i] = ld_cg_ordered(p + i * kEpiLanes);
#pragma unroll
                    for (int i = 0; i < CW; ++i) v[i] += piece[i];
                }
            }
#pragma unroll
            for (int i = 0; i < CW; ++i) v[i] = v[i] * sc + bs;
            if (c + G < NCH) SHREWQ_EPI_REQUEST(c + G);
        }
        if constexpr (GATED) {
            // neighbouring lanes swap halves: the up lane gives tokens [0, CW/2), the gate lane tokens [CW/2, CW)
            // (register arrays are indexed with constants only; the choice between the halves is a select)
            const int keep0 = is_up ? CW / 2 : 0;
            if (ok) {
#pragma unroll
                for (int i = 0; i < CW / 2; ++i) {
                    const float other = __shfl_xor_sync(0xFFFFFFFFu, is_up ? v[i] : v[CW / 2 + i], 1);
                    const float mine = is_up ? v[CW / 2 + i] : v[i];
                    const float g = is_up ? other : mine, u = is_up ? mine : other;
                    out_st[(keep0 + i) * CH + ch] = to_out<YT>(silu_f(g) * u);
                }
            }
        } else if (ok) {
#pragma unroll
            for (int i = 0; i < CW; ++i) {
                float o = v[i];
                if (relu) o = fmaxf(o, 0.0f);
                out_st[i * CH + ch] = to_out<YT>(o);
            }
        }
        named_bar_sync(2 + group, 128);  // the staging tile is complete
        if (ok && vec_ok) {
#pragma unroll
            for (int p = t; p < PIECES; p += 128) {
                const int tr = p / PPR, seg = p % PPR;
                const int m = m0 + c * CW + tr, nn = n0 + seg * EPV;
                if (m < M && nn < N) {
                    const size_t off = (size_t)m * ldy + nn;
                    if (nn + EPV <= N) {
                        const uint4 w = *reinterpret_cast<const uint4 *>(stage + tr * RB + seg * 16);
                        *reinterpret_cast<uint4 *>(y + off) = w;
                        for (int d = 0; d < extra.n; ++d) *reinterpret_cast<uint4 *>(static_cast<YT *>(extra.p[d]) + off) = w;
                    } else {
                        for (int e = 0; e < EPV && nn + e < N; ++e) {
                            const YT w = out_st[tr * CH + seg * EPV + e];
                            y[off + e] = w;
                            for (int d = 0; d < extra.n; ++d) static_cast<YT *>(extra.p[d])[off + e] = w;
                        }
                    }
                }
            }
        } else if (ok) {
            // rows that do not start on 16-byte boundaries (e.g. 50257 f32 channels): element stores, consecutive
            // threads on consecutive channels of one token, so that every store instruction writes whole sectors
#pragma unroll 4
            for (int e = t; e < CW * CH; e += 128) {
                const int tr = e / CH, cn = e % CH;
                const int m = m0 + c * CW + tr, nn = n0 + cn;
                if (m < M && nn < N) {
                    const size_t off = (size_t)m * ldy + nn;
                    const YT w = out_st[tr * CH + cn];
                    y[off] = w;
                    for (int d = 0; d < extra.n; ++d) static_cast<YT *>(extra.p[d])[off] = w;
                }
            }
        }
        named_bar_sync(2 + group, 128);  // the next chunk rewrites the staging tile
    }
#undef SHREWQ_EPI_REQUEST
}

}  // namespace
}  // namespace shrewq
