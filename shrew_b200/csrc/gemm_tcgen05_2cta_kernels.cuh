// Quantized Linear forward on CTA PAIRS (tcgen05.mma.cta_group::2), sm_100a only.
//
// Why: in the single-CTA kernel (gemm_tcgen05.cu) one thread issues every MMA; at ~80 cycles
// per issue plus ~380 cycles of wait / fence / commit per pipeline stage it needs ~700 cycles
// for a 128x256x64 block whose tensor work is 512 cycles.  A CTA pair doubles the work of each
// issued instruction (256 channels x 256 tokens x 16 k), and because each CTA of the pair
// holds only HALF of the activation tile (128 tokens), a 128-wide k stage fits four times in
// shared memory, which halves the per-stage overhead as well: ~1020 issue cycles for 1024
// cycles of tensor work per stage.
//
// Mapping (cluster of 2 CTAs along the channel dimension, rank r = 0 leader, 1 peer):
//   A  = 256 channels: CTA r converts rows n0 + 128 r .. +127 into ITS tensor memory.
//   B  = 256 tokens:   CTA r TMA-loads tokens m0 + 128 r .. +127 into ITS shared memory; the
//        pair MMA reads both halves through the same descriptor offset.
//   D  = 256 x 256 f32: CTA r's tensor memory holds its 128 channels x all 256 tokens.
// Barriers (mbarriers in each CTA's shared memory, same offsets in both):
//   wfull[s]  local : the CTA's own INT8 sub-blocks landed (plain TMA)          -> converters
//   xfull[s]  leader: the activation halves of BOTH CTAs landed (TMA .cta_group::2 completing
//                     on the leader's barrier; the leader expects the bytes of both)
//   aready[s] leader: 8 converter warps (4 per CTA) wrote and fenced their A stage (remote
//                     arrive from the peer)                                        -> MMA issuer
//   empty[s]  both  : tcgen05.commit.cta_group::2 multicast to both CTAs' barriers -> producers
//   accfull   both  : the same commit after the last stage                        -> epilogues
// Tensor memory is allocated and freed by both CTAs with the cta_group::2 forms, with a
// cluster barrier before the free.  Every mbarrier wait is bounded as in the single-CTA
// kernel; the cluster barriers are reached by every thread on every path.
//
// Device code only (no launch syntax, no runtime calls; PTX behind ptx_tcgen05.cuh, ptx_tcgen05_pair.cuh
// and ptx_small.cuh): it also compiles as plain C++ against the CUDA stand-in of the CPU tests
// (tests/cpu_emu/), which run the pair as two concurrent blocks over modelled cluster shared memory.
#pragma once

#include "../../include/shrewq.h"
#include "dests.cuh"
#include "ptx_small.cuh"
#include "ptx_tcgen05_pair.cuh"
#include "tcgen05_common.cuh"
#include "tcgen05_epilogue.cuh"

namespace shrewq {
namespace {

constexpr int kLanes = 128;     // TMEM lanes = weight rows per CTA
constexpr int kTokHalf = 128;   // tokens per CTA (half of the pair's tile)
constexpr int kTokPair = 256;   // MMA N
constexpr int kBlockK = 64;     // k per sub-block
constexpr int kSub = 2;         // sub-blocks per stage (128 k)
constexpr int kUmmaK = 16;
constexpr int kStages = 4;
constexpr int kGroups = 3;      // converter groups of 4 warps
constexpr int kThreads = 64 + 128 * kGroups;
constexpr int kWSub = kLanes * kBlockK;          // 8192 B of codes
constexpr int kXSub = kTokHalf * kBlockK * 2;    // 16384 B of bf16 activations
constexpr int kStageBytes = kSub * (kWSub + kXSub);  // 49152
constexpr int kXOff = kSub * kWSub;
constexpr int kAColsPerStage = kSub * (kBlockK / 2);  // 64
constexpr int kABase = kTokPair;                      // D occupies columns [0,256)
constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 1024;
static_assert(kABase + kStages * kAColsPerStage <= 512, "TMEM columns");
static_assert(kSmemBytes <= 227 * 1024, "shared memory");
static_assert(kStages * kStageBytes >= kGroups * kEpiGroupBytes, "the epilogue's staging tiles reuse the pipeline stages");

// In-kernel cycle trace (tracing build only): CTA (0,0,0), the pair's leader, stamps clock64() per role
// and pipeline round; layout and meaning as in the single-CTA kernel.
#ifdef SHREWQ_TRACE
__device__ long long *g_trace_pair = nullptr;  // [role 0..3][round 0..255][tag 0..3]
__device__ __forceinline__ void trace_rec_pair(long long *tr, int role, int kb, int tag) {
    if (tr && kb < 256) tr[(role * 256 + kb) * 4 + tag] = clock64();
}
#define TRACE2(role, kb, tag) do { if ((threadIdx.x & 31) == 0) trace_rec_pair(trace_buf, role, kb, tag); } while (0)
#define TRACE2_INIT long long *trace_buf = (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) ? g_trace_pair : nullptr;
#else
#define TRACE2(role, kb, tag)
#define TRACE2_INIT
#endif

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, Ctl *ctl, DeviceStatus *st, uint32_t role, uint32_t stage) {
    return mbar_wait_c<2>(bar, parity, ctl, st, role, stage);
}
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, Ctl *ctl, DeviceStatus *st, uint32_t role,
                                               uint32_t stage) {
    return mbar_wait_warp_c<2>(bar, parity, ctl, st, role, stage);
}

// Split-K (gridDim.z > 1): CTA (x, y, z) walks pipeline rounds [z * rounds_per_split, ...) of its tile
// and parks its raw accumulators in `partials`; the CTA arriving last at the tile's counter adds the
// slices in split order, applies the epilogue and resets the counter.  Every CTA of a pair is a tile
// of its own here (128 lanes x 256 tokens), so nothing crosses the pair in the reduction.
struct SplitK2 {
    float *partials;         // [tile][split][256 tokens][128 lanes] f32
    unsigned int *counters;  // one per CTA tile, zero between launches
    int rounds_per_split;
    // Tile-list mode (pairs_total > 0): the grid is a 1-D list of pair tiles (blockIdx.x / 2) starting at
    // tile_begin, channel pairs fastest, instead of the (channel pair, token tile) grid.  Lets one forward
    // be issued as two launches with different split counts (full waves whole, the short last wave split).
    int tile_begin;
    int pairs_total;
};

// GATED: as in the single-CTA kernel, the 128 lanes of a CTA carry 64 rows of a gate matrix (tmap_w,
// 64-row boxes) and the same 64 rows of an up matrix (tmap_w2); the epilogue pairs lane r with lane
// r + 64 and writes silu(gate) * up for 64 channels per CTA, 128 per pair.
template <typename YT, bool GATED>
__global__ void SHREWQ_CLUSTER_OF_2 __launch_bounds__(kThreads, 1)
linear_i8_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_w2,
                              const __grid_constant__ CUtensorMap tmap_x, Operands ops, YT *__restrict__ y, Dests extra,
                              int M, int N, int K, size_t ldy, int epilogue, SplitK2 sk, DeviceStatus *status) {
    constexpr int kChan = GATED ? kLanes / 2 : kLanes;  // output channels per CTA
    TRACE2_INIT
    pdl_launch_dependents();  // the next kernel of the stream may start its prologue (a no-op in an ordinary launch)
    SHREWQ_DYNAMIC_SMEM(uint8_t, smem_raw);
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *bar_area = smem + kStages * kStageBytes;
    uint64_t *bars = reinterpret_cast<uint64_t *>(bar_area);
    Ctl *ctl = reinterpret_cast<Ctl *>(bar_area + 512);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();          // 0 = leader
    int pair = blockIdx.x >> 1, m_tile = blockIdx.y;
    if (sk.pairs_total > 0) {
        const int t = sk.tile_begin + pair;
        pair = t % sk.pairs_total;
        m_tile = t / sk.pairs_total;
    } else {
        // token tiles fastest in launch order: the pairs that share a weight tile start together, so the tile
        // comes from DRAM once and from L2 for the others
        const int t = (int)blockIdx.y * (int)(gridDim.x >> 1) + pair;
        m_tile = t % (int)gridDim.y;
        pair = t / (int)gridDim.y;
    }
    const int n0 = pair * 2 * kChan + (int)rank * kChan;      // this CTA's first channel
    const int m0 = m_tile * kTokPair + (int)rank * kTokHalf;  // this CTA's first token (B half)
    const int m0_pair = m_tile * kTokPair;
    const int rounds_total = (K + kBlockK * kSub - 1) / (kBlockK * kSub);
    const int r_begin = (int)blockIdx.z * sk.rounds_per_split;
    const int rounds = min(rounds_total - r_begin, sk.rounds_per_split);  // >= 1 by construction of the grid
    int *s_is_last = reinterpret_cast<int *>(bar_area + 640);
    // barrier byte offsets
    constexpr uint32_t kWFull = 0, kXFull = kStages * 8, kAready = 2 * kStages * 8, kEmpty = 3 * kStages * 8,
                       kAcc = 4 * kStages * 8;
    const uint32_t bars_u32 = smem_u32(bars);
    const uint32_t smem_base = smem_u32(smem);

    if (threadIdx.x == 0) {
        ctl->abort_flag = 0;
        ctl->tmem_base = 0;
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bars_u32 + kWFull + s * 8, 1);
            mbar_init(bars_u32 + kXFull + s * 8, 1);    // used in the leader only
            mbar_init(bars_u32 + kAready + s * 8, 8);   // used in the leader only: 4 warps x 2 CTAs
            mbar_init(bars_u32 + kEmpty + s * 8, 1);
        }
        mbar_init(bars_u32 + kAcc, 1);
        mbar_fence_init();
    }
    if (warp == 1) {
        tc_alloc_512_pair(smem_u32(&ctl->tmem_base));
        tc_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    // both CTAs' barriers exist before anyone signals across the pair
    cluster_arrive();
    cluster_wait();
    tc_fence_after();
    const uint32_t tmem_base = ctl->tmem_base;

    if (warp == 0) {
        // ---------------- TMA producer (one thread per CTA) ----------------
        // Programmatic dependent launch: the WEIGHTS of the first stages are requested at once (they never depend on
        // an earlier kernel), the activations only when the previous kernel of the stream, whose output they may be,
        // has completed (griddepcontrol.wait; it returns at once in an ordinary launch).
        if (lane == 0) {
            auto load_w = [&](uint32_t dst, int kc, uint32_t wb) {
#pragma unroll
                for (int j = 0; j < kSub; ++j) {
                    if constexpr (GATED) {
                        tma_load_2d(dst + j * kWSub, &tmap_w, kc + j * kBlockK, n0, wb);
                        tma_load_2d(dst + j * kWSub + (kLanes / 2) * kBlockK, &tmap_w2, kc + j * kBlockK, n0, wb);
                    } else {
                        tma_load_2d(dst + j * kWSub, &tmap_w, kc + j * kBlockK, n0, wb);
                    }
                }
            };
            auto load_x = [&](uint32_t dst, int kc, uint32_t xb) {
                if (rank == 0) mbar_expect_tx(xb, 2 * kSub * kXSub);  // the halves of both CTAs
#pragma unroll
                for (int j = 0; j < kSub; ++j) tma_load_2d_pair(dst + kXOff + j * kXSub, &tmap_x, kc + j * kBlockK, m0, xb);
            };
            const int kc0 = r_begin * kSub * kBlockK;
            const int pre = rounds < kStages ? rounds : kStages;  // the stages that are free at the start
            for (int i = 0; i < pre; ++i) {
                const uint32_t wb = bars_u32 + kWFull + i * 8;
                mbar_expect_tx(wb, kSub * kWSub);
                load_w(smem_base + i * kStageBytes, kc0 + i * kSub * kBlockK, wb);
            }
            pdl_wait();
            for (int i = 0; i < pre; ++i) {
                load_x(smem_base + i * kStageBytes, kc0 + i * kSub * kBlockK, bars_u32 + kXFull + i * 8);
                TRACE2(0, i, 2);
            }
            uint32_t s = 0, ph = 0;  // the ring wrapped once: the producer now waits for the first release of a stage
            uint32_t dst = smem_base;
            int kc = kc0 + pre * kSub * kBlockK;
            for (int i = pre; i < rounds; ++i) {
                TRACE2(0, i, 0);
                if (!mbar_wait(bars_u32 + kEmpty + s * 8, ph, ctl, status, 0, s)) break;
                TRACE2(0, i, 1);
                const uint32_t wb = bars_u32 + kWFull + s * 8;
                mbar_expect_tx(wb, kSub * kWSub);
                load_w(dst, kc, wb);
                load_x(dst, kc, bars_u32 + kXFull + s * 8);
                TRACE2(0, i, 2);
                kc += kSub * kBlockK;
                dst += kStageBytes;
                if (++s == kStages) { s = 0; ph ^= 1; dst = smem_base; }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (one thread of the leader CTA) ----------------
        if (lane == 0 && rank == 0) {
            // D=f32, A=bf16 (K-major, TMEM), B=bf16 (K-major), M=256 (two CTAs), N=256
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kTokPair >> 3) << 17) |
                                       ((uint32_t)((2 * kLanes) >> 4) << 24);
            const uint64_t bdesc0 = make_b_desc(smem_base + kXOff);
            const uint32_t a0 = tmem_base + kABase;
            uint32_t s = 0, ph = 0, a_tmem = a0;
            uint64_t bdesc = bdesc0;
            bool ok = true;
            for (int i = 0; i < rounds; ++i) {
                TRACE2(1, i, 0);
                ok = mbar_wait(bars_u32 + kAready + s * 8, ph, ctl, status, 2, s) &&
                     mbar_wait(bars_u32 + kXFull + s * 8, ph, ctl, status, 1, s);
                if (!ok) break;
                TRACE2(1, i, 2);
                tc_fence_after();
#pragma unroll
                for (int j = 0; j < kSub; ++j) {
#pragma unroll
                    for (int jj = 0; jj < kBlockK / kUmmaK; ++jj)
                        tc_mma_ts_pair(tmem_base, a_tmem + j * (kBlockK / 2) + jj * (kUmmaK / 2),
                                       bdesc + (uint64_t)((j * kXSub + jj * kUmmaK * 2) >> 4), idesc,
                                       (i > 0 || j > 0 || jj > 0) ? 1u : 0u);
                }
                tc_commit_pair(bars_u32 + kEmpty + s * 8);  // frees stage s in both CTAs
                TRACE2(1, i, 3);
                a_tmem += kAColsPerStage;
                bdesc += (uint64_t)(kStageBytes >> 4);
                if (++s == kStages) { s = 0; ph ^= 1; a_tmem = a0; bdesc = bdesc0; }
            }
            if (ok) tc_commit_pair(bars_u32 + kAcc);  // accumulators complete, both CTAs
        }
        __syncwarp();
    } else {
        // ---------------- converters, then epilogue (both CTAs) ----------------
        const int group = (warp - 2) >> 2;
        const int quad = warp & 3;
        const int row = quad * 32 + lane;  // TMEM lane
        // gated tiles: gate row r (shared-memory row r) goes to lane 2r, up row r (row 64 + r) to lane 2r + 1
        const int srow = GATED ? ((row & 1) * (kLanes / 2) + (row >> 1)) : row;
        const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
        const int swz = (srow >> 1) & 3;
        const uint32_t aready_leader = map_to_cta(bars_u32 + kAready, 0);
        bool ok = true;
        // a group owns pipeline stages (s % kGroups), so that it passes through every phase of the
        // barriers it polls and a parity wait stays unambiguous under any TMA completion order
        for (int i = 0; i < rounds && ok; ++i) {
            const int s = i % kStages;
            if (s % kGroups != group) continue;
            const uint32_t ph = (i / kStages) & 1;
            if (quad == 0) TRACE2(2, i, 0);
            ok = mbar_wait_warp(bars_u32 + kWFull + s * 8, ph, ctl, status, 3, s);
            if (!ok) break;
            tc_fence_after();
            if (quad == 0) TRACE2(2, i, 1);
#pragma unroll
            for (int j = 0; j < kSub; ++j) {
                uint32_t packed[32];
                convert_row64(smem + s * kStageBytes + j * kWSub + srow * kBlockK, swz, packed);
                tc_st32(tmem_base + lane_addr + kABase + s * kAColsPerStage + j * (kBlockK / 2), packed);
            }
            if (quad == 0) TRACE2(2, i, 2);
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(aready_leader + s * 8);
            if (quad == 0) TRACE2(2, i, 3);
        }
        // epilogue: this CTA's channels x the pair's 256 tokens; 16-column chunks dealt to the groups
        pdl_wait();  // outputs, partial sums and counters may still be in use by the previous kernel of the stream
        if (ok) ok = mbar_wait_warp(bars_u32 + kAcc, 0, ctl, status, 4, 0);
        if (ok) tc_fence_after();
        const int splits = (int)gridDim.z;
        if (splits > 1) {
            const size_t tile = (size_t)blockIdx.y * gridDim.x + blockIdx.x;
            float *mine = sk.partials + (tile * splits + blockIdx.z) * (size_t)(kTokPair * kLanes);
            if (ok) {
                dump_partials<kTokPair, kGroups>(tmem_base, mine, group, quad, lane);
            }
            __threadfence();
            named_bar_sync(1, 128 * kGroups);
            if (threadIdx.x == 64) {
                const unsigned int old = atomicAdd(sk.counters + tile, 1u);
                *s_is_last = (old == (unsigned int)(splits - 1));
            }
            named_bar_sync(1, 128 * kGroups);
            if (*s_is_last) {
                __threadfence();
                epilogue_tile<kTokPair, kGroups, GATED, YT>(tmem_base, smem, group, quad, lane, ok, ops, y, extra, M, N, ldy, epilogue,
                                                            n0, m0_pair,
                                                            PartialSums{sk.partials + tile * splits * (size_t)(kTokPair * kLanes), splits, (size_t)(kTokPair * kLanes)});
                named_bar_sync(1, 128 * kGroups);
                if (threadIdx.x == 64) sk.counters[tile] = 0;  // ready for the next launch
            }
        } else {
            epilogue_tile<kTokPair, kGroups, GATED, YT>(tmem_base, smem, group, quad, lane, ok, ops, y, extra, M, N, ldy, epilogue, n0,
                                                        m0_pair, PartialSums{nullptr, 0, 0});
        }
    }

    // ---------------- teardown: both CTAs are done with tensor memory before it is freed ----------------
    tc_fence_before();
    __syncthreads();
    cluster_arrive();
    cluster_wait();
    if (warp == 1) {
        if (ctl->abort_flag) {
            for (int i = 0; i < 2000; ++i) __nanosleep(1000);
        }
        tc_fence_after();
        __syncwarp();
        tc_dealloc_512_pair(tmem_base);
    }
}

}  // namespace
}  // namespace shrewq
