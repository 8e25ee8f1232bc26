// Quantized Linear forward on the 5th-generation tensor cores (tcgen05 + TMEM + TMA),
// sm_100a only.
//
//   y[m,n] = epi( scale[n] * sum_k q[n,k] * x[m,k] + bias[n] )       (quantize.rs:463-476)
//
// Mapping.  The MMA computes D[128 x TOK] = A[128 x 16] * B[TOK x 16]^T per instruction:
//   A  = 128 weight rows (output channels).  The INT8 codes are TMA-loaded into shared
//        memory, widened to bf16 in registers (exact: |q| <= 127 fits bf16's 8-bit
//        significand) and written with tcgen05.st into TENSOR MEMORY, from where the MMA
//        reads its A operand.  The expanded weights therefore never occupy shared memory
//        and cost no shared-memory bandwidth on the MMA side.
//   B  = TOK tokens of bf16 activations, TMA-loaded with the 128-byte swizzle and read by
//        the MMA through a shared-memory descriptor (K-major).
//   D  = f32 accumulators in TMEM: lane = output channel, column = token.
// The epilogue (tcgen05_epilogue.cuh) reads D with tcgen05.ld, applies the per-channel scale, bias and
// the elementwise op, transposes through shared memory and stores whole token rows with 16-byte stores.
//
// GATED: the 128 lanes carry 64 rows of a gate matrix and the same 64 rows of an up matrix
// (two 64-row TMA boxes per sub-block), interleaved by the converters: gate row r in lane 2r, up row r in
// lane 2r+1; the epilogue pairs neighbouring lanes with a shuffle and writes silu(gate)*up for 64 channels.
//
// XSPLIT (f32 activations): x arrives as two bf16 matrices hi = bf16(x) and lo = bf16(x - hi), stacked
// as rows [0,M) and [M,2M) of one array; a stage holds both token tiles and every k-step issues two
// MMAs into the same accumulator, so the codes are converted once and the sum carries ~16 significand
// bits of x (the f32 path's 1e-4 tolerance) in one pass.
//
// Warp roles: warp 0 = TMA producer, warp 1 = TMEM allocator + MMA issuer, then G groups of
// 4 converter warps (one TMEM lane quadrant each) which also run the epilogue.  A pipeline
// stage holds KSUB sub-blocks of 64 k: full[s] (TMA bytes landed) -> converters (group g
// owns the stages s with s % G == g) -> aready[s] -> MMA (4*KSUB instructions, one commit) ->
// empty[s] -> producer.  One barrier round trip per stage costs the single MMA-issuing
// thread ~400 cycles, so small token tiles (short MMAs) use more sub-blocks per stage.
// Every wait is bounded: after the limit the waiter records where it gave up in a status
// block, raises a CTA-wide abort flag and all roles fall through to the common teardown,
// which frees TMEM.
//
// Device code only (no launch syntax, no runtime calls; PTX behind ptx_tcgen05.cuh and ptx_small.cuh):
// it also compiles as plain C++ against the CUDA stand-in of the CPU tests (tests/cpu_emu/), which
// model mbarriers, TMA, tensor memory and tcgen05.mma and run this kernel against reference results.
#pragma once

#include "../../include/shrewq.h"
#include "dests.cuh"
#include "ptx_small.cuh"
#include "ptx_tcgen05.cuh"
#include "tcgen05_common.cuh"
#include "tcgen05_epilogue.cuh"

namespace shrewq {
namespace {

constexpr int kTileN = 128;  // TMEM lanes = weight rows per CTA (64 + 64 when GATED)
constexpr int kBlockK = 64;  // k per sub-block (one 64-byte-swizzled INT8 box)
constexpr int kUmmaK = 16;
template <int TOK, int KSUB, bool XSPLIT = false>
struct Cfg {
    static constexpr int kWSub = kTileN * kBlockK;                   // 8192 B of codes per sub-block
    static constexpr int kXTile = TOK * kBlockK * 2;                 // one bf16 token tile of a sub-block
    static constexpr int kXSub = kXTile * (XSPLIT ? 2 : 1);          // bf16 activations per sub-block (hi, then lo)
    static constexpr int kStageBytes = KSUB * (kWSub + kXSub);
    static constexpr int kXOff = KSUB * kWSub;                       // activations follow the codes
    static constexpr int kAColsPerStage = KSUB * (kBlockK / 2);      // 32-bit TMEM columns
    static constexpr int kABase = (TOK + 31) / 32 * 32;
    static constexpr int kMaxStagesSmem = (200 * 1024) / kStageBytes;
    static constexpr int kMaxStagesTmem = (512 - kABase) / kAColsPerStage;
    static constexpr int kStagesRaw = kMaxStagesSmem < kMaxStagesTmem ? kMaxStagesSmem : kMaxStagesTmem;
    static constexpr int kStages = kStagesRaw > 12 ? 12 : kStagesRaw;
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*barriers*/ + 1024 /*alignment slack*/;
    // one CTA per SM is required (the CTA allocates all 512 TMEM columns)
    static constexpr int kSmemRequest = kSmemBytes > 120 * 1024 ? kSmemBytes : 120 * 1024;
    static_assert(kStages >= 2, "pipeline needs at least two stages");
    static_assert(kABase + kStages * kAColsPerStage <= 512, "TMEM columns");
    static_assert(kSmemRequest <= 227 * 1024, "shared memory");
    static_assert(kStageBytes % 1024 == 0, "stage bases must keep the 1024-byte swizzle alignment");
    static_assert(kStages * kStageBytes >= 3 * kEpiGroupBytes, "the epilogue's staging tiles reuse the pipeline stages");
};

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, Ctl *ctl, DeviceStatus *st, uint32_t role, uint32_t stage) {
    return mbar_wait_c<1>(bar, parity, ctl, st, role, stage);
}
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, Ctl *ctl, DeviceStatus *st, uint32_t role,
                                               uint32_t stage) {
    return mbar_wait_warp_c<1>(bar, parity, ctl, st, role, stage);
}

#ifdef SHREWQ_TRACE
__device__ long long *g_trace = nullptr;  // [role 0..3][stage index 0..255][tag 0..3]
__device__ __forceinline__ void trace_rec(long long *tr, int role, int kb, int tag) {
    if (tr && kb < 256) tr[(role * 256 + kb) * 4 + tag] = clock64();
}
#define TRACE(role, kb, tag) do { if ((threadIdx.x & 31) == 0) trace_rec(trace_buf, role, kb, tag); } while (0)
#define TRACE_INIT long long *trace_buf = (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) ? g_trace : nullptr;
#else
#define TRACE(role, kb, tag)
#define TRACE_INIT
#endif

struct SplitK {
    float *partials;         // [tile][split][TOK][128] f32, only when gridDim.z > 1
    unsigned int *counters;  // one per (n tile, token tile), zero between launches
    int rounds_per_split;    // pipeline rounds (KSUB sub-blocks each) per split
    // Tile-list mode (n_tiles_total > 0): the grid is a 1-D list of output tiles starting at
    // tile_begin in channel-major order, instead of the (channel tile, token tile) grid.
    // Lets one forward be issued as two launches with different split counts.
    int tile_begin;
    int n_tiles_total;
};

template <int TOK, int KSUB, int G, bool GATED, typename YT, bool XSPLIT = false>
__global__ void __launch_bounds__(64 + 128 * G, 1)
linear_i8_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_w2,
                         const __grid_constant__ CUtensorMap tmap_x, Operands ops, YT *__restrict__ y, Dests extra, int M, int N,
                         int K, size_t ldy, int epilogue, SplitK sk, DeviceStatus *status) {
    using C = Cfg<TOK, KSUB, XSPLIT>;
    static_assert(!(XSPLIT && GATED), "the hi/lo form exists for plain tiles");
    constexpr int kChan = GATED ? 64 : 128;  // output channels per CTA
    TRACE_INIT
    pdl_launch_dependents();  // the next kernel of the stream may start its prologue (a no-op in an ordinary launch)
    SHREWQ_DYNAMIC_SMEM(uint8_t, smem_raw);
    // 1024-byte alignment: required by the 128-byte swizzle with base_offset 0
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *bar_area = smem + C::kStages * C::kStageBytes;
    uint64_t *bars = reinterpret_cast<uint64_t *>(bar_area);
    Ctl *ctl = reinterpret_cast<Ctl *>(bar_area + 512);
    int *s_is_last = reinterpret_cast<int *>(bar_area + 640);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp == 2) TRACE(3, 1, 0);  // kernel entry
    int tile_x = blockIdx.x, tile_y = blockIdx.y;
    if (sk.n_tiles_total > 0) {
        const int tl = sk.tile_begin + (int)blockIdx.x;
        tile_x = tl % sk.n_tiles_total;
        tile_y = tl / sk.n_tiles_total;
    }
    const int n0 = tile_x * kChan;
    const int m0 = tile_y * TOK;
    const int rounds_total = (K + kBlockK * KSUB - 1) / (kBlockK * KSUB);
    const int r_begin = blockIdx.z * sk.rounds_per_split;
    const int nr = min(rounds_total - r_begin, sk.rounds_per_split);  // >= 1 by construction of the grid
    // barrier byte offsets: full[s], aready[s], empty[s], accfull
    constexpr uint32_t kFullBar = 0, kAreadyBar = C::kStages * 8, kEmptyBar = 2 * C::kStages * 8, kAccBar = 3 * C::kStages * 8;
    const uint32_t bars_u32 = smem_u32(bars);
    const uint32_t smem_base = smem_u32(smem);

    if (threadIdx.x == 0) {
        ctl->abort_flag = 0;
        ctl->tmem_base = 0;
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(bars_u32 + kFullBar + s * 8, 1);
            mbar_init(bars_u32 + kAreadyBar + s * 8, 4);
            mbar_init(bars_u32 + kEmptyBar + s * 8, 1);
        }
        mbar_init(bars_u32 + kAccBar, 1);
        mbar_fence_init();
    }
    if (warp == 1) {
        tc_alloc_512(smem_u32(&ctl->tmem_base));
        tc_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctl->tmem_base;
    if (warp == 2) TRACE(3, 1, 1);  // barriers initialised, tensor memory allocated

    if (warp == 0) {
        // ---------------- TMA producer (one thread) ----------------
        // Programmatic dependent launch: the WEIGHTS of the first stages are requested at once (they never depend on
        // an earlier kernel), the activations only when the previous kernel of the stream, whose output they may be,
        // has completed (griddepcontrol.wait; it returns at once in an ordinary launch).
        if (lane == 0) {
            auto load_w = [&](uint32_t dst, int kc, uint32_t fb) {
#pragma unroll
                for (int j = 0; j < KSUB; ++j) {
                    if constexpr (GATED) {
                        tma_load_2d(dst + j * C::kWSub, &tmap_w, kc + j * kBlockK, n0, fb);
                        tma_load_2d(dst + j * C::kWSub + 64 * kBlockK, &tmap_w2, kc + j * kBlockK, n0, fb);
                    } else {
                        tma_load_2d(dst + j * C::kWSub, &tmap_w, kc + j * kBlockK, n0, fb);
                    }
                }
            };
            auto load_x = [&](uint32_t dst, int kc, uint32_t fb) {
#pragma unroll
                for (int j = 0; j < KSUB; ++j) {
                    tma_load_2d(dst + C::kXOff + j * C::kXSub, &tmap_x, kc + j * kBlockK, m0, fb);
                    if constexpr (XSPLIT)  // the lo rows follow the M hi rows in the same array
                        tma_load_2d(dst + C::kXOff + j * C::kXSub + C::kXTile, &tmap_x, kc + j * kBlockK, m0 + M, fb);
                }
            };
            const int kc0 = r_begin * KSUB * kBlockK;
            const int pre = nr < C::kStages ? nr : C::kStages;  // the stages that are free at the start
            for (int i = 0; i < pre; ++i) {
                const uint32_t fb = bars_u32 + kFullBar + i * 8;
                mbar_expect_tx(fb, C::kStageBytes);
                load_w(smem_base + i * C::kStageBytes, kc0 + i * KSUB * kBlockK, fb);
            }
            pdl_wait();
            for (int i = 0; i < pre; ++i) {
                load_x(smem_base + i * C::kStageBytes, kc0 + i * KSUB * kBlockK, bars_u32 + kFullBar + i * 8);
                TRACE(0, i, 2);
            }
            uint32_t s = 0, ph = 0;  // the ring wrapped once: the producer now waits for the first release of a stage
            uint32_t dst = smem_base;
            int kc = kc0 + pre * KSUB * kBlockK;
            for (int i = pre; i < nr; ++i) {
                TRACE(0, i, 0);
                if (!mbar_wait(bars_u32 + kEmptyBar + s * 8, ph, ctl, status, 0, s)) break;
                TRACE(0, i, 1);
                const uint32_t fb = bars_u32 + kFullBar + s * 8;
                mbar_expect_tx(fb, C::kStageBytes);
                load_w(dst, kc, fb);
                load_x(dst, kc, fb);
                TRACE(0, i, 2);
                kc += KSUB * kBlockK;
                dst += C::kStageBytes;
                if (++s == C::kStages) { s = 0; ph ^= 1; dst = smem_base; }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (one thread) ----------------
        if (lane == 0) {
            // instruction descriptor: D=f32, A=bf16 (K-major, from TMEM), B=bf16 (K-major), M=128, N=TOK
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) |
                                       ((uint32_t)(TOK >> 3) << 17) | ((uint32_t)(kTileN >> 4) << 24);
            const uint64_t bdesc0 = make_b_desc(smem_base + C::kXOff);
            const uint32_t a0 = tmem_base + C::kABase;
            uint32_t s = 0, ph = 0, a_tmem = a0;
            uint64_t bdesc = bdesc0;
            bool ok = true;
            for (int i = 0; i < nr; ++i) {
                TRACE(1, i, 0);
                // aready[s] implies full[s] (the converters waited for it), so the second wait
                // returns at once; it gives this thread its own acquire on the activation tile
                ok = mbar_wait(bars_u32 + kAreadyBar + s * 8, ph, ctl, status, 2, s) &&
                     mbar_wait(bars_u32 + kFullBar + s * 8, ph, ctl, status, 1, s);
                if (!ok) break;
                TRACE(1, i, 2);
                tc_fence_after();
#pragma unroll
                for (int j = 0; j < KSUB; ++j) {
#pragma unroll
                    for (int jj = 0; jj < kBlockK / kUmmaK; ++jj) {
                        tc_mma_ts(tmem_base, a_tmem + j * (kBlockK / 2) + jj * (kUmmaK / 2),
                                  bdesc + (uint64_t)((j * C::kXSub + jj * kUmmaK * 2) >> 4), idesc,
                                  (i > 0 || j > 0 || jj > 0) ? 1u : 0u);
                        if constexpr (XSPLIT)
                            tc_mma_ts(tmem_base, a_tmem + j * (kBlockK / 2) + jj * (kUmmaK / 2),
                                      bdesc + (uint64_t)((j * C::kXSub + C::kXTile + jj * kUmmaK * 2) >> 4), idesc, 1u);
                    }
                }
                tc_commit(bars_u32 + kEmptyBar + s * 8);  // frees smem stage s and TMEM A stage s
                TRACE(1, i, 3);
                a_tmem += C::kAColsPerStage;
                bdesc += (uint64_t)(C::kStageBytes >> 4);
                if (++s == C::kStages) { s = 0; ph ^= 1; a_tmem = a0; bdesc = bdesc0; }
            }
            if (ok) tc_commit(bars_u32 + kAccBar);  // accumulators complete
        }
        __syncwarp();
    } else {
        // ---------------- converters, then epilogue ----------------
        const int group = (warp - 2) >> 2;
        const int quad = warp & 3;                 // TMEM lane quadrant this warp may access
        const int row = quad * 32 + lane;          // TMEM lane
        // the weight row of the tile this lane converts: plain tiles lane = row; gated tiles interleave the gate box
        // (shared-memory rows 0..63) and the up box (64..127), gate rows on even lanes, so that a channel's
        // gate and up accumulators sit in neighbouring lanes for the epilogue
        const int srow = GATED ? ((row & 1) * 64 + (row >> 1)) : row;
        const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
        const int swz = (srow >> 1) & 3;
        bool ok = true;
        // A group owns pipeline STAGES (stage s belongs to group s % G), not every G-th round: its
        // warps then pass through every phase of the barriers they poll, so a parity wait can never
        // mistake phase k-2 for phase k, whatever order the TMA loads complete in.
        for (int i = 0; i < nr && ok; ++i) {
            const int s = i % C::kStages;
            if (s % G != group) continue;
            const uint32_t ph = (i / C::kStages) & 1;
            if (((warp - 2) & 3) == 0) TRACE(2, i, 0);
            ok = mbar_wait_warp(bars_u32 + kFullBar + s * 8, ph, ctl, status, 3, s);
            if (!ok) break;
            tc_fence_after();
            if (((warp - 2) & 3) == 0) TRACE(2, i, 1);
#pragma unroll
            for (int j = 0; j < KSUB; ++j) {
                uint32_t packed[32];
                convert_row64(smem + s * C::kStageBytes + j * C::kWSub + srow * kBlockK, swz, packed);
                tc_st32(tmem_base + lane_addr + C::kABase + s * C::kAColsPerStage + j * (kBlockK / 2), packed);
            }
            if (((warp - 2) & 3) == 0) TRACE(2, i, 2);
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bars_u32 + kAreadyBar + s * 8);
            if (((warp - 2) & 3) == 0) TRACE(2, i, 3);
        }
        // ---------------- epilogue: 16-column chunks dealt round-robin to the groups ----------------
        pdl_wait();  // outputs, partial sums and counters may still be in use by the previous kernel of the stream
        if (warp == 2) TRACE(3, 0, 0);  // (tracing build: role 3 = the epilogue of the first converter warp)
        if (ok) ok = mbar_wait_warp(bars_u32 + kAccBar, 0, ctl, status, 4, 0);
        if (warp == 2) TRACE(3, 0, 1);  // accumulators complete
        const int splits = gridDim.z;
        if (splits == 1) {
            if (ok) tc_fence_after();
            epilogue_tile<TOK, G, GATED, YT>(tmem_base, smem, group, quad, lane, ok, ops, y, extra, M, N, ldy, epilogue, n0, m0,
                                             PartialSums{nullptr, 0, 0});
        } else {
            // split-K: every CTA parks its raw accumulators in scratch; the CTA that arrives
            // last at the tile's counter adds the slices in split order (so the sum does not
            // depend on arrival order), applies scale / bias / op and stores.
            const size_t tile = (size_t)blockIdx.y * gridDim.x + blockIdx.x;
            float *mine = sk.partials + (tile * splits + blockIdx.z) * (size_t)(TOK * kTileN);
            if (ok) {
                tc_fence_after();
                dump_partials<TOK, G>(tmem_base, mine, group, quad, lane);
            }
            if (warp == 2) TRACE(3, 0, 2);  // partial sums written
            __threadfence();
            named_bar_sync(1, 128 * G);
            if (threadIdx.x == 64) {
                const unsigned int old = atomicAdd(sk.counters + tile, 1u);
                *s_is_last = (old == (unsigned int)(splits - 1));
            }
            named_bar_sync(1, 128 * G);
            if (warp == 2) TRACE(3, 0, 3);  // this CTA's arrival counted
            if (*s_is_last) {
                __threadfence();
                epilogue_tile<TOK, G, GATED, YT>(tmem_base, smem, group, quad, lane, ok, ops, y, extra, M, N, ldy, epilogue, n0,
                                                 m0, PartialSums{sk.partials + tile * splits * (size_t)(TOK * kTileN), splits, (size_t)(TOK * kTileN)});
                named_bar_sync(1, 128 * G);
                if (threadIdx.x == 64) sk.counters[tile] = 0;  // ready for the next launch
            }
        }
    }

    // ---------------- teardown ----------------
    if (warp == 2) TRACE(3, 1, 2);  // this warp's epilogue done
    tc_fence_before();
    __syncthreads();
    if (warp == 2) TRACE(3, 1, 3);  // every warp done
    if (warp == 1) {
        if (ctl->abort_flag) {
            // give in-flight copies / MMAs a bounded moment to land before TMEM is released
            for (int i = 0; i < 2000; ++i) __nanosleep(1000);
        }
        tc_fence_after();
        __syncwarp();
        tc_dealloc_512(tmem_base);
    }
}

}  // namespace
}  // namespace shrewq
