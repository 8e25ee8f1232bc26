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
// The epilogue reads D with tcgen05.ld (one thread per channel), applies the per-channel
// scale, bias and the elementwise op, and stores; for a fixed token the 32 lanes of a warp
// write 32 consecutive channels.
//
// GATED: the 128 lanes carry 64 rows of a gate matrix and the same 64 rows of an up matrix
// (two 64-row TMA boxes per sub-block); the epilogue pairs lane r with lane r+64 and
// writes silu(gate)*up for 64 channels.
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
#include <cuda.h>

#include <cstdlib>

#include "common.cuh"

namespace shrewq {
namespace {

constexpr int kTileN = 128;  // TMEM lanes = weight rows per CTA (64 + 64 when GATED)
constexpr int kBlockK = 64;  // k per sub-block (one 64-byte-swizzled INT8 box)
constexpr int kUmmaK = 16;
constexpr uint32_t kSpinFast = 1u << 14;
constexpr uint32_t kSpinSlow = 1u << 21;  // x ~100 ns sleeps: a fraction of a second

template <int TOK, int KSUB>
struct Cfg {
    static constexpr int kWSub = kTileN * kBlockK;                   // 8192 B of codes per sub-block
    static constexpr int kXSub = TOK * kBlockK * 2;                  // bf16 activations per sub-block
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
};

// ---- PTX wrappers ---------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

struct Ctl {  // lives in shared memory
    volatile int abort_flag;
    uint32_t tmem_base;
};

// Slow path of the bounded wait, kept out of line so the hot loops only carry one try_wait.
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, Ctl *ctl, DeviceStatus *st,
                                            uint32_t role, uint32_t stage) {
    for (uint32_t i = 0; i < kSpinFast; ++i)
        if (mbar_try(bar, parity)) return true;
    for (uint32_t i = 0; i < kSpinSlow; ++i) {
        if (mbar_try(bar, parity)) return true;
        if (ctl->abort_flag) return false;
        __nanosleep(100);
    }
    ctl->abort_flag = 1;
    if (atomicCAS(&st->timeout_flag, 0u, 1u) == 0u) {
        st->where = (blockIdx.x << 8) | role;
        st->stage = stage;
        st->parity = parity;
    }
    return false;
}

// Bounded wait.  Returns false if it gave up or another role already did.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, Ctl *ctl, DeviceStatus *st,
                                          uint32_t role, uint32_t stage) {
    if (mbar_try(bar, parity)) return true;
    if (mbar_try(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, ctl, st, role, stage);
}

// Warp-level wait: lane 0 polls, the outcome is broadcast with a shuffle (which also
// synchronises the warp and orders memory among its lanes).  32 lanes polling the same
// mbarrier word serialise in the shared-memory pipe.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, Ctl *ctl, DeviceStatus *st,
                                               uint32_t role, uint32_t stage) {
    int ok = 1;
    if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, ctl, st, role, stage) ? 1 : 0;
    ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
    // every lane observes the completed phase itself (one try_wait that succeeds at once), so
    // each has its own acquire on the data the barrier guards
    if (ok) ok = mbar_try(bar, parity) ? 1 : 0;
    return __all_sync(0xFFFFFFFFu, ok) != 0;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void *tmap, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(tmap), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem desc]
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t *r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t *r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// 4 INT8 codes (one 32-bit word) -> two packed bf16x2 words, exactly.
// byte ^ 0x80 = q + 128 as an unsigned byte u; 0x4B0000uu is the float 2^23 + u; subtracting
// 2^23 + 128 leaves q; cvt.rn.bf16x2.f32 packs two of them (exact, |q| <= 128).
__device__ __forceinline__ void cvt_i8x4_bf16(uint32_t w, uint32_t &lo, uint32_t &hi) {
    const uint32_t u = w ^ 0x80808080u;
    const float f0 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7440)) - 8388736.0f;
    const float f1 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7441)) - 8388736.0f;
    const float f2 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7442)) - 8388736.0f;
    const float f3 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7443)) - 8388736.0f;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(lo) : "f"(f1), "f"(f0));
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(hi) : "f"(f3), "f"(f2));
}

// Shared-memory matrix descriptor for the activation tile: K-major, 128-byte swizzle,
// rows of 128 B, 8-row groups 1024 B apart (stride byte offset), descriptor version 1.
__device__ __forceinline__ uint64_t make_b_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);        // start address  [0,14)
    d |= (uint64_t)1 << 16;                             // leading byte offset (unused with swizzle)
    d |= (uint64_t)(1024 >> 4) << 32;                   // stride byte offset [32,46)
    d |= (uint64_t)1 << 46;                             // version = 1 (sm_100)
    d |= (uint64_t)2 << 61;                             // layout: SWIZZLE_128B
    return d;
}

template <typename YT>
__device__ __forceinline__ void store_out(YT *p, float v);
// the local store plus one store per peer destination (same element offset in each buffer)
template <typename YT>
__device__ __forceinline__ void store_all(YT *y, const Dests &extra, size_t off, float v);
template <>
__device__ __forceinline__ void store_out<float>(float *p, float v) { *p = v; }
template <>
__device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float load_prev(const float *p) { return *p; }
__device__ __forceinline__ float load_prev(const __nv_bfloat16 *p) { return __bfloat162float(*p); }

template <typename YT>
__device__ __forceinline__ void store_all(YT *y, const Dests &extra, size_t off, float v) {
    store_out<YT>(y + off, v);
    for (int d = 0; d < extra.n; ++d) store_out<YT>(static_cast<YT *>(extra.p[d]) + off, v);
}

__device__ __forceinline__ float silu_f(float g) { return g / (1.0f + __expf(-g)); }

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
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

struct Operands {
    const float *scales;   // per output channel
    const float *bias;     // or null
    const float *scales2;  // up matrix (GATED)
    const float *bias2;
};

template <int TOK, int KSUB, int G, bool GATED, typename YT>
__global__ void __launch_bounds__(64 + 128 * G, 1)
linear_i8_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_w2,
                         const __grid_constant__ CUtensorMap tmap_x, Operands ops, YT *__restrict__ y, Dests extra, int M, int N,
                         int K, size_t ldy, int epilogue, SplitK sk, DeviceStatus *status) {
    using C = Cfg<TOK, KSUB>;
    constexpr int kChan = GATED ? 64 : 128;  // output channels per CTA
    TRACE_INIT
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment: required by the 128-byte swizzle with base_offset 0
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *bar_area = smem + C::kStages * C::kStageBytes;
    uint64_t *bars = reinterpret_cast<uint64_t *>(bar_area);
    Ctl *ctl = reinterpret_cast<Ctl *>(bar_area + 512);
    int *s_is_last = reinterpret_cast<int *>(bar_area + 640);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
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
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(&ctl->tmem_base))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctl->tmem_base;

    if (warp == 0) {
        // ---------------- TMA producer (one thread) ----------------
        if (lane == 0) {
            uint32_t s = 0, ph = 1;  // waiting on parity 1 of a fresh barrier returns at once
            uint32_t dst = smem_base;
            int kc = r_begin * KSUB * kBlockK;
            for (int i = 0; i < nr; ++i) {
                TRACE(0, i, 0);
                if (!mbar_wait(bars_u32 + kEmptyBar + s * 8, ph, ctl, status, 0, s)) break;
                TRACE(0, i, 1);
                const uint32_t fb = bars_u32 + kFullBar + s * 8;
                mbar_expect_tx(fb, C::kStageBytes);
#pragma unroll
                for (int j = 0; j < KSUB; ++j) {
                    if constexpr (GATED) {
                        tma_load_2d(dst + j * C::kWSub, &tmap_w, kc + j * kBlockK, n0, fb);
                        tma_load_2d(dst + j * C::kWSub + 64 * kBlockK, &tmap_w2, kc + j * kBlockK, n0, fb);
                    } else {
                        tma_load_2d(dst + j * C::kWSub, &tmap_w, kc + j * kBlockK, n0, fb);
                    }
                    tma_load_2d(dst + C::kXOff + j * C::kXSub, &tmap_x, kc + j * kBlockK, m0, fb);
                }
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
                    for (int jj = 0; jj < kBlockK / kUmmaK; ++jj)
                        tc_mma_ts(tmem_base, a_tmem + j * (kBlockK / 2) + jj * (kUmmaK / 2),
                                  bdesc + (uint64_t)((j * C::kXSub + jj * kUmmaK * 2) >> 4), idesc,
                                  (i > 0 || j > 0 || jj > 0) ? 1u : 0u);
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
        const int row = quad * 32 + lane;          // weight row inside the tile == TMEM lane
        const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
        const int swz = (row >> 1) & 3;
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
                // 64 codes of this row; TMA wrote them with the 64-byte swizzle: the 16-byte
                // chunk c of row r sits at chunk position c ^ ((r >> 1) & 3)
                const uint8_t *rowp = smem + s * C::kStageBytes + j * C::kWSub + row * kBlockK;
                uint32_t packed[32];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const uint4 v = *reinterpret_cast<const uint4 *>(rowp + ((c ^ swz) << 4));
                    cvt_i8x4_bf16(v.x, packed[8 * c + 0], packed[8 * c + 1]);
                    cvt_i8x4_bf16(v.y, packed[8 * c + 2], packed[8 * c + 3]);
                    cvt_i8x4_bf16(v.z, packed[8 * c + 4], packed[8 * c + 5]);
                    cvt_i8x4_bf16(v.w, packed[8 * c + 6], packed[8 * c + 7]);
                }
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
        if (ok) ok = mbar_wait_warp(bars_u32 + kAccBar, 0, ctl, status, 4, 0);
        // this lane's channel: plain tiles map lane -> n0 + lane; gated tiles map lanes 0..63 to
        // the gate rows and lanes 64..127 to the up rows of channels n0 .. n0+63
        const bool is_up = GATED && row >= 64;
        const int n = n0 + (GATED ? (row & 63) : row);
        const bool n_ok = n < N;
        const float *sc_p = is_up ? ops.scales2 : ops.scales;
        const float *bs_p = is_up ? ops.bias2 : ops.bias;
        const float sc = n_ok ? sc_p[n] : 0.0f;
        const float bs = (n_ok && bs_p) ? bs_p[n] : 0.0f;
        const int splits = gridDim.z;
        if (splits == 1) {
            if (ok) tc_fence_after();
            // gated tiles: the up half hands its values to the gate half through shared memory
            // (the pipeline stages are idle once the accumulators are complete)
            float *xch = reinterpret_cast<float *>(smem) + group * (16 * 64);
#pragma unroll 1
            for (int c = group; c < TOK / 16; c += G) {
                uint32_t r[16];
                if (ok) {
                    tc_ld16(tmem_base + lane_addr + c * 16, r);
                    tc_wait_ld();
                }
                if constexpr (GATED) {
                    if (is_up && ok) {
#pragma unroll
                        for (int i = 0; i < 16; ++i) xch[i * 64 + (row - 64)] = __uint_as_float(r[i]) * sc + bs;
                    }
                    named_bar_sync(2 + group, 128);
                    if (!is_up && ok) {
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const int m = m0 + c * 16 + i;
                            const float g = __uint_as_float(r[i]) * sc + bs;
                            const float o = silu_f(g) * xch[i * 64 + row];
                            if (n_ok && m < M) store_all<YT>(y, extra, (size_t)m * ldy + n, o);
                        }
                    }
                    named_bar_sync(2 + group, 128);  // xch is rewritten by the next chunk
                } else if (ok) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const int m = m0 + c * 16 + i;
                        float o = __uint_as_float(r[i]) * sc + bs;
                        if ((epilogue & kEpilogueAccumulate) && n_ok && m < M) o += load_prev(y + (size_t)m * ldy + n);
                        if ((epilogue & 0xFF) == SHREWQ_EPILOGUE_RELU) o = fmaxf(o, 0.0f);
                        if (n_ok && m < M) store_all<YT>(y, extra, (size_t)m * ldy + n, o);
                    }
                }
            }
        } else {
            // split-K: every CTA parks its raw accumulators in scratch; the CTA that arrives
            // last at the tile's counter adds the slices in split order (so the sum does not
            // depend on arrival order), applies scale / bias / op and stores.
            const size_t tile = (size_t)blockIdx.y * gridDim.x + blockIdx.x;
            float *mine = sk.partials + (tile * splits + blockIdx.z) * (size_t)(TOK * kTileN);
            if (ok) {
                tc_fence_after();
#pragma unroll 1
                for (int c = group; c < TOK / 16; c += G) {
                    uint32_t r[16];
                    tc_ld16(tmem_base + lane_addr + c * 16, r);
                    tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 16; ++i) __stcg(mine + (c * 16 + i) * kTileN + row, __uint_as_float(r[i]));
                }
            }
            __threadfence();
            named_bar_sync(1, 128 * G);
            if (threadIdx.x == 64) {
                const unsigned int old = atomicAdd(sk.counters + tile, 1u);
                *s_is_last = (old == (unsigned int)(splits - 1));
            }
            named_bar_sync(1, 128 * G);
            if (*s_is_last) {
                __threadfence();
                const float *base = sk.partials + tile * splits * (size_t)(TOK * kTileN);
                if (ok && !is_up) {
#pragma unroll 1
                    for (int c = group; c < TOK / 16; c += G) {
#pragma unroll 4
                        for (int i = 0; i < 16; ++i) {
                            const int ml = c * 16 + i, m = m0 + ml;
                            float acc = 0.0f, acc2 = 0.0f;
                            for (int z = 0; z < splits; ++z) {
                                const float *p = base + (size_t)z * (TOK * kTileN) + ml * kTileN + row;
                                acc += __ldcg(p);
                                if constexpr (GATED) acc2 += __ldcg(p + 64);
                            }
                            float o = acc * sc + bs;
                            if constexpr (GATED) {
                                const float u = acc2 * (n_ok ? ops.scales2[n] : 0.0f) + ((n_ok && ops.bias2) ? ops.bias2[n] : 0.0f);
                                o = silu_f(o) * u;
                            } else {
                                if ((epilogue & kEpilogueAccumulate) && n_ok && m < M) o += load_prev(y + (size_t)m * ldy + n);
                                if ((epilogue & 0xFF) == SHREWQ_EPILOGUE_RELU) o = fmaxf(o, 0.0f);
                            }
                            if (n_ok && m < M) store_all<YT>(y, extra, (size_t)m * ldy + n, o);
                        }
                    }
                }
                named_bar_sync(1, 128 * G);
                if (threadIdx.x == 64) sk.counters[tile] = 0;  // ready for the next launch
            }
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        if (ctl->abort_flag) {
            // give in-flight copies / MMAs a bounded moment to land before TMEM is released
            for (int i = 0; i < 2000; ++i) __nanosleep(1000);
        }
        tc_fence_after();
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
    }
}

// ---- host side ------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

int encode_2d(shrewq_ctx *ctx, CUtensorMap *out, CUtensorMapDataType dt, int elem_bytes, const void *base,
              size_t inner, size_t outer, int box_inner, int box_outer, CUtensorMapSwizzle sw) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return set_err(ctx, SHREWQ_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
    cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
    cuuint64_t strides[1] = {(cuuint64_t)inner * elem_bytes};
    cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, dt, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_err(ctx, SHREWQ_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return SHREWQ_OK;
}

// ---- launch ---------------------------------------------------------------------------
struct Tuning {
    int groups;   // converter groups (1..3)
    bool splitk;  // allow split-K when the grid would leave SMs idle
    int tok;      // 0 = choose; else force the token tile
};

Tuning read_tuning() {
    Tuning t{3, true, 0};
    if (const char *e = getenv("SHREWQ_TC_GROUPS")) t.groups = atoi(e);
    if (const char *e = getenv("SHREWQ_TC_SPLITK")) t.splitk = atoi(e) != 0;
    if (const char *e = getenv("SHREWQ_TC_TOK")) t.tok = atoi(e);
    if (t.groups < 1) t.groups = 1;
    if (t.groups > 3) t.groups = 3;
    return t;
}

constexpr size_t kScratchCounterOff = 4096, kScratchPartialOff = 8192;

struct LaunchPlan {
    int n_tiles, m_tiles, splits, rounds_per_split;
};

template <int TOK, int KSUB>
LaunchPlan plan_launch(const ForwardArgs &a, int chan_per_tile, int sm_count, bool allow_split) {
    LaunchPlan p;
    p.n_tiles = (int)((a.N + chan_per_tile - 1) / chan_per_tile);
    p.m_tiles = (int)((a.M + TOK - 1) / TOK);
    const int rounds = (int)((a.K + kBlockK * KSUB - 1) / (kBlockK * KSUB));
    // split-K only for small token tiles (their partial sums are small) when the output
    // tiles alone leave most SMs idle: as many splits as fit in one wave, >= 2 rounds each
    int splits = 1;
    const long tiles = (long)p.n_tiles * p.m_tiles;
    // SHREWQ_TC_SPLITK_MAXTOK=128|256 (NOT yet run on a GPU, default 64) extends the rule to the
    // large token tiles, with at least 8 rounds per split: batches 65..256 on layers with few
    // channel tiles (N = 4096: 32 tiles) otherwise run on a fraction of the SMs.  The kernel's
    // split path is the same code for every tile width.
    static const int max_tok = [] {
        const char *e = getenv("SHREWQ_TC_SPLITK_MAXTOK");
        const int v = e ? atoi(e) : 64;
        return v < 64 ? 64 : v;
    }();
    const int min_rounds = TOK <= 64 ? 2 : 8;
    if (allow_split && TOK <= max_tok && tiles <= 1024) {
        int want = (int)(sm_count / tiles);
        if (want > rounds / min_rounds) want = rounds / min_rounds;
        if (want > 1) splits = want;
    }
    p.rounds_per_split = (rounds + splits - 1) / splits;
    p.splits = (rounds + p.rounds_per_split - 1) / p.rounds_per_split;  // no empty split
    return p;
}

// scratch == nullptr: use (and grow) the context's scratch; otherwise a caller-provided
// region of scratch_bytes laid out as [0,4096) counters, partial sums from 4096.
template <int TOK, int KSUB, int G, bool GATED, typename YT>
int launch_cfg(shrewq_ctx *ctx, const ForwardArgs &a, const CUtensorMap &tw, const CUtensorMap &tw2, bool allow_split,
               void *fixed_scratch, size_t fixed_scratch_bytes) {
    using C = Cfg<TOK, KSUB>;
    CUtensorMap tx;
    int rc = encode_2d(ctx, &tx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.x, a.K, a.M, kBlockK, TOK,
                       CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != SHREWQ_OK) return rc;
    auto kern = linear_i8_tcgen05_kernel<TOK, KSUB, G, GATED, YT>;
    static bool attr_set[64] = {false};  // per instantiation and per device (the attribute is per device)
    if (ctx->device < 0 || ctx->device >= 64 || !attr_set[ctx->device]) {
        SHREWQ_CUDA_TRY(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemRequest));
        if (ctx->device >= 0 && ctx->device < 64) attr_set[ctx->device] = true;
    }
    const LaunchPlan p = plan_launch<TOK, KSUB>(a, GATED ? 64 : 128, ctx->sm_count, allow_split);
    SplitK sk{nullptr, nullptr, p.rounds_per_split, 0, 0};
    Operands ops{a.scales, a.bias, a.scales_up, a.bias_up};
    // SHREWQ_TC_TAILSPLIT=1 (built, NOT yet run on a GPU, off by default): when large tiles
    // leave a short last wave, issue the full waves as one launch and the tiles of the last
    // wave as a second launch split along K so that it also fills the SMs.
    static const bool tail_split = getenv("SHREWQ_TC_TAILSPLIT") && atoi(getenv("SHREWQ_TC_TAILSPLIT")) != 0;
    if (tail_split && !fixed_scratch && TOK >= 128 && p.splits == 1) {
        const int tiles = p.n_tiles * p.m_tiles, rem = tiles % ctx->sm_count;
        const int rounds = p.rounds_per_split;
        int s_tail = rem > 0 ? ctx->sm_count / rem : 0;
        if (s_tail > 4) s_tail = 4;
        if (s_tail > rounds / 8) s_tail = rounds / 8;
        if (tiles > ctx->sm_count && rem > 0 && s_tail >= 2) {
            const size_t part_bytes = (size_t)rem * s_tail * TOK * kTileN * sizeof(float);
            if ((rc = ensure_scratch(ctx, kScratchPartialOff + part_bytes)) != SHREWQ_OK) return rc;
            if (!ctx->counters_zeroed) {
                SHREWQ_CUDA_TRY(ctx, cudaMemsetAsync(static_cast<char *>(ctx->scratch) + kScratchCounterOff, 0,
                                                     kScratchPartialOff - kScratchCounterOff, ctx->stream));
                ctx->counters_zeroed = true;
            }
            SplitK head{nullptr, nullptr, rounds, 0, p.n_tiles};
            kern<<<dim3((unsigned)(tiles - rem), 1, 1), 64 + 128 * G, C::kSmemRequest, ctx->stream>>>(
                tw, tw2, tx, ops, static_cast<YT *>(a.y), a.extra, (int)a.M, (int)a.N, (int)a.K, a.ldy, a.epilogue, head,
                ctx->dev_status);
            const int rps = (rounds + s_tail - 1) / s_tail;
            const int splits = (rounds + rps - 1) / rps;
            SplitK tail{reinterpret_cast<float *>(static_cast<char *>(ctx->scratch) + kScratchPartialOff),
                        reinterpret_cast<unsigned int *>(static_cast<char *>(ctx->scratch) + kScratchCounterOff), rps,
                        tiles - rem, p.n_tiles};
            kern<<<dim3((unsigned)rem, 1, (unsigned)splits), 64 + 128 * G, C::kSmemRequest, ctx->stream>>>(
                tw, tw2, tx, ops, static_cast<YT *>(a.y), a.extra, (int)a.M, (int)a.N, (int)a.K, a.ldy, a.epilogue, tail,
                ctx->dev_status);
            ctx->launches += 2;
            SHREWQ_CUDA_TRY(ctx, cudaGetLastError());
            return SHREWQ_OK;
        }
    }
    if (p.splits > 1) {
        const size_t tiles = (size_t)p.n_tiles * p.m_tiles;
        const size_t part_bytes = tiles * p.splits * TOK * kTileN * sizeof(float);
        if (fixed_scratch) {
            const size_t need = 4096 + part_bytes;
            if (need > fixed_scratch_bytes)
                return set_err(ctx, SHREWQ_ERR_UNSUPPORTED,
                               "forward_noalloc: this shape needs %zu bytes of split-K scratch, the built-in array holds %zu "
                               "(use shrewq_linear_forward, which allocates)", need, fixed_scratch_bytes);
            // the array keeps whatever the previous call left: the counters must start at zero
            SHREWQ_CUDA_TRY(ctx, cudaMemsetAsync(fixed_scratch, 0, 4096, ctx->stream));
            sk.counters = static_cast<unsigned int *>(fixed_scratch);
            sk.partials = reinterpret_cast<float *>(static_cast<unsigned char *>(fixed_scratch) + 4096);
        } else {
            // context scratch: [0,4096) quantizer words, [4096,8192) tile counters (at most one
            // per SM is ever in use), partial sums from 8192
            if ((rc = ensure_scratch(ctx, kScratchPartialOff + part_bytes)) != SHREWQ_OK) return rc;
            if (!ctx->counters_zeroed) {
                // fresh scratch: counters must start at zero (the kernels reset them after use)
                SHREWQ_CUDA_TRY(ctx, cudaMemsetAsync(static_cast<char *>(ctx->scratch) + kScratchCounterOff, 0,
                                                     kScratchPartialOff - kScratchCounterOff, ctx->stream));
                ctx->counters_zeroed = true;
            }
            sk.counters = reinterpret_cast<unsigned int *>(static_cast<char *>(ctx->scratch) + kScratchCounterOff);
            sk.partials = reinterpret_cast<float *>(static_cast<char *>(ctx->scratch) + kScratchPartialOff);
        }
    }
    dim3 grid((unsigned)p.n_tiles, (unsigned)p.m_tiles, (unsigned)p.splits);
    kern<<<grid, 64 + 128 * G, C::kSmemRequest, ctx->stream>>>(tw, tw2, tx, ops, static_cast<YT *>(a.y), a.extra, (int)a.M,
                                                                (int)a.N, (int)a.K, a.ldy, a.epilogue, sk,
                                                                ctx->dev_status);
    ctx->launches += 1;
    SHREWQ_CUDA_TRY(ctx, cudaGetLastError());
    return SHREWQ_OK;
}

template <int TOK, int KSUB, bool GATED, typename YT>
int launch_groups(shrewq_ctx *ctx, const ForwardArgs &a, const CUtensorMap &tw, const CUtensorMap &tw2, const Tuning &t,
                  void *fs, size_t fsb) {
    if (t.groups == 1) return launch_cfg<TOK, KSUB, 1, GATED, YT>(ctx, a, tw, tw2, t.splitk, fs, fsb);
    if (t.groups == 2) return launch_cfg<TOK, KSUB, 2, GATED, YT>(ctx, a, tw, tw2, t.splitk, fs, fsb);
    return launch_cfg<TOK, KSUB, 3, GATED, YT>(ctx, a, tw, tw2, t.splitk, fs, fsb);
}

// Token tile: the smallest tile that covers M up to 256; above that 256 tokens, unless
// 128-token tiles fill the SMs markedly better (few channel tiles, e.g. N = 4096 at M = 512).
int choose_tok(const ForwardArgs &a, int chan_per_tile, int sm_count) {
    if (a.M <= 16) return 16;
    if (a.M <= 32) return 32;
    if (a.M <= 64) return 64;
    if (a.M <= 128) return 128;
    const long n_tiles = (long)((a.N + chan_per_tile - 1) / chan_per_tile);
    auto fill = [&](int tok) {
        const long tiles = n_tiles * (long)((a.M + tok - 1) / tok);
        const long waves = (tiles + sm_count - 1) / sm_count;
        return (double)tiles / (double)(waves * sm_count);
    };
    return fill(128) * 0.85 > fill(256) ? 128 : 256;
}

template <bool GATED, typename YT>
int launch_y(shrewq_ctx *ctx, const ForwardArgs &a, const CUtensorMap &tw, const CUtensorMap &tw2, void *fs, size_t fsb) {
    const Tuning t = read_tuning();
    const int tok = t.tok ? t.tok : choose_tok(a, GATED ? 64 : 128, ctx->sm_count);
    switch (tok) {
        // small token tiles are HBM-bound: 2 sub-blocks per stage keeps the pipeline 6-7 stages
        // deep (TMEM columns limit the depth), i.e. ~100 KB of codes in flight per SM
        case 16: return launch_groups<16, 2, GATED, YT>(ctx, a, tw, tw2, t, fs, fsb);
        case 32: return launch_groups<32, 2, GATED, YT>(ctx, a, tw, tw2, t, fs, fsb);
        case 64: return launch_groups<64, 2, GATED, YT>(ctx, a, tw, tw2, t, fs, fsb);
        case 128: return launch_groups<128, 2, GATED, YT>(ctx, a, tw, tw2, t, fs, fsb);
        default: return launch_groups<256, 1, GATED, YT>(ctx, a, tw, tw2, t, fs, fsb);
    }
}

// ---- forward without any allocation ---------------------------------------------------
// Split-K scratch for shrewq_linear_forward_noalloc: a fixed array inside the library image
// instead of a cudaMalloc'd buffer.  Every GPU that loads the library holds these 4 MiB
// until the process exits.  Layout: [0,4096) tile counters, partial sums from 4096.
constexpr size_t kStaticScratchBytes = 4u << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code the array's name is only a handle for the runtime, not a device address:
// the address is looked up once per device (with that device current) and cached.
constexpr int kMaxDevices = 64;
static void *g_static_scratch_addr[kMaxDevices] = {nullptr};

int static_scratch_for_device(shrewq_ctx *ctx, void **out) {
    if (ctx->device < 0 || ctx->device >= kMaxDevices)
        return set_err(ctx, SHREWQ_ERR_UNSUPPORTED, "forward_noalloc: device index %d above %d", ctx->device, kMaxDevices - 1);
    if (!g_static_scratch_addr[ctx->device]) {
        void *p = nullptr;
        SHREWQ_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || !p)
            return set_err(ctx, SHREWQ_ERR_CUDA, "forward_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        g_static_scratch_addr[ctx->device] = p;
    }
    *out = g_static_scratch_addr[ctx->device];
    return SHREWQ_OK;
}

}  // namespace

#ifdef SHREWQ_TRACE
extern "C" __attribute__((visibility("default"))) int shrewq_debug_set_trace(long long *dev_buf) {
    return (int)cudaMemcpyToSymbol(g_trace, &dev_buf, sizeof(dev_buf));
}
#endif

bool tcgen05_supported(const ForwardArgs &a) {
    return a.x_dtype == SHREWQ_BF16 && a.K >= 16 && (a.K % 16) == 0 && a.M >= 1 && a.N >= 1 &&
           (reinterpret_cast<uintptr_t>(a.x) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.q) & 15) == 0 &&
           (!a.q_up || (reinterpret_cast<uintptr_t>(a.q_up) & 15) == 0) && a.K < (1u << 31) && a.N < (1u << 31) &&
           a.M < (1u << 31) && (a.M + 15) / 16 <= 65535 * 16;
}

// box_rows = 128 for plain tiles, 64 for the gate / up halves of a gated tile
int encode_weight_tmap(shrewq_ctx *ctx, const int8_t *q, size_t n, size_t k, int box_rows, void *tmap_out) {
    return encode_2d(ctx, static_cast<CUtensorMap *>(tmap_out), CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, q, k, n, kBlockK,
                     box_rows, CU_TENSOR_MAP_SWIZZLE_64B);
}

int launch_gemm_tcgen05_noalloc(shrewq_ctx *ctx, const ForwardArgs &a, const void *w_tmap) {
    const CUtensorMap &tw = *static_cast<const CUtensorMap *>(w_tmap);
    void *base = nullptr;
    int rc = static_scratch_for_device(ctx, &base);
    if (rc != SHREWQ_OK) return rc;
    if (a.y_dtype == SHREWQ_BF16) return launch_y<false, __nv_bfloat16>(ctx, a, tw, tw, base, kStaticScratchBytes);
    return launch_y<false, float>(ctx, a, tw, tw, base, kStaticScratchBytes);
}

// w_tmap: 128-row boxes of the weight (plain) or 64-row boxes of the gate matrix (gated, with
// w_up_tmap the 64-row boxes of the up matrix)
int launch_gemm_tcgen05(shrewq_ctx *ctx, const ForwardArgs &a, const void *w_tmap, const void *w_up_tmap) {
    const CUtensorMap &tw = *static_cast<const CUtensorMap *>(w_tmap);
    if (a.q_up) {
        const CUtensorMap &tw2 = *static_cast<const CUtensorMap *>(w_up_tmap);
        if (a.y_dtype == SHREWQ_BF16) return launch_y<true, __nv_bfloat16>(ctx, a, tw, tw2, nullptr, 0);
        return launch_y<true, float>(ctx, a, tw, tw2, nullptr, 0);
    }
    if (a.y_dtype == SHREWQ_BF16) return launch_y<false, __nv_bfloat16>(ctx, a, tw, tw, nullptr, 0);
    return launch_y<false, float>(ctx, a, tw, tw, nullptr, 0);
}

}  // namespace shrewq
