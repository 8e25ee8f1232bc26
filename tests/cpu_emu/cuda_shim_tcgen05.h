// Stand-ins for the PTX pieces of shrew_b200/csrc/ptx_tcgen05.cuh: mbarriers, 2-D TMA loads with
// shared-memory swizzle, tensor memory, tcgen05.mma (kind::f16, A from tensor memory, B through a
// shared-memory descriptor), named barriers.  Include after cuda_shim.h.
//
// TEST INFRASTRUCTURE ONLY.  The behaviour modelled here is the documented one as this project
// understands it; the single-CTA kernel that runs on top of it has passed its parity tests on B200s,
// which is what ties the model to the hardware (a model that read the swizzle, the descriptor or the
// tensor-memory layout differently would not reproduce that kernel's results).
//
// Asynchronous operations (TMA loads, MMAs, commits) complete at issue by default; in the deferred mode
// they are queued and performed later by polling threads (loads in an adversarial order, tensor-core
// work in issue order).  Shared-memory addresses are the low 32 bits of host addresses inside the
// block's dynamic shared memory.
#pragma once

#include <atomic>
#include <chrono>

#define __grid_constant__
#define __noinline__ __attribute__((noinline))

// What the kernel needs from a tensor map: a row-major 2-D tensor, a box, a swizzle mode.
struct CUtensorMap {
    const void *base;
    uint32_t elem_bytes;
    uint64_t dim_inner, dim_outer;   // elements
    uint64_t row_stride_bytes;
    uint32_t box_inner, box_outer;   // elements
    int swizzle_bytes;               // 0, 64 or 128
};

namespace emu {
// a shared-memory address of this block or, in a cluster, of any member (shared::cluster window)
inline uint8_t *smem_ptr(uint32_t addr) {
    const uintptr_t base = reinterpret_cast<uintptr_t>(g_block->region);
    const uintptr_t p = (base & ~uintptr_t(0xFFFFFFFFu)) | addr;
    if (!(p >= base && p + 16 <= base + g_block->region_bytes)) {
        static uint8_t sink[64];  // keep the run alive; it is reported as failed
        fail("shared-memory address outside the cluster's shared memory");
        return sink;
    }
    return reinterpret_cast<uint8_t *>(p);
}
// Fault injection for the tests of the bounded waits: the load with this running number (counted over
// the whole launch, first load = 0) is dropped: no data, no bytes counted on its barrier.  -1 = none.
inline std::atomic<int> g_drop_tma{-1};
inline std::atomic<int> g_tma_count{0};
inline std::mutex g_mbar_mu;
inline void tma_progress();  // deferred modes: whoever polls a barrier may perform a queued load ...
inline void tc_progress();   // ... or the next queued tensor-core job  // one lock for every modelled mbarrier (a barrier may be touched from the peer block)
// the XOR the TMA applies when it writes, and tcgen05.mma when it reads: 16-byte chunk index bits
// [4,7) ^= address bits [7,10) (128-byte mode) or bits [4,6) ^= bits [7,9) (64-byte mode)
inline uint32_t swizzle(uint32_t addr, int mode) {
    if (mode == 128) return addr ^ (((addr >> 7) & 7u) << 4);
    if (mode == 64) return addr ^ (((addr >> 7) & 3u) << 4);
    return addr;
}
struct MBar {  // the 8 bytes of an mbarrier object
    uint32_t phase : 1, pending : 15, init : 15;
    int32_t tx;
};
static_assert(sizeof(MBar) == 8, "mbarrier object is 8 bytes");
inline void mbar_settle(MBar *b) {
    if (b->pending == 0 && b->tx == 0) {
        b->phase ^= 1;
        b->pending = b->init;
    }
}
}  // namespace emu

static inline uint32_t smem_u32(const void *p) { return (uint32_t)reinterpret_cast<uintptr_t>(p); }

static inline void mbar_init(uint32_t bar, uint32_t count) {
    std::lock_guard<std::mutex> g(emu::g_mbar_mu);
    auto *b = reinterpret_cast<emu::MBar *>(emu::smem_ptr(bar));
    b->phase = 0; b->pending = count; b->init = count; b->tx = 0;
}
static inline void mbar_fence_init() {}
static inline void mbar_arrive(uint32_t bar) {
    std::lock_guard<std::mutex> g(emu::g_mbar_mu);
    auto *b = reinterpret_cast<emu::MBar *>(emu::smem_ptr(bar));
    if (b->pending == 0) { emu::fail("more arrivals than the barrier was initialised for"); return; }
    b->pending -= 1;
    emu::mbar_settle(b);
}
static inline void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    std::lock_guard<std::mutex> g(emu::g_mbar_mu);
    auto *b = reinterpret_cast<emu::MBar *>(emu::smem_ptr(bar));
    if (b->pending == 0) { emu::fail("expect_tx: more arrivals than the barrier was initialised for"); return; }
    b->tx += (int32_t)bytes;
    b->pending -= 1;
    emu::mbar_settle(b);
}
static inline bool mbar_try(uint32_t bar, uint32_t parity) {
    emu::tma_progress();
    emu::tc_progress();
    bool done;
    {
        std::lock_guard<std::mutex> g(emu::g_mbar_mu);
        done = reinterpret_cast<emu::MBar *>(emu::smem_ptr(bar))->phase != (parity & 1u);  // that phase has completed
    }
    if (!done) std::this_thread::yield();
    return done;
}

// cp.async.bulk.tensor.2d ... mbarrier::complete_tx::bytes: box at element coordinates (c0 inner,
// c1 outer), out-of-range elements read as zero, the full box is counted on the barrier
namespace emu {
struct PendingTma {
    uint32_t dst;
    CUtensorMap tm;
    int c0, c1;
    uint32_t bar;
};
// Deferred mode (tests of ordering assumptions): a load is queued at issue and performed later, in RANDOM
// order, by whichever thread polls an mbarrier next.  0 = loads complete at issue.
inline std::atomic<unsigned> g_tma_async_seed{0};
inline std::atomic<unsigned> g_tma_one_in{8};  // a poll performs a queued load once in this many polls
inline std::mutex g_tma_mu;
inline std::vector<PendingTma> g_tma_pending;
inline void tma_perform(uint32_t dst, const CUtensorMap &tm, int c0, int c1, uint32_t bar);
inline void tma_progress() {
    if (g_tma_async_seed.load() == 0) return;
    PendingTma job;
    {
        std::lock_guard<std::mutex> g(g_tma_mu);
        if (g_tma_pending.empty()) return;
        static thread_local unsigned rng = 0;
        if (rng == 0) rng = g_tma_async_seed.load() * 2654435761u + (unsigned)(uintptr_t)&rng;
        rng = rng * 1664525u + 1013904223u;
        if ((rng >> 12) % g_tma_one_in.load() != 0) return;  // mostly: not yet (loads stay in flight for many polls)
        // usually the most recently issued load lands first (the worst order for a consumer that assumes
        // issue order), otherwise a random one
        const size_t pick = ((rng >> 20) & 3) ? g_tma_pending.size() - 1 : (rng >> 8) % g_tma_pending.size();
        job = g_tma_pending[pick];
        g_tma_pending.erase(g_tma_pending.begin() + pick);
    }
    tma_perform(job.dst, job.tm, job.c0, job.c1, job.bar);
}
}  // namespace emu

// cp.async.bulk (1-D): `bytes` from global memory to shared memory, counted on the barrier
static inline void bulk_load_1d(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    EMU_CHECK((dst & 15u) == 0 && (reinterpret_cast<uintptr_t>(src) & 15u) == 0 && (bytes & 15u) == 0, "bulk copy: 16-byte alignment and size");
    memcpy(emu::smem_ptr(dst), src, bytes);
    std::lock_guard<std::mutex> g(emu::g_mbar_mu);
    auto *b = reinterpret_cast<emu::MBar *>(emu::smem_ptr(bar));
    b->tx -= (int32_t)bytes;
    emu::mbar_settle(b);
}

static inline void tma_load_2d(uint32_t dst, const void *tmap_v, int c0, int c1, uint32_t bar) {
    const CUtensorMap &tm = *static_cast<const CUtensorMap *>(tmap_v);
    if (emu::g_tma_count.fetch_add(1) == emu::g_drop_tma.load()) return;  // injected fault: this load never lands
    if (emu::g_tma_async_seed.load() != 0) {
        std::lock_guard<std::mutex> g(emu::g_tma_mu);
        emu::g_tma_pending.push_back(emu::PendingTma{dst, tm, c0, c1, bar});
        return;
    }
    emu::tma_perform(dst, tm, c0, c1, bar);
}

inline void emu::tma_perform(uint32_t dst, const CUtensorMap &tm, int c0, int c1, uint32_t bar) {
    const uint32_t row_bytes = tm.box_inner * tm.elem_bytes;
    EMU_CHECK((dst & 15u) == 0 && ((uint32_t)c0 * tm.elem_bytes) % 16 == 0, "TMA alignment rules");
    EMU_CHECK(tm.swizzle_bytes == 0 || row_bytes == (uint32_t)tm.swizzle_bytes, "tm.swizzle_bytes == 0 || row_bytes == (uint32_t)tm.swizzle_bytes");
    for (uint32_t r = 0; r < tm.box_outer; ++r) {
        const int64_t row = (int64_t)c1 + r;
        for (uint32_t e = 0; e < tm.box_inner; ++e) {
            const int64_t col = (int64_t)c0 + e;
            const bool in = row >= 0 && row < (int64_t)tm.dim_outer && col >= 0 && col < (int64_t)tm.dim_inner;
            for (uint32_t by = 0; by < tm.elem_bytes; ++by) {
                const uint32_t off = dst + r * row_bytes + e * tm.elem_bytes + by;
                uint8_t v = 0;
                if (in) v = static_cast<const uint8_t *>(tm.base)[(uint64_t)row * tm.row_stride_bytes + (uint64_t)col * tm.elem_bytes + by];
                *emu::smem_ptr(emu::swizzle(off, tm.swizzle_bytes)) = v;
            }
        }
    }
    std::lock_guard<std::mutex> g(emu::g_mbar_mu);
    auto *b = reinterpret_cast<emu::MBar *>(emu::smem_ptr(bar));
    b->tx -= (int32_t)(tm.box_outer * row_bytes);
    emu::mbar_settle(b);
}

namespace emu {
// Deferred mode for tensor-core work (same switch and pace as the deferred TMA): tcgen05.mma and
// tcgen05.commit are queued at issue and executed later, IN ORDER, by whichever thread polls an mbarrier.
// An operand overwritten before its MMA has run (a missing wait on `empty`) then shows as a wrong result.
struct TcJob {
    Block *blk;                       // the issuing block (its shared and tensor memory)
    std::function<void()> run;
};
inline std::mutex g_tc_mu;
inline std::vector<TcJob> g_tc_queue;
inline bool tc_deferred() { return g_tma_async_seed.load() != 0; }
inline void tc_push(std::function<void()> fn) {
    std::lock_guard<std::mutex> g(g_tc_mu);
    g_tc_queue.push_back(TcJob{g_block, std::move(fn)});
}
inline void tc_progress() {
    if (!tc_deferred()) return;
    static thread_local unsigned rng = 12345u + (unsigned)(uintptr_t)&rng;
    rng = rng * 1664525u + 1013904223u;
    if ((rng >> 12) % g_tma_one_in.load() != 0) return;
    std::lock_guard<std::mutex> g(g_tc_mu);  // held while the job runs: jobs execute one at a time, in order
    if (g_tc_queue.empty()) return;
    TcJob job = std::move(g_tc_queue.front());
    g_tc_queue.erase(g_tc_queue.begin());
    Block *mine = g_block;
    g_block = job.blk;
    job.run();
    g_block = mine;
}
}  // namespace emu

static inline void tc_fence_before() {}
static inline void tc_fence_after() {}
static inline void tc_wait_st() {}
static inline void tc_wait_ld() {}
// the barrier is arrived on once the MMAs issued so far have completed
static inline void tc_commit(uint32_t bar) {
    if (emu::tc_deferred()) emu::tc_push([bar] { mbar_arrive(bar); });
    else mbar_arrive(bar);
}

static inline void tc_alloc_512(uint32_t result_smem) {
    emu::Block *blk = emu::g_block;
    if ((threadIdx.x & 31) == 0) {
        std::lock_guard<std::mutex> g(blk->mu);
        blk->tmem.assign(128 * 512, 0xDEADBEEFu);   // tensor memory is not zeroed by an allocation
        *reinterpret_cast<uint32_t *>(emu::smem_ptr(result_smem)) = 0;  // lane 0, column 0
    }
    __syncwarp();
}
static inline void tc_relinquish() {}
static inline void tc_dealloc_512(uint32_t) {}

// tcgen05.st / ld .32x32b: lane i of the warp accesses tensor-memory lane (taddr.lane + i), consecutive columns
static inline void tc_st32(uint32_t taddr, const uint32_t *r) {
    const uint32_t lane = (taddr >> 16) + (threadIdx.x & 31), col = taddr & 0xFFFF;
    if (!(lane < 128 && col + 32 <= 512)) { emu::fail("tcgen05.st outside tensor memory"); return; }
    EMU_CHECK((taddr >> 16) == 32 * ((threadIdx.x >> 5) & 3), "a warp may only touch the lane quadrant warp % 4");
    for (int i = 0; i < 32; ++i) emu::g_block->tmem[lane * 512 + col + i] = r[i];
}
static inline void tc_ld16(uint32_t taddr, uint32_t *r) {
    const uint32_t lane = (taddr >> 16) + (threadIdx.x & 31), col = taddr & 0xFFFF;
    if (!(lane < 128 && col + 16 <= 512)) { emu::fail("tcgen05.ld outside tensor memory"); return; }
    EMU_CHECK((taddr >> 16) == 32 * ((threadIdx.x >> 5) & 3), "a warp may only touch the lane quadrant warp % 4");
    for (int i = 0; i < 16; ++i) r[i] = emu::g_block->tmem[lane * 512 + col + i];
}

static inline void tc_ld32(uint32_t taddr, uint32_t *r) {
    const uint32_t lane = (taddr >> 16) + (threadIdx.x & 31), col = taddr & 0xFFFF;
    if (!(lane < 128 && col + 32 <= 512)) { emu::fail("tcgen05.ld outside tensor memory"); return; }
    EMU_CHECK((taddr >> 16) == 32 * ((threadIdx.x >> 5) & 3), "a warp may only touch the lane quadrant warp % 4");
    for (int i = 0; i < 32; ++i) r[i] = emu::g_block->tmem[lane * 512 + col + i];
}

// tcgen05.mma.cta_group::1.kind::f16 [d], [a], b_desc, idesc, p:  D[128 x N] (+)= A[128 x 16] * B[N x 16]^T,
// bf16 B, bf16 or f16 A (the descriptor's format fields), f32 accumulators.  A: tensor-memory lane m, 8 columns
// of two 16-bit values (even k in the lower half).  B: shared memory, K-major rows of 128 bytes, 8-row groups `stride byte offset` apart, 128-byte swizzle.
namespace emu { inline std::atomic<int> g_last_a_format{-1}; }  // A operand format of the latest MMA (for the tests)
static inline void tc_mma_ts_now(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate);
static inline void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    if (emu::tc_deferred()) emu::tc_push([=] { tc_mma_ts_now(d_tmem, a_tmem, b_desc, idesc, accumulate); });
    else tc_mma_ts_now(d_tmem, a_tmem, b_desc, idesc, accumulate);
}
static inline void tc_mma_ts_now(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    emu::Block *blk = emu::g_block;
    const uint32_t N = ((idesc >> 17) & 0x3Fu) << 3, Mrows = ((idesc >> 24) & 0x1Fu) << 4;
    EMU_CHECK(Mrows == 128 && N >= 8 && N <= 256 && N % 8 == 0, "Mrows == 128 && N >= 8 && N <= 256 && N % 8 == 0");
    // operand formats of kind::f16: 0 = f16, 1 = bf16, named separately for A [7,10) and B [10,13)
    const uint32_t a_fmt = (idesc >> 7) & 7u;
    emu::g_last_a_format = (int)a_fmt;
    EMU_CHECK(((idesc >> 4) & 3u) == 1 && a_fmt <= 1 && ((idesc >> 10) & 7u) == 1, "D f32, A f16 or bf16, B bf16");
    EMU_CHECK(((b_desc >> 61) & 7u) == 2 && ((b_desc >> 46) & 1u) == 1, "128-byte swizzle, descriptor version 1");
    const uint32_t start = (uint32_t)(b_desc & 0x3FFFu) << 4, sbo = (uint32_t)((b_desc >> 32) & 0x3FFFu) << 4;
    const uint32_t smem_hi = smem_u32(blk->dyn);  // 256 KiB aligned; the descriptor keeps the 18 low address bits
    const uint32_t dcol = d_tmem & 0xFFFF, acol = a_tmem & 0xFFFF;
    if (!((d_tmem >> 16) == 0 && (a_tmem >> 16) == 0 && dcol + N <= 512 && acol + 8 <= 512 && N >= 8 && N <= 256)) {
        emu::fail("tcgen05.mma operands outside tensor memory");
        return;
    }
    std::vector<float> b((size_t)N * 16);
    for (uint32_t n = 0; n < N; ++n)
        for (uint32_t k = 0; k < 16; ++k) {
            const uint32_t addr = (smem_hi | start) + (n >> 3) * sbo + (n & 7) * 128 + k * 2;
            uint16_t h;
            memcpy(&h, emu::smem_ptr(emu::swizzle(addr, 128)), 2);
            b[n * 16 + k] = __uint_as_float((uint32_t)h << 16);
        }
    for (uint32_t m = 0; m < 128; ++m) {
        float a[16];
        for (uint32_t k = 0; k < 16; ++k) {
            const uint32_t w = blk->tmem[m * 512 + acol + (k >> 1)];
            const uint32_t h = (k & 1) ? (w >> 16) : (w & 0xFFFF);
            a[k] = a_fmt == 1 ? __uint_as_float(h << 16) : (float)emu_f16_of(h);
        }
        for (uint32_t n = 0; n < N; ++n) {
            double acc = accumulate ? (double)__uint_as_float(blk->tmem[m * 512 + dcol + n]) : 0.0;
            for (uint32_t k = 0; k < 16; ++k) acc += (double)a[k] * (double)b[n * 16 + k];
            blk->tmem[m * 512 + dcol + n] = __float_as_uint((float)acc);
        }
    }
}

// bar.sync id, nthreads
static inline void named_bar_sync(int id, int nthreads) {
    emu::Block *blk = emu::g_block;
    std::barrier<> *bar;
    {
        std::lock_guard<std::mutex> g(blk->mu);
        auto &slot = blk->named[id];
        if (!slot) slot = std::make_unique<std::barrier<>>(nthreads);
        bar = slot.get();
    }
    bar->arrive_and_wait();
}

// ---- the remaining builtins the kernel uses -----------------------------------------------------------
template <typename T>
static inline int __all_sync(unsigned, T pred) {
    emu::Block *b = emu::g_block;
    const unsigned me = threadIdx.x, w0 = me & ~31u;
    b->slots[me] = pred ? 1 : 0;
    b->warp[me >> 5]->arrive_and_wait();
    int all = 1;
    for (unsigned i = 0; i < 32 && w0 + i < b->threads; ++i) all &= (int)b->slots[w0 + i];
    b->warp[me >> 5]->arrive_and_wait();
    return all;
}
