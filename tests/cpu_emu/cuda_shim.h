// A small stand-in for the CUDA execution model, enough to run the library's scalar and warp-MMA
// kernels (quantize / dequantize families, the small-batch forward) on the CPU, thread by thread.
//
// TEST INFRASTRUCTURE ONLY.  Nothing in the shipped library includes this file; the product has
// no CPU path.  The CPU tests compile the device-code headers (shrew_b200/csrc/*_kernels.cuh)
// against this shim and compare what the kernels compute with the golden vectors, so that kernel
// logic (index arithmetic, reductions, rounding paths, special values) is exercised without a GPU.
//
// Model: one launch = grid.x blocks run one after the other; a block = blockDim.x real threads
// (std::thread) that share the kernel's `__shared__` variables (function-local statics) and meet at
// __syncthreads() (a std::barrier).  Warp shuffles exchange through a per-warp slot array between
// two warp barriers; every lane of a warp must take part, as with a full mask on the GPU.
// mma.sync.m16n8k16 is computed from its documented fragment layout; the other PTX pieces the
// warp-MMA kernels use (shrew_b200/csrc/ptx_small.cuh) have plain C++ stand-ins of the same name.
// Not modelled: memory ordering weaker than sequential, divergence inside a warp at a shuffle,
// tcgen05 / TMEM / TMA instructions.
#pragma once
#define SHREWQ_CPU_EMU 1

#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <atomic>
#include <barrier>
#include <chrono>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <thread>
#include <vector>

#define __global__
#define __device__
#define __host__
#define __forceinline__ inline
#define __restrict__
#define __launch_bounds__(...)
#define __shared__ static

struct emu_uint3 { unsigned x, y, z; };
struct float4 { float x, y, z, w; };
struct uint4 { unsigned x, y, z, w; };
static inline float4 make_float4(float x, float y, float z, float w) { return float4{x, y, z, w}; }
static inline uint4 make_uint4(unsigned x, unsigned y, unsigned z, unsigned w) { return uint4{x, y, z, w}; }

namespace emu {
// A violated rule of the model (more arrivals than a barrier expects, a tensor-memory access outside the
// warp's quadrant, ...) is recorded, not fatal: the harness reports it as a failed run.
inline std::atomic<bool> g_failed{false};
inline char g_fail_msg[256] = {0};
inline void fail(const char *what) {
    bool expected = false;
    if (g_failed.compare_exchange_strong(expected, true)) strncpy(g_fail_msg, what, sizeof(g_fail_msg) - 1);
}
#define EMU_CHECK(cond, what) do { if (!(cond)) emu::fail(what); } while (0)

struct Block {
    unsigned threads;
    std::barrier<> all;
    std::vector<std::unique_ptr<std::barrier<>>> warp;
    std::vector<uint64_t> slots;  // one 8-byte exchange slot per thread
    std::vector<uint32_t> frag;   // eight 32-bit registers per thread: MMA operand fragments
    unsigned char *dyn = nullptr;    // dynamic shared memory of the block, 256 KiB aligned: like real shared
    size_t dyn_bytes = 0;            // addresses, its offsets fit the 18 address bits a matrix descriptor keeps
    std::mutex mu;                   // serialises the modelled mbarrier / named-barrier bookkeeping
    std::vector<uint32_t> tmem;      // tensor memory: 128 lanes x 512 columns of 32 bits (allocated on first use)
    std::map<int, std::unique_ptr<std::barrier<>>> named;  // bar.sync id -> barrier
    // thread-block cluster (pairs): rank in the cluster, the member blocks, the cluster-wide barrier, and
    // the region that holds every member's shared memory back to back (256 KiB each)
    unsigned rank = 0;
    Block *cluster[2] = {nullptr, nullptr};
    std::barrier<> *cluster_bar = nullptr;
    unsigned char *region = nullptr;
    size_t region_bytes = 0;
    bool owns_region = false;
    // `shared`: this block's 256 KiB window inside a cluster region; null = allocate an own window
    explicit Block(unsigned t, size_t dyn_b = 0, unsigned char *shared = nullptr)
        : threads(t), all(t), slots(t), frag(8 * (size_t)t), dyn_bytes(dyn_b) {
        for (unsigned w = 0; w < (t + 31) / 32; ++w) {
            const unsigned lanes = std::min(32u, t - w * 32);
            warp.emplace_back(std::make_unique<std::barrier<>>(lanes));
        }
        cluster[0] = this;
        if (shared) {
            dyn = shared;
        } else {
            dyn = static_cast<unsigned char *>(std::aligned_alloc(size_t(1) << 18, size_t(1) << 18));
            region = dyn;
            region_bytes = size_t(1) << 18;
            owns_region = true;
        }
        memset(dyn, 0xA5, size_t(1) << 18);  // shared memory starts with whatever was there
    }
    ~Block() { if (owns_region) std::free(dyn); }
    Block(const Block &) = delete;
};
inline thread_local Block *g_block = nullptr;
}  // namespace emu

inline thread_local emu_uint3 threadIdx{0, 0, 0}, blockIdx{0, 0, 0};
inline thread_local emu_uint3 blockDim{1, 1, 1}, gridDim{1, 1, 1};

namespace emu {
// Runs `body` as a kernel of `grid` blocks of `block` threads (1-D) with `dyn_bytes` of dynamic
// shared memory per block.
inline void launch3(unsigned gx, unsigned gy, unsigned gz, unsigned block, size_t dyn_bytes, const std::function<void()> &body) {
    Block blk(block, dyn_bytes);
    std::vector<std::thread> pool;
    for (unsigned t = 0; t < block; ++t) {
        pool.emplace_back([&, t] {
            g_block = &blk;
            threadIdx = emu_uint3{t, 0, 0};
            blockDim = emu_uint3{block, 1, 1};
            gridDim = emu_uint3{gx, gy, gz};
            for (unsigned z = 0; z < gz; ++z)
                for (unsigned y = 0; y < gy; ++y)
                    for (unsigned x = 0; x < gx; ++x) {
                        blockIdx = emu_uint3{x, y, z};
                        body();
                        blk.all.arrive_and_wait();  // the next block reuses the shared variables
                    }
        });
    }
    for (auto &th : pool) th.join();
}
inline void launch(unsigned grid, unsigned block, size_t dyn_bytes, const std::function<void()> &body) {
    launch3(grid, 1, 1, block, dyn_bytes, body);
}
// Clusters of 2 blocks along x: the two blocks of a cluster run at the same time (2 * block threads),
// clusters one after the other.  gx must be even.
inline void launch_cluster2(unsigned gx, unsigned gy, unsigned gz, unsigned block, size_t dyn_bytes, const std::function<void()> &body) {
    unsigned char *region = static_cast<unsigned char *>(std::aligned_alloc(size_t(1) << 19, size_t(1) << 19));
    {
        Block b0(block, dyn_bytes, region), b1(block, dyn_bytes, region + (size_t(1) << 18));
        std::barrier<> cluster_bar(2 * block);
        Block *both[2] = {&b0, &b1};
        for (unsigned r = 0; r < 2; ++r) {
            both[r]->rank = r;
            both[r]->cluster[0] = &b0;
            both[r]->cluster[1] = &b1;
            both[r]->cluster_bar = &cluster_bar;
            both[r]->region = region;
            both[r]->region_bytes = size_t(1) << 19;
        }
        std::vector<std::thread> pool;
        for (unsigned r = 0; r < 2; ++r)
            for (unsigned t = 0; t < block; ++t) {
                pool.emplace_back([&, r, t] {
                    g_block = both[r];
                    threadIdx = emu_uint3{t, 0, 0};
                    blockDim = emu_uint3{block, 1, 1};
                    gridDim = emu_uint3{gx, gy, gz};
                    for (unsigned z = 0; z < gz; ++z)
                        for (unsigned y = 0; y < gy; ++y)
                            for (unsigned c = 0; c < gx / 2; ++c) {
                                blockIdx = emu_uint3{2 * c + r, y, z};
                                body();
                                cluster_bar.arrive_and_wait();  // the next cluster reuses the blocks' memories
                            }
                });
            }
        for (auto &th : pool) th.join();
    }
    std::free(region);
}
}  // namespace emu

namespace emu {
inline void launch(unsigned grid, unsigned block, const std::function<void()> &body) { launch(grid, block, 0, body); }
inline void *dynamic_smem() { return g_block->dyn; }
}  // namespace emu
#define SHREWQ_DYNAMIC_SMEM(T, name) T *name = static_cast<T *>(emu::dynamic_smem())

static inline void __syncthreads() { emu::g_block->all.arrive_and_wait(); }
static inline void __syncwarp(unsigned = 0xFFFFFFFFu) { emu::g_block->warp[threadIdx.x >> 5]->arrive_and_wait(); }

template <typename T>
static inline T __shfl_xor_sync(unsigned, T v, int lane_mask) {
    static_assert(sizeof(T) <= 8, "shuffle of at most 8 bytes");
    emu::Block *b = emu::g_block;
    const unsigned me = threadIdx.x, partner = (me & ~31u) | ((me ^ (unsigned)lane_mask) & 31u);
    uint64_t raw = 0;
    memcpy(&raw, &v, sizeof(T));
    b->slots[me] = raw;
    b->warp[me >> 5]->arrive_and_wait();
    const uint64_t got = partner < b->threads ? b->slots[partner] : raw;
    b->warp[me >> 5]->arrive_and_wait();
    T out;
    memcpy(&out, &got, sizeof(T));
    return out;
}
template <typename T>
static inline T __shfl_sync(unsigned, T v, int src_lane) {
    emu::Block *b = emu::g_block;
    const unsigned me = threadIdx.x, src = (me & ~31u) | ((unsigned)src_lane & 31u);
    uint64_t raw = 0;
    memcpy(&raw, &v, sizeof(T));
    b->slots[me] = raw;
    b->warp[me >> 5]->arrive_and_wait();
    const uint64_t got = b->slots[src];
    b->warp[me >> 5]->arrive_and_wait();
    T out;
    memcpy(&out, &got, sizeof(T));
    return out;
}

// ---- bit casts, rounding-mode intrinsics (compile with -ffp-contract=off) -------------------------
static inline unsigned __float_as_uint(float f) { unsigned u; memcpy(&u, &f, 4); return u; }
static inline float __uint_as_float(unsigned u) { float f; memcpy(&f, &u, 4); return f; }
static inline double __dmul_rn(double a, double b) { return a * b; }
static inline double __dadd_rn(double a, double b) { return a + b; }
static inline double __dsub_rn(double a, double b) { return a - b; }
static inline float __double2float_rz(double v) {
    float f = (float)v;  // to nearest
    if (v == v && fabs((double)f) > fabs(v)) f = nextafterf(f, 0.0f);  // pull back toward zero (Inf -> FLT_MAX)
    return f;
}

// ---- loads / stores with cache hints --------------------------------------------------------------
template <typename T> static inline T __ldg(const T *p) { return *p; }
template <typename T> static inline T __ldcs(const T *p) { return *p; }
template <typename T> static inline T __ldcg(const T *p) { return *p; }
template <typename T> static inline void __stcs(T *p, T v) { *p = v; }
template <typename T> static inline void __stcg(T *p, T v) { *p = v; }

// ---- atomics on 32-bit unsigned ---------------------------------------------------------------------
static inline unsigned atomicMax(unsigned *p, unsigned v) {
    unsigned old = __atomic_load_n(p, __ATOMIC_SEQ_CST);
    while (old < v && !__atomic_compare_exchange_n(p, &old, v, false, __ATOMIC_SEQ_CST, __ATOMIC_SEQ_CST)) {}
    return old;
}
static inline unsigned atomicMin(unsigned *p, unsigned v) {
    unsigned old = __atomic_load_n(p, __ATOMIC_SEQ_CST);
    while (old > v && !__atomic_compare_exchange_n(p, &old, v, false, __ATOMIC_SEQ_CST, __ATOMIC_SEQ_CST)) {}
    return old;
}

// ---- bf16 / f16 -----------------------------------------------------------------------------------
struct __nv_bfloat16 { uint16_t bits; };
static inline float __bfloat162float(__nv_bfloat16 h) { return __uint_as_float((unsigned)h.bits << 16); }
static inline __nv_bfloat16 __float2bfloat16_rn(float f) {
    unsigned u = __float_as_uint(f);
    if (f != f) return __nv_bfloat16{0x7FFF};
    u += 0x7FFFu + ((u >> 16) & 1u);
    return __nv_bfloat16{(uint16_t)(u >> 16)};
}
struct __half { _Float16 v; };
static inline __half __float2half_rn(float f) { return __half{(_Float16)f}; }
static inline unsigned short __half_as_ushort(__half h) { unsigned short u; memcpy(&u, &h.v, 2); return u; }
static inline float __half2float(__half h) { return (float)h.v; }
static inline __half __double2half(double v) { return __half{(_Float16)v}; }  // one rounding, to nearest even
static inline long long __double_as_longlong(double v) { long long b; memcpy(&b, &v, 8); return b; }
static inline double __longlong_as_double(long long b) { double v; memcpy(&v, &b, 8); return v; }
static inline unsigned long long atomicMax(unsigned long long *p, unsigned long long v) {
    unsigned long long old = __atomic_load_n(p, __ATOMIC_SEQ_CST);
    while (old < v && !__atomic_compare_exchange_n(p, &old, v, false, __ATOMIC_SEQ_CST, __ATOMIC_SEQ_CST)) {}
    return old;
}
static inline unsigned long long atomicMin(unsigned long long *p, unsigned long long v) {
    unsigned long long old = __atomic_load_n(p, __ATOMIC_SEQ_CST);
    while (old > v && !__atomic_compare_exchange_n(p, &old, v, false, __ATOMIC_SEQ_CST, __ATOMIC_SEQ_CST)) {}
    return old;
}

static inline unsigned atomicCAS(unsigned *p, unsigned cmp, unsigned val) {
    __atomic_compare_exchange_n(p, &cmp, val, false, __ATOMIC_SEQ_CST, __ATOMIC_SEQ_CST);
    return cmp;
}
static inline unsigned atomicAdd(unsigned *p, unsigned v) { return __atomic_fetch_add(p, v, __ATOMIC_SEQ_CST); }
static inline void __threadfence() { __atomic_thread_fence(__ATOMIC_SEQ_CST); }
static inline void __nanosleep(unsigned) { std::this_thread::sleep_for(std::chrono::microseconds(50)); }
// flags another GPU reads or writes: sequentially consistent atomics here
static inline void st_release_sys_u32(uint32_t *p, uint32_t v) { __atomic_store_n(p, v, __ATOMIC_SEQ_CST); }
static inline uint32_t ld_acquire_sys_u32(const uint32_t *p) { return __atomic_load_n(p, __ATOMIC_SEQ_CST); }
static inline void fence_sys() { __atomic_thread_fence(__ATOMIC_SEQ_CST); }
static inline void sleep_ns(uint32_t) { std::this_thread::sleep_for(std::chrono::microseconds(20)); }

using std::max;
using std::min;

// ---- the PTX pieces of shrew_b200/csrc/ptx_small.cuh -----------------------------------------------
static inline unsigned __byte_perm(unsigned x, unsigned y, unsigned sel) {
    const uint64_t both = ((uint64_t)y << 32) | x;
    unsigned out = 0;
    for (int i = 0; i < 4; ++i) out |= (unsigned)((both >> (8 * ((sel >> (4 * i)) & 7))) & 0xFF) << (8 * i);
    return out;
}
#define __expf expf
static inline float __fdividef(float a, float b) { return a / b; }
static inline uint4 ld_stream_16(const void *p) { uint4 v; memcpy(&v, p, 16); return v; }
static inline float ld_cg_ordered(const float *p) { return *p; }
static inline void pdl_launch_dependents() {}   // launches are sequential here
static inline void pdl_wait() {}
static inline void add_f32x2(float &a0, float &a1, float b0, float b1) { a0 += b0; a1 += b1; }
static inline uint32_t pack_bf16x2_rn(float hi, float lo) {
    return ((uint32_t)__float2bfloat16_rn(hi).bits << 16) | __float2bfloat16_rn(lo).bits;
}
static inline _Float16 emu_f16_of(uint32_t bits16) { uint16_t u = (uint16_t)bits16; _Float16 h; memcpy(&h, &u, 2); return h; }
static inline uint32_t emu_bits_of(_Float16 h) { uint16_t u; memcpy(&u, &h, 2); return u; }
static inline uint32_t sub_f16x2(uint32_t a, uint32_t b) {
    const _Float16 lo = emu_f16_of(a & 0xFFFF) - emu_f16_of(b & 0xFFFF), hi = emu_f16_of(a >> 16) - emu_f16_of(b >> 16);
    return emu_bits_of(lo) | (emu_bits_of(hi) << 16);
}

// mma.sync.aligned.m16n8k16.row.col.f32.{bf16|f16}.{bf16|f16}.f32: D[16x8] += A[16x16] * B[16x8].
// Lane (g = lane / 4, t = lane % 4) holds  a0: A[g][2t,2t+1]  a1: A[g+8][2t,2t+1]  a2: A[g][2t+8,2t+9]
// a3: A[g+8][2t+8,2t+9];  b0: B[2t,2t+1][g]  b1: B[2t+8,2t+9][g];  d0,d1: D[g][2t,2t+1]  d2,d3: D[g+8][2t,2t+1];
// the lower half of a register is the element with the even k.
template <bool F16>
static inline void emu_mma_16816(float *d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    emu::Block *blk = emu::g_block;
    const unsigned me = threadIdx.x, w0 = me & ~31u, lane = me & 31u, g = lane >> 2, t = lane & 3u;
    uint32_t *mine = &blk->frag[8 * (size_t)me];
    mine[0] = a0; mine[1] = a1; mine[2] = a2; mine[3] = a3; mine[4] = b0; mine[5] = b1;
    blk->warp[me >> 5]->arrive_and_wait();
    auto val = [](uint32_t reg, unsigned odd) -> double {
        const uint32_t h = odd ? (reg >> 16) : (reg & 0xFFFF);
        return F16 ? (double)emu_f16_of(h) : (double)__uint_as_float(h << 16);
    };
    auto A = [&](unsigned row, unsigned k) { return val(blk->frag[8 * (size_t)(w0 + (row & 7) * 4 + ((k & 7) >> 1)) + (row >> 3) + 2 * (k >> 3)], k & 1); };
    auto B = [&](unsigned k, unsigned n) { return val(blk->frag[8 * (size_t)(w0 + n * 4 + ((k & 7) >> 1)) + 4 + (k >> 3)], k & 1); };
    float out[4];
    for (unsigned r = 0; r < 4; ++r) {
        const unsigned row = g + ((r & 2) ? 8 : 0), col = 2 * t + (r & 1);
        double acc = d[r];
        for (unsigned k = 0; k < 16; ++k) acc += A(row, k) * B(k, col);
        out[r] = (float)acc;
    }
    blk->warp[me >> 5]->arrive_and_wait();  // everybody has read the fragments before they are overwritten
    for (unsigned r = 0; r < 4; ++r) d[r] = out[r];
}
static inline void mma_bf16_16816(float *d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    emu_mma_16816<false>(d, a0, a1, a2, a3, b0, b1);
}
static inline void mma_f16_16816(float *d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    emu_mma_16816<true>(d, a0, a1, a2, a3, b0, b1);
}

