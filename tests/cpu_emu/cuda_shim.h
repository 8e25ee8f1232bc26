// A small stand-in for the CUDA execution model, enough to run the library's scalar kernels
// (quantize / dequantize families) on the CPU, thread by thread.
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
// Not modelled: memory ordering weaker than sequential, divergence inside a warp at a shuffle,
// dynamic shared memory, tensor-core and TMA instructions.
#pragma once
#define SHREWQ_CPU_EMU 1

#include <math.h>
#include <stdint.h>
#include <string.h>

#include <algorithm>
#include <barrier>
#include <functional>
#include <memory>
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
struct Block {
    unsigned threads;
    std::barrier<> all;
    std::vector<std::unique_ptr<std::barrier<>>> warp;
    std::vector<uint64_t> slots;  // one 8-byte exchange slot per thread
    explicit Block(unsigned t) : threads(t), all(t), slots(t) {
        for (unsigned w = 0; w < (t + 31) / 32; ++w) {
            const unsigned lanes = std::min(32u, t - w * 32);
            warp.emplace_back(std::make_unique<std::barrier<>>(lanes));
        }
    }
};
inline thread_local Block *g_block = nullptr;
}  // namespace emu

inline thread_local emu_uint3 threadIdx{0, 0, 0}, blockIdx{0, 0, 0};
inline thread_local emu_uint3 blockDim{1, 1, 1}, gridDim{1, 1, 1};

namespace emu {
// Runs `body` as a kernel of `grid` blocks of `block` threads (1-D).
inline void launch(unsigned grid, unsigned block, const std::function<void()> &body) {
    Block blk(block);
    std::vector<std::thread> pool;
    for (unsigned t = 0; t < block; ++t) {
        pool.emplace_back([&, t] {
            g_block = &blk;
            threadIdx = emu_uint3{t, 0, 0};
            blockDim = emu_uint3{block, 1, 1};
            gridDim = emu_uint3{grid, 1, 1};
            for (unsigned b = 0; b < grid; ++b) {
                blockIdx = emu_uint3{b, 0, 0};
                body();
                blk.all.arrive_and_wait();  // the next block reuses the shared variables
            }
        });
    }
    for (auto &th : pool) th.join();
}
}  // namespace emu

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

using std::max;
using std::min;
