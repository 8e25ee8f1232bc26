// Pieces shared by the tcgen05 forward kernels: the bounded mbarrier waits, the INT8 -> bf16 widening of
// the converter warps and the shared-memory descriptor of the activation tile.
#pragma once

#include "dests.cuh"
#include "ptx_small.cuh"
#include "ptx_tcgen05.cuh"

namespace shrewq {
namespace {

// Limits of a bounded wait: a few polls back to back, then polls with pauses in between (a fraction of a
// second in all).  The pauses matter for more than power: a thread that polls an mbarrier in a tight loop keeps
// the shared-memory pipe busy, and in a persistent kernel the producer and the MMA issuer wait for microseconds
// while the other warps run the epilogue through that same pipe.  The CPU tests that make a wait run out on
// purpose compile with smaller limits.
#ifndef SHREWQ_SPIN_FAST_LIMIT
#define SHREWQ_SPIN_FAST_LIMIT 2048u
#endif
#ifndef SHREWQ_SPIN_SLOW_LIMIT
#define SHREWQ_SPIN_SLOW_LIMIT (1u << 21)
#endif
constexpr uint32_t kSpinFast = SHREWQ_SPIN_FAST_LIMIT;
constexpr uint32_t kSpinSlow = SHREWQ_SPIN_SLOW_LIMIT;

struct Ctl {  // lives in shared memory
    volatile int abort_flag;
    uint32_t tmem_base;
};

// Slow path of the bounded wait, kept out of line so the hot loops only carry one try_wait.
// `code` is what DeviceStatus::timeout_flag reports (1 single-CTA kernel, 2 CTA-pair kernels).
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, Ctl *ctl, DeviceStatus *st, uint32_t role,
                                            uint32_t stage, uint32_t code) {
    for (uint32_t i = 0; i < kSpinFast; ++i)
        if (mbar_try(bar, parity)) return true;
    for (uint32_t i = 0; i < kSpinSlow; ++i) {
        if (mbar_try(bar, parity)) return true;
        if ((i & 15) == 15 && ctl->abort_flag) return false;
        __nanosleep(i < 256 ? 64 : 256);
    }
    ctl->abort_flag = 1;
    if (atomicCAS(&st->timeout_flag, 0u, code) == 0u) {
        st->where = (blockIdx.x << 8) | role;
        st->stage = stage;
        st->parity = parity;
    }
    return false;
}

// Bounded wait.  Returns false if it gave up or another role already did.
template <uint32_t CODE>
__device__ __forceinline__ bool mbar_wait_c(uint32_t bar, uint32_t parity, Ctl *ctl, DeviceStatus *st, uint32_t role,
                                            uint32_t stage) {
    if (mbar_try(bar, parity)) return true;
    if (mbar_try(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, ctl, st, role, stage, CODE);
}

// Warp-level wait: lane 0 polls, the outcome is broadcast with a shuffle (which also
// synchronises the warp and orders memory among its lanes).  32 lanes polling the same
// mbarrier word serialise in the shared-memory pipe.
template <uint32_t CODE>
__device__ __forceinline__ bool mbar_wait_warp_c(uint32_t bar, uint32_t parity, Ctl *ctl, DeviceStatus *st, uint32_t role,
                                                 uint32_t stage) {
    int ok = 1;
    if ((threadIdx.x & 31) == 0) ok = mbar_wait_c<CODE>(bar, parity, ctl, st, role, stage) ? 1 : 0;
    ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
    // every lane observes the completed phase itself (one try_wait that succeeds at once), so
    // each has its own acquire on the data the barrier guards
    if (ok) ok = mbar_try(bar, parity) ? 1 : 0;
    return __all_sync(0xFFFFFFFFu, ok) != 0;
}

// 4 INT8 codes (one 32-bit word) -> two packed bf16x2 words, exactly.
// byte ^ 0x80 = q + 128 as an unsigned byte u; 0x4B0000uu is the float 2^23 + u; subtracting
// 2^23 + 128 leaves q; cvt.rn.bf16x2.f32 packs two of them (exact, |q| <= 128).
__device__ __forceinline__ void cvt_i8x4_bf16(uint32_t w, uint32_t &lo, uint32_t &hi) {
    const uint32_t u = w ^ 0x80808080u;
    const float f0 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7440)) - 8388736.0f;
    const float f1 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7441)) - 8388736.0f;
    const float f2 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7442)) - 8388736.0f;
    const float f3 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7443)) - 8388736.0f;
    lo = pack_bf16x2_rn(f1, f0);
    hi = pack_bf16x2_rn(f3, f2);
}

// One weight row's 64 codes of a 64-byte-swizzled INT8 sub-block -> 32 packed bf16x2 words.  TMA wrote the
// row with the 64-byte swizzle: the 16-byte chunk c of row r sits at chunk position c ^ ((r >> 1) & 3).
__device__ __forceinline__ void convert_row64(const uint8_t *rowp, int swz, uint32_t *packed) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const uint4 v = *reinterpret_cast<const uint4 *>(rowp + ((c ^ swz) << 4));
        cvt_i8x4_bf16(v.x, packed[8 * c + 0], packed[8 * c + 1]);
        cvt_i8x4_bf16(v.y, packed[8 * c + 2], packed[8 * c + 3]);
        cvt_i8x4_bf16(v.z, packed[8 * c + 4], packed[8 * c + 5]);
        cvt_i8x4_bf16(v.w, packed[8 * c + 6], packed[8 * c + 7]);
    }
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

}  // namespace
}  // namespace shrewq
