// The few PTX instructions the warp-MMA kernels use, each behind a small function, and the
// declaration of dynamic shared memory.  The CPU tests (tests/cpu_emu/) provide stand-ins with the
// same names and semantics, so the kernels that call them also compile as plain C++.
#pragma once

#ifndef SHREWQ_CPU_EMU
#include <cuda_runtime.h>
#include <stdint.h>

namespace shrewq {
namespace {

// 16 bytes through the read-only path, not kept in L1 (weights are read once)
__device__ __forceinline__ uint4 ld_stream_16(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// two f32 -> packed bf16x2, round to nearest even; `hi` lands in the upper half
__device__ __forceinline__ uint32_t pack_bf16x2_rn(float hi, float lo) {
    uint32_t d;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}

// per-half f16 subtraction a - b
// (a0, a1) += (b0, b1) as one packed f32x2 instruction (sm_100: half the issue slots of two scalar adds)
__device__ __forceinline__ void add_f32x2(float &a0, float &a1, float b0, float b1) {
    asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%0, %1};\n\tmov.b64 rb, {%2, %3};\n\tadd.rn.f32x2 rd, ra, rb;\n\t"
        "mov.b64 {%0, %1}, rd;\n\t}"
        : "+f"(a0), "+f"(a1)
        : "f"(b0), "f"(b1));
}

__device__ __forceinline__ uint32_t sub_f16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

// D[16x8] += A[16x16] * B[16x8], bf16 operands, f32 accumulate
__device__ __forceinline__ void mma_bf16_16816(float *d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// D[16x8] += A[16x16] * B[16x8], f16 operands, f32 accumulate
__device__ __forceinline__ void mma_f16_16816(float *d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// One f32 from L2 (not kept in L1), as an instruction the compiler may not reorder or merge with its
// neighbours: a run of these is issued back to back, so that all of them are in flight before the first
// value is consumed.
__device__ __forceinline__ float ld_cg_ordered(const float *p) {
    float v;
    asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}

// system-scope release store / acquire load of one word (flags that another GPU reads or writes)
__device__ __forceinline__ void st_release_sys_u32(uint32_t *p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void fence_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
__device__ __forceinline__ void sleep_ns(uint32_t ns) { asm volatile("nanosleep.u32 %0;" ::"r"(ns) : "memory"); }

// programmatic dependent launch: let the next kernel of the stream start / wait for the previous one
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

}  // namespace
}  // namespace shrewq

#define SHREWQ_DYNAMIC_SMEM(T, name) extern __shared__ __align__(16) T name[]
#endif  // SHREWQ_CPU_EMU
