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
// With NW == 2 the CTA carries two weight matrices (gate and up) over the same
// activations and two accumulators, and the epilogue writes silu(gate)*up.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM allocator + MMA issuer,
// warps 2..5 = converters (one TMEM lane quadrant each), which then run the epilogue.
// Pipeline per k-block of 64: full[s] (TMA bytes landed) -> converters -> aready[s] ->
// MMA -> tcgen05.commit -> empty[s] -> producer.  Every wait is bounded: after the limit
// the waiter records where it gave up in a status block, raises a CTA-wide abort flag and
// all roles fall through to the common teardown, which frees TMEM.
#include <cuda.h>

#include "common.cuh"

namespace shrewq {
namespace {

constexpr int kTileN = 128;  // weight rows per CTA (MMA M, TMEM lanes)
constexpr int kBlockK = 64;  // k per pipeline stage
constexpr int kUmmaK = 16;
constexpr int kThreads = 192;
constexpr uint32_t kSpinFast = 1u << 14;
constexpr uint32_t kSpinSlow = 1u << 21;  // x ~100 ns sleeps: a fraction of a second

template <int TOK, int NW>
struct Cfg {
    static constexpr int kWBytes = kTileN * kBlockK;                 // 8192 per matrix
    static constexpr int kXBytes = TOK * kBlockK * 2;                // bf16
    static constexpr int kStageBytes = NW * kWBytes + kXBytes;
    static constexpr int kAColsPerStage = NW * (kBlockK / 2);        // 32-bit TMEM columns
    static constexpr int kDCols = NW * TOK;
    static constexpr int kABase = (kDCols + 31) / 32 * 32;
    static constexpr int kMaxStagesSmem = (200 * 1024) / kStageBytes;
    static constexpr int kMaxStagesTmem = (512 - kABase) / kAColsPerStage;
    static constexpr int kStagesRaw = kMaxStagesSmem < kMaxStagesTmem ? kMaxStagesSmem : kMaxStagesTmem;
    static constexpr int kStages = kStagesRaw > 12 ? 12 : kStagesRaw;
    static constexpr int kBarBytes = 1024;
    static constexpr int kSmemBytes = kStages * kStageBytes + kBarBytes + 1024;  // + align slack
    // one CTA per SM is required (the CTA allocates all 512 TMEM columns)
    static constexpr int kSmemRequest = kSmemBytes > 120 * 1024 ? kSmemBytes : 120 * 1024;
    static_assert(kStages >= 2, "pipeline needs at least two stages");
    static_assert(kABase + kStages * kAColsPerStage <= 512, "TMEM columns");
    static_assert(kSmemRequest <= 227 * 1024, "shared memory");
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

// Bounded wait.  Returns false if it gave up or another role already did.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, Ctl *ctl, DeviceStatus *st,
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
template <>
__device__ __forceinline__ void store_out<float>(float *p, float v) { *p = v; }
template <>
__device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float silu_f(float g) { return g / (1.0f + __expf(-g)); }

template <int TOK, int NW, typename YT>
__global__ void __launch_bounds__(kThreads, 1)
linear_i8_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_w2,
                         const __grid_constant__ CUtensorMap tmap_x, const float *__restrict__ scales,
                         const float *__restrict__ bias, const float *__restrict__ scales2,
                         const float *__restrict__ bias2, YT *__restrict__ y, int M, int N, int K, size_t ldy,
                         int epilogue, DeviceStatus *status) {
    using C = Cfg<TOK, NW>;
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment: required by the 128-byte swizzle with base_offset 0
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *bar_area = smem + C::kStages * C::kStageBytes;
    uint64_t *bars = reinterpret_cast<uint64_t *>(bar_area);
    // barrier indices: full[s]=s, aready[s]=S+s, empty[s]=2S+s, accfull=3S
    Ctl *ctl = reinterpret_cast<Ctl *>(bar_area + 512);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * kTileN;
    const int m0 = blockIdx.y * TOK;
    const int num_kb = (K + kBlockK - 1) / kBlockK;
    auto bar = [&](int i) { return smem_u32(bars + i); };
    auto stage_w = [&](int s, int w) { return smem + s * C::kStageBytes + w * C::kWBytes; };
    auto stage_x = [&](int s) { return smem + s * C::kStageBytes + NW * C::kWBytes; };

    if (threadIdx.x == 0) {
        ctl->abort_flag = 0;
        ctl->tmem_base = 0;
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(bar(s), 1);
            mbar_init(bar(C::kStages + s), 4);
            mbar_init(bar(2 * C::kStages + s), 1);
        }
        mbar_init(bar(3 * C::kStages), 1);
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
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            for (int kb = 0; kb < num_kb; ++kb) {
                const int s = kb % C::kStages;
                const uint32_t ph = (kb / C::kStages) & 1;
                if (!mbar_wait(bar(2 * C::kStages + s), ph ^ 1, ctl, status, 0, s)) break;
                mbar_expect_tx(bar(s), C::kStageBytes);
                tma_load_2d(smem_u32(stage_w(s, 0)), &tmap_w, kb * kBlockK, n0, bar(s));
                if constexpr (NW == 2) tma_load_2d(smem_u32(stage_w(s, 1)), &tmap_w2, kb * kBlockK, n0, bar(s));
                tma_load_2d(smem_u32(stage_x(s)), &tmap_x, kb * kBlockK, m0, bar(s));
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            // instruction descriptor: D=f32, A=bf16 (K-major, from TMEM), B=bf16 (K-major), M=128, N=TOK
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TOK >> 3) << 17) |
                                       ((uint32_t)(kTileN >> 4) << 24);
            bool ok = true;
            for (int kb = 0; kb < num_kb && ok; ++kb) {
                const int s = kb % C::kStages;
                const uint32_t ph = (kb / C::kStages) & 1;
                ok = mbar_wait(bar(s), ph, ctl, status, 1, s) &&
                     mbar_wait(bar(C::kStages + s), ph, ctl, status, 2, s);
                if (!ok) break;
                tc_fence_after();
                const uint64_t bdesc = make_b_desc(smem_u32(stage_x(s)));
#pragma unroll
                for (int w = 0; w < NW; ++w) {
#pragma unroll
                    for (int j = 0; j < kBlockK / kUmmaK; ++j) {
                        const uint32_t a_tmem = tmem_base + C::kABase + s * C::kAColsPerStage + w * (kBlockK / 2) + j * (kUmmaK / 2);
                        tc_mma_ts(tmem_base + w * TOK, a_tmem, bdesc + (uint64_t)((j * kUmmaK * 2) >> 4), idesc,
                                  (kb > 0 || j > 0) ? 1u : 0u);
                    }
                }
                tc_commit(bar(2 * C::kStages + s));  // frees smem stage s and TMEM A stage s
            }
            if (ok) tc_commit(bar(3 * C::kStages));  // accumulators complete
        }
    } else {
        // ---------------- converters, then epilogue ----------------
        const int quad = warp & 3;                 // TMEM lane quadrant this warp may access
        const int row = quad * 32 + lane;          // weight row inside the tile == TMEM lane
        const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
        bool ok = true;
        for (int kb = 0; kb < num_kb && ok; ++kb) {
            const int s = kb % C::kStages;
            const uint32_t ph = (kb / C::kStages) & 1;
            ok = mbar_wait(bar(s), ph, ctl, status, 3, s);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) break;
            tc_fence_after();
#pragma unroll
            for (int w = 0; w < NW; ++w) {
                // 64 codes of this row; TMA wrote them with the 64-byte swizzle: the 16-byte
                // chunk c of row r sits at chunk position c ^ ((r >> 1) & 3)
                const uint8_t *rowp = stage_w(s, w) + row * kBlockK;
                uint32_t packed[32];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const uint4 v = *reinterpret_cast<const uint4 *>(rowp + ((c ^ ((row >> 1) & 3)) << 4));
                    cvt_i8x4_bf16(v.x, packed[8 * c + 0], packed[8 * c + 1]);
                    cvt_i8x4_bf16(v.y, packed[8 * c + 2], packed[8 * c + 3]);
                    cvt_i8x4_bf16(v.z, packed[8 * c + 4], packed[8 * c + 5]);
                    cvt_i8x4_bf16(v.w, packed[8 * c + 6], packed[8 * c + 7]);
                }
                tc_st32(tmem_base + lane_addr + C::kABase + s * C::kAColsPerStage + w * (kBlockK / 2), packed);
            }
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(C::kStages + s));
        }
        // epilogue
        if (ok) ok = mbar_wait(bar(3 * C::kStages), 0, ctl, status, 4, 0);
        ok = __all_sync(0xFFFFFFFFu, ok);
        if (ok) {
            tc_fence_after();
            const int n = n0 + row;
            const bool n_ok = n < N;
            const float sc = n_ok ? scales[n] : 0.0f;
            const float bs = (n_ok && bias) ? bias[n] : 0.0f;
            float sc2 = 0.0f, bs2 = 0.0f;
            if constexpr (NW == 2) {
                sc2 = n_ok ? scales2[n] : 0.0f;
                bs2 = (n_ok && bias2) ? bias2[n] : 0.0f;
            }
#pragma unroll 1
            for (int c = 0; c < TOK / 16; ++c) {
                uint32_t r[16], r2[16];
                tc_ld16(tmem_base + lane_addr + c * 16, r);
                if constexpr (NW == 2) tc_ld16(tmem_base + lane_addr + TOK + c * 16, r2);
                tc_wait_ld();
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int m = m0 + c * 16 + i;
                    float o = __uint_as_float(r[i]) * sc + bs;
                    if constexpr (NW == 2) {
                        const float u = __uint_as_float(r2[i]) * sc2 + bs2;
                        o = silu_f(o) * u;
                    } else if (epilogue == SHREWQ_EPILOGUE_RELU) {
                        o = fmaxf(o, 0.0f);
                    }
                    if (n_ok && m < M) store_out<YT>(y + (size_t)m * ldy + n, o);
                }
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

template <int TOK, int NW, typename YT>
int launch_cfg(shrewq_ctx *ctx, const ForwardArgs &a, const CUtensorMap &tw, const CUtensorMap &tw2) {
    using C = Cfg<TOK, NW>;
    CUtensorMap tx;
    int rc = encode_2d(ctx, &tx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.x, a.K, a.M, kBlockK, TOK,
                       CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != SHREWQ_OK) return rc;
    auto kern = linear_i8_tcgen05_kernel<TOK, NW, YT>;
    static bool attr_set = false;  // per instantiation
    if (!attr_set) {
        SHREWQ_CUDA_TRY(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemRequest));
        attr_set = true;
    }
    dim3 grid((unsigned)((a.N + kTileN - 1) / kTileN), (unsigned)((a.M + TOK - 1) / TOK));
    kern<<<grid, kThreads, C::kSmemRequest, ctx->stream>>>(tw, tw2, tx, a.scales, a.bias, a.scales_up, a.bias_up,
                                                           static_cast<YT *>(a.y), (int)a.M, (int)a.N, (int)a.K,
                                                           a.ldy, a.epilogue, ctx->dev_status);
    ctx->launches += 1;
    SHREWQ_CUDA_TRY(ctx, cudaGetLastError());
    return SHREWQ_OK;
}

template <typename YT>
int launch_y(shrewq_ctx *ctx, const ForwardArgs &a, const CUtensorMap &tw, const CUtensorMap &tw2) {
    if (a.q_up) {
        if (a.M <= 16) return launch_cfg<16, 2, YT>(ctx, a, tw, tw2);
        if (a.M <= 32) return launch_cfg<32, 2, YT>(ctx, a, tw, tw2);
        if (a.M <= 64) return launch_cfg<64, 2, YT>(ctx, a, tw, tw2);
        return launch_cfg<128, 2, YT>(ctx, a, tw, tw2);
    }
    if (a.M <= 16) return launch_cfg<16, 1, YT>(ctx, a, tw, tw2);
    if (a.M <= 32) return launch_cfg<32, 1, YT>(ctx, a, tw, tw2);
    if (a.M <= 64) return launch_cfg<64, 1, YT>(ctx, a, tw, tw2);
    if (a.M <= 128) return launch_cfg<128, 1, YT>(ctx, a, tw, tw2);
    return launch_cfg<256, 1, YT>(ctx, a, tw, tw2);
}

}  // namespace

bool tcgen05_supported(const ForwardArgs &a) {
    return a.x_dtype == SHREWQ_BF16 && a.K >= 16 && (a.K % 16) == 0 && a.M >= 1 && a.N >= 1 &&
           (reinterpret_cast<uintptr_t>(a.x) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.q) & 15) == 0 &&
           (!a.q_up || (reinterpret_cast<uintptr_t>(a.q_up) & 15) == 0) && a.K < (1u << 31) && a.N < (1u << 31) &&
           a.M < (1u << 31) && (a.M + 15) / 16 <= 65535 * 16;
}

int encode_weight_tmap(shrewq_ctx *ctx, const int8_t *q, size_t n, size_t k, void *tmap_out) {
    return encode_2d(ctx, static_cast<CUtensorMap *>(tmap_out), CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, q, k, n, kBlockK,
                     kTileN, CU_TENSOR_MAP_SWIZZLE_64B);
}

int launch_gemm_tcgen05(shrewq_ctx *ctx, const ForwardArgs &a, const void *w_tmap, const void *w_up_tmap) {
    const CUtensorMap &tw = *static_cast<const CUtensorMap *>(w_tmap);
    const CUtensorMap &tw2 = *static_cast<const CUtensorMap *>(w_up_tmap ? w_up_tmap : w_tmap);
    if (a.y_dtype == SHREWQ_BF16) return launch_y<__nv_bfloat16>(ctx, a, tw, tw2);
    return launch_y<float>(ctx, a, tw, tw2);
}

}  // namespace shrewq
