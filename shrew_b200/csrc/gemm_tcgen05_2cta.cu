// Host side of the CTA-pair forward (device code and its description: gemm_tcgen05_2cta_kernels.cuh).
#include <cuda.h>

#include <atomic>
#include <cstdlib>

#include "common.cuh"
#include "gemm_tcgen05_2cta_kernels.cuh"

namespace shrewq {
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int encode_x_half(shrewq_ctx *ctx, CUtensorMap *out, const void *x, size_t K, size_t M) {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess)
            return set_err(ctx, SHREWQ_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
        fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {(cuuint32_t)kBlockK, (cuuint32_t)kTokHalf};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(x), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_err(ctx, SHREWQ_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return SHREWQ_OK;
}

template <typename YT, bool GATED>
int launch_pair(shrewq_ctx *ctx, const ForwardArgs &a, const CUtensorMap &tw, const CUtensorMap &tw2) {
    CUtensorMap tx;
    int rc = encode_x_half(ctx, &tx, a.x, a.K, a.M);
    if (rc != SHREWQ_OK) return rc;
    auto kern = linear_i8_tcgen05_pair_kernel<YT, GATED>;
    static std::atomic<unsigned long long> attr_done{0};  // per instantiation: bit d = device d has the attribute
    if (ctx->device < 0 || ctx->device >= 64 || !((attr_done.load(std::memory_order_acquire) >> ctx->device) & 1ull)) {
        SHREWQ_CUDA_TRY(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
        if (ctx->device >= 0 && ctx->device < 64) attr_done.fetch_or(1ull << ctx->device, std::memory_order_release);
    }
    constexpr int kChanPair = GATED ? kLanes : 2 * kLanes;  // output channels per CTA pair
    const unsigned pairs = (unsigned)((a.N + kChanPair - 1) / kChanPair);
    const unsigned m_tiles = (unsigned)((a.M + kTokPair - 1) / kTokPair);
    // split-K when the CTA grid leaves SMs idle: as many splits as fit in one wave, >= 8 rounds each
    const int rounds = (int)((a.K + kBlockK * kSub - 1) / (kBlockK * kSub));
    const long ctas = 2L * pairs * m_tiles;
    int splits = 1;
    if (ctas <= 1024) {
        int want = (int)(ctx->sm_count / ctas);
        if (want > rounds / 8) want = rounds / 8;
        if (want > 1) splits = want;
    }
    const int rps = (rounds + splits - 1) / splits;
    splits = (rounds + rps - 1) / rps;  // no empty split
    SplitK2 sk{nullptr, nullptr, rps, 0, 0};
    Operands ops{a.scales, a.bias, a.scales_up, a.bias_up};
    // Option tc_tailsplit (as for the single-CTA kernel): when the pair tiles leave a short last wave, the
    // full waves go out as one launch of whole-K tiles and the tiles of the last wave as a second launch
    // split along K, so that it fills the SMs too.
    // By default (0) the tail goes out split when it is at most a quarter of a wave: measured on the MLP block at
    // batch 512, a tail of 12 of 74 pair tiles (the 2-GPU shard) 57.6 -> 53.4 us, a tail of 24 (one GPU) no gain.
    // 1 = whenever a tail exists, 2 = never.
    if (ctx->tuning.tc_tailsplit != 2 && splits == 1) {
        const int per_wave = ctx->sm_count / 2;  // pair tiles resident at once, one CTA per SM
        const int tiles = (int)(pairs * m_tiles), rem = per_wave > 0 ? tiles % per_wave : 0;
        int s_tail = rem > 0 ? per_wave / rem : 0;
        if (s_tail > 4) s_tail = 4;
        if (s_tail > rounds / 8) s_tail = rounds / 8;
        const bool wanted = ctx->tuning.tc_tailsplit == 1 || rem * 4 <= per_wave;
        if (wanted && tiles > per_wave && rem > 0 && s_tail >= 2) {
            const int rps_t = (rounds + s_tail - 1) / s_tail;
            const int splits_t = (rounds + rps_t - 1) / rps_t;
            const size_t part_bytes = (size_t)2 * rem * splits_t * kTokPair * kLanes * sizeof(float);
            if ((rc = ensure_scratch(ctx, 8192 + part_bytes)) != SHREWQ_OK) return rc;
            if (!ctx->counters_zeroed) {
                SHREWQ_CUDA_TRY(ctx, cudaMemsetAsync(static_cast<char *>(ctx->scratch) + 4096, 0, 4096, ctx->stream));
                ctx->counters_zeroed = true;
            }
            SplitK2 head{nullptr, nullptr, rounds, 0, (int)pairs};
            SHREWQ_CUDA_TRY(ctx, launch_maybe_pdl(kern, dim3(2u * (unsigned)(tiles - rem), 1, 1), dim3(kThreads), (size_t)kSmemBytes,
                                                  ctx->stream, a.pdl, tw, tw2, tx, ops, static_cast<YT *>(a.y), a.extra, (int)a.M,
                                                  (int)a.N, (int)a.K, a.ldy, a.epilogue, head, ctx->dev_status));
            SplitK2 tail{reinterpret_cast<float *>(static_cast<char *>(ctx->scratch) + 8192),
                         reinterpret_cast<unsigned int *>(static_cast<char *>(ctx->scratch) + 4096), rps_t, tiles - rem,
                         (int)pairs};
            // (the tail launch may start under the head launch's last wave: the two write disjoint tiles)
            SHREWQ_CUDA_TRY(ctx, launch_maybe_pdl(kern, dim3(2u * (unsigned)rem, 1, (unsigned)splits_t), dim3(kThreads),
                                                  (size_t)kSmemBytes, ctx->stream, a.pdl, tw, tw2, tx, ops, static_cast<YT *>(a.y),
                                                  a.extra, (int)a.M, (int)a.N, (int)a.K, a.ldy, a.epilogue, tail, ctx->dev_status));
            ctx->launches += 2;
            SHREWQ_CUDA_TRY(ctx, cudaGetLastError());
            return SHREWQ_OK;
        }
    }
    if (splits > 1) {
        // context scratch as in the single-CTA launcher: tile counters at 4096, partial sums from 8192
        const size_t part_bytes = (size_t)ctas * splits * kTokPair * kLanes * sizeof(float);
        if ((rc = ensure_scratch(ctx, 8192 + part_bytes)) != SHREWQ_OK) return rc;
        if (!ctx->counters_zeroed) {
            SHREWQ_CUDA_TRY(ctx, cudaMemsetAsync(static_cast<char *>(ctx->scratch) + 4096, 0, 4096, ctx->stream));
            ctx->counters_zeroed = true;
        }
        sk.counters = reinterpret_cast<unsigned int *>(static_cast<char *>(ctx->scratch) + 4096);
        sk.partials = reinterpret_cast<float *>(static_cast<char *>(ctx->scratch) + 8192);
    }
    dim3 grid(2 * pairs, m_tiles, (unsigned)splits);
    SHREWQ_CUDA_TRY(ctx, launch_maybe_pdl(kern, grid, dim3(kThreads), (size_t)kSmemBytes, ctx->stream, a.pdl, tw, tw2, tx, ops,
                                          static_cast<YT *>(a.y), a.extra, (int)a.M, (int)a.N, (int)a.K, a.ldy, a.epilogue, sk,
                                          ctx->dev_status));
    ctx->launches += 1;
    SHREWQ_CUDA_TRY(ctx, cudaGetLastError());
    return SHREWQ_OK;
}

}  // namespace

#ifdef SHREWQ_TRACE
extern "C" __attribute__((visibility("default"))) int shrewq_debug_set_trace_pair(long long *dev_buf) {
    return (int)cudaMemcpyToSymbol(g_trace_pair, &dev_buf, sizeof(dev_buf));
}
#endif

// Plain forward: w_tmap = the handle's 128-row INT8 boxes, w_up_tmap = nullptr.  Gate/up pair: the
// 64-row boxes of the gate and of the up handle (the descriptors the single-CTA kernel uses).
int launch_gemm_tcgen05_2cta(shrewq_ctx *ctx, const ForwardArgs &a, const void *w_tmap, const void *w_up_tmap) {
    const CUtensorMap &tw = *static_cast<const CUtensorMap *>(w_tmap);
    if (a.q_up) {
        if (!w_up_tmap) return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "tcgen05-2cta: the up matrix has no tensor map");
        const CUtensorMap &tw2 = *static_cast<const CUtensorMap *>(w_up_tmap);
        if (a.y_dtype == SHREWQ_BF16) return launch_pair<__nv_bfloat16, true>(ctx, a, tw, tw2);
        return launch_pair<float, true>(ctx, a, tw, tw2);
    }
    if (a.y_dtype == SHREWQ_BF16) return launch_pair<__nv_bfloat16, false>(ctx, a, tw, tw);
    return launch_pair<float, false>(ctx, a, tw, tw);
}

}  // namespace shrewq
