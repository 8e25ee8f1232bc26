// Launchers of the CUDA-core GEMV (device code and its description: gemv_kernels.cuh).
#include <cstdlib>

#include <atomic>

#include "common.cuh"
#include "gemv_kernels.cuh"
#include "gemv_ring_kernels.cuh"

namespace shrewq {
namespace {

template <int MT, int R, typename XT, typename YT, bool GATED>
void launch_one(shrewq_ctx *ctx, const ForwardArgs &a) {
    constexpr int NR = GATED ? R / 2 : R;
    const unsigned gx = (unsigned)((a.N + NR - 1) / NR);
    if (a.M > (size_t)MT) {
        // batches above MT tokens run as slices of MT tokens along grid.y (small layers with f32 activations: the
        // weights come from L2 for every slice but the first)
        gemv_i8_kernel<MT, R, XT, YT, GATED, false, true><<<dim3(gx, (unsigned)((a.M + MT - 1) / MT)), kThreads, 0, ctx->stream>>>(
            a.q, a.scales, a.bias, a.q_up, a.scales_up, a.bias_up, static_cast<const XT *>(a.x), static_cast<YT *>(a.y), a.extra,
            (int)a.M, (int)a.N, (int)a.K, a.ldy, a.epilogue);
        return;
    }
    // With a.pdl (and one or two tokens: from four tokens on the early weight fetch costs more registers than the
    // overlap returns) the launch takes the PDL variant of the kernel with programmatic stream serialization:
    // back-to-back GEMVs overlap launch latency, prologue and the first weight loads with the tail of the kernel before.
    if (a.pdl && MT <= 2) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(gx);
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = 0;
        cfg.stream = ctx->stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        cudaLaunchKernelEx(&cfg, gemv_i8_kernel<MT, R, XT, YT, GATED, true>, a.q, a.scales, a.bias, a.q_up, a.scales_up,
                           a.bias_up, static_cast<const XT *>(a.x), static_cast<YT *>(a.y), a.extra, (int)a.M, (int)a.N,
                           (int)a.K, a.ldy, a.epilogue);
        return;
    }
    gemv_i8_kernel<MT, R, XT, YT, GATED><<<gx, kThreads, 0, ctx->stream>>>(
        a.q, a.scales, a.bias, a.q_up, a.scales_up, a.bias_up, static_cast<const XT *>(a.x),
        static_cast<YT *>(a.y), a.extra, (int)a.M, (int)a.N, (int)a.K, a.ldy, a.epilogue);
}

template <typename XT, typename YT, bool GATED>
void dispatch_m(shrewq_ctx *ctx, const ForwardArgs &a) {
    if (a.M <= 1) launch_one<1, 4, XT, YT, GATED>(ctx, a);
    else if (a.M <= 2) launch_one<2, 4, XT, YT, GATED>(ctx, a);
    else if (a.M <= 4) launch_one<4, 4, XT, YT, GATED>(ctx, a);
    else if (a.M <= 8) launch_one<8, 2, XT, YT, GATED>(ctx, a);
    else launch_one<16, 2, XT, YT, GATED>(ctx, a);
}

// ---- the ring kernel (1..32 tokens, bf16 activations): bulk copies into a shared-memory ring + warp MMA ----
template <int NT, typename YT, bool GATED, int STAGES>
int launch_ring_stages(shrewq_ctx *ctx, const ForwardArgs &a) {
    constexpr int NCH = GATED ? kRingRows / 2 : kRingRows;
    constexpr size_t kSmem = RingCfg<kRingKC, STAGES>::kSmemBytes;
    auto kern = gemv_i8_ring_kernel<NT, kRingKC, kRingConsumers, YT, GATED, STAGES>;
    static std::atomic<unsigned long long> attr_done{0};  // per instantiation: bit d = device d has the attribute
    const int d = ctx->device;
    if (d < 0 || d >= 64 || !((attr_done.load(std::memory_order_acquire) >> d) & 1ull)) {
        SHREWQ_CUDA_TRY(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem));
        if (d >= 0 && d < 64) attr_done.fetch_or(1ull << d, std::memory_order_release);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((a.N + NCH - 1) / NCH));
    cfg.blockDim = dim3((kRingConsumers + 1) * 32);
    cfg.dynamicSmemBytes = kSmem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = a.pdl ? 1 : 0;
    SHREWQ_CUDA_TRY(ctx, cudaLaunchKernelEx(&cfg, kern, a.q, a.scales, a.bias, a.q_up, a.scales_up, a.bias_up,
                                            static_cast<const uint16_t *>(a.x), static_cast<YT *>(a.y), a.extra, (int)a.M,
                                            (int)a.N, (int)a.K, a.ldy, a.epilogue, ctx->dev_status));
    return SHREWQ_OK;
}

// three stages (two CTAs per SM) while all CTAs are resident at once, two stages (three CTAs per SM) for larger grids
template <int NT, typename YT, bool GATED>
int launch_ring_one(shrewq_ctx *ctx, const ForwardArgs &a) {
    constexpr int NCH = GATED ? kRingRows / 2 : kRingRows;
    const size_t ctas = (a.N + NCH - 1) / NCH;
    const int stages = ctx->tuning.ring_stages == 2 || ctx->tuning.ring_stages == 3 ? ctx->tuning.ring_stages
                                                                                     : (ctas <= (size_t)2 * ctx->sm_count ? 3 : 2);
    if (stages == 2) return launch_ring_stages<NT, YT, GATED, 2>(ctx, a);
    return launch_ring_stages<NT, YT, GATED, 3>(ctx, a);
}

template <typename YT, bool GATED>
int launch_ring_m(shrewq_ctx *ctx, const ForwardArgs &a) {
    if (a.M <= 8) return launch_ring_one<1, YT, GATED>(ctx, a);
    if (a.M <= 16) return launch_ring_one<2, YT, GATED>(ctx, a);
    return launch_ring_one<4, YT, GATED>(ctx, a);
}

}  // namespace

int launch_gemv(shrewq_ctx *ctx, const ForwardArgs &a) {
    if (a.M == 0 || a.N == 0) return SHREWQ_OK;
    if (a.M > 128 || (a.K % 16) != 0 || a.K == 0 || a.N > 0x7FFFFFFF || a.K > 0x7FFFFFFF)
        return set_err(ctx, SHREWQ_ERR_UNSUPPORTED, "gemv: needs M<=128 and K a positive multiple of 16");
    const bool gated = a.q_up != nullptr;
    const bool xb = a.x_dtype == SHREWQ_BF16, yb = a.y_dtype == SHREWQ_BF16;
#define SHREWQ_GEMV_CASE(XT, YT)                       \
    do {                                               \
        if (gated) dispatch_m<XT, YT, true>(ctx, a);   \
        else dispatch_m<XT, YT, false>(ctx, a);        \
    } while (0)
    if (xb && yb) SHREWQ_GEMV_CASE(__nv_bfloat16, __nv_bfloat16);
    else if (xb && !yb) SHREWQ_GEMV_CASE(__nv_bfloat16, float);
    else if (!xb && !yb) SHREWQ_GEMV_CASE(float, float);
    else SHREWQ_GEMV_CASE(float, __nv_bfloat16);
#undef SHREWQ_GEMV_CASE
    ctx->launches += 1;
    SHREWQ_CUDA_TRY(ctx, cudaGetLastError());
    return SHREWQ_OK;
}

bool gemv_ring_supported(const ForwardArgs &a) {
    return a.x_dtype == SHREWQ_BF16 && a.M >= 1 && a.M <= 32 && a.K >= 64 && (a.K % 64) == 0 &&
           (reinterpret_cast<uintptr_t>(a.x) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.q) & 15) == 0 &&
           (!a.q_up || (reinterpret_cast<uintptr_t>(a.q_up) & 15) == 0) && a.N <= 0x7FFFFFFF && a.K <= 0x7FFFFFFF;
}

int launch_gemv_ring(shrewq_ctx *ctx, const ForwardArgs &a) {
    if (a.M == 0 || a.N == 0) return SHREWQ_OK;
    if (!gemv_ring_supported(a))
        return set_err(ctx, SHREWQ_ERR_UNSUPPORTED, "ring gemv: needs bf16 activations, M <= 32, K a multiple of 64, 16-byte alignment");
    const bool gated = a.q_up != nullptr;
    int rc;
    if (a.y_dtype == SHREWQ_BF16) rc = gated ? launch_ring_m<__nv_bfloat16, true>(ctx, a) : launch_ring_m<__nv_bfloat16, false>(ctx, a);
    else rc = gated ? launch_ring_m<float, true>(ctx, a) : launch_ring_m<float, false>(ctx, a);
    if (rc != SHREWQ_OK) return rc;
    ctx->launches += 1;
    SHREWQ_CUDA_TRY(ctx, cudaGetLastError());
    return SHREWQ_OK;
}

}  // namespace shrewq
