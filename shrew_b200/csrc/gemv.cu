// Launchers of the CUDA-core GEMV (device code and its description: gemv_kernels.cuh).
#include <cstdlib>

#include "common.cuh"
#include "gemv_kernels.cuh"

namespace shrewq {
namespace {

template <int MT, int R, typename XT, typename YT, bool GATED>
void launch_one(shrewq_ctx *ctx, const ForwardArgs &a) {
    constexpr int NR = GATED ? R / 2 : R;
    const unsigned grid = (unsigned)((a.N + NR - 1) / NR);
    // Option gemv_pdl launches the PDL variant of the kernel with programmatic stream
    // serialization: back-to-back GEMVs overlap launch latency, prologue and the first weight
    // loads with the tail of the kernel before.
    const bool pdl = ctx->tuning.gemv_pdl != 0;
    if (pdl) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(grid);
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
    gemv_i8_kernel<MT, R, XT, YT, GATED><<<grid, kThreads, 0, ctx->stream>>>(
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

}  // namespace

int launch_gemv(shrewq_ctx *ctx, const ForwardArgs &a) {
    if (a.M == 0 || a.N == 0) return SHREWQ_OK;
    if (a.M > 16 || (a.K % 16) != 0 || a.K == 0 || a.N > 0x7FFFFFFF || a.K > 0x7FFFFFFF)
        return set_err(ctx, SHREWQ_ERR_UNSUPPORTED, "gemv: needs M<=16 and K a positive multiple of 16");
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

}  // namespace shrewq
