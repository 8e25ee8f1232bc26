// Launchers of the general f32 forward kernel (device code and its description: gemm_simt_kernels.cuh).
#include "common.cuh"
#include "gemm_simt_kernels.cuh"

namespace shrewq {
namespace {

template <typename XT, typename YT>
void launch_t(shrewq_ctx *ctx, const ForwardArgs &a) {
    dim3 grid((unsigned)((a.N + BN - 1) / BN), (unsigned)((a.M + BM - 1) / BM));
    if (a.q_up)
        gemm_i8_simt_kernel<XT, YT, true><<<grid, 256, 0, ctx->stream>>>(
            a.q, a.scales, a.bias, a.q_up, a.scales_up, a.bias_up, static_cast<const XT *>(a.x),
            static_cast<YT *>(a.y), a.M, a.N, a.K, a.ldy, a.epilogue);
    else
        gemm_i8_simt_kernel<XT, YT, false><<<grid, 256, 0, ctx->stream>>>(
            a.q, a.scales, a.bias, nullptr, nullptr, nullptr, static_cast<const XT *>(a.x),
            static_cast<YT *>(a.y), a.M, a.N, a.K, a.ldy, a.epilogue);
}

}  // namespace

int launch_gemm_simt(shrewq_ctx *ctx, const ForwardArgs &a) {
    if (a.M == 0 || a.N == 0) return SHREWQ_OK;
    if ((a.M + BM - 1) / BM > 65535) return set_err(ctx, SHREWQ_ERR_UNSUPPORTED, "simt gemm: M too large");
    const bool xb = a.x_dtype == SHREWQ_BF16, yb = a.y_dtype == SHREWQ_BF16;
    if (xb && yb) launch_t<__nv_bfloat16, __nv_bfloat16>(ctx, a);
    else if (xb && !yb) launch_t<__nv_bfloat16, float>(ctx, a);
    else if (!xb && !yb) launch_t<float, float>(ctx, a);
    else launch_t<float, __nv_bfloat16>(ctx, a);
    ctx->launches += 1;
    SHREWQ_CUDA_TRY(ctx, cudaGetLastError());
    return SHREWQ_OK;
}

}  // namespace shrewq
