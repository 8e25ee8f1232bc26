// Launchers of the warp-MMA small-batch forward (device code and its description:
// gemv_mma_kernels.cuh).
#include <cstdlib>

#include "common.cuh"
#include "gemv_mma_kernels.cuh"

namespace shrewq {
namespace {

template <int MT16, typename YT, bool GATED, bool F16>
void launch_one(shrewq_ctx *ctx, const ForwardArgs &a, const void *x, const int *xshift) {
    constexpr int kChan = GATED ? 8 : 8 * NB;
    const unsigned grid = (unsigned)((a.N + kChan - 1) / kChan);
    gemv_mma_kernel<MT16, YT, GATED, F16, false><<<grid, kThreads, 0, ctx->stream>>>(
        a.q, a.scales, a.bias, a.q_up, a.scales_up, a.bias_up, static_cast<const uint16_t *>(x), xshift,
        static_cast<YT *>(a.y), a.extra, (int)a.M, (int)a.N, (int)a.K, a.ldy, a.epilogue);
}

template <typename YT, bool GATED, bool F16>
void dispatch_m(shrewq_ctx *ctx, const ForwardArgs &a, const void *x, const int *xshift) {
    if (a.M <= 16) launch_one<1, YT, GATED, F16>(ctx, a, x, xshift);
    else if (a.M <= 32) launch_one<2, YT, GATED, F16>(ctx, a, x, xshift);
    else launch_one<4, YT, GATED, F16>(ctx, a, x, xshift);
}

template <bool F16>
void dispatch_y(shrewq_ctx *ctx, const ForwardArgs &a, const void *x, const int *xshift) {
    const bool gated = a.q_up != nullptr;
    if (a.y_dtype == SHREWQ_BF16) {
        if (gated) dispatch_m<__nv_bfloat16, true, F16>(ctx, a, x, xshift);
        else dispatch_m<__nv_bfloat16, false, F16>(ctx, a, x, xshift);
    } else {
        if (gated) dispatch_m<float, true, F16>(ctx, a, x, xshift);
        else dispatch_m<float, false, F16>(ctx, a, x, xshift);
    }
}

// packed INT4 weights (f16 operands only): batch 1..4 staged in the kernel, else the staging kernel
// with the permuted store
template <int MT16, typename YT, bool GATED, bool XS>
void launch_w4(shrewq_ctx *ctx, const ForwardArgs &a, const void *x, const int *xshift, size_t smem) {
    constexpr int kChan = GATED ? 8 : 8 * NB;
    const unsigned grid = (unsigned)((a.N + kChan - 1) / kChan);
    gemv_mma_kernel<MT16, YT, GATED, true, XS, true><<<grid, kThreads, smem, ctx->stream>>>(
        a.q, a.scales, a.bias, a.q_up, a.scales_up, a.bias_up, static_cast<const uint16_t *>(x), xshift,
        static_cast<YT *>(a.y), a.extra, (int)a.M, (int)a.N, (int)a.K, a.ldy, a.epilogue);
}

template <typename YT, bool GATED>
int forward_w4(shrewq_ctx *ctx, const ForwardArgs &a) {
    if (a.M <= (size_t)kStageMaxTokens && a.M * a.K * sizeof(uint16_t) <= (size_t)kStageMaxBytes) {
        launch_w4<1, YT, GATED, true>(ctx, a, a.x, nullptr, a.M * a.K * sizeof(uint16_t));
        ctx->launches += 1;
        return SHREWQ_OK;
    }
    const size_t xbytes = a.M * a.K * sizeof(__half);
    int rc = ensure_xsplit(ctx, xbytes + a.M * sizeof(int));
    if (rc != SHREWQ_OK) return rc;
    __half *x16 = static_cast<__half *>(ctx->xsplit);
    int *xshift = reinterpret_cast<int *>(static_cast<char *>(ctx->xsplit) + xbytes);
    x_to_f16_kernel<<<(unsigned)a.M, 256, 0, ctx->stream>>>(static_cast<const __nv_bfloat16 *>(a.x), x16, xshift, (int)a.K, 1);
    if (a.M <= 16) launch_w4<1, YT, GATED, false>(ctx, a, x16, xshift, 0);
    else launch_w4<2, YT, GATED, false>(ctx, a, x16, xshift, 0);
    ctx->launches += 2;
    return SHREWQ_OK;
}

}  // namespace

// q / q_up of `a` point at packed INT4 rows (K/2 bytes each)
bool gemv_mma_w4_supported(const ForwardArgs &a) {
    return a.x_dtype == SHREWQ_BF16 && a.M >= 1 && a.M <= 32 && a.K >= 128 && (a.K % 128) == 0 &&
           (reinterpret_cast<uintptr_t>(a.x) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.q) & 15) == 0 &&
           (!a.q_up || (reinterpret_cast<uintptr_t>(a.q_up) & 15) == 0) && a.N <= 0x7FFFFFFF && a.K <= 0x7FFFFFFF;
}

int launch_gemv_mma_w4(shrewq_ctx *ctx, const ForwardArgs &a) {
    if (a.M == 0 || a.N == 0) return SHREWQ_OK;
    if (!gemv_mma_w4_supported(a))
        return set_err(ctx, SHREWQ_ERR_UNSUPPORTED,
                       "packed INT4 forward: needs bf16 activations, M <= 32, K a multiple of 128, 16-byte alignment");
    const bool gated = a.q_up != nullptr;
    int rc;
    if (a.y_dtype == SHREWQ_BF16) rc = gated ? forward_w4<__nv_bfloat16, true>(ctx, a) : forward_w4<__nv_bfloat16, false>(ctx, a);
    else rc = gated ? forward_w4<float, true>(ctx, a) : forward_w4<float, false>(ctx, a);
    if (rc != SHREWQ_OK) return rc;
    SHREWQ_CUDA_TRY(ctx, cudaGetLastError());
    return SHREWQ_OK;
}

bool gemv_mma_supported(const ForwardArgs &a) {
    return a.x_dtype == SHREWQ_BF16 && a.M >= 1 && a.M <= 64 && a.K >= 64 && (a.K % 64) == 0 &&
           (reinterpret_cast<uintptr_t>(a.x) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.q) & 15) == 0 &&
           (!a.q_up || (reinterpret_cast<uintptr_t>(a.q_up) & 15) == 0) && a.N <= 0x7FFFFFFF && a.K <= 0x7FFFFFFF;
}

int launch_gemv_mma(shrewq_ctx *ctx, const ForwardArgs &a) {
    if (a.M == 0 || a.N == 0) return SHREWQ_OK;
    if (!gemv_mma_supported(a))
        return set_err(ctx, SHREWQ_ERR_UNSUPPORTED, "mma gemv: needs bf16 activations, M<=64, K a multiple of 64, 16-byte alignment");
    dispatch_y<false>(ctx, a, a.x, nullptr);
    ctx->launches += 1;
    SHREWQ_CUDA_TRY(ctx, cudaGetLastError());
    return SHREWQ_OK;
}

}  // namespace shrewq
