// CPU run of the warp-MMA small-batch forward (shrew_b200/csrc/gemv_mma_kernels.cuh) under the CUDA
// stand-in, mma.sync emulated from its documented fragment layout.  The choice of kernel variant
// mirrors launch_gemv_mma in shrew_b200/csrc/gemv_mma.cu.  TEST INFRASTRUCTURE ONLY; see cuda_shim.h.
#include "cuda_shim.h"
#include "../../shrew_b200/csrc/gemv_mma_kernels.cuh"

using namespace shrewq;

namespace {
struct Args {
    const int8_t *q, *q_up;
    const float *scales, *bias, *scales_up, *bias_up;
    const void *x;
    void *y;
    int M, N, K;
    size_t ldy;
    int epilogue;
};

template <int MT16, typename YT, bool GATED, bool F16>
void run_one(const Args &a, const void *x, const int *xshift) {
    constexpr int kChan = GATED ? 8 : 8 * NB;
    const unsigned grid = (unsigned)((a.N + kChan - 1) / kChan);
    Dests none{};
    emu::launch(grid, kThreads, [&] {
        gemv_mma_kernel<MT16, YT, GATED, F16, false>(a.q, a.scales, a.bias, a.q_up, a.scales_up, a.bias_up,
                                                     static_cast<const uint16_t *>(x), xshift, static_cast<YT *>(a.y), none,
                                                     a.M, a.N, a.K, a.ldy, a.epilogue);
    });
}

template <typename YT, bool GATED>
void run_staged(const Args &a) {
    constexpr int kChan = GATED ? 8 : 8 * NB;
    const unsigned grid = (unsigned)((a.N + kChan - 1) / kChan);
    Dests none{};
    emu::launch(grid, kThreads, (size_t)a.M * a.K * sizeof(uint16_t), [&] {
        gemv_mma_kernel<1, YT, GATED, true, true>(a.q, a.scales, a.bias, a.q_up, a.scales_up, a.bias_up,
                                                  static_cast<const uint16_t *>(a.x), nullptr, static_cast<YT *>(a.y), none, a.M,
                                                  a.N, a.K, a.ldy, a.epilogue);
    });
}

template <typename YT, bool GATED, bool F16>
void run_m(const Args &a, const void *x, const int *xshift) {
    if (a.M <= 16) run_one<1, YT, GATED, F16>(a, x, xshift);
    else if (a.M <= 32) run_one<2, YT, GATED, F16>(a, x, xshift);
    else run_one<4, YT, GATED, F16>(a, x, xshift);
}

template <typename YT>
int run_y(const Args &a, int f16, int *staged_out) {
    const bool gated = a.q_up != nullptr;
    *staged_out = 0;
    if (f16 && a.M <= kStageMaxTokens && (size_t)a.M * a.K * sizeof(uint16_t) <= (size_t)kStageMaxBytes) {
        *staged_out = 1;
        if (gated) run_staged<YT, true>(a); else run_staged<YT, false>(a);
    } else if (f16) {
        std::vector<uint16_t> x16((size_t)a.M * a.K);
        std::vector<int> shift(a.M);
        emu::launch((unsigned)a.M, 256, [&] {
            x_to_f16_kernel(static_cast<const __nv_bfloat16 *>(a.x), reinterpret_cast<__half *>(x16.data()), shift.data(), a.K);
        });
        if (gated) run_m<YT, true, true>(a, x16.data(), shift.data()); else run_m<YT, false, true>(a, x16.data(), shift.data());
    } else {
        if (gated) run_m<YT, true, false>(a, a.x, nullptr); else run_m<YT, false, false>(a, a.x, nullptr);
    }
    return 0;
}
}  // namespace

// x: bf16 bits [M,K]; y: f32 or bf16 bits [M, ldy]; q_up == NULL: plain forward, else silu(gate)*up.
// Returns 0, or -1 for shapes gemv_mma_supported refuses.  *staged = 1 when x was staged inside the kernel.
extern "C" int emu_gemv_mma(const int8_t *q, const float *scales, const float *bias, const int8_t *q_up, const float *scales_up,
                            const float *bias_up, const void *x, void *y, int M, int N, int K, size_t ldy, int epilogue,
                            int f16, int y_bf16, int *staged) {
    if (M < 1 || M > 64 || K < 64 || (K % 64) != 0 || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(q) & 15) ||
        (q_up && (reinterpret_cast<uintptr_t>(q_up) & 15)))
        return -1;
    const Args a{q, q_up, scales, bias, scales_up, bias_up, x, y, M, N, K, ldy, epilogue};
    return y_bf16 ? run_y<__nv_bfloat16>(a, f16, staged) : run_y<float>(a, f16, staged);
}

namespace {
template <int MT16, typename YT, bool GATED, bool XS>
void run_w4(const Args &a, const void *x, const int *xshift, size_t smem) {
    constexpr int kChan = GATED ? 8 : 8 * NB;
    const unsigned grid = (unsigned)((a.N + kChan - 1) / kChan);
    Dests none{};
    emu::launch(grid, kThreads, smem, [&] {
        gemv_mma_kernel<MT16, YT, GATED, true, XS, true>(a.q, a.scales, a.bias, a.q_up, a.scales_up, a.bias_up,
                                                         static_cast<const uint16_t *>(x), xshift, static_cast<YT *>(a.y), none,
                                                         a.M, a.N, a.K, a.ldy, a.epilogue);
    });
}

template <typename YT, bool GATED>
int forward_w4(const Args &a, int *staged_out) {
    *staged_out = 0;
    if (a.M <= kStageMaxTokens && (size_t)a.M * a.K * sizeof(uint16_t) <= (size_t)kStageMaxBytes) {
        *staged_out = 1;
        run_w4<1, YT, GATED, true>(a, a.x, nullptr, (size_t)a.M * a.K * sizeof(uint16_t));
        return 0;
    }
    std::vector<uint16_t> x16((size_t)a.M * a.K);
    std::vector<int> shift(a.M);
    emu::launch((unsigned)a.M, 256, [&] {
        x_to_f16_kernel(static_cast<const __nv_bfloat16 *>(a.x), reinterpret_cast<__half *>(x16.data()), shift.data(), a.K, 1);
    });
    if (a.M <= 16) run_w4<1, YT, GATED, false>(a, x16.data(), shift.data(), 0);
    else run_w4<2, YT, GATED, false>(a, x16.data(), shift.data(), 0);
    return 0;
}
}  // namespace

// packed INT4 weights: q / q_up are [N][K/2] bytes (code 2j + 8 in the low, code 2j+1 + 8 in the high nibble)
extern "C" int emu_gemv_mma_w4(const uint8_t *q, const float *scales, const float *bias, const uint8_t *q_up,
                               const float *scales_up, const float *bias_up, const void *x, void *y, int M, int N, int K,
                               size_t ldy, int epilogue, int y_bf16, int *staged) {
    if (M < 1 || M > 32 || K < 128 || (K % 128) != 0 || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(q) & 15) ||
        (q_up && (reinterpret_cast<uintptr_t>(q_up) & 15)))
        return -1;
    const Args a{reinterpret_cast<const int8_t *>(q), reinterpret_cast<const int8_t *>(q_up), scales, bias, scales_up, bias_up, x, y,
                 M, N, K, ldy, epilogue};
    const bool gated = q_up != nullptr;
    if (y_bf16) return gated ? forward_w4<__nv_bfloat16, true>(a, staged) : forward_w4<__nv_bfloat16, false>(a, staged);
    return gated ? forward_w4<float, true>(a, staged) : forward_w4<float, false>(a, staged);
}

