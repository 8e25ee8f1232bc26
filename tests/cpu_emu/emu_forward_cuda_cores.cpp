// CPU run of the CUDA-core forward kernels (shrew_b200/csrc/gemv_kernels.cuh and gemm_simt_kernels.cuh)
// under the CUDA stand-in; kernel variants chosen as launch_gemv / launch_gemm_simt choose them.
// TEST INFRASTRUCTURE ONLY; see cuda_shim.h.
#include "cuda_shim.h"
#include "cuda_shim_tcgen05.h"
#include "../../shrew_b200/csrc/gemv_kernels.cuh"
#include "../../shrew_b200/csrc/gemv_ring_kernels.cuh"
#include "../../shrew_b200/csrc/gemm_simt_kernels.cuh"

using namespace shrewq;

namespace {
Dests g_peers{};

struct Args {
    const int8_t *q, *q_up;
    const float *scales, *bias, *scales_up, *bias_up;
    const void *x;
    void *y;
    int M, N, K;
    size_t ldy;
    int epilogue, pdl;
};

template <int MT, int R, typename XT, typename YT, bool GATED>
void gemv_one(const Args &a) {
    constexpr int NR = GATED ? R / 2 : R;
    const unsigned grid = (unsigned)((a.N + NR - 1) / NR), gy = (unsigned)((a.M + MT - 1) / MT);  // as launch_one
    if (gy > 1) {  // as launch_one: the sliced instantiation
        emu::launch3(grid, gy, 1, kThreads, 0, [&] {
            gemv_i8_kernel<MT, R, XT, YT, GATED, false, true>(a.q, a.scales, a.bias, a.q_up, a.scales_up, a.bias_up,
                                                              static_cast<const XT *>(a.x), static_cast<YT *>(a.y), g_peers, a.M,
                                                              a.N, a.K, a.ldy, a.epilogue);
        });
        return;
    }
    // pdl: the variant that fetches its first weights before waiting for the previous kernel
    if (a.pdl)
        emu::launch(grid, kThreads, [&] {
            gemv_i8_kernel<MT, R, XT, YT, GATED, true>(a.q, a.scales, a.bias, a.q_up, a.scales_up, a.bias_up,
                                                       static_cast<const XT *>(a.x), static_cast<YT *>(a.y), g_peers, a.M, a.N,
                                                       a.K, a.ldy, a.epilogue);
        });
    else
        emu::launch(grid, kThreads, [&] {
            gemv_i8_kernel<MT, R, XT, YT, GATED>(a.q, a.scales, a.bias, a.q_up, a.scales_up, a.bias_up, static_cast<const XT *>(a.x),
                                                 static_cast<YT *>(a.y), g_peers, a.M, a.N, a.K, a.ldy, a.epilogue);
        });
}
template <typename XT, typename YT, bool GATED>
void gemv_m(const Args &a) {
    if (a.M <= 1) gemv_one<1, 4, XT, YT, GATED>(a);
    else if (a.M <= 2) gemv_one<2, 4, XT, YT, GATED>(a);
    else if (a.M <= 4) gemv_one<4, 4, XT, YT, GATED>(a);
    else if (a.M <= 8) gemv_one<8, 2, XT, YT, GATED>(a);
    else gemv_one<16, 2, XT, YT, GATED>(a);
}
template <typename XT, typename YT>
void gemv_g(const Args &a) {
    if (a.q_up) gemv_m<XT, YT, true>(a); else gemv_m<XT, YT, false>(a);
}

// the ring kernel (bulk copies into a shared-memory ring + warp MMA), instantiated as launch_gemv_ring does
DeviceStatus g_ring_status{};
int g_ring_kc = kRingKC;
bool g_ring_two_stages = false;
template <int NT, int KC, typename YT, bool GATED>
void ring_one_kc(const Args &a) {
    constexpr int NCH = GATED ? kRingRows / 2 : kRingRows;
    const unsigned grid = (unsigned)((a.N + NCH - 1) / NCH);
    if (g_ring_two_stages) {  // the launcher's choice for grids of several waves
        emu::launch(grid, (kRingConsumers + 1) * 32, RingCfg<KC, 2>::kSmemBytes, [&] {
            gemv_i8_ring_kernel<NT, KC, kRingConsumers, YT, GATED, 2>(a.q, a.scales, a.bias, a.q_up, a.scales_up, a.bias_up,
                                                                      static_cast<const uint16_t *>(a.x), static_cast<YT *>(a.y),
                                                                      g_peers, a.M, a.N, a.K, a.ldy, a.epilogue, &g_ring_status);
        });
        return;
    }
    emu::launch(grid, (kRingConsumers + 1) * 32, RingCfg<KC>::kSmemBytes, [&] {
        gemv_i8_ring_kernel<NT, KC, kRingConsumers, YT, GATED>(a.q, a.scales, a.bias, a.q_up, a.scales_up, a.bias_up,
                                                               static_cast<const uint16_t *>(a.x), static_cast<YT *>(a.y), g_peers,
                                                               a.M, a.N, a.K, a.ldy, a.epilogue, &g_ring_status);
    });
}
template <int NT, typename YT, bool GATED>
void ring_one(const Args &a) {
    if (g_ring_kc == 512) ring_one_kc<NT, 512, YT, GATED>(a);
    else if (g_ring_kc == 2048) ring_one_kc<NT, 2048, YT, GATED>(a);
    else ring_one_kc<NT, 1024, YT, GATED>(a);
}
template <typename YT, bool GATED>
void ring_m(const Args &a) {
    if (a.M <= 8) ring_one<1, YT, GATED>(a);
    else if (a.M <= 16) ring_one<2, YT, GATED>(a);
    else ring_one<4, YT, GATED>(a);
}

template <typename XT, typename YT>
void simt_t(const Args &a) {
    const unsigned gx = (unsigned)((a.N + BN - 1) / BN), gy = (unsigned)((a.M + BM - 1) / BM);
    if (a.q_up)
        emu::launch3(gx, gy, 1, 256, 0, [&] {
            gemm_i8_simt_kernel<XT, YT, true>(a.q, a.scales, a.bias, a.q_up, a.scales_up, a.bias_up, static_cast<const XT *>(a.x),
                                              static_cast<YT *>(a.y), (size_t)a.M, (size_t)a.N, (size_t)a.K, a.ldy, a.epilogue);
        });
    else
        emu::launch3(gx, gy, 1, 256, 0, [&] {
            gemm_i8_simt_kernel<XT, YT, false>(a.q, a.scales, a.bias, nullptr, nullptr, nullptr, static_cast<const XT *>(a.x),
                                               static_cast<YT *>(a.y), (size_t)a.M, (size_t)a.N, (size_t)a.K, a.ldy, a.epilogue);
        });
}
}  // namespace

extern "C" void emu_set_ring_kc(int kc) { g_ring_kc = kc; }
extern "C" void emu_set_ring_two_stages(int on) { g_ring_two_stages = on != 0; }

extern "C" void emu_set_peers(void **p, int n) {
    g_peers = Dests{};
    for (int i = 0; i < n && i < kMaxPeers; ++i) g_peers.p[i] = p[i];
    g_peers.n = n;
}

// kernel: 0 = gemv (M <= 128, in slices of 16 tokens above 16; K % 16 == 0, 16-byte aligned q and x), 1 = general f32 kernel, 2 = ring kernel
// (bf16 activations, M <= 32, K % 64 == 0, same alignment).
// x_bf16 / y_bf16: element types.  Returns -1 for a shape the launcher refuses.
extern "C" int emu_forward_cuda_cores(int kernel, const int8_t *q, const float *scales, const float *bias, const int8_t *q_up,
                                      const float *scales_up, const float *bias_up, const void *x, void *y, int M, int N, int K,
                                      size_t ldy, int epilogue, int x_bf16, int y_bf16, int pdl) {
    const Args a{q, q_up, scales, bias, scales_up, bias_up, x, y, M, N, K, ldy, epilogue, pdl};
    if (kernel == 0) {
        if (M < 1 || M > 128 || K % 16 != 0 || K == 0 || (reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(x) & 15)) return -1;
        if (x_bf16 && y_bf16) gemv_g<__nv_bfloat16, __nv_bfloat16>(a);
        else if (x_bf16) gemv_g<__nv_bfloat16, float>(a);
        else if (!y_bf16) gemv_g<float, float>(a);
        else gemv_g<float, __nv_bfloat16>(a);
        return 0;
    }
    if (kernel == 2) {
        if (!x_bf16 || M < 1 || M > 32 || K % 64 != 0 || K == 0 || (reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(x) & 15)) return -1;
        g_ring_status = DeviceStatus{};
        if (y_bf16) { if (a.q_up) ring_m<__nv_bfloat16, true>(a); else ring_m<__nv_bfloat16, false>(a); }
        else { if (a.q_up) ring_m<float, true>(a); else ring_m<float, false>(a); }
        return g_ring_status.timeout_flag ? -2 : 0;
    }
    if (x_bf16 && y_bf16) simt_t<__nv_bfloat16, __nv_bfloat16>(a);
    else if (x_bf16) simt_t<__nv_bfloat16, float>(a);
    else if (!y_bf16) simt_t<float, float>(a);
    else simt_t<float, __nv_bfloat16>(a);
    return 0;
}
