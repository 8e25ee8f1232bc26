// CPU run of the CTA-pair forward kernel (shrew_b200/csrc/gemm_tcgen05_2cta_kernels.cuh): the two blocks of
// a pair run concurrently over modelled cluster shared memory.  Grid and tensor maps as launch_pair in
// shrew_b200/csrc/gemm_tcgen05_2cta.cu sets them up.  TEST INFRASTRUCTURE ONLY; see cuda_shim.h.
#include "cuda_shim.h"
#include "cuda_shim_tcgen05.h"
#include "cuda_shim_tcgen05_pair.h"
#include "../../shrew_b200/csrc/gemm_tcgen05_2cta_kernels.cuh"

using namespace shrewq;

namespace {
template <typename YT>
int run(const int8_t *q, const float *scales, const float *bias, const uint16_t *x, void *y, int M, int N, int K, size_t ldy,
        int epilogue, DeviceStatus *st) {
    const CUtensorMap tw{q, 1, (uint64_t)K, (uint64_t)N, (uint64_t)K, kBlockK, 128, 64};
    const CUtensorMap tx{x, 2, (uint64_t)K, (uint64_t)M, (uint64_t)K * 2, kBlockK, kTokHalf, 128};
    const unsigned pairs = (unsigned)((N + 2 * kLanes - 1) / (2 * kLanes));
    Operands2 ops{scales, bias};
    Dests none{};
    emu::launch_cluster2(2 * pairs, (unsigned)((M + kTokPair - 1) / kTokPair), kThreads, kSmemBytes, [&] {
        linear_i8_tcgen05_pair_kernel<YT>(tw, tx, ops, static_cast<YT *>(y), none, M, N, K, ldy, epilogue, st);
    });
    return 0;
}
}  // namespace

// Returns 0; -1 for a shape the launcher refuses; -2 when a bounded wait of the kernel gave up.
extern "C" int emu_gemm_tcgen05_pair(const int8_t *q, const float *scales, const float *bias, const void *x, void *y, int M,
                                     int N, int K, size_t ldy, int epilogue, int y_bf16) {
    if (K % 16 != 0 || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(q) & 15) || M < 1) return -1;
    DeviceStatus st{0, 0, 0, 0};
    emu::g_failed = false;
    if (y_bf16) run<__nv_bfloat16>(q, scales, bias, static_cast<const uint16_t *>(x), y, M, N, K, ldy, epilogue, &st);
    else run<float>(q, scales, bias, static_cast<const uint16_t *>(x), y, M, N, K, ldy, epilogue, &st);
    if (emu::g_failed) return -4;  // a rule of the model was violated (emu_fail_message)
    return st.timeout_flag ? -2 : 0;
}

// fault injection: drop the n-th TMA load of the next launches (-1 = none); resets the running count
extern "C" void emu_drop_tma(int n) {
    emu::g_drop_tma = n;
    emu::g_tma_count = 0;
}

// deferred TMA: loads complete later, mostly newest first (seed != 0; a poll performs one queued load
// once in `one_in` polls), or at issue (seed 0)
extern "C" void emu_tma_async(unsigned seed, unsigned one_in) {
    emu::g_tma_async_seed = seed;
    emu::g_tma_one_in = one_in ? one_in : 8;
}

// the first violated rule of the model during the last run ("" if none)
extern "C" const char *emu_fail_message() { return emu::g_failed ? emu::g_fail_msg : ""; }

