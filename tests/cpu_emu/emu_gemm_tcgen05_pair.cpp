// CPU run of the CTA-pair forward kernel (shrew_b200/csrc/gemm_tcgen05_2cta_kernels.cuh): the two blocks of
// a pair run concurrently over modelled cluster shared memory.  Grid and tensor maps as launch_pair in
// shrew_b200/csrc/gemm_tcgen05_2cta.cu sets them up.  TEST INFRASTRUCTURE ONLY; see cuda_shim.h.
#include "cuda_shim.h"
#include "cuda_shim_tcgen05.h"
#include "cuda_shim_tcgen05_pair.h"
#include "../../shrew_b200/csrc/gemm_tcgen05_2cta_kernels.cuh"

using namespace shrewq;

namespace {
template <typename YT, bool GATED>
int run(const int8_t *q, const int8_t *q_up, const Operands &ops, const uint16_t *x, void *y, int M, int N, int K, size_t ldy,
        int epilogue, int splits, int tile_list, DeviceStatus *st) {
    const uint32_t box_rows = GATED ? 64 : 128;
    const CUtensorMap tw{q, 1, (uint64_t)K, (uint64_t)N, (uint64_t)K, kBlockK, box_rows, 64};
    const CUtensorMap tw2{GATED ? q_up : q, 1, (uint64_t)K, (uint64_t)N, (uint64_t)K, kBlockK, box_rows, 64};
    const CUtensorMap tx{x, 2, (uint64_t)K, (uint64_t)M, (uint64_t)K * 2, kBlockK, kTokHalf, 128};
    const int chan_pair = GATED ? kLanes : 2 * kLanes;
    const unsigned pairs = (unsigned)((N + chan_pair - 1) / chan_pair);
    Dests none{};
    const unsigned m_tiles = (unsigned)((M + kTokPair - 1) / kTokPair);
    const int rounds = (K + kBlockK * kSub - 1) / (kBlockK * kSub);
    if (splits < 1) splits = 1;
    const int rps = (rounds + splits - 1) / splits;
    splits = (rounds + rps - 1) / rps;  // no empty split
    const size_t ctas = (size_t)2 * pairs * m_tiles;
    std::vector<float> partials(splits > 1 ? ctas * splits * kTokPair * kLanes : 0, -12345.0f);
    std::vector<unsigned int> counters(ctas, 0u);
    SplitK2 sk{splits > 1 ? partials.data() : nullptr, splits > 1 ? counters.data() : nullptr, rps, 0, 0};
    auto body = [&] {
        linear_i8_tcgen05_pair_kernel<YT, GATED>(tw, tw2, tx, ops, static_cast<YT *>(y), none, M, N, K, ldy, epilogue, sk, st);
    };
    if (tile_list >= 2) {
        // the two-launch scheme of launch_pair for a short last wave, `tile_list` standing for the pair tiles
        // that are resident at once: full waves as one launch of whole-K tiles, the rest split along K
        const int tiles = (int)(pairs * m_tiles), rem = tiles % tile_list;
        if (tiles <= tile_list || rem == 0) return -1;
        sk = SplitK2{nullptr, nullptr, rounds, 0, (int)pairs};
        emu::launch_cluster2(2u * (unsigned)(tiles - rem), 1, 1, kThreads, kSmemBytes, body);
        sk = SplitK2{splits > 1 ? partials.data() : nullptr, splits > 1 ? counters.data() : nullptr, rps, tiles - rem, (int)pairs};
        emu::launch_cluster2(2u * (unsigned)rem, 1, (unsigned)splits, kThreads, kSmemBytes, body);
    } else if (tile_list == 1) {  // the 1-D tile list as one launch over all pair tiles
        sk.pairs_total = (int)pairs;
        emu::launch_cluster2(2 * pairs * m_tiles, 1, (unsigned)splits, kThreads, kSmemBytes, body);
    } else {
        emu::launch_cluster2(2 * pairs, m_tiles, (unsigned)splits, kThreads, kSmemBytes, body);
    }
    for (unsigned int c : counters)
        if (c != 0) return -3;  // the kernel leaves the tile counters at zero for the next launch
    return 0;
}
}  // namespace

extern "C" int emu_last_a_format() { return emu::g_last_a_format.load(); }  // 0 = f16, 1 = bf16

// q_up == NULL: plain forward; else silu(gate) * up.  splits: K splits (blockIdx.z).  Returns 0; -1 for a shape
// the launcher refuses; -2 when a bounded wait of the kernel gave up; -3 when a tile counter was left set;
// -4 when a rule of the model was violated.  tile_list: 0 = (channel pair, token tile) grid; 1 = 1-D list of
// pair tiles; >= 2 = two launches (see run).
extern "C" int emu_gemm_tcgen05_pair(const int8_t *q, const float *scales, const float *bias, const int8_t *q_up,
                                     const float *scales_up, const float *bias_up, const void *x, void *y, int M, int N, int K,
                                     size_t ldy, int epilogue, int y_bf16, int splits, int tile_list) {
    if (K % 16 != 0 || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(q) & 15) || M < 1) return -1;
    DeviceStatus st{0, 0, 0, 0};
    emu::g_failed = false;
    const Operands ops{scales, bias, scales_up, bias_up};
    const uint16_t *xs = static_cast<const uint16_t *>(x);
    int rc;
    if (q_up) {
        if (y_bf16) rc = run<__nv_bfloat16, true>(q, q_up, ops, xs, y, M, N, K, ldy, epilogue, splits, tile_list, &st);
        else rc = run<float, true>(q, q_up, ops, xs, y, M, N, K, ldy, epilogue, splits, tile_list, &st);
    } else {
        if (y_bf16) rc = run<__nv_bfloat16, false>(q, q_up, ops, xs, y, M, N, K, ldy, epilogue, splits, tile_list, &st);
        else rc = run<float, false>(q, q_up, ops, xs, y, M, N, K, ldy, epilogue, splits, tile_list, &st);
    }
    if (emu::g_failed) return -4;  // a rule of the model was violated (emu_fail_message)
    if (st.timeout_flag) return -2;
    return rc;
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

