// CPU run of the tcgen05 forward kernel (shrew_b200/csrc/gemm_tcgen05_kernels.cuh) under the CUDA
// stand-in with modelled mbarriers, TMA, tensor memory and tcgen05.mma.  Tensor maps, grid and split-K
// scratch are set up as launch_cfg in shrew_b200/csrc/gemm_tcgen05.cu does; the token tile, the number
// of converter groups and the number of K splits are chosen by the caller.
// TEST INFRASTRUCTURE ONLY; see cuda_shim.h.
#include "cuda_shim.h"
#include "cuda_shim_tcgen05.h"
#include "../../shrew_b200/csrc/gemm_tcgen05_kernels.cuh"

using namespace shrewq;

namespace {
Dests g_peers{};  // extra destinations of the next launches (the fused all-gather's peer buffers)

struct Args {
    const int8_t *q, *q_up;
    const float *scales, *bias, *scales_up, *bias_up;
    const uint16_t *x;
    void *y;
    int M, N, K;
    size_t ldy;
    int epilogue, splits, tile_list;
};

CUtensorMap map2d(const void *base, uint32_t elem, uint64_t inner, uint64_t outer, uint32_t box_inner, uint32_t box_outer, int sw) {
    return CUtensorMap{base, elem, inner, outer, inner * elem, box_inner, box_outer, sw};
}

template <int TOK, int KSUB, int G, bool GATED, typename YT>
int run(const Args &a, DeviceStatus *status) {
    using C = Cfg<TOK, KSUB>;
    const int chan = GATED ? 64 : 128;
    const CUtensorMap tw = map2d(a.q, 1, a.K, a.N, kBlockK, GATED ? 64 : 128, 64);
    const CUtensorMap tw2 = GATED ? map2d(a.q_up, 1, a.K, a.N, kBlockK, 64, 64) : tw;
    const CUtensorMap tx = map2d(a.x, 2, a.K, a.M, kBlockK, TOK, 128);
    const int n_tiles = (a.N + chan - 1) / chan, m_tiles = (a.M + TOK - 1) / TOK;
    const int rounds = (a.K + kBlockK * KSUB - 1) / (kBlockK * KSUB);
    int splits = a.splits < 1 ? 1 : a.splits;
    const int rps = (rounds + splits - 1) / splits;
    splits = (rounds + rps - 1) / rps;  // no empty split
    std::vector<float> partials;
    std::vector<unsigned int> counters((size_t)n_tiles * m_tiles, 0u);
    SplitK sk{nullptr, nullptr, rps, 0, 0};
    if (splits > 1) {
        partials.assign((size_t)n_tiles * m_tiles * splits * TOK * kTileN, -12345.0f);
        sk.partials = partials.data();
        sk.counters = counters.data();
    }
    Operands ops{a.scales, a.bias, a.scales_up, a.bias_up};
    auto body = [&] {
        linear_i8_tcgen05_kernel<TOK, KSUB, G, GATED, YT>(tw, tw2, tx, ops, static_cast<YT *>(a.y), g_peers, a.M, a.N, a.K, a.ldy,
                                                          a.epilogue, sk, status);
    };
    if (a.tile_list >= 2) {
        // the two-launch scheme of launch_cfg for a short last wave, with `tile_list` standing for the SM
        // count: full waves as one launch of whole-K tiles, the remaining tiles as a second launch split
        // along K (a.splits ways); both launches use the 1-D tile list
        const int tiles = n_tiles * m_tiles, rem = tiles % a.tile_list;
        if (tiles <= a.tile_list || rem == 0) return -1;
        sk = SplitK{nullptr, nullptr, rounds, 0, n_tiles};
        emu::launch3((unsigned)(tiles - rem), 1, 1, 64 + 128 * G, C::kSmemRequest, body);
        sk = SplitK{partials.data(), counters.data(), rps, tiles - rem, n_tiles};
        if (splits == 1) sk.partials = nullptr, sk.counters = nullptr;
        emu::launch3((unsigned)rem, 1, (unsigned)splits, 64 + 128 * G, C::kSmemRequest, body);
        for (unsigned int c : counters)
            if (c != 0) return -3;
        return 0;
    }
    if (a.tile_list == 1) {  // the 1-D tile list of the two-launch scheme, here as one launch over all tiles
        sk.tile_begin = 0;
        sk.n_tiles_total = n_tiles;
        emu::launch3((unsigned)(n_tiles * m_tiles), 1, (unsigned)splits, 64 + 128 * G, C::kSmemRequest, body);
    } else {
        emu::launch3((unsigned)n_tiles, (unsigned)m_tiles, (unsigned)splits, 64 + 128 * G, C::kSmemRequest, body);
    }
    for (unsigned int c : counters)
        if (c != 0) return -3;  // the kernels leave the tile counters at zero for the next launch
    return 0;
}

template <int TOK, int KSUB, bool GATED, typename YT>
int run_g(const Args &a, int groups, DeviceStatus *st) {
    if (groups == 1) return run<TOK, KSUB, 1, GATED, YT>(a, st);
    if (groups == 2) return run<TOK, KSUB, 2, GATED, YT>(a, st);
    return run<TOK, KSUB, 3, GATED, YT>(a, st);
}

template <bool GATED, typename YT>
int run_tok(const Args &a, int tok, int groups, DeviceStatus *st) {
    switch (tok) {
        case 16: return run_g<16, 2, GATED, YT>(a, groups, st);
        case 32: return run_g<32, 2, GATED, YT>(a, groups, st);
        case 64: return run_g<64, 2, GATED, YT>(a, groups, st);
        case 128: return run_g<128, 2, GATED, YT>(a, groups, st);
        case 256: return run_g<256, 1, GATED, YT>(a, groups, st);
        default: return -1;
    }
}
}  // namespace

// x: bf16 bits [M,K]; y: f32 or bf16 bits [M, ldy].  Returns 0; -1 for an unknown token tile or a shape
// tcgen05_supported refuses; -2 when a bounded wait of the kernel gave up; -3 when a tile counter was
// left non-zero.
extern "C" int emu_gemm_tcgen05(const int8_t *q, const float *scales, const float *bias, const int8_t *q_up,
                                const float *scales_up, const float *bias_up, const void *x, void *y, int M, int N, int K,
                                size_t ldy, int epilogue, int y_bf16, int tok, int groups, int splits, int tile_list) {
    if (K % 16 != 0 || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(q) & 15) || M < 1) return -1;
    Args a{q, q_up, scales, bias, scales_up, bias_up, static_cast<const uint16_t *>(x), y, M, N, K, ldy, epilogue, splits, tile_list};
    DeviceStatus st{0, 0, 0, 0};
    emu::g_failed = false;
    int rc;
    if (q_up) rc = y_bf16 ? run_tok<true, __nv_bfloat16>(a, tok, groups, &st) : run_tok<true, float>(a, tok, groups, &st);
    else rc = y_bf16 ? run_tok<false, __nv_bfloat16>(a, tok, groups, &st) : run_tok<false, float>(a, tok, groups, &st);
    if (emu::g_failed) return -4;  // a rule of the model was violated (emu_fail_message)
    if (st.timeout_flag) return -2;
    return rc;
}

// f32 activations as a bf16 hi/lo pair (x: [2M, K] bf16 bits, the lo rows under the hi rows), 128- or 256-token
// tiles, one sub-block per stage, as launch_gemm_tcgen05_xsplit sets the launch up.  Same return codes as above.
template <int TOK>
static int run_xsplit(const int8_t *q, const float *scales, const float *bias, const void *x_hi_lo, void *y, int M, int N, int K,
                      size_t ldy, int epilogue, int y_bf16, int splits) {
    using C = Cfg<TOK, 1, true>;
    const CUtensorMap tw = map2d(q, 1, K, N, kBlockK, 128, 64);
    const CUtensorMap tx = map2d(x_hi_lo, 2, K, 2 * (uint64_t)M, kBlockK, TOK, 128);
    const int n_tiles = (N + 127) / 128, m_tiles = (M + TOK - 1) / TOK;
    const int rounds = (K + kBlockK - 1) / kBlockK;
    if (splits < 1) splits = 1;
    const int rps = (rounds + splits - 1) / splits;
    splits = (rounds + rps - 1) / rps;
    std::vector<float> partials(splits > 1 ? (size_t)n_tiles * m_tiles * splits * TOK * kTileN : 0, -12345.0f);
    std::vector<unsigned int> counters((size_t)n_tiles * m_tiles, 0u);
    SplitK sk{splits > 1 ? partials.data() : nullptr, splits > 1 ? counters.data() : nullptr, rps, 0, 0};
    Operands ops{scales, bias, nullptr, nullptr};
    DeviceStatus st{0, 0, 0, 0};
    emu::g_failed = false;
    Dests none{};
    auto body = [&] {
        if (y_bf16) linear_i8_tcgen05_kernel<TOK, 1, 3, false, __nv_bfloat16, true>(tw, tw, tx, ops, static_cast<__nv_bfloat16 *>(y), none, M, N, K, ldy, epilogue, sk, &st);
        else linear_i8_tcgen05_kernel<TOK, 1, 3, false, float, true>(tw, tw, tx, ops, static_cast<float *>(y), none, M, N, K, ldy, epilogue, sk, &st);
    };
    emu::launch3((unsigned)n_tiles, (unsigned)m_tiles, (unsigned)splits, 64 + 128 * 3, C::kSmemRequest, body);
    if (emu::g_failed) return -4;
    if (st.timeout_flag) return -2;
    for (unsigned int c : counters)
        if (c != 0) return -3;
    return 0;
}
extern "C" int emu_gemm_tcgen05_xsplit(const int8_t *q, const float *scales, const float *bias, const void *x_hi_lo, void *y, int M,
                                       int N, int K, size_t ldy, int epilogue, int y_bf16, int splits, int tok) {
    if (K % 16 != 0 || (reinterpret_cast<uintptr_t>(x_hi_lo) & 15) || (reinterpret_cast<uintptr_t>(q) & 15) || M < 1) return -1;
    if (tok == 256) return run_xsplit<256>(q, scales, bias, x_hi_lo, y, M, N, K, ldy, epilogue, y_bf16, splits);
    return run_xsplit<128>(q, scales, bias, x_hi_lo, y, M, N, K, ldy, epilogue, y_bf16, splits);
}

extern "C" int emu_last_a_format() { return emu::g_last_a_format.load(); }  // 0 = f16, 1 = bf16

// peer destinations of the next launches: every output value is also stored at the same offset there
extern "C" void emu_set_peers(void **p, int n) {
    g_peers = Dests{};
    for (int i = 0; i < n && i < kMaxPeers; ++i) g_peers.p[i] = p[i];
    g_peers.n = n;
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

