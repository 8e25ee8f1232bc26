// Host side of the tcgen05 forward: tensor maps, launch plan, launchers (device code and its
// description: gemm_tcgen05_kernels.cuh).
#include <cuda.h>

#include <atomic>
#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "gemm_tcgen05_kernels.cuh"

namespace shrewq {
namespace {

// ---- host side ------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

int encode_2d(shrewq_ctx *ctx, CUtensorMap *out, CUtensorMapDataType dt, int elem_bytes, const void *base,
              size_t inner, size_t outer, int box_inner, int box_outer, CUtensorMapSwizzle sw) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return set_err(ctx, SHREWQ_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
    cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
    cuuint64_t strides[1] = {(cuuint64_t)inner * elem_bytes};
    cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, dt, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_err(ctx, SHREWQ_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return SHREWQ_OK;
}

// ---- launch ---------------------------------------------------------------------------
constexpr size_t kScratchCounterOff = 4096, kScratchPartialOff = 8192;

struct LaunchPlan {
    int n_tiles, m_tiles, splits, rounds_per_split;
};

// Split-K when the output tiles alone leave most SMs idle: as many splits as fit in one wave, each with at
// least 2 pipeline rounds (token tiles up to 64, whose partial sums are small) or 8 (larger tiles).
// split_max_tok: the widest token tile that may be split (the no-allocation entry point keeps its
// partial sums in a fixed array and splits the small tiles only).
template <int TOK, int KSUB>
LaunchPlan plan_launch(const ForwardArgs &a, int chan_per_tile, int sm_count, bool allow_split, int split_max_tok = 256) {
    LaunchPlan p;
    p.n_tiles = (int)((a.N + chan_per_tile - 1) / chan_per_tile);
    p.m_tiles = (int)((a.M + TOK - 1) / TOK);
    const int rounds = (int)((a.K + kBlockK * KSUB - 1) / (kBlockK * KSUB));
    int splits = 1;
    const long tiles = (long)p.n_tiles * p.m_tiles;
    const int min_rounds = TOK <= 64 ? 2 : 8;
    if (allow_split && TOK <= split_max_tok && tiles <= 1024) {
        int want = (int)(sm_count / tiles);
        if (want > rounds / min_rounds) want = rounds / min_rounds;
        if (want > 1) splits = want;
    }
    p.rounds_per_split = (rounds + splits - 1) / splits;
    p.splits = (rounds + p.rounds_per_split - 1) / p.rounds_per_split;  // no empty split
    return p;
}

// cudaFuncSetAttribute once per kernel instantiation and device (bit d of `done`: device d has it)
template <typename Kern>
int set_smem_attr_once(shrewq_ctx *ctx, Kern kern, int bytes, std::atomic<unsigned long long> &done) {
    const int d = ctx->device;
    if (d >= 0 && d < 64 && ((done.load(std::memory_order_acquire) >> d) & 1ull)) return SHREWQ_OK;
    SHREWQ_CUDA_TRY(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    if (d >= 0 && d < 64) done.fetch_or(1ull << d, std::memory_order_release);
    return SHREWQ_OK;
}

// scratch == nullptr: use (and grow) the context's scratch; otherwise a caller-provided
// region of scratch_bytes laid out as [0,4096) counters, partial sums from 4096.
// XSPLIT: a.x is the bf16 hi/lo pair of f32 activations, lo rows stacked under the M hi rows
template <int TOK, int KSUB, int G, bool GATED, typename YT, bool XSPLIT = false>
int launch_cfg(shrewq_ctx *ctx, const ForwardArgs &a, const CUtensorMap &tw, const CUtensorMap &tw2, bool allow_split,
               void *fixed_scratch, size_t fixed_scratch_bytes) {
    using C = Cfg<TOK, KSUB, XSPLIT>;
    CUtensorMap tx;
    int rc = encode_2d(ctx, &tx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.x, a.K, XSPLIT ? 2 * a.M : a.M, kBlockK, TOK,
                       CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != SHREWQ_OK) return rc;
    auto kern = linear_i8_tcgen05_kernel<TOK, KSUB, G, GATED, YT, XSPLIT>;
    static std::atomic<unsigned long long> attr_done{0};  // per instantiation
    if ((rc = set_smem_attr_once(ctx, kern, C::kSmemRequest, attr_done)) != SHREWQ_OK) return rc;
    const LaunchPlan p = plan_launch<TOK, KSUB>(a, GATED ? 64 : 128, ctx->sm_count, allow_split, fixed_scratch ? 64 : 256);
    SplitK sk{nullptr, nullptr, p.rounds_per_split, 0, 0};
    Operands ops{a.scales, a.bias, a.scales_up, a.bias_up};
    // Option tc_tailsplit: when large tiles leave a short last wave, issue the full waves as one
    // launch and the tiles of the last wave as a second launch split along K so that it also fills
    // the SMs.
    const bool tail_split = ctx->tuning.tc_tailsplit == 1;
    if (tail_split && !fixed_scratch && TOK >= 128 && p.splits == 1) {
        const int tiles = p.n_tiles * p.m_tiles, rem = tiles % ctx->sm_count;
        const int rounds = p.rounds_per_split;
        int s_tail = rem > 0 ? ctx->sm_count / rem : 0;
        if (s_tail > 4) s_tail = 4;
        if (s_tail > rounds / 8) s_tail = rounds / 8;
        if (tiles > ctx->sm_count && rem > 0 && s_tail >= 2) {
            const size_t part_bytes = (size_t)rem * s_tail * TOK * kTileN * sizeof(float);
            if ((rc = ensure_scratch(ctx, kScratchPartialOff + part_bytes)) != SHREWQ_OK) return rc;
            if (!ctx->counters_zeroed) {
                SHREWQ_CUDA_TRY(ctx, cudaMemsetAsync(static_cast<char *>(ctx->scratch) + kScratchCounterOff, 0,
                                                     kScratchPartialOff - kScratchCounterOff, ctx->stream));
                ctx->counters_zeroed = true;
            }
            SplitK head{nullptr, nullptr, rounds, 0, p.n_tiles};
            SHREWQ_CUDA_TRY(ctx, launch_maybe_pdl(kern, dim3((unsigned)(tiles - rem), 1, 1), dim3(64 + 128 * G), (size_t)C::kSmemRequest,
                                                  ctx->stream, a.pdl, tw, tw2, tx, ops, static_cast<YT *>(a.y), a.extra, (int)a.M,
                                                  (int)a.N, (int)a.K, a.ldy, a.epilogue, head, ctx->dev_status));
            const int rps = (rounds + s_tail - 1) / s_tail;
            const int splits = (rounds + rps - 1) / rps;
            SplitK tail{reinterpret_cast<float *>(static_cast<char *>(ctx->scratch) + kScratchPartialOff),
                        reinterpret_cast<unsigned int *>(static_cast<char *>(ctx->scratch) + kScratchCounterOff), rps,
                        tiles - rem, p.n_tiles};
            SHREWQ_CUDA_TRY(ctx, launch_maybe_pdl(kern, dim3((unsigned)rem, 1, (unsigned)splits), dim3(64 + 128 * G),
                                                  (size_t)C::kSmemRequest, ctx->stream, a.pdl, tw, tw2, tx, ops, static_cast<YT *>(a.y),
                                                  a.extra, (int)a.M, (int)a.N, (int)a.K, a.ldy, a.epilogue, tail, ctx->dev_status));
            ctx->launches += 2;
            SHREWQ_CUDA_TRY(ctx, cudaGetLastError());
            return SHREWQ_OK;
        }
    }
    if (p.splits > 1) {
        const size_t tiles = (size_t)p.n_tiles * p.m_tiles;
        const size_t part_bytes = tiles * p.splits * TOK * kTileN * sizeof(float);
        if (fixed_scratch) {
            const size_t need = 4096 + part_bytes;
            if (need > fixed_scratch_bytes)
                return set_err(ctx, SHREWQ_ERR_UNSUPPORTED,
                               "forward_noalloc: this shape needs %zu bytes of split-K scratch, the built-in array holds %zu "
                               "(use shrewq_linear_forward, which allocates)", need, fixed_scratch_bytes);
            // the array keeps whatever the previous call left: the counters must start at zero
            SHREWQ_CUDA_TRY(ctx, cudaMemsetAsync(fixed_scratch, 0, 4096, ctx->stream));
            sk.counters = static_cast<unsigned int *>(fixed_scratch);
            sk.partials = reinterpret_cast<float *>(static_cast<unsigned char *>(fixed_scratch) + 4096);
        } else {
            // context scratch: [0,4096) quantizer words, [4096,8192) tile counters (at most one
            // per SM is ever in use), partial sums from 8192
            if ((rc = ensure_scratch(ctx, kScratchPartialOff + part_bytes)) != SHREWQ_OK) return rc;
            if (!ctx->counters_zeroed) {
                // fresh scratch: counters must start at zero (the kernels reset them after use)
                SHREWQ_CUDA_TRY(ctx, cudaMemsetAsync(static_cast<char *>(ctx->scratch) + kScratchCounterOff, 0,
                                                     kScratchPartialOff - kScratchCounterOff, ctx->stream));
                ctx->counters_zeroed = true;
            }
            sk.counters = reinterpret_cast<unsigned int *>(static_cast<char *>(ctx->scratch) + kScratchCounterOff);
            sk.partials = reinterpret_cast<float *>(static_cast<char *>(ctx->scratch) + kScratchPartialOff);
        }
    }
    dim3 grid((unsigned)p.n_tiles, (unsigned)p.m_tiles, (unsigned)p.splits);
    SHREWQ_CUDA_TRY(ctx, launch_maybe_pdl(kern, grid, dim3(64 + 128 * G), (size_t)C::kSmemRequest, ctx->stream, a.pdl, tw, tw2, tx, ops,
                                          static_cast<YT *>(a.y), a.extra, (int)a.M, (int)a.N, (int)a.K, a.ldy, a.epilogue, sk,
                                          ctx->dev_status));
    ctx->launches += 1;
    SHREWQ_CUDA_TRY(ctx, cudaGetLastError());
    return SHREWQ_OK;
}

template <int TOK, int KSUB, bool GATED, typename YT>
int launch_groups(shrewq_ctx *ctx, const ForwardArgs &a, const CUtensorMap &tw, const CUtensorMap &tw2, void *fs, size_t fsb) {
    const bool sk = ctx->tuning.tc_splitk != 0;
    if (ctx->tuning.tc_groups == 1) return launch_cfg<TOK, KSUB, 1, GATED, YT>(ctx, a, tw, tw2, sk, fs, fsb);
    if (ctx->tuning.tc_groups == 2) return launch_cfg<TOK, KSUB, 2, GATED, YT>(ctx, a, tw, tw2, sk, fs, fsb);
    return launch_cfg<TOK, KSUB, 3, GATED, YT>(ctx, a, tw, tw2, sk, fs, fsb);
}

// Token tile: the smallest tile that covers M up to 128.  Above that a gate/up launch takes 256 tokens
// (twice the tokens per converted weight byte; measured 12 % shorter on the 4096 -> 11008 block at batch 512),
// a plain launch 256 tokens unless 128-token tiles fill the SMs markedly better (few channel tiles, e.g.
// N = 4096 at M = 512: 128 CTAs instead of 64).
int choose_tok(const ForwardArgs &a, bool gated, int sm_count, const Tuning &t) {
    const int forced = (gated && t.tc_tok_gated) ? t.tc_tok_gated : t.tc_tok;
    if (forced == 16 || forced == 32 || forced == 64 || forced == 128 || forced == 256) return forced;
    if (a.M <= 16) return 16;
    if (a.M <= 32) return 32;
    if (a.M <= 64) return 64;
    if (a.M <= 128) return 128;
    if (gated) return 256;
    const long n_tiles = (long)((a.N + 127) / 128);
    auto fill = [&](int tok) {
        const long tiles = n_tiles * (long)((a.M + tok - 1) / tok);
        const long waves = (tiles + sm_count - 1) / sm_count;
        return (double)tiles / (double)(waves * sm_count);
    };
    return fill(128) * 0.85 > fill(256) ? 128 : 256;
}

template <bool GATED, typename YT>
int launch_y(shrewq_ctx *ctx, const ForwardArgs &a, const CUtensorMap &tw, const CUtensorMap &tw2, void *fs, size_t fsb) {
    switch (choose_tok(a, GATED, ctx->sm_count, ctx->tuning)) {
        // small token tiles are HBM-bound: 2 sub-blocks per stage keeps the pipeline 6-7 stages
        // deep (TMEM columns limit the depth), i.e. ~100 KB of codes in flight per SM
        case 16: return launch_groups<16, 2, GATED, YT>(ctx, a, tw, tw2, fs, fsb);
        case 32: return launch_groups<32, 2, GATED, YT>(ctx, a, tw, tw2, fs, fsb);
        case 64: return launch_groups<64, 2, GATED, YT>(ctx, a, tw, tw2, fs, fsb);
        case 128: return launch_groups<128, 2, GATED, YT>(ctx, a, tw, tw2, fs, fsb);
        default: return launch_groups<256, 1, GATED, YT>(ctx, a, tw, tw2, fs, fsb);
    }
}

// ---- forward without any allocation ---------------------------------------------------
// Split-K scratch for shrewq_linear_forward_noalloc: a fixed array inside the library image
// instead of a cudaMalloc'd buffer.  Every GPU that loads the library holds these 4 MiB
// until the process exits.  Layout: [0,4096) tile counters, partial sums from 4096.
constexpr size_t kStaticScratchBytes = 4u << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code the array's name is only a handle for the runtime, not a device address:
// the address is looked up once per device (with that device current) and cached.
constexpr int kMaxDevices = 64;
static std::atomic<void *> g_static_scratch_addr[kMaxDevices];

int static_scratch_for_device(shrewq_ctx *ctx, void **out) {
    if (ctx->device < 0 || ctx->device >= kMaxDevices)
        return set_err(ctx, SHREWQ_ERR_UNSUPPORTED, "forward_noalloc: device index %d above %d", ctx->device, kMaxDevices - 1);
    if (!g_static_scratch_addr[ctx->device].load(std::memory_order_acquire)) {
        void *p = nullptr;
        SHREWQ_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || !p)
            return set_err(ctx, SHREWQ_ERR_CUDA, "forward_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        g_static_scratch_addr[ctx->device].store(p, std::memory_order_release);  // every thread looks up the same address
    }
    *out = g_static_scratch_addr[ctx->device].load(std::memory_order_acquire);
    return SHREWQ_OK;
}

}  // namespace

#ifdef SHREWQ_TRACE
extern "C" __attribute__((visibility("default"))) int shrewq_debug_set_trace(long long *dev_buf) {
    return (int)cudaMemcpyToSymbol(g_trace, &dev_buf, sizeof(dev_buf));
}
#endif

bool tcgen05_supported(const ForwardArgs &a) {
    return a.x_dtype == SHREWQ_BF16 && a.K >= 16 && (a.K % 16) == 0 && a.M >= 1 && a.N >= 1 &&
           (reinterpret_cast<uintptr_t>(a.x) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.q) & 15) == 0 &&
           (!a.q_up || (reinterpret_cast<uintptr_t>(a.q_up) & 15) == 0) && a.K < (1u << 31) && a.N < (1u << 31) &&
           a.M < (1u << 31) && (a.M + 15) / 16 <= 65535 * 16;
}

// box_rows = 128 for plain tiles, 64 for the gate / up halves of a gated tile
int encode_weight_tmap(shrewq_ctx *ctx, const int8_t *q, size_t n, size_t k, int box_rows, void *tmap_out) {
    return encode_2d(ctx, static_cast<CUtensorMap *>(tmap_out), CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, q, k, n, kBlockK,
                     box_rows, CU_TENSOR_MAP_SWIZZLE_64B);
}

// f32 activations: a.x points at the bf16 hi matrix [M,K] with the lo matrix right behind it
int launch_gemm_tcgen05_xsplit(shrewq_ctx *ctx, const ForwardArgs &a, const void *w_tmap) {
    const CUtensorMap &tw = *static_cast<const CUtensorMap *>(w_tmap);
    const bool sk = ctx->tuning.tc_splitk != 0;
    // token tile: 256 (half the tiles, twice the work per prologue and per byte of weights) when such tiles still
    // keep three quarters of the SMs busy, 128 otherwise; option tc_tok overrides.  Measured at 4096 tokens:
    // 50257 x 256: 666 against 910 us; 1024 x 256: 14.8 against 19.6 us; 256 x 1024 (32 tiles): 28.4 against 21.5 us.
    const size_t tiles256 = ((a.N + kTileN - 1) / kTileN) * ((a.M + 255) / 256);
    const int tok = ctx->tuning.tc_tok == 128 || ctx->tuning.tc_tok == 256 ? ctx->tuning.tc_tok
                    : (tiles256 * 4 >= (size_t)ctx->sm_count * 3 ? 256 : 128);
    if (tok == 256) {
        if (a.y_dtype == SHREWQ_BF16) return launch_cfg<256, 1, 3, false, __nv_bfloat16, true>(ctx, a, tw, tw, sk, nullptr, 0);
        return launch_cfg<256, 1, 3, false, float, true>(ctx, a, tw, tw, sk, nullptr, 0);
    }
    if (a.y_dtype == SHREWQ_BF16) return launch_cfg<128, 1, 3, false, __nv_bfloat16, true>(ctx, a, tw, tw, sk, nullptr, 0);
    return launch_cfg<128, 1, 3, false, float, true>(ctx, a, tw, tw, sk, nullptr, 0);
}

int launch_gemm_tcgen05_noalloc(shrewq_ctx *ctx, const ForwardArgs &a, const void *w_tmap) {
    const CUtensorMap &tw = *static_cast<const CUtensorMap *>(w_tmap);
    void *base = nullptr;
    int rc = static_scratch_for_device(ctx, &base);
    if (rc != SHREWQ_OK) return rc;
    if (a.y_dtype == SHREWQ_BF16) return launch_y<false, __nv_bfloat16>(ctx, a, tw, tw, base, kStaticScratchBytes);
    return launch_y<false, float>(ctx, a, tw, tw, base, kStaticScratchBytes);
}

// w_tmap: 128-row boxes of the weight (plain) or 64-row boxes of the gate matrix (gated, with
// w_up_tmap the 64-row boxes of the up matrix)
// The launch plan of the tcgen05 forward for a shape, without launching anything (pure host arithmetic:
// token tile, tile grid, K splits, pipeline rounds per split).
int plan_gemm_tcgen05(size_t M, size_t N, size_t K, bool gated, int sm_count, int *tok, int *n_tiles, int *m_tiles,
                      int *splits, int *rounds_per_split) {
    ForwardArgs a{};
    a.M = M; a.N = N; a.K = K;
    const Tuning t;  // the defaults
    const int chan = gated ? 64 : 128;
    const int tk = choose_tok(a, gated, sm_count, t);
    LaunchPlan p;
    switch (tk) {
        case 16: p = plan_launch<16, 2>(a, chan, sm_count, true); break;
        case 32: p = plan_launch<32, 2>(a, chan, sm_count, true); break;
        case 64: p = plan_launch<64, 2>(a, chan, sm_count, true); break;
        case 128: p = plan_launch<128, 2>(a, chan, sm_count, true); break;
        case 256: p = plan_launch<256, 1>(a, chan, sm_count, true); break;
        default: return SHREWQ_ERR_INVALID_ARG;
    }
    *tok = tk; *n_tiles = p.n_tiles; *m_tiles = p.m_tiles; *splits = p.splits; *rounds_per_split = p.rounds_per_split;
    return SHREWQ_OK;
}

int launch_gemm_tcgen05(shrewq_ctx *ctx, const ForwardArgs &a, const void *w_tmap, const void *w_up_tmap) {
    const CUtensorMap &tw = *static_cast<const CUtensorMap *>(w_tmap);
    if (a.q_up) {
        const CUtensorMap &tw2 = *static_cast<const CUtensorMap *>(w_up_tmap);
        if (a.y_dtype == SHREWQ_BF16) return launch_y<true, __nv_bfloat16>(ctx, a, tw, tw2, nullptr, 0);
        return launch_y<true, float>(ctx, a, tw, tw2, nullptr, 0);
    }
    if (a.y_dtype == SHREWQ_BF16) return launch_y<false, __nv_bfloat16>(ctx, a, tw, tw, nullptr, 0);
    return launch_y<false, float>(ctx, a, tw, tw, nullptr, 0);
}

}  // namespace shrewq
