// Internal declarations shared by the translation units of libshrewq.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdarg>
#include <vector>
#include <cstdio>
#include <cstring>

#include "../../include/shrewq.h"
#include "dests.cuh"

namespace shrewq {

constexpr int kErrLen = 512;

// Launch options of a context (shrewq_ctx_set_option); the defaults are the measured choices.
struct Tuning {
    int tc_groups = 3;      // converter groups of the tcgen05 kernel (1..3)
    int tc_splitk = 1;      // split K when the tile grid leaves SMs idle
    int tc_tok = 0;         // 0 = choose; else force the token tile (16, 32, 64, 128, 256)
    int tc_tok_gated = 0;   // the same for gate/up launches only
    int tc_tailsplit = 0;   // a short last wave as a second launch split along K: 0 = pair kernel, tails up to a quarter wave; 1 = always; 2 = never
    int tc_pair = 1;        // CTA pairs (tcgen05.mma.cta_group::2) for large batches: 0 never, 1 where they win, 2 whenever M > 128
    int ring_stages = 0;    // stages of the ring kernel: 0 = by grid size, 2 or 3 forced
    int pdl = 1;            // programmatic dependent launch of the forward kernels (after a handle's first forward)
};

}  // namespace shrewq

// Opaque in the ABI.
struct shrewq_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    int sm_count = 0;
    char err[shrewq::kErrLen] = {0};
    std::atomic<uint64_t> launches{0};
    shrewq::Tuning tuning;
    // scratch: per-tensor amax word, split-K partial sums and tile counters
    void *scratch = nullptr;
    size_t scratch_bytes = 0;
    // split-K tile counters live in scratch; they are zeroed once and reset by the kernels
    bool counters_zeroed = false;
    // the gated block's host-buffer entry point: two staging slots and two copy streams, so that the copies of
    // one call overlap the kernels of its neighbours (created on first use)
    cudaStream_t copy_in = nullptr, copy_out = nullptr;
    cudaEvent_t ev_in[2] = {nullptr, nullptr}, ev_cmp[2] = {nullptr, nullptr}, ev_out[2] = {nullptr, nullptr};
    void *mlp_stage = nullptr;
    size_t mlp_stage_bytes = 0;
    uint64_t mlp_calls = 0;
    // staging for the *_host entry points
    void *stage_dev = nullptr;
    size_t stage_dev_bytes = 0;
    void *stage_pinned = nullptr;
    size_t stage_pinned_bytes = 0;
    // bf16 hi/lo split of f32 activations (tensor-core route for f32 inputs)
    void *xsplit = nullptr;
    size_t xsplit_bytes = 0;
    // f32 [M,N] accumulators + per-token activation sums of a forward through zero points
    void *ytmp = nullptr;
    size_t ytmp_bytes = 0;
    // Workspaces that were outgrown: kept until the context is destroyed, because a CUDA graph captured earlier
    // still launches kernels with their addresses (device pointers, and pinned host pointers with the flag set)
    std::vector<std::pair<void *, bool>> retired;
    // device status block + pinned mirror
    shrewq::DeviceStatus *dev_status = nullptr;
};

struct shrewq_linear {
    shrewq_ctx *ctx = nullptr;
    const int8_t *q = nullptr;
    const float *bias = nullptr;
    float *scales_f32 = nullptr;  // owned, out_features entries (per-tensor scale broadcast)
    float *czp = nullptr;         // owned, scale * zero_point per output channel; null = symmetric
    bool int4_packed = false;     // q points at packed INT4 rows (in_features / 2 bytes each)
    size_t n = 0, k = 0;
    int granularity = 0;
    // TMA descriptors for the INT8 weight matrix (128 B each, opaque CUtensorMap), valid when
    // tmap_ok: 64-byte k boxes over 128 weight rows, and over 64 rows (gate / up halves).
    alignas(64) unsigned char w_tmap[128];
    alignas(64) unsigned char w_tmap64[128];
    bool tmap_ok = false;
    // a forward of this handle has been enqueued: its weights, scales and bias are then older than every later
    // kernel of the stream, which is what lets later small-batch forwards prefetch them early
    std::atomic<bool> forwarded{false};
};

namespace shrewq {

int set_err(shrewq_ctx *ctx, int code, const char *fmt, ...);
int ensure_scratch(shrewq_ctx *ctx, size_t bytes);
int ensure_stage(shrewq_ctx *ctx, size_t dev_bytes, size_t pinned_bytes);

#define SHREWQ_CUDA_TRY(ctx, expr)                                                         \
    do {                                                                                   \
        cudaError_t e__ = (expr);                                                          \
        if (e__ != cudaSuccess)                                                            \
            return shrewq::set_err((ctx), SHREWQ_ERR_CUDA, "%s failed: %s", #expr,          \
                                   cudaGetErrorString(e__));                               \
    } while (0)

// Launch with or without programmatic stream serialization (the attribute lets the kernel start while the previous
// kernel of the stream still runs; the kernels wait for it before they touch anything but weights).
template <typename Kern, typename... Args>
inline cudaError_t launch_maybe_pdl(Kern kern, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, bool pdl, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, args...);
}

// ---- launchers implemented in the kernel translation units -------------------------
int launch_quantize_batch(shrewq_ctx *ctx, const shrewq_quant_item *items, size_t n_items, int granularity);
int launch_quantize(shrewq_ctx *ctx, const float *w, size_t rows, size_t cols, int granularity,
                    int8_t *q, double *scales);
int launch_absmax(shrewq_ctx *ctx, const float *w, size_t n, float *amax_dev);
int launch_quantize_given_amax(shrewq_ctx *ctx, const float *w, size_t n, const float *amax_dev, int8_t *q, double *scale);
int launch_dequantize(shrewq_ctx *ctx, const int8_t *q, const double *scales, size_t rows,
                      size_t cols, int granularity, int out_dtype, void *out);
int launch_scales_to_f32(shrewq_ctx *ctx, const double *scales, int granularity, size_t n, float *out);
int launch_split_f32(shrewq_ctx *ctx, const float *x, size_t n, void *hi_bf16, void *lo_bf16);
int ensure_xsplit(shrewq_ctx *ctx, size_t bytes);
int launch_quantize_ex(shrewq_ctx *ctx, const float *w, size_t rows, size_t cols, int granularity, int bits, int mode,
                       int8_t *q, double *scales, double *zps);
int launch_quantize_any(shrewq_ctx *ctx, const void *w, int w_dtype, size_t rows, size_t cols, int granularity, int bits,
                        int mode, int8_t *q, double *scales, double *zps);
int launch_dequantize_ex(shrewq_ctx *ctx, const int8_t *q, const double *scales, const double *zps, size_t rows,
                         size_t cols, int granularity, int out_dtype, void *out);
int launch_scale_zp_to_f32(shrewq_ctx *ctx, const double *scales, const double *zps, int granularity, size_t n, float *out);
int launch_row_sums(shrewq_ctx *ctx, const void *x, int x_dtype, size_t M, size_t K, float *sums);
int launch_zero_point_fix(shrewq_ctx *ctx, const float *acc, const float *czp, const float *xsum, size_t M, size_t N,
                          size_t ldy, int relu, int y_dtype, void *y);


struct ForwardArgs {
    const int8_t *q;       // [N,K]
    const float *scales;   // [N] f32
    const float *bias;     // [N] or null
    const void *x;         // [M,K]
    int x_dtype;
    void *y;               // [M, ldy]
    int y_dtype;
    size_t M, N, K, ldy;
    int epilogue;
    // gate/up fusion: when q_up != null the output is silu(gate)*up
    const int8_t *q_up = nullptr;
    const float *scales_up = nullptr;
    const float *bias_up = nullptr;
    Dests extra = {{nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr}, 0};
    // launch with programmatic stream serialization: the kernel may fetch WEIGHTS before the previous kernel of the
    // stream has completed (set only when the weights are known to be older than that kernel)
    bool pdl = false;
};

int launch_gemv(shrewq_ctx *ctx, const ForwardArgs &a);
int launch_gemm_simt(shrewq_ctx *ctx, const ForwardArgs &a);
bool gemv_mma_supported(const ForwardArgs &a);
int launch_gemv_mma(shrewq_ctx *ctx, const ForwardArgs &a);
bool gemv_ring_supported(const ForwardArgs &a);
int launch_gemv_ring(shrewq_ctx *ctx, const ForwardArgs &a);
bool gemv_mma_w4_supported(const ForwardArgs &a);
int launch_gemv_mma_w4(shrewq_ctx *ctx, const ForwardArgs &a);
int launch_pack_int4(shrewq_ctx *ctx, const int8_t *q, size_t n_pairs, uint8_t *packed);
bool tcgen05_supported(const ForwardArgs &a);
int launch_gemm_tcgen05(shrewq_ctx *ctx, const ForwardArgs &a, const void *w_tmap, const void *w_up_tmap);
int plan_gemm_tcgen05(size_t M, size_t N, size_t K, bool gated, int sm_count, int *tok, int *n_tiles, int *m_tiles,
                      int *splits, int *rounds_per_split);
int launch_gemm_tcgen05_2cta(shrewq_ctx *ctx, const ForwardArgs &a, const void *w_tmap, const void *w_up_tmap);
int launch_gemm_tcgen05_noalloc(shrewq_ctx *ctx, const ForwardArgs &a, const void *w_tmap);
int launch_gemm_tcgen05_xsplit(shrewq_ctx *ctx, const ForwardArgs &a, const void *w_tmap);
int encode_weight_tmap(shrewq_ctx *ctx, const int8_t *q, size_t n, size_t k, int box_rows, void *tmap_out);

// bf16 <-> f32 helpers usable on host and device
__host__ __device__ inline float bf16_bits_to_float(uint16_t h) {
    uint32_t b = (uint32_t)h << 16;
    float f;
    memcpy(&f, &b, 4);
    return f;
}

}  // namespace shrewq
