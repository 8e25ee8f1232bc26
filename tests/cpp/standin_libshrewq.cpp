// Test infrastructure, never shipped: a CPU stand-in for libshrewq.so and for the handful of CUDA
// runtime calls the C++ host mirror (include/shrewq.hpp, shrewq_checkpoint.hpp) makes, so that the
// C++ restatement of the reference's unit tests (test_quantize_api.cpp) and the checkpoint round trip
// can run where there is no GPU.  "Device" memory is host memory; the arithmetic of every entry point
// is the CPU oracle's (oracle/shrew_oracle.c).  What this checks is the host code above the C ABI:
// argument order, shapes, ownership, the file format — not the kernels.
//
// Built by tests/test_cpp_mirror_standin.py as tests/cpp/build/standin/libshrewq.so and linked in place
// of both the real library and libcudart.
#include <cuda_runtime_api.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "shrewq.h"

extern "C" {
// oracle/shrew_oracle.c
int shrew_oracle_quantize_f32(const float *w, size_t rows, size_t cols, int granularity, int8_t *q, double *scales);
void shrew_oracle_dequantize_f32(const int8_t *q, const double *scales, size_t rows, size_t cols, int granularity,
                                 float *out);
void shrew_oracle_dequantize_bf16(const int8_t *q, const double *scales, size_t rows, size_t cols, int granularity,
                                  uint16_t *out);
void shrew_oracle_linear_forward_f32(const int8_t *q, const double *scales, int granularity, const float *bias,
                                     const float *x, size_t M, size_t N, size_t K, int relu, float *y);
uint16_t shrew_oracle_f64_to_bf16(double v);
float shrew_oracle_bf16_to_f32(uint16_t h);
}

struct shrewq_ctx {
    char err[256];
    uint64_t launches;
};
struct shrewq_linear {
    shrewq_ctx *ctx;
    const int8_t *q;
    std::vector<double> scales;
    const float *bias;
    size_t n, k;
    int granularity;
};

static char g_err[256] = "";
static int fail(shrewq_ctx *ctx, int code, const char *msg) {
    snprintf(ctx ? ctx->err : g_err, 256, "%s", msg);
    return code;
}

extern "C" {

// ---- the CUDA runtime calls of the mirror: device memory is host memory ----
cudaError_t cudaSetDevice(int) { return cudaSuccess; }
cudaError_t cudaMalloc(void **p, size_t n) {
    *p = malloc(n ? n : 1);
    return *p ? cudaSuccess : cudaErrorMemoryAllocation;
}
cudaError_t cudaFree(void *p) {
    free(p);
    return cudaSuccess;
}
cudaError_t cudaMemcpy(void *dst, const void *src, size_t n, cudaMemcpyKind) {
    memcpy(dst, src, n);
    return cudaSuccess;
}
cudaError_t cudaMemset(void *p, int v, size_t n) {
    memset(p, v, n);
    return cudaSuccess;
}

// ---- the C ABI entry points the mirror binds ----
int shrewq_ctx_create(int device, void *, shrewq_ctx **out) {
    if (!out || device < 0) return fail(nullptr, SHREWQ_ERR_INVALID_ARG, "ctx_create: bad argument");
    *out = new shrewq_ctx{{0}, 0};
    return SHREWQ_OK;
}
int shrewq_ctx_set_stream(shrewq_ctx *ctx, void *) { return ctx ? SHREWQ_OK : SHREWQ_ERR_INVALID_ARG; }
int shrewq_ctx_synchronize(shrewq_ctx *ctx) { return ctx ? SHREWQ_OK : SHREWQ_ERR_INVALID_ARG; }
void shrewq_ctx_destroy(shrewq_ctx *ctx) { delete ctx; }
const char *shrewq_last_error(const shrewq_ctx *ctx) { return ctx ? ctx->err : g_err; }
const char *shrewq_version(void) { return "cpu stand-in (tests only)"; }
uint64_t shrewq_ctx_launch_count(const shrewq_ctx *ctx) { return ctx ? ctx->launches : 0; }

int shrewq_quantize_f32(shrewq_ctx *ctx, const float *w, size_t rows, size_t cols, int granularity, int8_t *q,
                        double *scales) {
    if (!ctx) return fail(nullptr, SHREWQ_ERR_INVALID_ARG, "quantize: ctx is NULL");
    if (granularity != SHREWQ_PER_TENSOR && granularity != SHREWQ_PER_CHANNEL)
        return fail(ctx, SHREWQ_ERR_INVALID_ARG, "quantize: bad granularity");
    if (!scales || (rows * cols > 0 && (!w || !q))) return fail(ctx, SHREWQ_ERR_INVALID_ARG, "quantize: NULL buffer");
    ctx->launches++;
    return shrew_oracle_quantize_f32(w, rows, cols, granularity, q, scales) == 0 ? SHREWQ_OK : SHREWQ_ERR_ALLOC;
}

int shrewq_dequantize(shrewq_ctx *ctx, const int8_t *q, const double *scales, size_t rows, size_t cols, int granularity,
                      int out_dtype, void *out) {
    if (!ctx) return fail(nullptr, SHREWQ_ERR_INVALID_ARG, "dequantize: ctx is NULL");
    if (rows * cols > 0 && (!q || !scales || !out)) return fail(ctx, SHREWQ_ERR_INVALID_ARG, "dequantize: NULL buffer");
    if (out_dtype == SHREWQ_F32) shrew_oracle_dequantize_f32(q, scales, rows, cols, granularity, static_cast<float *>(out));
    else if (out_dtype == SHREWQ_BF16)
        shrew_oracle_dequantize_bf16(q, scales, rows, cols, granularity, static_cast<uint16_t *>(out));
    else return fail(ctx, SHREWQ_ERR_INVALID_ARG, "dequantize: bad out_dtype");
    ctx->launches++;
    return SHREWQ_OK;
}

int shrewq_linear_create(shrewq_ctx *ctx, const int8_t *q, const double *scales, const float *bias, size_t n, size_t k,
                         int granularity, shrewq_linear **out) {
    if (!ctx) return fail(nullptr, SHREWQ_ERR_INVALID_ARG, "linear_create: ctx is NULL");
    if (!out) return fail(ctx, SHREWQ_ERR_INVALID_ARG, "linear_create: out is NULL");
    *out = nullptr;
    if (!q || !scales || n == 0 || k == 0) return fail(ctx, SHREWQ_ERR_INVALID_ARG, "linear_create: bad argument");
    // like the library, the handle keeps q and bias by pointer and copies the scales
    *out = new shrewq_linear{ctx, q, std::vector<double>(scales, scales + (granularity == SHREWQ_PER_CHANNEL ? n : 1)),
                             bias, n, k, granularity};
    return SHREWQ_OK;
}
void shrewq_linear_destroy(shrewq_linear *lin) { delete lin; }
size_t shrewq_linear_in_features(const shrewq_linear *lin) { return lin ? lin->k : 0; }
size_t shrewq_linear_out_features(const shrewq_linear *lin) { return lin ? lin->n : 0; }
size_t shrewq_linear_memory_savings_bytes(const shrewq_linear *lin) { return lin ? lin->n * lin->k * 3 : 0; }
const char *shrewq_linear_last_kernel(const shrewq_linear *) { return "cpu stand-in"; }

int shrewq_linear_forward(shrewq_linear *lin, const void *x, int x_dtype, size_t M, void *y, int y_dtype, size_t ldy,
                          int epilogue) {
    if (!lin) return fail(nullptr, SHREWQ_ERR_INVALID_ARG, "forward: handle is NULL");
    if (M == 0) return SHREWQ_OK;
    if (!x || !y || ldy < lin->n) return fail(lin->ctx, SHREWQ_ERR_INVALID_ARG, "forward: bad argument");
    std::vector<float> xf(M * lin->k), yf(M * lin->n);
    for (size_t i = 0; i < xf.size(); ++i)
        xf[i] = x_dtype == SHREWQ_BF16 ? shrew_oracle_bf16_to_f32(static_cast<const uint16_t *>(x)[i])
                                       : static_cast<const float *>(x)[i];
    shrew_oracle_linear_forward_f32(lin->q, lin->scales.data(), lin->granularity, lin->bias, xf.data(), M, lin->n, lin->k,
                                    epilogue == SHREWQ_EPILOGUE_RELU, yf.data());
    for (size_t m = 0; m < M; ++m)
        for (size_t n = 0; n < lin->n; ++n) {
            if (y_dtype == SHREWQ_BF16) static_cast<uint16_t *>(y)[m * ldy + n] = shrew_oracle_f64_to_bf16(yf[m * lin->n + n]);
            else static_cast<float *>(y)[m * ldy + n] = yf[m * lin->n + n];
        }
    lin->ctx->launches++;
    return SHREWQ_OK;
}

}  // extern "C"
