// Host side of the device barrier between GPUs (device code and its description: exchange_kernels.cuh).
#include <new>

#include "common.cuh"
#include "exchange_kernels.cuh"

struct shrewq_exchange {
    shrewq_ctx *ctx = nullptr;
    shrewq::ExchangeArgs args{};
};

using namespace shrewq;

extern "C" {

int shrewq_exchange_create(shrewq_ctx *ctx, int rank, int world, void *const *flag_blocks_dev, shrewq_exchange **out) {
    if (!ctx) return set_err(nullptr, SHREWQ_ERR_INVALID_ARG, "exchange_create: ctx is NULL");
    if (!out) return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "exchange_create: out is NULL");
    *out = nullptr;
    if (world < 1 || world > kExchangeMaxWorld || rank < 0 || rank >= world)
        return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "exchange_create: need 1 <= world <= %d and 0 <= rank < world",
                       kExchangeMaxWorld);
    if (!flag_blocks_dev) return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "exchange_create: flag_blocks_dev is NULL");
    shrewq_exchange *ex = new (std::nothrow) shrewq_exchange();
    if (!ex) return set_err(ctx, SHREWQ_ERR_ALLOC, "out of host memory");
    ex->ctx = ctx;
    ex->args.rank = rank;
    ex->args.world = world;
    for (int r = 0; r < world; ++r) {
        if (!flag_blocks_dev[r] || (reinterpret_cast<uintptr_t>(flag_blocks_dev[r]) & 3)) {
            delete ex;
            return set_err(ctx, SHREWQ_ERR_INVALID_ARG, "exchange_create: flag block %d is NULL or not 4-byte aligned", r);
        }
        ex->args.flags[r] = static_cast<uint32_t *>(flag_blocks_dev[r]);
    }
    *out = ex;
    return SHREWQ_OK;
}

int shrewq_exchange_barrier(shrewq_exchange *ex) {
    if (!ex) return set_err(nullptr, SHREWQ_ERR_INVALID_ARG, "exchange_barrier: handle is NULL");
    shrewq_ctx *ctx = ex->ctx;
    SHREWQ_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    // with programmatic stream serialization the barrier kernel may start (and let ITS successor start its prologue)
    // while the kernel before it still runs; it signals nothing before that kernel has completed
    SHREWQ_CUDA_TRY(ctx, launch_maybe_pdl(exchange_barrier_kernel, dim3(1), dim3(32), (size_t)0, ctx->stream, ctx->tuning.pdl != 0,
                                          ex->args, ctx->dev_status));
    ctx->launches += 1;
    SHREWQ_CUDA_TRY(ctx, cudaGetLastError());
    return SHREWQ_OK;
}

void shrewq_exchange_destroy(shrewq_exchange *ex) { delete ex; }

}  // extern "C"
