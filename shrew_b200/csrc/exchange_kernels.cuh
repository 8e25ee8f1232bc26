// Device-side barrier between the GPUs that write output slices into each other's buffers.
//
// A sharded layer's kernels store their column slice of y into every rank's copy of the output
// (peer stores over NVLink).  Before a rank may read its copy, every rank's stores must have
// landed; before a rank may overwrite a peer's copy again, that peer must be done reading it.
// Both are the same exchange: "I have finished everything enqueued before this point" told to
// every peer, and a wait until every peer has said the same.
//
// Each rank owns a flag block in memory that all ranks have mapped:
//   word r (r < world)  : the number of the latest barrier rank r has entered, written by rank r
//   word kEpochWord     : this rank's own barrier count, touched only by this rank's barrier kernels
// One launch of 32 threads per barrier: thread 0 advances the local count; thread r writes it
// into word `rank` of peer r's block (release, system scope: everything this GPU wrote before,
// peer stores of earlier kernels included, is visible before the flag is) and then polls word r
// of the local block until it has reached the same count.  The count lives in device memory, so
// a barrier captured in a CUDA graph counts on at every replay.  Flags only grow (compared as a
// wrapping difference), a peer can be at most one barrier ahead.
// The wait is bounded: after the limit the thread records the missing peer in the status block and
// the kernel ends; the host learns of it from shrewq_ctx_synchronize (SHREWQ_ERR_TIMEOUT).  No trap,
// no endless spin.
//
// Device code only: also compiles against the CUDA stand-in of the CPU tests (tests/cpu_emu/), where
// several ranks run as concurrent host threads and a missing rank makes the wait run out.
#pragma once

#include "dests.cuh"
#include "ptx_small.cuh"

namespace shrewq {
namespace {

constexpr int kExchangeMaxWorld = 8;
constexpr int kEpochWord = 32;  // index of the rank's own barrier count inside its flag block
// polls without a pause, then polls with pauses of kExchangeSleepNs: about one second in all
#ifndef SHREWQ_EXCHANGE_FAST_POLLS
#define SHREWQ_EXCHANGE_FAST_POLLS (1u << 12)
#endif
#ifndef SHREWQ_EXCHANGE_SLOW_POLLS
#define SHREWQ_EXCHANGE_SLOW_POLLS (1u << 20)
#endif
constexpr uint32_t kExchangeFastPolls = SHREWQ_EXCHANGE_FAST_POLLS;
constexpr uint32_t kExchangeSlowPolls = SHREWQ_EXCHANGE_SLOW_POLLS;
constexpr uint32_t kExchangeSleepNs = 256;
constexpr unsigned int kTimeoutExchange = 3;  // DeviceStatus::timeout_flag of a barrier that gave up

struct ExchangeArgs {
    uint32_t *flags[kExchangeMaxWorld];  // flag block of every rank as mapped here; [rank] is local memory
    int rank, world;
};

__device__ __forceinline__ bool exchange_reached(const uint32_t *p, uint32_t epoch) {
    return (int32_t)(ld_acquire_sys_u32(p) - epoch) >= 0;
}

__global__ void __launch_bounds__(32) exchange_barrier_kernel(ExchangeArgs a, DeviceStatus *status) {
    // Programmatic dependent launch: the kernel after the barrier may start its prologue now; this kernel says
    // "everything before me is done" only once the kernel before it has completed and its stores are visible.
    pdl_launch_dependents();
    pdl_wait();
    uint32_t *mine = a.flags[a.rank];
    uint32_t epoch = 0;
    if (threadIdx.x == 0) {
        epoch = mine[kEpochWord] + 1;
        mine[kEpochWord] = epoch;
    }
    epoch = __shfl_sync(0xFFFFFFFFu, epoch, 0);  // one warp: no shared memory needed
    const int r = (int)threadIdx.x;
    if (r >= a.world || r == a.rank) return;
    fence_sys();
    st_release_sys_u32(a.flags[r] + a.rank, epoch);
    const uint32_t *from = mine + r;
    for (uint32_t i = 0; i < kExchangeFastPolls; ++i)
        if (exchange_reached(from, epoch)) return;
    for (uint32_t i = 0; i < kExchangeSlowPolls; ++i) {
        if (exchange_reached(from, epoch)) return;
        sleep_ns(kExchangeSleepNs);
    }
    if (atomicCAS(&status->timeout_flag, 0u, kTimeoutExchange) == 0u) {
        status->where = ((unsigned)a.rank << 8) | (unsigned)r;  // (waiting rank, rank that never arrived)
        status->stage = epoch;
        status->parity = ld_acquire_sys_u32(from);
    }
}

}  // namespace
}  // namespace shrewq
