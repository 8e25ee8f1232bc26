// CPU run of the device barrier between GPUs (shrew_b200/csrc/exchange_kernels.cuh): every rank is a host
// thread that launches the barrier kernel `rounds` times on flag blocks in ordinary memory, writing a
// payload word into every rank's buffer before each barrier and checking what it reads after it.  A rank
// listed as absent never launches anything, which is how a wait is made to run out (compile with small
// SHREWQ_EXCHANGE_*_POLLS).  TEST INFRASTRUCTURE ONLY; see cuda_shim.h.
#include "cuda_shim.h"
#include "../../shrew_b200/csrc/exchange_kernels.cuh"

using namespace shrewq;

// Returns 0 when every present rank passed every barrier and read what its peers wrote before it;
// 1 when some rank read stale data after a barrier; 2 when a wait gave up (status[r] then holds the
// record of rank r).  delay_us[r]: pause of rank r before each of its barriers (ranks arrive out of step).
extern "C" int emu_exchange_run(int world, int rounds, const int *absent, const int *delay_us, DeviceStatus *status) {
    std::vector<std::vector<uint32_t>> flags(world, std::vector<uint32_t>(64, 0u));
    std::vector<std::vector<uint32_t>> payload(world, std::vector<uint32_t>(world, 0u));  // payload[dst][src]
    std::atomic<int> stale{0};
    std::vector<std::thread> ranks;
    for (int r = 0; r < world; ++r) {
        status[r] = DeviceStatus{0, 0, 0, 0};
        if (absent[r]) continue;
        ranks.emplace_back([&, r] {
            ExchangeArgs a{};
            a.rank = r;
            a.world = world;
            for (int p = 0; p < world; ++p) a.flags[p] = flags[p].data();
            for (int it = 1; it <= rounds; ++it) {
                for (int p = 0; p < world; ++p) __atomic_store_n(&payload[p][r], (uint32_t)it, __ATOMIC_RELAXED);  // "peer stores"
                if (delay_us[r]) std::this_thread::sleep_for(std::chrono::microseconds(delay_us[r]));
                emu::launch(1, 32, [&] { exchange_barrier_kernel(a, &status[r]); });
                if (status[r].timeout_flag) return;
                for (int p = 0; p < world; ++p)
                    if (!absent[p] && (int)__atomic_load_n(&payload[r][p], __ATOMIC_RELAXED) < it) stale.fetch_add(1);
            }
        });
    }
    for (auto &t : ranks) t.join();
    for (int r = 0; r < world; ++r)
        if (status[r].timeout_flag) return 2;
    return stale.load() ? 1 : 0;
}
