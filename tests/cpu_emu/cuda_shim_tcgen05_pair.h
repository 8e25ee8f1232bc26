// Stand-ins for shrew_b200/csrc/ptx_tcgen05_pair.cuh: a thread-block cluster of two blocks (distributed
// shared memory, remote mbarrier arrival, cluster barrier) and the cta_group::2 forms of TMA, tensor-memory
// allocation, tcgen05.mma and tcgen05.commit.  Include after cuda_shim_tcgen05.h; launch with
// emu::launch_cluster2.
//
// TEST INFRASTRUCTURE ONLY.  Unlike the single-CTA model, nothing that has run on a GPU ties this part
// to the hardware yet: it states how this project READS the documentation of cta_group::2 (each CTA
// holds 128 of the 256 accumulator rows and 128 of the 256 rows of B; one instruction issued by the
// leader works on both), and checks the kernel against that reading.
#pragma once

#define SHREWQ_CLUSTER_OF_2

static inline uint32_t cluster_ctarank() { return emu::g_block->rank; }
static inline void cluster_arrive() {}
static inline void cluster_wait() { emu::g_block->cluster_bar->arrive_and_wait(); }  // arrive + wait, always paired in the kernel
static inline uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
    return (smem_u32(emu::g_block->region) + (rank << 18)) | (local_addr & 0x3FFFFu);
}
static inline void mbar_arrive_cluster(uint32_t cluster_addr) { mbar_arrive(cluster_addr); }
static inline void tma_load_2d_pair(uint32_t dst, const void *tmap, int c0, int c1, uint32_t bar_local) {
    tma_load_2d(dst, tmap, c0, c1, map_to_cta(bar_local, 0));  // data here, bytes counted on the leader's barrier
}
static inline void tc_commit_pair(uint32_t bar) {
    const uint32_t b0 = map_to_cta(bar, 0), b1 = map_to_cta(bar, 1);
    if (emu::tc_deferred()) emu::tc_push([=] { mbar_arrive(b0); mbar_arrive(b1); });
    else { mbar_arrive(b0); mbar_arrive(b1); }
}
static inline void tc_alloc_512_pair(uint32_t result_smem) { tc_alloc_512(result_smem); }  // each block: its own tensor memory
static inline void tc_relinquish_pair() {}
static inline void tc_dealloc_512_pair(uint32_t) {}

// tcgen05.mma.cta_group::2.kind::f16: D[256 x N] (+)= A[256 x 16] * B[N x 16]^T issued by one thread of the
// leader.  Rows 128 r .. 128 r + 127 of A and D live in block r's tensor memory (same columns in both);
// rows 128 r .. of B live in block r's shared memory at the descriptor's offset.
static inline void tc_mma_ts_pair_now(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate);
static inline void tc_mma_ts_pair(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    if (emu::tc_deferred()) emu::tc_push([=] { tc_mma_ts_pair_now(d_tmem, a_tmem, b_desc, idesc, accumulate); });
    else tc_mma_ts_pair_now(d_tmem, a_tmem, b_desc, idesc, accumulate);
}
static inline void tc_mma_ts_pair_now(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    emu::Block *me = emu::g_block;
    EMU_CHECK(me->rank == 0, "the leader CTA issues the pair MMA");
    const uint32_t N = ((idesc >> 17) & 0x3Fu) << 3, Mrows = ((idesc >> 24) & 0x1Fu) << 4;
    EMU_CHECK(Mrows == 256 && N == 256, "Mrows == 256 && N == 256");
    const uint32_t a_fmt = (idesc >> 7) & 7u;  // 0 = f16, 1 = bf16
    emu::g_last_a_format = (int)a_fmt;
    EMU_CHECK(((idesc >> 4) & 3u) == 1 && a_fmt <= 1 && ((idesc >> 10) & 7u) == 1, "D f32, A f16 or bf16, B bf16");
    EMU_CHECK(((b_desc >> 61) & 7u) == 2 && ((b_desc >> 46) & 1u) == 1, "128-byte swizzle, descriptor version 1");
    const uint32_t start = (uint32_t)(b_desc & 0x3FFFu) << 4, sbo = (uint32_t)((b_desc >> 32) & 0x3FFFu) << 4;
    const uint32_t dcol = d_tmem & 0xFFFF, acol = a_tmem & 0xFFFF;
    if (!((d_tmem >> 16) == 0 && (a_tmem >> 16) == 0 && dcol + N <= 512 && acol + 8 <= 512 && N == 256 && Mrows == 256)) {
        emu::fail("pair tcgen05.mma operands outside tensor memory or not 256 x 256");
        return;
    }
    std::vector<float> b((size_t)N * 16);
    for (uint32_t n = 0; n < N; ++n) {
        const uint32_t owner = n >> 7, row = n & 127;
        const uint32_t base = smem_u32(me->cluster[owner]->dyn);
        for (uint32_t k = 0; k < 16; ++k) {
            const uint32_t addr = (base | start) + (row >> 3) * sbo + (row & 7) * 128 + k * 2;
            uint16_t h;
            memcpy(&h, emu::smem_ptr(emu::swizzle(addr, 128)), 2);
            b[n * 16 + k] = __uint_as_float((uint32_t)h << 16);
        }
    }
    for (uint32_t r = 0; r < 2; ++r) {
        std::vector<uint32_t> &tm = me->cluster[r]->tmem;
        for (uint32_t m = 0; m < 128; ++m) {
            float a[16];
            for (uint32_t k = 0; k < 16; ++k) {
                const uint32_t w = tm[m * 512 + acol + (k >> 1)];
                const uint32_t h = (k & 1) ? (w >> 16) : (w & 0xFFFF);
                a[k] = a_fmt == 1 ? __uint_as_float(h << 16) : (float)emu_f16_of(h);
            }
            for (uint32_t n = 0; n < N; ++n) {
                double acc = accumulate ? (double)__uint_as_float(tm[m * 512 + dcol + n]) : 0.0;
                for (uint32_t k = 0; k < 16; ++k) acc += (double)a[k] * (double)b[n * 16 + k];
                tm[m * 512 + dcol + n] = __float_as_uint((float)acc);
            }
        }
    }
}
