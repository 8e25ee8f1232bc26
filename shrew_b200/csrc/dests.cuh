// Small types shared by the kernels and the host side.
#pragma once

namespace shrewq {

// Extra destinations of a forward: the same output slice is also stored into these buffers
// (peer GPUs' memory, mapped into this process) — the all-gather fused into the epilogue.
constexpr int kMaxPeers = 7;
struct Dests {
    void *p[kMaxPeers];
    int n;
};

// Device-visible record a kernel writes when one of its bounded waits runs out.
struct DeviceStatus {
    unsigned int timeout_flag;  // 0 = fine; otherwise a code naming the wait that gave up
    unsigned int where;         // (blockIdx.x << 8) | role
    unsigned int stage;
    unsigned int parity;
};

// internal epilogue flag (above the public SHREWQ_EPILOGUE_* values): add the f32 value already
// stored at the output position before the elementwise op
constexpr int kEpilogueAccumulate = 0x100;

}  // namespace shrewq
