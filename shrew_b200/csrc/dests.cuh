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

}  // namespace shrewq
