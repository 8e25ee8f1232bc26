// Extra destinations of a forward: the same output slice is also stored into these buffers
// (peer GPUs' memory, mapped into this process) — the all-gather fused into the epilogue.
#pragma once

namespace shrewq {

constexpr int kMaxPeers = 7;
struct Dests {
    void *p[kMaxPeers];
    int n;
};

}  // namespace shrewq
