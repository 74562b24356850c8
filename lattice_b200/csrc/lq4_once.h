// Per-device "done once" bookkeeping for kernel attributes (host code, no CUDA types).
//
// cudaFuncSetAttribute(..., MaxDynamicSharedMemorySize, ...) applies to ONE device (the current
// primary context), so a process that drives several GPUs has to opt in once per device, not
// once per process.  One DeviceOnce per kernel instantiation remembers which devices are done;
// it is safe to call from several host threads (a lost race only repeats the cheap opt-in).
#pragma once

#include <atomic>
#include <cstdint>

namespace lq4 {

struct DeviceOnce {
    static constexpr int kMaxDevices = 256;
    std::atomic<uint64_t> bits[kMaxDevices / 64];

    constexpr DeviceOnce() : bits{} {}

    // True if `device` still needs the one-time call (devices outside the table always do).
    bool needs(int device) const {
        if (device < 0 || device >= kMaxDevices) return true;
        return ((bits[device >> 6].load(std::memory_order_acquire) >> (device & 63)) & 1u) == 0;
    }
    void mark(int device) {
        if (device < 0 || device >= kMaxDevices) return;
        bits[device >> 6].fetch_or(uint64_t(1) << (device & 63), std::memory_order_release);
    }
    void reset() {
        for (auto& b : bits) b.store(0, std::memory_order_release);
    }
};

}  // namespace lq4
