#pragma once
// Set-up that CUDA keeps per device (a kernel's opt-in to large dynamic shared
// memory, for one) must be repeated on every GPU a process drives, not once per
// process. One bit per device ordinal records where it has been done.

#include <atomic>

namespace mcd {

class PerDeviceOnce {
public:
    // True the first time it is asked about `device` (and again after forget): the caller then does the set-up.
    // Ordinals outside 0..63 are never remembered, so their set-up simply repeats.
    bool first_use(int device) {
        if (device < 0 || device >= 64) return true;
        const unsigned long long bit = 1ull << device;
        return (done_.fetch_or(bit, std::memory_order_acq_rel) & bit) == 0;
    }
    // After a failed set-up: the next launch on `device` tries again.
    void forget(int device) {
        if (device >= 0 && device < 64) done_.fetch_and(~(1ull << device), std::memory_order_acq_rel);
    }

private:
    std::atomic<unsigned long long> done_{0};
};

}  // namespace mcd
