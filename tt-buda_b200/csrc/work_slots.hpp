// Hand-out of the device work counters that the staged pack / unpack kernels draw their items from.
//
// A launch takes one counter ("slot"); its CTAs share it and the CTA that leaves last zeroes it.  Two launches must
// therefore never hold the same slot at the same time.  The ring below makes that impossible for ordinary launches:
// a slot is given out again only after the launch that used it last is known to have finished (the backend keeps one
// completion marker per slot -- a CUDA event in the library, a fake in the unit test; between acquire() and release()
// the slot is "in hand" and skipped by everyone else).  Launches that are being
// recorded into a CUDA graph cannot be tracked with events (a graph may be replayed any number of times, later), so
// they take their slots from a reserved range, each of which is given out once per process; when that range is used
// up the launch is refused instead of sharing.  What remains the caller's duty: not to replay one captured graph
// concurrently with itself.
//
// Pure C++ (no CUDA types) so that the hand-out logic can be tested without a GPU.
#pragma once

#include <mutex>

namespace buda {

// Backend: bool busy(int slot)   -- the launch that last used `slot` may still be running
//          void wait(int slot)   -- block until it has finished
template <int kSlots, int kCaptureSlots>
class WorkSlotRing {
    static_assert(kCaptureSlots >= 0 && kCaptureSlots < kSlots, "reserved range must leave ordinary slots");

public:
    static constexpr int kOrdinary = kSlots - kCaptureSlots;

    // Slot for an ordinary launch: the next slot of the ring that is free.  Busy slots are skipped; if one full turn
    // finds every slot busy, waits for the one the ring points at (the oldest).
    template <class Backend>
    int acquire(Backend &b)
    {
        std::lock_guard<std::mutex> lock(mu_);
        for (int tries = 0; tries < kOrdinary; tries++) {
            const int slot = next_;
            next_ = (next_ + 1) % kOrdinary;
            if (in_hand_[slot]) continue;   // taken, its launch not yet issued and marked
            if (!used_[slot] || !b.busy(slot)) {
                used_[slot] = in_hand_[slot] = true;
                return slot;
            }
        }
        // every slot busy: wait for the oldest that is not in another thread's hands
        for (int tries = 0; tries < kOrdinary; tries++) {
            const int slot = next_;
            next_ = (next_ + 1) % kOrdinary;
            if (in_hand_[slot]) continue;
            b.wait(slot);
            in_hand_[slot] = true;
            return slot;
        }
        return -1;   // more threads inside a launch at once than there are slots
    }

    // The launch that took `slot` has been issued and its completion marker recorded.
    void release(int slot)
    {
        std::lock_guard<std::mutex> lock(mu_);
        if (slot >= 0 && slot < kOrdinary) in_hand_[slot] = false;
    }

    // Slot for a launch that is being captured into a graph: never handed out twice.  -1 when the range is used up.
    int acquire_for_capture()
    {
        std::lock_guard<std::mutex> lock(mu_);
        if (captured_ >= kCaptureSlots) return -1;
        return kOrdinary + captured_++;
    }

    int captured() const { return captured_; }

private:
    std::mutex mu_;
    int next_ = 0;
    int captured_ = 0;
    bool used_[kSlots] = {};
    bool in_hand_[kSlots] = {};
};

}  // namespace buda
