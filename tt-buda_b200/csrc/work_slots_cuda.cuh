// CUDA side of the work-counter hand-out (work_slots.hpp): one completion event per slot and device.
#pragma once

#include <cuda_runtime.h>

#include <mutex>

#include "buda_common.cuh"
#include "work_slots.hpp"

namespace buda {

constexpr int kCaptureSlots = 256;   // of kWorkSlots: reserved for launches recorded into CUDA graphs

class SlotEvents {
public:
    bool busy(int slot)
    {
        std::lock_guard<std::mutex> lock(mu_);
        return ev_[slot] != nullptr && cudaEventQuery(ev_[slot]) == cudaErrorNotReady;
    }
    void wait(int slot)
    {
        cudaEvent_t e;
        {
            std::lock_guard<std::mutex> lock(mu_);
            e = ev_[slot];
        }
        if (e) (void)cudaEventSynchronize(e);
    }
    cudaError_t mark(int slot, cudaStream_t stream)
    {
        std::lock_guard<std::mutex> lock(mu_);
        if (!ev_[slot]) {
            cudaError_t e = cudaEventCreateWithFlags(&ev_[slot], cudaEventDisableTiming);
            if (e != cudaSuccess) return e;
        }
        return cudaEventRecord(ev_[slot], stream);
    }

private:
    std::mutex mu_;
    cudaEvent_t ev_[kWorkSlots] = {};
};

struct DeviceWorkSlots {
    WorkSlotRing<kWorkSlots, kCaptureSlots> ring;
    SlotEvents events;
};

// Slot for a launch on `stream` of the current device.  *tracked: the slot must be marked and released after the launch
// (false for a launch that is being captured: its slot is never reused).  Negative: no slot can be given.
inline int take_work_slot(DeviceWorkSlots &d, cudaStream_t stream, bool *tracked)
{
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cs) != cudaSuccess) {
        (void)cudaGetLastError();
        cs = cudaStreamCaptureStatusNone;
    }
    if (cs != cudaStreamCaptureStatusNone) {
        *tracked = false;
        return d.ring.acquire_for_capture();
    }
    *tracked = true;
    return d.ring.acquire(d.events);
}

inline void work_slot_launched(DeviceWorkSlots &d, int slot, cudaStream_t stream, bool tracked)
{
    if (!tracked) return;
    (void)d.events.mark(slot, stream);
    d.ring.release(slot);
}

}  // namespace buda
