/* event.h -- CUDA-event timer with the interface of the reference's include/event.h:13-51. */
#ifndef BAM_COMPAT_EVENT_H
#define BAM_COMPAT_EVENT_H
#include <cuda_runtime.h>
#include <stdexcept>
struct Event {
    cudaEvent_t event;
    explicit Event(cudaStream_t stream = 0)
    {
        if (cudaEventCreate(&event) != cudaSuccess) throw std::runtime_error("Failed to create event");
        if (cudaEventRecord(event, stream) != cudaSuccess) throw std::runtime_error("Failed to record event");
    }
    ~Event() { cudaEventDestroy(event); }
    /* elapsed microseconds from `other` to this event */
    double operator-(const Event& other) const
    {
        float ms = 0;
        cudaEventSynchronize(event);
        if (cudaEventElapsedTime(&ms, other.event, event) != cudaSuccess) throw std::runtime_error("Failed to read event time");
        return (double)ms * 1e3;
    }
};
#endif
