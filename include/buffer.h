/* buffer.h -- BufferPtr / createBuffer as in the reference's include/buffer.h:31-33, :224-259:
 * reference-counted host (pinned) or device buffers that free themselves.  createDma (DMA windows
 * registered with the kernel module, :175-219 there) has no counterpart: with the emulated
 * controller a bus address is the device virtual address, nothing has to be mapped. */
#ifndef BAM_COMPAT_BUFFER_H
#define BAM_COMPAT_BUFFER_H
#include <cuda_runtime.h>

#include <memory>
#include <stdexcept>
#include <string>

typedef std::shared_ptr<void> BufferPtr;

inline BufferPtr createBuffer(size_t size)
{
    void* p = nullptr;
    cudaError_t e = cudaHostAlloc(&p, size, cudaHostAllocDefault);
    if (e != cudaSuccess) throw std::runtime_error(std::string("Failed to allocate host memory: ") + cudaGetErrorString(e));
    return BufferPtr(p, [](void* q) { cudaFreeHost(q); });
}

/* cudaDevice < 0: pinned host memory; otherwise device memory on that GPU, 64 KiB aligned (queue
 * memory must be, include/buffer.h:90-91 there). */
inline BufferPtr createBuffer(size_t size, int cudaDevice)
{
    if (cudaDevice < 0) return createBuffer(size);
    cudaError_t e = cudaSetDevice(cudaDevice);
    if (e != cudaSuccess) throw std::runtime_error(std::string("Failed to set CUDA device: ") + cudaGetErrorString(e));
    void* base = nullptr;
    const size_t align = 64 * 1024;
    e = cudaMalloc(&base, size + align);
    if (e != cudaSuccess) throw std::runtime_error(std::string("Failed to allocate device memory: ") + cudaGetErrorString(e));
    void* aligned = reinterpret_cast<void*>((reinterpret_cast<uintptr_t>(base) + align - 1) / align * align);
    /* the owner frees the allocation's base, users see the aligned address */
    std::shared_ptr<void> owner(base, [](void* q) { cudaFree(q); });
    return BufferPtr(owner, aligned);
}
#endif
