/*
 * bam_noalloc.cu -- bam_cache_audit_noalloc: the cache audit for callers that must not allocate.
 *
 * bam_cache_audit (bam_lib.cu) obtains its violation counter with cudaMalloc, frees it with
 * cudaFree and synchronises the whole device around the kernel.  That is fine for a test, but
 * some users of this library cannot afford it:
 *   - a service that audits the cache between launches while other streams keep the GPU busy:
 *     cudaMalloc/cudaFree serialise against all work on the device and stall those streams;
 *   - a process whose device memory is owned by one allocator (a framework's caching allocator,
 *     a fixed arena carved at start-up) and that forbids stray driver allocations, or that runs
 *     so close to the memory limit that an allocation may fail at the worst moment;
 *   - code on a path where allocation calls are not permitted at all, such as work being
 *     recorded into a stream for later replay.
 * For them this file holds the audit's scratch in a fixed array that lives in the library's
 * device image: BAM_AUDIT_NOALLOC_WORDS 64-bit words = 8 KiB on every GPU that loads the library,
 * kept until the process exits.  The entry point only enqueues a memset and a kernel on the
 * caller's stream: no cudaMalloc, no cudaFree, no synchronisation, no allocating library call.
 *
 * The array's name is only meaningful in device code.  Host code in this file asks the runtime
 * for the array's device address once per device (cudaGetSymbolAddress, with that device
 * current) and hands that address to the kernel.
 */
#include <cuda_runtime.h>

#include <mutex>

#include "bam_abi.h"
#include "bam/array.cuh"
#include "bam_internal.h"

using namespace bam;

/* Layout of the scratch: word 0 counts blocks that have finished; word 1+b is the number of
 * violations block b found.  Block b audits BAM_AUDIT_NOALLOC_SLOTS_PER_BLOCK cache slots and
 * an equal share of the page-table buckets, so the largest cache this entry point accepts has
 * (BAM_AUDIT_NOALLOC_WORDS - 1) * BAM_AUDIT_NOALLOC_SLOTS_PER_BLOCK = 8,380,416 slots. */
static __device__ __align__(256) unsigned long long g_audit_scratch[BAM_AUDIT_NOALLOC_WORDS];

__global__ void __launch_bounds__(256)
k_audit_fixed_scratch(page_cache_d_t pc, uint64_t n_buckets, uint64_t buckets_per_block,
                      unsigned long long* scratch, unsigned long long* violations_out)
{
    __shared__ unsigned long long s_part[8];
    __shared__ bool s_last;
    unsigned long long bad = 0;

    /* the same invariants bam_cache_audit checks: no pin left, no fill or eviction in progress,
     * tag and VALID bit agree, every resident page is found through the table ... */
    const uint64_t s0 = (uint64_t)blockIdx.x * BAM_AUDIT_NOALLOC_SLOTS_PER_BLOCK;
    uint64_t s1 = s0 + BAM_AUDIT_NOALLOC_SLOTS_PER_BLOCK;
    if (s1 > pc.n_slots) s1 = pc.n_slots;
    for (uint64_t s = s0 + threadIdx.x; s < s1; s += blockDim.x) {
        const uint32_t st = pc.slots[s].state;
        const uint64_t tag = pc.slots[s].tag;
        if (st & BAM_CNT_MASK) bad++;
        if (st & BAM_BUSY) bad++;
        if ((st & BAM_VALID) && tag == BAM_TAG_NONE) bad++;
        if (!(st & BAM_VALID) && tag != BAM_TAG_NONE) bad++;
        if (st & BAM_VALID) {
            const uint64_t h = pt_hash(tag);
            if (pt_lookup(pc, tag, (uint32_t)h & pc.bucket_mask, (uint32_t)(h >> 56)) != (uint32_t)s) bad++;
        }
    }
    /* ... and every table entry points at a slot whose tag has the entry's fingerprint */
    const uint64_t b0 = (uint64_t)blockIdx.x * buckets_per_block;
    uint64_t b1 = b0 + buckets_per_block;
    if (b1 > n_buckets) b1 = n_buckets;
    for (uint64_t b = b0 + threadIdx.x; b < b1; b += blockDim.x) {
        const uint32_t* w = pc.table + b * BAM_BUCKET_WORDS;
        if (w[0] & BAM_BUCKET_LOCK) bad++;
        for (int i = 1; i < BAM_BUCKET_WORDS; i++) {
            if (w[i] == BAM_ENTRY_EMPTY) continue;
            const uint32_t s = w[i] & 0xffffffu;
            if (s >= pc.n_slots) { bad++; continue; }
            const uint64_t tag = pc.slots[s].tag;
            if (tag == BAM_TAG_NONE || (uint32_t)(pt_hash(tag) >> 56) != (w[i] >> 24)) bad++;
        }
    }

    /* block total -> this block's scratch word */
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) bad += __shfl_xor_sync(0xffffffffu, bad, o);
    if ((threadIdx.x & 31u) == 0u) s_part[threadIdx.x >> 5] = bad;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long t = 0;
        for (uint32_t w = 0; w < (blockDim.x >> 5); w++) t += s_part[w];
        scratch[1 + blockIdx.x] = t;
        __threadfence();
        s_last = (atomicAdd(&scratch[0], 1ull) == (unsigned long long)gridDim.x - 1ull);
    }
    __syncthreads();
    /* the block that finishes last adds the per-block words up and writes the result */
    if (s_last) {
        __threadfence();
        unsigned long long t = 0;
        for (uint32_t b = threadIdx.x; b < gridDim.x; b += blockDim.x)
            t += *reinterpret_cast<volatile unsigned long long*>(&scratch[1 + b]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        __syncthreads();
        if ((threadIdx.x & 31u) == 0u) s_part[threadIdx.x >> 5] = t;
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned long long sum = 0;
            for (uint32_t w = 0; w < (blockDim.x >> 5); w++) sum += s_part[w];
            *violations_out = sum;
        }
    }
}

/* Device address of g_audit_scratch on each device, looked up on first use. */
#define BAM_NOALLOC_MAX_DEVICES 64
static std::mutex g_scratch_mu;
static unsigned long long* g_scratch_addr[BAM_NOALLOC_MAX_DEVICES];

static int scratch_address(int device, unsigned long long** out)
{
    if (device < 0 || device >= BAM_NOALLOC_MAX_DEVICES) return BAM_EINVAL;
    std::lock_guard<std::mutex> lock(g_scratch_mu);
    if (!g_scratch_addr[device]) {
        void* p = nullptr;
        /* `device` is current here (the caller set it); the symbol's name is not an address the
         * GPU can use, the runtime translates it to one */
        cudaError_t e = cudaGetSymbolAddress(&p, g_audit_scratch);
        if (e != cudaSuccess || !p) { (void)cudaGetLastError(); return BAM_ECUDA; }
        g_scratch_addr[device] = static_cast<unsigned long long*>(p);
    }
    *out = g_scratch_addr[device];
    return BAM_OK;
}

extern "C" int bam_cache_audit_noalloc(bam_cache_t pc, uint64_t* violations_out_dev, void* stream)
{
    if (!pc || !violations_out_dev) return BAM_EINVAL;
    if (pc->d.n_slots > BAM_AUDIT_NOALLOC_MAX_SLOTS) return BAM_E2BIG;      /* beyond the fixed scratch */
    if (cudaSetDevice(pc->ctrl->device) != cudaSuccess) { (void)cudaGetLastError(); return BAM_ECUDA; }
    unsigned long long* scratch = nullptr;
    int rc = scratch_address(pc->ctrl->device, &scratch);
    if (rc != BAM_OK) return rc;
    const uint32_t n_blocks = (uint32_t)((pc->d.n_slots + BAM_AUDIT_NOALLOC_SLOTS_PER_BLOCK - 1) / BAM_AUDIT_NOALLOC_SLOTS_PER_BLOCK);
    const uint64_t buckets_per_block = (pc->n_buckets + n_blocks - 1) / n_blocks;
    cudaStream_t s = (cudaStream_t)stream;
    /* the array still holds the previous call's counter and partial sums: clear what this call uses */
    if (cudaMemsetAsync(scratch, 0, (size_t)(1 + n_blocks) * sizeof(unsigned long long), s) != cudaSuccess) {
        (void)cudaGetLastError();
        return BAM_ECUDA;
    }
    k_audit_fixed_scratch<<<n_blocks, 256, 0, s>>>(pc->d, pc->n_buckets, buckets_per_block, scratch,
                                                    reinterpret_cast<unsigned long long*>(violations_out_dev));
    if (cudaGetLastError() != cudaSuccess) return BAM_ECUDA;
    return BAM_OK;
}
