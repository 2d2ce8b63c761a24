/*
 * bam_exchange.cu -- the exchange steps of the multi-GPU traversals.
 *
 * The reference runs BFS and CC on one GPU (benchmarks/bfs/main.cu:1577-1736,
 * benchmarks/cc/main.cu:1418-1623); it has no counterpart for this file.  Here a graph is sharded
 * by vertex range, every GPU keeps a replica of the label array, and after each level / sweep the
 * ranks exchange what they changed:
 *
 *   compact   one pass over the replica appends this rank's changes -- BFS: the vertices it labelled
 *             in this level; CC: (vertex, label) of every vertex it lowered -- to a send buffer that
 *             the collective library reads in place (warp-aggregated cursor: one atomic per warp);
 *             the buffer's header carries the entry count and the status code of the rank's
 *             controller, so one all-gather of the headers tells every rank how much to expect,
 *             whether the traversal is over and whether any rank has failed;
 *   (all-gather of the payloads by the host, into this GPU's own memory)
 *   apply     one pass over the received entries of the OTHER ranks: BFS stores the level into
 *             unreached vertices (every writer stores the same value), CC takes the minimum and flags
 *             the vertices this rank owns for its next sweep.  Both rules are order independent, so
 *             every rank count gives the same bits.
 *
 * CC also has a dense form for sweeps in which most labels change (an element-wise MIN all-reduce of
 * the replicas by the host): cc_dense_flag then flags the owned vertices whose label fell.
 *
 * These are ordinary kernels on the caller's stream: nothing here waits for another kernel or rank.
 */
#include <cuda_runtime.h>

#include "bam_abi.h"
#include "bam_fused.cuh"

using namespace bam;

#define BAM_XCHG_THREADS 256

static int xchg_grid(uint64_t n)
{
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const uint64_t want = (n + BAM_XCHG_THREADS - 1) / BAM_XCHG_THREADS;
    const uint64_t cap = (uint64_t)sms * 8;
    return (int)(want < 1 ? 1 : (want < cap ? want : cap));
}

/* Append the lanes with keep == true to out[]; one atomic per warp. */
template <typename E>
__device__ __forceinline__ void warp_append(bool keep, E entry, E* out, uint64_t capacity, unsigned long long* cursor)
{
    const uint32_t m = __ballot_sync(0xffffffffu, keep);
    if (m == 0u) return;
    const uint32_t lane = threadIdx.x & 31u;
    unsigned long long base = 0;
    if (lane == (uint32_t)(__ffs(m) - 1)) base = atomicAdd(cursor, (unsigned long long)__popc(m));
    base = __shfl_sync(0xffffffffu, base, __ffs(m) - 1);
    const uint64_t at = base + __popc(m & ((1u << lane) - 1u));
    if (keep && at < capacity) out[at] = entry;
}

__global__ void __launch_bounds__(BAM_XCHG_THREADS)
k_frontier_compact(const uint32_t* __restrict__ label, uint64_t n, uint32_t level_value, uint32_t* out, uint64_t capacity,
                   unsigned long long* hdr, const bam_status_t* status)
{
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x, nthr = (uint64_t)gridDim.x * blockDim.x;
    if (tid == 0) hdr[1] = status ? status->code : 0u;
    for (uint64_t v0 = tid - (threadIdx.x & 31u); v0 < n; v0 += nthr) {
        const uint64_t v = v0 + (threadIdx.x & 31u);
        warp_append<uint32_t>(v < n && label[v] == level_value, (uint32_t)v, out, capacity, hdr);
    }
}

__global__ void __launch_bounds__(BAM_XCHG_THREADS)
k_frontier_apply(uint32_t* label, uint64_t n, uint32_t level_value, const uint32_t* __restrict__ recv, uint64_t stride,
                 const unsigned long long* __restrict__ hdrs, uint32_t world, uint32_t my_rank)
{
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x, nthr = (uint64_t)gridDim.x * blockDim.x;
    for (uint32_t r = 0; r < world; r++) {
        if (r == my_rank) continue;
        const uint64_t cnt = hdrs[2 * r] < stride ? hdrs[2 * r] : stride;
        const uint32_t* seg = recv + (uint64_t)r * stride;
        for (uint64_t k = tid; k < cnt; k += nthr) {
            const uint32_t v = seg[k];
            if (v < n && label[v] == 0xffffffffu) label[v] = level_value;
        }
    }
}

__global__ void __launch_bounds__(BAM_XCHG_THREADS)
k_cc_compact(const unsigned long long* __restrict__ comp, const uint8_t* __restrict__ next_visit, uint64_t n,
             unsigned long long* out, uint64_t capacity, unsigned long long* hdr, const bam_status_t* status)
{
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x, nthr = (uint64_t)gridDim.x * blockDim.x;
    if (tid == 0) hdr[1] = status ? status->code : 0u;
    for (uint64_t v0 = tid - (threadIdx.x & 31u); v0 < n; v0 += nthr) {
        const uint64_t v = v0 + (threadIdx.x & 31u);
        const bool keep = v < n && next_visit[v] != 0;
        const unsigned long long entry = keep ? ((unsigned long long)v << 32) | (comp[v] & 0xffffffffull) : 0ull;
        warp_append<unsigned long long>(keep, entry, out, capacity, hdr);
    }
}

__global__ void __launch_bounds__(BAM_XCHG_THREADS)
k_cc_apply(unsigned long long* comp, uint8_t* next_visit, uint64_t n, uint64_t own_begin, uint64_t own_end,
           const unsigned long long* __restrict__ recv, uint64_t stride, const unsigned long long* __restrict__ hdrs,
           uint32_t world, uint32_t my_rank)
{
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x, nthr = (uint64_t)gridDim.x * blockDim.x;
    for (uint32_t r = 0; r < world; r++) {
        if (r == my_rank) continue;
        const uint64_t cnt = hdrs[2 * r] < stride ? hdrs[2 * r] : stride;
        const unsigned long long* seg = recv + (uint64_t)r * stride;
        for (uint64_t k = tid; k < cnt; k += nthr) {
            const unsigned long long e = seg[k];
            const uint64_t v = e >> 32;
            const unsigned long long lab = e & 0xffffffffull;
            if (v >= n) continue;
            if (*reinterpret_cast<volatile unsigned long long*>(&comp[v]) > lab && atomicMin(&comp[v], lab) > lab &&
                v >= own_begin && v < own_end)
                next_visit[v] = 1;
        }
    }
}

__global__ void __launch_bounds__(BAM_XCHG_THREADS)
k_cc_dense_flag(const unsigned long long* __restrict__ comp, const unsigned long long* __restrict__ before_own, uint8_t* next_visit,
                uint64_t own_begin, uint64_t own_end)
{
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x, nthr = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t v = own_begin + tid; v < own_end; v += nthr)
        if (comp[v] < before_own[v - own_begin]) next_visit[v] = 1;
}

static const bam_status_t* status_of(bam_cache_t pc) { return pc ? pc->d.status : nullptr; }

extern "C" int bam_launch_frontier_compact(bam_cache_t pc, const uint32_t* label_dev, uint64_t n_vertices, uint32_t level_value,
                                           uint32_t* out_dev, uint64_t capacity, uint64_t* hdr_dev, void* stream)
{
    if (!label_dev || !out_dev || !hdr_dev || n_vertices > (1ull << 32)) return BAM_EINVAL;
    if (pc) CK(cudaSetDevice(pc->ctrl->device));
    cudaStream_t s = (cudaStream_t)stream;
    CK(cudaMemsetAsync(hdr_dev, 0, 8, s));
    k_frontier_compact<<<xchg_grid(n_vertices), BAM_XCHG_THREADS, 0, s>>>(label_dev, n_vertices, level_value, out_dev, capacity,
                                                                        reinterpret_cast<unsigned long long*>(hdr_dev), status_of(pc));
    CK(cudaGetLastError());
    return BAM_OK;
}

extern "C" int bam_launch_frontier_apply(uint32_t* label_dev, uint64_t n_vertices, uint32_t level_value, const uint32_t* recv_dev,
                                         uint64_t stride, const uint64_t* hdrs_dev, uint32_t world, uint32_t my_rank, void* stream)
{
    if (!label_dev || !recv_dev || !hdrs_dev || world == 0 || my_rank >= world) return BAM_EINVAL;
    k_frontier_apply<<<xchg_grid(stride * world), BAM_XCHG_THREADS, 0, (cudaStream_t)stream>>>(
        label_dev, n_vertices, level_value, recv_dev, stride, reinterpret_cast<const unsigned long long*>(hdrs_dev), world, my_rank);
    CK(cudaGetLastError());
    return BAM_OK;
}

extern "C" int bam_launch_cc_compact(bam_cache_t pc, const uint64_t* comp_dev, const uint8_t* next_visit_dev, uint64_t n_vertices,
                                     uint64_t* out_pairs_dev, uint64_t capacity, uint64_t* hdr_dev, void* stream)
{
    if (!comp_dev || !next_visit_dev || !out_pairs_dev || !hdr_dev || n_vertices > (1ull << 32)) return BAM_EINVAL;
    if (pc) CK(cudaSetDevice(pc->ctrl->device));
    cudaStream_t s = (cudaStream_t)stream;
    CK(cudaMemsetAsync(hdr_dev, 0, 8, s));
    k_cc_compact<<<xchg_grid(n_vertices), BAM_XCHG_THREADS, 0, s>>>(reinterpret_cast<const unsigned long long*>(comp_dev), next_visit_dev,
                                                                   n_vertices, reinterpret_cast<unsigned long long*>(out_pairs_dev), capacity,
                                                                   reinterpret_cast<unsigned long long*>(hdr_dev), status_of(pc));
    CK(cudaGetLastError());
    return BAM_OK;
}

extern "C" int bam_launch_cc_apply(uint64_t* comp_dev, uint8_t* next_visit_dev, uint64_t n_vertices, uint64_t own_begin, uint64_t own_end,
                                   const uint64_t* recv_pairs_dev, uint64_t stride, const uint64_t* hdrs_dev, uint32_t world,
                                   uint32_t my_rank, void* stream)
{
    if (!comp_dev || !next_visit_dev || !recv_pairs_dev || !hdrs_dev || world == 0 || my_rank >= world || own_begin > own_end ||
        own_end > n_vertices)
        return BAM_EINVAL;
    k_cc_apply<<<xchg_grid(stride * world), BAM_XCHG_THREADS, 0, (cudaStream_t)stream>>>(
        reinterpret_cast<unsigned long long*>(comp_dev), next_visit_dev, n_vertices, own_begin, own_end,
        reinterpret_cast<const unsigned long long*>(recv_pairs_dev), stride, reinterpret_cast<const unsigned long long*>(hdrs_dev), world,
        my_rank);
    CK(cudaGetLastError());
    return BAM_OK;
}

extern "C" int bam_launch_cc_dense_flag(const uint64_t* comp_dev, const uint64_t* before_own_dev, uint8_t* next_visit_dev,
                                        uint64_t own_begin, uint64_t own_end, void* stream)
{
    if (!comp_dev || !before_own_dev || !next_visit_dev || own_begin > own_end) return BAM_EINVAL;
    k_cc_dense_flag<<<xchg_grid(own_end - own_begin), BAM_XCHG_THREADS, 0, (cudaStream_t)stream>>>(
        reinterpret_cast<const unsigned long long*>(comp_dev), reinterpret_cast<const unsigned long long*>(before_own_dev), next_visit_dev,
        own_begin, own_end);
    CK(cudaGetLastError());
    return BAM_OK;
}
