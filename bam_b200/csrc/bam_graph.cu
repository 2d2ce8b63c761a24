/*
 * bam_graph.cu -- graph consumers of bam::array: level-synchronous BFS and label-propagation
 * connected components over a CSR graph whose row offsets AND column indices live in the backing
 * store and are read only through the page cache.
 *
 * Reference kernels: benchmarks/bfs/main.cu:658-689 and benchmarks/cc/main.cu:123-144, :595-617
 * (the "coalesce coarse ptr_pc" variants the published runs use).  There a warp walks one
 * vertex's 16-aligned neighbour list through a bam_ptr and the row offsets stay in plain GPU
 * memory.  Here a warp takes 32 consecutive vertices: their labels are one coalesced load, their
 * offsets one or two cached pages, and each active vertex's neighbour list is consumed page by
 * page -- one pin per 4 KiB page of edges for the whole warp, 256 contiguous bytes per step.
 *
 * One level / sweep = one fused launch (controller blocks + workers), so the host sees the
 * `changed` flag between launches exactly as the reference's drivers do (bfs/main.cu:1577-1736,
 * cc/main.cu:1418-1623).
 */
#include <cuda_runtime.h>

#include "bam_abi.h"
#include "bam_synth.h"
#include "bam_fused.cuh"

using namespace bam;

#define BAM_BFS_INF 0xffffffffu

/* Pin the page of `r` holding element index i for the whole warp (lane 0 asks). */
BAM_DEV const uint64_t* warp_page_of(const range_d_t<uint64_t>& r, uint64_t i, uint32_t queue, uint32_t& slot)
{
    const uint64_t page = r.get_page(i);
    slot = range_pin_page(r, 0xffffffffu, (threadIdx.x & 31u) == 0u, page, 1, queue);
    slot = __shfl_sync(0xffffffffu, slot, 0);
    if (slot == BAM_SLOT_ERR) return nullptr;
    return reinterpret_cast<const uint64_t*>(r.get_cache_page_addr(slot));
}

/* offsets[v] and offsets[v+1] for the 32 vertices v0+lane of a chunk (active lanes only) */
BAM_DEV void chunk_offsets(const range_d_t<uint64_t>& off, uint64_t v, bool act, uint32_t queue, uint64_t& s, uint64_t& e)
{
    s = e = 0;
    if (act) {
        s = range_read<uint64_t>(off, v, queue);
        e = range_read<uint64_t>(off, v + 1, queue);
    }
    __syncwarp();
}

struct BfsLevelWork {
    range_d_t<uint64_t> off, col;
    uint64_t v_begin, v_end;
    uint32_t level;
    uint32_t* label;
    uint32_t* changed;
    uint64_t* scanned;

    __device__ void operator()(uint32_t vb, uint32_t nvb) const
    {
        const uint32_t lane = threadIdx.x & 31u;
        const uint32_t wpb = blockDim.x >> 5;
        const uint64_t warp = (uint64_t)vb * wpb + (threadIdx.x >> 5);
        const uint64_t nwarps = (uint64_t)nvb * wpb;
        const uint32_t queue = (uint32_t)warp;
        const uint32_t epp_log = col.cache.page_size_log - 3;
        uint64_t edges = 0;
        bool ch = false;
        for (uint64_t c0 = v_begin + warp * 32; c0 < v_end; c0 += nwarps * 32) {
            const uint64_t v = c0 + lane;
            const bool act = v < v_end && label[v] == level;
            uint32_t am = __ballot_sync(0xffffffffu, act);
            if (am == 0) continue;
            uint64_t s, e;
            chunk_offsets(off, v, act, queue, s, e);
            edges += e - s;
            while (am) {
                const int src = __ffs(am) - 1;
                am &= am - 1;
                const uint64_t vs = __shfl_sync(0xffffffffu, s, src);
                const uint64_t ve = __shfl_sync(0xffffffffu, e, src);
                for (uint64_t i = vs; i < ve;) {
                    uint64_t pend = ((i >> epp_log) + 1) << epp_log;       /* first index of the next page */
                    if (pend > ve) pend = ve;
                    uint32_t slot;
                    const uint64_t* base = warp_page_of(col, i, queue, slot);
                    if (!base) { i = ve; am = 0; break; }
                    const uint64_t page_first = (i >> epp_log) << epp_log;
                    for (uint64_t j = i + lane; j < pend; j += 32) {
                        const uint64_t nb = base[j - page_first];
                        if (label[nb] == BAM_BFS_INF) { label[nb] = level + 1; ch = true; }
                    }
                    __syncwarp();
                    if (lane == 0) col.release_page(slot, 1);
                    i = pend;
                }
            }
        }
        __syncwarp();
        if (__any_sync(0xffffffffu, ch) && lane == 0) *changed = 1u;
        warp_sum_to(edges, scanned);
    }
};

struct CcSweepWork {
    range_d_t<uint64_t> off, col;
    uint64_t v_begin, v_end;
    unsigned long long* comp;
    const uint8_t* curr_visit;
    uint8_t* next_visit;
    uint32_t* changed;
    uint64_t* scanned;

    __device__ void operator()(uint32_t vb, uint32_t nvb) const
    {
        const uint32_t lane = threadIdx.x & 31u;
        const uint32_t wpb = blockDim.x >> 5;
        const uint64_t warp = (uint64_t)vb * wpb + (threadIdx.x >> 5);
        const uint64_t nwarps = (uint64_t)nvb * wpb;
        const uint32_t queue = (uint32_t)warp;
        const uint32_t epp_log = col.cache.page_size_log - 3;
        uint64_t edges = 0;
        bool ch = false;
        for (uint64_t c0 = v_begin + warp * 32; c0 < v_end; c0 += nwarps * 32) {
            const uint64_t v = c0 + lane;
            const bool act = v < v_end && curr_visit[v] != 0;
            uint32_t am = __ballot_sync(0xffffffffu, act);
            if (am == 0) continue;
            uint64_t s, e;
            chunk_offsets(off, v, act, queue, s, e);
            edges += e - s;
            while (am) {
                const int src = __ffs(am) - 1;
                am &= am - 1;
                const uint64_t vs = __shfl_sync(0xffffffffu, s, src);
                const uint64_t ve = __shfl_sync(0xffffffffu, e, src);
                const uint64_t u = c0 + src;
                for (uint64_t i = vs; i < ve;) {
                    uint64_t pend = ((i >> epp_log) + 1) << epp_log;
                    if (pend > ve) pend = ve;
                    uint32_t slot;
                    const uint64_t* base = warp_page_of(col, i, queue, slot);
                    if (!base) { i = ve; am = 0; break; }
                    const uint64_t page_first = (i >> epp_log) << epp_log;
                    for (uint64_t j = i + lane; j < pend; j += 32) {
                        const uint64_t nb = base[j - page_first];
                        /* the relaxation of cc_compute: the larger label takes the smaller one */
                        const unsigned long long cu = *reinterpret_cast<volatile unsigned long long*>(&comp[u]);
                        const unsigned long long cn = *reinterpret_cast<volatile unsigned long long*>(&comp[nb]);
                        if (cu < cn) { atomicMin(&comp[nb], cu); next_visit[nb] = 1; ch = true; }
                        else if (cn < cu) { atomicMin(&comp[u], cn); next_visit[u] = 1; ch = true; }
                    }
                    __syncwarp();
                    if (lane == 0) col.release_page(slot, 1);
                    i = pend;
                }
            }
        }
        __syncwarp();
        if (__any_sync(0xffffffffu, ch) && lane == 0) *changed = 1u;
        warp_sum_to(edges, scanned);
    }
};

__global__ void k_bfs_init(uint32_t* label, uint64_t n, uint64_t src)
{
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x, nthr = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = tid; i < n; i += nthr) label[i] = (i == src) ? 0u : BAM_BFS_INF;
}

__global__ void k_cc_init(unsigned long long* comp, uint8_t* curr, uint8_t* next, uint64_t n)
{
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x, nthr = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = tid; i < n; i += nthr) { comp[i] = i; curr[i] = 1; next[i] = 0; }
}

/* R-MAT edge e -> the two directed keys (u<<32|v), (v<<32|u); a self loop gives two ~0 keys
 * (sorted to the end and dropped by the caller). */
__global__ void k_rmat_keys(uint64_t* keys, uint64_t e_begin, uint64_t e_end, uint64_t seed, uint32_t scale, bam_rmat_thresh_t t)
{
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x, nthr = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t e = e_begin + tid; e < e_end; e += nthr) {
        uint64_t u, v;
        bam_rmat_edge(seed, e, scale, t, &u, &v);
        const uint64_t k = 2 * (e - e_begin);
        if (u == v) { keys[k] = ~0ull; keys[k + 1] = ~0ull; }
        else { keys[k] = (u << 32) | v; keys[k + 1] = (v << 32) | u; }
    }
}

static int check_graph_args(bam_array_t offsets, bam_array_t cols)
{
    if (!offsets || !cols) return BAM_EINVAL;
    if (offsets->elem_bytes != 8 || cols->elem_bytes != 8) return BAM_EINVAL;
    if (offsets->pc != cols->pc) return BAM_EINVAL;
    return BAM_OK;
}

extern "C" int bam_launch_bfs_level(bam_array_t offsets, bam_array_t cols, uint64_t v_begin, uint64_t v_end, uint32_t level,
                                    uint32_t* label_dev, uint32_t* changed_dev, uint64_t* scanned_dev, void* stream)
{
    int rc = check_graph_args(offsets, cols);
    if (rc) return rc;
    if (!label_dev || !changed_dev || v_end > offsets->n_elems - 1 || v_begin > v_end) return BAM_EINVAL;
    bam_ctrl* c = offsets->pc->ctrl;
    CK(cudaSetDevice(c->device));
    BfsLevelWork w;
    w.off = offsets->h_range; w.col = cols->h_range; w.v_begin = v_begin; w.v_end = v_end; w.level = level;
    w.label = label_dev; w.changed = changed_dev; w.scanned = scanned_dev;
    return launch_fused(c, w, (cudaStream_t)stream);
}

extern "C" int bam_launch_cc_sweep(bam_array_t offsets, bam_array_t cols, uint64_t v_begin, uint64_t v_end,
                                   uint64_t* comp_dev, const uint8_t* curr_visit_dev, uint8_t* next_visit_dev,
                                   uint32_t* changed_dev, uint64_t* scanned_dev, void* stream)
{
    int rc = check_graph_args(offsets, cols);
    if (rc) return rc;
    if (!comp_dev || !curr_visit_dev || !next_visit_dev || !changed_dev || v_end > offsets->n_elems - 1 || v_begin > v_end) return BAM_EINVAL;
    bam_ctrl* c = offsets->pc->ctrl;
    CK(cudaSetDevice(c->device));
    CcSweepWork w;
    w.off = offsets->h_range; w.col = cols->h_range; w.v_begin = v_begin; w.v_end = v_end;
    w.comp = reinterpret_cast<unsigned long long*>(comp_dev); w.curr_visit = curr_visit_dev; w.next_visit = next_visit_dev;
    w.changed = changed_dev; w.scanned = scanned_dev;
    return launch_fused(c, w, (cudaStream_t)stream);
}

/* Whole traversals on one GPU: the host loops of benchmarks/bfs/main.cu:1577-1736 and
 * benchmarks/cc/main.cu:1418-1623 (launch, read `changed`, repeat). */
extern "C" int bam_bfs_run(bam_array_t offsets, bam_array_t cols, uint64_t n_vertices, uint64_t source,
                           uint32_t* label_dev, uint32_t* n_levels_out, uint64_t* edges_scanned_out)
{
    int rc = check_graph_args(offsets, cols);
    if (rc) return rc;
    if (!label_dev || source >= n_vertices || n_vertices + 1 > offsets->n_elems) return BAM_EINVAL;
    bam_ctrl* c = offsets->pc->ctrl;
    CK(cudaSetDevice(c->device));
    uint32_t* d_changed = nullptr;
    uint64_t* d_scanned = nullptr;
    CK(cudaMalloc(&d_changed, 4));
    cudaError_t e = cudaMalloc(&d_scanned, 8);
    if (e != cudaSuccess) { cudaFree(d_changed); g_last_cuda = e; return BAM_ENOMEM; }
    cudaMemset(d_scanned, 0, 8);
    k_bfs_init<<<c->num_sms * 4, 256>>>(label_dev, n_vertices, source);
    uint32_t level = 0;
    rc = BAM_OK;
    for (;; level++) {
        cudaMemsetAsync(d_changed, 0, 4, 0);
        rc = bam_launch_bfs_level(offsets, cols, 0, n_vertices, level, label_dev, d_changed, d_scanned, nullptr);
        if (rc) break;
        uint32_t changed = 0;
        e = cudaMemcpy(&changed, d_changed, 4, cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) { g_last_cuda = e; rc = BAM_ECUDA; break; }
        bam_status_t st;
        cudaMemcpy(&st, c->d_status, sizeof st, cudaMemcpyDeviceToHost);
        if (st.code) { rc = (int)st.code; break; }
        if (!changed) break;
    }
    if (n_levels_out) *n_levels_out = level + 1;              /* levels 0..level hold vertices */
    if (edges_scanned_out) cudaMemcpy(edges_scanned_out, d_scanned, 8, cudaMemcpyDeviceToHost);
    cudaFree(d_changed); cudaFree(d_scanned);
    return rc;
}

extern "C" int bam_cc_run(bam_array_t offsets, bam_array_t cols, uint64_t n_vertices, uint64_t* comp_dev,
                          uint32_t* n_sweeps_out, uint64_t* edges_scanned_out)
{
    int rc = check_graph_args(offsets, cols);
    if (rc) return rc;
    if (!comp_dev || n_vertices + 1 > offsets->n_elems) return BAM_EINVAL;
    bam_ctrl* c = offsets->pc->ctrl;
    CK(cudaSetDevice(c->device));
    uint32_t* d_changed = nullptr;
    uint64_t* d_scanned = nullptr;
    uint8_t* d_visit = nullptr;
    cudaError_t e = cudaMalloc(&d_changed, 4);
    if (e == cudaSuccess) e = cudaMalloc(&d_scanned, 8);
    if (e == cudaSuccess) e = cudaMalloc(&d_visit, 2 * n_vertices);
    if (e != cudaSuccess) { cudaFree(d_changed); cudaFree(d_scanned); cudaFree(d_visit); g_last_cuda = e; (void)cudaGetLastError(); return BAM_ENOMEM; }
    cudaMemset(d_scanned, 0, 8);
    uint8_t* curr = d_visit;
    uint8_t* next = d_visit + n_vertices;
    k_cc_init<<<c->num_sms * 4, 256>>>(reinterpret_cast<unsigned long long*>(comp_dev), curr, next, n_vertices);
    uint32_t sweeps = 0;
    rc = BAM_OK;
    for (;;) {
        cudaMemsetAsync(d_changed, 0, 4, 0);
        rc = bam_launch_cc_sweep(offsets, cols, 0, n_vertices, comp_dev, curr, next, d_changed, d_scanned, nullptr);
        if (rc) break;
        sweeps++;
        uint32_t changed = 0;
        e = cudaMemcpy(&changed, d_changed, 4, cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) { g_last_cuda = e; rc = BAM_ECUDA; break; }
        bam_status_t st;
        cudaMemcpy(&st, c->d_status, sizeof st, cudaMemcpyDeviceToHost);
        if (st.code) { rc = (int)st.code; break; }
        if (!changed) break;
        cudaMemsetAsync(curr, 0, n_vertices, 0);              /* the visited set becomes the next one */
        uint8_t* t = curr; curr = next; next = t;
    }
    if (n_sweeps_out) *n_sweeps_out = sweeps;
    if (edges_scanned_out) cudaMemcpy(edges_scanned_out, d_scanned, 8, cudaMemcpyDeviceToHost);
    cudaFree(d_changed); cudaFree(d_scanned); cudaFree(d_visit);
    return rc;
}

extern "C" int bam_gen_rmat_keys(uint64_t* keys_dev, uint64_t e_begin, uint64_t e_end, uint64_t seed, uint32_t scale,
                                 uint32_t ta, uint32_t tab, uint32_t tabc, void* stream)
{
    if (!keys_dev || e_end < e_begin || scale == 0 || scale > 31) return BAM_EINVAL;
    bam_rmat_thresh_t t = { ta, tab, tabc };
    k_rmat_keys<<<1184, 256, 0, (cudaStream_t)stream>>>(keys_dev, e_begin, e_end, seed, scale, t);
    CK(cudaGetLastError());
    return BAM_OK;
}

extern "C" int bam_ctrl_write_store_from_device(bam_ctrl_t c, uint64_t byte_offset, const void* src_dev, uint64_t bytes, void* stream)
{
    if (!c || !src_dev || byte_offset + bytes > c->store_bytes || byte_offset + bytes < byte_offset) return BAM_EINVAL;
    CK(cudaSetDevice(c->device));
    CK(cudaMemcpyAsync(c->store_host + byte_offset, src_dev, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    return BAM_OK;
}
