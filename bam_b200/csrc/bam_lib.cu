/*
 * bam_lib.cu -- host side of libbam_b200.so (the C ABI of include/bam_abi.h) and the fused
 * kernels it launches.  sm_100a only; there is no CPU path.
 *
 * Launch model.  A workload kernel waits on completions that the emulated controller produces,
 * so both must be running at the same time.  They are therefore ONE cooperative launch
 * (co-residency of all blocks is guaranteed by cudaLaunchCooperativeKernel or the launch fails):
 * blocks [0, n_ctrl_blocks) run bam::emu_controller_main, the remaining blocks are persistent
 * workers that stride over the workload.  The controller blocks leave when the last worker
 * block has finished.
 */
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

#include "bam_abi.h"
#include "bam_synth.h"
#include "bam/array.cuh"
#include "bam/emu_ctrl.cuh"
#include "bam_internal.h"
#include "bam_fused.cuh"

using namespace bam;

thread_local cudaError_t g_last_cuda = cudaSuccess;

/* ====================================================================================== */
/* small kernels: initialisation, store fill, audit                                       */
/* ====================================================================================== */

__global__ void k_init_cache(bam_slot_t* slots, uint32_t n_slots, uint32_t* table, uint64_t n_words)
{
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t nthr = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = tid; i < n_slots; i += nthr) { slots[i].tag = BAM_TAG_NONE; slots[i].state = 0; slots[i].gen = 0; }
    for (uint64_t i = tid; i < n_words; i += nthr) table[i] = (i % BAM_BUCKET_WORDS) ? BAM_ENTRY_EMPTY : 0u;
}

__global__ void k_fill_store(uint64_t* dst, uint64_t n_elems, uint64_t seed, uint64_t first_elem)
{
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t nthr = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = tid * 2; i < n_elems; i += nthr * 2) {
        ulonglong2 v;
        v.x = bam_store_elem(seed, first_elem + i);
        v.y = bam_store_elem(seed, first_elem + i + 1);
        if (i + 1 < n_elems) *reinterpret_cast<ulonglong2*>(dst + i) = v;
        else dst[i] = v.x;
    }
}

/* Access streams of the synthetic workloads, materialised as index lists in device memory. */
/* The share of a striped store that controller `stripe` of `n_stripes` holds: its page j is page
 * j * n_stripes + stripe of the logical store. */
__global__ void k_fill_store_striped(uint64_t* dst, uint64_t n_elems, uint64_t seed, uint64_t first_elem, uint32_t page_elems_log2,
                                     uint32_t stripe, uint32_t n_stripes)
{
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t nthr = (uint64_t)gridDim.x * blockDim.x;
    const uint64_t mask = (1ull << page_elems_log2) - 1;
    for (uint64_t i = tid; i < n_elems; i += nthr) {
        const uint64_t logical = (((i >> page_elems_log2) * n_stripes + stripe) << page_elems_log2) | (i & mask);
        dst[i] = bam_store_elem(seed, first_elem + logical);
    }
}

__global__ void k_gen_uniform(uint64_t* out, uint64_t n_lanes, uint64_t reqs_per_lane, uint64_t access_seed, uint64_t n_elems)
{
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t nthr = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t lane = tid; lane < n_lanes; lane += nthr) {
        bam_pcg32_t g;
        bam_lane_stream(&g, access_seed, lane);
        for (uint64_t k = 0; k < reqs_per_lane; k++) out[lane * reqs_per_lane + k] = bam_uniform_index(&g, n_elems);
    }
}

__global__ void k_gen_zipf(uint64_t* out, uint64_t n_lanes, uint64_t reqs_per_lane, uint64_t access_seed,
                           const uint64_t* cdf, uint64_t n_pages, uint32_t elems_per_page, uint64_t perm_seed)
{
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t nthr = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t lane = tid; lane < n_lanes; lane += nthr) {
        bam_pcg32_t g;
        bam_lane_stream(&g, access_seed, lane);
        for (uint64_t k = 0; k < reqs_per_lane; k++)
            out[lane * reqs_per_lane + k] = bam_zipf_access(&g, cdf, n_pages, elems_per_page, perm_seed);
    }
}

/* Wrapping sum of store element (first_elem + idx[i]) recomputed from its definition: the value a
 * cached read of that index must return.  Used to verify full-size runs on the device. */
__global__ void k_direct_checksum(const uint64_t* idx, uint64_t n, uint64_t seed, uint64_t first_elem, uint64_t* out)
{
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t nthr = (uint64_t)gridDim.x * blockDim.x;
    uint64_t sum = 0;
    for (uint64_t i = tid; i < n; i += nthr) sum += bam_store_elem(seed, first_elem + idx[i]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if ((threadIdx.x & 31u) == 0u) atomicAdd((unsigned long long*)out, (unsigned long long)sum);
}

/* Page of every request of the block random-read workload. */
__global__ void k_gen_block_pages(uint64_t* out, uint64_t n_reqs, uint64_t req_seed, uint64_t n_pages)
{
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t nthr = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t r = tid; r < n_reqs; r += nthr) out[r] = bam_block_request_page(req_seed, r, n_pages);
}

/* Wrapping sum of every word of every listed page, recomputed from the store's definition
 * (one warp per page). */
__global__ void k_page_sums(const uint64_t* pages, uint64_t n, uint64_t seed, uint32_t words_per_page, uint64_t* out)
{
    const uint32_t lane = threadIdx.x & 31u;
    const uint64_t warp = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint64_t nwarps = ((uint64_t)gridDim.x * blockDim.x) >> 5;
    uint64_t sum = 0;
    for (uint64_t i = warp; i < n; i += nwarps) {
        const uint64_t first = pages[i] * words_per_page;
        for (uint32_t w = lane; w < words_per_page; w += 32) sum += bam_store_elem(seed, first + w);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) atomicAdd((unsigned long long*)out, (unsigned long long)sum);
}

/* Post-launch audit of the cache invariants; counts violations. */
__global__ void k_audit(page_cache_d_t pc, uint64_t n_buckets, unsigned long long* violations)
{
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t nthr = (uint64_t)gridDim.x * blockDim.x;
    unsigned long long bad = 0;
    for (uint64_t s = tid; s < pc.n_slots; s += nthr) {
        const uint32_t st = pc.slots[s].state;
        const uint64_t tag = pc.slots[s].tag;
        if (st & BAM_CNT_MASK) bad++;                                  /* a pin was leaked          */
        if (st & BAM_BUSY) bad++;                                      /* a fill/evict never ended  */
        if ((st & BAM_VALID) && tag == BAM_TAG_NONE) bad++;
        if (!(st & BAM_VALID) && tag != BAM_TAG_NONE) bad++;
        if (st & BAM_VALID) {
            const uint64_t h = pt_hash(tag);
            if (pt_lookup(pc, tag, (uint32_t)h & pc.bucket_mask, (uint32_t)(h >> 56)) != (uint32_t)s) bad++;
        }
    }
    for (uint64_t b = tid; b < n_buckets; b += nthr) {
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
    if (bad) atomicAdd(violations, bad);
}

/* ---- block benchmark ---------------------------------------------------------------------
 * Every thread keeps io_depth requests in flight (io_depth = 1: the block benchmark,
 * benchmarks/block/main.cu:137-200; io_depth > 1: the iodepth-block benchmark,
 * benchmarks/iodepth-block/main.cu:97-147), each landing in a private cache slot. */
#define BAM_MAX_IO_DEPTH 8
struct BlockReadWork {
    page_cache_d_t pc;
    uint64_t n_reqs;
    const uint64_t* pages;
    uint64_t req_seed;
    uint64_t n_store_pages;
    uint32_t* crc_out;
    uint64_t* sum_out;
    uint32_t io_depth;

    __device__ void operator()(uint32_t vb, uint32_t nvb) const
    {
        __shared__ uint32_t crc_tab[256];
        if (crc_out) {
            for (uint32_t i = threadIdx.x; i < 256; i += blockDim.x) {
                uint32_t c = i;
                for (int k = 0; k < 8; k++) c = (c >> 1) ^ (0xEDB88320u & (0u - (c & 1u)));
                crc_tab[i] = c;
            }
            __syncthreads();
        }
        const uint64_t gid = (uint64_t)vb * blockDim.x + threadIdx.x;
        const uint64_t nthr = (uint64_t)nvb * blockDim.x;
        Controller* c = pc.d_ctrl;
        QueuePair* qp = c->d_qps + ((uint32_t)(gid >> 5) % c->n_qps);
        uint64_t sum = 0;
        const uint64_t warp_first = gid & ~31ull;             /* requests are issued by whole warps */
        const uint32_t depth = io_depth;
        for (uint64_t r0 = warp_first; r0 < n_reqs; r0 += nthr * depth) {
            uint32_t cid[BAM_MAX_IO_DEPTH];
            uint64_t req[BAM_MAX_IO_DEPTH];
            bool fail = false;
#pragma unroll
            for (uint32_t d = 0; d < BAM_MAX_IO_DEPTH; d++) {
                if (d < depth) {
                    req[d] = r0 + (uint64_t)d * nthr + (threadIdx.x & 31u);
                    const bool active = req[d] < n_reqs;
                    uint64_t pg = 0;
                    if (active) pg = pages ? pages[req[d]] : bam_block_request_page(req_seed, req[d], n_store_pages);
                    const uint64_t bus = slot_bus_addr(pc, (uint32_t)(gid * depth + d));     /* private slot */
                    /* one request per thread: the blocking form, which also copes with queues shallower
                     * than a warp; several per thread: submit now, wait below */
                    if (depth == 1) cid[d] = (uint32_t)warp_io(0xffffffffu, active, qp, pg * pc.n_blocks_per_page, pc.n_blocks_per_page,
                                                               bus, pc.page_size > 4096 ? bus + 4096 : 0, NVM_IO_READ);
                    else cid[d] = warp_io_submit(0xffffffffu, active, qp, pg * pc.n_blocks_per_page, pc.n_blocks_per_page, bus,
                                                 pc.page_size > 4096 ? bus + 4096 : 0, NVM_IO_READ);
                }
            }
#pragma unroll
            for (uint32_t d = 0; d < BAM_MAX_IO_DEPTH; d++) {
                if (d < depth) {
                    const bool active = req[d] < n_reqs;
                    const int rc = depth == 1 ? (int)cid[d] : warp_io_wait(0xffffffffu, active, qp, cid[d]);
                    if (__any_sync(0xffffffffu, rc != BAM_OK)) fail = true;
                    if (active && rc == BAM_OK && (crc_out || sum_out)) {
                        uint32_t crc = ~0u;
                        const uint8_t* p = reinterpret_cast<const uint8_t*>(slot_bus_addr(pc, (uint32_t)(gid * depth + d)));
                        for (uint32_t o = 0; o < pc.page_size; o += 16) {
                            const uint4 v = ld_cg_v4(p + o);
                            sum += (((uint64_t)v.y << 32) | v.x) + (((uint64_t)v.w << 32) | v.z);
                            if (crc_out) {
                                const uint32_t w[4] = { v.x, v.y, v.z, v.w };
#pragma unroll
                                for (int j = 0; j < 4; j++) {
                                    uint32_t x = w[j];
#pragma unroll
                                    for (int bb = 0; bb < 4; bb++) { crc = (crc >> 8) ^ crc_tab[(crc ^ x) & 0xffu]; x >>= 8; }
                                }
                            }
                        }
                        if (crc_out) crc_out[req[d]] = ~crc;
                    }
                    __syncwarp();
                }
            }
            if (fail) break;
        }
        __syncwarp();
        warp_sum_to(sum, sum_out);
    }
};

/* ---- array benchmark --------------------------------------------------------------------- */
#ifndef BAM_ARRAY_READ_BATCH
#define BAM_ARRAY_READ_BATCH 4
#endif
struct ArrayReadWork {
    /* two resident blocks per SM (128 registers per thread): the batched reader keeps four look-ups, slot
     * records and element loads per lane in registers; measured against three blocks of 80 registers, all-hit
     * random reads 12.4 -> 16.4 G/s, the miss-bound scan unchanged */
    static constexpr int min_blocks = 2;
    range_d_t<uint64_t> r;
    uint64_t n_lanes, reqs_per_lane;
    const uint64_t* idx;
    uint64_t access_seed;
    uint64_t* sum_out;

    __device__ void operator()(uint32_t vb, uint32_t nvb) const
    {
        const uint64_t gid = (uint64_t)vb * blockDim.x + threadIdx.x;
        const uint64_t nthr = (uint64_t)nvb * blockDim.x;
        const uint32_t queue = (uint32_t)(gid >> 5);
        const uint64_t n_elems = r.count - r.index_start;
        uint64_t sum = 0;
        uint32_t hits = 0;
        opt_memo_t memo;
        /* a lane's requests are served BAM_ARRAY_READ_BATCH at a time, so that it has that many
         * independent look-ups and element loads in flight; the indices of the next batch are loaded
         * while the current one is served */
        for (uint64_t lane = gid; lane < n_lanes; lane += nthr) {
            bam_pcg32_t g;
            bam_lane_stream(&g, access_seed, lane);
            size_t nx[BAM_ARRAY_READ_BATCH];
            auto fetch = [&](uint64_t k) {
#pragma unroll
                for (uint32_t b = 0; b < BAM_ARRAY_READ_BATCH; b++) {
                    nx[b] = r.index_start;
                    if (k + b < reqs_per_lane) nx[b] = idx ? idx[lane * reqs_per_lane + k + b] : r.index_start + bam_uniform_index(&g, n_elems);
                }
            };
            fetch(0);
            for (uint64_t k = 0; k < reqs_per_lane; k += BAM_ARRAY_READ_BATCH) {
                size_t ii[BAM_ARRAY_READ_BATCH];
                uint64_t vv[BAM_ARRAY_READ_BATCH];
                const uint32_t n = reqs_per_lane - k < BAM_ARRAY_READ_BATCH ? (uint32_t)(reqs_per_lane - k) : BAM_ARRAY_READ_BATCH;
#pragma unroll
                for (uint32_t b = 0; b < BAM_ARRAY_READ_BATCH; b++) { ii[b] = nx[b]; vv[b] = 0; }
                if (k + BAM_ARRAY_READ_BATCH < reqs_per_lane) fetch(k + BAM_ARRAY_READ_BATCH);
                range_read_n<uint64_t, BAM_ARRAY_READ_BATCH>(r, ii, n, vv, queue, hits, memo);
#pragma unroll
                for (uint32_t b = 0; b < BAM_ARRAY_READ_BATCH; b++) if (b < n) sum += vv[b];
            }
        }
        __syncwarp();
        const uint32_t wh = __reduce_add_sync(0xffffffffu, hits);
        if (wh && (threadIdx.x & 31u) == 0u) count_hit(r.cache, wh);
        warp_sum_to(sum, sum_out);
    }
};

/* The same benchmark over an array of several ranges: every read is array[i] (array_d_t::seq_read looks the
 * range up, page_cache.h:1318-1329 and :1541-1574 in the reference). */
struct ArrayReadRangesWork {
    array_d_t<uint64_t> arr;
    uint64_t n_lanes, reqs_per_lane;
    const uint64_t* idx;
    uint64_t access_seed;
    uint64_t* sum_out;

    __device__ void operator()(uint32_t vb, uint32_t nvb) const
    {
        const uint64_t gid = (uint64_t)vb * blockDim.x + threadIdx.x;
        const uint64_t nthr = (uint64_t)nvb * blockDim.x;
        uint64_t sum = 0;
        for (uint64_t lane = gid; lane < n_lanes; lane += nthr) {
            bam_pcg32_t g;
            bam_lane_stream(&g, access_seed, lane);
            for (uint64_t k = 0; k < reqs_per_lane; k++) {
                const uint64_t i = idx ? idx[lane * reqs_per_lane + k] : bam_uniform_index(&g, arr.n_elems);
                sum += arr[i];
            }
        }
        __syncwarp();
        warp_sum_to(sum, sum_out);
    }
};

/* ---- write path ----------------------------------------------------------------------------------
 * Element writes and atomic adds through the cache (the vectoradd-style consumers of the
 * reference, benchmarks/vectoradd/main.cu:103-118), and the write-back of every dirty page
 * (page_cache.h:584-629 __flush there). */
struct ArrayWriteWork {
    array_d_t<uint64_t> arr;            /* by value: n_ranges = 1, d_ranges points at the device descriptor */
    uint64_t n;
    const uint64_t* idx;
    uint64_t val_seed;
    uint64_t addend;                    /* 0: a[i] = splitmix64(val_seed ^ i); else a[i] += addend (atomic) */

    __device__ void operator()(uint32_t vb, uint32_t nvb) const
    {
        const uint64_t gid = (uint64_t)vb * blockDim.x + threadIdx.x;
        const uint64_t nthr = (uint64_t)nvb * blockDim.x;
        for (uint64_t k = gid; k < n; k += nthr) {
            const uint64_t i = idx[k];
            if (addend) arr.AtomicAdd(i, addend);
            else arr.seq_write(i, bam_splitmix64(val_seed ^ i));
        }
    }
};

/* ---- the per-thread protocol ------------------------------------------------------------------------
 * Every participating lane pins a page, reads its first element and unpins it entirely on its own, the way a
 * diverged caller uses range_d_t::acquire_page(page, count, write, queue) (page_cache.h:1122-1224 in the
 * reference: no warp-mates to share look-ups, slot claims or write-backs with).  `lanes` says which lanes of
 * every warp take part; the others sit the launch out. */
struct ThreadAcquireWork {
    range_d_t<uint64_t> r;
    uint64_t first_page, n_pages;
    uint32_t lanes;
    uint64_t* first_words;              /* first_words[k] = element 0 of page first_page + k */

    __device__ void operator()(uint32_t vb, uint32_t nvb) const
    {
        const uint32_t lane = threadIdx.x & 31u;
        const uint64_t warp = ((uint64_t)vb * blockDim.x + threadIdx.x) >> 5, nwarps = ((uint64_t)nvb * blockDim.x) >> 5;
        if ((lanes >> lane) & 1u) {
            const uint32_t per_warp = __popc(lanes), rank = __popc(lanes & ((1u << lane) - 1u));
            for (uint64_t k = warp * per_warp + rank; k < n_pages; k += nwarps * per_warp) {
                const uint32_t slot = r.acquire_page(first_page + k, 1, false, (uint32_t)warp);
                if (slot > BAM_SLOT_MAX) break;                       /* the status block says why */
                first_words[k] = ld_strong(reinterpret_cast<const uint64_t*>(r.get_cache_page_addr(slot)));
                r.release_page(slot, 1);
            }
        }
    }
};

/* ---- bulk transfer between cache memory and the store (benchmarks/readwrite/main.cu:283-390) -------
 * The reference's loader copies a chunk of a file into the cache's memory and lets a kernel issue one
 * NVMe WRITE per cache page (sequential_access_kernel with WRITE, :93-130 there); reading back is the
 * same with READ.  Request r moves cache slot first_slot + r <-> store page first_store_page + r. */
struct BulkIoWork {
    page_cache_d_t pc;
    uint64_t n_pages, first_store_page, first_slot;
    uint8_t opcode;

    __device__ void operator()(uint32_t vb, uint32_t nvb) const
    {
        const uint32_t lane = threadIdx.x & 31u;
        const uint64_t gid = (uint64_t)vb * blockDim.x + threadIdx.x;
        const uint64_t nthr = (uint64_t)nvb * blockDim.x;
        const uint32_t queue = (uint32_t)(gid >> 5);
        for (uint64_t base = gid - lane; base < n_pages; base += nthr) {
            const uint64_t r = base + lane;
            const bool active = r < n_pages;
            const uint32_t slot = (uint32_t)(first_slot + r);
            const int rc = warp_io(0xffffffffu, active, pick_queue(pc, 0, queue), (first_store_page + r) * pc.n_blocks_per_page,
                                   pc.n_blocks_per_page, active ? slot_bus_addr(pc, slot) : 0, active ? slot_prp2(pc, slot) : 0, opcode);
            if (__any_sync(0xffffffffu, active && rc != BAM_OK)) break;
        }
    }
};

/* ---- access patterns through bam_ptr cursors (benchmarks/pattern/main.cu) ------------------------
 * The *_pc kernels of the reference's pattern benchmark: every thread owns a bam_ptr and sums the
 * elements it visits.  SEQUENTIAL (:131-146): element i goes to thread i mod T.  SEQUENTIAL_WARP
 * (:232-265): warp w reads n_pages_per_warp consecutive pages; warp ids are interleaved by `stride`
 * as there.  RANDOM (:155-170): thread t reads a[assignment[i]] for i = t, t + T, ...  RANDOM_WARP:
 * warp w reads the whole pages assignment[w * n_pages_per_warp + k]. */
#define BAM_PATTERN_SEQUENTIAL 0u
#define BAM_PATTERN_SEQUENTIAL_WARP 1u
#define BAM_PATTERN_RANDOM 2u
#define BAM_PATTERN_RANDOM_WARP 3u

#ifndef BAM_PATTERN_ROWS
#define BAM_PATTERN_ROWS 4            /* rows of a page the array[] form reads per batch */
#endif
#define BAM_IMPL_PTR 0u            /* every thread reads through a bam_ptr cursor (the benchmarks' "bam_ptr" type)  */
#define BAM_IMPL_ARRAY 1u          /* every read is array[i] (their "ORIG" type, benchmarks/cache/main.cu:70)       */

struct PatternWork {
    array_d_t<uint64_t> arr;
    range_d_t<uint64_t> rng;            /* the array's single range, by value: what the array[] form reads through */
    uint32_t pattern, impl;
    uint64_t n_elems, n_warps, n_pages_per_warp, stride;
    const uint64_t* assignment;
    uint64_t* sum_out;

    __device__ void operator()(uint32_t vb, uint32_t nvb) const
    {
        const uint32_t lane = threadIdx.x & 31u;
        const uint64_t gid = (uint64_t)vb * blockDim.x + threadIdx.x;
        const uint64_t nthr = (uint64_t)nvb * blockDim.x;
        const uint64_t epp = rng.cache.page_size / sizeof(uint64_t);
        uint64_t v = 0;
        if (impl == BAM_IMPL_ARRAY) {
            /* the same walks with array[] reads: indices are computed, the 16 rows of a 4 KiB page are read
             * BAM_PATTERN_ROWS at a time, and after the first read of a page the thread's translation memo serves the rest */
            const bool by_warp = pattern == BAM_PATTERN_SEQUENTIAL_WARP || pattern == BAM_PATTERN_RANDOM_WARP;
            const uint64_t nep = by_warp ? (n_warps + stride - 1) / stride : 1;
            const uint64_t w_end = by_warp ? n_warps : (n_elems + 31) / 32;
            const uint64_t rows = by_warp ? epp / 32 : 1;
            const uint64_t pages = by_warp ? n_pages_per_warp : 1;
            const uint64_t limit = by_warp ? arr.n_elems : n_elems;
            const uint32_t queue = (uint32_t)(gid >> 5);
            opt_memo_t memo;
            uint32_t hits = 0;
            for (uint64_t w = gid >> 5; w < w_end; w += nthr >> 5) {
                const uint64_t warp_id = pattern == BAM_PATTERN_SEQUENTIAL_WARP ? (w / nep) + (w % nep) * stride : w;
                if (warp_id >= w_end) continue;
                for (uint64_t k = 0; k < pages; k++) {
                    uint64_t first;
                    if (pattern == BAM_PATTERN_SEQUENTIAL_WARP) first = (warp_id * pages + k) * epp;
                    else if (pattern == BAM_PATTERN_RANDOM_WARP) first = assignment[warp_id * pages + k] * epp;
                    else first = warp_id * 32;
                    for (uint64_t r = 0; r < rows; r += BAM_PATTERN_ROWS) {
                        size_t ii[BAM_PATTERN_ROWS];
                        uint64_t x[BAM_PATTERN_ROWS];
                        uint32_t n = 0;
#pragma unroll
                        for (int u = 0; u < BAM_PATTERN_ROWS; u++) {
                            uint64_t i = first + (r + u) * 32 + lane;
                            const bool ok = r + u < rows && i < limit;
                            if (ok && pattern == BAM_PATTERN_RANDOM) i = assignment[i];
                            ii[u] = ok ? i : 0;
                            x[u] = 0;
                            n += ok ? 1u : 0u;          /* the valid rows are a prefix: indices grow with u */
                        }
                        range_read_n<uint64_t, BAM_PATTERN_ROWS>(rng, ii, n, x, queue, hits, memo);
#pragma unroll
                        for (int u = 0; u < BAM_PATTERN_ROWS; u++) v += (uint32_t)u < n ? x[u] : 0;
                    }
                }
            }
            __syncwarp();
            const uint32_t wh = __reduce_add_sync(0xffffffffu, hits);
            if (wh && lane == 0) count_hit(rng.cache, wh);
        } else {
            bam_ptr<uint64_t> ptr(&arr);
            /* one loop for all patterns, so that the cursor's code exists once: (w, k, j) walk warp
             * items, pages of an item and element rows of a page; the element patterns use w only */
            const bool by_warp = pattern == BAM_PATTERN_SEQUENTIAL_WARP || pattern == BAM_PATTERN_RANDOM_WARP;
            const uint64_t nep = by_warp ? (n_warps + stride - 1) / stride : 1;
            const uint64_t w_end = by_warp ? n_warps : (n_elems + 31) / 32;
            const uint64_t rows = by_warp ? epp / 32 : 1;
            const uint64_t pages = by_warp ? n_pages_per_warp : 1;
            for (uint64_t w = gid >> 5; w < w_end; w += nthr >> 5) {
                const uint64_t warp_id = pattern == BAM_PATTERN_SEQUENTIAL_WARP ? (w / nep) + (w % nep) * stride : w;
                if (warp_id >= w_end) continue;
                for (uint64_t k = 0; k < pages; k++) {
                    uint64_t first;                                  /* element index of lane 0 in row 0 */
                    if (pattern == BAM_PATTERN_SEQUENTIAL_WARP) first = (warp_id * pages + k) * epp;
                    else if (pattern == BAM_PATTERN_RANDOM_WARP) first = assignment[warp_id * pages + k] * epp;
                    else first = warp_id * 32;
                    /* row 0 moves the cursor to the page; the other rows of the page are then read four
                     * at a time (four loads in flight per lane) */
                    uint64_t i0 = first + lane;
                    const bool ok0 = by_warp ? i0 < arr.n_elems : i0 < n_elems;
                    if (ok0 && pattern == BAM_PATTERN_RANDOM) i0 = assignment[i0];
                    if (ok0) v += ptr.read(i0);
                    for (uint64_t r = 1; r < rows; r += 4) {
                        size_t idx[4];
                        uint64_t x[4];
                        bool ok[4];
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            const uint64_t i = first + (r + u) * 32 + lane;
                            ok[u] = r + u < rows && i < arr.n_elems;
                            idx[u] = ok[u] ? i : i0;
                        }
                        if (ok0) {
                            ptr.read_n<4>(idx, x);
#pragma unroll
                            for (int u = 0; u < 4; u++) v += ok[u] ? x[u] : 0;
                        }
                    }
                }
            }
            ptr.fini();
        }
        warp_sum_to(v, sum_out);
    }
};

struct FlushWork {
    page_cache_d_t pc;

    __device__ void operator()(uint32_t vb, uint32_t nvb) const
    {
        const uint32_t lane = threadIdx.x & 31u;
        const uint32_t wpb = blockDim.x >> 5;
        const uint64_t warp = (uint64_t)vb * wpb + (threadIdx.x >> 5);
        const uint64_t nwarps = (uint64_t)nvb * wpb;
        for (uint64_t s0 = warp * 32; s0 < pc.n_slots; s0 += nwarps * 32) {
            const uint64_t s = s0 + lane;
            uint32_t st = 0;
            uint64_t tag = BAM_TAG_NONE;
            if (s < pc.n_slots) { st = ld_acquire_gpu(&pc.slots[s].state); tag = ld_relaxed_gpu(&pc.slots[s].tag); }
            const bool dirty = (st & (BAM_VALID | BAM_DIRTY)) == (BAM_VALID | BAM_DIRTY) && tag != BAM_TAG_NONE;
            if (!__any_sync(0xffffffffu, dirty)) continue;
            const int rc = warp_write_back(0xffffffffu, dirty, pc, tag, (uint32_t)s);
            if (dirty && rc == BAM_OK) atom_and_release(&pc.slots[s].state, ~BAM_DIRTY);
            if (__any_sync(0xffffffffu, rc != BAM_OK)) break;
        }
    }
};

/* ---- cache benchmark: a warp reads whole pages -----------------------------------------------
 * Hit data is staged through shared memory: the warp pins 32 pages at once (one look-up and one
 * pin per lane, side by side), then streams them through its two 4 KiB stages of the block's
 * dynamic shared memory with bulk-async loads (two pages in flight per warp), sums each page from
 * shared memory with 128-bit loads, and finally unpins all 32. */
struct PageScanWork {
    range_d_t<uint64_t> r;
    uint64_t n_pages;
    const uint64_t* pages;
    uint64_t first_page;
    uint64_t* sum_out;

    __device__ void operator()(uint32_t vb, uint32_t nvb) const
    {
        const uint32_t lane = threadIdx.x & 31u;
        const uint32_t wib = threadIdx.x >> 5;
        const uint32_t wpb = blockDim.x >> 5;
        const uint64_t warp = (uint64_t)vb * wpb + wib;
        const uint64_t nwarps = (uint64_t)nvb * wpb;
        const uint32_t psz = (uint32_t)r.cache.page_size;
        /* two stages per warp; pages larger than a stage are streamed in 4 KiB pieces */
        const uint32_t stage0 = smem_u32(bam_dyn_smem + (size_t)(wib * 2) * BAM_EMU_STAGE_BYTES);
        const uint32_t bar0 = smem_u32(bam_dyn_smem + (size_t)BAM_EMU_STAGES * BAM_EMU_STAGE_BYTES + (wib * 2) * 8);
        if (lane == 0) { mbar_init(bar0, 1); mbar_init(bar0 + 8, 1); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        uint32_t parity = 0;                                   /* bit s = parity stage s completes next */
        uint64_t sum = 0;
        bool failed = false;
        for (uint64_t p0 = warp * 32; p0 < n_pages && !failed; p0 += nwarps * 32) {
            const uint64_t pi = p0 + lane;
            const bool have = pi < n_pages;
            const uint64_t page = have ? (pages ? pages[pi] : first_page + pi) : 0;
            const uint32_t slot = range_pin_page(r, 0xffffffffu, have, page, 1, (uint32_t)warp);
            const uint32_t ok = __ballot_sync(0xffffffffu, have && slot != BAM_SLOT_ERR);
            if (__any_sync(0xffffffffu, have && slot == BAM_SLOT_ERR)) failed = true;
            /* the pieces of all pinned pages, in order: piece q = (lane q / ppp, offset (q % ppp) * 4 KiB) */
            const uint32_t ppp = (psz + BAM_EMU_STAGE_BYTES - 1) / BAM_EMU_STAGE_BYTES;
            const uint32_t plen = psz < BAM_EMU_STAGE_BYTES ? psz : BAM_EMU_STAGE_BYTES;
            const uint32_t n_lanes_ok = __popc(ok);
            const uint32_t n_pieces = n_lanes_ok * ppp;
            const uint64_t my_base = (ok >> lane) & 1u ? r.get_cache_page_addr(slot) : 0;
            /* issue piece q into stage q & 1 */
            uint32_t inflight = 0;                                 /* bit s: stage s has a bulk load under way */
            auto issue = [&](uint32_t q) {
                const uint32_t src_lane = __fns(ok, 0, (int)(q / ppp) + 1);
                const uint64_t base = __shfl_sync(0xffffffffu, my_base, src_lane);
                const uint32_t st = q & 1u;
                if (lane == 0) {
                    mbar_expect_tx(bar0 + st * 8, plen);
                    bulk_load(stage0 + st * BAM_EMU_STAGE_BYTES, reinterpret_cast<const void*>(base + (uint64_t)(q % ppp) * BAM_EMU_STAGE_BYTES), plen, bar0 + st * 8);
                }
                inflight |= 1u << st;
            };
            /* wait for stage st's load, bounded like every other wait of the library; false = gave up */
            auto wait_stage = [&](uint32_t st, uint64_t detail) {
                const uint64_t t0 = global_timer_ns();
                uint32_t polls = 0;
                while (!mbar_test(bar0 + st * 8, (parity >> st) & 1u)) {
                    if (((++polls) & 1023u) == 0u) {
                        if (global_timer_ns() - t0 > r.cache.status->spin_timeout_ns) {
                            status_fail(r.cache.status, BAM_ETIMEDOUT, BAM_AT_TMA, detail);
                            return false;
                        }
                    }
                }
                parity ^= 1u << st;
                inflight &= ~(1u << st);
                return true;
            };
            if (n_pieces > 0) issue(0);
            if (n_pieces > 1) issue(1);
            for (uint32_t q = 0; q < n_pieces; q++) {
                const uint32_t st = q & 1u;
                /* a failure anywhere in the launch ends the scan: nothing more is read or issued */
                if (!wait_stage(st, q) || status_bad(r.cache.status)) { failed = true; break; }
                const uint8_t* sm = bam_dyn_smem + (size_t)(wib * 2 + st) * BAM_EMU_STAGE_BYTES;
#pragma unroll
                for (uint32_t o = lane * 16; o < BAM_EMU_STAGE_BYTES; o += 512) {
                    if (o < plen) {
                        const uint4 v = *reinterpret_cast<const uint4*>(sm + o);
                        sum += (((uint64_t)v.y << 32) | v.x) + (((uint64_t)v.w << 32) | v.z);
                    }
                }
                __syncwarp();                                      /* everyone has read the stage       */
                if (q + 2 < n_pieces) issue(q + 2);
            }
            /* leaving early: let the loads that are still under way land first (bounded), so that no bulk
             * copy targets this block's shared memory after the block has gone */
            if (failed) {
                for (uint32_t st = 0; st < 2; st++)
                    if ((inflight >> st) & 1u) (void)wait_stage(st, 0xffffffffull);
            }
            if ((ok >> lane) & 1u) r.release_page(slot, 1);
        }
        __syncwarp();
        warp_sum_to(sum, sum_out);
    }
};

/* ====================================================================================== */
/* C ABI                                                                                   */
/* ====================================================================================== */

extern "C" const char* bam_version(void) { return "bam_b200 0.1 (sm_100a)"; }

extern "C" const char* bam_strerror(int code)
{
    switch (code) {
    case BAM_OK: return "success";
    case BAM_EIO: return "I/O error (NVMe completion status or earlier device-side failure)";
    case BAM_E2BIG: return "size exceeds the fixed limit of this entry point";
    case BAM_ENOMEM: return "out of memory";
    case BAM_EBUSY: return "resource busy";
    case BAM_EINVAL: return "invalid argument";
    case BAM_ENOSPC: return "page table full";
    case BAM_ERANGE: return "index outside the array";
    case BAM_ETIMEDOUT: return "a device-side wait exceeded its limit";
    case BAM_ECUDA: return cudaGetErrorString(g_last_cuda);
    default: return "unknown error";
    }
}

static size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
static uint32_t log2_u32(uint64_t x) { uint32_t l = 0; while ((1ull << l) < x) l++; return l; }

/* The status block a controller's waits report into: its own, or its group's. */
static bam_status_t* status_block(bam_ctrl* c) { return c->lead ? c->lead->d_status : c->d_status; }

/* Build the power-on image of every queue structure on the host and upload it. */
static int upload_queue_image(bam_ctrl* c)
{
    std::vector<uint8_t> img(c->arena_bytes, 0);
    std::vector<bam_emu_qp_t> emu_qps(c->n_qps);
    memset(emu_qps.data(), 0, emu_qps.size() * sizeof(bam_emu_qp_t));
    /* a controller that backs a multi-controller cache reports into the status block of the
     * cache's first controller, so that every waiter of a launch sees the same error state */
    bam_status_t* const d_status = status_block(c);
    uint8_t* dev = (uint8_t*)c->arena;
    auto host_of = [&](void* devp) { return img.data() + ((uint8_t*)devp - dev); };
    const uint32_t qs = c->qdepth;
    for (uint32_t q = 0; q < c->n_qps; q++) {
        QueuePair* qp = (QueuePair*)host_of(c->d_qps + q);
        qp->pageSize = 4096;
        qp->block_size = c->lba_bytes;
        qp->block_size_log = log2_u32(c->lba_bytes);
        qp->block_size_minus_1 = c->lba_bytes - 1;
        qp->nvmNamespace = 1;
        qp->qp_id = (uint16_t)(q + 1);
        for (int is_cq = 0; is_cq < 2; is_cq++) {
            nvm_queue_t* nq = is_cq ? &qp->cq : &qp->sq;
            nq->qs = qs; nq->qs_minus_1 = qs - 1; nq->qs_log2 = log2_u32(qs);
            nq->no = (uint16_t)(q + 1);
            nq->es = is_cq ? sizeof(nvm_cpl_t) : sizeof(nvm_cmd_t);
            nq->phase = 1; nq->local = c->sys_scope ? 0 : 1;
            nq->status = d_status;
            nq->db = c->d_doorbells + (size_t)(2 * (q + 1) + is_cq) * BAM_DB_STRIDE_WORDS;
            nq->vaddr = is_cq ? (void*)(c->d_cq_mem + (size_t)q * qs) : (void*)(c->d_sq_mem + (size_t)q * qs);
            nq->ioaddr = (uint64_t)nq->vaddr;
            nq->tickets = c->d_tickets + (size_t)q * qs;
            nq->tail_mark = c->d_marks + (size_t)q * qs;
            nq->cid = c->d_cids + (size_t)q * BAM_CID_SPACE;
        }
        uint32_t* tk = (uint32_t*)host_of(c->d_tickets + (size_t)q * qs);
        for (uint32_t i = 0; i < qs; i++) tk[i] = i;            /* slot i is first used by ticket i */
        bam_emu_qp_t* e = &emu_qps[q];
        e->sq_mem = c->d_sq_mem + (size_t)q * qs;
        e->cq_mem = c->d_cq_mem + (size_t)q * qs;
        e->sq_db = c->d_doorbells + (size_t)(2 * (q + 1)) * BAM_DB_STRIDE_WORDS;
        e->cq_db = c->d_doorbells + (size_t)(2 * (q + 1) + 1) * BAM_DB_STRIDE_WORDS;
        e->qs = qs; e->qs_log2 = log2_u32(qs);
        e->cq_qs = qs; e->cq_qs_log2 = e->qs_log2;
        e->sqid = e->cqid = (uint16_t)(q + 1);
        e->ctrl_index = c->group_index;
        e->store = c->store_dev; e->store_bytes = c->store_bytes;
        e->fault = c->d_fault; e->served = c->d_served;
    }
    Controller* ctl = (Controller*)host_of(c->d_ctrl);
    ctl->d_qps = c->d_qps; ctl->n_qps = c->n_qps; ctl->page_size = 4096;
    ctl->blk_size = c->lba_bytes; ctl->blk_size_log = log2_u32(c->lba_bytes);
    ctl->status = d_status;
    bam_status_t* st = (bam_status_t*)host_of(c->d_status);
    st->spin_timeout_ns = c->spin_timeout_ns;
    st->launch_timeout_ns = c->launch_timeout_ns;
    CK(cudaMemcpy(c->arena, img.data(), c->arena_bytes, cudaMemcpyHostToDevice));
    /* the controller-side queue state lives in the arena, or in the group's array once grouped */
    CK(cudaMemcpy(c->d_emu_qps, emu_qps.data(), emu_qps.size() * sizeof(bam_emu_qp_t), cudaMemcpyHostToDevice));
    return BAM_OK;
}

extern "C" int bam_ctrl_create(bam_ctrl_t* out, int device, uint64_t store_bytes, uint32_t lba_bytes,
                               uint32_t n_queues, uint32_t queue_depth)
{
    if (!out) return BAM_EINVAL;
    *out = nullptr;
    if (lba_bytes != 512 && lba_bytes != 4096) return BAM_EINVAL;
    if (n_queues == 0 || n_queues > 1024) return BAM_EINVAL;
    if (queue_depth < 2 || queue_depth > 1024 || (queue_depth & (queue_depth - 1))) return BAM_EINVAL;
    if (store_bytes == 0 || store_bytes % 4096) return BAM_EINVAL;
    CK(cudaSetDevice(device));
    bam_ctrl* c = new (std::nothrow) bam_ctrl();
    if (!c) return BAM_ENOMEM;
    c->device = device;
    cudaDeviceProp prop;
    cudaError_t e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) { g_last_cuda = e; delete c; return BAM_ECUDA; }
    c->num_sms = prop.multiProcessorCount;
    c->store_bytes = store_bytes; c->lba_bytes = lba_bytes;
    c->n_qps = n_queues; c->qdepth = queue_depth;
    c->spin_timeout_ns = 20ull * 1000 * 1000 * 1000;
    c->launch_timeout_ns = 300ull * 1000 * 1000 * 1000;

    e = cudaHostAlloc((void**)&c->store_host, store_bytes, cudaHostAllocMapped | cudaHostAllocPortable);
    if (e != cudaSuccess) { g_last_cuda = e; (void)cudaGetLastError(); delete c; return BAM_ENOMEM; }
    e = cudaHostGetDevicePointer((void**)&c->store_dev, c->store_host, 0);
    if (e != cudaSuccess) { g_last_cuda = e; cudaFreeHost(c->store_host); delete c; return BAM_ECUDA; }

    /* one device arena for every queue structure */
    const size_t qs = queue_depth, nq = n_queues;
    size_t off = 0;
    auto take = [&](size_t bytes, size_t align) { off = align_up(off, align); size_t o = off; off += bytes; return o; };
    const size_t o_sq = take(nq * qs * sizeof(nvm_cmd_t), 4096);
    const size_t o_cq = take(nq * qs * sizeof(nvm_cpl_t), 4096);
    const size_t o_tk = take(nq * qs * 4, 256);
    const size_t o_mk = take(nq * qs * 4, 256);
    const size_t o_cid = take(nq * (size_t)BAM_CID_SPACE * 4, 256);
    const size_t o_db = take((2 * (nq + 1)) * BAM_DB_STRIDE_WORDS * 4, 256);
    const size_t o_eqp = take(nq * sizeof(bam_emu_qp_t), 256);
    const size_t o_qp = take(nq * sizeof(QueuePair), 256);
    const size_t o_ctl = take(sizeof(Controller), 256);
    const size_t o_st = take(sizeof(bam_status_t), 256);
    const size_t o_rem = take(4, 256);
    const size_t o_flt = take(sizeof(bam_fault_t), 256);
    const size_t o_srv = take(8, 256);
    c->arena_bytes = align_up(off, 4096);
    e = cudaMalloc(&c->arena, c->arena_bytes);
    if (e != cudaSuccess) { g_last_cuda = e; (void)cudaGetLastError(); cudaFreeHost(c->store_host); delete c; return BAM_ENOMEM; }
    uint8_t* a = (uint8_t*)c->arena;
    c->d_sq_mem = (nvm_cmd_t*)(a + o_sq); c->d_cq_mem = (nvm_cpl_t*)(a + o_cq);
    c->d_tickets = (uint32_t*)(a + o_tk); c->d_marks = (uint32_t*)(a + o_mk); c->d_cids = (uint32_t*)(a + o_cid);
    c->d_doorbells = (uint32_t*)(a + o_db); c->d_emu_qps = (bam_emu_qp_t*)(a + o_eqp);
    c->d_qps = (QueuePair*)(a + o_qp); c->d_ctrl = (Controller*)(a + o_ctl);
    c->d_status = (bam_status_t*)(a + o_st); c->d_remaining = (uint32_t*)(a + o_rem);
    c->d_fault = (bam_fault_t*)(a + o_flt); c->d_served = (uint64_t*)(a + o_srv);

    c->emu.qps = c->d_emu_qps; c->emu.n_qps = n_queues;
    c->emu.n_ctrl_blocks = BAM_DEFAULT_CTRL_BLOCKS;
    c->emu.lba_log2 = log2_u32(lba_bytes); c->emu.mps_log2 = 12;
    c->emu.batch = 32; c->emu.sys_scope = c->sys_scope;
    c->emu.consumers_remaining = c->d_remaining; c->emu.status = c->d_status;
    int rc = upload_queue_image(c);
    if (rc != BAM_OK) { cudaFree(c->arena); cudaFreeHost(c->store_host); delete c; return rc; }
    *out = c;
    return BAM_OK;
}

extern "C" int bam_ctrl_destroy(bam_ctrl_t c)
{
    if (!c) return BAM_EINVAL;
    cudaSetDevice(c->device);
    cudaDeviceSynchronize();
    cudaFree(c->arena);
    cudaFreeHost(c->store_host);
    delete c;
    return BAM_OK;
}

extern "C" void* bam_ctrl_store_host(bam_ctrl_t c) { return c ? c->store_host : nullptr; }
extern "C" uint64_t bam_ctrl_store_bytes(bam_ctrl_t c) { return c ? c->store_bytes : 0; }

extern "C" int bam_ctrl_fill_store(bam_ctrl_t c, uint64_t seed, uint64_t first_elem, void* stream)
{
    if (!c) return BAM_EINVAL;
    CK(cudaSetDevice(c->device));
    k_fill_store<<<c->num_sms * 8, 256, 0, (cudaStream_t)stream>>>((uint64_t*)c->store_dev, c->store_bytes / 8, seed, first_elem);
    CK(cudaGetLastError());
    return BAM_OK;
}

extern "C" int bam_ctrl_fill_store_striped(bam_ctrl_t c, uint64_t seed, uint64_t first_elem, uint32_t page_bytes, uint32_t stripe,
                                           uint32_t n_stripes, void* stream)
{
    if (!c || n_stripes == 0 || stripe >= n_stripes || page_bytes < 8 || (page_bytes & (page_bytes - 1))) return BAM_EINVAL;
    CK(cudaSetDevice(c->device));
    k_fill_store_striped<<<c->num_sms * 8, 256, 0, (cudaStream_t)stream>>>((uint64_t*)c->store_dev, c->store_bytes / 8, seed, first_elem,
                                                                         log2_u32(page_bytes / 8), stripe, n_stripes);
    CK(cudaGetLastError());
    return BAM_OK;
}

extern "C" int bam_ctrl_write_store(bam_ctrl_t c, uint64_t byte_offset, const void* src, uint64_t bytes)
{
    if (!c || !src || byte_offset + bytes > c->store_bytes || byte_offset + bytes < byte_offset) return BAM_EINVAL;
    memcpy(c->store_host + byte_offset, src, bytes);
    return BAM_OK;
}

extern "C" int bam_ctrl_set_launch_timeout(bam_ctrl_t c, uint64_t launch_timeout_ns)
{
    if (!c || launch_timeout_ns == 0) return BAM_EINVAL;
    CK(cudaSetDevice(c->device));
    CK(cudaDeviceSynchronize());
    c->launch_timeout_ns = launch_timeout_ns;
    CK(cudaMemcpy(&status_block(c)->launch_timeout_ns, &launch_timeout_ns, 8, cudaMemcpyHostToDevice));
    return BAM_OK;
}

extern "C" int bam_ctrl_configure(bam_ctrl_t c, uint32_t n_ctrl_blocks, uint32_t batch, uint64_t spin_timeout_ns)
{
    if (!c) return BAM_EINVAL;
    CK(cudaSetDevice(c->device));
    if (n_ctrl_blocks) c->emu.n_ctrl_blocks = n_ctrl_blocks;
    if (batch) { if (batch > 32) return BAM_EINVAL; c->emu.batch = batch; }
    if (spin_timeout_ns) {
        c->spin_timeout_ns = spin_timeout_ns;
        CK(cudaDeviceSynchronize());
        CK(cudaMemcpy(&status_block(c)->spin_timeout_ns, &spin_timeout_ns, 8, cudaMemcpyHostToDevice));
    }
    return BAM_OK;
}

extern "C" int bam_ctrl_set_scope(bam_ctrl_t c, int system_scope)
{
    if (!c) return BAM_EINVAL;
    CK(cudaSetDevice(c->device));
    CK(cudaDeviceSynchronize());
    c->sys_scope = system_scope ? 1u : 0u;
    c->emu.sys_scope = c->sys_scope;
    return upload_queue_image(c);
}

extern "C" int bam_ctrl_set_max_grid(bam_ctrl_t c, uint32_t max_grid)
{
    if (!c) return BAM_EINVAL;
    c->max_grid = max_grid;
    c->emu.max_grid = max_grid;         /* launches through the device header see it in the descriptor */
    return BAM_OK;
}

extern "C" int bam_ctrl_inject_fault(bam_ctrl_t c, uint32_t mode, uint64_t nth, uint32_t status)
{
    if (!c || mode > BAM_FAULT_STATUS) return BAM_EINVAL;
    CK(cudaSetDevice(c->device));
    CK(cudaDeviceSynchronize());
    bam_fault_t f = { mode, status, nth, 0 };
    CK(cudaMemcpy(c->d_fault, &f, sizeof f, cudaMemcpyHostToDevice));
    return BAM_OK;
}

extern "C" int bam_ctrl_status(bam_ctrl_t c, bam_status_out_t* out, int clear)
{
    if (!c || !out) return BAM_EINVAL;
    CK(cudaSetDevice(c->device));
    CK(cudaDeviceSynchronize());
    bam_status_t st;
    CK(cudaMemcpy(&st, status_block(c), sizeof st, cudaMemcpyDeviceToHost));
    out->code = st.code; out->where = st.where; out->detail = st.detail;
    if (clear && st.code) {
        st.code = 0; st.where = 0; st.detail = 0;
        CK(cudaMemcpy(status_block(c), &st, sizeof st, cudaMemcpyHostToDevice));
    }
    return BAM_OK;
}

extern "C" int bam_ctrl_profile(bam_ctrl_t c, uint64_t* out32, int reset)
{
    if (!c || !out32) return BAM_EINVAL;
    CK(cudaSetDevice(c->device));
    CK(cudaDeviceSynchronize());
    CK(cudaMemcpy(out32, status_block(c)->prof, sizeof(uint64_t) * 32, cudaMemcpyDeviceToHost));
    if (reset) CK(cudaMemset(status_block(c)->prof, 0, sizeof(uint64_t) * 32));
    return BAM_OK;
}

extern "C" int bam_ctrl_served(bam_ctrl_t c, uint64_t* out, int reset)
{
    if (!c || !out) return BAM_EINVAL;
    CK(cudaSetDevice(c->device));
    CK(cudaDeviceSynchronize());
    CK(cudaMemcpy(out, c->d_served, 8, cudaMemcpyDeviceToHost));
    if (reset) CK(cudaMemset(c->d_served, 0, 8));
    return BAM_OK;
}

extern "C" int bam_ctrl_reset_queues(bam_ctrl_t c)
{
    if (!c) return BAM_EINVAL;
    CK(cudaSetDevice(c->device));
    CK(cudaDeviceSynchronize());
    return upload_queue_image(c);
}

extern "C" void* bam_ctrl_device_controller(bam_ctrl_t c) { return c ? c->d_ctrl : nullptr; }

extern "C" int bam_ctrl_emu_descriptor(bam_ctrl_t c, void* out, size_t out_bytes)
{
    if (!c || !out || out_bytes < sizeof(bam_emu_d_t)) return BAM_EINVAL;
    memcpy(out, &c->emu, sizeof(bam_emu_d_t));
    return BAM_OK;
}

/* ---- cache -------------------------------------------------------------------------------- */

static int cache_reset_device(bam_cache* pc)
{
    k_init_cache<<<pc->ctrl->num_sms * 4, 256>>>(pc->d.slots, pc->d.n_slots, pc->d.table, pc->n_buckets * BAM_BUCKET_WORDS);
    CK(cudaGetLastError());
    CK(cudaMemset(pc->d.clock_hand, 0, 8 * BAM_HAND_STRIDE * BAM_MAX_HANDS));
    CK(cudaMemset(pc->d.stats, 0, sizeof(bam_stat_stripe_t) * BAM_STAT_STRIPES));
    CK(cudaDeviceSynchronize());
    return BAM_OK;
}

static void cache_free_device(bam_cache* pc)
{
    page_cache_d_t& d = pc->d;
    cudaFree(d.base_addr); cudaFree(d.slots); cudaFree(d.table); cudaFree(d.clock_hand);
    cudaFree(d.stats); cudaFree(d.range_page_starts); cudaFree(d.range_dists); cudaFree(pc->prp_lists_raw);
    cudaFree(d.d_ctrls); cudaFree(pc->d_group_qps);
}

/* Undo the grouping of bam_cache_create_multi: every member gets its own controller-side queue
 * state and status block back (queues are reset; nothing is in flight when a cache is destroyed). */
static void cache_ungroup(bam_cache* pc)
{
    for (bam_ctrl* m : pc->members) {
        if (m->group != pc) continue;
        m->group = nullptr; m->lead = nullptr; m->group_index = 0;
        m->d_emu_qps = m->own_emu_qps;
        m->emu.qps = m->own_emu_qps; m->emu.n_qps = m->n_qps;
        (void)upload_queue_image(m);
    }
}

extern "C" int bam_cache_create_multi(bam_cache_t* out, const bam_ctrl_t* ctrls, uint32_t n_ctrls, uint32_t page_size,
                                      uint64_t n_pages)
{
    if (!out) return BAM_EINVAL;
    *out = nullptr;
    if (!ctrls || n_ctrls == 0 || n_ctrls > BAM_MAX_CTRLS || n_pages == 0 || n_pages > BAM_MAX_CACHE_SLOTS) return BAM_EINVAL;
    bam_ctrl* ctrl = ctrls[0];
    if (!ctrl) return BAM_EINVAL;
    if (page_size < 512 || (page_size & (page_size - 1)) || page_size < ctrl->lba_bytes || page_size > (1u << 20)) return BAM_EINVAL;
    for (uint32_t k = 0; k < n_ctrls; k++) {
        bam_ctrl* m = ctrls[k];
        if (!m || m->device != ctrl->device || m->lba_bytes != ctrl->lba_bytes || m->sys_scope != ctrl->sys_scope) return BAM_EINVAL;
        for (uint32_t j = 0; j < k; j++) if (ctrls[j] == m) return BAM_EINVAL;
        if (n_ctrls > 1 && m->group) return BAM_EBUSY;      /* a controller backs one multi-controller cache at a time */
    }
    CK(cudaSetDevice(ctrl->device));
    bam_cache* pc = new (std::nothrow) bam_cache();
    if (!pc) return BAM_ENOMEM;
    pc->ctrl = ctrl;
    uint64_t want = (n_pages * 2 + 6) / 7;           /* load factor <= 0.5 over 7-entry buckets */
    pc->n_buckets = 1; while (pc->n_buckets < want) pc->n_buckets <<= 1;
    page_cache_d_t& d = pc->d;
    memset(&d, 0, sizeof d);
    d.page_size = page_size; d.page_size_minus_1 = page_size - 1; d.page_size_log = log2_u32(page_size);
    d.n_slots = (uint32_t)n_pages;
    for (d.n_hands = 1; d.n_hands < BAM_MAX_HANDS && (uint64_t)d.n_hands * 2 * BAM_SLOTS_PER_HAND <= n_pages;) d.n_hands <<= 1;
    d.bucket_mask = (uint32_t)(pc->n_buckets - 1);
    d.n_blocks_per_page = page_size / ctrl->lba_bytes;
    d.d_ctrl = ctrl->d_ctrl; d.status = status_block(ctrl); d.n_ctrls = n_ctrls;
    d.n_ranges_bits = BAM_RANGE_BITS; d.n_ranges_mask = BAM_MAX_RANGES - 1;
    const uint32_t chunks = page_size / 4096;
    /* a slot's PRP list has chunks - 1 entries.  Lists are laid out at a power-of-two stride from a
     * page-aligned base, so none crosses a memory page: the last 8 bytes of a list page mean "link to
     * the next list page" to an NVMe controller whenever entries still follow */
    const uint32_t list_entries = chunks > 2 ? chunks - 1 : 0;
    d.prp_list_stride = 0;
    if (list_entries) for (d.prp_list_stride = 1; d.prp_list_stride < list_entries;) d.prp_list_stride <<= 1;
    uint32_t total_qps = 0;
    for (uint32_t k = 0; k < n_ctrls; k++) total_qps += ctrls[k]->n_qps;
    cudaError_t e = cudaSuccess;
    auto alloc = [&](void** p, size_t bytes) { if (e == cudaSuccess) e = cudaMalloc(p, bytes); };
    alloc((void**)&d.base_addr, n_pages * (size_t)page_size);
    alloc((void**)&d.slots, n_pages * sizeof(bam_slot_t));
    alloc((void**)&d.table, pc->n_buckets * BAM_BUCKET_WORDS * 4);
    alloc((void**)&d.clock_hand, 8 * BAM_HAND_STRIDE * BAM_MAX_HANDS);
    alloc((void**)&d.stats, sizeof(bam_stat_stripe_t) * BAM_STAT_STRIPES);
    alloc((void**)&d.range_page_starts, 8 * BAM_MAX_RANGES);
    alloc((void**)&d.range_dists, 4 * BAM_MAX_RANGES);
    alloc((void**)&d.d_ctrls, sizeof(Controller*) * n_ctrls);
    if (d.prp_list_stride) {
        alloc(&pc->prp_lists_raw, n_pages * d.prp_list_stride * 8 + 4096);
        d.prp_lists = reinterpret_cast<uint64_t*>(((uintptr_t)pc->prp_lists_raw + 4095) / 4096 * 4096);
    }
    if (n_ctrls > 1) alloc((void**)&pc->d_group_qps, sizeof(bam_emu_qp_t) * total_qps);
    if (e != cudaSuccess) {
        g_last_cuda = e; (void)cudaGetLastError();
        cache_free_device(pc);
        delete pc;
        return BAM_ENOMEM;
    }
    auto fail = [&](int rc) { cache_ungroup(pc); cache_free_device(pc); delete pc; return rc; };
    if (d.prp_list_stride) {
        std::vector<uint64_t> lists(n_pages * d.prp_list_stride);
        for (uint64_t s = 0; s < n_pages; s++)
            for (uint32_t k = 0; k < list_entries; k++)
                lists[s * d.prp_list_stride + k] = (uint64_t)(d.base_addr + s * page_size + (size_t)(k + 1) * 4096);
        if (cudaMemcpy(d.prp_lists, lists.data(), lists.size() * 8, cudaMemcpyHostToDevice) != cudaSuccess) return fail(BAM_ECUDA);
    }
    std::vector<Controller*> h_ctrls(n_ctrls);
    for (uint32_t k = 0; k < n_ctrls; k++) h_ctrls[k] = ctrls[k]->d_ctrl;
    if (cudaMemcpy(d.d_ctrls, h_ctrls.data(), sizeof(Controller*) * n_ctrls, cudaMemcpyHostToDevice) != cudaSuccess ||
        cudaMemset(d.range_page_starts, 0, 8 * BAM_MAX_RANGES) != cudaSuccess ||
        cudaMemset(d.range_dists, 0, 4 * BAM_MAX_RANGES) != cudaSuccess)
        return fail(BAM_ECUDA);
    if (n_ctrls > 1) {
        /* One launch serves every member: their controller-side queue state moves into one
         * contiguous array, which the first controller's launch descriptor then covers, and all of
         * them report into the first controller's status block. */
        if (cudaDeviceSynchronize() != cudaSuccess) return fail(BAM_ECUDA);
        uint32_t at = 0;
        for (uint32_t k = 0; k < n_ctrls; k++) {
            bam_ctrl* m = ctrls[k];
            pc->members.push_back(m);
            m->group = pc; m->lead = (k == 0) ? nullptr : ctrl; m->group_index = k;
            m->own_emu_qps = m->emu.qps;
            m->d_emu_qps = pc->d_group_qps + at;
            m->emu.qps = m->d_emu_qps;
            at += m->n_qps;
            const int rc = upload_queue_image(m);
            if (rc != BAM_OK) return fail(rc);
        }
        ctrl->emu.qps = pc->d_group_qps; ctrl->emu.n_qps = total_qps;
    }
    int rc = cache_reset_device(pc);
    if (rc != BAM_OK) return fail(rc);
    *out = pc;
    return BAM_OK;
}

extern "C" int bam_cache_create(bam_cache_t* out, bam_ctrl_t ctrl, uint32_t page_size, uint64_t n_pages)
{
    return bam_cache_create_multi(out, &ctrl, 1, page_size, n_pages);
}

extern "C" int bam_cache_destroy(bam_cache_t pc)
{
    if (!pc) return BAM_EINVAL;
    cudaSetDevice(pc->ctrl->device);
    cudaDeviceSynchronize();
    cache_ungroup(pc);
    cache_free_device(pc);
    delete pc;
    return BAM_OK;
}

extern "C" int bam_cache_stats(bam_cache_t pc, bam_cache_stats_t* out, int reset)
{
    if (!pc || !out) return BAM_EINVAL;
    CK(cudaSetDevice(pc->ctrl->device));
    CK(cudaDeviceSynchronize());
    bam_stat_stripe_t h[BAM_STAT_STRIPES];
    CK(cudaMemcpy(h, pc->d.stats, sizeof h, cudaMemcpyDeviceToHost));
    out->hits = out->misses = out->read_ios = 0;
    for (int i = 0; i < BAM_STAT_STRIPES; i++) { out->hits += h[i].hits; out->misses += h[i].misses; out->read_ios += h[i].read_ios; }
    if (reset) CK(cudaMemset(pc->d.stats, 0, sizeof h));
    return BAM_OK;
}

extern "C" int bam_cache_invalidate(bam_cache_t pc)
{
    if (!pc) return BAM_EINVAL;
    CK(cudaSetDevice(pc->ctrl->device));
    CK(cudaDeviceSynchronize());
    return cache_reset_device(pc);
}

extern "C" int bam_cache_invalidate_async(bam_cache_t pc, void* stream)
{
    if (!pc) return BAM_EINVAL;
    CK(cudaSetDevice(pc->ctrl->device));
    cudaStream_t s = (cudaStream_t)stream;
    k_init_cache<<<pc->ctrl->num_sms * 4, 256, 0, s>>>(pc->d.slots, pc->d.n_slots, pc->d.table, pc->n_buckets * BAM_BUCKET_WORDS);
    CK(cudaGetLastError());
    CK(cudaMemsetAsync(pc->d.clock_hand, 0, 8 * BAM_HAND_STRIDE * BAM_MAX_HANDS, s));
    return BAM_OK;
}

extern "C" int bam_cache_audit(bam_cache_t pc, uint64_t* violations)
{
    if (!pc || !violations) return BAM_EINVAL;
    CK(cudaSetDevice(pc->ctrl->device));
    CK(cudaDeviceSynchronize());
    unsigned long long* d_bad = nullptr;
    CK(cudaMalloc(&d_bad, 8));
    CK(cudaMemset(d_bad, 0, 8));
    k_audit<<<pc->ctrl->num_sms * 4, 256>>>(pc->d, pc->n_buckets, d_bad);
    cudaError_t e = cudaDeviceSynchronize();
    unsigned long long bad = 0;
    if (e == cudaSuccess) e = cudaMemcpy(&bad, d_bad, 8, cudaMemcpyDeviceToHost);
    cudaFree(d_bad);
    if (e != cudaSuccess) { g_last_cuda = e; return BAM_ECUDA; }
    *violations = bad;
    return BAM_OK;
}

extern "C" int bam_cache_descriptor(bam_cache_t pc, void* out, size_t out_bytes)
{
    if (!pc || !out || out_bytes < sizeof(page_cache_d_t)) return BAM_EINVAL;
    memcpy(out, &pc->d, sizeof(page_cache_d_t));
    return BAM_OK;
}

/* ---- arrays ----------------------------------------------------------------------------------- */

extern "C" int bam_array_create_ranges(bam_array_t* out, bam_cache_t pc, uint64_t n_elems, uint32_t elem_bytes,
                                       const bam_range_desc_t* ranges, uint32_t n_ranges)
{
    if (!out) return BAM_EINVAL;
    *out = nullptr;
    if (!pc || n_elems == 0 || (elem_bytes != 4 && elem_bytes != 8) || !ranges || n_ranges == 0) return BAM_EINVAL;
    if (pc->n_ranges + n_ranges > BAM_MAX_RANGES) return BAM_ENOSPC;
    const uint64_t psz = pc->d.page_size;
    const uint32_t n_ctrls = pc->d.n_ctrls;
    std::vector<range_d_t<uint64_t>> h(n_ranges);
    for (uint32_t k = 0; k < n_ranges; k++) {
        const bam_range_desc_t& d = ranges[k];
        if (d.index_end <= d.index_start || d.index_end > n_elems) return BAM_EINVAL;
        if (d.dist != BAM_DIST_REPLICATE && d.dist != BAM_DIST_STRIPE) return BAM_EINVAL;
        if (d.store_byte_offset % psz || d.page_start_offset >= psz || d.page_start_offset % elem_bytes) return BAM_EINVAL;
        for (uint32_t j = 0; j < k; j++)            /* index ranges must not overlap */
            if (d.index_start < ranges[j].index_end && ranges[j].index_start < d.index_end) return BAM_EINVAL;
        const uint64_t bytes = d.page_start_offset + (d.index_end - d.index_start) * elem_bytes;
        const uint64_t page_count = (bytes + psz - 1) / psz;
        /* bytes of the range that each controller must hold, from store_byte_offset on */
        const uint64_t per_ctrl = (d.dist == BAM_DIST_STRIPE && n_ctrls > 1) ? (page_count + n_ctrls - 1) / n_ctrls * psz : bytes;
        if (pc->members.empty()) {
            if (d.store_byte_offset + per_ctrl > pc->ctrl->store_bytes) return BAM_EINVAL;
        } else {
            for (bam_ctrl* m : pc->members)
                if (d.store_byte_offset + per_ctrl > m->store_bytes) return BAM_EINVAL;
        }
        range_d_t<uint64_t>& r = h[k];
        r.index_start = d.index_start; r.count = d.index_end; r.range_id = pc->n_ranges + k;
        r.page_start_offset = d.page_start_offset;
        r.page_start = d.store_byte_offset / psz;
        r.page_count = page_count;
        r.n_elems_per_page = psz / elem_bytes;
        r.dist = d.dist; r.pad_ = 0;
        r.cache = pc->d;
    }
    CK(cudaSetDevice(pc->ctrl->device));
    bam_array* a = new (std::nothrow) bam_array();
    if (!a) return BAM_ENOMEM;
    a->pc = pc; a->elem_bytes = elem_bytes; a->n_elems = n_elems; a->n_ranges = n_ranges;
    a->h_range = h[0];
    struct { uint64_t n_elems, start_offset, n_ranges; void* d_ranges; } h_arr;
    cudaError_t e = cudaMalloc(&a->d_range, sizeof(range_d_t<uint64_t>) * n_ranges);
    if (e == cudaSuccess) e = cudaMalloc(&a->d_array, sizeof h_arr);
    if (e == cudaSuccess) e = cudaMemcpy(a->d_range, h.data(), sizeof(range_d_t<uint64_t>) * n_ranges, cudaMemcpyHostToDevice);
    h_arr.n_elems = n_elems; h_arr.start_offset = ranges[0].store_byte_offset; h_arr.n_ranges = n_ranges; h_arr.d_ranges = a->d_range;
    if (e == cudaSuccess) e = cudaMemcpy(a->d_array, &h_arr, sizeof h_arr, cudaMemcpyHostToDevice);
    for (uint32_t k = 0; k < n_ranges && e == cudaSuccess; k++) {
        e = cudaMemcpy(pc->d.range_page_starts + h[k].range_id, &h[k].page_start, 8, cudaMemcpyHostToDevice);
        if (e == cudaSuccess) e = cudaMemcpy(pc->d.range_dists + h[k].range_id, &h[k].dist, 4, cudaMemcpyHostToDevice);
    }
    if (e != cudaSuccess) { g_last_cuda = e; cudaFree(a->d_range); cudaFree(a->d_array); delete a; return BAM_ECUDA; }
    pc->n_ranges += n_ranges;
    *out = a;
    return BAM_OK;
}

extern "C" int bam_array_create_dist(bam_array_t* out, bam_cache_t pc, uint64_t n_elems, uint32_t elem_bytes,
                                     uint64_t store_byte_offset, uint32_t dist)
{
    const bam_range_desc_t one = { 0, n_elems, store_byte_offset, 0, dist, 0 };
    return bam_array_create_ranges(out, pc, n_elems, elem_bytes, &one, 1);
}

extern "C" int bam_array_create(bam_array_t* out, bam_cache_t pc, uint64_t n_elems, uint32_t elem_bytes,
                                uint64_t store_byte_offset)
{
    return bam_array_create_dist(out, pc, n_elems, elem_bytes, store_byte_offset, BAM_DIST_REPLICATE);
}

extern "C" int bam_array_destroy(bam_array_t a)
{
    if (!a) return BAM_EINVAL;
    cudaSetDevice(a->pc->ctrl->device);
    cudaDeviceSynchronize();
    cudaFree(a->d_range); cudaFree(a->d_array);
    delete a;
    return BAM_OK;
}

extern "C" void* bam_array_device_ptr(bam_array_t a) { return a ? a->d_array : nullptr; }

/* ---- launchers --------------------------------------------------------------------------------- */

extern "C" int bam_launch_block_read_depth(bam_cache_t pc, uint64_t n_reqs, const uint64_t* pages_dev, uint64_t req_seed,
                                           uint32_t io_depth, uint32_t* crc_out_dev, uint64_t* sum_out_dev, void* stream)
{
    if (!pc || io_depth == 0 || io_depth > BAM_MAX_IO_DEPTH) return BAM_EINVAL;
    bam_ctrl* c = pc->ctrl;
    CK(cudaSetDevice(c->device));
    if (pc->d.page_size > 8192) return BAM_EINVAL;
    /* a warp's outstanding commands must stay below half the queue depth */
    if (32u * io_depth >= c->qdepth / 2 && io_depth > 1) return BAM_EINVAL;
    uint32_t grid = 0;
    int rc = fused_geometry<BlockReadWork>(c, &grid);
    if (rc) return rc;
    if (grid <= c->emu.n_ctrl_blocks) return BAM_EINVAL;
    /* every worker thread owns io_depth cache slots as its landing buffers */
    if ((uint64_t)(grid - c->emu.n_ctrl_blocks) * BAM_THREADS * io_depth > pc->d.n_slots) return BAM_ENOSPC;
    BlockReadWork w;
    w.pc = pc->d; w.n_reqs = n_reqs; w.pages = pages_dev; w.req_seed = req_seed;
    w.n_store_pages = c->store_bytes / pc->d.page_size;
    w.crc_out = crc_out_dev; w.sum_out = sum_out_dev; w.io_depth = io_depth;
    return launch_fused(c, w, (cudaStream_t)stream);
}

extern "C" int bam_launch_block_read(bam_cache_t pc, uint64_t n_reqs, const uint64_t* pages_dev, uint64_t req_seed,
                                     uint32_t* crc_out_dev, uint64_t* sum_out_dev, void* stream)
{
    return bam_launch_block_read_depth(pc, n_reqs, pages_dev, req_seed, 1, crc_out_dev, sum_out_dev, stream);
}

extern "C" int bam_launch_array_read(bam_array_t a, uint64_t n_lanes, uint64_t reqs_per_lane, const uint64_t* idx_dev,
                                     uint64_t access_seed, uint64_t* sum_out_dev, void* stream)
{
    if (!a || a->elem_bytes != 8) return BAM_EINVAL;
    bam_ctrl* c = a->pc->ctrl;
    CK(cudaSetDevice(c->device));
    if (a->n_ranges > 1) {
        ArrayReadRangesWork m;
        m.arr.n_elems = a->n_elems; m.arr.start_offset = 0; m.arr.n_ranges = a->n_ranges;
        m.arr.d_ranges = static_cast<range_d_t<uint64_t>*>(a->d_range);
        m.n_lanes = n_lanes; m.reqs_per_lane = reqs_per_lane; m.idx = idx_dev; m.access_seed = access_seed; m.sum_out = sum_out_dev;
        return launch_fused(c, m, (cudaStream_t)stream);
    }
    ArrayReadWork w;
    w.r = a->h_range; w.n_lanes = n_lanes; w.reqs_per_lane = reqs_per_lane; w.idx = idx_dev;
    w.access_seed = access_seed; w.sum_out = sum_out_dev;
    return launch_fused(c, w, (cudaStream_t)stream);
}

extern "C" int bam_launch_array_write(bam_array_t a, uint64_t n, const uint64_t* idx_dev, uint64_t val_seed, uint64_t addend,
                                      void* stream)
{
    if (!a || a->elem_bytes != 8 || !idx_dev) return BAM_EINVAL;
    bam_ctrl* c = a->pc->ctrl;
    CK(cudaSetDevice(c->device));
    ArrayWriteWork w;
    w.arr.n_elems = a->n_elems; w.arr.start_offset = 0; w.arr.n_ranges = a->n_ranges;
    w.arr.d_ranges = static_cast<range_d_t<uint64_t>*>(a->d_range);
    w.n = n; w.idx = idx_dev; w.val_seed = val_seed; w.addend = addend;
    return launch_fused(c, w, (cudaStream_t)stream);
}

extern "C" int bam_launch_thread_acquire(bam_array_t a, uint64_t first_page, uint64_t n_pages, uint32_t lanes,
                                         uint64_t* first_words_dev, void* stream)
{
    if (!a || a->elem_bytes != 8 || a->n_ranges != 1 || !first_words_dev || lanes == 0 || n_pages == 0) return BAM_EINVAL;
    if (first_page + n_pages > a->h_range.page_count || a->h_range.page_start_offset) return BAM_EINVAL;
    bam_ctrl* c = a->pc->ctrl;
    CK(cudaSetDevice(c->device));
    ThreadAcquireWork w;
    w.r = a->h_range; w.first_page = first_page; w.n_pages = n_pages; w.lanes = lanes; w.first_words = first_words_dev;
    return launch_fused(c, w, (cudaStream_t)stream);
}

extern "C" int bam_launch_bulk_io(bam_cache_t pc, uint64_t n_pages, uint64_t first_store_page, uint64_t first_slot, int write,
                                  void* stream)
{
    if (!pc || n_pages == 0) return BAM_EINVAL;
    bam_ctrl* c = pc->ctrl;
    if (first_slot + n_pages > pc->d.n_slots) return BAM_EINVAL;
    if ((first_store_page + n_pages) * pc->d.page_size > c->store_bytes) return BAM_EINVAL;
    CK(cudaSetDevice(c->device));
    BulkIoWork w;
    w.pc = pc->d; w.n_pages = n_pages; w.first_store_page = first_store_page; w.first_slot = first_slot;
    w.opcode = write ? NVM_IO_WRITE : NVM_IO_READ;
    return launch_fused(c, w, (cudaStream_t)stream);
}

extern "C" int bam_cache_copy(bam_cache_t pc, uint64_t first_slot, void* host, uint64_t bytes, int to_cache, void* stream)
{
    if (!pc || !host || first_slot * pc->d.page_size + bytes > (uint64_t)pc->d.n_slots * pc->d.page_size) return BAM_EINVAL;
    CK(cudaSetDevice(pc->ctrl->device));
    uint8_t* dev = pc->d.base_addr + first_slot * pc->d.page_size;
    if (to_cache) CK(cudaMemcpyAsync(dev, host, bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream));
    else CK(cudaMemcpyAsync(host, dev, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    return BAM_OK;
}

extern "C" int bam_launch_pattern_read_impl(bam_array_t a, uint32_t pattern, uint32_t impl, uint64_t n_elems, uint64_t n_warps,
                                            uint64_t n_pages_per_warp, uint64_t stride, const uint64_t* assignment_dev,
                                            uint64_t* sum_out_dev, void* stream)
{
    if (!a || a->elem_bytes != 8 || pattern > BAM_PATTERN_RANDOM_WARP || impl > BAM_IMPL_ARRAY || n_elems > a->n_elems) return BAM_EINVAL;
    const bool by_warp = pattern == BAM_PATTERN_SEQUENTIAL_WARP || pattern == BAM_PATTERN_RANDOM_WARP;
    if (by_warp && (n_warps == 0 || n_pages_per_warp == 0 || stride == 0)) return BAM_EINVAL;
    if ((pattern == BAM_PATTERN_RANDOM || pattern == BAM_PATTERN_RANDOM_WARP) && !assignment_dev) return BAM_EINVAL;
    bam_ctrl* c = a->pc->ctrl;
    CK(cudaSetDevice(c->device));
    if (a->n_ranges > 1 && impl == BAM_IMPL_ARRAY) return BAM_EINVAL;       /* that form reads through one range held by value */
    PatternWork w;
    w.arr.n_elems = a->n_elems; w.arr.start_offset = 0; w.arr.n_ranges = a->n_ranges;
    w.arr.d_ranges = static_cast<range_d_t<uint64_t>*>(a->d_range);
    w.rng = a->h_range;
    w.pattern = pattern; w.impl = impl; w.n_elems = n_elems; w.n_warps = n_warps; w.n_pages_per_warp = n_pages_per_warp; w.stride = stride;
    w.assignment = assignment_dev; w.sum_out = sum_out_dev;
    return launch_fused(c, w, (cudaStream_t)stream);
}

extern "C" int bam_launch_pattern_read(bam_array_t a, uint32_t pattern, uint64_t n_elems, uint64_t n_warps, uint64_t n_pages_per_warp,
                                       uint64_t stride, const uint64_t* assignment_dev, uint64_t* sum_out_dev, void* stream)
{
    return bam_launch_pattern_read_impl(a, pattern, BAM_IMPL_PTR, n_elems, n_warps, n_pages_per_warp, stride, assignment_dev, sum_out_dev,
                                        stream);
}

/* ---- command encoding, exposed for checks against other encoders ------------------------------------ */

__global__ void k_encode_rw(uint32_t cid, uint8_t opcode, uint32_t ns_id, uint64_t prp1, uint64_t prp2, uint64_t slba, uint32_t n_blks,
                            uint4* out)
{
    uint4 c0, c1, c2, c3;
    bam::nvm_cmd_rw_quarters(cid, opcode, ns_id, prp1, prp2, slba, n_blks, c0, c1, c2, c3);
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

extern "C" int bam_encode_rw_command(void* out64, uint16_t cid, uint8_t opcode, uint32_t ns_id, uint64_t prp1, uint64_t prp2,
                                     uint64_t start_lba, uint16_t n_blks, int on_device)
{
    if (!out64 || n_blks == 0) return BAM_EINVAL;
    if (!on_device) {
        /* the builders a host program (or a kernel) calls one after the other */
        nvm_cmd_t cmd;
        memset(&cmd, 0, sizeof cmd);
        bam::nvm_cmd_header(&cmd, cid, opcode, ns_id);
        bam::nvm_cmd_data_ptr(&cmd, prp1, prp2);
        bam::nvm_cmd_rw_blks(&cmd, start_lba, n_blks);
        /* and the register form the submission paths use must agree with them */
        uint4 q[4];
        bam::nvm_cmd_rw_quarters(cid, opcode, ns_id, prp1, prp2, start_lba, n_blks, q[0], q[1], q[2], q[3]);
        if (memcmp(q, &cmd, 64) != 0) return BAM_EIO;
        memcpy(out64, &cmd, 64);
        return BAM_OK;
    }
    uint4* d = nullptr;
    CK(cudaMalloc(&d, 64));
    k_encode_rw<<<1, 1>>>(cid, opcode, ns_id, prp1, prp2, start_lba, n_blks, d);
    cudaError_t e = cudaMemcpy(out64, d, 64, cudaMemcpyDeviceToHost);
    cudaFree(d);
    if (e != cudaSuccess) { g_last_cuda = e; return BAM_ECUDA; }
    return BAM_OK;
}

extern "C" int bam_cache_flush(bam_cache_t pc, void* stream)
{
    if (!pc) return BAM_EINVAL;
    bam_ctrl* c = pc->ctrl;
    CK(cudaSetDevice(c->device));
    FlushWork w;
    w.pc = pc->d;
    return launch_fused(c, w, (cudaStream_t)stream);
}

extern "C" int bam_launch_page_scan(bam_array_t a, uint64_t n_pages, const uint64_t* pages_dev, uint64_t first_page,
                                    uint64_t* sum_out_dev, void* stream)
{
    if (!a || a->elem_bytes != 8 || a->n_ranges != 1 || a->h_range.page_start_offset != 0) return BAM_EINVAL;
    bam_ctrl* c = a->pc->ctrl;
    CK(cudaSetDevice(c->device));
    PageScanWork w;
    w.r = a->h_range; w.n_pages = n_pages; w.pages = pages_dev; w.first_page = first_page; w.sum_out = sum_out_dev;
    return launch_fused(c, w, (cudaStream_t)stream);
}

extern "C" int bam_gen_uniform_indices(uint64_t* out_dev, uint64_t n_lanes, uint64_t reqs_per_lane, uint64_t access_seed,
                                       uint64_t n_elems, void* stream)
{
    if (!out_dev || n_elems == 0) return BAM_EINVAL;
    k_gen_uniform<<<1184, 256, 0, (cudaStream_t)stream>>>(out_dev, n_lanes, reqs_per_lane, access_seed, n_elems);
    CK(cudaGetLastError());
    return BAM_OK;
}

extern "C" int bam_gen_zipf_indices(uint64_t* out_dev, uint64_t n_lanes, uint64_t reqs_per_lane, uint64_t access_seed,
                                    const uint64_t* cdf_dev, uint64_t n_pages, uint32_t elems_per_page,
                                    uint64_t perm_seed, void* stream)
{
    if (!out_dev || !cdf_dev || n_pages == 0 || elems_per_page == 0) return BAM_EINVAL;
    k_gen_zipf<<<1184, 256, 0, (cudaStream_t)stream>>>(out_dev, n_lanes, reqs_per_lane, access_seed, cdf_dev, n_pages,
                                                       elems_per_page, perm_seed);
    CK(cudaGetLastError());
    return BAM_OK;
}

extern "C" int bam_gen_block_pages(uint64_t* out_dev, uint64_t n_reqs, uint64_t req_seed, uint64_t n_pages, void* stream)
{
    if (!out_dev || n_pages == 0) return BAM_EINVAL;
    k_gen_block_pages<<<1184, 256, 0, (cudaStream_t)stream>>>(out_dev, n_reqs, req_seed, n_pages);
    CK(cudaGetLastError());
    return BAM_OK;
}

extern "C" int bam_direct_page_sums(const uint64_t* pages_dev, uint64_t n, uint64_t store_seed, uint32_t words_per_page,
                                    uint64_t* sum_out_dev, void* stream)
{
    if (!pages_dev || !sum_out_dev || words_per_page == 0) return BAM_EINVAL;
    k_page_sums<<<1184, 256, 0, (cudaStream_t)stream>>>(pages_dev, n, store_seed, words_per_page, sum_out_dev);
    CK(cudaGetLastError());
    return BAM_OK;
}

extern "C" int bam_direct_checksum(const uint64_t* idx_dev, uint64_t n, uint64_t store_seed, uint64_t first_elem,
                                   uint64_t* sum_out_dev, void* stream)
{
    if (!idx_dev || !sum_out_dev) return BAM_EINVAL;
    k_direct_checksum<<<1184, 256, 0, (cudaStream_t)stream>>>(idx_dev, n, store_seed, first_elem, sum_out_dev);
    CK(cudaGetLastError());
    return BAM_OK;
}

extern "C" int bam_launch_geometry(bam_ctrl_t c, uint32_t* grid, uint32_t* ctrl_blocks, uint32_t* threads)
{
    if (!c) return BAM_EINVAL;
    CK(cudaSetDevice(c->device));
    uint32_t g = 0;
    int rc = fused_geometry<BlockReadWork>(c, &g);        /* the largest grid any launcher uses (three blocks per SM) */
    if (rc) return rc;
    if (grid) *grid = g;
    if (ctrl_blocks) *ctrl_blocks = c->emu.n_ctrl_blocks;
    if (threads) *threads = BAM_THREADS;
    return BAM_OK;
}
