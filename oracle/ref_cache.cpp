/*
 * ref_cache.cpp -- TEST INFRASTRUCTURE: the REFERENCE's page cache and array read path
 * (include/page_cache.h: array_d_t<T>::seq_read :1541-1574, coalesce_page :1332-1366, range_d_t<T>::
 * acquire_page :1122-1224 / release_page, page_cache_d_t::find_slot :1786-1927, read_data :2009-2054 with its
 * enqueue_second) on top of its parallel queue protocol (include/nvm_parallel_queue.h), compiled for the
 * host from the reference's headers where they lie (recipe: oracle/Makefile, target _ref/libref_cache.so)
 * and run by host threads that play the role of GPU threads (one thread = a warp with one active lane: the
 * header's own host stubs give __activemask() == 1).
 *
 * What the recipe has to work around, without touching the reference's files:
 *  - page_cache.h:679 launches a kernel with <<< >>> inside a host method that is never called here, and
 *    :1190 initialises a variable inside a switch where a later case label jumps past it (an error for g++);
 *    the Makefile writes a copy of the header without the launch and with that declaration split from its
 *    assignment into _ref/gen/ and puts it first on the include path;
 *  - nvm_util.h defines lane_id / warp_id / get_smid with PTX special registers; they are compiled under
 *    other names and replaced by host versions below (get_smid = the calling thread's number, so that
 *    "queue = smid % n_qps" spreads the threads over the queue pairs as SMs would);
 *  - the doorbell store st.mmio.relaxed.sys.global.u32 becomes a plain store through an assembler macro;
 *  - <simt/atomic> comes from oracle/ref_shim.
 * The host classes of the header (page_cache_t, range_t, array_t, Controller, QueuePair) need a kernel module
 * and a GPU; their DEVICE descriptors are plain data and are filled in here the way those constructors do
 * (page_cache.h:697-875, :978-1030; queue.h:58-221; ctrl.h:148-199).
 *
 * What it is for: tests run the same access list through this code and through the restatement in
 * bam_oracle.c and compare results and counters, which pins the restatement to the reference.
 */
#include <pthread.h>
#include <time.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include <vector_types.h>
#include <cuda_runtime.h>

struct refc_dim3 { unsigned x, y, z; };
static refc_dim3 refc_zero_dim = { 0, 0, 0 };
#define threadIdx refc_zero_dim
#define blockIdx refc_zero_dim
#define blockDim refc_zero_dim
#define gridDim refc_zero_dim
#define __global__
inline unsigned __activemask() { return 1u; }
inline int __any_sync(unsigned, int p) { return p; }
inline unsigned __ballot_sync(unsigned, int p) { return p ? 1u : 0u; }

__asm__(".macro st.mmio.relaxed.sys.global.u32 addr, val\n"
        ".intel_syntax prefix\n"
        "mov DWORD PTR \\addr, \\val\n"
        ".att_syntax prefix\n"
        ".endm\n");

#define lane_id refc_ptx_lane_id
#define warp_id refc_ptx_warp_id
#define get_smid refc_ptx_get_smid
#include <nvm_util.h>
#undef lane_id
#undef warp_id
#undef get_smid
static thread_local uint32_t refc_thread_no = 0;
inline uint32_t lane_id() { return 0; }
inline unsigned warp_id() { return 0; }
inline uint32_t get_smid() { return refc_thread_no; }

#include <nvm_queue.h>
#include "page_cache.h"            /* _ref/gen/page_cache.h: the reference's header minus the one kernel launch */

#define REFC_API extern "C" __attribute__((visibility("default")))

struct refc_stats { uint64_t checksum, accesses, misses, hits, read_ios, extra_reads; };

struct refc_world {
    nvm_ctrl_t nvm;
    Controller* ctrl;               /* raw storage: only the members the device code reads are set */
    QueuePair* qps;
    uint32_t n_qps;
    page_cache_d_t pc;
    range_d_t<uint64_t>* range;
    array_d_t<uint64_t> arr;
    void** owned;
    uint32_t n_owned;
};

static void* zalloc(refc_world* w, size_t bytes, size_t align = 64)
{
    void* p = nullptr;
    bytes = (bytes + align - 1) / align * align;
    if (posix_memalign(&p, align, bytes) != 0) return nullptr;
    memset(p, 0, bytes);
    w->owned[w->n_owned++] = p;
    return p;
}

/* n_qps queue pairs of depth qs over caller memory (sq_mem[q], cq_mem[q]; doorbells in the register window
 * mm_ptr), a cache of n_slots pages of page_size bytes, one range of u64 elements over n_store_pages pages
 * of the namespace starting at page 0. */
REFC_API void* refc_new2(void* mm_ptr, uint32_t n_qps, uint32_t qs, void* const* sq_mem, void* const* cq_mem, uint32_t page_size,
                         uint64_t n_slots, uint64_t n_store_pages, uint32_t lba_bytes, void* cache_mem, uint64_t cache_bus_addr);

REFC_API void* refc_new(void* mm_ptr, uint32_t n_qps, uint32_t qs, void* const* sq_mem, void* const* cq_mem, uint32_t page_size,
                        uint64_t n_slots, uint64_t n_store_pages, uint32_t lba_bytes)
{
    return refc_new2(mm_ptr, n_qps, qs, sq_mem, cq_mem, page_size, n_slots, n_store_pages, lba_bytes, nullptr, 0);
}

/* The same with the cache's memory supplied by the caller (cache_mem: n_slots pages; cache_bus_addr: the
 * address a controller uses for it), for controllers that cannot reach ordinary host memory. */
REFC_API void* refc_new2(void* mm_ptr, uint32_t n_qps, uint32_t qs, void* const* sq_mem, void* const* cq_mem, uint32_t page_size,
                         uint64_t n_slots, uint64_t n_store_pages, uint32_t lba_bytes, void* cache_mem, uint64_t cache_bus_addr)
{
    refc_world* w = static_cast<refc_world*>(calloc(1, sizeof(refc_world)));
    w->owned = static_cast<void**>(calloc(64 + 5 * n_qps, sizeof(void*)));
    w->nvm.page_size = 4096; w->nvm.dstrd = 0; w->nvm.timeout = 5000; w->nvm.max_qs = 1024; w->nvm.mm_size = 0x2000; w->nvm.mm_ptr = mm_ptr;
    w->n_qps = n_qps;
    /* queue pairs: QueuePair's constructor and init_gpu_specific_struct (queue.h:58-82, :89-221) */
    w->qps = static_cast<QueuePair*>(zalloc(w, sizeof(QueuePair) * n_qps));
    uint32_t lg = 0; while ((1u << lg) < qs) lg++;
    uint32_t blk_log = 0; while ((1u << blk_log) < lba_bytes) blk_log++;
    for (uint32_t q = 0; q < n_qps; q++) {
        QueuePair* qp = &w->qps[q];
        if (nvm_queue_clear(&qp->cq, &w->nvm, true, (uint16_t)(q + 1), qs, true, cq_mem[q], (uint64_t)(uintptr_t)cq_mem[q]) != 0 ||
            nvm_queue_clear(&qp->sq, &w->nvm, false, (uint16_t)(q + 1), qs, true, sq_mem[q], (uint64_t)(uintptr_t)sq_mem[q]) != 0) return nullptr;
        qp->sq.tickets = static_cast<padded_struct*>(zalloc(w, qs * sizeof(padded_struct)));
        qp->sq.tail_mark = static_cast<padded_struct*>(zalloc(w, qs * sizeof(padded_struct)));
        qp->sq.cid = static_cast<padded_struct*>(zalloc(w, 65536 * sizeof(padded_struct)));
        qp->cq.head_mark = static_cast<padded_struct*>(zalloc(w, qs * sizeof(padded_struct)));
        qp->cq.pos_locks = static_cast<padded_struct*>(zalloc(w, qs * sizeof(padded_struct)));
        qp->sq.qs_minus_1 = qp->cq.qs_minus_1 = qs - 1;
        qp->sq.qs_log2 = qp->cq.qs_log2 = lg;
        qp->pageSize = 4096;
        qp->block_size = lba_bytes; qp->block_size_minus_1 = lba_bytes - 1; qp->block_size_log = blk_log;
        qp->nvmNamespace = 1;
        qp->qp_id = (uint16_t)(q + 1);
    }
    /* controller: the members kernels read (ctrl.h:39-59) */
    w->ctrl = static_cast<Controller*>(zalloc(w, sizeof(Controller)));
    w->ctrl->n_qps = (uint16_t)n_qps;
    w->ctrl->d_qps = w->qps;
    w->ctrl->page_size = 4096;
    w->ctrl->blk_size = lba_bytes;
    w->ctrl->blk_size_log = blk_log;
    /* cache descriptor: page_cache_t's constructor (page_cache.h:697-875) */
    page_cache_d_t& pc = w->pc;
    memset(&pc, 0, sizeof pc);
    pc.page_size = page_size; pc.page_size_minus_1 = page_size - 1;
    while ((1ull << pc.page_size_log) < page_size) pc.page_size_log++;
    pc.n_pages = n_slots; pc.n_pages_minus_1 = n_slots - 1;
    pc.ctrl_page_size = 4096;
    pc.n_ctrls = 1;
    pc.d_ctrls = static_cast<Controller**>(zalloc(w, sizeof(Controller*)));
    pc.d_ctrls[0] = w->ctrl;
    pc.n_blocks_per_page = page_size / lba_bytes;
    pc.n_cachelines_for_states = n_slots / STATES_PER_CACHELINE;
    pc.range_cap = 64; pc.n_ranges = 0; pc.n_ranges_bits = 6; pc.n_ranges_mask = 63;
    pc.ranges = static_cast<pages_t*>(zalloc(w, 64 * sizeof(pages_t)));
    pc.ranges_page_starts = static_cast<uint64_t*>(zalloc(w, 64 * sizeof(uint64_t)));
    pc.ranges_dists = static_cast<data_dist_t*>(zalloc(w, 64 * sizeof(data_dist_t)));
    pc.cache_pages = static_cast<cache_page_t*>(zalloc(w, n_slots * sizeof(cache_page_t)));
    for (uint64_t i = 0; i < n_slots; i++) pc.cache_pages[i].page_take_lock = FREE;
    pc.page_ticket = static_cast<padded_struct_pc*>(zalloc(w, sizeof(padded_struct_pc)));
    typedef simt::atomic<uint64_t, simt::thread_scope_device> a64;
    pc.ctrl_counter = static_cast<a64*>(zalloc(w, sizeof(a64)));
    pc.q_head = static_cast<a64*>(zalloc(w, sizeof(a64)));
    pc.q_tail = static_cast<a64*>(zalloc(w, sizeof(a64)));
    pc.q_lock = static_cast<a64*>(zalloc(w, sizeof(a64)));
    pc.extra_reads = static_cast<a64*>(zalloc(w, sizeof(a64)));
    pc.base_addr = cache_mem ? static_cast<uint8_t*>(cache_mem) : static_cast<uint8_t*>(zalloc(w, n_slots * (size_t)page_size, 4096));
    const uint64_t bus0 = cache_mem ? cache_bus_addr : (uint64_t)(uintptr_t)pc.base_addr;          /* bus address == address here */
    pc.prp1 = static_cast<uint64_t*>(zalloc(w, n_slots * sizeof(uint64_t)));
    for (uint64_t i = 0; i < n_slots; i++) pc.prp1[i] = bus0 + i * page_size;
    pc.prps = false;
    /* one range over the whole namespace: range_t's constructor and page_cache_t::add_range (:978-1030, :685-695) */
    range_d_t<uint64_t>* r = static_cast<range_d_t<uint64_t>*>(zalloc(w, sizeof(range_d_t<uint64_t>)));
    r->access_cnt = 0; r->miss_cnt = 0; r->hit_cnt = 0; r->read_io_cnt = 0;
    r->index_start = 0;
    r->count = n_store_pages * (page_size / 8);
    r->page_start = 0; r->page_count = n_store_pages;
    r->page_size = page_size; r->page_start_offset = 0;
    r->dist = REPLICATE;
    r->n_elems_per_page = page_size / 8;
    r->pages = static_cast<data_page_t*>(zalloc(w, n_store_pages * sizeof(data_page_t)));
    for (uint64_t i = 0; i < n_store_pages; i++) r->pages[i].state = INVALID;
    r->range_id = pc.n_ranges++;
    pc.ranges[0] = r->pages; pc.ranges_page_starts[0] = 0; pc.ranges_dists[0] = REPLICATE;
    r->cache = pc;
    w->range = r;
    w->arr.n_elems = r->count; w->arr.start_offset = 0; w->arr.n_ranges = 1; w->arr.src = nullptr; w->arr.d_ranges = r;
    return w;
}

REFC_API void refc_free(void* h)
{
    refc_world* w = static_cast<refc_world*>(h);
    for (uint32_t i = 0; i < w->n_owned; i++) free(w->owned[i]);
    free(w->owned);
    free(w);
}

struct refc_job { refc_world* w; const uint64_t* idx; uint64_t first, step, n; uint32_t thread_no; uint64_t sum; volatile uint64_t* done; };

static void* refc_worker(void* arg)
{
    refc_job* j = static_cast<refc_job*>(arg);
    refc_thread_no = j->thread_no;
    uint64_t sum = 0;
    for (uint64_t k = j->first; k < j->n; k += j->step) {
        sum += j->w->arr.seq_read(j->idx[k]);
        __atomic_fetch_add(j->done, 1, __ATOMIC_RELEASE);
    }
    j->sum = sum;
    return nullptr;
}

/* The array benchmark's kernel body (benchmarks/array/main.cu:54-65) on n_threads host threads: thread t reads
 * elements idx[t], idx[t + n_threads], ... through seq_read.  0 = done, -1 = time limit passed. */
REFC_API int refc_array_read(void* h, const uint64_t* idx, uint64_t n, uint32_t n_threads, uint64_t timeout_ms, refc_stats* out)
{
    refc_world* w = static_cast<refc_world*>(h);
    uint64_t* done = static_cast<uint64_t*>(calloc(1, sizeof(uint64_t)));
    refc_job* jobs = static_cast<refc_job*>(calloc(n_threads, sizeof(refc_job)));
    pthread_t* th = static_cast<pthread_t*>(calloc(n_threads, sizeof(pthread_t)));
    for (uint32_t t = 0; t < n_threads; t++) {
        jobs[t] = { w, idx, t, n_threads, n, t, 0, done };
        if (pthread_create(&th[t], nullptr, refc_worker, &jobs[t]) != 0) return -2;
    }
    struct timespec t0, t;
    clock_gettime(CLOCK_MONOTONIC, &t0);
    for (;;) {
        if (__atomic_load_n(done, __ATOMIC_ACQUIRE) == n) break;
        clock_gettime(CLOCK_MONOTONIC, &t);
        const uint64_t ms = (uint64_t)(t.tv_sec - t0.tv_sec) * 1000ull + (uint64_t)((t.tv_nsec - t0.tv_nsec) / 1000000);
        if (ms > timeout_ms) { for (uint32_t k = 0; k < n_threads; k++) pthread_detach(th[k]); return -1; }
        struct timespec nap = { 0, 200000 };
        nanosleep(&nap, nullptr);
    }
    memset(out, 0, sizeof *out);
    for (uint32_t k = 0; k < n_threads; k++) { pthread_join(th[k], nullptr); out->checksum += jobs[k].sum; }
    out->accesses = w->range->access_cnt.load(); out->misses = w->range->miss_cnt.load();
    out->hits = w->range->hit_cnt.load(); out->read_ios = w->range->read_io_cnt.load();
    out->extra_reads = w->pc.extra_reads->load();
    free(jobs); free(done); free(th);
    return 0;
}

/* The state word and slot of a data page, and the page a cache slot holds (to compare final cache contents). */
REFC_API uint32_t refc_page_state(void* h, uint64_t page) { return static_cast<refc_world*>(h)->range->pages[page].state.load(); }
REFC_API uint32_t refc_page_slot(void* h, uint64_t page) { return static_cast<refc_world*>(h)->range->pages[page].offset; }
