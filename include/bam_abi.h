/*
 * bam_abi.h -- C ABI of libbam_b200.so.
 *
 * Plain pointers, sizes and opaque handles only.  Every function returns 0 or a BAM_E*
 * code (bam/abi_types.h) and never throws.  Kernel launchers are asynchronous on the given
 * stream (a cudaStream_t passed as void*; NULL = default stream); device-side failures
 * (a wait that ran out, an NVMe error status) are reported by bam_ctrl_status(), which
 * synchronises the device first.  There is no CPU fallback: without a CUDA device every
 * create call fails with BAM_ECUDA.
 *
 * Each entry point names the reference interface it stands in for.
 */
#ifndef BAM_ABI_H
#define BAM_ABI_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct bam_ctrl* bam_ctrl_t;     /* emulated NVMe controller + its queue pairs  */
typedef struct bam_cache* bam_cache_t;   /* page cache                                  */
typedef struct bam_array* bam_array_t;   /* array of fixed-size elements over the cache */

typedef struct {
    uint64_t hits, misses, read_ios;
} bam_cache_stats_t;

typedef struct {
    uint32_t code, where;
    uint64_t detail;
} bam_status_out_t;

const char* bam_version(void);
const char* bam_strerror(int code);                              /* nvm_strerror, include/nvm_error.h:67 */

/* ---- controller ------------------------------------------------------------------------
 * Replaces Controller::Controller(path, ns, gpu, queueDepth, numQueues) (include/ctrl.h:148-199)
 * and the QueuePair constructor (include/queue.h:89-221): instead of opening /dev/libnvm*,
 * it creates the emulated controller on `device` with a pinned, device-mapped backing store of
 * `store_bytes` (logical block size `lba_bytes`, 512 or 4096) and `n_queues` I/O queue pairs of
 * `queue_depth` entries (a power of two, 2..65536... capped at 1024 like MAX_SQ_ENTRIES_64K,
 * include/queue.h:55) in device memory. */
int bam_ctrl_create(bam_ctrl_t* out, int device, uint64_t store_bytes, uint32_t lba_bytes,
                    uint32_t n_queues, uint32_t queue_depth);
int bam_ctrl_destroy(bam_ctrl_t c);
/* Host pointer of the backing store ("the media"); the caller may fill it directly. */
void* bam_ctrl_store_host(bam_ctrl_t c);
uint64_t bam_ctrl_store_bytes(bam_ctrl_t c);
/* Fill the store with element[i] = splitmix64(seed ^ (first_elem + i)) (bam_synth.h) from the
 * GPU through the mapping.  Stands in for loading a dataset onto the SSD
 * (benchmarks/readwrite/main.cu:283-316). */
int bam_ctrl_fill_store(bam_ctrl_t c, uint64_t seed, uint64_t first_elem, void* stream);
/* The same for controller `stripe` of `n_stripes` behind a striped range (BAM_DIST_STRIPE): its
 * page j receives the elements of logical page j * n_stripes + stripe. */
int bam_ctrl_fill_store_striped(bam_ctrl_t c, uint64_t seed, uint64_t first_elem, uint32_t page_bytes, uint32_t stripe,
                                uint32_t n_stripes, void* stream);
/* Copy caller data into the store at a byte offset (host memcpy). */
int bam_ctrl_write_store(bam_ctrl_t c, uint64_t byte_offset, const void* src, uint64_t bytes);
/* Controller warps: n_blocks blocks of the fused launches run the command processor;
 * batch = the most commands a warp reserves from a queue at a time (at most 32; a queue shallower than
 * 16 x batch is cut into batches of a sixteenth of its depth, 8 at least).  0 keeps the current value.
 * At most 32 processor warps serve one queue. */
int bam_ctrl_configure(bam_ctrl_t c, uint32_t n_ctrl_blocks, uint32_t batch, uint64_t spin_timeout_ns);
/* Upper limit for one fused launch (default 300 s): the controller blocks flag BAM_ETIMEDOUT and
 * every wait in the launch drains. */
int bam_ctrl_set_launch_timeout(bam_ctrl_t c, uint64_t launch_timeout_ns);
/* Scope of the acquire/release operations on doorbells and completion entries.  1 = system scope
 * (what a controller outside this GPU needs), 0 = device scope (sufficient, and the default, for
 * the emulated controller, which runs inside the same launch on the same GPU).  Re-initialises
 * the queue pairs. */
int bam_ctrl_set_scope(bam_ctrl_t c, int system_scope);
/* Cap the grid of the fused launches (0 = as many blocks as are co-resident).  Small caches
 * need it: each resident warp may pin up to 32 pages at once.  The cap also travels in the descriptor
 * bam_ctrl_emu_descriptor returns, so bam::launch_fused of the device headers applies it to user
 * kernels; fetch the descriptor after this call. */
int bam_ctrl_set_max_grid(bam_ctrl_t c, uint32_t max_grid);
/* Fault injection on the controller side (host-configured, never faults the GPU):
 * mode BAM_FAULT_DROP_CPL swallows the completion of the nth command from now,
 * BAM_FAULT_STATUS completes it with `status`. */
int bam_ctrl_inject_fault(bam_ctrl_t c, uint32_t mode, uint64_t nth, uint32_t status);
/* Synchronise the device and read the status block; clear = reset it afterwards. */
int bam_ctrl_status(bam_ctrl_t c, bam_status_out_t* out, int clear);
/* Commands served since creation (Controller::print_reset_stats, include/ctrl.h:86-92). */
int bam_ctrl_served(bam_ctrl_t c, uint64_t* out, int reset);
/* The 32 profiling counters of the status block (all zero unless the library was built with
 * -DBAM_PROFILE): cycles and event counts of the protocol stages, for tuning. */
int bam_ctrl_profile(bam_ctrl_t c, uint64_t* out32, int reset);
/* Re-initialise every queue pair to its power-on state (nvm_queue_clear, src/queue.cpp:12-42).
 * Needed after an injected fault left commands unaccounted for. */
int bam_ctrl_reset_queues(bam_ctrl_t c);
/* Device pointers for callers that write their own kernels (include/bam/*.cuh). */
void* bam_ctrl_device_controller(bam_ctrl_t c);   /* Controller*            */
int bam_ctrl_emu_descriptor(bam_ctrl_t c, void* out, size_t out_bytes); /* bam_emu_d_t by value */

/* ---- page cache --------------------------------------------------------------------------
 * Replaces page_cache_t::page_cache_t(page_size, n_pages, gpu, ctrl, max_range, ctrls)
 * (include/page_cache.h:697-875).  n_pages is at most BAM_MAX_CACHE_SLOTS (2^24 - 2 = 16,777,214: the
 * page table addresses slots with 24 bits; 64 GiB of 4 KiB pages); more is refused with BAM_EINVAL. */
int bam_cache_create(bam_cache_t* out, bam_ctrl_t ctrl, uint32_t page_size, uint64_t n_pages);
/* The same constructor with its `ctrls` vector of several controllers (page_cache.h:714-720: one
 * cache in front of n SSDs).  All controllers must sit on the same GPU with the same block size.
 * From here until bam_cache_destroy the controllers form a group: one fused launch serves the
 * queues of all of them, they report into the first controller's status block (bam_ctrl_status of
 * any member reads it) and bam_ctrl_configure of the FIRST controller sets the launch geometry.
 * A controller can back one multi-controller cache at a time (BAM_EBUSY otherwise); destroy the
 * cache before its controllers.  How a range's pages map to the controllers is chosen per array:
 * bam_array_create_dist. */
int bam_cache_create_multi(bam_cache_t* out, const bam_ctrl_t* ctrls, uint32_t n_ctrls, uint32_t page_size,
                           uint64_t n_pages);
int bam_cache_destroy(bam_cache_t pc);
/* range_d_t counters (page_cache.h:904-907, printed by array_t::print_reset_stats :1731-1752). */
int bam_cache_stats(bam_cache_t pc, bam_cache_stats_t* out, int reset);
/* Drop every cached page (all slots free, table empty). */
int bam_cache_invalidate(bam_cache_t pc);
/* The same, enqueued on `stream` without synchronising; the counters are left alone. */
int bam_cache_invalidate_async(bam_cache_t pc, void* stream);
/* Audit after a launch: no pins left, no BUSY bits, every VALID slot is found through the page
 * table, every table entry points at a slot with a matching tag.  *violations = 0 when clean. */
int bam_cache_audit(bam_cache_t pc, uint64_t* violations);
int bam_cache_descriptor(bam_cache_t pc, void* out, size_t out_bytes);  /* page_cache_d_t by value */
/* The same audit for callers that must not allocate or stall the device (no counterpart in the
 * reference).  bam_cache_audit takes its counter from cudaMalloc/cudaFree and synchronises the
 * device; a caller that audits while other streams run, whose device memory belongs to a single
 * allocator, or that is on a path where allocation calls are not allowed, uses this instead:
 * it enqueues a memset and one kernel on `stream` and returns at once.  The count is written to
 * *violations_out_dev (device memory, overwritten) when the kernel has run.
 * Scratch is a fixed 8 KiB array inside the library's device image (held on every GPU that loads
 * the library until exit), so caches of more than 8,380,416 slots are refused with BAM_E2BIG.
 * All calls share that array: calls that can overlap on the GPU (different streams, no ordering
 * between them) race and give wrong counts; calls on one stream are safe.  The first call on each
 * device also looks up the array's device address; make that first call outside any stream
 * capture.  Like every entry point that takes a cache, the call makes the cache's GPU the calling
 * thread's current device (cudaSetDevice) and leaves it so. */
int bam_cache_audit_noalloc(bam_cache_t pc, uint64_t* violations_out_dev, void* stream);

/* ---- arrays --------------------------------------------------------------------------------
 * Replaces range_t<T>(index_start, count, page_start, page_count, page_start_offset, page_size,
 * cache, gpu) + array_t<T>(n_elems, disk_start_offset, {range}) (page_cache.h:978-1030,
 * :1754-1772) for a single-range array of `elem_bytes`-sized elements (4 or 8) that starts at
 * byte `store_byte_offset` (page aligned) of the backing store. */
int bam_array_create(bam_array_t* out, bam_cache_t pc, uint64_t n_elems, uint32_t elem_bytes,
                     uint64_t store_byte_offset);
/* The same with the range's data_dist_t (page_cache.h:42, :558-582, :978): BAM_DIST_REPLICATE (0,
 * what bam_array_create uses: every controller holds the whole range at store_byte_offset, a page
 * read goes to any one of them, a write-back to all) or BAM_DIST_STRIPE (1: page p of the range
 * lives on controller p % n at backing page store_byte_offset / page_size + p / n). */
int bam_array_create_dist(bam_array_t* out, bam_cache_t pc, uint64_t n_elems, uint32_t elem_bytes,
                          uint64_t store_byte_offset, uint32_t dist);
/* array_t<T> over a vector of range_t<T> (page_cache.h:1754-1772; the device side looks an index up with
 * find_range, :1318-1329): range k covers the element indices [index_start, index_end) and its element
 * index_start lives page_start_offset bytes into the backing page at store_byte_offset (range_t's
 * page_start * page_size and page_start_offset, :985-1030 -- the shape benchmarks/bfs/main.cu:1481-1484 builds
 * for an edge list that starts at a file offset).  store_byte_offset must be page aligned,
 * page_start_offset smaller than a page and a multiple of elem_bytes; index ranges must not overlap;
 * indices outside every range fail with BAM_ERANGE in the status block.  bam_launch_array_read,
 * bam_launch_array_write and the cursor patterns accept such arrays; the launchers that walk whole pages
 * of one range (page scan, graph traversals, the array[] pattern form) need a single range with
 * page_start_offset 0 and return BAM_EINVAL otherwise. */
typedef struct {
    uint64_t index_start, index_end;
    uint64_t store_byte_offset;
    uint64_t page_start_offset;
    uint32_t dist;               /* BAM_DIST_REPLICATE / BAM_DIST_STRIPE */
    uint32_t reserved;
} bam_range_desc_t;
int bam_array_create_ranges(bam_array_t* out, bam_cache_t pc, uint64_t n_elems, uint32_t elem_bytes,
                            const bam_range_desc_t* ranges, uint32_t n_ranges);
int bam_array_destroy(bam_array_t a);
void* bam_array_device_ptr(bam_array_t a);         /* array_d_t<T>* (array_t::d_array_ptr) */

/* ---- kernel launchers -----------------------------------------------------------------------
 * The reference exports no kernels (they live in benchmarks/...); these are the same
 * workloads as launchable entry points.  Every launcher runs ONE fused cooperative kernel:
 * the first blocks are the emulated controller's command processor, the rest the workload. */

/* Block benchmark (benchmarks/block/main.cu:137-200): request r reads 4 KiB-aligned page
 * pages[r] (or, if pages == NULL, bam_block_request_page(req_seed, r, n_store_pages)) of
 * `page_bytes` straight into a private cache slot through read_data, bypassing the cache
 * look-up.  crc_out (device, n_reqs u32, may be NULL) receives the CRC-32 of what arrived;
 * sum_out (device u64, may be NULL) is incremented by the wrapping sum of all words read. */
int bam_launch_block_read(bam_cache_t pc, uint64_t n_reqs, const uint64_t* pages_dev, uint64_t req_seed,
                          uint32_t* crc_out_dev, uint64_t* sum_out_dev, void* stream);

/* The same with io_depth (1..8) requests in flight per thread, each in its own cache slot: the
 * iodepth-block benchmark (benchmarks/iodepth-block/main.cu:97-147, access_data_async x N then
 * poll_async x N, page_cache.h:1930-1959).  Needs 32 * io_depth < queue_depth / 2 and
 * worker threads * io_depth cache slots. */
int bam_launch_block_read_depth(bam_cache_t pc, uint64_t n_reqs, const uint64_t* pages_dev, uint64_t req_seed,
                                uint32_t io_depth, uint32_t* crc_out_dev, uint64_t* sum_out_dev, void* stream);

/* Array benchmark (benchmarks/array/main.cu:54-65): n_lanes reader lanes x reqs_per_lane
 * element reads through array[]; indices from idx_dev[lane*reqs_per_lane + k], or if idx_dev ==
 * NULL from PCG32 stream `lane` seeded with access_seed (bam_synth.h).  *sum_out_dev (device u64)
 * is incremented by the wrapping sum of the values read. */
int bam_launch_array_read(bam_array_t a, uint64_t n_lanes, uint64_t reqs_per_lane, const uint64_t* idx_dev,
                          uint64_t access_seed, uint64_t* sum_out_dev, void* stream);

/* Element updates through the cache (array_d_t<T>::seq_write / operator() / AtomicAdd,
 * page_cache.h:1577-1711; the write side of benchmarks/vectoradd/main.cu:103-118): for k < n,
 * addend == 0: a[idx[k]] = splitmix64(val_seed ^ idx[k]); addend != 0: a[idx[k]] += addend
 * (atomic, wrapping).  Pages become DIRTY; a dirty page that is evicted is written back first. */
int bam_launch_array_write(bam_array_t a, uint64_t n, const uint64_t* idx_dev, uint64_t val_seed, uint64_t addend,
                           void* stream);

/* The per-thread protocol: the lanes named by `lanes` (bit l = lane l of every warp) each pin page
 * first_page + k of the array's single range, read its first element into first_words_dev[k] and unpin it,
 * every lane on its own with no help from its warp-mates -- range_d_t<T>::acquire_page(page, count, write,
 * queue) / release_page as a diverged caller uses them (page_cache.h:1122-1224, find_slot :1786-1927).  A
 * miss whose victim is dirty writes it back itself. */
int bam_launch_thread_acquire(bam_array_t a, uint64_t first_page, uint64_t n_pages, uint32_t lanes,
                              uint64_t* first_words_dev, void* stream);

/* Bulk transfer between the cache's memory and the store, one NVMe command per cache page (the loader
 * and the read-back of benchmarks/readwrite/main.cu:283-390): request r moves cache slot first_slot + r
 * to (write != 0) or from store page first_store_page + r.  The cache's page table is not involved: use
 * it on an invalidated cache.  bam_cache_copy moves bytes between host memory and the cache's memory
 * (slot first_slot onwards) on `stream`, which is how a file gets there. */
int bam_launch_bulk_io(bam_cache_t pc, uint64_t n_pages, uint64_t first_store_page, uint64_t first_slot, int write,
                       void* stream);
int bam_cache_copy(bam_cache_t pc, uint64_t first_slot, void* host, uint64_t bytes, int to_cache, void* stream);

/* Pattern benchmark (benchmarks/pattern/main.cu, the *_pc kernels): every thread sums the elements
 * it visits through a bam_ptr cursor; *sum_out_dev (device u64) is incremented by the wrapping sum.
 * pattern 0 SEQUENTIAL (:131-146): elements [0, n_elems) dealt round-robin to the threads;
 * 1 SEQUENTIAL_WARP (:232-265): warp w of n_warps reads n_pages_per_warp consecutive pages, warp ids
 * interleaved by `stride` (1 = in order); 2 RANDOM (:155-170): a[assignment_dev[i]] for i in
 * [0, n_elems); 3 RANDOM_WARP: warp w reads the whole pages assignment_dev[w * n_pages_per_warp + k].
 * A cursor keeps its page pinned: the cache needs more slots than worker threads. */
int bam_launch_pattern_read(bam_array_t a, uint32_t pattern, uint64_t n_elems, uint64_t n_warps, uint64_t n_pages_per_warp,
                            uint64_t stride, const uint64_t* assignment_dev, uint64_t* sum_out_dev, void* stream);
/* The same walks with the element access chosen as the benchmarks' `type` option does
 * (benchmarks/cache/main.cu:69-74, benchmarks/pattern/main.cu): impl 0 = through a bam_ptr cursor (what
 * bam_launch_pattern_read runs), impl 1 = every read is array[i] ("ORIG"); pattern 1 with impl 1 is the
 * cache benchmark's sequential_access_warp (benchmarks/cache/main.cu:82-112), pattern 3 its
 * random_access_warp (:45-79).  array[] reads of resident pages pin nothing, so impl 1 puts no demand on
 * the number of cache slots. */
int bam_launch_pattern_read_impl(bam_array_t a, uint32_t pattern, uint32_t impl, uint64_t n_elems, uint64_t n_warps,
                                 uint64_t n_pages_per_warp, uint64_t stride, const uint64_t* assignment_dev,
                                 uint64_t* sum_out_dev, void* stream);
/* Write every dirty page back to the backing store (page_cache_t::flush_cache, page_cache.h:675-682,
 * kernel __flush :584-629).  Call it when no other launch is using the cache. */
int bam_cache_flush(bam_cache_t pc, void* stream);

/* Cache benchmark (benchmarks/cache/main.cu:44-114): each warp reads whole pages of the
 * array (page list pages_dev[n_pages], or pages first_page .. first_page+n_pages-1 when NULL),
 * all 32 lanes striding the page; wrapping sum of every element into *sum_out_dev. */
int bam_launch_page_scan(bam_array_t a, uint64_t n_pages, const uint64_t* pages_dev, uint64_t first_page,
                         uint64_t* sum_out_dev, void* stream);

/* ---- graph consumers -------------------------------------------------------------------------
 * CSR graph in the backing store: `offsets` (n_vertices + 1 u64 row offsets) and `cols` (u64
 * column indices) are two arrays over the SAME cache; both are read only through the cache
 * (the reference keeps the offsets in plain GPU memory, benchmarks/bfs/main.cu:1244-1259). */

/* One BFS level over local vertices [v_begin, v_end) (benchmarks/bfs/main.cu:658-689): every vertex
 * with label == level relaxes its neighbours; unreached = 0xFFFFFFFF.  *changed_dev is set to 1 if
 * any label was written, *scanned_dev (may be NULL) is incremented by the edges read.  When the
 * graph is sharded by vertex range, `offsets`/`cols` hold this shard's rows (local vertex v is
 * global vertex v_base + v), column indices and the label array stay global. */
int bam_launch_bfs_level(bam_array_t offsets, bam_array_t cols, uint64_t v_begin, uint64_t v_end, uint64_t v_base,
                         uint32_t level, uint32_t* label_dev, uint32_t* changed_dev, uint64_t* scanned_dev,
                         void* scratch_dev, uint64_t scratch_bytes, void* stream);
/* One label-propagation sweep over the vertices of [v_begin, v_end) flagged in curr_visit
 * (benchmarks/cc/main.cu:123-144, :595-617): for every edge the larger component label takes
 * the smaller (atomicMin), the written vertex is flagged in next_visit. */
int bam_launch_cc_sweep(bam_array_t offsets, bam_array_t cols, uint64_t v_begin, uint64_t v_end, uint64_t v_base,
                        uint64_t* comp_dev, const uint8_t* curr_visit_dev, uint8_t* next_visit_dev,
                        uint32_t* changed_dev, uint64_t* scanned_dev, void* scratch_dev, uint64_t scratch_bytes,
                        void* stream);
/* scratch_dev (may be NULL) is device memory of bam_graph_scratch_bytes(number of edges) bytes that
 * the launch clears and uses to split adjacency lists of hub vertices into work items shared by
 * all warps; without it every list is walked by one warp. */
uint64_t bam_graph_scratch_bytes(uint64_t n_edges);
/* Whole traversals on one GPU (the host loops of benchmarks/bfs/main.cu:1577-1736 and
 * benchmarks/cc/main.cu:1418-1623).  label_dev: n_vertices u32 levels; comp_dev: n_vertices u64
 * labels, at the fixed point the minimum vertex id of each component.  Synchronous. */
int bam_bfs_run(bam_array_t offsets, bam_array_t cols, uint64_t n_vertices, uint64_t source,
                uint32_t* label_dev, uint32_t* n_levels_out, uint64_t* edges_scanned_out);
int bam_cc_run(bam_array_t offsets, bam_array_t cols, uint64_t n_vertices, uint64_t* comp_dev,
               uint32_t* n_sweeps_out, uint64_t* edges_scanned_out);

/* ---- exchange steps of the multi-GPU traversals ---------------------------------------------------
 * No counterpart in the reference, whose BFS and CC run on one GPU (benchmarks/bfs/main.cu:1577-1736,
 * benchmarks/cc/main.cu:1418-1623).  With the graph sharded by vertex range and the label array
 * replicated, every rank runs, after each level / sweep:  compact -> all-gather of the 16-byte headers
 * -> all-gather of the payloads (both by the caller, into this GPU's own memory) -> apply.
 * A header is two u64: {entries appended, status code of `pc`'s controller (0 = fine)}; the gathered
 * headers hdrs_dev[2 * world] tell every rank how many entries each rank sent, whether the traversal is
 * over (no entries at all) and whether a rank failed.  Received payloads sit `stride` entries apart:
 * rank r's entries are recv[r * stride .. r * stride + hdrs[2 r]).  The entries of my_rank are skipped.
 * Vertex ids must fit 32 bits (n_vertices <= 2^32).  Plain kernels on `stream`; pc may be NULL. */
/* BFS: append every vertex v with label[v] == level_value (the vertices this rank labelled in the
 * level it just ran) to out_dev[capacity] (u32). */
int bam_launch_frontier_compact(bam_cache_t pc, const uint32_t* label_dev, uint64_t n_vertices, uint32_t level_value,
                                uint32_t* out_dev, uint64_t capacity, uint64_t* hdr_dev, void* stream);
/* BFS: label[v] = level_value for every received v that is still unreached (0xFFFFFFFF). */
int bam_launch_frontier_apply(uint32_t* label_dev, uint64_t n_vertices, uint32_t level_value, const uint32_t* recv_dev,
                              uint64_t stride, const uint64_t* hdrs_dev, uint32_t world, uint32_t my_rank, void* stream);
/* CC: append (v << 32 | comp[v]) for every vertex flagged in next_visit_dev (the vertices whose label
 * this rank lowered in the sweep it just ran) to out_pairs_dev[capacity] (u64). */
int bam_launch_cc_compact(bam_cache_t pc, const uint64_t* comp_dev, const uint8_t* next_visit_dev, uint64_t n_vertices,
                          uint64_t* out_pairs_dev, uint64_t capacity, uint64_t* hdr_dev, void* stream);
/* CC: comp[v] = min(comp[v], label) for every received pair; a vertex of [own_begin, own_end) whose
 * label fell is flagged in next_visit_dev for this rank's next sweep. */
int bam_launch_cc_apply(uint64_t* comp_dev, uint8_t* next_visit_dev, uint64_t n_vertices, uint64_t own_begin, uint64_t own_end,
                        const uint64_t* recv_pairs_dev, uint64_t stride, const uint64_t* hdrs_dev, uint32_t world,
                        uint32_t my_rank, void* stream);
/* CC, dense form for sweeps that change most labels: after the caller has combined the replicas with
 * an element-wise MIN all-reduce, flag the owned vertices whose label is now below before_own_dev
 * (the caller's copy of comp[own_begin .. own_end) taken before the all-reduce). */
int bam_launch_cc_dense_flag(const uint64_t* comp_dev, const uint64_t* before_own_dev, uint8_t* next_visit_dev,
                             uint64_t own_begin, uint64_t own_end, void* stream);

/* Single-source shortest paths over a weighted CSR graph (benchmarks/sssp/main.cu): `weights` is a
 * third array over the same cache, u32 elements, weights[j] belongs to edge cols[j] (the .val file
 * of the reference, :379-431).  One sweep (kernel_*_pc, :115-146): every vertex flagged in label_dev
 * (u8 per vertex) offers cost + weight to its neighbours with atomicMin on new_cost_dev and clears
 * its flag (with a graph sharded by vertex range, local vertex v is global vertex v_base + v; the
 * label and cost arrays and the column indices stay global).  bam_sssp_run is the host loop (:640-720) with the update kernel (:282-292) between
 * sweeps; cost_dev receives n_vertices u32 distances, 0xFFFFFFFF = unreachable.  Synchronous. */
int bam_launch_sssp_sweep(bam_array_t offsets, bam_array_t cols, bam_array_t weights, uint64_t v_begin, uint64_t v_end,
                          uint64_t v_base, uint8_t* label_dev, uint32_t* new_cost_dev, uint64_t* scanned_dev, void* scratch_dev,
                          uint64_t scratch_bytes, void* stream);
int bam_sssp_run(bam_array_t offsets, bam_array_t cols, bam_array_t weights, uint64_t n_vertices, uint64_t source,
                 uint32_t* cost_dev, uint32_t* n_iters_out, uint64_t* edges_scanned_out);

/* Push-based delta PageRank (benchmarks/pagerank/main.cu:107-115, 137-160, 412-421, host loop
 * :678-772).  All quantities are 64-bit fixed-point numbers with BAM_PR_FRAC_BITS (40) fraction
 * bits and the damping factor is alpha_num / alpha_den (the reference: float, alpha 0.85,
 * tolerance 0.001, at most 100 sweeps), which makes the result independent of the order in which
 * the atomic adds land: bit-identical on every run.  One sweep: every vertex flagged in label_dev
 * adds delta_dev[v] to residual_dev of each neighbour and clears its flag.  bam_launch_degrees
 * writes the out-degree of every vertex (read once through the cache).  bam_pagerank_run is the
 * whole loop; value_dev receives n_vertices fixed-point ranks.  Synchronous. */
int bam_launch_pr_sweep(bam_array_t offsets, bam_array_t cols, uint64_t v_begin, uint64_t v_end, uint64_t v_base,
                        uint8_t* label_dev,
                        const uint64_t* delta_dev, uint64_t* residual_dev, uint64_t* scanned_dev, void* scratch_dev,
                        uint64_t scratch_bytes, void* stream);
int bam_launch_degrees(bam_array_t offsets, uint64_t n_vertices, uint32_t* deg_dev, void* stream);
int bam_pagerank_run(bam_array_t offsets, bam_array_t cols, uint64_t n_vertices, uint64_t alpha_num, uint64_t alpha_den,
                     uint64_t tolerance_q, uint32_t max_iters, uint64_t* value_dev, uint32_t* n_iters_out,
                     uint64_t* edges_scanned_out);
/* R-MAT edges [e_begin, e_end) of bam_synth.h as directed 64-bit keys (u<<32|v and v<<32|u per
 * edge, ~0 for self loops) into keys_dev[2*(e_end-e_begin)]; sorting and de-duplicating the keys
 * gives the CSR (stands in for benchmarks/bam_data_conversion.py + the dataset files). */
int bam_gen_rmat_keys(uint64_t* keys_dev, uint64_t e_begin, uint64_t e_end, uint64_t seed, uint32_t scale,
                      uint32_t ta, uint32_t tab, uint32_t tabc, void* stream);
/* Copy device data into the backing store (loading a dataset onto the "SSD",
 * benchmarks/readwrite/main.cu:283-316). */
int bam_ctrl_write_store_from_device(bam_ctrl_t c, uint64_t byte_offset, const void* src_dev, uint64_t bytes, void* stream);

/* ---- synthetic access streams ------------------------------------------------------------------
 * The reference benchmarks build their access lists on the host with rand()
 * (benchmarks/array/main.cu:150-162, benchmarks/pattern/main.cu:560-600); these write the seeded
 * streams of bam_synth.h as u64 element indices, out[lane*reqs_per_lane + k], on the device. */
int bam_gen_uniform_indices(uint64_t* out_dev, uint64_t n_lanes, uint64_t reqs_per_lane, uint64_t access_seed,
                            uint64_t n_elems, void* stream);
/* Zipf page popularity from a 64-bit fixed-point CDF table (device, n_pages entries), rank ->
 * page through the seeded permutation, uniform element offset inside the page. */
int bam_gen_zipf_indices(uint64_t* out_dev, uint64_t n_lanes, uint64_t reqs_per_lane, uint64_t access_seed,
                         const uint64_t* cdf_dev, uint64_t n_pages, uint32_t elems_per_page, uint64_t perm_seed,
                         void* stream);

/* Pages of the block random-read workload's requests (bam_block_request_page of bam_synth.h). */
int bam_gen_block_pages(uint64_t* out_dev, uint64_t n_reqs, uint64_t req_seed, uint64_t n_pages, void* stream);
/* Wrapping sum of every word of every listed page, recomputed from the store's definition: what
 * bam_launch_block_read's sum_out must equal (verification of full-size runs). */
int bam_direct_page_sums(const uint64_t* pages_dev, uint64_t n, uint64_t store_seed, uint32_t words_per_page,
                         uint64_t* sum_out_dev, void* stream);
/* Wrapping sum of splitmix64(store_seed ^ (first_elem + idx[i])) over an index list, recomputed
 * from the store's definition without touching cache or queues: the value every cached read of
 * those indices must add up to (verification of full-size runs; no counterpart in the reference,
 * whose array benchmark discards the values it reads, benchmarks/array/main.cu:49,61). */
int bam_direct_checksum(const uint64_t* idx_dev, uint64_t n, uint64_t store_seed, uint64_t first_elem,
                        uint64_t* sum_out_dev, void* stream);

/* The 4096-byte IDENTIFY page an emulated controller returns (cns 1: controller data; cns 0: namespace 1 of a
 * store of store_bytes bytes in logical blocks of lba_bytes), at the offsets of the NVMe specification that the
 * reference parses (src/admin.cpp:139-152, :189-198).  Needs no controller and no GPU. */
int bam_identify_page(uint32_t cns, uint64_t store_bytes, uint32_t lba_bytes, void* out4096);
/* The 64-byte NVMe read/write command the library writes into a submission queue for these fields
 * (nvm_cmd_header / nvm_cmd_data_ptr / nvm_cmd_rw_blks, include/nvm_cmd.h:54-88), for checks against
 * other encoders; on_device != 0 runs the register-built form in a kernel. */
int bam_encode_rw_command(void* out64, uint16_t cid, uint8_t opcode, uint32_t ns_id, uint64_t prp1, uint64_t prp2,
                          uint64_t start_lba, uint16_t n_blks, int on_device);
/* The largest grid a launcher uses on this controller's GPU (three blocks per SM; some workloads run two):
 * total blocks, controller blocks among them, threads per block.  Callers size the per-thread landing slots of
 * bam_launch_block_read(_depth) with it. */
int bam_launch_geometry(bam_ctrl_t c, uint32_t* grid, uint32_t* ctrl_blocks, uint32_t* threads);

#ifdef __cplusplus
}
#endif
#endif /* BAM_ABI_H */
