/*
 * bam/abi_types.h -- plain-old-data types shared by host code, device code and the C ABI.
 *
 * Names follow libnvm / BaM so that code written against the reference reads the same
 * (nvm_cmd_t, nvm_cpl_t, nvm_queue_t, QueuePair, Controller, page_cache_d_t); the layouts
 * are this library's own.  Reference counterparts: include/nvm_types.h:123-193 (queue,
 * command, completion), include/queue.h:27-53 (QueuePair), include/ctrl.h:39-59 (Controller),
 * include/page_cache.h:57-70 (state bits), :96-102, :487-493, :501-550 (cache descriptors).
 *
 * All members are plain integers; device code operates on them with explicit
 * acquire/release PTX at gpu or sys scope (bam/sync.cuh), host code with __atomic builtins.
 */
#ifndef BAM_ABI_TYPES_H
#define BAM_ABI_TYPES_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
#define BAM_ALIGNAS(n) alignas(n)
#else
#define BAM_ALIGNAS(n) _Alignas(n)
#endif

/* ---- status codes (errno values; NVMe status is reported as -(SCT<<8|SC) like
 * include/nvm_error.h:37-59) -------------------------------------------------------- */
#define BAM_OK 0
#define BAM_EIO 5
#define BAM_E2BIG 7          /* a size exceeds the fixed limit of the entry point */
#define BAM_ENOMEM 12
#define BAM_EBUSY 16
#define BAM_EINVAL 22
#define BAM_ENOSPC 28
#define BAM_ERANGE 34
#define BAM_ETIMEDOUT 110
#define BAM_ECUDA 1000   /* a CUDA runtime call failed; detail = cudaError_t */

/* where a device-side wait gave up (bam_status_t.where) */
#define BAM_AT_NONE 0
#define BAM_AT_CID 1          /* no free command id                         */
#define BAM_AT_SQ_TURN 2      /* waiting for the SQ slot's turn             */
#define BAM_AT_SQ_DOORBELL 3  /* waiting for the tail to pass my slot       */
#define BAM_AT_CQ_WAIT 4      /* waiting for my completion                  */
#define BAM_AT_PAGE_BUSY 5    /* waiting for another thread's page fill     */
#define BAM_AT_FIND_SLOT 6    /* clock sweep found nothing to evict         */
#define BAM_AT_BUCKET_LOCK 7  /* page-table bucket lock                     */
#define BAM_AT_TABLE_FULL 8   /* no free page-table entry within the probe distance */
#define BAM_AT_NVME_STATUS 9  /* completion carried a non-zero status; detail = status */
#define BAM_AT_CTRL_CQ_FULL 10
#define BAM_AT_RANGE 11       /* index outside every range of the array     */
#define BAM_AT_TMA 12         /* bulk-copy mbarrier wait                    */
#define BAM_AT_LAUNCH 13      /* the whole launch outlived launch_timeout_ns */
#define BAM_AT_SQ_ORDER 14    /* controller: an earlier batch of the queue never handed its entries back */

/* Per-controller error/status block in device memory.  code is written once (first error
 * wins); every bounded wait also polls it so that one failure drains the whole launch. */
typedef struct {
    uint32_t code;
    uint32_t where;
    uint64_t detail;
    uint64_t spin_timeout_ns;   /* limit for any single device-side wait */
    uint64_t launch_timeout_ns; /* limit for one fused launch, enforced by the controller blocks */
    /* cycle/event counters, only updated by builds with -DBAM_PROFILE.  Consumers: 0 commands, 1 SQ-turn
     * cycles, 2 cid cycles, 3 publish cycles, 4 completion-wait cycles, 5 reaps, 6 reap cycles, 7 entries
     * reaped; cache: 10 inserts that lost the race for a page, 11 slots claimed by evicting a valid page,
     * 12 free slots claimed, 13 clock-sweep probes; controller: 16 batches, 17 commands, 18 fetch cycles,
     * 20 bulk-load cycles, 21 bulk-store cycles, 22 completion cycles. */
    uint64_t prof[32];
} bam_status_t;

/* ---- NVMe queue entries -------------------------------------------------------------- */
typedef struct BAM_ALIGNAS(64) { uint32_t dword[16]; } nvm_cmd_t;   /* 64-byte submission entry */
typedef struct BAM_ALIGNAS(16) { uint32_t dword[4]; } nvm_cpl_t;    /* 16-byte completion entry */

#define NVM_IO_FLUSH 0x00
#define NVM_IO_WRITE 0x01
#define NVM_IO_READ 0x02

/* cid table words: 0 = free, BAM_CID_INFLIGHT = owned, BAM_CID_DONE|status = completed */
#define BAM_CID_INFLIGHT 1u
#define BAM_CID_DONE 0x80000000u
#define BAM_CID_SPACE 65536u

/* ---- queue descriptor (one per SQ and one per CQ) -----------------------------------------
 * head/tail are virtual (never wrapped) counters; doorbell registers carry them modulo qs as
 * the NVMe specification requires. */
typedef struct {
    BAM_ALIGNAS(64) uint32_t head_lock;   /* CQ: held by the thread reaping completions      */
    BAM_ALIGNAS(64) uint32_t tail_lock;   /* SQ: held by the thread advancing the tail        */
    BAM_ALIGNAS(64) uint32_t head;        /* SQ: entries the controller has fetched; CQ: reaped */
    BAM_ALIGNAS(64) uint32_t tail;        /* SQ: entries published through the doorbell        */
    BAM_ALIGNAS(64) uint32_t in_ticket;   /* SQ: next slot ticket                              */
    BAM_ALIGNAS(64) uint32_t cid_ticket;  /* SQ: rotating start point of the command-id search */
    BAM_ALIGNAS(64) uint32_t* tickets;    /* SQ [qs]: ticket whose turn it is to use the slot  */
    uint32_t* tail_mark;                  /* SQ [qs]: 1 = command written, not yet published   */
    uint32_t* cid;                        /* SQ [65536]: command-id lock + completion mailbox  */
    bam_status_t* status;
    uint32_t qs, qs_minus_1, qs_log2;
    uint16_t no;                          /* queue number (unique per SQ/CQ pair)              */
    uint16_t es;                          /* entry size in bytes                               */
    int8_t phase;
    int8_t local;                         /* 1: the controller runs on this GPU (device scope suffices) */
    uint32_t last;
    volatile uint32_t* db;                /* doorbell register of this queue                   */
    volatile void* vaddr;                 /* queue memory                                      */
    uint64_t ioaddr;                      /* bus address of the queue memory (== vaddr here)   */
} nvm_queue_t;

typedef struct {
    uint32_t pageSize;
    uint32_t block_size, block_size_log, block_size_minus_1;
    uint32_t nvmNamespace;
    uint16_t qp_id;
    nvm_queue_t sq;
    nvm_queue_t cq;
} QueuePair;

/* ---- host-side controller handle and identify data (include/nvm_types.h:19-28, :198-232 in the
 * reference); the functions that fill them are declared in nvm_host_api.h -------------------------- */
typedef struct {
    size_t page_size;          /* memory page size used by the controller (MPS)        */
    uint8_t dstrd;             /* doorbell stride, encoded: registers are 4 << dstrd bytes apart */
    uint64_t timeout;          /* controller time-out in milliseconds                  */
    uint32_t max_qs;           /* maximum queue entries supported                      */
    size_t mm_size;            /* size of the register window                          */
    volatile void* mm_ptr;     /* register window: pinned host memory, doorbells at 0x1000 + ... */
} nvm_ctrl_t;

struct nvm_admin_reference;
typedef struct nvm_admin_reference* nvm_aq_ref;

struct nvm_ctrl_info {
    uint32_t nvme_version;
    size_t page_size, db_stride;
    uint64_t timeout;
    int contiguous;
    uint16_t max_entries;
    uint8_t pci_vendor[4];
    char serial_no[20], model_no[40], firmware[8];
    size_t max_data_size, max_data_pages, cq_entry_size, sq_entry_size, max_out_cmds, max_n_ns;
};
struct nvm_ns_info {
    uint32_t ns_id;
    size_t size, capacity, utilization;      /* in logical blocks */
    size_t lba_data_size, metadata_size;
};

/* One controller.  The leading members are what kernels use to pick a queue and count I/O (the
 * copy in device memory, Controller::d_ctrl_ptr, holds only those); the trailing members belong
 * to the host object.  In C++ the struct also carries the reference's constructor
 * Controller(path, nvmNamespace, cudaDevice, queueDepth, numQueues) (include/ctrl.h:148 there),
 * defined in this library's ctrl.h on top of the C ABI. */
#ifdef __cplusplus
struct bam_ctrl;
struct Controller {
    uint64_t access_counter;
    uint64_t queue_counter;
    QueuePair* d_qps;
    uint32_t n_qps;
    uint32_t page_size;
    uint32_t blk_size, blk_size_log;
    bam_status_t* status;
    /* host side */
    bam_ctrl* h;
    void* d_ctrl_ptr;
    uint32_t deviceId;
    uint32_t reserved_;
    nvm_ctrl_t* ctrl;                 /* libnvm handle over the same emulated controller */
    nvm_aq_ref aq_ref;
    struct nvm_ctrl_info info;
    struct nvm_ns_info ns;
    uint16_t n_sqs, n_cqs;

    Controller() = default;
    inline Controller(const char* path, uint32_t nvmNamespace, uint32_t cudaDevice, uint64_t queueDepth,
                      uint64_t numQueues, uint64_t store_bytes = 0);
    inline void close();
    inline void print_reset_stats();
};
#else
typedef struct {
    uint64_t access_counter;
    uint64_t queue_counter;
    QueuePair* d_qps;
    uint32_t n_qps;
    uint32_t page_size;
    uint32_t blk_size, blk_size_log;
    bam_status_t* status;
    void* h;
    void* d_ctrl_ptr;
    uint32_t deviceId;
    uint32_t reserved_;
    nvm_ctrl_t* ctrl;
    nvm_aq_ref aq_ref;
    struct nvm_ctrl_info info;
    struct nvm_ns_info ns;
    uint16_t n_sqs, n_cqs;
} Controller;
#endif

/* ---- emulated NVMe controller (device-resident command processor) ----------------------- */
typedef struct BAM_ALIGNAS(64) {
    uint32_t lock;          /* one controller warp reserves commands of this SQ at a time */
    uint32_t sq_fetch;      /* virtual SQ head: next entry to fetch               */
    uint32_t cq_tail;       /* virtual CQ tail: next completion slot to hand out   */
    uint32_t cq_head;       /* virtual CQ head reconstructed from the doorbell     */
    nvm_cmd_t* sq_mem;
    nvm_cpl_t* cq_mem;
    uint32_t* sq_db;
    uint32_t* cq_db;
    uint32_t qs, qs_log2;
    uint16_t sqid, cqid;
    uint32_t ctrl_index;    /* which controller of a multi-controller launch owns this queue */
    /* the media behind this queue: several controllers can be served by one launch, every queue
     * carries its own controller's store, fault plan and statistics */
    uint8_t* store;         /* backing store: device-visible mapping of pinned host memory   */
    uint64_t store_bytes;
    struct bam_fault_s* fault;
    uint64_t* served;       /* commands completed, for statistics                            */
    uint32_t cq_qs, cq_qs_log2;   /* depth of the completion queue (may differ from the SQ's)  */
    uint32_t sq_decoded;    /* virtual SQ position up to which entries have been read out: batches are reserved
                             * under `lock`, decoded outside it, and handed back here in order */
    uint32_t pad32_;
    uint64_t pad[2];
} bam_emu_qp_t;

#define BAM_FAULT_NONE 0
#define BAM_FAULT_DROP_CPL 1     /* swallow the completion of the nth command           */
#define BAM_FAULT_STATUS 2       /* complete the nth command with `status`               */
typedef struct bam_fault_s {
    uint32_t mode;
    uint32_t status;
    uint64_t nth;
    uint64_t counter;
} bam_fault_t;

typedef struct {
    bam_emu_qp_t* qps;
    uint32_t n_qps;
    uint32_t n_ctrl_blocks;     /* blocks [0, n_ctrl_blocks) of a fused launch run the controller */
    uint32_t lba_log2;          /* logical block size                                            */
    uint32_t mps_log2;          /* controller memory page size (PRP granule)                     */
    uint32_t batch;             /* commands one warp fetches per lock hold                        */
    uint32_t sys_scope;         /* 1: doorbells/completions use system scope, 0: device scope      */
    uint32_t* consumers_remaining;
    bam_status_t* status;
    /* Memory that commands may name as their data pointers, for submitters the controller does not trust
     * (host programs): a PRP outside every window completes with a data transfer error instead of being
     * touched.  NULL = no check (the library's own kernels build their PRPs from cache slots). */
    const struct bam_dma_window_s* windows;
    uint32_t n_windows;
    uint32_t procs_per_queue;   /* command processors (warps) that may serve one queue; 0 = the default of 8 */
    uint32_t max_grid;          /* host side only: cap on the blocks of a fused launch (bam_ctrl_set_max_grid), 0 = none */
    uint32_t reserved_;
} bam_emu_d_t;

typedef struct bam_dma_window_s { uint64_t base, bytes; } bam_dma_window_t;

/* ---- page cache -------------------------------------------------------------------------
 * Slot state word (32 bits, updated with CAS / fetch-ops):
 *   VALID | BUSY | DIRTY | pin count (29 bits) -- encodings of include/page_cache.h:57-62.
 * Unlike the reference the word belongs to the cache SLOT, not to the data page: the page
 * table is hashed (O(cache) memory) instead of direct-mapped (O(backing store)).
 * The bucket entries address slots with 24 bits: a cache holds at most 2^24 - 2 slots. */
#define BAM_VALID 0x80000000u
#define BAM_BUSY 0x40000000u
#define BAM_DIRTY 0x20000000u
#define BAM_CNT_MASK 0x1fffffffu
#define BAM_TAG_NONE 0xffffffffffffffffull
#define BAM_SLOT_NONE 0xffffffffu
#define BAM_SLOT_ERR 0xfffffffeu
#define BAM_SLOT_RETRY 0xfffffffdu   /* no slot could be claimed right now: release what you hold and ask again */
#define BAM_SLOT_MAX 0xfffffffcu     /* largest value that is a real slot index */
#define BAM_MAX_CACHE_SLOTS 0xfffffeull   /* 2^24 - 2: bucket entries hold 24-bit slot indices */

typedef struct BAM_ALIGNAS(16) {
    uint64_t tag;        /* (page index in range << range bits) | range id; BAM_TAG_NONE if unassigned */
    uint32_t state;
    uint32_t gen;        /* recycle generation: incremented when an eviction claims the slot, before its tag is
                          * cleared and long before new data can land in it.  Readers that pin nothing sample
                          * {state, gen} (one aligned 64-bit load) before and after they read page data. */
} bam_slot_t;

/* One page-table bucket = 32 bytes = one DRAM sector: a control word and seven entries.
 * control: bit 31 = insert lock, bits 30:0 = keys whose home is this bucket but live further on.
 * entry:   0xffffffff = empty, else (8-bit fingerprint << 24) | slot index. */
#define BAM_BUCKET_WORDS 8
#define BAM_BUCKET_LOCK 0x80000000u
#define BAM_ENTRY_EMPTY 0xffffffffu
#define BAM_MAX_PROBE 8

#define BAM_MAX_HANDS 16          /* clock hands of a large cache: an SM draws from hand smid % n_hands */
#define BAM_SLOTS_PER_HAND 4096   /* a cache gets a further hand for every so many slots, up to BAM_MAX_HANDS */
#define BAM_HAND_STRIDE 4         /* u64 words between two hands: one 32-byte sector each */
#define BAM_STAT_STRIPES 64
typedef struct BAM_ALIGNAS(32) { uint64_t hits, misses, read_ios, pad; } bam_stat_stripe_t;

/* How a range's pages are laid out over the controllers of a cache (data_dist_t of
 * include/page_cache.h:42, :558-582 in the reference): REPLICATE = every controller holds the whole
 * range, a read may go to any of them and a write-back goes to all; STRIPE = page p of the range
 * lives on controller p % n at backing page page_start + p / n. */
#define BAM_DIST_REPLICATE 0u
#define BAM_DIST_STRIPE 1u
#define BAM_ALL_CTRLS 0xffffffffu
#define BAM_MAX_CTRLS 16

#define BAM_MAX_RANGES 64
#define BAM_RANGE_BITS 6

typedef struct {
    uint8_t* base_addr;          /* n_slots * page_size bytes of cache in HBM   */
    uint64_t page_size, page_size_minus_1;
    uint32_t page_size_log;
    uint32_t n_slots;
    bam_slot_t* slots;
    uint32_t* table;             /* n_buckets * 8 words                          */
    uint32_t bucket_mask;        /* n_buckets - 1 (power of two)                 */
    uint32_t n_blocks_per_page;  /* logical blocks per cache page                */
    uint64_t* clock_hand;        /* the sweep positions (page_ticket in the reference): n_hands counters, one per
                                  * 32-byte sector; hand h sweeps the slots s with s % n_hands == h */
    Controller* d_ctrl;          /* backing controller (the first one when there are several) */
    Controller** d_ctrls;        /* [n_ctrls] all backing controllers             */
    uint32_t n_ctrls;
    uint32_t n_hands;            /* power of two; 1 for caches of fewer than BAM_SLOTS_PER_HAND * 2 slots */
    uint32_t* range_dists;       /* [BAM_MAX_RANGES] BAM_DIST_* of each range      */
    bam_stat_stripe_t* stats;    /* [BAM_STAT_STRIPES]                           */
    bam_status_t* status;
    uint32_t n_ranges_bits, n_ranges_mask;
    uint64_t* range_page_starts; /* [BAM_MAX_RANGES] first backing page of each range */
    uint64_t* prp_lists;         /* per-slot PRP lists, only when page_size > 2 controller pages */
    uint32_t prp_list_stride;    /* entries per slot in prp_lists */
} page_cache_d_t;

#endif /* BAM_ABI_TYPES_H */
