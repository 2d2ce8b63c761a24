/*
 * bam_internal.h -- host-side objects behind the opaque handles of bam_abi.h.
 */
#ifndef BAM_INTERNAL_H
#define BAM_INTERNAL_H

#include <vector>

#include "bam/abi_types.h"
#include "bam/array.cuh"
#include "bam/launch.cuh"

#define BAM_DEFAULT_CTRL_BLOCKS 48    /* controller blocks unless configured otherwise       */
#define BAM_DB_STRIDE_WORDS 8         /* doorbell stride: 32 bytes, one sector per register   */

/* fixed scratch of bam_cache_audit_noalloc (bam_noalloc.cu) */
#define BAM_AUDIT_NOALLOC_WORDS 1024
#define BAM_AUDIT_NOALLOC_SLOTS_PER_BLOCK 8192
#define BAM_AUDIT_NOALLOC_MAX_SLOTS ((uint64_t)(BAM_AUDIT_NOALLOC_WORDS - 1) * BAM_AUDIT_NOALLOC_SLOTS_PER_BLOCK)

struct bam_ctrl {
    int device = 0;
    int num_sms = 0;
    uint8_t* store_host = nullptr;
    uint8_t* store_dev = nullptr;
    uint64_t store_bytes = 0;
    uint32_t lba_bytes = 0;
    uint32_t n_qps = 0, qdepth = 0;
    uint64_t spin_timeout_ns = 0;
    uint64_t launch_timeout_ns = 0;
    void* arena = nullptr;
    size_t arena_bytes = 0;
    nvm_cmd_t* d_sq_mem = nullptr;
    nvm_cpl_t* d_cq_mem = nullptr;
    uint32_t* d_tickets = nullptr;
    uint32_t* d_marks = nullptr;
    uint32_t* d_cids = nullptr;
    uint32_t* d_doorbells = nullptr;
    bam_emu_qp_t* d_emu_qps = nullptr;
    QueuePair* d_qps = nullptr;
    Controller* d_ctrl = nullptr;
    bam_status_t* d_status = nullptr;
    uint32_t* d_remaining = nullptr;
    bam_fault_t* d_fault = nullptr;
    uint64_t* d_served = nullptr;
    bam_emu_d_t emu = {};
    uint32_t sys_scope = 0;           /* scope of doorbell/completion synchronisation          */
    uint32_t max_grid = 0;            /* 0 = as many blocks as fit                            */
    uint32_t last_grid = 0;
    /* membership in a multi-controller cache (bam_cache_create_multi) */
    struct bam_cache* group = nullptr;
    bam_ctrl* lead = nullptr;         /* first controller of the group: owner of the shared status block */
    uint32_t group_index = 0;
    bam_emu_qp_t* own_emu_qps = nullptr;   /* the arena's array, while d_emu_qps points into the group's */
};

struct bam_cache {
    bam_ctrl* ctrl = nullptr;         /* the (first) backing controller: launches run with its descriptor */
    std::vector<bam_ctrl*> members;   /* all backing controllers when there are several */
    bam_emu_qp_t* d_group_qps = nullptr;   /* controller-side state of all members' queues, contiguous */
    void* prp_lists_raw = nullptr;    /* the allocation d.prp_lists (page-aligned) lies in */
    page_cache_d_t d;
    uint64_t n_buckets = 0;
    uint32_t n_ranges = 0;
};

struct bam_array {
    bam_cache* pc = nullptr;
    uint32_t elem_bytes = 0;
    uint64_t n_elems = 0;
    bam::range_d_t<uint64_t> h_range;   /* the first range; layout does not depend on the element type */
    uint32_t n_ranges = 1;              /* launchers that take one range by value need n_ranges == 1 */
    void* d_range = nullptr;            /* device array of n_ranges descriptors */
    void* d_array = nullptr;
};

#endif
