/*
 * bam/emu_ctrl.cuh -- the emulated NVMe controller's command processor, as device code.
 *
 * The reference talks to a physical SSD; its device code relies on this much of the NVMe
 * contract (include/nvm_parallel_queue.h:168-330, :379-535; src/queue.cpp:12-42;
 * include/nvm_cmd.h:54-88): the controller consumes SQ entries up to the SQ tail doorbell,
 * executes READ/WRITE by moving (NLB+1) logical blocks between SLBA and the PRP-described
 * buffer, posts a 16-byte completion {DW2 = SQHD | SQID<<16, DW3 = CID | phase<<16 |
 * status<<17} whose phase bit starts at 1 and flips on every wrap of the CQ, never
 * overwrites completions the host has not released through the CQ head doorbell, and may
 * complete commands out of order.
 *
 * Here that controller is a set of threads: blocks [0, n_ctrl_blocks) of a fused launch run
 * emu_controller_main() while the remaining blocks run the workload.  The backing store is
 * pinned host memory mapped into the device address space, so every page a command reads
 * crosses the host link exactly once, as it would from an SSD.
 *
 * Data movement uses the bulk-copy engine (TMA, cp.async.bulk) and costs no registers: a lane
 * issues an asynchronous bulk load (media -> its 4 KiB shared-memory stage, completion counted on
 * an mbarrier), then an asynchronous bulk store (stage -> PRP target), and after the store has
 * completed releases the completion entry.  What limits a software controller is not the copy
 * but the chain of dependent protocol steps per command (doorbell read, lock, SQ entry read,
 * completion release at system scope), so those are overlapped SIMT-style: a processor is one
 * warp, it reserves a BATCH of commands from one queue under that queue's lock, all lanes read
 * one SQ entry each, and then BAM_EMU_LANES lanes transfer and complete the commands side by side.
 * Several processors may serve one queue; the lock covers only the reservation, and the batches
 * hand their SQ entries back in order (emu_hand_back) before any of their completions is posted.
 */
#ifndef BAM_EMU_CTRL_CUH
#define BAM_EMU_CTRL_CUH

#include "sync.cuh"

namespace bam {

#define BAM_SC_SUCCESS 0x00u
#define BAM_SC_INVALID_OPCODE 0x01u
#define BAM_SC_INVALID_FIELD 0x02u
#define BAM_SC_DATA_XFER_ERROR 0x04u
#define BAM_SC_PRP_OFFSET_INVALID 0x13u
#define BAM_SC_LBA_OUT_OF_RANGE 0x80u

#define BAM_EMU_STAGE_BYTES 4096
#define BAM_EMU_LANES 4             /* lanes of a controller warp that process commands (one stage each) */
#define BAM_EMU_WARPS 4             /* warps of a controller block that are command processors            */
#define BAM_EMU_MAX_PROCS_PER_QUEUE 32u
#define BAM_EMU_STAGES (BAM_EMU_LANES * BAM_EMU_WARPS)     /* 4 KiB stages per controller block           */
/* dynamic shared memory a controller block needs: the stages and one mbarrier per stage */
#define BAM_EMU_SMEM_BYTES (BAM_EMU_STAGES * BAM_EMU_STAGE_BYTES + 256)

/* ---- bulk-copy / mbarrier primitives ------------------------------------------------------- */
BAM_DEV uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
BAM_DEV void mbar_init(uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory"); }
BAM_DEV void mbar_expect_tx(uint32_t bar, uint32_t bytes) { asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory"); }
BAM_DEV bool mbar_test(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{ .reg .pred p; mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
BAM_DEV void bulk_load(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
BAM_DEV void bulk_store(void* dst, uint32_t src_smem, uint32_t bytes)
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src_smem), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
/* the stage can be overwritten once the bulk store has READ it; the data may still be on its way */
BAM_DEV void bulk_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
BAM_DEV void bulk_store_wait_all()
{
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    asm volatile("fence.proxy.async.global;" ::: "memory");
}

/* One fetched command, decoded. */
struct emu_cmd_t {
    uint64_t prp1, prp2, media_off;
    uint32_t bytes;        /* transfer length                               */
    uint32_t cq_virt;      /* completion slot handed out at fetch time      */
    uint32_t q;            /* queue pair index                              */
    uint32_t cid, sqhd, opc, status;
};

/* Post the completion of a command (release at system scope, after its payload). */
BAM_DEV void emu_post_completion(const bam_emu_d_t& c, const emu_cmd_t& m, uint32_t status)
{
    bam_emu_qp_t* s = &c.qps[m.q];
    bool drop = false;
    bam_fault_t* fault = s->fault;
    if (fault) {
        const uint32_t mode = ld_relaxed_gpu(&fault->mode);
        if (mode != BAM_FAULT_NONE) {
            const uint64_t k = atom_add_relaxed(&fault->counter, 1ull);
            if (k == fault->nth) {
                if (mode == BAM_FAULT_DROP_CPL) drop = true;
                else if (mode == BAM_FAULT_STATUS) status = fault->status;
            }
        }
    }
    if (!drop) {
        const uint32_t mask = s->cq_qs - 1u;
        const uint32_t phase = (~(m.cq_virt >> s->cq_qs_log2)) & 1u;
        nvm_cpl_t* e = &s->cq_mem[m.cq_virt & mask];
        *reinterpret_cast<volatile uint64_t*>(&e->dword[0]) = 0ull;
        const uint64_t dw2 = m.sqhd | ((uint32_t)s->sqid << 16);
        const uint64_t dw3 = m.cid | (phase << 16) | (status << 17);
        st_release_scoped(reinterpret_cast<uint64_t*>(&e->dword[2]), dw2 | (dw3 << 32), c.sys_scope != 0);
    }
}

/* What a processor needs from the queue descriptor to post the completions of a batch, loaded once per
 * batch instead of once per command (the descriptor lives in global memory: five dependent loads). */
struct emu_cq_view_t {
    nvm_cpl_t* cq_mem;
    uint32_t cq_mask, cq_log2, sqid;
    bool plain;                 /* no fault plan armed: completions are posted as they are */
};

BAM_DEV emu_cq_view_t emu_cq_view(const bam_emu_d_t& c, uint32_t q)
{
    const bam_emu_qp_t* s = &c.qps[q];
    emu_cq_view_t v;
    v.cq_mem = s->cq_mem;
    v.cq_mask = s->cq_qs - 1u;
    v.cq_log2 = s->cq_qs_log2;
    v.sqid = s->sqid;
    v.plain = s->fault == nullptr || ld_relaxed_gpu(&s->fault->mode) == BAM_FAULT_NONE;
    return v;
}

/* emu_post_completion for the common case (no fault plan), from the per-batch view; the caller counts the
 * served commands once per batch. */
BAM_DEV void emu_post_completion_plain(const bam_emu_d_t& c, const emu_cq_view_t& v, const emu_cmd_t& m, uint32_t status)
{
    const uint32_t phase = (~(m.cq_virt >> v.cq_log2)) & 1u;
    nvm_cpl_t* e = &v.cq_mem[m.cq_virt & v.cq_mask];
    *reinterpret_cast<volatile uint64_t*>(&e->dword[0]) = 0ull;
    const uint64_t dw2 = m.sqhd | (v.sqid << 16);
    const uint64_t dw3 = m.cid | (phase << 16) | (status << 17);
    st_release_scoped(reinterpret_cast<uint64_t*>(&e->dword[2]), dw2 | (dw3 << 32), c.sys_scope != 0);
}

/* Lane 0 of a processor: look at queue pair q and, if commands are waiting, take the queue's lock,
 * reserve up to `want` of them together with their completion slots, and release the lock.  Returns
 * the number reserved (0: nothing taken).  The doorbells are polled with relaxed loads; one
 * acquire fence follows only when there is work. */
BAM_DEV uint32_t emu_reserve(const bam_emu_d_t& c, uint32_t q, uint32_t want, uint32_t& fetch, uint32_t& cqbase)
{
    bam_emu_qp_t* s = &c.qps[q];
    const uint32_t mask = s->qs - 1u;
    if (ld_relaxed_sys(s->sq_db) == (ld_relaxed_gpu(&s->sq_fetch) & mask)) return 0;
    if (atom_cas_acquire(&s->lock, 0u, 1u) != 0u) return 0;
    fetch = ld_relaxed_gpu(&s->sq_fetch);
    const uint32_t tail = ld_relaxed_sys(s->sq_db);
    const uint32_t hdb = ld_relaxed_sys(s->cq_db);
    uint32_t cq_head = ld_relaxed_gpu(&s->cq_head);
    cqbase = ld_relaxed_gpu(&s->cq_tail);
    const uint32_t avail = (tail - fetch) & mask;
    const uint32_t cmask = s->cq_qs - 1u;
    cq_head += (hdb - cq_head) & cmask;
    const uint32_t space = cmask - (cqbase - cq_head);         /* keep one completion slot open */
    uint32_t n = avail < space ? avail : space;
    /* a shallow queue is spread over more processors: a sixteenth of its depth per batch (8 at least) keeps
     * more of its commands in transfer at once than two or three full batches would */
    uint32_t most = s->qs >> 4;
    if (most < 8u) most = 8u;
    if (most > want) most = want;
    if (n > most) n = most;
    if (n == 0) { st_release_gpu(&s->lock, 0u); return 0; }
    fence_acq_rel_scoped(c.sys_scope != 0);                    /* acquire the command bytes      */
    st_relaxed_gpu(&s->cq_head, cq_head);
    st_relaxed_gpu(&s->cq_tail, cqbase + n);
    st_relaxed_gpu(&s->sq_fetch, fetch + n);
    st_release_gpu(&s->lock, 0u);                              /* the next batch can be reserved while this one is read out */
    return n;
}

/* Lane 0 of a processor, after its warp has read the SQ entries [fetch, fetch + n) of queue q: hand them
 * back IN ORDER.  A completion's SQ-head value says that every entry below it has been consumed, and the
 * completions of a later batch may be posted before those of an earlier one; with this step the value is
 * true at the moment it is posted.  (A submitter that consumes completions strictly in queue order -- this
 * library's reaper, the reference's move_head_cq -- would be safe without it, because completion slots are
 * reserved in SQ order and an earlier batch posts only after it has read its entries; one that looks ahead
 * in the completion queue and trusts what it sees there would not.) */
BAM_DEV void emu_hand_back(const bam_emu_d_t& c, uint32_t q, uint32_t fetch, uint32_t n)
{
    uint32_t* dec = &c.qps[q].sq_decoded;
    const uint64_t t0 = global_timer_ns();
    uint32_t polls = 0;
    while (ld_acquire_gpu(dec) != fetch) {
        if (((++polls) & 255u) == 0u && global_timer_ns() - t0 > c.status->spin_timeout_ns) {
            status_fail(c.status, BAM_ETIMEDOUT, BAM_AT_SQ_ORDER, fetch);
            return;                                            /* the launch is draining: leave the counter alone */
        }
    }
    st_release_gpu(dec, fetch + n);
}

/* Read and decode SQ entry `fetch_i` of queue pair q. */
BAM_DEV void emu_decode(const bam_emu_d_t& c, uint32_t q, uint32_t fetch_i, uint32_t cq_virt, uint32_t sqhd, emu_cmd_t& m)
{
    bam_emu_qp_t* s = &c.qps[q];
    const uint8_t* p = reinterpret_cast<const uint8_t*>(&s->sq_mem[fetch_i & (s->qs - 1u)]);
    const uint4 a = ld_cg_v4(p), b = ld_cg_v4(p + 16), d = ld_cg_v4(p + 32), e = ld_cg_v4(p + 48);
    m.opc = a.x & 0x7fu;
    m.cid = a.x >> 16;
    m.prp1 = ((uint64_t)b.w << 32) | b.z;
    m.prp2 = ((uint64_t)d.y << 32) | d.x;
    const uint64_t slba = ((uint64_t)d.w << 32) | d.z;
    const uint64_t bytes = (uint64_t)((e.x & 0xffffu) + 1u) << c.lba_log2;
    m.media_off = slba << c.lba_log2;
    m.bytes = (uint32_t)bytes;
    m.cq_virt = cq_virt;
    m.q = q;
    m.sqhd = sqhd;
    m.status = BAM_SC_SUCCESS;
    if (m.opc != NVM_IO_READ && m.opc != NVM_IO_WRITE) m.status = BAM_SC_INVALID_OPCODE;
    else if (m.media_off + bytes > s->store_bytes || m.media_off + bytes < m.media_off) m.status = BAM_SC_LBA_OUT_OF_RANGE;
    else if ((m.prp1 & 15u) || (bytes & 15u)) m.status = BAM_SC_INVALID_FIELD;
}

/* Whether [mem, mem + len) lies inside one of the memory windows commands of this controller may name. */
BAM_DEV bool emu_in_window(const bam_emu_d_t& c, uint64_t mem, uint64_t len)
{
    for (uint32_t k = 0; k < c.n_windows; k++)
        if (mem >= c.windows[k].base && mem + len <= c.windows[k].base + c.windows[k].bytes && mem + len >= mem) return true;
    return false;
}

/* The next data-page address of a PRP list.  The list lies in memory pages; when entries still follow,
 * the last 8 bytes of a list page hold the address of the next list page instead of a data page
 * (`more_follow`: this entry is not the transfer's last). */
struct emu_list_step { uint64_t mem, next; uint32_t status; };
BAM_DEV __noinline__ emu_list_step emu_list_entry(const bam_emu_d_t& c, uint64_t mps, uint64_t list_ptr, bool more_follow)
{
    emu_list_step r = { 0, 0, BAM_SC_PRP_OFFSET_INVALID };
    for (int hop = 0; hop < 2; hop++) {
        if (list_ptr & 7u) return r;
        if (c.windows && !emu_in_window(c, list_ptr, 8)) { r.status = BAM_SC_DATA_XFER_ERROR; return r; }
        const uint64_t e = ld_relaxed_sys(reinterpret_cast<const uint64_t*>(list_ptr));
        const bool last_of_page = ((list_ptr + 8) & (mps - 1)) == 0;
        if (hop == 0 && last_of_page && more_follow) { list_ptr = e; continue; }     /* follow the link, then read the entry there */
        r.mem = e;
        r.next = list_ptr + 8;
        r.status = BAM_SC_SUCCESS;
        return r;
    }
    return r;
}

/* Move the data of one command through this lane's stage, segment by segment (a 4 KiB page is
 * one segment).  Returns the NVMe status. */
BAM_DEV uint32_t emu_transfer(const bam_emu_d_t& c, const emu_cmd_t& m, uint32_t stage_smem, uint32_t bar, uint32_t& parity)
{
    const uint64_t mps = 1ull << c.mps_log2;
    /* a PRP segment is moved through one stage in one piece: the controller's memory page size must be the
     * stage size (both 4 KiB; bam_ctrl_create and the libnvm layer set mps_log2 = 12) */
    if (mps != BAM_EMU_STAGE_BYTES) return BAM_SC_INVALID_FIELD;
    uint8_t* const store = c.qps[m.q].store;               /* the media of the controller that owns the queue */
    uint64_t first = mps - (m.prp1 & (mps - 1));
    if (first > m.bytes) first = m.bytes;
    const bool use_list = (m.bytes - first) > mps;
    uint32_t done = 0;
    uint64_t list_ptr = m.prp2;                            /* with use_list: where the next list entry lies */
    while (done < m.bytes) {
        uint64_t mem;
        uint32_t len;
        if (done == 0) { mem = m.prp1; len = (uint32_t)first; }
        else {
            if (use_list) {
                const emu_list_step e = emu_list_entry(c, mps, list_ptr, m.bytes - done > mps);
                if (e.status != BAM_SC_SUCCESS) return e.status;
                mem = e.mem;
                list_ptr = e.next;
            } else mem = m.prp2;
            if (mem & (mps - 1)) return BAM_SC_INVALID_FIELD;
            len = m.bytes - done < mps ? m.bytes - done : (uint32_t)mps;
        }
        if (len > BAM_EMU_STAGE_BYTES) len = BAM_EMU_STAGE_BYTES;
        if (c.windows && !emu_in_window(c, mem, len)) return BAM_SC_DATA_XFER_ERROR;     /* an untrusted submitter */
        uint8_t* media = store + m.media_off + done;
        const void* src = (m.opc == NVM_IO_READ) ? (const void*)media : (const void*)mem;
        void* dst = (m.opc == NVM_IO_READ) ? (void*)mem : (void*)media;
        BAM_PROF_T0();
        /* a WRITE's source is a cache page other threads wrote with ordinary stores: order them
         * before the bulk engine's read */
        asm volatile("fence.proxy.async.global;" ::: "memory");
        mbar_expect_tx(bar, len);
        bulk_load(stage_smem, src, len, bar);
        const uint64_t t0 = global_timer_ns();
        uint32_t polls = 0;
        while (!mbar_test(bar, parity)) {
            if (((++polls) & 1023u) == 0u) {
                const uint64_t waited = global_timer_ns() - t0;
                if (waited > c.status->spin_timeout_ns) status_fail(c.status, BAM_ETIMEDOUT, BAM_AT_TMA, (uint64_t)dst);
                if (waited > 2 * c.status->spin_timeout_ns) return 0xffffffffu;     /* the copy never landed */
            }
        }
        parity ^= 1u;
        BAM_PROF_LAP(c.status, 20);
        bulk_store(dst, stage_smem, len);
        bulk_store_wait_all();
        BAM_PROF_LAP(c.status, 21);
        done += len;
    }
    return BAM_SC_SUCCESS;
}

/* A transfer of one segment that fits a stage -- every 4 KiB page read or write of the cache -- can be split
 * in two so that a mover lane overlaps the landing of one page with the load of the next:
 * emu_load_page_overlapped starts the load into the stage, runs `while_in_flight` (the caller's chance to let
 * the previous page land and post its completion), then waits for the load (returns false with *status set
 * when the command must not be transferred, or with *status == 0xffffffff when the load never completed).
 * The caller then starts the store with bulk_store and may start the next load as soon as
 * bulk_store_wait_read() says the stage has been read. */
BAM_DEV bool emu_one_segment(const bam_emu_d_t& c, const emu_cmd_t& m)
{
    const uint64_t mps = 1ull << c.mps_log2;
    return mps == BAM_EMU_STAGE_BYTES && m.bytes <= mps - (m.prp1 & (mps - 1));
}

template <class WhileInFlight>
BAM_DEV bool emu_load_page_overlapped(const bam_emu_d_t& c, const emu_cmd_t& m, uint32_t stage_smem, uint32_t bar, uint32_t& parity,
                                      void*& dst, uint32_t* status, WhileInFlight while_in_flight)
{
    if (c.windows && !emu_in_window(c, m.prp1, m.bytes)) { while_in_flight(); *status = BAM_SC_DATA_XFER_ERROR; return false; }
    uint8_t* media = c.qps[m.q].store + m.media_off;
    const void* src = (m.opc == NVM_IO_READ) ? (const void*)media : (const void*)m.prp1;
    dst = (m.opc == NVM_IO_READ) ? (void*)m.prp1 : (void*)media;
    BAM_PROF_T0();
    /* a WRITE's source is a cache page other threads wrote with ordinary stores: order them
     * before the bulk engine's read */
    asm volatile("fence.proxy.async.global;" ::: "memory");
    mbar_expect_tx(bar, m.bytes);
    bulk_load(stage_smem, src, m.bytes, bar);
    while_in_flight();
    const uint64_t t0 = global_timer_ns();
    uint32_t polls = 0;
    while (!mbar_test(bar, parity)) {
        if (((++polls) & 1023u) == 0u) {
            const uint64_t waited = global_timer_ns() - t0;
            if (waited > c.status->spin_timeout_ns) status_fail(c.status, BAM_ETIMEDOUT, BAM_AT_TMA, (uint64_t)dst);
            if (waited > 2 * c.status->spin_timeout_ns) { *status = 0xffffffffu; return false; }     /* the copy never landed */
        }
    }
    parity ^= 1u;
    BAM_PROF_LAP(c.status, 20);
    return true;
}

/* Body of a controller block.  Warps [0, BAM_EMU_WARPS) are command processors; in each, lanes
 * [0, BAM_EMU_LANES) own one 4 KiB stage and one mbarrier.  A processor reserves a batch of up to 32
 * commands from one queue under that queue's lock (held for the reservation only), every lane decodes
 * one of them side by side, the entries are handed back in order, and the stage-owning lanes transfer and complete the commands
 * BAM_EMU_LANES at a time, so the latencies of a round overlap and the lock is held once per batch.  Runs until
 * every workload block of the launch has finished (consumers_remaining == 0) or an error has been
 * flagged.  `smem` is the block's dynamic shared memory (BAM_EMU_SMEM_BYTES, 128-byte aligned). */
BAM_DEV void emu_controller_main(const bam_emu_d_t& c, uint8_t* smem)
{
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t wib = threadIdx.x >> 5;
    if (wib >= BAM_EMU_WARPS) return;
    const uint32_t full = 0xffffffffu;
    const bool mover = lane < BAM_EMU_LANES;               /* lanes that own a stage and move data */
    const uint32_t me = blockIdx.x * BAM_EMU_WARPS + wib;
    const uint32_t n_procs = c.n_ctrl_blocks * BAM_EMU_WARPS;
    const uint32_t my_stage = wib * BAM_EMU_LANES + (lane & (BAM_EMU_LANES - 1));
    const uint32_t stage_smem = smem_u32(smem + (size_t)my_stage * BAM_EMU_STAGE_BYTES);
    const uint32_t bar = smem_u32(smem + (size_t)BAM_EMU_STAGES * BAM_EMU_STAGE_BYTES + my_stage * 8);
    if (mover) mbar_init(bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp(full);

    const uint64_t t_start = global_timer_ns();
    /* with few queues, more than a few dozen processors per queue only add polling traffic on its lock */
    const bool spare = me >= c.n_qps * (c.procs_per_queue ? c.procs_per_queue : BAM_EMU_MAX_PROCS_PER_QUEUE);
    const uint32_t rounds = (c.n_qps + n_procs - 1) / n_procs;
    uint32_t want = c.batch < 32u ? c.batch : 32u;
    if (want == 0) want = 1;
    uint32_t parity = 0;
    uint32_t q = me % c.n_qps;
    uint32_t idle_ns = 32, idle_rounds = 0;

    for (;;) {
        uint32_t n = 0, fetch = 0, cqbase = 0, bq = 0;
#ifdef BAM_PROFILE
        long long pt = clock64();
#endif
        if (lane == 0 && !spare) {
            for (uint32_t r = 0; r < rounds && n == 0; r++) {
                n = emu_reserve(c, q, want, fetch, cqbase);
                bq = q;
                q += n_procs;
                while (q >= c.n_qps) q -= c.n_qps;
            }
        }
        n = __shfl_sync(full, n, 0);
        if (n) {
            fetch = __shfl_sync(full, fetch, 0);
            cqbase = __shfl_sync(full, cqbase, 0);
            bq = __shfl_sync(full, bq, 0);
            __syncwarp(full);                                  /* lane 0's acquire fence covers the batch */
            const uint32_t qmask = c.qps[bq].qs - 1u;
            /* every lane decodes one SQ entry of the batch (the queue's lock is free again already) */
            emu_cmd_t m;
            m.prp1 = m.prp2 = m.media_off = 0; m.bytes = m.cq_virt = m.cid = m.opc = 0; m.status = BAM_SC_SUCCESS;
            if (lane < n) emu_decode(c, bq, fetch + lane, cqbase + lane, (fetch + n) & qmask, m);
            __syncwarp(full);
            const emu_cq_view_t cqv = emu_cq_view(c, bq);
            if (lane == 0) {
                emu_hand_back(c, bq, fetch, n);
#ifdef BAM_PROFILE
                { long long t = clock64(); BAM_PROF_ADD(c.status, 16, 1); BAM_PROF_ADD(c.status, 17, n); BAM_PROF_ADD(c.status, 18, t - pt); pt = t; }
#endif
            }
            /* the mover lanes work through the batch, BAM_EMU_LANES commands per round.  A lane keeps the store of
             * its previous page in flight while it loads the next one: the stage is free again as soon as the bulk
             * store has read it, and the previous command's completion is posted once its page has landed */
            emu_cmd_t prev;
            bool have_prev = false;
            auto post = [&](const emu_cmd_t& w, uint32_t status) {
#ifdef BAM_PROFILE
                long long t1 = clock64();
#endif
                if (status != 0xffffffffu) {
                    if (cqv.plain) emu_post_completion_plain(c, cqv, w, status);
                    else emu_post_completion(c, w, status);
                }
#ifdef BAM_PROFILE
                BAM_PROF_ADD(c.status, 22, clock64() - t1);
#endif
            };
            auto land_prev = [&]() {                       /* the previous page has landed: complete its command */
                if (have_prev) { bulk_store_wait_all(); post(prev, BAM_SC_SUCCESS); have_prev = false; }
            };
            for (uint32_t r0 = 0; r0 < n; r0 += BAM_EMU_LANES) {
                const uint32_t src = r0 + (lane & (BAM_EMU_LANES - 1));
                emu_cmd_t w;
                w.prp1 = __shfl_sync(full, m.prp1, src);
                w.prp2 = __shfl_sync(full, m.prp2, src);
                w.media_off = __shfl_sync(full, m.media_off, src);
                w.bytes = __shfl_sync(full, m.bytes, src);
                w.cq_virt = __shfl_sync(full, m.cq_virt, src);
                w.cid = __shfl_sync(full, m.cid, src);
                w.opc = __shfl_sync(full, m.opc, src);
                w.status = __shfl_sync(full, m.status, src);
                w.q = bq;
                w.sqhd = (fetch + n) & qmask;
                if (mover && src < n) {
                    uint32_t status = w.status;
                    if (status == BAM_SC_SUCCESS && emu_one_segment(c, w)) {
                        if (have_prev) bulk_store_wait_read();           /* the stage is free for the next load */
                        void* dst = nullptr;
                        /* (the load is started inside; while it is in flight the previous page lands) */
                        const bool loaded = emu_load_page_overlapped(c, w, stage_smem, bar, parity, dst, &status, land_prev);
                        if (loaded) { bulk_store(dst, stage_smem, w.bytes); prev = w; have_prev = true; }
                        else post(w, status);
                    } else {
                        land_prev();
                        if (status == BAM_SC_SUCCESS) status = emu_transfer(c, w, stage_smem, bar, parity);
                        post(w, status);
                    }
                }
                __syncwarp(full);
            }
            if (mover) land_prev();
            if (lane == 0) red_add_relaxed(c.qps[bq].served, (uint64_t)n);      /* statistics: once per batch */
#ifdef BAM_PROFILE
            if (lane == 0) BAM_PROF_ADD(c.status, 19, clock64() - pt);
#endif
            idle_ns = 32; idle_rounds = 0;
            continue;
        }
        uint32_t stop = 0;
        if (lane == 0) {
            stop = ((c.sys_scope ? ld_acquire_sys(c.consumers_remaining) : ld_acquire_gpu(c.consumers_remaining)) == 0u) || status_bad(c.status);
            if (!stop && ((++idle_rounds) & 63u) == 0u && global_timer_ns() - t_start > c.status->launch_timeout_ns) {
                status_fail(c.status, BAM_ETIMEDOUT, BAM_AT_LAUNCH, 0);
                stop = 1;
            }
        }
        stop = __shfl_sync(full, stop, 0);
#ifdef BAM_PROFILE
        if (lane == 0) { BAM_PROF_ADD(c.status, 23, 1); BAM_PROF_ADD(c.status, 24, clock64() - pt); }
#endif
        if (stop) break;
        __nanosleep(spare ? 2000u : idle_ns);
        if (idle_ns < 512) idle_ns <<= 1;
    }
}

}  // namespace bam
#endif
