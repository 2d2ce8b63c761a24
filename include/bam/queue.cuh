/*
 * bam/queue.cuh -- the GPU-parallel NVMe submission/completion protocol.
 *
 * Same contract as the reference's include/nvm_parallel_queue.h (thousands of threads share
 * one SQ/CQ pair without a global lock; doorbells are batched), redesigned:
 *
 *   get_cid / put_cid   (ref :36-57)   The 65536-entry table is kept, but each word is both the
 *                                      lock and the completion mailbox of that command id.
 *   sq_enqueue          (ref :168-330) Ticket -> slot.  A slot has ONE turn word holding the
 *                                      ticket allowed to write it (the reference uses a 2-step
 *                                      even/odd turn id, :28-31, :327, :113-115).  Writers mark
 *                                      their slot; whoever holds tail_lock publishes every
 *                                      contiguous marked slot with one release.sys doorbell store.
 *   cq_poll             (ref :379-422) The reference lets every waiter rescan the CQ from head
 *                                      (O(depth) per attempt per waiter).  Here a waiter spins on
 *                                      its own mailbox word; whoever holds head_lock reaps the CQ
 *                                      in order, phase bit by phase bit, and posts each
 *                                      completion's status to the mailbox of its command id:
 *                                      O(1) work per completion in total.
 *   cq_dequeue /        (ref :425-535, The reaper also does what cq_dequeue + move_head_cq do:
 *   move_head_cq         :83-123)      reads SQHD from the newest completion, re-opens the SQ
 *                                      slots the controller has fetched, advances the CQ head and
 *                                      rings the CQ head doorbell once per batch.
 *
 * Memory model: command bytes -> st.release.gpu(mark) -> ld.acquire.gpu(mark) by the
 * publisher -> st.release.sys(doorbell).  Completion: controller st.release.sys(DW2|DW3 as
 * one 64-bit word) -> reaper ld.relaxed.sys + fence.acq_rel.sys -> st.release.gpu(mailbox) ->
 * waiter ld.acquire.gpu(mailbox) -> page payload visible.  No extra "flush" read is needed
 * (the reference issues one: page_cache.h:1961-2007).
 */
#ifndef BAM_QUEUE_CUH
#define BAM_QUEUE_CUH

#include "sync.cuh"

namespace bam {

/* ---- command builders (same field placement as include/nvm_cmd.h:54-88) ---------------- */
__host__ __device__ __forceinline__ void nvm_cmd_header(nvm_cmd_t* cmd, uint16_t cid, uint8_t opcode, uint32_t ns_id)
{
    cmd->dword[0] = ((uint32_t)cid << 16) | (opcode & 0x7fu);   /* PSDT = 0 (PRP), FUSE = 0 */
    cmd->dword[1] = ns_id;
}

__host__ __device__ __forceinline__ void nvm_cmd_data_ptr(nvm_cmd_t* cmd, uint64_t prp1, uint64_t prp2)
{
    cmd->dword[0] &= ~((0x03u << 14) | (0x03u << 8));
    cmd->dword[6] = (uint32_t)prp1;
    cmd->dword[7] = (uint32_t)(prp1 >> 32);
    cmd->dword[8] = (uint32_t)prp2;
    cmd->dword[9] = (uint32_t)(prp2 >> 32);
}

__host__ __device__ __forceinline__ void nvm_cmd_rw_blks(nvm_cmd_t* cmd, uint64_t start_lba, uint16_t n_blks)
{
    cmd->dword[10] = (uint32_t)start_lba;
    cmd->dword[11] = (uint32_t)(start_lba >> 32);
    cmd->dword[12] = (cmd->dword[12] & 0xffff0000u) | ((uint32_t)(n_blks - 1) & 0xffffu);
}

#define BAM_CID_ERR 0xffffffffu
#define BAM_POS_ERR 0xffffffffu
#define BAM_CPL_ERR 0xffffffffu

/* Claim a command id.  Returns BAM_CID_ERR if none could be claimed within the wait limit. */
BAM_DEV uint32_t get_cid(nvm_queue_t* sq)
{
    spin_t sp;
    for (;;) {
        uint32_t id = atom_add_relaxed(&sq->cid_ticket, 1u) & (BAM_CID_SPACE - 1u);
        if (atom_cas_acquire(&sq->cid[id], 0u, BAM_CID_INFLIGHT) == 0u) return id;
        if (sp.expired(sq->status, BAM_AT_CID)) return BAM_CID_ERR;
    }
}

BAM_DEV void put_cid(nvm_queue_t* sq, uint32_t id) { st_release_gpu(&sq->cid[id], 0u); }

/* Submit one command given as four 16-byte quarters (kept in registers).  Returns the SQ slot it
 * was written to, or BAM_POS_ERR. */
BAM_DEV uint32_t sq_enqueue_regs(nvm_queue_t* sq, uint4 c0, uint4 c1, uint4 c2, uint4 c3)
{
    bam_status_t* st = sq->status;
    const uint32_t mask = sq->qs_minus_1;
    const uint32_t ticket = atom_add_relaxed(&sq->in_ticket, 1u);
    const uint32_t pos = ticket & mask;

    spin_t sp;
    while (ld_acquire_gpu(&sq->tickets[pos]) != ticket)
        if (sp.expired(st, BAM_AT_SQ_TURN, ticket)) return BAM_POS_ERR;

    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<nvm_cmd_t*>(const_cast<void*>(sq->vaddr)) + pos);
    dst[0] = c0; dst[1] = c1; dst[2] = c2; dst[3] = c3;
    st_release_gpu(&sq->tail_mark[pos], 1u);

    sp.reset();
    while (ld_relaxed_gpu(&sq->tail_mark[pos]) == 1u) {
        if (ld_relaxed_gpu(&sq->tail_lock) == 0u && atom_cas_acquire(&sq->tail_lock, 0u, 1u) == 0u) {
            const uint32_t tail = ld_relaxed_gpu(&sq->tail);
            const uint32_t head = ld_acquire_gpu(&sq->head);
            uint32_t n = 0;
            /* a queue of qs entries holds at most qs-1 (tail == head means empty) */
            while ((tail + n - head) < mask && ld_acquire_gpu(&sq->tail_mark[(tail + n) & mask]) == 1u) {
                st_relaxed_gpu(&sq->tail_mark[(tail + n) & mask], 0u);
                n++;
            }
            if (n) {
                st_release_sys(const_cast<uint32_t*>(sq->db), (tail + n) & mask);
                st_release_gpu(&sq->tail, tail + n);
            }
            st_release_gpu(&sq->tail_lock, 0u);
            if (n) continue;
        }
        if (sp.expired(st, BAM_AT_SQ_DOORBELL, ticket)) return BAM_POS_ERR;
    }
    return pos;
}

/* Same, from a command in memory (the reference's signature, nvm_parallel_queue.h:168). */
BAM_DEV uint32_t sq_enqueue(nvm_queue_t* sq, const nvm_cmd_t* cmd)
{
    const uint4* src = reinterpret_cast<const uint4*>(cmd);
    return sq_enqueue_regs(sq, src[0], src[1], src[2], src[3]);
}

/* Reap the completion queue (caller holds cq->head_lock).  Returns entries consumed. */
BAM_DEV uint32_t cq_reap(QueuePair* qp)
{
    nvm_queue_t* sq = &qp->sq;
    nvm_queue_t* cq = &qp->cq;
    const uint32_t mask = cq->qs_minus_1;
    const uint32_t lg = cq->qs_log2;
    nvm_cpl_t* mem = reinterpret_cast<nvm_cpl_t*>(const_cast<void*>(cq->vaddr));
    const uint32_t h = ld_relaxed_gpu(&cq->head);
    uint32_t total = 0;
    uint32_t sqhd = 0;
    for (;;) {
        uint64_t e[4];
#pragma unroll
        for (int i = 0; i < 4; i++)
            e[i] = ld_relaxed_sys(reinterpret_cast<const uint64_t*>(&mem[(h + total + i) & mask].dword[2]));
        uint32_t k = 0;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            uint32_t want = (~((h + total + i) >> lg)) & 1u;
            uint32_t have = (uint32_t)(e[i] >> 48) & 1u;
            if (k == (uint32_t)i && have == want) k++;
        }
        if (total + k > mask) k = mask - total;          /* never more than qs-1 per pass */
        if (k == 0) break;
        fence_acq_rel_sys();                               /* acquire the k payloads */
#pragma unroll
        for (int i = 0; i < 4; i++) {
            if ((uint32_t)i < k) {
                uint32_t dw3 = (uint32_t)(e[i] >> 32);
                st_release_gpu(&sq->cid[dw3 & 0xffffu], BAM_CID_DONE | (dw3 >> 17));
                sqhd = (uint32_t)e[i] & 0xffffu;
            }
        }
        total += k;
        if (k < 4 || total >= mask) break;
    }
    if (total) {
        /* re-open the SQ slots the controller has fetched (SQHD of the newest completion) */
        const uint32_t cur = ld_relaxed_gpu(&sq->head);
        const uint32_t delta = (sqhd - cur) & sq->qs_minus_1;
        for (uint32_t i = 0; i < delta; i++)
            st_release_gpu(&sq->tickets[(cur + i) & sq->qs_minus_1], cur + i + sq->qs);
        if (delta) st_release_gpu(&sq->head, cur + delta);
        st_release_gpu(&cq->head, h + total);
        st_release_sys(const_cast<uint32_t*>(cq->db), (h + total) & mask);
    }
    return total;
}

/* Wait for the completion of command `cid`.  Returns the NVMe status field (0 = success) or
 * BAM_CPL_ERR when the wait was abandoned. */
BAM_DEV uint32_t cq_poll(QueuePair* qp, uint32_t cid)
{
    nvm_queue_t* sq = &qp->sq;
    nvm_queue_t* cq = &qp->cq;
    spin_t sp;
    for (;;) {
        uint32_t v = ld_acquire_gpu(&sq->cid[cid]);
        if (v & BAM_CID_DONE) return v & 0x7fffu;
        if (ld_relaxed_gpu(&cq->head_lock) == 0u && atom_cas_acquire(&cq->head_lock, 0u, 1u) == 0u) {
            uint32_t n = cq_reap(qp);
            st_release_gpu(&cq->head_lock, 0u);
            if (n) continue;
        }
        if (sp.expired(sq->status, BAM_AT_CQ_WAIT, cid)) return BAM_CPL_ERR;
    }
}

/* Kept for source compatibility with callers of the reference API: the reaper inside cq_poll
 * has already consumed the entry, advanced the head and rung the doorbell. */
BAM_DEV void cq_dequeue(nvm_queue_t*, uint32_t, nvm_queue_t*) {}

/* One blocking I/O: build the command, submit, wait, retire.  Counterpart of read_data /
 * write_data / access_data (include/page_cache.h:2009-2132); `bus_addr` is PRP1 (the cache
 * slot), `bus_addr2` PRP2 when the transfer spans more than one controller page.
 * Returns 0, or a BAM_E* code after recording it in the status block. */
BAM_DEV int access_data_raw(QueuePair* qp, uint64_t starting_lba, uint32_t n_blocks,
                            uint64_t bus_addr, uint64_t bus_addr2, uint8_t opcode)
{
    bam_status_t* st = qp->sq.status;
    if (status_bad(st)) return BAM_EIO;
    uint32_t cid = get_cid(&qp->sq);
    if (cid == BAM_CID_ERR) return BAM_ETIMEDOUT;
    /* DW0 = CID | opcode, DW1 = NSID, DW6-9 = PRP1/PRP2, DW10-11 = SLBA, DW12 = NLB-1
     * (the fields nvm_cmd_header / nvm_cmd_data_ptr / nvm_cmd_rw_blks set), built in registers */
    const uint4 c0 = make_uint4((cid << 16) | (opcode & 0x7fu), qp->nvmNamespace, 0u, 0u);
    const uint4 c1 = make_uint4(0u, 0u, (uint32_t)bus_addr, (uint32_t)(bus_addr >> 32));
    const uint4 c2 = make_uint4((uint32_t)bus_addr2, (uint32_t)(bus_addr2 >> 32), (uint32_t)starting_lba, (uint32_t)(starting_lba >> 32));
    const uint4 c3 = make_uint4((n_blocks - 1u) & 0xffffu, 0u, 0u, 0u);
    if (sq_enqueue_regs(&qp->sq, c0, c1, c2, c3) == BAM_POS_ERR) return BAM_ETIMEDOUT;
    uint32_t status = cq_poll(qp, cid);
    if (status == BAM_CPL_ERR) return BAM_ETIMEDOUT;   /* the id stays claimed: its completion may still arrive */
    put_cid(&qp->sq, cid);
    if (status != 0) { status_fail(st, BAM_EIO, BAM_AT_NVME_STATUS, status); return BAM_EIO; }
    return BAM_OK;
}

}  // namespace bam
#endif
