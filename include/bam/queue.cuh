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

#include <stddef.h>
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

/* The same read/write command as four 16-byte quarters kept in registers (what the submission paths
 * store into the queue): DW0 = CID | opcode, DW1 = NSID, DW6-9 = PRP1 / PRP2, DW10-11 = SLBA,
 * DW12 = NLB - 1; everything else zero. */
__host__ __device__ __forceinline__ void nvm_cmd_rw_quarters(uint32_t cid, uint8_t opcode, uint32_t ns_id, uint64_t prp1, uint64_t prp2,
                                                             uint64_t start_lba, uint32_t n_blks, uint4& c0, uint4& c1, uint4& c2, uint4& c3)
{
    c0 = make_uint4((cid << 16) | (opcode & 0x7fu), ns_id, 0u, 0u);
    c1 = make_uint4(0u, 0u, (uint32_t)prp1, (uint32_t)(prp1 >> 32));
    c2 = make_uint4((uint32_t)prp2, (uint32_t)(prp2 >> 32), (uint32_t)start_lba, (uint32_t)(start_lba >> 32));
    c3 = make_uint4((n_blks - 1u) & 0xffffu, 0u, 0u, 0u);
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

/* Reserve an SQ slot: draw a ticket and wait for the slot's turn.  Returns the ticket through
 * *ticket_out and the slot position, or BAM_POS_ERR. */
BAM_DEV uint32_t sq_reserve(nvm_queue_t* sq, uint32_t* ticket_out)
{
    const uint32_t ticket = atom_add_relaxed(&sq->in_ticket, 1u);
    const uint32_t pos = ticket & sq->qs_minus_1;
    spin_t sp;
    while (ld_acquire_gpu(&sq->tickets[pos]) != ticket)
        if (sp.expired(sq->status, BAM_AT_SQ_TURN, ticket)) return BAM_POS_ERR;
    *ticket_out = ticket;
    return pos;
}

/* Write the command into the reserved slot, mark it, and publish: whoever holds tail_lock
 * advances the tail over every contiguous marked slot with one doorbell store. */
BAM_DEV uint32_t sq_publish(nvm_queue_t* sq, uint32_t pos, uint32_t ticket, uint4 c0, uint4 c1, uint4 c2, uint4 c3)
{
    bam_status_t* st = sq->status;
    const uint32_t mask = sq->qs_minus_1;
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<nvm_cmd_t*>(const_cast<void*>(sq->vaddr)) + pos);
    dst[0] = c0; dst[1] = c1; dst[2] = c2; dst[3] = c3;
    st_release_gpu(&sq->tail_mark[pos], 1u);

    spin_t sp;
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
                st_release_scoped(const_cast<uint32_t*>(sq->db), (tail + n) & mask, sq->local == 0);
                st_release_gpu(&sq->tail, tail + n);
                BAM_PROF_ADD(st, 8, 1); BAM_PROF_ADD(st, 9, n);
            }
            st_release_gpu(&sq->tail_lock, 0u);
            if (n) continue;
        }
        if (sp.expired(st, BAM_AT_SQ_DOORBELL, ticket)) return BAM_POS_ERR;
    }
    return pos;
}

/* Submit one command given as four 16-byte quarters (kept in registers).  Returns the SQ slot it
 * was written to, or BAM_POS_ERR. */
BAM_DEV uint32_t sq_enqueue_regs(nvm_queue_t* sq, uint4 c0, uint4 c1, uint4 c2, uint4 c3)
{
    uint32_t ticket;
    const uint32_t pos = sq_reserve(sq, &ticket);
    if (pos == BAM_POS_ERR) return BAM_POS_ERR;
    return sq_publish(sq, pos, ticket, c0, c1, c2, c3);
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
        fence_acq_rel_scoped(cq->local == 0);              /* acquire the k payloads */
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
        st_release_scoped(const_cast<uint32_t*>(cq->db), (h + total) & mask, cq->local == 0);
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
            BAM_PROF_T0();
            uint32_t n = cq_reap(qp);
            st_release_gpu(&cq->head_lock, 0u);
            BAM_PROF_ADD(sq->status, 5, 1); BAM_PROF_LAP(sq->status, 6); BAM_PROF_ADD(sq->status, 7, n);
            if (n) continue;
        }
        if (sp.expired(sq->status, BAM_AT_CQ_WAIT, cid)) return BAM_CPL_ERR;
    }
}

/* The reference's parameter lists (include/nvm_parallel_queue.h:333, :379, :425), so that its call sequence
 *     sq_pos = sq_enqueue(&qp->sq, &cmd); cq_pos = cq_poll(&qp->cq, cid); sq_dequeue(&qp->sq, sq_pos);
 *     cq_dequeue(&qp->cq, cq_pos); put_cid(&qp->sq, cid);        (benchmarks/block/main.cu:86-93)
 * compiles and works unchanged.  cq_poll finds the queue pair that embeds `cq`; what it returns is the NVMe
 * status of the command (0 = success), not a queue position: the reaper inside it has already consumed the
 * entry, re-opened the submission slot, advanced the head and rung the doorbell, so sq_dequeue and
 * cq_dequeue have nothing left to do and ignore their position argument. */
BAM_DEV uint32_t cq_poll(nvm_queue_t* cq, uint16_t search_cid, uint32_t* loc_ = nullptr, uint32_t* cq_head = nullptr)
{
    QueuePair* qp = reinterpret_cast<QueuePair*>(reinterpret_cast<char*>(cq) - offsetof(QueuePair, cq));
    const uint32_t status = cq_poll(qp, (uint32_t)search_cid);
    if (loc_) *loc_ = 0;
    if (cq_head) *cq_head = ld_relaxed_gpu(&cq->head);
    return status;
}
BAM_DEV void sq_dequeue(nvm_queue_t*, uint16_t) {}
BAM_DEV void cq_dequeue(nvm_queue_t*, uint16_t, nvm_queue_t* = nullptr, uint32_t = 0, uint32_t = 0) {}

/* ================================================================================================
 * Warp-cooperative I/O.
 *
 * The single-thread functions above are correct from any divergent context, but 32 lanes that
 * each spin and sleep on their own serialise one another (a warp runs one divergent path at a
 * time, and every path sleeps).  The functions below are called by all lanes of `mask` together
 * and keep every wait CONVERGED: each lane tests its own condition, the warp votes, and it backs
 * off once for all lanes.  They also aggregate: one fetch-add reserves the tickets of the whole
 * group, and the holder of tail_lock / head_lock sweeps the SQ marks and reaps the CQ with all
 * lanes at once (32 entries per round trip instead of one).
 * ============================================================================================== */

/* number of lanes of `mask` below this lane */
BAM_DEV uint32_t rank_in(uint32_t mask) { return __popc(mask & ((1u << lane_id()) - 1u)); }

/* how many lanes, in rank order from the first lane of `mask`, have their bit set in `votes` */
BAM_DEV uint32_t leading_votes(uint32_t mask, uint32_t votes)
{
    const uint32_t miss = mask & ~votes;
    if (miss == 0u) return __popc(mask);
    return __popc(mask & ((1u << (__ffs(miss) - 1)) - 1u));
}

/* Publish every contiguous marked SQ slot (caller's leader holds tail_lock; all lanes of mask help). */
BAM_DEV void sq_sweep_warp(uint32_t mask, uint32_t leader, nvm_queue_t* sq)
{
    const uint32_t qmask = sq->qs_minus_1;
    const uint32_t nl = __popc(mask), rank = rank_in(mask);
    uint32_t tail = 0, head = 0;
    if (lane_id() == leader) { tail = ld_relaxed_gpu(&sq->tail); head = ld_acquire_gpu(&sq->head); }
    tail = __shfl_sync(mask, tail, leader);
    head = __shfl_sync(mask, head, leader);
    uint32_t total = 0;
    for (;;) {
        const uint32_t idx = tail + total + rank;
        /* a queue of qs entries holds at most qs-1 (tail == head means empty) */
        const bool ok = (idx - head) < qmask && ld_acquire_gpu(&sq->tail_mark[idx & qmask]) == 1u;
        const uint32_t k = leading_votes(mask, __ballot_sync(mask, ok));
        if (rank < k) st_relaxed_gpu(&sq->tail_mark[idx & qmask], 0u);
        total += k;
        if (k < nl) break;
    }
    __syncwarp(mask);
    if (total && lane_id() == leader) {
        st_release_scoped(const_cast<uint32_t*>(sq->db), (tail + total) & qmask, sq->local == 0);
        st_release_gpu(&sq->tail, tail + total);
        BAM_PROF_ADD(sq->status, 8, 1); BAM_PROF_ADD(sq->status, 9, total);
    }
}

/* Reap the completion queue with all lanes of mask (leader holds cq->head_lock).  Returns the
 * number of entries consumed (same value in every lane). */
BAM_DEV uint32_t cq_reap_warp(uint32_t mask, uint32_t leader, QueuePair* qp)
{
    nvm_queue_t* sq = &qp->sq;
    nvm_queue_t* cq = &qp->cq;
    const uint32_t qmask = cq->qs_minus_1, lg = cq->qs_log2;
    const uint32_t nl = __popc(mask), rank = rank_in(mask);
    nvm_cpl_t* mem = reinterpret_cast<nvm_cpl_t*>(const_cast<void*>(cq->vaddr));
    uint32_t h = 0;
    if (lane_id() == leader) h = ld_relaxed_gpu(&cq->head);
    h = __shfl_sync(mask, h, leader);
    uint32_t total = 0, sqhd = 0;
    for (;;) {
        const uint32_t idx = h + total + rank;
        const uint64_t e = ld_relaxed_sys(reinterpret_cast<const uint64_t*>(&mem[idx & qmask].dword[2]));
        const bool ok = ((uint32_t)(e >> 48) & 1u) == ((~(idx >> lg)) & 1u);
        uint32_t k = leading_votes(mask, __ballot_sync(mask, ok));
        if (total + k > qmask) k = qmask - total;               /* never more than qs-1 per pass */
        if (k == 0) break;
        if (rank < k) {
            fence_acq_rel_scoped(cq->local == 0);                /* acquire the payload           */
            const uint32_t dw3 = (uint32_t)(e >> 32);
            st_release_gpu(&sq->cid[dw3 & 0xffffu], BAM_CID_DONE | (dw3 >> 17));
        }
        /* SQ head reported by the newest consumed entry (the lane of rank k-1 holds it) */
        sqhd = __shfl_sync(mask, (uint32_t)e & 0xffffu, __ffs(__ballot_sync(mask, rank == k - 1u)) - 1);
        total += k;
        if (k < nl || total >= qmask) break;
    }
    if (total) {
        /* re-open the SQ slots the controller has fetched */
        uint32_t cur = 0;
        if (lane_id() == leader) cur = ld_relaxed_gpu(&sq->head);
        cur = __shfl_sync(mask, cur, leader);
        const uint32_t delta = (sqhd - cur) & sq->qs_minus_1;
        for (uint32_t i = rank; i < delta; i += nl)
            st_release_gpu(&sq->tickets[(cur + i) & sq->qs_minus_1], cur + i + sq->qs);
        __syncwarp(mask);
        if (lane_id() == leader) {
            if (delta) st_release_gpu(&sq->head, cur + delta);
            st_release_gpu(&cq->head, h + total);
            st_release_scoped(const_cast<uint32_t*>(cq->db), (h + total) & qmask, cq->local == 0);
        }
    }
    return total;
}

/* Submit half of a group: the lanes of `g` (a subset of mask, all on queue pair qp) write one
 * command each and get it published.  Every lane of mask takes part in the votes and helps
 * sweeping.  Returns the command id of the lane's command (BAM_CID_ERR for lanes outside g, or when
 * a wait ran out). */
BAM_DEV uint32_t warp_submit_group(uint32_t mask, uint32_t g, QueuePair* qp, uint64_t starting_lba, uint32_t n_blocks,
                                   uint64_t bus_addr, uint64_t bus_addr2, uint8_t opcode)
{
    nvm_queue_t* sq = &qp->sq;
    bam_status_t* st = sq->status;
    const uint32_t lane = lane_id();
    const bool mine = (g >> lane) & 1u;
    const uint32_t gl = __ffs(g) - 1;
    const uint32_t qmask = sq->qs_minus_1;
    spin_t sp;
#ifdef BAM_PROFILE
    long long pt = clock64();
#endif
    /* one fetch-add reserves the tickets of the whole group */
    uint32_t base = 0;
    if (lane == gl) base = atom_add_relaxed(&sq->in_ticket, (uint32_t)__popc(g));
    base = __shfl_sync(mask, base, gl);
    const uint32_t ticket = base + __popc(g & ((1u << lane) - 1u));
    const uint32_t pos = ticket & qmask;
    for (;;) {
        const bool ok = !mine || ld_acquire_gpu(&sq->tickets[pos]) == ticket;
        if (__all_sync(mask, ok)) break;
        if (__any_sync(mask, sp.expired(st, BAM_AT_SQ_TURN, ticket))) return BAM_CID_ERR;
    }
#ifdef BAM_PROFILE
    { long long n = clock64(); if (mine) { BAM_PROF_ADD(st, 0, 1); BAM_PROF_ADD(st, 1, n - pt); } pt = n; }
#endif
    /* command ids: held only from here to the completion.  One fetch-add moves the rotating
     * start point for the whole group; a lane whose word is taken steps on by the group size. */
    uint32_t cid = BAM_CID_ERR;
    {
        uint32_t cbase = 0;
        if (lane == gl) cbase = atom_add_relaxed(&sq->cid_ticket, (uint32_t)__popc(g));
        cbase = __shfl_sync(mask, cbase, gl);
        uint32_t probe = cbase + __popc(g & ((1u << lane) - 1u));
        sp.reset();
        for (;;) {
            if (mine && cid == BAM_CID_ERR) {
                const uint32_t id = probe & (BAM_CID_SPACE - 1u);
                if (atom_cas_acquire(&sq->cid[id], 0u, BAM_CID_INFLIGHT) == 0u) cid = id;
                else probe += 32u;
            }
            if (__all_sync(mask, !mine || cid != BAM_CID_ERR)) break;
            if (__any_sync(mask, sp.expired(st, BAM_AT_CID))) return BAM_CID_ERR;
        }
    }
#ifdef BAM_PROFILE
    { long long n = clock64(); if (mine) BAM_PROF_ADD(st, 2, n - pt); pt = n; }
#endif
    if (mine) {
        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<nvm_cmd_t*>(const_cast<void*>(sq->vaddr)) + pos);
        uint4 c0, c1, c2, c3;
        nvm_cmd_rw_quarters(cid, opcode, qp->nvmNamespace, bus_addr, bus_addr2, starting_lba, n_blocks, c0, c1, c2, c3);
        dst[0] = c0; dst[1] = c1; dst[2] = c2; dst[3] = c3;
        st_release_gpu(&sq->tail_mark[pos], 1u);
    }
    /* publish: whoever gets tail_lock sweeps with the whole warp */
    sp.reset();
    for (;;) {
        uint32_t locked = 0;
        if (lane == gl) locked = (ld_relaxed_gpu(&sq->tail_lock) == 0u && atom_cas_acquire(&sq->tail_lock, 0u, 1u) == 0u);
        locked = __shfl_sync(mask, locked, gl);
        if (locked) {
            sq_sweep_warp(mask, gl, sq);
            if (lane == gl) st_release_gpu(&sq->tail_lock, 0u);
        }
        const bool cleared = !mine || ld_relaxed_gpu(&sq->tail_mark[pos]) == 0u;
        if (__all_sync(mask, cleared)) break;
        if (__any_sync(mask, sp.expired(st, BAM_AT_SQ_DOORBELL, ticket))) return BAM_CID_ERR;
    }
#ifdef BAM_PROFILE
    { long long n = clock64(); if (mine) BAM_PROF_ADD(st, 3, n - pt); pt = n; }
#endif
    return mine ? cid : BAM_CID_ERR;
}

/* Wait half: the lanes of `g` wait for the completions of their commands `cid`; whoever gets
 * head_lock reaps with the whole warp.  Returns BAM_OK / BAM_E* (per lane; BAM_OK if not in g). */
BAM_DEV int warp_wait_group(uint32_t mask, uint32_t g, QueuePair* qp, uint32_t cid)
{
    nvm_queue_t* sq = &qp->sq;
    nvm_queue_t* cq = &qp->cq;
    bam_status_t* st = sq->status;
    const uint32_t lane = lane_id();
    const bool mine = ((g >> lane) & 1u) && cid != BAM_CID_ERR;
    const uint32_t gl = __ffs(g) - 1;
#ifdef BAM_PROFILE
    long long pt = clock64();
#endif
    uint32_t status = BAM_CPL_ERR;
    spin_t sp;
    for (;;) {
        if (mine && status == BAM_CPL_ERR) {
            const uint32_t v = ld_acquire_gpu(&sq->cid[cid]);
            if (v & BAM_CID_DONE) status = v & 0x7fffu;
        }
        if (__all_sync(mask, !mine || status != BAM_CPL_ERR)) break;
        /* take the reaper lock only if the entry at the head carries the phase of a new completion */
        uint32_t locked = 0;
        if (lane == gl && ld_relaxed_gpu(&cq->head_lock) == 0u) {
            const uint32_t h = ld_relaxed_gpu(&cq->head);
            const uint64_t e = ld_relaxed_sys(reinterpret_cast<const uint64_t*>(
                &reinterpret_cast<nvm_cpl_t*>(const_cast<void*>(cq->vaddr))[h & cq->qs_minus_1].dword[2]));
            if ((((uint32_t)(e >> 48)) & 1u) == ((~(h >> cq->qs_log2)) & 1u))
                locked = atom_cas_acquire(&cq->head_lock, 0u, 1u) == 0u;
        }
        locked = __shfl_sync(mask, locked, gl);
        if (locked) {
            BAM_PROF_T0();
            const uint32_t n = cq_reap_warp(mask, gl, qp);
            if (lane == gl) {
                st_release_gpu(&cq->head_lock, 0u);
                BAM_PROF_ADD(st, 5, 1); BAM_PROF_LAP(st, 6); BAM_PROF_ADD(st, 7, n);
            }
            if (n) continue;
        }
        if (__any_sync(mask, sp.expired(st, BAM_AT_CQ_WAIT, cid))) break;
    }
#ifdef BAM_PROFILE
    { long long n = clock64(); if (mine) BAM_PROF_ADD(st, 4, n - pt); pt = n; }
#endif
    if (!mine) return ((g >> lane) & 1u) ? BAM_ETIMEDOUT : BAM_OK;      /* a lane of g without an id never submitted */
    if (status == BAM_CPL_ERR) return BAM_ETIMEDOUT;       /* the id stays claimed: its completion may still arrive */
    put_cid(sq, cid);
    if (status != 0u) { status_fail(st, BAM_EIO, BAM_AT_NVME_STATUS, status); return BAM_EIO; }
    return BAM_OK;
}

/* One group, blocking: submit, then wait. */
BAM_DEV int warp_io_group(uint32_t mask, uint32_t g, QueuePair* qp, uint64_t starting_lba, uint32_t n_blocks,
                          uint64_t bus_addr, uint64_t bus_addr2, uint8_t opcode)
{
    const uint32_t cid = warp_submit_group(mask, g, qp, starting_lba, n_blocks, bus_addr, bus_addr2, opcode);
    return warp_wait_group(mask, g, qp, cid);
}

/* Asynchronous pair for callers that keep several requests per thread in flight (the reference's
 * access_data_async / poll_async, page_cache.h:1930-1959): every lane of `mask` calls them
 * together, all on the same queue pair.  Submit as many rounds as wanted, then wait for each round
 * with the ids it returned.  The commands a warp has outstanding must stay below half the queue
 * depth (32 x rounds < qs / 2), or a later round would wait for slots its own commands occupy. */
BAM_DEV uint32_t warp_io_submit(uint32_t mask, bool active, QueuePair* qp, uint64_t starting_lba, uint32_t n_blocks,
                                uint64_t bus_addr, uint64_t bus_addr2, uint8_t opcode)
{
    const uint32_t g = __ballot_sync(mask, active);
    if (g == 0u || __any_sync(mask, status_bad(qp->sq.status))) return BAM_CID_ERR;
    return warp_submit_group(mask, g, qp, starting_lba, n_blocks, bus_addr, bus_addr2, opcode);
}

BAM_DEV int warp_io_wait(uint32_t mask, bool active, QueuePair* qp, uint32_t cid)
{
    const uint32_t g = __ballot_sync(mask, active);
    if (g == 0u) return BAM_OK;
    return warp_wait_group(mask, g, qp, cid);
}

/* Blocking I/O for a warp: every lane of `mask` calls this together; lanes with active == true
 * run one command each.  Lanes are grouped by queue pair and chunked to half the queue depth (a
 * group must never need a slot that one of its own commands still occupies). */
BAM_DEV int warp_io(uint32_t mask, bool active, QueuePair* qp, uint64_t starting_lba, uint32_t n_blocks,
                    uint64_t bus_addr, uint64_t bus_addr2, uint8_t opcode)
{
    const uint32_t lane = lane_id();
    int rc = BAM_OK;
    uint32_t todo = __ballot_sync(mask, active);
    while (todo) {
        const uint32_t first = __ffs(todo) - 1;
        QueuePair* gqp = reinterpret_cast<QueuePair*>(__shfl_sync(mask, reinterpret_cast<uint64_t>(qp), first));
        bool mine = ((todo >> lane) & 1u) && qp == gqp;
        uint32_t g = __ballot_sync(mask, mine);
        uint32_t cap = gqp->sq.qs >> 1;
        if (cap == 0) cap = 1;
        if ((uint32_t)__popc(g) > cap) {
            mine = mine && (uint32_t)__popc(g & ((1u << lane) - 1u)) < cap;
            g = __ballot_sync(mask, mine);
        }
        if (__any_sync(mask, status_bad(gqp->sq.status))) { if (mine) rc = BAM_EIO; }
        else {
            const int r = warp_io_group(mask, g, gqp, starting_lba, n_blocks, bus_addr, bus_addr2, opcode);
            if (mine) rc = r;
        }
        todo &= ~g;
    }
    return rc;
}

/* Submit half of one thread's I/O: build the command, claim a slot and an id, publish.  On
 * success *cid_out names the command for access_data_complete. */
BAM_DEV int access_data_submit(QueuePair* qp, uint64_t starting_lba, uint32_t n_blocks, uint64_t bus_addr, uint64_t bus_addr2,
                               uint8_t opcode, uint32_t* cid_out, uint32_t* pos_out)
{
    bam_status_t* st = qp->sq.status;
    if (status_bad(st)) return BAM_EIO;
    /* slot first, command id second: ids are then held only by commands that are in the queue
     * or at the controller (a few thousand), never by the threads still waiting for a slot */
    uint32_t ticket;
#ifdef BAM_PROFILE
    long long pt = clock64();
#endif
    const uint32_t pos = sq_reserve(&qp->sq, &ticket);
    if (pos == BAM_POS_ERR) return BAM_ETIMEDOUT;
#ifdef BAM_PROFILE
    { long long n = clock64(); BAM_PROF_ADD(st, 0, 1); BAM_PROF_ADD(st, 1, n - pt); pt = n; }
#endif
    const uint32_t cid = get_cid(&qp->sq);
    if (cid == BAM_CID_ERR) return BAM_ETIMEDOUT;
#ifdef BAM_PROFILE
    { long long n = clock64(); BAM_PROF_ADD(st, 2, n - pt); pt = n; }
#endif
    /* DW0 = CID | opcode, DW1 = NSID, DW6-9 = PRP1/PRP2, DW10-11 = SLBA, DW12 = NLB-1
     * (the fields nvm_cmd_header / nvm_cmd_data_ptr / nvm_cmd_rw_blks set), built in registers */
    uint4 c0, c1, c2, c3;
    nvm_cmd_rw_quarters(cid, opcode, qp->nvmNamespace, bus_addr, bus_addr2, starting_lba, n_blocks, c0, c1, c2, c3);
    if (sq_publish(&qp->sq, pos, ticket, c0, c1, c2, c3) == BAM_POS_ERR) return BAM_ETIMEDOUT;
#ifdef BAM_PROFILE
    { long long n = clock64(); BAM_PROF_ADD(st, 3, n - pt); pt = n; }
#endif
    *cid_out = cid;
    if (pos_out) *pos_out = pos;
    return BAM_OK;
}

/* Wait half: wait for the completion of command `cid`, retire its id. */
BAM_DEV int access_data_complete(QueuePair* qp, uint32_t cid)
{
    bam_status_t* st = qp->sq.status;
    BAM_PROF_T0();
    const uint32_t status = cq_poll(qp, cid);
    BAM_PROF_LAP(st, 4);
    if (status == BAM_CPL_ERR) return BAM_ETIMEDOUT;   /* the id stays claimed: its completion may still arrive */
    put_cid(&qp->sq, cid);
    if (status != 0) { status_fail(st, BAM_EIO, BAM_AT_NVME_STATUS, status); return BAM_EIO; }
    return BAM_OK;
}

/* One blocking I/O: build the command, submit, wait, retire.  Counterpart of read_data /
 * write_data / access_data (page_cache.h:2009-2132 in the reference). */
BAM_DEV int access_data_raw(QueuePair* qp, uint64_t starting_lba, uint32_t n_blocks,
                            uint64_t bus_addr, uint64_t bus_addr2, uint8_t opcode)
{
    uint32_t cid = 0;
    const int rc = access_data_submit(qp, starting_lba, n_blocks, bus_addr, bus_addr2, opcode, &cid, nullptr);
    if (rc != BAM_OK) return rc;
    return access_data_complete(qp, cid);
}

}  // namespace bam
#endif
