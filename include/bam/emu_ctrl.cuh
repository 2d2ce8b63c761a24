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
 * Here that controller is a set of warps: blocks [0, n_ctrl_blocks) of a fused launch
 * (bam/launch.cuh) run emu_controller_main() while the remaining blocks run the workload.
 * The backing store is pinned host memory mapped into the device address space, so every
 * page a command reads crosses the host link exactly once, as it would from an SSD.
 * Several warps may serve one queue: a per-queue lock serialises only the fetch of a small
 * batch of commands (and the hand-out of their completion slots); the data movement of
 * different batches overlaps.
 */
#ifndef BAM_EMU_CTRL_CUH
#define BAM_EMU_CTRL_CUH

#include "sync.cuh"

namespace bam {

#define BAM_SC_SUCCESS 0x00u
#define BAM_SC_INVALID_OPCODE 0x01u
#define BAM_SC_INVALID_FIELD 0x02u
#define BAM_SC_LBA_OUT_OF_RANGE 0x80u

/* Copy `bytes` (a multiple of 16, both pointers 16-byte aligned) with the whole warp.
 * Up to eight 128-bit loads per lane are in flight before the first store. */
BAM_DEV void warp_copy_16(uint8_t* dst, const uint8_t* src, uint32_t bytes, uint32_t lane)
{
    const uint32_t n16 = bytes >> 4;
    for (uint32_t base = 0; base < n16; base += 256) {
        uint4 v[8];
#pragma unroll
        for (int k = 0; k < 8; k++) {
            uint32_t i = base + k * 32 + lane;
            if (i < n16) v[k] = ld_cg_v4(src + ((size_t)i << 4));
        }
#pragma unroll
        for (int k = 0; k < 8; k++) {
            uint32_t i = base + k * 32 + lane;
            if (i < n16) *reinterpret_cast<uint4*>(dst + ((size_t)i << 4)) = v[k];
        }
    }
}

/* Execute one READ or WRITE with the whole warp.  Returns the NVMe status code. */
BAM_DEV uint32_t emu_execute(const bam_emu_d_t& c, uint32_t dw0, uint64_t prp1, uint64_t prp2,
                             uint64_t slba, uint32_t nlb, uint32_t lane)
{
    const uint32_t opc = dw0 & 0x7fu;
    if (opc != NVM_IO_READ && opc != NVM_IO_WRITE) return BAM_SC_INVALID_OPCODE;
    const uint64_t bytes = (uint64_t)(nlb + 1u) << c.lba_log2;
    const uint64_t off = slba << c.lba_log2;
    if (off + bytes > c.store_bytes || off + bytes < off) return BAM_SC_LBA_OUT_OF_RANGE;
    if (prp1 & 15u) return BAM_SC_INVALID_FIELD;
    const uint64_t mps = 1ull << c.mps_log2;
    uint8_t* media = c.store + off;
    /* first chunk: from PRP1 to the end of its memory page */
    uint64_t first = mps - (prp1 & (mps - 1));
    if (first > bytes) first = bytes;
    uint64_t done = 0;
    uint64_t seg_addr = prp1, seg_len = first;
    uint32_t list_i = 0;
    const bool use_list = (bytes - first) > mps;
    while (done < bytes) {
        uint8_t* mem = reinterpret_cast<uint8_t*>(seg_addr);
        uint8_t* med = media + done;
        warp_copy_16(opc == NVM_IO_READ ? mem : med, opc == NVM_IO_READ ? med : mem, (uint32_t)seg_len, lane);
        done += seg_len;
        if (done >= bytes) break;
        if (!use_list) seg_addr = prp2;
        else seg_addr = ld_relaxed_gpu(reinterpret_cast<const uint64_t*>(prp2) + list_i++);
        if (seg_addr & (mps - 1)) return BAM_SC_INVALID_FIELD;
        seg_len = bytes - done < mps ? bytes - done : mps;
    }
    return BAM_SC_SUCCESS;
}

/* Try to fetch and execute one batch from queue pair q.  Returns true if any command ran. */
BAM_DEV bool emu_serve_queue(const bam_emu_d_t& c, uint32_t q, uint32_t lane)
{
    bam_emu_qp_t* s = &c.qps[q];
    const uint32_t mask = s->qs - 1u;
    uint32_t n = 0, fetch = 0, cqbase = 0;
    if (lane == 0) {
        uint32_t tail = ld_acquire_sys(s->sq_db);
        if (tail != (ld_relaxed_gpu(&s->sq_fetch) & mask) && atom_cas_acquire(&s->lock, 0u, 1u) == 0u) {
            fetch = ld_relaxed_gpu(&s->sq_fetch);
            tail = ld_acquire_sys(s->sq_db);
            uint32_t avail = (tail - fetch) & mask;
            uint32_t hdb = ld_acquire_sys(s->cq_db);
            uint32_t cq_head = ld_relaxed_gpu(&s->cq_head);
            cq_head += (hdb - cq_head) & mask;
            st_relaxed_gpu(&s->cq_head, cq_head);
            cqbase = ld_relaxed_gpu(&s->cq_tail);
            uint32_t space = mask - (cqbase - cq_head);      /* keep one completion slot open */
            n = avail < space ? avail : space;
            if (n > c.batch) n = c.batch;
            if (n) st_relaxed_gpu(&s->cq_tail, cqbase + n);
            else st_release_gpu(&s->lock, 0u);
        }
    }
    n = __shfl_sync(0xffffffffu, n, 0);
    if (n == 0) return false;
    fetch = __shfl_sync(0xffffffffu, fetch, 0);
    cqbase = __shfl_sync(0xffffffffu, cqbase, 0);

    /* lane i reads command i of the batch into registers, then the SQ slots are released */
    uint32_t dw0 = 0, nlb = 0;
    uint64_t prp1 = 0, prp2 = 0, slba = 0;
    if (lane < n) {
        const uint8_t* p = reinterpret_cast<const uint8_t*>(&s->sq_mem[(fetch + lane) & mask]);
        uint4 a = ld_cg_v4(p), b = ld_cg_v4(p + 16), d = ld_cg_v4(p + 32), e = ld_cg_v4(p + 48);
        dw0 = a.x;
        prp1 = ((uint64_t)b.w << 32) | b.z;
        prp2 = ((uint64_t)d.y << 32) | d.x;
        slba = ((uint64_t)d.w << 32) | d.z;
        nlb = e.x & 0xffffu;
    }
    __syncwarp();
    if (lane == 0) {
        st_relaxed_gpu(&s->sq_fetch, fetch + n);
        st_release_gpu(&s->lock, 0u);
    }
    const uint32_t sqhd = (fetch + n) & mask;

    /* fault injection is decided per command by lane 0 */
    const uint32_t fault_mode = c.fault ? ld_relaxed_gpu(&c.fault->mode) : BAM_FAULT_NONE;

    for (uint32_t i = 0; i < n; i++) {
        uint32_t c_dw0 = __shfl_sync(0xffffffffu, dw0, i);
        uint32_t c_nlb = __shfl_sync(0xffffffffu, nlb, i);
        uint64_t c_prp1 = __shfl_sync(0xffffffffu, prp1, i);
        uint64_t c_prp2 = __shfl_sync(0xffffffffu, prp2, i);
        uint64_t c_slba = __shfl_sync(0xffffffffu, slba, i);
        uint32_t status = emu_execute(c, c_dw0, c_prp1, c_prp2, c_slba, c_nlb, lane);
        __threadfence();          /* every lane's payload stores are ordered before ...       */
        __syncwarp();             /* ... lane 0's release of the completion entry              */
        if (lane == 0) {
            bool drop = false;
            if (fault_mode != BAM_FAULT_NONE) {
                uint64_t k = atom_add_relaxed(&c.fault->counter, 1ull);
                if (k == c.fault->nth) {
                    if (fault_mode == BAM_FAULT_DROP_CPL) drop = true;
                    else if (fault_mode == BAM_FAULT_STATUS) status = c.fault->status;
                }
            }
            if (!drop) {
                uint32_t v = cqbase + i;
                uint32_t phase = (~(v >> s->qs_log2)) & 1u;
                nvm_cpl_t* e = &s->cq_mem[v & mask];
                *reinterpret_cast<volatile uint64_t*>(&e->dword[0]) = 0ull;
                uint64_t dw2 = sqhd | ((uint32_t)s->sqid << 16);
                uint64_t dw3 = (c_dw0 >> 16) | (phase << 16) | (status << 17);
                st_release_sys(reinterpret_cast<uint64_t*>(&e->dword[2]), dw2 | (dw3 << 32));
            }
            red_add_relaxed(c.served, 1ull);
        }
    }
    return true;
}

/* Body of a controller block.  Runs until every workload block of the launch has finished
 * (consumers_remaining == 0) or an error has been flagged. */
BAM_DEV void emu_controller_main(const bam_emu_d_t& c)
{
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t warps_per_block = blockDim.x >> 5;
    const uint32_t warp = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
    const uint32_t n_warps = c.n_ctrl_blocks * warps_per_block;
    const uint32_t rounds = (c.n_qps + n_warps - 1) / n_warps;
    uint32_t idle_ns = 32;
    const uint64_t t_start = global_timer_ns();
    for (;;) {
        bool any = false;
        uint32_t q = warp % c.n_qps;
        for (uint32_t r = 0; r < rounds; r++) {
            any |= emu_serve_queue(c, q, lane);
            q += n_warps;
            if (q >= c.n_qps) q -= c.n_qps;
            if (q >= c.n_qps) q %= c.n_qps;
        }
        if (any) { idle_ns = 32; continue; }
        uint32_t stop = 0;
        if (lane == 0) {
            stop = (ld_acquire_gpu(c.consumers_remaining) == 0u) || status_bad(c.status);
            if (!stop && global_timer_ns() - t_start > c.status->launch_timeout_ns) {
                status_fail(c.status, BAM_ETIMEDOUT, BAM_AT_LAUNCH, 0);
                stop = 1;
            }
        }
        stop = __shfl_sync(0xffffffffu, stop, 0);
        if (stop) break;
        __nanosleep(idle_ns);
        if (idle_ns < 1024) idle_ns <<= 1;
    }
}

}  // namespace bam
#endif
