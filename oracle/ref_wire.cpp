/*
 * ref_wire.cpp -- TEST INFRASTRUCTURE: a thin extern "C" face on the REFERENCE's own host-compilable
 * wire-format code, compiled from the reference's sources where they lie (recipe: oracle/Makefile,
 * target _ref/libref_wire.so; nothing of the reference is copied into this repository):
 *   include/nvm_cmd.h    nvm_cmd_header / nvm_cmd_data_ptr / nvm_cmd_rw_blks (command encoding),
 *                        nvm_cmd_data / nvm_prp_list / nvm_prp_list_chain (PRP lists)
 *   include/nvm_queue.h  nvm_sq_enqueue / nvm_sq_submit / nvm_cq_poll / nvm_cq_dequeue / nvm_sq_update /
 *                        nvm_cq_update (the classic host-side queue protocol)
 *   src/queue.cpp        nvm_queue_clear / nvm_queue_reset / nvm_cq_dequeue_block
 *   src/error.cpp        nvm_strerror, with include/nvm_error.h's status packing
 *   include/nvm_util.h   NVM_CPL_* / NVM_CMD_* field accessors, page arithmetic macros
 * <simt/atomic> comes from oracle/ref_shim (a stand-in for the reference's un-vendored submodule).
 * Only tests use this library: they let the reference's host code drive the emulated controller and
 * compare its command encoding with the library's.
 */
#include <nvm_types.h>
#include <nvm_cmd.h>
#include <nvm_queue.h>
#include <nvm_error.h>
#include <nvm_util.h>

#include <cstdlib>
#include <cstring>

#define REFW_API extern "C" __attribute__((visibility("default")))

struct refw_queue {
    nvm_ctrl_t ctrl;         /* only what nvm_queue_clear reads: mm_ptr, dstrd, max_qs */
    nvm_queue_t q;
};

/* A queue descriptor of the reference over caller memory; the doorbell address is computed by the
 * reference (SQ_DBL / CQ_DBL, src/regs.h:40-48) from the register window mm_ptr. */
REFW_API void* refw_queue_new(void* mm_ptr, int is_cq, uint16_t no, uint32_t qs, void* vaddr, uint64_t ioaddr)
{
    refw_queue* r = static_cast<refw_queue*>(calloc(1, sizeof(refw_queue)));
    if (!r) return nullptr;
    r->ctrl.page_size = 4096;
    r->ctrl.dstrd = 0;
    r->ctrl.timeout = 5000;
    r->ctrl.max_qs = 1024;
    r->ctrl.mm_size = 0x2000;
    r->ctrl.mm_ptr = mm_ptr;
    if (nvm_queue_clear(&r->q, &r->ctrl, is_cq != 0, no, qs, true, vaddr, ioaddr) != 0) { free(r); return nullptr; }
    return r;
}

REFW_API void refw_queue_free(void* q) { free(q); }

REFW_API uint64_t refw_queue_doorbell_offset(void* q)
{
    refw_queue* r = static_cast<refw_queue*>(q);
    return (uint64_t)((volatile unsigned char*)r->q.db - (volatile unsigned char*)r->ctrl.mm_ptr);
}

/* The 64 bytes the reference's builders produce for one read/write command. */
REFW_API void refw_encode_rw(uint16_t cid, uint8_t opcode, uint32_t ns_id, uint64_t prp1, uint64_t prp2, uint64_t start_lba,
                             uint16_t n_blks, void* out64)
{
    nvm_cmd_t cmd;
    memset(&cmd, 0, sizeof cmd);
    nvm_cmd_header(&cmd, cid, opcode, ns_id);
    nvm_cmd_data_ptr(&cmd, prp1, prp2);
    nvm_cmd_rw_blks(&cmd, start_lba, n_blks);
    memcpy(out64, &cmd, 64);
}

/* Enqueue one read/write command with the reference's nvm_sq_enqueue; -1 when the queue is full. */
REFW_API int refw_sq_put_rw(void* sq, uint16_t cid, uint8_t opcode, uint32_t ns_id, uint64_t prp1, uint64_t prp2, uint64_t start_lba,
                            uint16_t n_blks)
{
    refw_queue* r = static_cast<refw_queue*>(sq);
    nvm_cmd_t* cmd = nvm_sq_enqueue(&r->q);
    if (!cmd) return -1;
    memset(cmd, 0, sizeof *cmd);
    nvm_cmd_header(cmd, cid, opcode, ns_id);
    nvm_cmd_data_ptr(cmd, prp1, prp2);
    nvm_cmd_rw_blks(cmd, start_lba, n_blks);
    return 0;
}

REFW_API void refw_sq_submit(void* sq) { nvm_sq_submit(&static_cast<refw_queue*>(sq)->q); }

/* Take one completion with the reference's nvm_cq_dequeue_block, release the SQ entry and ring the CQ
 * doorbell as its users do (nvm_sq_update, nvm_cq_update).  Returns 0, or -1 on time-out.  The fields
 * come out through the reference's accessors. */
REFW_API int refw_cq_take(void* cq, void* sq, uint64_t timeout_ms, uint16_t* cid, uint16_t* sqhd, uint16_t* sqid, uint8_t* sct,
                          uint8_t* sc, int* packed)
{
    refw_queue* c = static_cast<refw_queue*>(cq);
    refw_queue* s = static_cast<refw_queue*>(sq);
    nvm_cpl_t* cpl = nvm_cq_dequeue_block(&c->q, timeout_ms);
    if (!cpl) return -1;
    *cid = *NVM_CPL_CID(cpl);
    *sqhd = *NVM_CPL_SQHD(cpl);
    *sqid = *NVM_CPL_SQID(cpl);
    *sct = NVM_ERR_SCT(cpl);
    *sc = NVM_ERR_SC(cpl);
    *packed = NVM_ERR_PACK(cpl, 0);
    nvm_sq_update(&s->q);
    nvm_cq_update(&c->q);
    return 0;
}

/* The reference's nvm_cmd_data for a transfer of n_pages pages named by ioaddrs, with n_lists list pages of
 * page_size bytes each at list_mem + l * page_size (bus addresses list_ioaddrs[l]).  dptr4 receives command
 * dwords 6..9; returns the addresses consumed. */
REFW_API uint64_t refw_cmd_data(uint64_t n_lists, void* list_mem, const uint64_t* list_ioaddrs, uint64_t page_size, uint64_t n_pages,
                                const uint64_t* ioaddrs, uint32_t* dptr4)
{
    nvm_prp_list_t lists[16];
    if (n_lists > 16) return 0;
    for (uint64_t l = 0; l < n_lists; l++) {
        lists[l].vaddr = static_cast<unsigned char*>(list_mem) + l * page_size;
        lists[l].local = 1;
        lists[l].page_size = page_size;
        lists[l].ioaddr = list_ioaddrs[l];
    }
    nvm_cmd_t cmd;
    memset(&cmd, 0, sizeof cmd);
    const size_t used = nvm_cmd_data(&cmd, n_lists, n_lists ? lists : NULL, n_pages, ioaddrs);
    memcpy(dptr4, &cmd.dword[6], 16);
    return used;
}

REFW_API const char* refw_strerror(int status) { return nvm_strerror(status); }
REFW_API int refw_unpack_sct(int status) { return NVM_ERR_UNPACK_SCT(status); }
REFW_API int refw_unpack_sc(int status) { return NVM_ERR_UNPACK_SC(status); }
REFW_API uint64_t refw_page_align(uint64_t size, uint64_t page_size) { return NVM_PAGE_ALIGN(size, page_size); }
REFW_API uint64_t refw_page_to_block(uint64_t page_size, uint64_t block_size, uint64_t pageno) { return NVM_PAGE_TO_BLOCK(page_size, block_size, pageno); }
REFW_API uint64_t refw_sq_pages(uint64_t page_size, uint32_t qs) { nvm_ctrl_t c; c.page_size = page_size; return NVM_SQ_PAGES(&c, qs); }
REFW_API uint64_t refw_cq_pages(uint64_t page_size, uint32_t qs) { nvm_ctrl_t c; c.page_size = page_size; return NVM_CQ_PAGES(&c, qs); }
REFW_API uint32_t refw_default_cid(uint32_t tail, int phase, uint32_t qs)
{
    nvm_queue_t q;
    memset(&q, 0, sizeof q);
    q.tail = tail; q.phase = (int8_t)phase; q.qs = qs;
    return NVM_DEFAULT_CID(&q);
}
REFW_API uint32_t refw_opcode(int gen, int fun, int data) { return NVM_CMD_OPCODE(gen, fun, data); }
REFW_API uint32_t refw_sizeof_queue(void) { return (uint32_t)sizeof(nvm_queue_t); }
