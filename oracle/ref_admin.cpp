/*
 * ref_admin.cpp -- TEST INFRASTRUCTURE: the REFERENCE's own admin layer (src/admin.cpp: nvm_admin_ctrl_info,
 * nvm_admin_ns_info, nvm_admin_*_num_queues, nvm_admin_cq_create / sq_create / cq_delete / sq_delete, with its
 * src/queue.cpp and src/error.cpp), compiled from the reference's sources where they lie (recipe:
 * oracle/Makefile, target _ref/libref_admin.so; nothing of the reference is copied into this repository).
 * The two functions that layer calls downwards -- nvm_raw_rpc, which submits an admin command, and
 * nvm_ctrl_from_aq_ref -- are forwarded to function pointers a test binds to the library under test, so the
 * reference's code builds its admin commands, parses the identify pages and fills its own queue descriptors
 * while the emulated controller executes the commands.  Only tests use this library.
 */
#include <nvm_types.h>
#include <nvm_admin.h>
#include <nvm_rpc.h>
#include <nvm_util.h>
#include <nvm_queue.h>
#include <nvm_cmd.h>
#include <nvm_error.h>

#include <cerrno>
#include <cstdlib>
#include <cstring>

#define REFA_API extern "C" __attribute__((visibility("default")))

static int (*g_rpc)(void*, void*, void*) = nullptr;
static const void* (*g_ctrl_of)(void*) = nullptr;

/* what src/admin.cpp calls (declared in the reference's nvm_rpc.h and nvm_util.h) */
int nvm_raw_rpc(nvm_aq_ref ref, nvm_cmd_t* cmd, nvm_cpl_t* cpl) { return g_rpc ? g_rpc(ref, cmd, cpl) : ENOSYS; }
extern "C" const nvm_ctrl_t* nvm_ctrl_from_aq_ref(nvm_aq_ref ref) { return g_ctrl_of ? static_cast<const nvm_ctrl_t*>(g_ctrl_of(ref)) : nullptr; }

REFA_API void refa_bind(void* raw_rpc, void* ctrl_from_aq_ref)
{
    g_rpc = reinterpret_cast<int (*)(void*, void*, void*)>(raw_rpc);
    g_ctrl_of = reinterpret_cast<const void* (*)(void*)>(ctrl_from_aq_ref);
}

REFA_API int refa_ctrl_info(void* aq, struct nvm_ctrl_info* info, void* buffer, uint64_t ioaddr)
{
    return nvm_admin_ctrl_info(static_cast<nvm_aq_ref>(aq), info, buffer, ioaddr);
}
REFA_API int refa_ns_info(void* aq, struct nvm_ns_info* info, uint32_t ns_id, void* buffer, uint64_t ioaddr)
{
    return nvm_admin_ns_info(static_cast<nvm_aq_ref>(aq), info, ns_id, buffer, ioaddr);
}
REFA_API int refa_request_num_queues(void* aq, uint16_t* n_cqs, uint16_t* n_sqs)
{
    return nvm_admin_request_num_queues(static_cast<nvm_aq_ref>(aq), n_cqs, n_sqs);
}
REFA_API int refa_get_num_queues(void* aq, uint16_t* n_cqs, uint16_t* n_sqs)
{
    return nvm_admin_get_num_queues(static_cast<nvm_aq_ref>(aq), n_cqs, n_sqs);
}

/* queue descriptors of the reference's layout, owned by this library */
REFA_API void* refa_queue_alloc(void) { return calloc(1, sizeof(nvm_queue_t)); }
REFA_API void refa_queue_free(void* q) { free(q); }
REFA_API uint32_t refa_queue_qs(void* q) { return static_cast<nvm_queue_t*>(q)->qs; }
REFA_API uint64_t refa_queue_doorbell_offset(void* q, void* mm_ptr)
{
    return (uint64_t)((volatile unsigned char*)static_cast<nvm_queue_t*>(q)->db - (volatile unsigned char*)mm_ptr);
}

REFA_API int refa_cq_create(void* aq, void* cq, uint16_t id, const void* dma, uint64_t offset, uint64_t qs)
{
    return nvm_admin_cq_create(static_cast<nvm_aq_ref>(aq), static_cast<nvm_queue_t*>(cq), id, static_cast<const nvm_dma_t*>(dma), offset, qs);
}
REFA_API int refa_sq_create(void* aq, void* sq, const void* cq, uint16_t id, const void* dma, uint64_t offset, uint64_t qs)
{
    return nvm_admin_sq_create(static_cast<nvm_aq_ref>(aq), static_cast<nvm_queue_t*>(sq), static_cast<const nvm_queue_t*>(cq), id,
                               static_cast<const nvm_dma_t*>(dma), offset, qs);
}
REFA_API int refa_cq_delete(void* aq, void* cq) { return nvm_admin_cq_delete(static_cast<nvm_aq_ref>(aq), static_cast<nvm_queue_t*>(cq)); }
REFA_API int refa_sq_delete(void* aq, void* sq, const void* cq)
{
    return nvm_admin_sq_delete(static_cast<nvm_aq_ref>(aq), static_cast<nvm_queue_t*>(sq), static_cast<const nvm_queue_t*>(cq));
}

/* one read/write command through the reference's classic queue functions on descriptors made above */
REFA_API int refa_rw(void* sq, void* cq, uint8_t opcode, uint32_t ns_id, uint64_t prp1, uint64_t start_lba, uint16_t n_blks, uint64_t timeout_ms)
{
    nvm_queue_t* s = static_cast<nvm_queue_t*>(sq);
    nvm_queue_t* c = static_cast<nvm_queue_t*>(cq);
    nvm_cmd_t* cmd = nvm_sq_enqueue(s);
    if (!cmd) return EAGAIN;
    memset(cmd, 0, sizeof *cmd);
    nvm_cmd_header(cmd, NVM_DEFAULT_CID(s), opcode, ns_id);
    nvm_cmd_data_ptr(cmd, prp1, 0);
    nvm_cmd_rw_blks(cmd, start_lba, n_blks);
    nvm_sq_submit(s);
    nvm_cpl_t* cpl = nvm_cq_dequeue_block(c, timeout_ms);
    if (!cpl) return ETIMEDOUT;
    const int st = NVM_ERR_PACK(cpl, 0);
    nvm_sq_update(s);
    nvm_cq_update(c);
    return st;
}
