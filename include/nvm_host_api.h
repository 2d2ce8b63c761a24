/*
 * nvm_host_api.h -- the host-side libnvm interface of the reference, served by the emulated
 * controller (reference: include/nvm_types.h:19-66,180-232, nvm_ctrl.h:36-76, nvm_dma.h:35-147,
 * nvm_aq.h:23-38, nvm_admin.h:18-117, nvm_queue.h:30-286, nvm_rpc.h:33-53).
 *
 * What the names mean here.  There is no kernel module and no PCI device: a controller handle
 * (nvm_ctrl_t) is made from an emulated controller (nvm_emu_ctrl_init), its "register window"
 * (mm_ptr) is a page of pinned host memory with the doorbell registers at their NVMe offsets, a DMA
 * mapping pins memory and reports device-visible addresses as bus addresses (ioaddr == the address
 * the GPU uses), and admin commands are executed on the host by nvm_raw_rpc, the way the controller
 * would execute them from its admin queue (there is no admin queue memory to poll).  I/O queue pairs created with nvm_admin_cq_create / nvm_admin_sq_create
 * live in caller memory (a DMA mapping of host memory) and are driven from the HOST with the
 * classic single-threaded queue functions below; their commands are executed by the controller's
 * command processor running as a service kernel on the GPU (started by nvm_admin_sq_create,
 * stopped by nvm_emu_service_stop / nvm_ctrl_free).  While the service kernel runs, fused launches
 * (bam_launch_*) on the same GPU must wait, and CUDA calls that wait for the whole device to go idle
 * (cudaDeviceSynchronize, cudaFree) do not return before it stops: stop the service first.  The DMA
 * functions below pause and resume it themselves.  The service kernel leaves on its own after the
 * controller's launch time limit (bam_ctrl_set_launch_timeout, 300 s by default).
 *
 * Errors: 0 = success, positive errno values, as in the reference (nvm_error.h).
 */
#ifndef BAM_NVM_HOST_API_H
#define BAM_NVM_HOST_API_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#include "bam_abi.h"
#include "bam/abi_types.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---- controller handle: nvm_ctrl_t is defined in bam/abi_types.h (nvm_types.h:19-28 there) ------ */
/* The reference opens /dev/libnvm* (a kernel module bound to a raw SSD); not available: ENODEV. */
int nvm_ctrl_init(nvm_ctrl_t** ctrl, int fd);
/* A handle from a memory-mapped register window (nvm_ctrl.h:53 there).  The windows that exist here are
 * those of emulated controllers (mm_ptr of a handle made by nvm_emu_ctrl_init): such a window gives
 * another handle to the same controller, counted by nvm_ctrl_free; anything else is ENODEV.  The window
 * holds CAP, VS, CC, CSTS, AQA, ASQ and ACQ at their NVMe offsets, consistent with the handle's fields. */
#define NVM_CTRL_MEM_MINSIZE 0x2000
int nvm_raw_ctrl_init(nvm_ctrl_t** ctrl, volatile void* mm_ptr, size_t mm_size);
/* Reset the controller (nvm_ctrl.h:76 there): all I/O queue pairs are gone afterwards, doorbells read 0
 * and ASQ / ACQ hold the given page-aligned addresses (EINVAL otherwise). */
int nvm_raw_ctrl_reset(const nvm_ctrl_t* ctrl, uint64_t acq_ioaddr, uint64_t asq_ioaddr);
/* A handle over an emulated controller made by bam_ctrl_create (which stays owned by the caller). */
int nvm_emu_ctrl_init(nvm_ctrl_t** ctrl, bam_ctrl_t emu);
void nvm_ctrl_free(nvm_ctrl_t* ctrl);
/* Start / stop the command processor that serves the host-driven queue pairs (see above). */
int nvm_emu_service_start(const nvm_ctrl_t* ctrl);
int nvm_emu_service_stop(const nvm_ctrl_t* ctrl);
/* Whether the service kernel is (believed to be) running, the error state it recorded (BAM_E* code and
 * BAM_AT_* place, 0 = none) and the number of commands it has completed.  Returns 0, or 1000 + the CUDA
 * error when the kernel or the query failed. */
int nvm_emu_service_status(const nvm_ctrl_t* ctrl, uint32_t* running, uint32_t* code, uint32_t* where, uint64_t* served);

/* ---- DMA mappings (nvm_types.h:52-66, nvm_dma.h) ------------------------------------------------ */
typedef struct {
    void* vaddr;               /* virtual address of the region (may be NULL)           */
    int8_t local;              /* host memory of this machine                           */
    int8_t contiguous;
    size_t page_size;          /* controller page size                                  */
    size_t n_ioaddrs;          /* number of controller pages                            */
    uint64_t ioaddrs[];        /* bus address of every page                             */
} nvm_dma_t;

int nvm_dma_map(nvm_dma_t** map, const nvm_ctrl_t* ctrl, void* vaddr, size_t page_size, size_t n_pages, const uint64_t* ioaddrs);
int nvm_dma_map_host(nvm_dma_t** map, const nvm_ctrl_t* ctrl, void* vaddr, size_t size);      /* pins the memory */
int nvm_dma_map_device(nvm_dma_t** map, const nvm_ctrl_t* ctrl, void* devptr, size_t size);   /* cudaMalloc'd memory */
int nvm_dma_create(nvm_dma_t** map, const nvm_ctrl_t* ctrl, size_t size);                     /* allocates pinned memory */
/* Another descriptor of the memory of other_map (nvm_dma.h:48 there); pinned or allocated memory is
 * released when the last descriptor is unmapped. */
int nvm_dma_remap(nvm_dma_t** new_map, const nvm_dma_t* other_map);
void nvm_dma_unmap(nvm_dma_t* map);
/* The controller a mapping / an admin reference belongs to (nvm_util.h:234-250 there). */
const nvm_ctrl_t* nvm_ctrl_from_dma(const nvm_dma_t* dma);

/* ---- admin queue reference and identify data (nvm_aq.h, nvm_admin.h, nvm_types.h:198-232) ------- */
/* struct nvm_ctrl_info and struct nvm_ns_info are defined in bam/abi_types.h */

/* dma: memory for the admin queues (unused by the emulator, accepted for source compatibility) */
int nvm_aq_create(nvm_aq_ref* ref, const nvm_ctrl_t* ctrl, const nvm_dma_t* dma);
void nvm_aq_destroy(nvm_aq_ref ref);
const nvm_ctrl_t* nvm_ctrl_from_aq_ref(nvm_aq_ref ref);
void nvm_rpc_unbind(nvm_aq_ref ref);                     /* references are always local here: does nothing */
int nvm_admin_ctrl_info(nvm_aq_ref ref, struct nvm_ctrl_info* info, void* buffer, uint64_t ioaddr);
int nvm_admin_ns_info(nvm_aq_ref ref, struct nvm_ns_info* info, uint32_t ns_id, void* buffer, uint64_t ioaddr);
int nvm_admin_set_num_queues(nvm_aq_ref ref, uint16_t n_cqs, uint16_t n_sqs);
int nvm_admin_get_num_queues(nvm_aq_ref ref, uint16_t* n_cqs, uint16_t* n_sqs);
int nvm_admin_request_num_queues(nvm_aq_ref ref, uint16_t* n_cqs, uint16_t* n_sqs);
/* Create the completion / submission queue `id` (1..) in page `offset` of the mapping `dma`, which
 * must be host memory; qs entries (0 = as many as fit one controller page). */
int nvm_admin_cq_create(nvm_aq_ref ref, nvm_queue_t* cq, uint16_t id, const nvm_dma_t* dma, size_t offset, size_t qs);
int nvm_admin_cq_delete(nvm_aq_ref ref, nvm_queue_t* cq);
int nvm_admin_sq_create(nvm_aq_ref ref, nvm_queue_t* sq, const nvm_queue_t* cq, uint16_t id, const nvm_dma_t* dma, size_t offset, size_t qs);
int nvm_admin_sq_delete(nvm_aq_ref ref, nvm_queue_t* sq, const nvm_queue_t* cq);
/* Admin pass-through (nvm_rpc.h:53 there): the command is executed the way the controller would execute it
 * from its admin queue -- IDENTIFY (CNS 1 controller, CNS 0 namespace; the page goes to PRP1, which must lie
 * in memory mapped with nvm_dma_*), SET / GET FEATURES 0x07 (number of queues), CREATE / DELETE I/O completion
 * and submission queue (contiguous, power-of-two sizes, host memory), GET LOG PAGE 1..3 (empty logs) -- and
 * the completion is filled in.  Returns 0, an errno, or the packed NVMe status -(SCT << 8 | SC).  The
 * nvm_admin_* functions above are clients of this call, as in the reference (src/admin.cpp). */
int nvm_raw_rpc(nvm_aq_ref ref, nvm_cmd_t* cmd, nvm_cpl_t* cpl);
int nvm_admin_get_log_page(nvm_aq_ref ref, uint32_t ns_id, void* ptr, uint64_t ioaddr, uint8_t log_id, uint64_t log_offset);

/* ---- classic host-side queue functions (nvm_queue.h:30-286, src/queue.cpp:12-80) ----------------- */
int nvm_queue_clear(nvm_queue_t* q, const nvm_ctrl_t* ctrl, bool cq, uint16_t no, uint32_t qs, bool local, volatile void* vaddr,
                    uint64_t ioaddr);
void nvm_queue_reset(nvm_queue_t* q);
nvm_cpl_t* nvm_cq_dequeue_block(nvm_queue_t* cq, uint64_t timeout_ms);

#define NVM_SQ_DBL_OFFSET(no, dstrd) (0x1000 + (size_t)(2 * (no)) * ((size_t)4 << (dstrd)))
#define NVM_CQ_DBL_OFFSET(no, dstrd) (0x1000 + (size_t)(2 * (no) + 1) * ((size_t)4 << (dstrd)))

/* Next free submission entry, or NULL when the queue is full; the caller fills it in. */
static inline nvm_cmd_t* nvm_sq_enqueue(nvm_queue_t* sq)
{
    if ((uint32_t)(sq->tail - sq->head + sq->qs) % sq->qs == sq->qs - 1) return NULL;
    nvm_cmd_t* cmd = (nvm_cmd_t*)((unsigned char*)sq->vaddr + (size_t)sq->es * sq->tail);
    if (++sq->tail == sq->qs) { sq->tail = 0; sq->phase = !sq->phase; }
    return cmd;
}
/* Ring the submission doorbell if entries were added since the last time. */
static inline void nvm_sq_submit(nvm_queue_t* sq)
{
    if (sq->last != sq->tail && sq->db != NULL) {
        __atomic_thread_fence(__ATOMIC_RELEASE);          /* the entries before the doorbell */
        *sq->db = sq->tail;
        sq->last = sq->tail;
    }
}
/* The completion at the head if its phase bit says it is new, else NULL. */
static inline nvm_cpl_t* nvm_cq_poll(const nvm_queue_t* cq)
{
    nvm_cpl_t* cpl = (nvm_cpl_t*)((unsigned char*)cq->vaddr + (size_t)cq->es * cq->head);
    const uint32_t dw3 = __atomic_load_n(&cpl->dword[3], __ATOMIC_ACQUIRE);
    if (((dw3 >> 16) & 1u) != (uint32_t)(cq->phase != 0)) return NULL;
    return cpl;
}
static inline nvm_cpl_t* nvm_cq_dequeue(nvm_queue_t* cq)
{
    nvm_cpl_t* cpl = nvm_cq_poll(cq);
    if (cpl != NULL && ++cq->head == cq->qs) { cq->head = 0; cq->phase = !cq->phase; }
    return cpl;
}
/* One submission entry has been consumed (call once per completion taken). */
static inline void nvm_sq_update(nvm_queue_t* sq)
{
    if (sq->db != NULL && ++sq->head == sq->qs) sq->head = 0;
}
/* Tell the controller how far the completion queue has been read. */
static inline void nvm_cq_update(nvm_queue_t* cq)
{
    if (cq->last != cq->head && cq->db != NULL) {
        *cq->db = cq->head;
        cq->tail = cq->last = cq->head;
    }
}

#ifdef __cplusplus
}
#endif
#endif
