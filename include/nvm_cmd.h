/* nvm_cmd.h -- command builders under the reference's header name (include/nvm_cmd.h:20-236 there):
 * opcodes, nvm_cmd_header / nvm_cmd_data_ptr / nvm_cmd_rw_blks, and the PRP-list helpers a host
 * program uses for transfers of more than two controller pages. */
#ifndef BAM_COMPAT_NVM_CMD_H
#define BAM_COMPAT_NVM_CMD_H
#include "bam/queue.cuh"
#include "nvm_util.h"
using bam::nvm_cmd_data_ptr;
using bam::nvm_cmd_header;
using bam::nvm_cmd_rw_blks;

#define NVM_CMD_NS_ALL 0xffffffffu
/* opcode byte: bit 7 generic-command flag, bits 6:2 function, bits 1:0 data transfer direction */
#define NVM_CMD_OPCODE(gen, fun, data) ((((gen) & 1u) << 7) | (((fun) & 0x1fu) << 2) | ((data) & 3u))
#define NVM_IO_WRITE_ZEROES 0x08
enum nvm_admin_command_set {
    NVM_ADMIN_DELETE_SQ = 0x00, NVM_ADMIN_CREATE_SQ = 0x01, NVM_ADMIN_GET_LOG_PAGE = 0x02, NVM_ADMIN_DELETE_CQ = 0x04,
    NVM_ADMIN_CREATE_CQ = 0x05, NVM_ADMIN_IDENTIFY = 0x06, NVM_ADMIN_ABORT = 0x08, NVM_ADMIN_SET_FEATURES = 0x09,
    NVM_ADMIN_GET_FEATURES = 0x0a
};

/* One memory page that holds a list of page addresses (nvm_types.h:169-178 there). */
typedef struct BAM_ALIGNAS(32) {
    volatile void* vaddr;      /* where the program writes the entries    */
    int16_t local;
    size_t page_size;
    uint64_t ioaddr;           /* the address the controller reads them at */
} nvm_prp_list_t;

static inline nvm_prp_list_t nvm_prp_list_init(volatile void* vaddr, int local, size_t page_size, uint64_t ioaddr)
{
    nvm_prp_list_t l;
    l.vaddr = vaddr; l.local = (int16_t)(local != 0); l.page_size = page_size; l.ioaddr = ioaddr;
    return l;
}
#define NVM_PRP_LIST_INIT(vaddr, local, page_size, ioaddr) nvm_prp_list_init((vaddr), (local), (page_size), (ioaddr))
/* the list page is page `offset` of a DMA mapping */
#define NVM_PRP_LIST(dma_ptr, offset) \
    NVM_PRP_LIST_INIT(NVM_DMA_OFFSET(dma_ptr, offset), (dma_ptr)->local, (dma_ptr)->page_size, (dma_ptr)->ioaddrs[(offset)])

/* Fill one list page with the addresses of up to n_pages data pages.  When they do not all fit, the
 * last entry of the page stays free for the link to the next list page.  Returns the entries written. */
__host__ __device__ static inline size_t nvm_prp_list(const nvm_prp_list_t* list, size_t n_pages, const uint64_t* ioaddrs)
{
    const size_t cap = list->page_size / sizeof(uint64_t);
    const size_t n = n_pages > cap ? cap - 1 : n_pages;
    volatile uint64_t* e = (volatile uint64_t*)list->vaddr;
    for (size_t i = 0; i < n; i++) e[i] = ioaddrs[i];
    return n;
}

/* Spread n_pages addresses over a chain of list pages, each full page ending in the address of the
 * next one.  Returns the data-page entries written. */
__host__ __device__ static inline size_t nvm_prp_list_chain(size_t n_lists, const nvm_prp_list_t* lists, size_t n_pages, const uint64_t* ioaddrs)
{
    size_t written = 0;
    for (size_t l = 0; l < n_lists && lists != NULL && written < n_pages; l++) {
        const size_t n = nvm_prp_list(&lists[l], n_pages - written, ioaddrs + written);
        written += n;
        if (written < n_pages && l + 1 < n_lists) ((volatile uint64_t*)lists[l].vaddr)[n] = lists[l + 1].ioaddr;
    }
    return written;
}

/* Set a command's data pointer for a transfer of n_pages controller pages: one page -> PRP1 only, two
 * -> PRP1 and PRP2, more -> PRP1 and a list (built in `lists`) named by PRP2.  Returns the number of
 * addresses consumed from ioaddrs. */
__host__ __device__ static inline size_t nvm_cmd_data(nvm_cmd_t* cmd, size_t n_lists, const nvm_prp_list_t* lists, size_t n_pages, const uint64_t* ioaddrs)
{
    if (n_pages == 0) return 0;
    if (lists == NULL) n_lists = 0;
    size_t used = 1;
    uint64_t second = 0;
    if (n_pages > 2 && n_lists != 0) {
        used += nvm_prp_list_chain(n_lists, lists, n_pages - 1, ioaddrs + 1);
        second = lists[0].ioaddr;
    } else if (n_pages >= 2) {
        second = ioaddrs[used++];
    }
    nvm_cmd_data_ptr(cmd, ioaddrs[0], second);
    return used;
}
#endif
