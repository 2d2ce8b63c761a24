/* nvm_util.h -- the page / block arithmetic helpers benchmarks take from the reference's
 * include/nvm_util.h:106-150 (sizes are powers of two or plain multiples as there). */
#ifndef BAM_COMPAT_NVM_UTIL_H
#define BAM_COMPAT_NVM_UTIL_H
#include <stddef.h>
#include <stdint.h>

#define NVM_MIN(a, b) ((a) <= (b) ? (a) : (b))
#define NVM_MAX(a, b) ((a) >= (b) ? (a) : (b))
/* number of blocks that precede page `pageno`, and the page a block falls into */
#define NVM_PAGE_TO_BLOCK(page_size, block_size, pageno) (((uint64_t)(page_size) * (pageno)) / (block_size))
#define NVM_BLOCK_TO_PAGE(page_size, block_size, blockno) (((uint64_t)(block_size) * (blockno)) / (page_size))
#define NVM_PAGE_MASK(page_size) (~((uint64_t)(page_size) - 1))
#define NVM_ADDR_MASK(addr, page_size) (((uint64_t)(addr)) & NVM_PAGE_MASK(page_size))
/* size rounded up to whole pages */
#define NVM_PAGE_ALIGN(size, page_size) ((((uint64_t)(size)) + (page_size) - 1) & NVM_PAGE_MASK(page_size))
#define NVM_ADDR_OFFSET(addr, page_size, pageno) (((uint64_t)(addr)) + ((uint64_t)(page_size)) * (pageno))
#define NVM_PTR_OFFSET(ptr, page_size, pageno) ((void*)(((unsigned char*)(ptr)) + ((uint64_t)(page_size)) * (pageno)))

/* sizes in units of the controller's page (ctrl_ptr: nvm_ctrl_t*) or of a DMA mapping's page (dma_ptr: nvm_dma_t*) */
#define NVM_CTRL_ALIGN(ctrl_ptr, size) NVM_PAGE_ALIGN((size), (ctrl_ptr)->page_size)
#define NVM_CTRL_PAGES(ctrl_ptr, size) (NVM_CTRL_ALIGN((ctrl_ptr), (size)) / (ctrl_ptr)->page_size)
#define NVM_DMA_ALIGN(dma_ptr, size) NVM_PAGE_ALIGN((size), (dma_ptr)->page_size)
#define NVM_DMA_OFFSET(dma_ptr, pageno) NVM_PTR_OFFSET((dma_ptr)->vaddr, (dma_ptr)->page_size, (pageno))
/* pages a queue of qs entries occupies (64-byte submission, 16-byte completion entries), and the
 * entries that fit one page */
#define NVM_SQ_PAGES(ctrl_ptr, qs) ((((uint16_t)((qs) - 1)) * (size_t)64) / (ctrl_ptr)->page_size + 1)
#define NVM_CQ_PAGES(ctrl_ptr, qs) ((((uint16_t)((qs) - 1)) * (size_t)16) / (ctrl_ptr)->page_size + 1)
#define NVM_SQ_SIZE(ctrl_ptr, num_pages) ((ctrl_ptr)->page_size / 64)
#define NVM_CQ_SIZE(ctrl_ptr, num_pages) ((ctrl_ptr)->page_size / 16)

/* fields of a submission entry (p: nvm_cmd_t*) and of a completion entry (p: nvm_cpl_t*), as pointers */
#define NVM_FIELD_PTR(p, byte_offset, type) ((volatile type*)(((volatile unsigned char*)(p)) + (byte_offset)))
#define NVM_CMD_CID(p) NVM_FIELD_PTR(p, 2, uint16_t)
#define NVM_CMD_NSID(p) NVM_FIELD_PTR(p, 4, uint32_t)
#define NVM_CPL_SQHD(p) NVM_FIELD_PTR(p, 8, uint16_t)
#define NVM_CPL_SQID(p) NVM_FIELD_PTR(p, 10, uint16_t)
#define NVM_CPL_CID(p) NVM_FIELD_PTR(p, 12, uint16_t)
#define NVM_CPL_SF(p) NVM_FIELD_PTR(p, 14, uint16_t)         /* phase tag in bit 0, status above it */
#define NVM_CPL_STATUS(p) NVM_CPL_SF(p)
/* a command id that is unique among the commands a host-driven queue can have in flight */
#define NVM_DEFAULT_CID(sq) ((uint16_t)((sq)->tail + (!(sq)->phase) * (sq)->qs))
#endif
