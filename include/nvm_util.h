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
#endif
