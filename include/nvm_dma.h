/* nvm_dma.h -- nvm_dma_t, nvm_dma_map / map_host / map_device / create / unmap (include/nvm_dma.h:35-147 there).
 * Served by the emulated controller: declarations and semantics in nvm_host_api.h. */
#ifndef BAM_COMPAT_NVM_DMA_H
#define BAM_COMPAT_NVM_DMA_H
#include "nvm_host_api.h"
#endif
