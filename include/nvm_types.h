/* nvm_types.h -- nvm_queue_t, nvm_cmd_t, nvm_cpl_t, nvm_ctrl_t, nvm_dma_t, nvm_aq_ref, nvm_ctrl_info,
 * nvm_ns_info under the reference's header name (include/nvm_types.h:19-232 there). */
#ifndef BAM_COMPAT_NVM_TYPES_H
#define BAM_COMPAT_NVM_TYPES_H
#include "bam/abi_types.h"
#include "nvm_host_api.h"
#endif
