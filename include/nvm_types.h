/* nvm_types.h -- nvm_queue_t, nvm_cmd_t, nvm_cpl_t under the reference's header name. */
#ifndef BAM_COMPAT_NVM_TYPES_H
#define BAM_COMPAT_NVM_TYPES_H
#include "bam/abi_types.h"
#endif
