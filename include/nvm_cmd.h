/* nvm_cmd.h -- command builders under the reference's header name (include/nvm_cmd.h:54-88 there). */
#ifndef BAM_COMPAT_NVM_CMD_H
#define BAM_COMPAT_NVM_CMD_H
#include "bam/queue.cuh"
using bam::nvm_cmd_data_ptr;
using bam::nvm_cmd_header;
using bam::nvm_cmd_rw_blks;
#endif
