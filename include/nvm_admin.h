/* nvm_admin.h -- nvm_admin_ctrl_info / ns_info / *_num_queues / cq_create / sq_create / *_delete (include/nvm_admin.h:18-117 there).
 * Served by the emulated controller: declarations and semantics in nvm_host_api.h. */
#ifndef BAM_COMPAT_NVM_ADMIN_H
#define BAM_COMPAT_NVM_ADMIN_H
#include "nvm_host_api.h"
#endif
