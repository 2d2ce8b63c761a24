/* nvm_queue.h -- nvm_queue_clear / nvm_queue_reset and the classic host-side queue functions nvm_sq_enqueue, nvm_sq_submit, nvm_cq_poll, nvm_cq_dequeue(_block), nvm_sq_update, nvm_cq_update (include/nvm_queue.h:30-286 there).
 * Served by the emulated controller: declarations and semantics in nvm_host_api.h. */
#ifndef BAM_COMPAT_NVM_QUEUE_H
#define BAM_COMPAT_NVM_QUEUE_H
#include "nvm_host_api.h"
#endif
