/* nvm_aq.h -- nvm_aq_ref, nvm_aq_create, nvm_aq_destroy (include/nvm_aq.h:23-38 there).
 * Served by the emulated controller: declarations and semantics in nvm_host_api.h. */
#ifndef BAM_COMPAT_NVM_AQ_H
#define BAM_COMPAT_NVM_AQ_H
#include "nvm_host_api.h"
#endif
