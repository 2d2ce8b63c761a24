/* nvm_ctrl.h -- nvm_ctrl_t, nvm_ctrl_init, nvm_emu_ctrl_init, nvm_ctrl_free (include/nvm_ctrl.h:36-76 there).
 * Served by the emulated controller: declarations and semantics in nvm_host_api.h. */
#ifndef BAM_COMPAT_NVM_CTRL_H
#define BAM_COMPAT_NVM_CTRL_H
#include "nvm_host_api.h"
#endif
