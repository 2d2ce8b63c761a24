/* nvm_rpc.h -- nvm_raw_rpc (include/nvm_rpc.h:33-53 there): admin pass-through, executed on the host the way the controller would.
 * Served by the emulated controller: declarations and semantics in nvm_host_api.h. */
#ifndef BAM_COMPAT_NVM_RPC_H
#define BAM_COMPAT_NVM_RPC_H
#include "nvm_host_api.h"
#endif
