/* nvm_io.h -- the I/O command helpers live in nvm_cmd.h; this name only completes the include list (include/nvm_io.h there).
 * Served by the emulated controller: declarations and semantics in nvm_host_api.h. */
#ifndef BAM_COMPAT_NVM_IO_H
#define BAM_COMPAT_NVM_IO_H
#include "nvm_host_api.h"
#endif
