/* nvm_io.h -- present so that programs written against the reference's include list compile.  The
 * reference's nvm_io.h declares part of its host-side control plane (controller bring-up over a
 * kernel module, admin queue, DMA windows, host-side queue polling); the emulated controller of
 * this library is created and driven through bam_abi.h (bam_ctrl_create, bam_ctrl_reset_queues,
 * ...) and needs none of it. */
#ifndef BAM_COMPAT_NVM_IO_H
#define BAM_COMPAT_NVM_IO_H
#include "bam_abi.h"
#include "nvm_types.h"
#endif
