/* nvm_error.h -- status conventions of the reference's include/nvm_error.h:37-67: 0 = success, a
 * positive value is an errno, a negative value packs an NVMe completion status as
 * -((status code type << 8) | status code). */
#ifndef BAM_COMPAT_NVM_ERROR_H
#define BAM_COMPAT_NVM_ERROR_H
#include "bam_abi.h"

#define nvm_ok(status) (!(status))
#define NVM_ERR_UNPACK_ERRNO(status) (((status) > 0) ? (status) : 0)
#define NVM_ERR_UNPACK_SCT(status) (((status) < 0) ? ((-(status) >> 8) & 0xff) : 0)
#define NVM_ERR_UNPACK_SC(status) (((status) < 0) ? (-(status) & 0xff) : 0)
/* The packed form of the 15-bit status field a completion carries (bam_status_out_t.detail after
 * BAM_AT_NVME_STATUS): bits 7:0 status code, bits 10:8 status code type. */
#define NVM_ERR_FROM_STATUS_FIELD(sf) (-(int)((((sf) >> 8) & 0x7) << 8 | ((sf) & 0xff)))

static inline const char* nvm_strerror(int status)
{
    if (status < 0) return "NVMe completion status";
    return bam_strerror(status);
}
#endif
