/* nvm_error.h -- status conventions of the reference's include/nvm_error.h:15-67: 0 = success, a
 * positive value is an errno, a negative value packs an NVMe completion status as
 * -((status code type << 8) | status code). */
#ifndef BAM_COMPAT_NVM_ERROR_H
#define BAM_COMPAT_NVM_ERROR_H
#include "bam_abi.h"
#include "nvm_util.h"

/* fields of a completion's status half-word (bit 0 is the phase tag): status code 8:1, status code
 * type 11:9, "more" 14, "do not retry" 15 */
#define NVM_ERR_SC(cpl) ((uint8_t)((*NVM_CPL_STATUS(cpl) >> 1) & 0xff))
#define NVM_ERR_SCT(cpl) ((uint8_t)((*NVM_CPL_STATUS(cpl) >> 9) & 0x7))
#define NVM_ERR_MORE(cpl) (((*NVM_CPL_STATUS(cpl) >> 14) & 1) != 0)
#define NVM_ERR_DNR(cpl) (((*NVM_CPL_STATUS(cpl) >> 15) & 1) != 0)
#define NVM_ERR_OK(cpl) (!NVM_ERR_SCT(cpl) && !NVM_ERR_SC(cpl))
/* a completion (may be NULL) as a packed status; an errno, when there is one, wins */
#define NVM_ERR_STATUS(cpl) ((int)((cpl) != NULL ? -((NVM_ERR_SCT(cpl) << 8) | NVM_ERR_SC(cpl)) : 0))
#define NVM_ERR_PACK(cpl, err) ((int)((err) != 0 ? (err) : NVM_ERR_STATUS(cpl)))

#define nvm_ok(status) (!(status))
#define NVM_ERR_UNPACK_ERRNO(status) (((status) > 0) ? (status) : 0)
#define NVM_ERR_UNPACK_SCT(status) (((status) < 0) ? ((-(status) >> 8) & 0xff) : 0)
#define NVM_ERR_UNPACK_SC(status) (((status) < 0) ? (-(status) & 0xff) : 0)
/* The packed form of the 15-bit status field a completion carries (bam_status_out_t.detail after
 * BAM_AT_NVME_STATUS): bits 7:0 status code, bits 10:8 status code type. */
#define NVM_ERR_FROM_STATUS_FIELD(sf) (-(int)((((sf) >> 8) & 0x7) << 8 | ((sf) & 0xff)))

#ifdef __cplusplus
extern "C" {
#endif
/* Text for a packed status: the library's message for 0 and errno values, the NVMe name of the
 * status for negative ones. */
const char* nvm_strerror(int status);
#ifdef __cplusplus
}
#endif
#endif
