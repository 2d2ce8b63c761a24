/*
 * ctrl.h -- host-side Controller, source compatible with the reference's include/ctrl.h:
 *   Controller(path, nvmNamespace, cudaDevice, queueDepth, numQueues)   (ctrl.h:148-199 there)
 *   d_ctrl_ptr, n_qps, print_reset_stats()                              (ctrl.h:39-92)
 * Instead of opening /dev/libnvm* and creating queue pairs through admin commands, the
 * constructor creates this library's emulated controller through the C ABI.  The size of the
 * emulated namespace comes from the extra argument store_bytes, or from a path of the form
 * "emu:<bytes>" / "emu:<n>G|M|K", or from the environment variable BAM_STORE_BYTES, else 1 GiB.
 * Failures throw std::runtime_error, as the reference does (ctrl.h:98-101).
 */
#ifndef BAM_COMPAT_CTRL_H
#define BAM_COMPAT_CTRL_H

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <stdexcept>
#include <string>

#include "bam_abi.h"
#include "bam/abi_types.h"
#include "nvm_host_api.h"

#define MAX_QUEUES 1024

inline uint64_t bam_parse_size(const char* s)
{
    char* end = nullptr;
    double v = strtod(s, &end);
    uint64_t mul = 1;
    if (end && (*end == 'G' || *end == 'g')) mul = 1ull << 30;
    else if (end && (*end == 'M' || *end == 'm')) mul = 1ull << 20;
    else if (end && (*end == 'K' || *end == 'k')) mul = 1ull << 10;
    return (uint64_t)(v * (double)mul);
}

inline Controller::Controller(const char* path, uint32_t nvmNamespace, uint32_t cudaDevice, uint64_t queueDepth,
                              uint64_t numQueues, uint64_t store_bytes)
{
    (void)nvmNamespace;
    memset(static_cast<void*>(this), 0, sizeof(*this));
    if (store_bytes == 0 && path && strncmp(path, "emu:", 4) == 0) store_bytes = bam_parse_size(path + 4);
    if (store_bytes == 0 && getenv("BAM_STORE_BYTES")) store_bytes = bam_parse_size(getenv("BAM_STORE_BYTES"));
    if (store_bytes == 0) store_bytes = 1ull << 30;
    store_bytes = (store_bytes + 4095) / 4096 * 4096;
    if (queueDepth > 1024) queueDepth = 1024;            /* MAX_SQ_ENTRIES_64K, queue.h:55 of the reference */
    bam_ctrl_t handle = nullptr;
    int rc = bam_ctrl_create(&handle, (int)cudaDevice, store_bytes, 512, (uint32_t)numQueues, (uint32_t)queueDepth);
    if (rc != 0) throw std::runtime_error(std::string("Failed to create controller: ") + bam_strerror(rc));
    h = handle;
    d_ctrl_ptr = bam_ctrl_device_controller(handle);
    n_qps = (uint32_t)numQueues;
    page_size = 4096;
    blk_size = 512;
    blk_size_log = 9;
    deviceId = cudaDevice;
    /* the libnvm view of the same controller, as the reference's constructor leaves it (ctrl.h:148-199 there) */
    if (nvm_emu_ctrl_init(&ctrl, handle) == 0 && nvm_aq_create(&aq_ref, ctrl, nullptr) == 0) {
        nvm_admin_ctrl_info(aq_ref, &info, nullptr, 0);
        nvm_admin_ns_info(aq_ref, &ns, nvmNamespace ? nvmNamespace : 1, nullptr, 0);
        n_sqs = n_cqs = (uint16_t)numQueues;
    }
}

inline void Controller::close()
{
    if (aq_ref) { nvm_aq_destroy(aq_ref); aq_ref = nullptr; }
    if (ctrl) { nvm_ctrl_free(ctrl); ctrl = nullptr; }
    if (h) { bam_ctrl_destroy(h); h = nullptr; }
}

inline void Controller::print_reset_stats()
{
    uint64_t n = 0;
    bam_ctrl_served(h, &n, 1);
    printf("------------------------------------\n#SSDAccesses:\t%llu\n", (unsigned long long)n);
}

#endif
