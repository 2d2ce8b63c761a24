/*
 * include_compat.cu -- compile-only check: the include list of the reference's benchmarks
 * (benchmarks/array/main.cu:1-27) resolves against this library's headers, and the names those
 * programs use exist with the expected shapes.
 */
#include <cuda.h>
#include <nvm_ctrl.h>
#include <nvm_types.h>
#include <nvm_queue.h>
#include <nvm_util.h>
#include <nvm_admin.h>
#include <nvm_error.h>
#include <nvm_cmd.h>
#include <string>
#include <stdexcept>
#include <vector>
#include <cstdio>
#include <cstdint>
#include <ctrl.h>
#include <buffer.h>
#include <event.h>
#include <queue.h>
#include <nvm_parallel_queue.h>
#include <nvm_io.h>
#include <page_cache.h>
#include <util.h>
#include <bafs_ptr.h>

static_assert(sizeof(nvm_cmd_t) == 64 && sizeof(nvm_cpl_t) == 16, "NVMe entry sizes");
static_assert(NVM_PAGE_ALIGN(4097, 4096) == 8192 && NVM_PAGE_TO_BLOCK(4096, 512, 3) == 24, "page arithmetic");
static_assert(NVM_ERR_UNPACK_SCT(-0x281) == 2 && NVM_ERR_UNPACK_SC(-0x281) == 0x81 && NVM_ERR_UNPACK_ERRNO(5) == 5, "status packing");
static_assert(REPLICATE == 0 && STRIPE == 1, "data_dist_t");

__global__ void touch(array_d_t<uint64_t>* a, QueuePair* qp, Controller* c, unsigned long long* out)
{
    bam_ptr<uint64_t> p(a);
    bafs_ptr<uint64_t> q(a, 0);
    __shared__ tlb<uint64_t, 8> t;
    t.init(a);
    bam_ptr_tlb<uint64_t, 8> pt(a, &t);
    *out = (unsigned long long)((uint64_t)p[0] + q[1] + (uint64_t)pt[2] + qp->sq.qs + c->n_qps);
    pt.fini();
    t.fini();
}

int main()
{
    BufferPtr b = createBuffer(64);
    (void)b;
    /* the members benchmarks read from a Controller (ctrl.h:39-59 of the reference) */
    Controller* c = nullptr;
    static_assert(sizeof(c->ns.lba_data_size) == sizeof(size_t) && sizeof(c->info.max_entries) == 2, "identify data");
    static_assert(sizeof(c->ctrl->page_size) == sizeof(size_t) && sizeof(c->n_qps) == 4 && sizeof(c->d_qps->block_size_log) == 4, "handle");
    nvm_queue_t q;
    nvm_queue_reset(&q);
    (void)nvm_sq_enqueue;
    (void)nvm_cq_dequeue;
    printf("%s\n", nvm_strerror(0));
    return 0;
}
