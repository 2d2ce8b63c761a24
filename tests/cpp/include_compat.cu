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
#include <nvm_dma.h>
#include <nvm_aq.h>
#include <nvm_rpc.h>
#include <string>
#include <stdexcept>
#include <vector>
#include <cstdio>
#include <cstdint>
#include <cstdlib>
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

/* the signatures of the reference's host library (include/nvm_ctrl.h:36-76, nvm_dma.h:35-147, nvm_aq.h:23-38,
 * nvm_admin.h:18-117, nvm_rpc.h:33-53, nvm_queue.h:30-50,220, nvm_util.h:234-250, nvm_error.h:67): a pointer of
 * the reference's type must accept the function of that name (nvm_admin_cq_create / sq_create: without the
 * trailing `need_prp` argument, which has a default there and is always physically-contiguous here) */
static int (*const sig_ctrl_init)(nvm_ctrl_t**, int) = nvm_ctrl_init;
static int (*const sig_raw_ctrl_init)(nvm_ctrl_t**, volatile void*, size_t) = nvm_raw_ctrl_init;
static void (*const sig_ctrl_free)(nvm_ctrl_t*) = nvm_ctrl_free;
static int (*const sig_raw_ctrl_reset)(const nvm_ctrl_t*, uint64_t, uint64_t) = nvm_raw_ctrl_reset;
static int (*const sig_dma_map)(nvm_dma_t**, const nvm_ctrl_t*, void*, size_t, size_t, const uint64_t*) = nvm_dma_map;
static int (*const sig_dma_remap)(nvm_dma_t**, const nvm_dma_t*) = nvm_dma_remap;
static void (*const sig_dma_unmap)(nvm_dma_t*) = nvm_dma_unmap;
static int (*const sig_dma_map_host)(nvm_dma_t**, const nvm_ctrl_t*, void*, size_t) = nvm_dma_map_host;
static int (*const sig_dma_map_device)(nvm_dma_t**, const nvm_ctrl_t*, void*, size_t) = nvm_dma_map_device;
static int (*const sig_dma_create)(nvm_dma_t**, const nvm_ctrl_t*, size_t) = nvm_dma_create;
static int (*const sig_aq_create)(nvm_aq_ref*, const nvm_ctrl_t*, const nvm_dma_t*) = nvm_aq_create;
static void (*const sig_aq_destroy)(nvm_aq_ref) = nvm_aq_destroy;
static int (*const sig_ctrl_info)(nvm_aq_ref, struct nvm_ctrl_info*, void*, uint64_t) = nvm_admin_ctrl_info;
static int (*const sig_ns_info)(nvm_aq_ref, struct nvm_ns_info*, uint32_t, void*, uint64_t) = nvm_admin_ns_info;
static int (*const sig_set_nq)(nvm_aq_ref, uint16_t, uint16_t) = nvm_admin_set_num_queues;
static int (*const sig_get_nq)(nvm_aq_ref, uint16_t*, uint16_t*) = nvm_admin_get_num_queues;
static int (*const sig_req_nq)(nvm_aq_ref, uint16_t*, uint16_t*) = nvm_admin_request_num_queues;
static int (*const sig_cq_create)(nvm_aq_ref, nvm_queue_t*, uint16_t, const nvm_dma_t*, size_t, size_t) = nvm_admin_cq_create;
static int (*const sig_cq_delete)(nvm_aq_ref, nvm_queue_t*) = nvm_admin_cq_delete;
static int (*const sig_sq_create)(nvm_aq_ref, nvm_queue_t*, const nvm_queue_t*, uint16_t, const nvm_dma_t*, size_t, size_t) = nvm_admin_sq_create;
static int (*const sig_sq_delete)(nvm_aq_ref, nvm_queue_t*, const nvm_queue_t*) = nvm_admin_sq_delete;
static int (*const sig_log_page)(nvm_aq_ref, uint32_t, void*, uint64_t, uint8_t, uint64_t) = nvm_admin_get_log_page;
static int (*const sig_raw_rpc)(nvm_aq_ref, nvm_cmd_t*, nvm_cpl_t*) = nvm_raw_rpc;
static void (*const sig_rpc_unbind)(nvm_aq_ref) = nvm_rpc_unbind;
static int (*const sig_queue_clear)(nvm_queue_t*, const nvm_ctrl_t*, bool, uint16_t, uint32_t, bool, volatile void*, uint64_t) = nvm_queue_clear;
static void (*const sig_queue_reset)(nvm_queue_t*) = nvm_queue_reset;
static nvm_cpl_t* (*const sig_dequeue_block)(nvm_queue_t*, uint64_t) = nvm_cq_dequeue_block;
static const nvm_ctrl_t* (*const sig_from_aq)(nvm_aq_ref) = nvm_ctrl_from_aq_ref;
static const nvm_ctrl_t* (*const sig_from_dma)(const nvm_dma_t*) = nvm_ctrl_from_dma;
static const char* (*const sig_strerror)(int) = nvm_strerror;
static_assert(NVM_CMD_OPCODE(0, 0, 2) == NVM_IO_READ && NVM_CMD_OPCODE(0, 0, 1) == NVM_IO_WRITE && NVM_CMD_OPCODE(0, 2, 0) == NVM_IO_WRITE_ZEROES &&
              NVM_CMD_OPCODE(0, 1, 2) == NVM_ADMIN_IDENTIFY && NVM_CMD_OPCODE(0, 2, 1) == NVM_ADMIN_SET_FEATURES, "opcode packing");
static_assert(NVM_CTRL_MEM_MINSIZE == 0x2000 && sizeof(nvm_prp_list_t) == 32, "register window, list descriptor");

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

/* the reference's raw access sequence (benchmarks/block/main.cu:66-93, access_data there), compiled as written */
__device__ void ref_access_data(QueuePair* qp, uint64_t starting_lba, uint64_t n_blocks, uint64_t prp1, uint64_t prp2)
{
    nvm_cmd_t cmd;
    uint16_t cid = get_cid(&(qp->sq));
    nvm_cmd_header(&cmd, cid, NVM_IO_READ, qp->nvmNamespace);
    nvm_cmd_data_ptr(&cmd, prp1, prp2);
    nvm_cmd_rw_blks(&cmd, starting_lba, n_blocks);
    uint16_t sq_pos = sq_enqueue(&qp->sq, &cmd);
    uint32_t cq_pos = cq_poll(&qp->cq, cid);
    sq_dequeue(&qp->sq, sq_pos);
    cq_dequeue(&qp->cq, cq_pos);
    put_cid(&qp->sq, cid);
}

__global__ void touch_raw(QueuePair* qp, uint64_t prp1) { ref_access_data(qp, 0, 8, prp1, 0); }

/* --prp n_lists n_pages: what nvm_cmd_data makes of a transfer of n_pages pages at 0x100000 + i * 4096 with
 * list pages at bus addresses 0xa000, 0xb000, ... (initialised to all ones), as JSON */
static int show_prp(size_t n_lists, size_t n_pages)
{
    std::vector<std::vector<uint64_t>> pages(n_lists, std::vector<uint64_t>(512, ~0ull));
    std::vector<nvm_prp_list_t> lists;
    for (size_t l = 0; l < n_lists; l++) lists.push_back(NVM_PRP_LIST_INIT(pages[l].data(), 1, 4096, 0xa000 + l * 0x1000));
    std::vector<uint64_t> addrs(n_pages + 1);
    for (size_t i = 0; i < addrs.size(); i++) addrs[i] = 0x100000ull + i * 4096;
    nvm_cmd_t cmd = {};
    const size_t used = nvm_cmd_data(&cmd, n_lists, n_lists ? lists.data() : NULL, n_pages, addrs.data());
    printf("{\"used\": %zu, \"dptr\": [%u, %u, %u, %u], \"lists\": [", used, cmd.dword[6], cmd.dword[7], cmd.dword[8], cmd.dword[9]);
    for (size_t l = 0; l < n_lists; l++) {
        printf("%s[", l ? ", " : "");
        for (size_t i = 0; i < 512; i++) printf("%s%llu", i ? ", " : "", (unsigned long long)pages[l][i]);
        printf("]");
    }
    printf("]}\n");
    return 0;
}

int main(int argc, char** argv)
{
    if (argc == 4 && std::string(argv[1]) == "--prp") return show_prp(strtoull(argv[2], nullptr, 0), strtoull(argv[3], nullptr, 0));
    if (argc > 1) {                        /* needs a GPU; without arguments the program only runs host code */
        BufferPtr b = createBuffer(64);
        (void)b;
    }
    /* the members benchmarks read from a Controller (ctrl.h:39-59 of the reference) */
    Controller* c = nullptr;
    static_assert(sizeof(c->ns.lba_data_size) == sizeof(size_t) && sizeof(c->info.max_entries) == 2, "identify data");
    static_assert(sizeof(c->ctrl->page_size) == sizeof(size_t) && sizeof(c->n_qps) == 4 && sizeof(c->d_qps->block_size_log) == 4, "handle");
    nvm_queue_t q;
    nvm_queue_reset(&q);
    (void)nvm_sq_enqueue;
    (void)nvm_cq_dequeue;
    printf("%s\n", nvm_strerror(0));

    /* host-side helpers: queue sizing, entry fields, status packing, PRP lists (nvm_util.h:157-227, nvm_error.h:15-48,
     * nvm_cmd.h:113-236 of the reference) */
    int bad = 0;
    bad += !sig_ctrl_init || !sig_raw_ctrl_init || !sig_ctrl_free || !sig_raw_ctrl_reset || !sig_dma_map || !sig_dma_remap || !sig_dma_unmap ||
           !sig_dma_map_host || !sig_dma_map_device || !sig_dma_create || !sig_aq_create || !sig_aq_destroy || !sig_ctrl_info || !sig_ns_info ||
           !sig_set_nq || !sig_get_nq || !sig_req_nq || !sig_cq_create || !sig_cq_delete || !sig_sq_create || !sig_sq_delete || !sig_log_page ||
           !sig_raw_rpc || !sig_rpc_unbind || !sig_queue_clear || !sig_queue_reset || !sig_dequeue_block || !sig_from_aq || !sig_from_dma ||
           !sig_strerror;
    nvm_ctrl_t hc = {};
    hc.page_size = 4096;
    bad += NVM_SQ_PAGES(&hc, 1024) != 16 || NVM_CQ_PAGES(&hc, 1024) != 4 || NVM_SQ_PAGES(&hc, 64) != 1 || NVM_CQ_PAGES(&hc, 257) != 2;
    bad += NVM_SQ_SIZE(&hc, 1) != 64 || NVM_CQ_SIZE(&hc, 1) != 256 || NVM_CTRL_PAGES(&hc, 4097) != 2 || NVM_CTRL_ALIGN(&hc, 1) != 4096;
    nvm_cpl_t cpl = {};
    cpl.dword[2] = 0x0003002au;                                  /* SQID 3, SQHD 42 */
    cpl.dword[3] = 0x1234u | (1u << 16) | ((0x80u | (2u << 8)) << 17) | (1u << 31);     /* CID, phase, SC 0x80 / SCT 2, DNR */
    bad += *NVM_CPL_CID(&cpl) != 0x1234 || *NVM_CPL_SQHD(&cpl) != 42 || *NVM_CPL_SQID(&cpl) != 3;
    bad += NVM_ERR_SC(&cpl) != 0x80 || NVM_ERR_SCT(&cpl) != 2 || !NVM_ERR_DNR(&cpl) || NVM_ERR_MORE(&cpl) || NVM_ERR_OK(&cpl);
    bad += NVM_ERR_STATUS(&cpl) != -0x280 || NVM_ERR_PACK(&cpl, 0) != -0x280 || NVM_ERR_PACK(&cpl, 5) != 5 || NVM_ERR_PACK((nvm_cpl_t*)NULL, 0) != 0;
    nvm_cmd_t cmd = {};
    nvm_cmd_header(&cmd, 0xbeef, NVM_IO_READ, 9);
    bad += *NVM_CMD_CID(&cmd) != 0xbeef || *NVM_CMD_NSID(&cmd) != 9;
    nvm_queue_t sq = {};
    sq.qs = 64; sq.tail = 5; sq.phase = 1;
    bad += NVM_DEFAULT_CID(&sq) != 5;
    sq.phase = 0;
    bad += NVM_DEFAULT_CID(&sq) != 69;

    std::vector<uint64_t> page_a(512, ~0ull), page_b(512, ~0ull), addrs(700);
    for (size_t i = 0; i < addrs.size(); i++) addrs[i] = 0x100000ull + i * 4096;
    nvm_prp_list_t lists[2] = { NVM_PRP_LIST_INIT(page_a.data(), 1, 4096, 0xa000), NVM_PRP_LIST_INIT(page_b.data(), 1, 4096, 0xb000) };
    bad += nvm_cmd_data(&cmd, 2, lists, 1, addrs.data()) != 1 || cmd.dword[6] != 0x100000u || cmd.dword[8] != 0 || cmd.dword[9] != 0;
    bad += nvm_cmd_data(&cmd, 2, lists, 2, addrs.data()) != 2 || cmd.dword[8] != 0x101000u;
    bad += nvm_cmd_data(&cmd, 2, lists, 17, addrs.data()) != 17 || cmd.dword[8] != 0xa000u || page_a[0] != addrs[1] || page_a[15] != addrs[16] || page_a[16] != ~0ull;
    /* 1 + 600 pages: the first list page takes 511 addresses and the link, the second the other 89 */
    bad += nvm_cmd_data(&cmd, 2, lists, 601, addrs.data()) != 601 || page_a[510] != addrs[511] || page_a[511] != 0xb000 || page_b[0] != addrs[512] ||
           page_b[88] != addrs[600];
    /* exactly one list page: 512 addresses, no link */
    bad += nvm_cmd_data(&cmd, 1, lists, 513, addrs.data()) != 513 || page_a[511] != addrs[512];
    bad += nvm_cmd_data(&cmd, 0, NULL, 3, addrs.data()) != 2;                 /* no list memory: two pages at most */
    printf("{\"bad\": %d}\n", bad);
    return bad != 0;
}
