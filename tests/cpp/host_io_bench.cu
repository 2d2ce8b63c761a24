/*
 * host_io_bench.cu -- a host program in the style of the reference's libnvm examples
 * (deprecated/examples/integrity/transfer.c:42-138): bring up a controller handle, query it through
 * the admin functions, create one I/O queue pair in host memory, and move data with NVMe WRITE and
 * READ commands that the HOST submits with the classic queue functions -- all served by the
 * emulated controller.  Checks every byte and prints one JSON line.
 */
#include <cerrno>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include <nvm_types.h>
#include <nvm_ctrl.h>
#include <nvm_dma.h>
#include <nvm_aq.h>
#include <nvm_admin.h>
#include <nvm_queue.h>
#include <nvm_cmd.h>
#include <nvm_error.h>
#include <nvm_util.h>
#include <nvm_rpc.h>
#include "bam_synth.h"

#define CHECK(x) do { int rc_ = (x); if (rc_) { fprintf(stderr, "%s failed: %s\n", #x, nvm_strerror(rc_)); return 1; } } while (0)

int main()
{
    const uint64_t store_bytes = 64ull << 20, seed = 23;
    bam_ctrl_t emu = nullptr;
    CHECK(bam_ctrl_create(&emu, 0, store_bytes, 512, 1, 64));
    bam_ctrl_set_launch_timeout(emu, 60ull * 1000 * 1000 * 1000);       /* the service kernel leaves after a minute at most */
    uint64_t* media = (uint64_t*)bam_ctrl_store_host(emu);
    for (uint64_t i = 0; i < store_bytes / 8; i++) media[i] = bam_store_elem(seed, i);

    /* device memory is allocated before the queues exist: while the service kernel runs, calls that may wait
     * for an idle device are best avoided */
    const size_t n_pages = 96;
    void* d_mem = nullptr;
    if (cudaMalloc(&d_mem, n_pages * 4096) != cudaSuccess) return 1;

    nvm_ctrl_t* ctrl = nullptr;
    CHECK(nvm_emu_ctrl_init(&ctrl, emu));
    nvm_aq_ref aq = nullptr;
    nvm_dma_t* aq_mem = nullptr;
    CHECK(nvm_dma_create(&aq_mem, ctrl, 2 * ctrl->page_size));
    CHECK(nvm_aq_create(&aq, ctrl, aq_mem));
    struct nvm_ctrl_info ci;
    struct nvm_ns_info ni;
    CHECK(nvm_admin_ctrl_info(aq, &ci, aq_mem->vaddr, aq_mem->ioaddrs[0]));
    CHECK(nvm_admin_ns_info(aq, &ni, 1, aq_mem->vaddr, aq_mem->ioaddrs[0]));
    uint16_t n_cqs = 4, n_sqs = 4;
    CHECK(nvm_admin_request_num_queues(aq, &n_cqs, &n_sqs));

    /* queue memory: page 0 = CQ (256 entries fit one page), page 1 = SQ (64 entries) */
    nvm_dma_t* q_mem = nullptr;
    CHECK(nvm_dma_create(&q_mem, ctrl, 2 * ctrl->page_size));
    nvm_queue_t cq, sq;
    CHECK(nvm_admin_cq_create(aq, &cq, 1, q_mem, 0, 0));
    CHECK(nvm_admin_sq_create(aq, &sq, &cq, 1, q_mem, 1, 0));

    /* data buffers: one the library allocates, one of the program's own (malloc'd, pinned by the mapping), one in GPU memory */
    const size_t page = ctrl->page_size, blocks_per_page = page / ni.lba_data_size;
    nvm_dma_t *buf = nullptr, *own = nullptr, *devbuf = nullptr;
    CHECK(nvm_dma_create(&buf, ctrl, n_pages * page));
    void* own_mem = nullptr;
    if (posix_memalign(&own_mem, 4096, n_pages * page)) return 1;
    CHECK(nvm_dma_map_host(&own, ctrl, own_mem, n_pages * page));
    CHECK(nvm_dma_map_device(&devbuf, ctrl, d_mem, n_pages * page));

    /* submit `n` one-page commands, at most qs - 1 in flight, and reap them; returns the number of failed completions */
    auto transfer = [&](uint8_t opcode, const nvm_dma_t* dma, uint64_t first_media_page, size_t n) -> int {
        size_t sent = 0, done = 0;
        int bad = 0;
        while (done < n) {
            while (sent < n) {
                nvm_cmd_t* cmd = nvm_sq_enqueue(&sq);
                if (!cmd) break;                                         /* queue full: reap first */
                memset(cmd, 0, sizeof *cmd);
                nvm_cmd_header(cmd, (uint16_t)sent, opcode, ni.ns_id);
                nvm_cmd_data_ptr(cmd, dma->ioaddrs[sent], 0);
                nvm_cmd_rw_blks(cmd, (first_media_page + sent) * blocks_per_page, (uint16_t)blocks_per_page);
                sent++;
            }
            nvm_sq_submit(&sq);
            nvm_cpl_t* cpl = nvm_cq_dequeue_block(&cq, ctrl->timeout);
            if (!cpl) return -1;                                         /* the controller did not answer */
            if ((cpl->dword[3] >> 17) != 0) bad++;
            nvm_sq_update(&sq);
            nvm_cq_update(&cq);
            done++;
        }
        return bad;
    };

    int bad_read = 0, bad_write = 0, bad_own = 0, bad_dev = 0, bad_status = 0;
    /* READ pages [100, 196) of the media into the library's buffer */
    int rc = transfer(NVM_IO_READ, buf, 100, n_pages);
    if (rc < 0) { fprintf(stderr, "read timed out\n"); return 1; }
    bad_status += rc;
    bad_read = memcmp(buf->vaddr, media + 100 * page / 8, n_pages * page) != 0;
    /* WRITE a pattern from the program's own pinned memory to pages [5000, 5096), READ it back into GPU memory */
    uint64_t* pat = (uint64_t*)own_mem;
    for (size_t i = 0; i < n_pages * page / 8; i++) pat[i] = bam_splitmix64(i ^ 0xabcdef);
    rc = transfer(NVM_IO_WRITE, own, 5000, n_pages);
    if (rc < 0) { fprintf(stderr, "write timed out\n"); return 1; }
    bad_status += rc;
    bad_write = memcmp(media + 5000 * page / 8, pat, n_pages * page) != 0;
    rc = transfer(NVM_IO_READ, devbuf, 5000, n_pages);
    if (rc < 0) { fprintf(stderr, "read to device timed out\n"); return 1; }
    bad_status += rc;
    std::vector<uint64_t> back(n_pages * page / 8);
    cudaMemcpy(back.data(), d_mem, n_pages * page, cudaMemcpyDeviceToHost);
    bad_dev = memcmp(back.data(), pat, n_pages * page) != 0;
    /* and the media pages next to the written range are untouched */
    bad_own = media[4999 * page / 8 + 7] != bam_store_elem(seed, 4999 * page / 8 + 7) || media[5096 * page / 8] != bam_store_elem(seed, 5096 * page / 8);
    /* a request beyond the namespace completes with an error status instead of touching memory */
    nvm_cmd_t* cmd = nvm_sq_enqueue(&sq);
    memset(cmd, 0, sizeof *cmd);
    nvm_cmd_header(cmd, 7, NVM_IO_READ, ni.ns_id);
    nvm_cmd_data_ptr(cmd, buf->ioaddrs[0], 0);
    nvm_cmd_rw_blks(cmd, ni.size, (uint16_t)blocks_per_page);
    nvm_sq_submit(&sq);
    nvm_cpl_t* cpl = nvm_cq_dequeue_block(&cq, ctrl->timeout);
    const unsigned oob_status = cpl ? (cpl->dword[3] >> 17) : 0xffffu;
    const unsigned oob_cid = cpl ? (cpl->dword[3] & 0xffffu) : 0xffffu;
    if (cpl) { nvm_sq_update(&sq); nvm_cq_update(&cq); }

    /* ---- transfers of several pages: PRP2 as second pointer, a PRP list, a list that continues in a second
     * list page, and list memory the controller was never given ---------------------------------------------- */
    auto one = [&](uint8_t opcode, uint64_t first_media_page, size_t pages, const nvm_cmd_t& dptr_of) -> int {
        nvm_cmd_t* c = nvm_sq_enqueue(&sq);
        if (!c) return -2;
        memset(c, 0, sizeof *c);
        nvm_cmd_header(c, NVM_DEFAULT_CID(&sq), opcode, ni.ns_id);
        c->dword[6] = dptr_of.dword[6]; c->dword[7] = dptr_of.dword[7]; c->dword[8] = dptr_of.dword[8]; c->dword[9] = dptr_of.dword[9];
        nvm_cmd_rw_blks(c, first_media_page * blocks_per_page, (uint16_t)(pages * blocks_per_page));
        nvm_sq_submit(&sq);
        nvm_cpl_t* done = nvm_cq_dequeue_block(&cq, ctrl->timeout);
        if (!done) return -1;
        const int st = NVM_ERR_PACK(done, 0);
        nvm_sq_update(&sq);
        nvm_cq_update(&cq);
        return st;
    };
    nvm_dma_t* list_mem = nullptr;
    CHECK(nvm_dma_create(&list_mem, ctrl, 2 * page));
    int bad_multi = 0, st_two = 0, st_list = 0, st_chain = 0, st_foreign = 0;
    nvm_cmd_t dp;
    memset(buf->vaddr, 0, n_pages * page);
    /* two pages: PRP1 + PRP2 */
    bad_multi += nvm_cmd_data(&dp, 0, NULL, 2, &buf->ioaddrs[10]) != 2;
    st_two = one(NVM_IO_READ, 300, 2, dp);
    bad_multi += memcmp(NVM_DMA_OFFSET(buf, 10), media + 300 * page / 8, 2 * page) != 0;
    /* 37 pages through one list page; the destination pages are taken in reverse order so that the list matters */
    std::vector<uint64_t> scattered(37);
    for (size_t i = 0; i < scattered.size(); i++) scattered[i] = buf->ioaddrs[50 - i];
    nvm_prp_list_t list0 = NVM_PRP_LIST(list_mem, 0);
    bad_multi += nvm_cmd_data(&dp, 1, &list0, scattered.size(), scattered.data()) != scattered.size();
    st_list = one(NVM_IO_READ, 1000, scattered.size(), dp);
    for (size_t i = 0; i < scattered.size(); i++)
        bad_multi += memcmp(NVM_DMA_OFFSET(buf, 50 - i), media + (1000 + i) * page / 8, page) != 0;
    /* 1 + 20 pages with the list starting 11 entries before the end of its page: 11 addresses, the link, 9 more */
    uint64_t* la = (uint64_t*)NVM_DMA_OFFSET(list_mem, 0);
    uint64_t* lb = (uint64_t*)NVM_DMA_OFFSET(list_mem, 1);
    memset(la, 0xff, page); memset(lb, 0xff, page);
    for (size_t i = 0; i < 11; i++) la[500 + i] = buf->ioaddrs[61 + i];
    la[511] = list_mem->ioaddrs[1];
    for (size_t i = 0; i < 9; i++) lb[i] = buf->ioaddrs[72 + i];
    memset(&dp, 0, sizeof dp);
    nvm_cmd_data_ptr(&dp, buf->ioaddrs[60], list_mem->ioaddrs[0] + 500 * 8);
    st_chain = one(NVM_IO_READ, 2000, 21, dp);
    bad_multi += memcmp(NVM_DMA_OFFSET(buf, 60), media + 2000 * page / 8, 21 * page) != 0;
    /* a list in memory that was never mapped for the controller: refused, nothing read through it */
    nvm_cmd_data_ptr(&dp, buf->ioaddrs[0], (uint64_t)(uintptr_t)d_mem + 64 * 1024 * 1024);
    st_foreign = one(NVM_IO_READ, 0, 5, dp);

    /* ---- handles: a second handle from the register window, the owners of a mapping and of an admin reference,
     * a second descriptor of a mapping that outlives the first --------------------------------------------------- */
    int bad_handles = 0;
    nvm_ctrl_t* again = nullptr;
    bad_handles += nvm_raw_ctrl_init(&again, ctrl->mm_ptr, NVM_CTRL_MEM_MINSIZE) != 0 || again != ctrl;
    bad_handles += nvm_raw_ctrl_init(&again, &bad_handles, NVM_CTRL_MEM_MINSIZE) != ENODEV || again != nullptr;
    bad_handles += nvm_raw_ctrl_init(&again, ctrl->mm_ptr, 0x1000) != EINVAL;
    nvm_ctrl_free(ctrl);                                                   /* drops the second handle only */
    const uint64_t cap = *(volatile uint64_t*)ctrl->mm_ptr;
    bad_handles += (cap & 0xffff) + 1 != ctrl->max_qs || ((cap >> 32) & 0xf) != ctrl->dstrd || (*(volatile uint32_t*)((volatile char*)ctrl->mm_ptr + 0x1c) & 1) != 1;
    bad_handles += nvm_ctrl_from_dma(buf) != ctrl || nvm_ctrl_from_aq_ref(aq) != ctrl;
    nvm_rpc_unbind(aq);
    nvm_dma_t* second = nullptr;
    CHECK(nvm_dma_remap(&second, buf));
    bad_handles += second->n_ioaddrs != buf->n_ioaddrs || second->ioaddrs[7] != buf->ioaddrs[7] || second->vaddr != buf->vaddr;
    nvm_dma_unmap(buf);
    buf = second;
    memset(buf->vaddr, 0, 2 * page);                                       /* the memory is still there and still a DMA window */
    bad_multi += nvm_cmd_data(&dp, 0, NULL, 2, &buf->ioaddrs[0]) != 2;
    const int st_remap = one(NVM_IO_READ, 4000, 2, dp);
    bad_handles += st_remap != 0 || memcmp(buf->vaddr, media + 4000 * page / 8, 2 * page) != 0;

    /* ---- admin commands through the pass-through: what the controller answers, and what it refuses ------------ */
    int bad_admin = 0;
    {
        nvm_cmd_t ac; nvm_cpl_t ap;
        uint8_t* apage = (uint8_t*)NVM_DMA_OFFSET(aq_mem, 1);
        memset(&ac, 0, sizeof ac);
        nvm_cmd_header(&ac, 77, NVM_ADMIN_IDENTIFY, 0);
        nvm_cmd_data_ptr(&ac, aq_mem->ioaddrs[1], 0);
        ac.dword[10] = 1;                                                  /* identify controller */
        memset(apage, 0xee, page);
        bad_admin += nvm_raw_rpc(aq, &ac, &ap) != 0 || !NVM_ERR_OK(&ap) || *NVM_CPL_CID(&ap) != 77;
        bad_admin += memcmp(apage + 4, ci.serial_no, 20) != 0 || memcmp(apage + 24, ci.model_no, 40) != 0 || apage[77] != 8 ||
                     apage[512] != 0x66 || apage[513] != 0x44 || ci.max_data_size != (1u << 20) || ci.nvme_version != 0x00010400;
        ac.dword[10] = 0; ac.dword[1] = 1;                                 /* identify namespace 1, into GPU memory */
        nvm_cmd_data_ptr(&ac, devbuf->ioaddrs[0], 0);
        bad_admin += nvm_raw_rpc(aq, &ac, &ap) != 0;
        uint64_t nsze = 0;
        cudaMemcpy(&nsze, d_mem, 8, cudaMemcpyDeviceToHost);
        bad_admin += nsze != ni.size;
        ac.dword[1] = 2;                                                   /* no such namespace */
        bad_admin += nvm_raw_rpc(aq, &ac, &ap) != -0x00b;
        memset(&ac, 0, sizeof ac);
        nvm_cmd_header(&ac, 1, NVM_ADMIN_GET_FEATURES, 0);
        ac.dword[10] = 0x07;
        bad_admin += nvm_raw_rpc(aq, &ac, &ap) != 0 || ap.dword[0] != ((3u << 16) | 3u);       /* 4 + 4 queues, zero-based */
        ac.dword[10] = 0x02;                                               /* a feature the controller does not have */
        bad_admin += nvm_raw_rpc(aq, &ac, &ap) != -0x002;
        memset(&ac, 0, sizeof ac);
        nvm_cmd_header(&ac, 2, 0x7f, 0);
        bad_admin += nvm_raw_rpc(aq, &ac, &ap) != -0x001 || NVM_ERR_SC(&ap) != 0x01;
        /* queue 9 was never granted; queue 1 exists; the completion queue cannot go while its submission queue lives */
        nvm_queue_t extra;
        memset(&extra, 0, sizeof extra);
        extra.no = 7;                                                      /* stands for a completion queue that does not exist */
        bad_admin += nvm_admin_cq_create(aq, &extra, 9, list_mem, 0, 0) != -0x101;
        bad_admin += nvm_admin_cq_create(aq, &extra, 1, list_mem, 0, 0) != -0x101;
        nvm_queue_t cq_copy = cq;
        bad_admin += nvm_admin_cq_delete(aq, &cq_copy) != -0x10c || strstr(nvm_strerror(-0x10c), "deletion") == NULL;
        bad_admin += nvm_admin_sq_create(aq, &extra, &extra, 2, list_mem, 0, 0) != -0x100;       /* no such completion queue */
        /* a queue in memory the controller was never given */
        memset(&ac, 0, sizeof ac);
        nvm_cmd_header(&ac, 3, NVM_ADMIN_CREATE_CQ, 0);
        nvm_cmd_data_ptr(&ac, (uint64_t)(uintptr_t)&ac, 0);
        ac.dword[10] = (255u << 16) | 2; ac.dword[11] = 1;
        bad_admin += nvm_raw_rpc(aq, &ac, &ap) != -0x004;
        /* log pages: empty health log; an unknown log id */
        memset(apage, 0xee, page);
        bad_admin += nvm_admin_get_log_page(aq, NVM_CMD_NS_ALL, apage, aq_mem->ioaddrs[1], 2, 0) != 0 || apage[0] != 0 || apage[4095] != 0;
        bad_admin += nvm_admin_get_log_page(aq, NVM_CMD_NS_ALL, apage, aq_mem->ioaddrs[1], 9, 0) != -0x109;
        /* I/O still works after all of this */
        bad_multi += nvm_cmd_data(&dp, 0, NULL, 1, &buf->ioaddrs[3]) != 1;
        bad_admin += one(NVM_IO_READ, 77, 1, dp) != 0 || memcmp(NVM_DMA_OFFSET(buf, 3), media + 77 * page / 8, page) != 0;
    }

    printf("{\"page_size\": %zu, \"max_entries\": %u, \"sq_entry\": %zu, \"cq_entry\": %zu, \"ns_blocks\": %zu, \"lba\": %zu, \"queues\": [%u, %u], "
           "\"sq_depth\": %u, \"cq_depth\": %u, \"bad_read\": %d, \"bad_write\": %d, \"bad_neighbours\": %d, \"bad_device_read\": %d, "
           "\"bad_status\": %d, \"oob_status\": %u, \"oob_cid\": %u, \"bad_multi\": %d, \"st_two\": %d, \"st_list\": %d, \"st_chain\": %d, "
           "\"st_foreign\": %d, \"foreign_text\": \"%s\", \"bad_handles\": %d, \"bad_admin\": %d}\n",
           ci.page_size, (unsigned)ci.max_entries, ci.sq_entry_size, ci.cq_entry_size, ni.size, ni.lba_data_size, n_cqs, n_sqs, sq.qs, cq.qs,
           bad_read, bad_write, bad_own, bad_dev, bad_status, oob_status, oob_cid, bad_multi, st_two, st_list, st_chain, st_foreign,
           nvm_strerror(st_foreign), bad_handles, bad_admin);

    CHECK(nvm_admin_sq_delete(aq, &sq, &cq));
    CHECK(nvm_admin_cq_delete(aq, &cq));
    /* a reset takes the admin queue addresses; misaligned ones are refused */
    if (nvm_raw_ctrl_reset(ctrl, aq_mem->ioaddrs[0] + 8, aq_mem->ioaddrs[1]) != EINVAL) { fprintf(stderr, "reset accepted a misaligned address\n"); return 1; }
    CHECK(nvm_raw_ctrl_reset(ctrl, aq_mem->ioaddrs[0], aq_mem->ioaddrs[1]));
    if (*(volatile uint64_t*)((volatile char*)ctrl->mm_ptr + 0x30) != aq_mem->ioaddrs[0]) { fprintf(stderr, "ACQ register not set\n"); return 1; }
    nvm_dma_unmap(list_mem);
    nvm_dma_unmap(devbuf); nvm_dma_unmap(own); nvm_dma_unmap(buf); nvm_dma_unmap(q_mem); nvm_dma_unmap(aq_mem);
    cudaFree(d_mem);
    free(own_mem);
    nvm_aq_destroy(aq);
    nvm_ctrl_free(ctrl);
    bam_ctrl_destroy(emu);
    return 0;
}
