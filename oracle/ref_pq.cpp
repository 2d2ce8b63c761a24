/*
 * ref_pq.cpp -- TEST INFRASTRUCTURE: the REFERENCE's parallel queue protocol (include/nvm_parallel_queue.h:
 * get_cid / put_cid, sq_enqueue + move_tail, cq_poll, cq_dequeue + move_head_cq), compiled for the host from
 * the reference's header where it lies (recipe: oracle/Makefile, target _ref/libref_pq.so) and run by host
 * threads that play the role of GPU threads.  The reference writes its doorbells with the PTX instruction
 * st.mmio.relaxed.sys.global.u32 in inline assembly (:303, :481); an assembler macro of that name, defined
 * below, turns it into the plain 32-bit store it is.  <simt/atomic> comes from oracle/ref_shim.
 *
 * What it is for: tests let this code submit and complete commands against the emulated controller of the
 * library (queue memory and doorbells in host memory), which pins the controller's side of the protocol --
 * SQ entry consumption, completion layout, phase bit, SQ-head reporting, doorbell semantics -- against the
 * code the reference's GPU threads run.
 */
#include <pthread.h>
#include <time.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include <vector_types.h>          /* ulonglong4: the reference copies a command as two of them */

struct refpq_dim3 { unsigned x, y, z; };
static refpq_dim3 threadIdx = { 0, 0, 0 }, blockIdx = { 0, 0, 0 }, blockDim = { 1, 1, 1 };   /* named by the header's debug prints */

__asm__(".macro st.mmio.relaxed.sys.global.u32 addr, val\n"
        ".intel_syntax prefix\n"
        "mov DWORD PTR \\addr, \\val\n"
        ".att_syntax prefix\n"
        ".endm\n");

#include <nvm_types.h>
#include <nvm_util.h>
#include <nvm_cmd.h>
#include <nvm_queue.h>
#include <nvm_parallel_queue.h>

#define REFPQ_API extern "C" __attribute__((visibility("default")))

struct refpq_pair {
    nvm_ctrl_t ctrl;
    nvm_queue_t sq, cq;
    uint32_t ns_id;
    void* aux[5];
};

static padded_struct* zeroed(size_t n)
{
    void* p = nullptr;
    if (posix_memalign(&p, 64, n * sizeof(padded_struct)) != 0) return nullptr;
    memset(p, 0, n * sizeof(padded_struct));
    return static_cast<padded_struct*>(p);
}

/* A queue pair as QueuePair's constructor leaves it (include/queue.h:58-82, :89-221): descriptors from
 * nvm_queue_clear over caller memory, plus the zeroed per-slot arrays of the parallel protocol. */
REFPQ_API void* refpq_pair_new(void* mm_ptr, uint16_t no, uint32_t sq_qs, void* sq_vaddr, uint64_t sq_ioaddr, uint32_t cq_qs,
                               void* cq_vaddr, uint64_t cq_ioaddr, uint32_t ns_id)
{
    refpq_pair* p = static_cast<refpq_pair*>(calloc(1, sizeof(refpq_pair)));
    if (!p) return nullptr;
    p->ctrl.page_size = 4096; p->ctrl.dstrd = 0; p->ctrl.timeout = 5000; p->ctrl.max_qs = 1024;
    p->ctrl.mm_size = 0x2000; p->ctrl.mm_ptr = mm_ptr;
    p->ns_id = ns_id;
    if (nvm_queue_clear(&p->cq, &p->ctrl, true, no, cq_qs, true, cq_vaddr, cq_ioaddr) != 0 ||
        nvm_queue_clear(&p->sq, &p->ctrl, false, no, sq_qs, true, sq_vaddr, sq_ioaddr) != 0) { free(p); return nullptr; }
    p->sq.tickets = zeroed(sq_qs);       p->aux[0] = p->sq.tickets;
    p->sq.tail_mark = zeroed(sq_qs);     p->aux[1] = p->sq.tail_mark;
    p->sq.cid = zeroed(65536);           p->aux[2] = p->sq.cid;
    p->cq.head_mark = zeroed(cq_qs);     p->aux[3] = p->cq.head_mark;
    p->cq.pos_locks = zeroed(cq_qs);     p->aux[4] = p->cq.pos_locks;
    p->sq.qs_minus_1 = sq_qs - 1; p->cq.qs_minus_1 = cq_qs - 1;
    while ((1u << p->sq.qs_log2) < sq_qs) p->sq.qs_log2++;
    while ((1u << p->cq.qs_log2) < cq_qs) p->cq.qs_log2++;
    for (int i = 0; i < 5; i++) if (!p->aux[i]) return nullptr;
    return p;
}

REFPQ_API void refpq_pair_free(void* pair)
{
    refpq_pair* p = static_cast<refpq_pair*>(pair);
    for (int i = 0; i < 5; i++) free(p->aux[i]);
    free(p);
}

/* One blocking I/O: the queue calls of read_data (include/page_cache.h:2009-2054) in its order and with its
 * arguments; what read_data does besides (the page cache's own q_head / q_tail bookkeeping and its
 * enqueue_second) is not part of the queue protocol and is left out. */
static void one_io(refpq_pair* p, uint8_t opcode, uint64_t prp1, uint64_t start_lba, uint16_t n_blks)
{
    nvm_cmd_t cmd;
    memset(&cmd, 0, sizeof cmd);
    uint16_t cid = get_cid(&p->sq);
    nvm_cmd_header(&cmd, cid, opcode, p->ns_id);
    nvm_cmd_data_ptr(&cmd, prp1, 0);
    nvm_cmd_rw_blks(&cmd, start_lba, n_blks);
    sq_enqueue(&p->sq, &cmd);
    uint32_t head, head_;
    uint32_t cq_pos = cq_poll(&p->cq, cid, &head, &head_);
    cq_dequeue(&p->cq, (uint16_t)cq_pos, &p->sq, head, head_);
    put_cid(&p->sq, cid);
}

struct refpq_job {
    refpq_pair* pair;
    uint8_t opcode;
    const uint64_t* lbas;       /* request r: start block                        */
    const uint64_t* prps;       /* request r: bus address of its 4 KiB buffer    */
    uint16_t n_blks;
    uint64_t first, step, n;    /* this thread does requests first, first + step, ... < n */
    volatile uint64_t* done;
};

static void* worker(void* arg)
{
    refpq_job* j = static_cast<refpq_job*>(arg);
    for (uint64_t r = j->first; r < j->n; r += j->step) {
        one_io(j->pair, j->opcode, j->prps[r], j->lbas[r], j->n_blks);
        __atomic_fetch_add(j->done, 1, __ATOMIC_RELEASE);
    }
    return nullptr;
}

/* n requests issued by n_threads host threads sharing the queue pair, as the threads of a GPU kernel
 * share it.  Returns 0 when all completed, -1 when the time limit passed first (the reference's waits
 * have no limit of their own: the threads are then left behind, detached). */
REFPQ_API int refpq_run(void* pair, uint32_t n_threads, uint8_t opcode, const uint64_t* lbas, const uint64_t* prps, uint16_t n_blks,
                        uint64_t n, uint64_t timeout_ms)
{
    refpq_pair* p = static_cast<refpq_pair*>(pair);
    uint64_t* done = static_cast<uint64_t*>(calloc(1, sizeof(uint64_t)));
    refpq_job* jobs = static_cast<refpq_job*>(calloc(n_threads, sizeof(refpq_job)));
    pthread_t* th = static_cast<pthread_t*>(calloc(n_threads, sizeof(pthread_t)));
    for (uint32_t t = 0; t < n_threads; t++) {
        jobs[t] = { p, opcode, lbas, prps, n_blks, t, n_threads, n, done };
        if (pthread_create(&th[t], nullptr, worker, &jobs[t]) != 0) return -2;
    }
    struct timespec t0, t;
    clock_gettime(CLOCK_MONOTONIC, &t0);
    for (;;) {
        if (__atomic_load_n(done, __ATOMIC_ACQUIRE) == n) {
            for (uint32_t k = 0; k < n_threads; k++) pthread_join(th[k], nullptr);     /* they are on their way out */
            free(jobs); free(done); free(th);
            return 0;
        }
        clock_gettime(CLOCK_MONOTONIC, &t);
        const uint64_t ms = (uint64_t)(t.tv_sec - t0.tv_sec) * 1000ull + (uint64_t)((t.tv_nsec - t0.tv_nsec) / 1000000);
        if (ms > timeout_ms) {
            /* the workers may be spinning for good and still use jobs and done: leave everything to them */
            for (uint32_t k = 0; k < n_threads; k++) pthread_detach(th[k]);
            return -1;
        }
        struct timespec nap = { 0, 200000 };
        nanosleep(&nap, nullptr);
    }
}

/* Where the reference's descriptors stand afterwards (for consistency checks). */
REFPQ_API void refpq_state(void* pair, uint32_t* sq_head, uint32_t* sq_tail, uint32_t* cq_head, uint32_t* cq_tail, uint32_t* in_ticket)
{
    refpq_pair* p = static_cast<refpq_pair*>(pair);
    *sq_head = p->sq.head.load(); *sq_tail = p->sq.tail.load();
    *cq_head = p->cq.head.load(); *cq_tail = p->cq.tail.load();
    *in_ticket = p->sq.in_ticket.load();
}
