/*
 * bam_nvm_host.cu -- the reference's host-side libnvm interface over the emulated controller
 * (declarations and the meaning of every name: include/nvm_host_api.h).
 *
 * A handle owns: the register window (one page of pinned, mapped host memory holding the doorbell
 * registers at their NVMe offsets), a table of host-driven queue pairs in the format the command
 * processor consumes (bam_emu_qp_t, with queue memory and doorbells in mapped host memory), and the
 * service kernel that runs the command processor for those queue pairs until it is told to stop.
 * Everything the host shares with that kernel is synchronised at system scope.
 */
#include <cuda_runtime.h>

#include <cerrno>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <ctime>
#include <mutex>
#include <new>
#include <vector>

#include "bam/emu_ctrl.cuh"
#include "bam_internal.h"
#include "nvm_host_api.h"

#define NVM_HOST_MAX_QUEUES 64                 /* host-driven queue pairs per handle            */
#define NVM_HOST_SERVICE_BLOCKS 2              /* command-processor blocks of the service kernel */
#define NVM_HOST_MAX_WINDOWS 256               /* DMA mappings whose memory commands may name      */

namespace {

struct host_ctrl;
struct dma_backing {                            /* what a mapping pinned or allocated; shared with its remaps */
    int refs = 1;
    void* registered = nullptr;                 /* memory pinned with cudaHostRegister              */
    void* allocated = nullptr;                  /* memory allocated with cudaHostAlloc              */
};
struct host_dma {                               /* container of an nvm_dma_t (the public part comes last) */
    host_ctrl* owner = nullptr;
    dma_backing* backing = nullptr;             /* nullptr: the caller's memory, nothing to release  */
    bool device = false;
    bool page_windows = false;                  /* one DMA window per page (a list of addresses) instead of one for the region */
};

struct host_ctrl {
    nvm_ctrl_t pub;                             /* must stay the first member: handles are cast back */
    bam_ctrl* emu = nullptr;
    std::mutex lock;
    int refs = 1;                               /* handles given out for this controller (guarded by g_handles_lock) */
    uint8_t* regs_raw = nullptr;                /* the allocation the register window lies in        */
    uint8_t* regs_host = nullptr;               /* register window                                   */
    uint8_t* regs_dev = nullptr;
    uint32_t* stop_host = nullptr;              /* 1 while the service should run (inside the window) */
    bam_emu_qp_t* d_qps = nullptr;              /* [NVM_HOST_MAX_QUEUES]                              */
    bam_emu_qp_t h_qps[NVM_HOST_MAX_QUEUES];
    bool have_cq[NVM_HOST_MAX_QUEUES + 1] = {};
    bool have_sq[NVM_HOST_MAX_QUEUES + 1] = {};
    nvm_cpl_t* cq_mem_dev[NVM_HOST_MAX_QUEUES + 1] = {};
    uint32_t cq_qs[NVM_HOST_MAX_QUEUES + 1] = {};
    uint32_t n_qps = 0;
    bam_status_t* d_status = nullptr;
    bam_fault_t* d_fault = nullptr;
    uint64_t* d_served = nullptr;
    cudaStream_t stream = nullptr;
    bool running = false;
    uint16_t granted_cqs = NVM_HOST_MAX_QUEUES, granted_sqs = NVM_HOST_MAX_QUEUES;
    bam_dma_window_t windows[NVM_HOST_MAX_WINDOWS];
    uint32_t n_windows = 0;
    bam_dma_window_t* d_windows = nullptr;
};

struct nvm_dma_box { host_dma priv; nvm_dma_t pub; };

host_ctrl* of(const nvm_ctrl_t* c) { return reinterpret_cast<host_ctrl*>(const_cast<nvm_ctrl_t*>(c)); }

std::mutex g_handles_lock;                      /* live handles, so that a register window can be recognised */
std::vector<host_ctrl*> g_handles;

__global__ void __launch_bounds__(BAM_THREADS, 1) k_nvm_host_service(const __grid_constant__ bam_emu_d_t emu)
{
    extern __shared__ __align__(128) uint8_t smem[];
    bam::emu_controller_main(emu, smem);
}

/* device-visible address of host memory that is already pinned, or 0 */
uint64_t device_address_of_host(void* p)
{
    void* d = nullptr;
    if (cudaHostGetDevicePointer(&d, p, 0) != cudaSuccess) { (void)cudaGetLastError(); return 0; }
    return (uint64_t)(uintptr_t)d;
}

int stop_service_locked(host_ctrl* h)
{
    if (!h->running) return 0;
    __atomic_store_n(h->stop_host, 0u, __ATOMIC_RELEASE);
    cudaError_t e = cudaStreamSynchronize(h->stream);
    h->running = false;
    /* keep where every queue stands (fetch position, completion tail) for the next start */
    if (e == cudaSuccess && h->n_qps) e = cudaMemcpy(h->h_qps, h->d_qps, sizeof(bam_emu_qp_t) * h->n_qps, cudaMemcpyDeviceToHost);
    return e == cudaSuccess ? 0 : EIO;
}

int start_service_locked(host_ctrl* h)
{
    if (h->running) return 0;
    if (h->n_qps == 0) return 0;
    if (cudaSetDevice(h->emu->device) != cudaSuccess) return EIO;
    if (cudaMemcpy(h->d_qps, h->h_qps, sizeof(bam_emu_qp_t) * h->n_qps, cudaMemcpyHostToDevice) != cudaSuccess) return EIO;
    bam_status_t st;
    memset(&st, 0, sizeof st);
    st.spin_timeout_ns = h->emu->spin_timeout_ns;
    st.launch_timeout_ns = h->emu->launch_timeout_ns;
    if (cudaMemcpy(h->d_status, &st, sizeof st, cudaMemcpyHostToDevice) != cudaSuccess) return EIO;
    __atomic_store_n(h->stop_host, 1u, __ATOMIC_RELEASE);
    bam_emu_d_t emu;
    memset(&emu, 0, sizeof emu);
    emu.qps = h->d_qps; emu.n_qps = h->n_qps;
    emu.n_ctrl_blocks = NVM_HOST_SERVICE_BLOCKS;
    emu.lba_log2 = h->emu->emu.lba_log2; emu.mps_log2 = 12;
    emu.batch = 32; emu.sys_scope = 1;
    emu.consumers_remaining = reinterpret_cast<uint32_t*>(h->regs_dev + (reinterpret_cast<uint8_t*>(h->stop_host) - h->regs_host));
    emu.status = h->d_status;
    /* the data pointers of host-submitted commands are checked against the memory mapped for DMA */
    if (cudaMemcpy(h->d_windows, h->windows, sizeof(bam_dma_window_t) * NVM_HOST_MAX_WINDOWS, cudaMemcpyHostToDevice) != cudaSuccess) return EIO;
    emu.windows = h->d_windows; emu.n_windows = h->n_windows;
#ifdef BAM_NVM_DEBUG          /* a build-time aid: dumps every pointer the service kernel is handed */
    {
        auto show = [](const char* what, const void* p) {
            cudaPointerAttributes a;
            cudaError_t e = cudaPointerGetAttributes(&a, p);
            fprintf(stderr, "[nvm] %-22s %p  type %d (err %d) dev %p host %p\n", what, p, e == cudaSuccess ? (int)a.type : -1, (int)e,
                    e == cudaSuccess ? a.devicePointer : nullptr, e == cudaSuccess ? a.hostPointer : nullptr);
            (void)cudaGetLastError();
        };
        show("qps table", emu.qps); show("status", emu.status); show("stop flag", emu.consumers_remaining); show("windows", emu.windows);
        for (uint32_t q = 0; q < h->n_qps; q++) {
            const bam_emu_qp_t& e = h->h_qps[q];
            show("sq_mem", e.sq_mem); show("cq_mem", e.cq_mem); show("sq_db", e.sq_db); show("cq_db", e.cq_db);
            show("store", e.store); show("fault", e.fault); show("served", e.served);
            fprintf(stderr, "[nvm] qp %u: qs %u cq_qs %u sqid %u cqid %u store_bytes %llu fetch %u cq_tail %u\n", q, e.qs, e.cq_qs, e.sqid, e.cqid,
                    (unsigned long long)e.store_bytes, e.sq_fetch, e.cq_tail);
        }
        for (uint32_t k = 0; k < h->n_windows; k++)
            fprintf(stderr, "[nvm] window %u: %p + %llu\n", k, (void*)(uintptr_t)h->windows[k].base, (unsigned long long)h->windows[k].bytes);
    }
#endif
    if (cudaFuncSetAttribute(k_nvm_host_service, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)BAM_EMU_SMEM_BYTES) != cudaSuccess) return EIO;
    k_nvm_host_service<<<NVM_HOST_SERVICE_BLOCKS, BAM_THREADS, BAM_EMU_SMEM_BYTES, h->stream>>>(emu);
    if (cudaGetLastError() != cudaSuccess) return EIO;
    h->running = true;
    return 0;
}

/* Pinning, allocating and freeing memory can make the CUDA runtime wait for the device to go idle,
 * which a running service kernel never is: such calls are made with the service paused. */
struct pause_guard {
    host_ctrl* h;
    bool was_running;
    explicit pause_guard(host_ctrl* c) : h(c), was_running(false)
    {
        h->lock.lock();
        cudaSetDevice(h->emu->device);
        was_running = h->running;
        if (was_running) stop_service_locked(h);
    }
    ~pause_guard()
    {
        if (was_running) start_service_locked(h);
        h->lock.unlock();
    }
};

/* The read-only registers a program may look at, at their NVMe offsets: CAP (0x00: MQES 15:0, CQR 16,
 * TO 31:24 in 500 ms units, DSTRD 35:32, CSS 37 = NVM command set, MPSMIN 51:48, MPSMAX 55:52),
 * VS (0x08) = 1.4, CC (0x14: EN 0, MPS 10:7, IOSQES 19:16 = 6, IOCQES 23:20 = 4), CSTS (0x1c: RDY 0),
 * AQA / ASQ / ACQ (0x24 / 0x28 / 0x30). */
void write_registers(host_ctrl* h, uint64_t asq, uint64_t acq)
{
    const uint64_t cap = (uint64_t)(h->pub.max_qs - 1) | (1ull << 16) | ((h->pub.timeout / 500) << 24) | ((uint64_t)h->pub.dstrd << 32) |
                         (1ull << 37);
    *reinterpret_cast<volatile uint64_t*>(h->regs_host + 0x00) = cap;
    *reinterpret_cast<volatile uint32_t*>(h->regs_host + 0x08) = 0x00010400u;
    *reinterpret_cast<volatile uint32_t*>(h->regs_host + 0x14) = 1u | (6u << 16) | (4u << 20);
    *reinterpret_cast<volatile uint32_t*>(h->regs_host + 0x1c) = 1u;
    *reinterpret_cast<volatile uint32_t*>(h->regs_host + 0x24) = ((uint32_t)(h->pub.page_size / 16 - 1) << 16) | (uint32_t)(h->pub.page_size / 64 - 1);
    *reinterpret_cast<volatile uint64_t*>(h->regs_host + 0x28) = asq;
    *reinterpret_cast<volatile uint64_t*>(h->regs_host + 0x30) = acq;
}

/* rebuild the table the service kernel reads: one entry per complete (CQ, SQ) pair */
void rebuild_table(host_ctrl* h)
{
    h->n_qps = 0;
    for (uint16_t id = 1; id <= NVM_HOST_MAX_QUEUES; id++)
        if (h->have_sq[id]) h->n_qps++;
}

}  // namespace

extern "C" int nvm_ctrl_init(nvm_ctrl_t** ctrl, int)
{
    if (ctrl) *ctrl = nullptr;
    return ENODEV;                     /* no kernel module, no raw SSD: use nvm_emu_ctrl_init */
}

extern "C" int nvm_emu_ctrl_init(nvm_ctrl_t** ctrl, bam_ctrl_t emu)
{
    if (!ctrl) return EINVAL;
    *ctrl = nullptr;
    if (!emu) return EINVAL;
    if (cudaSetDevice(emu->device) != cudaSuccess) { (void)cudaGetLastError(); return ENODEV; }
    host_ctrl* h = new (std::nothrow) host_ctrl();
    if (!h) return ENOMEM;
    h->emu = emu;
    h->pub.page_size = 4096;
    h->pub.dstrd = 0;
    h->pub.timeout = 5000;
    h->pub.max_qs = 1024;
    h->pub.mm_size = 0x2000;
    cudaError_t e = cudaHostAlloc((void**)&h->regs_raw, h->pub.mm_size + 4096, cudaHostAllocMapped | cudaHostAllocPortable);
    if (e == cudaSuccess) {
        h->regs_host = reinterpret_cast<uint8_t*>(((uintptr_t)h->regs_raw + 4095) / 4096 * 4096);     /* a register window starts on a page */
        e = cudaHostGetDevicePointer((void**)&h->regs_dev, h->regs_host, 0);
    }
    if (e == cudaSuccess) e = cudaMalloc(&h->d_qps, sizeof(bam_emu_qp_t) * NVM_HOST_MAX_QUEUES);
    if (e == cudaSuccess) e = cudaMalloc(&h->d_status, sizeof(bam_status_t));
    if (e == cudaSuccess) e = cudaMalloc(&h->d_fault, sizeof(bam_fault_t));
    if (e == cudaSuccess) e = cudaMalloc(&h->d_served, 8);
    if (e == cudaSuccess) e = cudaMalloc(&h->d_windows, sizeof(bam_dma_window_t) * NVM_HOST_MAX_WINDOWS);
    if (e == cudaSuccess) e = cudaMemset(h->d_fault, 0, sizeof(bam_fault_t));
    if (e == cudaSuccess) e = cudaMemset(h->d_served, 0, 8);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&h->stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        cudaFreeHost(h->regs_raw); cudaFree(h->d_qps); cudaFree(h->d_status); cudaFree(h->d_fault); cudaFree(h->d_served); cudaFree(h->d_windows);
        delete h;
        return ENOMEM;
    }
    memset(h->regs_host, 0, h->pub.mm_size);
    h->pub.mm_ptr = h->regs_host;
    h->stop_host = reinterpret_cast<uint32_t*>(h->regs_host + 0x40);    /* a word of the window the NVMe layout leaves unused */
    memset(h->h_qps, 0, sizeof h->h_qps);
    write_registers(h, 0, 0);
    {
        std::lock_guard<std::mutex> g(g_handles_lock);
        g_handles.push_back(h);
    }
    *ctrl = &h->pub;
    return 0;
}

/* The reference reads the controller's capabilities from a memory-mapped PCI BAR; here the only
 * register windows that exist are those of emulated controllers, which this call recognises by
 * address and hands out again (nvm_ctrl_free counts the handles). */
extern "C" int nvm_raw_ctrl_init(nvm_ctrl_t** ctrl, volatile void* mm_ptr, size_t mm_size)
{
    if (!ctrl) return EINVAL;
    *ctrl = nullptr;
    if (!mm_ptr || mm_size < NVM_CTRL_MEM_MINSIZE) return EINVAL;
    std::lock_guard<std::mutex> g(g_handles_lock);
    for (host_ctrl* h : g_handles)
        if (h->pub.mm_ptr == mm_ptr) {
            /* what the reference derives from CAP: page size from MPSMIN, stride from DSTRD, time-out from TO, entries from MQES */
            const uint64_t cap = *reinterpret_cast<volatile uint64_t*>(h->regs_host);
            if (h->pub.page_size != ((size_t)1 << (12 + ((cap >> 48) & 0xf))) || h->pub.dstrd != ((cap >> 32) & 0xf) ||
                h->pub.timeout != ((cap >> 24) & 0xff) * 500 || h->pub.max_qs != (cap & 0xffff) + 1)
                return EIO;
            h->refs++;
            *ctrl = &h->pub;
            return 0;
        }
    return ENODEV;
}

/* Controller reset with new admin queue addresses (controller pages): every I/O queue pair is
 * deleted, the doorbells are cleared and the admin queue registers take the addresses. */
extern "C" int nvm_raw_ctrl_reset(const nvm_ctrl_t* ctrl, uint64_t acq_ioaddr, uint64_t asq_ioaddr)
{
    if (!ctrl) return EINVAL;
    host_ctrl* h = of(ctrl);
    if ((acq_ioaddr | asq_ioaddr) & (ctrl->page_size - 1)) return EINVAL;
    std::lock_guard<std::mutex> g(h->lock);
    cudaSetDevice(h->emu->device);
    const int rc = stop_service_locked(h);
    for (uint16_t id = 0; id <= NVM_HOST_MAX_QUEUES; id++) h->have_cq[id] = h->have_sq[id] = false;
    h->n_qps = 0;
    memset(h->h_qps, 0, sizeof h->h_qps);
    memset(h->regs_host, 0, h->pub.mm_size);
    write_registers(h, asq_ioaddr, acq_ioaddr);
    return rc;
}

extern "C" void nvm_ctrl_free(nvm_ctrl_t* ctrl)
{
    if (!ctrl) return;
    host_ctrl* h = of(ctrl);
    {
        std::lock_guard<std::mutex> g(g_handles_lock);
        if (--h->refs > 0) return;                         /* nvm_raw_ctrl_init handed the controller out more than once */
        for (size_t i = 0; i < g_handles.size(); i++)
            if (g_handles[i] == h) { g_handles[i] = g_handles.back(); g_handles.pop_back(); break; }
    }
    {
        std::lock_guard<std::mutex> g(h->lock);
        cudaSetDevice(h->emu->device);
        stop_service_locked(h);
    }
    cudaStreamDestroy(h->stream);
    cudaFreeHost(h->regs_raw); cudaFree(h->d_qps); cudaFree(h->d_status); cudaFree(h->d_fault); cudaFree(h->d_served); cudaFree(h->d_windows);
    delete h;
}

extern "C" int nvm_emu_service_start(const nvm_ctrl_t* ctrl)
{
    if (!ctrl) return EINVAL;
    host_ctrl* h = of(ctrl);
    std::lock_guard<std::mutex> g(h->lock);
    return start_service_locked(h);
}

extern "C" int nvm_emu_service_stop(const nvm_ctrl_t* ctrl)
{
    if (!ctrl) return EINVAL;
    host_ctrl* h = of(ctrl);
    std::lock_guard<std::mutex> g(h->lock);
    cudaSetDevice(h->emu->device);
    return stop_service_locked(h);
}

extern "C" int nvm_emu_service_status(const nvm_ctrl_t* ctrl, uint32_t* running, uint32_t* code, uint32_t* where, uint64_t* served)
{
    if (!ctrl) return EINVAL;
    host_ctrl* h = of(ctrl);
    std::lock_guard<std::mutex> g(h->lock);
    if (cudaSetDevice(h->emu->device) != cudaSuccess) return EIO;
    /* has the kernel left on its own (time limit, recorded error) or failed? */
    if (h->running) {
        const cudaError_t q = cudaStreamQuery(h->stream);
        if (q == cudaSuccess) h->running = false;
        else if (q != cudaErrorNotReady) { (void)cudaGetLastError(); h->running = false; if (running) *running = 0; return 1000 + (int)q; }
    }
    if (running) *running = h->running ? 1u : 0u;
    /* the service kernel may be running: read on a stream of our own, not on the legacy default stream */
    bam_status_t st;
    uint64_t n = 0;
    cudaStream_t s = nullptr;
    cudaError_t e = cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaMemcpyAsync(&st, h->d_status, sizeof st, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(&n, h->d_served, 8, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (s) cudaStreamDestroy(s);
    if (e != cudaSuccess) { (void)cudaGetLastError(); return 1000 + (int)e; }
    if (code) *code = st.code;
    if (where) *where = st.where;
    if (served) *served = n;
    return 0;
}

/* ---- DMA mappings ---------------------------------------------------------------------------------- */

static int make_map(nvm_dma_t** map, void* vaddr, size_t page_size, size_t n_pages, uint64_t base, const uint64_t* ioaddrs,
                    const host_dma& priv, bool local)
{
    nvm_dma_box* box = static_cast<nvm_dma_box*>(calloc(1, sizeof(nvm_dma_box) + n_pages * sizeof(uint64_t)));
    if (!box) return ENOMEM;
    new (&box->priv) host_dma(priv);
    box->priv.page_windows = ioaddrs != nullptr;
    box->pub.vaddr = vaddr;
    box->pub.local = local;
    box->pub.contiguous = 1;
    box->pub.page_size = page_size;
    box->pub.n_ioaddrs = n_pages;
    for (size_t i = 0; i < n_pages; i++) box->pub.ioaddrs[i] = ioaddrs ? ioaddrs[i] : base + i * page_size;
    /* commands may name this memory from now on (a mapping given as a list of pages counts page by page) */
    host_ctrl* h = priv.owner;
    if (h) {
        const size_t n_w = ioaddrs ? n_pages : 1;
        if (h->n_windows + n_w > NVM_HOST_MAX_WINDOWS) { free(box); return ENOSPC; }
        for (size_t i = 0; i < n_w; i++) {
            h->windows[h->n_windows].base = ioaddrs ? ioaddrs[i] : base;
            h->windows[h->n_windows].bytes = ioaddrs ? page_size : n_pages * page_size;
            h->n_windows++;
        }
    }
    *map = &box->pub;
    return 0;
}

static nvm_dma_box* box_of(const nvm_dma_t* map)
{
    return reinterpret_cast<nvm_dma_box*>(reinterpret_cast<uint8_t*>(const_cast<nvm_dma_t*>(map)) - offsetof(nvm_dma_box, pub));
}

extern "C" int nvm_dma_map(nvm_dma_t** map, const nvm_ctrl_t* ctrl, void* vaddr, size_t page_size, size_t n_pages, const uint64_t* ioaddrs)
{
    if (!map) return EINVAL;
    *map = nullptr;
    if (!ctrl || !ioaddrs || n_pages == 0 || page_size == 0) return EINVAL;
    pause_guard pause(of(ctrl));                       /* the service picks the new windows up when it resumes */
    host_dma priv;
    priv.owner = of(ctrl);
    return make_map(map, vaddr, page_size, n_pages, 0, ioaddrs, priv, true);
}

/* A second descriptor of the same memory.  What the first one pinned or allocated stays until the
 * last of them is unmapped. */
extern "C" int nvm_dma_remap(nvm_dma_t** new_map, const nvm_dma_t* other_map)
{
    if (!new_map) return EINVAL;
    *new_map = nullptr;
    if (!other_map) return EINVAL;
    nvm_dma_box* other = box_of(other_map);
    if (!other->priv.owner) return EINVAL;
    pause_guard pause(other->priv.owner);
    host_dma priv = other->priv;
    const int rc = make_map(new_map, other_map->vaddr, other_map->page_size, other_map->n_ioaddrs, other_map->ioaddrs[0],
                            other->priv.page_windows ? other_map->ioaddrs : nullptr, priv, other_map->local != 0);
    if (rc == 0 && priv.backing) priv.backing->refs++;
    return rc;
}

extern "C" int nvm_dma_map_host(nvm_dma_t** map, const nvm_ctrl_t* ctrl, void* vaddr, size_t size)
{
    if (!map) return EINVAL;
    *map = nullptr;
    if (!ctrl || !vaddr || size == 0) return EINVAL;
    const size_t ps = ctrl->page_size;
    if (((uintptr_t)vaddr & (ps - 1)) != 0) return EINVAL;
    pause_guard pause(of(ctrl));
    host_dma priv;
    priv.owner = of(ctrl);
    uint64_t dev = device_address_of_host(vaddr);
    if (dev == 0) {                                   /* not pinned yet: pin and map it */
        cudaError_t e = cudaHostRegister(vaddr, size, cudaHostRegisterMapped | cudaHostRegisterPortable);
        if (e != cudaSuccess) { (void)cudaGetLastError(); return EFAULT; }
        dev = device_address_of_host(vaddr);
        priv.backing = dev ? new (std::nothrow) dma_backing() : nullptr;
        if (!priv.backing) { cudaHostUnregister(vaddr); return dev ? ENOMEM : EFAULT; }
        priv.backing->registered = vaddr;
    }
    int rc = make_map(map, vaddr, ps, (size + ps - 1) / ps, dev, nullptr, priv, true);
    if (rc && priv.backing) { cudaHostUnregister(vaddr); delete priv.backing; }
    return rc;
}

extern "C" int nvm_dma_map_device(nvm_dma_t** map, const nvm_ctrl_t* ctrl, void* devptr, size_t size)
{
    if (!map) return EINVAL;
    *map = nullptr;
    if (!ctrl || !devptr || size == 0) return EINVAL;
    const size_t ps = ctrl->page_size;
    if (((uintptr_t)devptr & (ps - 1)) != 0) return EINVAL;
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, devptr) != cudaSuccess || attr.type != cudaMemoryTypeDevice) { (void)cudaGetLastError(); return EINVAL; }
    pause_guard pause(of(ctrl));
    host_dma priv;
    priv.owner = of(ctrl);
    priv.device = true;
    return make_map(map, devptr, ps, (size + ps - 1) / ps, (uint64_t)(uintptr_t)devptr, nullptr, priv, false);
}

extern "C" int nvm_dma_create(nvm_dma_t** map, const nvm_ctrl_t* ctrl, size_t size)
{
    if (!map) return EINVAL;
    *map = nullptr;
    if (!ctrl || size == 0) return EINVAL;
    const size_t ps = ctrl->page_size;
    size = (size + ps - 1) / ps * ps;
    pause_guard pause(of(ctrl));
    /* pinned allocations come with the allocator's own alignment (512 bytes for small ones), DMA memory is
     * page-granular: allocate one page more and start at the first page boundary */
    void* raw = nullptr;
    if (cudaHostAlloc(&raw, size + ps, cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) { (void)cudaGetLastError(); return ENOMEM; }
    void* p = reinterpret_cast<void*>(((uintptr_t)raw + ps - 1) / ps * ps);
    memset(p, 0, size);
    host_dma priv;
    priv.owner = of(ctrl);
    priv.backing = new (std::nothrow) dma_backing();
    if (!priv.backing) { cudaFreeHost(raw); return ENOMEM; }
    priv.backing->allocated = raw;
    const uint64_t dev = device_address_of_host(p);
    int rc = (dev && (dev & (ps - 1)) == 0) ? make_map(map, p, ps, size / ps, dev, nullptr, priv, true) : EFAULT;
    if (rc) { cudaFreeHost(raw); delete priv.backing; }
    return rc;
}

extern "C" void nvm_dma_unmap(nvm_dma_t* map)
{
    if (!map) return;
    nvm_dma_box* box = box_of(map);
    host_ctrl* h = box->priv.owner;
    if (h) {
        pause_guard pause(h);
        /* the memory may no longer be named by commands -- unless another descriptor still maps it:
         * exactly the windows this descriptor added are taken out, one entry each */
        const size_t n_w = box->priv.page_windows ? map->n_ioaddrs : 1;
        for (size_t i = 0; i < n_w; i++) {
            const uint64_t bytes = box->priv.page_windows ? map->page_size : map->n_ioaddrs * map->page_size;
            for (uint32_t k = 0; k < h->n_windows; k++)
                if (h->windows[k].base == map->ioaddrs[i] && h->windows[k].bytes == bytes) { h->windows[k] = h->windows[--h->n_windows]; break; }
        }
        dma_backing* b = box->priv.backing;
        if (b && --b->refs == 0) {
            if (b->registered) cudaHostUnregister(b->registered);
            if (b->allocated) cudaFreeHost(b->allocated);
            delete b;
        }
    }
    free(box);
}

extern "C" const nvm_ctrl_t* nvm_ctrl_from_dma(const nvm_dma_t* dma)
{
    if (!dma) return nullptr;
    host_ctrl* h = box_of(dma)->priv.owner;
    return h ? &h->pub : nullptr;
}

/* ---- status text ------------------------------------------------------------------------------------ */

/* Names of the NVMe completion statuses a program is likely to meet, by status code type (0 generic,
 * 1 command specific, 2 media and data integrity) and status code (reference: src/error.cpp:139-182
 * maps the same packing to text). */
extern "C" const char* nvm_strerror(int status)
{
    if (status == 0) return "success";
    if (status > 0) {
        switch (status) {
        case BAM_EIO: case BAM_E2BIG: case BAM_ENOMEM: case BAM_EBUSY: case BAM_EINVAL: case BAM_ENOSPC: case BAM_ERANGE: case BAM_ETIMEDOUT:
        case BAM_ECUDA: return bam_strerror(status);
        default: return strerror(status);
        }
    }
    const unsigned sct = ((unsigned)(-status) >> 8) & 0xff, sc = (unsigned)(-status) & 0xff;
    if (sct == 0) {
        switch (sc) {
        case 0x00: return "NVMe: successful completion";
        case 0x01: return "NVMe: invalid command opcode";
        case 0x02: return "NVMe: invalid field in command";
        case 0x03: return "NVMe: command identifier conflict";
        case 0x04: return "NVMe: data transfer error";
        case 0x05: return "NVMe: aborted, power loss notification";
        case 0x06: return "NVMe: internal controller error";
        case 0x07: return "NVMe: abort requested";
        case 0x08: return "NVMe: aborted, submission queue deleted";
        case 0x0b: return "NVMe: invalid namespace or format";
        case 0x0c: return "NVMe: command sequence error";
        case 0x13: return "NVMe: PRP offset invalid";
        case 0x80: return "NVMe: LBA out of range";
        case 0x81: return "NVMe: capacity exceeded";
        case 0x82: return "NVMe: namespace not ready";
        default: return "NVMe: generic command status";
        }
    }
    if (sct == 1) {
        switch (sc) {
        case 0x00: return "NVMe: completion queue invalid";
        case 0x01: return "NVMe: invalid queue identifier";
        case 0x02: return "NVMe: invalid queue size";
        case 0x0c: return "NVMe: invalid queue deletion";
        default: return "NVMe: command specific status";
        }
    }
    if (sct == 2) {
        switch (sc) {
        case 0x80: return "NVMe: write fault";
        case 0x81: return "NVMe: unrecovered read error";
        case 0x85: return "NVMe: compare failure";
        case 0x86: return "NVMe: access denied";
        default: return "NVMe: media or data integrity error";
        }
    }
    return "NVMe: unknown status code type";
}

/* ---- admin ---------------------------------------------------------------------------------------------- */

struct nvm_admin_reference { host_ctrl* h; };

extern "C" int nvm_aq_create(nvm_aq_ref* ref, const nvm_ctrl_t* ctrl, const nvm_dma_t*)
{
    if (!ref) return EINVAL;
    *ref = nullptr;
    if (!ctrl) return EINVAL;
    nvm_admin_reference* r = new (std::nothrow) nvm_admin_reference();
    if (!r) return ENOMEM;
    r->h = of(ctrl);
    *ref = r;
    return 0;
}

extern "C" void nvm_aq_destroy(nvm_aq_ref ref) { delete ref; }

extern "C" const nvm_ctrl_t* nvm_ctrl_from_aq_ref(nvm_aq_ref ref) { return ref ? &ref->h->pub : nullptr; }

/* References to a remote machine's admin queues do not exist here: every reference is local, and
 * unbinding a local reference does nothing. */
extern "C" void nvm_rpc_unbind(nvm_aq_ref) {}

/* ---- the controller's side of the admin commands ------------------------------------------------------
 * What an NVMe controller does when it executes an admin command, as functions over the handle's state.
 * They return an NVMe status (status code | status code type << 8; 0 = success).  h->lock is held. */

#define ADM_SC_INVALID_OPCODE 0x001u
#define ADM_SC_INVALID_FIELD 0x002u
#define ADM_SC_DATA_XFER 0x004u
#define ADM_SC_INVALID_NS 0x00bu
#define ADM_SC_CQ_INVALID 0x100u
#define ADM_SC_QID_INVALID 0x101u
#define ADM_SC_QSIZE_INVALID 0x102u
#define ADM_SC_LOG_PAGE_INVALID 0x109u
#define ADM_SC_QUEUE_DELETION 0x10cu

static uint32_t log2_of(uint32_t x) { uint32_t l = 0; while ((1u << l) < x) l++; return l; }

/* host pointer behind a bus address that lies, with `bytes` bytes, inside memory mapped for this controller;
 * *device is set when the memory is GPU memory (then the returned pointer is the device pointer) */
static void* admin_memory(host_ctrl* h, uint64_t ioaddr, size_t bytes, bool* device)
{
    bool ok = false;
    for (uint32_t k = 0; k < h->n_windows && !ok; k++)
        ok = ioaddr >= h->windows[k].base && ioaddr + bytes <= h->windows[k].base + h->windows[k].bytes;
    if (!ok) return nullptr;
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, reinterpret_cast<void*>((uintptr_t)ioaddr)) != cudaSuccess) { (void)cudaGetLastError(); return nullptr; }
    *device = attr.type == cudaMemoryTypeDevice;
    if (*device) return attr.devicePointer;
    return attr.type == cudaMemoryTypeHost ? attr.hostPointer : nullptr;
}

static uint32_t ctrl_cq_create(host_ctrl* h, uint32_t id, uint32_t qs, uint64_t dev)
{
    if (id == 0 || id > NVM_HOST_MAX_QUEUES || id > h->granted_cqs || h->have_cq[id]) return ADM_SC_QID_INVALID;
    if (qs < 2 || qs > h->pub.max_qs || (qs & (qs - 1))) return ADM_SC_QSIZE_INVALID;      /* the command processor wants a power of two */
    h->have_cq[id] = true;
    h->cq_mem_dev[id] = reinterpret_cast<nvm_cpl_t*>((uintptr_t)dev);
    h->cq_qs[id] = qs;
    return 0;
}

static uint32_t ctrl_sq_create(host_ctrl* h, uint32_t id, uint32_t cqid, uint32_t qs, uint64_t dev, int* host_error)
{
    if (id == 0 || id > NVM_HOST_MAX_QUEUES || id > h->granted_sqs || h->have_sq[id]) return ADM_SC_QID_INVALID;
    if (cqid == 0 || cqid > NVM_HOST_MAX_QUEUES || !h->have_cq[cqid]) return ADM_SC_CQ_INVALID;
    if (qs < 2 || qs > h->pub.max_qs || (qs & (qs - 1))) return ADM_SC_QSIZE_INVALID;
    cudaSetDevice(h->emu->device);
    if ((*host_error = stop_service_locked(h)) != 0) return 0;
    uint32_t slot = 0;                                     /* position in the table = creation order */
    for (uint16_t k = 1; k <= NVM_HOST_MAX_QUEUES; k++) if (h->have_sq[k]) slot++;
    bam_emu_qp_t* e = &h->h_qps[slot];
    memset(e, 0, sizeof *e);
    e->sq_mem = reinterpret_cast<nvm_cmd_t*>((uintptr_t)dev);
    e->cq_mem = h->cq_mem_dev[cqid];
    e->sq_db = reinterpret_cast<uint32_t*>(h->regs_dev + NVM_SQ_DBL_OFFSET(id, h->pub.dstrd));
    e->cq_db = reinterpret_cast<uint32_t*>(h->regs_dev + NVM_CQ_DBL_OFFSET(cqid, h->pub.dstrd));
    e->qs = qs; e->qs_log2 = log2_of(qs);
    e->cq_qs = h->cq_qs[cqid]; e->cq_qs_log2 = log2_of(e->cq_qs);
    e->sqid = (uint16_t)id; e->cqid = (uint16_t)cqid;
    e->store = h->emu->store_dev; e->store_bytes = h->emu->store_bytes;
    e->fault = h->d_fault; e->served = h->d_served;
    *reinterpret_cast<volatile uint32_t*>(h->regs_host + NVM_SQ_DBL_OFFSET(id, h->pub.dstrd)) = 0;
    *reinterpret_cast<volatile uint32_t*>(h->regs_host + NVM_CQ_DBL_OFFSET(cqid, h->pub.dstrd)) = 0;
    h->have_sq[id] = true;
    rebuild_table(h);
    *host_error = start_service_locked(h);
    return 0;
}

static uint32_t ctrl_cq_delete(host_ctrl* h, uint32_t id)
{
    if (id == 0 || id > NVM_HOST_MAX_QUEUES || !h->have_cq[id]) return ADM_SC_QID_INVALID;
    for (uint32_t k = 0; k < h->n_qps; k++)
        if (h->h_qps[k].cqid == id) return ADM_SC_QUEUE_DELETION;           /* a submission queue still completes into it */
    h->have_cq[id] = false;
    return 0;
}

static uint32_t ctrl_sq_delete(host_ctrl* h, uint32_t id, int* host_error)
{
    if (id == 0 || id > NVM_HOST_MAX_QUEUES || !h->have_sq[id]) return ADM_SC_QID_INVALID;
    cudaSetDevice(h->emu->device);
    *host_error = stop_service_locked(h);
    /* close the gap in the table */
    uint32_t slot = 0, n = 0;
    for (uint16_t k = 1; k <= NVM_HOST_MAX_QUEUES; k++) { if (k == id) slot = n; if (h->have_sq[k]) n++; }
    for (uint32_t k = slot; k + 1 < n; k++) h->h_qps[k] = h->h_qps[k + 1];
    h->have_sq[id] = false;
    rebuild_table(h);
    if (*host_error == 0) *host_error = start_service_locked(h);
    return 0;
}

/* Identify data at the offsets of the NVMe specification (the ones the reference reads: src/admin.cpp:139-152
 * for the controller, :189-198 for a namespace). */
static void identify_ctrl_page(uint8_t* page)
{
    memset(page, 0, 4096);
    page[0] = 0xde; page[1] = 0x10;                            /* PCI vendor id of the GPU's maker; subsystem vendor 0 */
    memcpy(page + 4, "BAMB200EMU0000000001", 20);               /* serial number */
    memset(page + 24, ' ', 40);
    memcpy(page + 24, "emulated NVMe controller (pinned memory)", 40);
    memcpy(page + 64, "1.0     ", 8);                           /* firmware revision */
    page[77] = 8;                                               /* MDTS: 2^8 pages of 4 KiB = 1 MiB, the largest cache page the library accepts */
    page[512] = 0x66;                                           /* SQES: 64-byte entries required and maximum */
    page[513] = 0x44;                                           /* CQES: 16-byte entries */
    const uint16_t maxcmd = 0xffff;                             /* command ids in flight per queue (the field's largest value) */
    memcpy(page + 514, &maxcmd, 2);
    const uint32_t nn = 1;
    memcpy(page + 516, &nn, 4);
}

static void identify_ns_page(uint64_t store_bytes, uint32_t lba_bytes, uint8_t* page)
{
    memset(page, 0, 4096);
    const uint64_t blocks = store_bytes / lba_bytes;
    memcpy(page + 0, &blocks, 8);                               /* NSZE */
    memcpy(page + 8, &blocks, 8);                               /* NCAP */
    memcpy(page + 16, &blocks, 8);                              /* NUSE */
    page[25] = 0;                                               /* NLBAF: one format */
    page[26] = 0;                                               /* FLBAS: format 0 */
    const uint32_t lbaf0 = log2_of(lba_bytes) << 16;    /* no metadata, LBADS in bits 23:16 */
    memcpy(page + 128, &lbaf0, 4);
}

/* The identify page an emulated controller answers with (cns 1: controller; cns 0: namespace 1 of a store of
 * store_bytes bytes in logical blocks of lba_bytes), without a controller or a GPU. */
extern "C" int bam_identify_page(uint32_t cns, uint64_t store_bytes, uint32_t lba_bytes, void* out4096)
{
    if (!out4096 || cns > 1) return BAM_EINVAL;
    if (cns == 1) { identify_ctrl_page(static_cast<uint8_t*>(out4096)); return BAM_OK; }
    if (lba_bytes < 512 || (lba_bytes & (lba_bytes - 1)) || store_bytes < lba_bytes) return BAM_EINVAL;
    identify_ns_page(store_bytes, lba_bytes, static_cast<uint8_t*>(out4096));
    return BAM_OK;
}

/* copy `bytes` bytes to the memory behind a command's PRP1; NVMe status */
static uint32_t admin_write_out(host_ctrl* h, uint64_t prp1, const void* src, size_t bytes)
{
    bool device = false;
    void* dst = admin_memory(h, prp1, bytes, &device);
    if (!dst) return ADM_SC_DATA_XFER;
    if (!device) { memcpy(dst, src, bytes); return 0; }
    /* GPU memory: a synchronous copy can wait for the device to go idle, which a running service kernel never is */
    cudaSetDevice(h->emu->device);
    const bool was_running = h->running;
    if (was_running) stop_service_locked(h);
    const cudaError_t e = cudaMemcpy(dst, src, bytes, cudaMemcpyHostToDevice);
    if (was_running) start_service_locked(h);
    if (e != cudaSuccess) { (void)cudaGetLastError(); return ADM_SC_DATA_XFER; }
    return 0;
}

/* Execute one admin command the way the controller would (nvm_rpc.h:53 in the reference submits it to the
 * admin queue pair and waits): IDENTIFY (controller, namespace), SET / GET FEATURES "number of queues",
 * CREATE / DELETE of I/O completion and submission queues, GET LOG PAGE (error, health and firmware logs, all
 * empty).  The completion is filled in; the return value is 0, an errno, or the packed NVMe status. */
extern "C" int nvm_raw_rpc(nvm_aq_ref ref, nvm_cmd_t* cmd, nvm_cpl_t* cpl)
{
    if (!ref || !cmd || !cpl) return EINVAL;
    host_ctrl* h = ref->h;
    std::lock_guard<std::mutex> g(h->lock);
    const uint32_t opcode = cmd->dword[0] & 0xffu, cid = cmd->dword[0] >> 16, nsid = cmd->dword[1];
    const uint64_t prp1 = ((uint64_t)cmd->dword[7] << 32) | cmd->dword[6];
    const uint32_t dw10 = cmd->dword[10], dw11 = cmd->dword[11];
    uint32_t status = 0, result = 0;
    int host_error = 0;
    uint8_t page[4096];
    switch (opcode) {
    case 0x06:                                                     /* IDENTIFY: CNS 1 = controller, 0 = namespace */
        if ((dw10 & 0xff) == 1) identify_ctrl_page(page);
        else if ((dw10 & 0xff) == 0) { if (nsid != 1) { status = ADM_SC_INVALID_NS; break; } identify_ns_page(h->emu->store_bytes, h->emu->lba_bytes, page); }
        else { status = ADM_SC_INVALID_FIELD; break; }
        status = admin_write_out(h, prp1, page, sizeof page);
        break;
    case 0x09:                                                     /* SET FEATURES */
    case 0x0a:                                                     /* GET FEATURES */
        if ((dw10 & 0xff) != 0x07) { status = ADM_SC_INVALID_FIELD; break; }
        if (opcode == 0x09) {                                      /* requested counts are zero-based */
            const uint32_t want_sq = (dw11 & 0xffff) + 1, want_cq = (dw11 >> 16) + 1;
            h->granted_sqs = (uint16_t)(want_sq < NVM_HOST_MAX_QUEUES ? want_sq : NVM_HOST_MAX_QUEUES);
            h->granted_cqs = (uint16_t)(want_cq < NVM_HOST_MAX_QUEUES ? want_cq : NVM_HOST_MAX_QUEUES);
        }
        result = ((uint32_t)(h->granted_cqs - 1) << 16) | (uint32_t)(h->granted_sqs - 1);
        break;
    case 0x05: {                                                   /* CREATE I/O COMPLETION QUEUE: physically contiguous only */
        const uint32_t qs = (dw10 >> 16) + 1;
        bool device = false;
        void* mem = (dw11 & 1u) ? admin_memory(h, prp1, (size_t)qs * sizeof(nvm_cpl_t), &device) : nullptr;
        if (!(dw11 & 1u)) { status = ADM_SC_INVALID_FIELD; break; }
        if (!mem || device) { status = ADM_SC_DATA_XFER; break; }  /* host-driven queues live in host memory */
        status = ctrl_cq_create(h, dw10 & 0xffff, qs, prp1);
        if (status == 0) memset(mem, 0, (size_t)qs * sizeof(nvm_cpl_t));
        break;
    }
    case 0x01: {                                                   /* CREATE I/O SUBMISSION QUEUE */
        const uint32_t qs = (dw10 >> 16) + 1;
        bool device = false;
        void* mem = (dw11 & 1u) ? admin_memory(h, prp1, (size_t)qs * sizeof(nvm_cmd_t), &device) : nullptr;
        if (!(dw11 & 1u)) { status = ADM_SC_INVALID_FIELD; break; }
        if (!mem || device) { status = ADM_SC_DATA_XFER; break; }
        memset(mem, 0, (size_t)qs * sizeof(nvm_cmd_t));
        status = ctrl_sq_create(h, dw10 & 0xffff, dw11 >> 16, qs, prp1, &host_error);
        break;
    }
    case 0x04: status = ctrl_cq_delete(h, dw10 & 0xffff); break;
    case 0x00: status = ctrl_sq_delete(h, dw10 & 0xffff, &host_error); break;
    case 0x02: {                                                   /* GET LOG PAGE: NUMD (zero-based dwords) in 27:16, LID in 7:0 */
        const uint32_t lid = dw10 & 0xff;
        const size_t bytes = (size_t)(((dw10 >> 16) & 0xfff) + 1) * 4;
        if (lid < 1 || lid > 3) { status = ADM_SC_LOG_PAGE_INVALID; break; }
        if (bytes > sizeof page) { status = ADM_SC_INVALID_FIELD; break; }
        memset(page, 0, sizeof page);                              /* no errors logged, no wear, one firmware slot */
        status = admin_write_out(h, prp1, page, bytes);
        break;
    }
    default: status = ADM_SC_INVALID_OPCODE; break;
    }
    cpl->dword[0] = result;
    cpl->dword[1] = 0;
    cpl->dword[2] = 0;                                             /* admin queue: SQ head 0, SQ id 0 */
    cpl->dword[3] = cid | (1u << 16) | (status << 17);
    if (host_error) return host_error;
    return status ? -(int)status : 0;
}

/* ---- the admin functions programs call: thin clients of nvm_raw_rpc, as in the reference (src/admin.cpp) --- */

static void admin_command(nvm_cmd_t* cmd, uint8_t opcode, uint32_t nsid, uint64_t prp1, uint32_t dw10, uint32_t dw11)
{
    memset(cmd, 0, sizeof *cmd);
    cmd->dword[0] = opcode;
    cmd->dword[1] = nsid;
    cmd->dword[6] = (uint32_t)prp1; cmd->dword[7] = (uint32_t)(prp1 >> 32);
    cmd->dword[10] = dw10; cmd->dword[11] = dw11;
}

extern "C" int nvm_admin_ctrl_info(nvm_aq_ref ref, struct nvm_ctrl_info* info, void* buffer, uint64_t ioaddr)
{
    if (!ref || !info) return EINVAL;
    host_ctrl* h = ref->h;
    memset(info, 0, sizeof *info);
    const uint8_t* regs = h->regs_host;
    const uint64_t cap = *reinterpret_cast<const volatile uint64_t*>(regs);
    info->nvme_version = *reinterpret_cast<const volatile uint32_t*>(regs + 0x08);
    info->page_size = h->pub.page_size;
    info->db_stride = (size_t)1 << h->pub.dstrd;               /* in doorbell registers, as the reference reports it */
    info->timeout = ((cap >> 24) & 0xff) * 500;
    info->contiguous = (int)((cap >> 16) & 1);
    info->max_entries = (uint16_t)((cap & 0xffff) + 1);
    uint8_t local[4096];
    const uint8_t* page = local;
    if (buffer && ioaddr) {                                    /* through the command interface, into the caller's page */
        nvm_cmd_t cmd; nvm_cpl_t cpl;
        admin_command(&cmd, 0x06, 0, ioaddr, 1, 0);
        const int rc = nvm_raw_rpc(ref, &cmd, &cpl);
        if (rc) return rc;
        page = static_cast<const uint8_t*>(buffer);
    } else {
        std::lock_guard<std::mutex> g(h->lock);
        identify_ctrl_page(local);
    }
    memcpy(info->pci_vendor, page, 4);
    memcpy(info->serial_no, page + 4, 20);
    memcpy(info->model_no, page + 24, 40);
    memcpy(info->firmware, page + 64, 8);
    info->max_data_size = ((size_t)1 << page[77]) * ((size_t)1 << (12 + ((cap >> 48) & 0xf)));
    info->max_data_pages = info->max_data_size / info->page_size;
    info->sq_entry_size = (size_t)1 << (page[512] & 0xf);
    info->cq_entry_size = (size_t)1 << (page[513] & 0xf);
    uint16_t maxcmd; memcpy(&maxcmd, page + 514, 2);
    uint32_t nn; memcpy(&nn, page + 516, 4);
    info->max_out_cmds = maxcmd;
    info->max_n_ns = nn;
    return 0;
}

extern "C" int nvm_admin_ns_info(nvm_aq_ref ref, struct nvm_ns_info* info, uint32_t ns_id, void* buffer, uint64_t ioaddr)
{
    if (!ref || !info) return EINVAL;
    host_ctrl* h = ref->h;
    memset(info, 0, sizeof *info);
    uint8_t local[4096];
    const uint8_t* page = local;
    if (buffer && ioaddr) {
        nvm_cmd_t cmd; nvm_cpl_t cpl;
        admin_command(&cmd, 0x06, ns_id, ioaddr, 0, 0);
        const int rc = nvm_raw_rpc(ref, &cmd, &cpl);
        if (rc) return rc;
        page = static_cast<const uint8_t*>(buffer);
    } else {
        if (ns_id != 1) return EINVAL;
        std::lock_guard<std::mutex> g(h->lock);
        identify_ns_page(h->emu->store_bytes, h->emu->lba_bytes, local);
    }
    info->ns_id = ns_id;
    uint64_t v;
    memcpy(&v, page + 0, 8); info->size = v;
    memcpy(&v, page + 8, 8); info->capacity = v;
    memcpy(&v, page + 16, 8); info->utilization = v;
    uint32_t lbaf; memcpy(&lbaf, page + 128 + 4 * (page[26] & 0xf), 4);
    info->lba_data_size = (size_t)1 << ((lbaf >> 16) & 0xff);
    info->metadata_size = lbaf & 0xffff;
    return 0;
}

extern "C" int nvm_admin_set_num_queues(nvm_aq_ref ref, uint16_t n_cqs, uint16_t n_sqs)
{
    if (!ref || n_cqs == 0 || n_sqs == 0) return EINVAL;
    nvm_cmd_t cmd; nvm_cpl_t cpl;
    admin_command(&cmd, 0x09, 0, 0, 0x07, ((uint32_t)(n_cqs - 1) << 16) | (uint32_t)(n_sqs - 1));
    return nvm_raw_rpc(ref, &cmd, &cpl);
}

extern "C" int nvm_admin_get_num_queues(nvm_aq_ref ref, uint16_t* n_cqs, uint16_t* n_sqs)
{
    if (!ref || !n_cqs || !n_sqs) return EINVAL;
    nvm_cmd_t cmd; nvm_cpl_t cpl;
    admin_command(&cmd, 0x0a, 0, 0, 0x07, 0);
    const int rc = nvm_raw_rpc(ref, &cmd, &cpl);
    if (rc) return rc;
    *n_sqs = (uint16_t)((cpl.dword[0] & 0xffff) + 1);
    *n_cqs = (uint16_t)((cpl.dword[0] >> 16) + 1);
    return 0;
}

extern "C" int nvm_admin_request_num_queues(nvm_aq_ref ref, uint16_t* n_cqs, uint16_t* n_sqs)
{
    if (!ref || !n_cqs || !n_sqs) return EINVAL;
    int rc = nvm_admin_set_num_queues(ref, *n_cqs, *n_sqs);
    if (rc) return rc;
    return nvm_admin_get_num_queues(ref, n_cqs, n_sqs);
}

static int queue_memory(const nvm_dma_t* dma, size_t offset, size_t qs, size_t es, void** host, uint64_t* dev)
{
    if (!dma || !dma->vaddr || !dma->local || offset >= dma->n_ioaddrs) return EINVAL;
    if (qs * es > (dma->n_ioaddrs - offset) * dma->page_size) return EINVAL;
    *host = static_cast<uint8_t*>(dma->vaddr) + offset * dma->page_size;
    *dev = dma->ioaddrs[offset];
    return 0;
}

extern "C" int nvm_admin_cq_create(nvm_aq_ref ref, nvm_queue_t* cq, uint16_t id, const nvm_dma_t* dma, size_t offset, size_t qs)
{
    if (!ref || !cq || id == 0) return EINVAL;
    host_ctrl* h = ref->h;
    if (qs == 0) qs = h->pub.page_size / sizeof(nvm_cpl_t);
    if (qs < 2 || qs > 0x10000 || qs > h->pub.max_qs) return EINVAL;
    void* host; uint64_t dev;
    int rc = queue_memory(dma, offset, qs, sizeof(nvm_cpl_t), &host, &dev);
    if (rc) return rc;
    nvm_queue_t queue;
    rc = nvm_queue_clear(&queue, &h->pub, true, id, (uint32_t)qs, true, host, dev);
    if (rc) return rc;
    nvm_cmd_t cmd; nvm_cpl_t cpl;
    admin_command(&cmd, 0x05, 0, dev, ((uint32_t)(qs - 1) << 16) | id, 1u);
    rc = nvm_raw_rpc(ref, &cmd, &cpl);
    if (rc) return rc;
    memcpy((void*)cq, &queue, sizeof queue);
    return 0;
}

extern "C" int nvm_admin_sq_create(nvm_aq_ref ref, nvm_queue_t* sq, const nvm_queue_t* cq, uint16_t id, const nvm_dma_t* dma, size_t offset,
                                   size_t qs)
{
    if (!ref || !sq || !cq || id == 0) return EINVAL;
    host_ctrl* h = ref->h;
    if (qs == 0) qs = h->pub.page_size / sizeof(nvm_cmd_t);
    if (qs < 2 || qs > 0x10000 || qs > h->pub.max_qs) return EINVAL;
    void* host; uint64_t dev;
    int rc = queue_memory(dma, offset, qs, sizeof(nvm_cmd_t), &host, &dev);
    if (rc) return rc;
    nvm_queue_t queue;
    rc = nvm_queue_clear(&queue, &h->pub, false, id, (uint32_t)qs, true, host, dev);
    if (rc) return rc;
    nvm_cmd_t cmd; nvm_cpl_t cpl;
    admin_command(&cmd, 0x01, 0, dev, ((uint32_t)(qs - 1) << 16) | id, ((uint32_t)cq->no << 16) | 1u);
    rc = nvm_raw_rpc(ref, &cmd, &cpl);
    if (rc) return rc;
    memcpy((void*)sq, &queue, sizeof queue);
    return 0;
}

extern "C" int nvm_admin_cq_delete(nvm_aq_ref ref, nvm_queue_t* cq)
{
    if (!ref || !cq || cq->db == nullptr) return EINVAL;
    nvm_cmd_t cmd; nvm_cpl_t cpl;
    admin_command(&cmd, 0x04, 0, 0, cq->no, 0);
    const int rc = nvm_raw_rpc(ref, &cmd, &cpl);
    if (rc) return rc;
    cq->db = nullptr;
    return 0;
}

extern "C" int nvm_admin_sq_delete(nvm_aq_ref ref, nvm_queue_t* sq, const nvm_queue_t*)
{
    if (!ref || !sq || sq->db == nullptr) return EINVAL;
    nvm_cmd_t cmd; nvm_cpl_t cpl;
    admin_command(&cmd, 0x00, 0, 0, sq->no, 0);
    const int rc = nvm_raw_rpc(ref, &cmd, &cpl);
    if (rc) return rc;
    sq->db = nullptr;
    return 0;
}

/* `ptr` is where the caller will read the page, `ioaddr` the bus address of the same memory (nvm_admin.h:111-117
 * in the reference).  One controller page at most; the logs of the emulated controller are empty. */
extern "C" int nvm_admin_get_log_page(nvm_aq_ref ref, uint32_t ns_id, void* ptr, uint64_t ioaddr, uint8_t log_id, uint64_t log_offset)
{
    if (!ref || !ptr || !ioaddr) return EINVAL;
    nvm_cmd_t cmd; nvm_cpl_t cpl;
    admin_command(&cmd, 0x02, ns_id, ioaddr, ((uint32_t)(4096 / 4 - 1) << 16) | log_id, 0);
    cmd.dword[12] = (uint32_t)log_offset; cmd.dword[13] = (uint32_t)(log_offset >> 32);
    return nvm_raw_rpc(ref, &cmd, &cpl);
}

/* ---- host-side queue descriptors -------------------------------------------------------------------------- */

extern "C" int nvm_queue_clear(nvm_queue_t* q, const nvm_ctrl_t* ctrl, bool cq, uint16_t no, uint32_t qs, bool local, volatile void* vaddr,
                               uint64_t ioaddr)
{
    if (!q || !ctrl || qs < 2 || qs > 0x10000 || qs > ctrl->max_qs) return EINVAL;
    memset(q, 0, sizeof *q);
    q->no = no;
    q->qs = qs; q->qs_minus_1 = qs - 1;
    while ((1u << q->qs_log2) < qs) q->qs_log2++;
    q->es = cq ? sizeof(nvm_cpl_t) : sizeof(nvm_cmd_t);
    q->phase = 1;
    q->local = local ? 1 : 0;
    uint8_t* regs = static_cast<uint8_t*>(const_cast<void*>(ctrl->mm_ptr));
    q->db = reinterpret_cast<volatile uint32_t*>(regs + (cq ? NVM_CQ_DBL_OFFSET(no, ctrl->dstrd) : NVM_SQ_DBL_OFFSET(no, ctrl->dstrd)));
    q->vaddr = vaddr;
    q->ioaddr = ioaddr;
    return 0;
}

extern "C" void nvm_queue_reset(nvm_queue_t* q)
{
    if (!q) return;
    q->head = 0; q->tail = 0; q->last = 0; q->phase = 1;
}

extern "C" nvm_cpl_t* nvm_cq_dequeue_block(nvm_queue_t* cq, uint64_t timeout_ms)
{
    struct timespec t0, t;
    clock_gettime(CLOCK_MONOTONIC, &t0);
    for (;;) {
        nvm_cpl_t* cpl = nvm_cq_dequeue(cq);
        if (cpl) return cpl;
        clock_gettime(CLOCK_MONOTONIC, &t);
        const uint64_t ms = (uint64_t)(t.tv_sec - t0.tv_sec) * 1000ull + (uint64_t)((t.tv_nsec - t0.tv_nsec) / 1000000);
        if (ms >= timeout_ms) return nullptr;
    }
}
