/*
 * device_api_bench.cu -- the remaining device entry points of the reference's array and raw-I/O API,
 * driven from user kernels and checked on the host against the store's definition:
 *   array_d_t::get_raw / release_raw, acquire_page / release_page, memcpy  (page_cache.h:1256-1537)
 *   bafs_ptr::memcpy_to_array_aligned                                      (bafs_ptr.h:121-123)
 *   bafs_ptr: *p, p[i], p + i, p - i, ++p, p++, --p, p--, ==, !=, p(i, v)   (bafs_ptr.h:17-132)
 *   read_data / write_data / access_data_async / poll_async                (page_cache.h:1930-2132)
 * Prints one JSON line with the number of mismatches of each part.
 */
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "bafs_ptr.h"
#include "bam_synth.h"
#include "page_cache.h"
#include "util.h"

struct RawViewKernel {                /* out[k] = a[idx[k]] via get_raw, out2[k] = a[idx[k]] via acquire_page */
    array_d_t<uint64_t>* a;
    const uint64_t* idx;
    uint64_t n;
    uint64_t *out, *out2;

    __device__ void operator()(uint32_t vb, uint32_t nvb) const
    {
        const uint64_t stride = (uint64_t)nvb * blockDim.x;
        for (uint64_t base = (uint64_t)vb * blockDim.x + (threadIdx.x & ~31u); base < n; base += stride) {
            const uint64_t k = base + (threadIdx.x & 31u);
            if (k < n) {
                auto v = a->get_raw(idx[k]);
                out[k] = v.addr ? v.addr[v.offset] : 0;
                a->release_raw(idx[k], v);
                uint32_t slot;
                size_t start, end;
                uint64_t* p = a->acquire_page(idx[k], slot, start, end);
                out2[k] = (p && idx[k] >= start && idx[k] < end) ? p[idx[k] - start] : 0;
                a->release_page(idx[k], slot);
            }
        }
    }
};

struct BafsOpsKernel {                /* thread k works on a pointer to element 5 k; four reads and the comparisons per thread */
    array_d_t<uint64_t>* a;
    uint64_t n;
    uint64_t* out;                    /* out[4 k ..]: *p, p[3], *(p + 7), the element after three steps from p + 7 */
    unsigned int* bad_cmp;

    __device__ void operator()(uint32_t vb, uint32_t nvb) const
    {
        const uint64_t stride = (uint64_t)nvb * blockDim.x;
        for (uint64_t base = (uint64_t)vb * blockDim.x + (threadIdx.x & ~31u); base < n; base += stride) {
            const uint64_t k = base + (threadIdx.x & 31u);
            if (k < n) {
                bafs_ptr<uint64_t> p(a, 5 * k);
                out[4 * k] = *p;
                out[4 * k + 1] = p[3];
                bafs_ptr<uint64_t> q = p + 7;
                out[4 * k + 2] = *q;
                ++q; q++; --q;                                   /* 5 k + 8 */
                bafs_ptr<uint64_t> r = q--;                      /* r at 5 k + 8, q back at 5 k + 7 */
                out[4 * k + 3] = *r;
                const bool ok = (p + 7 == q) && (r - 1 == q) && (p != q) && !(p == r) && ((p + 8) == r);
                if (!ok) atomicAdd(bad_cmp, 1u);
            }
        }
    }
};

struct MemcpyKernel {                 /* warp w copies `len` elements from first + w * step into dst + w * len */
    array_d_t<uint64_t>* a;
    uint64_t first, step, len, n_copies;
    uint64_t* dst;

    __device__ void operator()(uint32_t vb, uint32_t nvb) const
    {
        const uint64_t warp = ((uint64_t)vb * blockDim.x + threadIdx.x) >> 5, nwarps = ((uint64_t)nvb * blockDim.x) >> 5;
        bafs_ptr<uint64_t> p(a, first);
        for (uint64_t w = warp; w < n_copies; w += nwarps) {
            if (w & 1) p.memcpy_to_array_aligned(w * step, len, dst + w * len);
            else a->memcpy(first + w * step, len, dst + w * len);
        }
    }
};

struct RawIoKernel {                  /* thread t: read page src[t] into its slot, write it to page dst[t]; then 4 async reads */
    page_cache_d_t pc;
    Controller* ctrl;
    const uint64_t *src, *dst;
    uint64_t n;
    uint64_t n_async;
    const uint64_t* apages;           /* n_async * 4 pages */
    uint64_t* asum;                   /* per async thread: sum of the first word of its 4 pages */
    unsigned int* errors;

    __device__ void operator()(uint32_t vb, uint32_t nvb) const
    {
        const uint64_t tid = (uint64_t)vb * blockDim.x + threadIdx.x, nthr = (uint64_t)nvb * blockDim.x;
        QueuePair* qp = ctrl->d_qps + (tid >> 5) % ctrl->n_qps;
        const uint64_t bpp = pc.n_blocks_per_page;
        for (uint64_t t = tid; t < n; t += nthr) {
            const unsigned long long slot = tid * 4;                        /* private landing slots: 4 per thread */
            int rc = read_data(&pc, qp, src[t] * bpp, bpp, slot);
            if (rc == 0) rc = write_data(&pc, qp, dst[t] * bpp, bpp, slot);
            if (rc) atomicAdd(errors, 1u);
        }
        for (uint64_t t = tid; t < n_async; t += nthr) {
            uint16_t cid[4], pos[4];
            int rc = 0;
            for (int d = 0; d < 4 && rc == 0; d++)
                rc = access_data_async(&pc, qp, apages[t * 4 + d] * bpp, bpp, tid * 4 + d, NVM_IO_READ, &cid[d], &pos[d]);
            uint64_t s = 0;
            for (int d = 0; d < 4 && rc == 0; d++) {
                rc = poll_async(qp, cid[d], pos[d]);
                if (rc == 0) s += *reinterpret_cast<volatile uint64_t*>(pc.base_addr + (tid * 4 + d) * pc.page_size);
            }
            if (rc) atomicAdd(errors, 1u);
            asum[t] = s;
        }
    }
};

int main()
{
    const uint64_t n_elems = 1ull << 20, page_size = 4096, n_pages = n_elems * 8 / page_size, seed = 19;
    int bad_raw = 0, bad_acq = 0, bad_cpy = 0, bad_io = 0, bad_async = 0;
    try {
        Controller ctrl("emu:0", 1, 0, 1024, 8, 2 * n_elems * sizeof(uint64_t));      /* second half: target of the raw writes */
        uint64_t* store = (uint64_t*)bam_ctrl_store_host(ctrl.h);
        for (uint64_t i = 0; i < n_elems; i++) { store[i] = bam_store_elem(seed, i); store[n_elems + i] = 0; }
        std::vector<Controller*> ctrls{ &ctrl };
        bam_emu_d_t emu;
        bam_ctrl_emu_descriptor(ctrl.h, &emu, sizeof emu);
        uint32_t grid = 0, ctrl_blocks = 0, threads = 0;
        bam_launch_geometry(ctrl.h, &grid, &ctrl_blocks, &threads);
        page_cache_t h_pc(page_size, (uint64_t)grid * threads * 4, 0, ctrl, 64, ctrls);
        range_t<uint64_t> h_range(0, n_elems, 0, n_pages, 0, page_size, &h_pc, 0);
        std::vector<range_t<uint64_t>*> vr{ &h_range };
        array_t<uint64_t> a(n_elems, 0, vr, 0);

        /* 1. get_raw / acquire_page */
        const uint64_t n = 1 << 16;
        std::vector<uint64_t> idx(n);
        bam_pcg32_t g;
        bam_lane_stream(&g, 5, 0);
        for (uint64_t k = 0; k < n; k++) idx[k] = (k % 3 == 0) ? (k * 7) % n_elems : bam_uniform_index(&g, n_elems);
        uint64_t *d_idx, *d_out, *d_out2;
        cuda_err_chk(cudaMalloc(&d_idx, n * 8)); cuda_err_chk(cudaMalloc(&d_out, n * 8)); cuda_err_chk(cudaMalloc(&d_out2, n * 8));
        cuda_err_chk(cudaMemcpy(d_idx, idx.data(), n * 8, cudaMemcpyHostToDevice));
        cuda_err_chk(bam::launch_fused(h_pc.emu(), RawViewKernel{ a.d_array_ptr, d_idx, n, d_out, d_out2 }));
        cuda_err_chk(cudaDeviceSynchronize());
        std::vector<uint64_t> out(n), out2(n);
        cuda_err_chk(cudaMemcpy(out.data(), d_out, n * 8, cudaMemcpyDeviceToHost));
        cuda_err_chk(cudaMemcpy(out2.data(), d_out2, n * 8, cudaMemcpyDeviceToHost));
        for (uint64_t k = 0; k < n; k++) { bad_raw += out[k] != store[idx[k]]; bad_acq += out2[k] != store[idx[k]]; }

        /* 1b. the pointer operators of bafs_ptr, on the device */
        const uint64_t n_ops = 1 << 15;
        uint64_t* d_ops;
        unsigned int* d_badcmp;
        cuda_err_chk(cudaMalloc(&d_ops, n_ops * 4 * 8)); cuda_err_chk(cudaMalloc(&d_badcmp, 4));
        cuda_err_chk(cudaMemset(d_badcmp, 0, 4));
        cuda_err_chk(bam::launch_fused(h_pc.emu(), BafsOpsKernel{ a.d_array_ptr, n_ops, d_ops, d_badcmp }));
        cuda_err_chk(cudaDeviceSynchronize());
        std::vector<uint64_t> ops(n_ops * 4);
        unsigned int badcmp = 0;
        cuda_err_chk(cudaMemcpy(ops.data(), d_ops, ops.size() * 8, cudaMemcpyDeviceToHost));
        cuda_err_chk(cudaMemcpy(&badcmp, d_badcmp, 4, cudaMemcpyDeviceToHost));
        int bad_ops = (int)badcmp;
        for (uint64_t k = 0; k < n_ops; k++)
            bad_ops += (ops[4 * k] != store[5 * k]) + (ops[4 * k + 1] != store[5 * k + 3]) + (ops[4 * k + 2] != store[5 * k + 7]) +
                       (ops[4 * k + 3] != store[5 * k + 8]);

        /* 2. memcpy: 300 copies of 1000 elements from odd offsets (every copy crosses pages, half are unaligned) */
        const uint64_t n_copies = 300, len = 1000, first = 3, step = 3001;
        uint64_t* d_dst;
        cuda_err_chk(cudaMalloc(&d_dst, n_copies * len * 8));
        cuda_err_chk(cudaMemset(d_dst, 0, n_copies * len * 8));
        cuda_err_chk(bam::launch_fused(h_pc.emu(), MemcpyKernel{ a.d_array_ptr, first, step, len, n_copies, d_dst }));
        cuda_err_chk(cudaDeviceSynchronize());
        std::vector<uint64_t> dst(n_copies * len);
        cuda_err_chk(cudaMemcpy(dst.data(), d_dst, dst.size() * 8, cudaMemcpyDeviceToHost));
        for (uint64_t w = 0; w < n_copies; w++)
            for (uint64_t k = 0; k < len; k++) bad_cpy += dst[w * len + k] != store[first + w * step + k];

        /* 3. raw block I/O: page p of the first half is copied to page n_pages + perm(p) of the second half */
        uint64_t bad_audit = 0;
        bam_cache_audit(h_pc.h, &bad_audit);
        bam_cache_invalidate(h_pc.h);
        /* 4 commands per thread in flight: the warps that share a queue must stay below its depth (4 x 128 < 1024) */
        const uint64_t n_io = n_pages, n_async = 1024;       /* every page of the first half lands somewhere in the second */
        std::vector<uint64_t> src(n_io), dstp(n_io), ap(n_async * 4);
        for (uint64_t t = 0; t < n_io; t++) { src[t] = bam_permute(t, n_pages, 3); dstp[t] = n_pages + t; }
        for (uint64_t t = 0; t < n_async * 4; t++) ap[t] = bam_permute(t, n_pages, 4);
        uint64_t *d_src, *d_dstp, *d_ap, *d_asum;
        unsigned int* d_err;
        cuda_err_chk(cudaMalloc(&d_src, n_io * 8)); cuda_err_chk(cudaMalloc(&d_dstp, n_io * 8));
        cuda_err_chk(cudaMalloc(&d_ap, ap.size() * 8)); cuda_err_chk(cudaMalloc(&d_asum, n_async * 8)); cuda_err_chk(cudaMalloc(&d_err, 4));
        cuda_err_chk(cudaMemcpy(d_src, src.data(), n_io * 8, cudaMemcpyHostToDevice));
        cuda_err_chk(cudaMemcpy(d_dstp, dstp.data(), n_io * 8, cudaMemcpyHostToDevice));
        cuda_err_chk(cudaMemcpy(d_ap, ap.data(), ap.size() * 8, cudaMemcpyHostToDevice));
        cuda_err_chk(cudaMemset(d_err, 0, 4));
        cuda_err_chk(bam::launch_fused(h_pc.emu(), RawIoKernel{ h_pc.pdt, (Controller*)ctrl.d_ctrl_ptr, d_src, d_dstp, n_io, n_async, d_ap, d_asum, d_err }));
        cuda_err_chk(cudaDeviceSynchronize());
        unsigned int errs = 0;
        cuda_err_chk(cudaMemcpy(&errs, d_err, 4, cudaMemcpyDeviceToHost));
        std::vector<uint64_t> asum(n_async);
        cuda_err_chk(cudaMemcpy(asum.data(), d_asum, n_async * 8, cudaMemcpyDeviceToHost));
        bad_io = (int)errs;
        for (uint64_t t = 0; t < n_io; t++)
            bad_io += memcmp(store + dstp[t] * 512, store + src[t] * 512, page_size) != 0;
        for (uint64_t t = 0; t < n_async; t++) {
            uint64_t want = 0;
            for (int d = 0; d < 4; d++) want += store[ap[t * 4 + d] * 512];
            bad_async += asum[t] != want;
        }
        bam_status_out_t st;
        bam_ctrl_status(ctrl.h, &st, 0);
        printf("{\"bad_get_raw\": %d, \"bad_acquire_page\": %d, \"bad_bafs_ptr_ops\": %d, \"bad_memcpy\": %d, \"bad_raw_io\": %d, "
               "\"bad_async\": %d, \"status\": %u, \"where\": %u, \"audit\": %llu}\n", bad_raw, bad_acq, bad_ops, bad_cpy, bad_io, bad_async,
               st.code, st.where, (unsigned long long)bad_audit);
        ctrl.close();
    } catch (const std::exception& ex) {
        fprintf(stderr, "error: %s\n", ex.what());
        return 1;
    }
    return 0;
}
