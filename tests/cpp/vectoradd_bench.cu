/*
 * vectoradd_bench.cu -- the reference's vector-add benchmark (benchmarks/vectoradd/main.cu:103-118,
 * kernel_baseline_ptr_pc: C[tid] = A[tid] + B[tid] with three bam_ptr cursors) written against this
 * library's drop-in headers.  A, B and C are three arrays behind one page cache; C is written
 * through the cache, flushed, and compared on the host with A + B.  --tlb 1 runs the same kernel
 * with bam_ptr_tlb cursors over block-level translation buffers in shared memory
 * (include/page_cache.h:158-411 of the reference).  Prints one JSON line.
 */
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "bam_synth.h"
#include "event.h"
#include "page_cache.h"
#include "util.h"

struct VectorAddPtr {
    array_d_t<uint64_t>*da, *db, *dc;
    uint64_t n_elems;

    __device__ void operator()(uint32_t worker_block, uint32_t n_worker_blocks) const
    {
        bam_ptr<uint64_t> Aptr(da), Bptr(db), Cptr(dc);
        /* whole warps enter the loop body together: the cursors are warp-cooperative */
        const uint64_t stride = (uint64_t)n_worker_blocks * blockDim.x;
        const uint64_t first = (uint64_t)worker_block * blockDim.x + threadIdx.x;
        for (uint64_t base = first - (threadIdx.x & 31u); base < n_elems; base += stride) {
            const uint64_t tid = base + (threadIdx.x & 31u);
            if (tid < n_elems) Cptr[tid] = Aptr[tid] + Bptr[tid];
        }
        Aptr.fini(); Bptr.fini(); Cptr.fini();
    }
};

#define TLB_N 16
struct VectorAddTlb {
    array_d_t<uint64_t>*da, *db, *dc;
    uint64_t n_elems;

    __device__ void operator()(uint32_t worker_block, uint32_t n_worker_blocks) const
    {
        __shared__ tlb<uint64_t, TLB_N> ta, tb, tc;
        ta.init(da); tb.init(db); tc.init(dc);
        {
            bam_ptr_tlb<uint64_t, TLB_N> Aptr(da, &ta), Bptr(db, &tb), Cptr(dc, &tc);
            /* a block works on a contiguous chunk, so its warps keep meeting the same pages */
            const uint64_t per_block = (n_elems + n_worker_blocks - 1) / n_worker_blocks;
            const uint64_t lo = (uint64_t)worker_block * per_block;
            const uint64_t hi = lo + per_block < n_elems ? lo + per_block : n_elems;
            for (uint64_t base = lo + (threadIdx.x & ~31u); base < hi; base += blockDim.x) {
                const uint64_t tid = base + (threadIdx.x & 31u);
                if (tid < hi) Cptr[tid] = Aptr[tid] + Bptr[tid];
            }
            Aptr.fini(); Bptr.fini(); Cptr.fini();
        }
        ta.fini(); tb.fini(); tc.fini();
    }
};

static uint64_t arg_u64(int argc, char** argv, const char* name, uint64_t def)
{
    for (int i = 1; i + 1 < argc; i++)
        if (strcmp(argv[i], name) == 0) return strtoull(argv[i + 1], nullptr, 0);
    return def;
}

int main(int argc, char** argv)
{
    const uint64_t n_elems = arg_u64(argc, argv, "--num_elems", 1ull << 20);
    const uint64_t pages = arg_u64(argc, argv, "--pages", 1ull << 16);
    const uint64_t page_size = 4096;
    const uint64_t qd = arg_u64(argc, argv, "--queue_depth", 64);
    const uint64_t nq = arg_u64(argc, argv, "--num_queues", 8);
    const uint64_t seed = arg_u64(argc, argv, "--seed", 7);
    const uint64_t use_tlb = arg_u64(argc, argv, "--tlb", 0);
    try {
        const uint64_t arr_pages = (n_elems * 8 + page_size - 1) / page_size;
        Controller ctrl("emu:0", 1, 0, qd, nq, 3 * arr_pages * page_size);
        uint64_t* store = (uint64_t*)bam_ctrl_store_host(ctrl.h);
        const uint64_t arr_words = arr_pages * page_size / 8;
        for (uint64_t i = 0; i < n_elems; i++) {
            store[i] = bam_store_elem(seed, i);                       /* A */
            store[arr_words + i] = bam_store_elem(seed + 1, i);       /* B */
            store[2 * arr_words + i] = 0xdeadbeefull;                 /* C: must be overwritten */
        }
        std::vector<Controller*> ctrls{ &ctrl };
        page_cache_t h_pc(page_size, pages, 0, ctrl, 64, ctrls);
        range_t<uint64_t> ra(0, n_elems, 0, arr_pages, 0, page_size, &h_pc, 0);
        range_t<uint64_t> rb(0, n_elems, arr_pages, arr_pages, 0, page_size, &h_pc, 0);
        range_t<uint64_t> rc(0, n_elems, 2 * arr_pages, arr_pages, 0, page_size, &h_pc, 0);
        std::vector<range_t<uint64_t>*> va{ &ra }, vb{ &rb }, vc{ &rc };
        array_t<uint64_t> a(n_elems, 0, va, 0), b(n_elems, arr_pages * page_size, vb, 0), c(n_elems, 2 * arr_pages * page_size, vc, 0);

        Event before;
        cudaError_t e;
        if (use_tlb) e = bam::launch_fused(h_pc.emu(), VectorAddTlb{ a.d_array_ptr, b.d_array_ptr, c.d_array_ptr, n_elems });
        else e = bam::launch_fused(h_pc.emu(), VectorAddPtr{ a.d_array_ptr, b.d_array_ptr, c.d_array_ptr, n_elems });
        Event after;
        cuda_err_chk(e);
        cuda_err_chk(cudaDeviceSynchronize());
        const double us = after - before;
        bam_status_out_t st;
        bam_ctrl_status(ctrl.h, &st, 0);
        bam_cache_stats_t cs;
        bam_cache_stats(h_pc.h, &cs, 0);
        h_pc.flush_cache();
        bam_status_out_t st2;
        bam_ctrl_status(ctrl.h, &st2, 0);
        uint64_t bad = 0;
        bam_cache_audit(h_pc.h, &bad);
        uint64_t mismatches = 0, checksum = 0;
        for (uint64_t i = 0; i < n_elems; i++) {
            const uint64_t want = bam_store_elem(seed, i) + bam_store_elem(seed + 1, i);
            if (store[2 * arr_words + i] != want) mismatches++;
            checksum += store[2 * arr_words + i];
        }
        printf("{\"checksum\": %llu, \"mismatches\": %llu, \"elapsed_us\": %.1f, \"elems_per_s\": %.1f, \"status\": %u, \"flush_status\": %u, "
               "\"where\": %u, \"hits\": %llu, \"misses\": %llu, \"read_ios\": %llu, \"audit\": %llu}\n",
               (unsigned long long)checksum, (unsigned long long)mismatches, us, (double)n_elems / (us * 1e-6), st.code, st2.code, st.where,
               (unsigned long long)cs.hits, (unsigned long long)cs.misses, (unsigned long long)cs.read_ios, (unsigned long long)bad);
        ctrl.close();
    } catch (const std::exception& ex) {
        fprintf(stderr, "error: %s\n", ex.what());
        return 1;
    }
    return 0;
}
