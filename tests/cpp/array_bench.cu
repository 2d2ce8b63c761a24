/*
 * array_bench.cu -- the reference's nvm-array-bench (benchmarks/array/main.cu) written against this
 * library's drop-in headers: Controller, page_cache_t, range_t, array_t on the host,
 * array_d_t<T>::operator[] on the device (--bam_ptr 1: bam_ptr cursors, --bam_ptr 2: bam_ptr_tlb
 * cursors over a block-level tlb in shared memory).  Differences from the reference program: the access
 * pattern is the seeded PCG32 stream of bam_synth.h instead of rand(), the values read are summed
 * (the reference discards them), and the kernel is launched fused with the emulated controller.
 * Prints one JSON line.
 */
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "bam_synth.h"
#include "event.h"
#include "page_cache.h"
#include "util.h"

struct RandomAccessKernel {
    array_d_t<uint64_t>* dr;
    uint64_t n_threads;
    const uint64_t* assignment;
    uint64_t reqs_per_thread;
    unsigned long long* sum;

    __device__ void operator()(uint32_t worker_block, uint32_t n_worker_blocks) const
    {
        unsigned long long v = 0;
        for (uint64_t tid = (uint64_t)worker_block * blockDim.x + threadIdx.x; tid < n_threads;
             tid += (uint64_t)n_worker_blocks * blockDim.x)
            for (uint64_t i = 0; i < reqs_per_thread; i++) v += (*dr)[assignment[tid * reqs_per_thread + i]];
        atomicAdd(sum, v);
    }
};

struct BamPtrKernel {                 /* the same reads through a bam_ptr cursor */
    array_d_t<uint64_t>* dr;
    uint64_t n_threads;
    const uint64_t* assignment;
    uint64_t reqs_per_thread;
    unsigned long long* sum;

    __device__ void operator()(uint32_t worker_block, uint32_t n_worker_blocks) const
    {
        unsigned long long v = 0;
        bam_ptr<uint64_t> ptr(dr);
        for (uint64_t tid = (uint64_t)worker_block * blockDim.x + threadIdx.x; tid < n_threads;
             tid += (uint64_t)n_worker_blocks * blockDim.x)
            for (uint64_t i = 0; i < reqs_per_thread; i++) v += ptr[assignment[tid * reqs_per_thread + i]];
        ptr.fini();
        atomicAdd(sum, v);
    }
};

struct TlbPtrKernel {                 /* the same reads through bam_ptr_tlb cursors over a block-level tlb */
    array_d_t<uint64_t>* dr;
    uint64_t n_threads;
    const uint64_t* assignment;
    uint64_t reqs_per_thread;
    unsigned long long* sum;

    __device__ void operator()(uint32_t worker_block, uint32_t n_worker_blocks) const
    {
        __shared__ tlb<uint64_t, 32> t;
        t.init(dr);
        unsigned long long v = 0;
        {
            bam_ptr_tlb<uint64_t, 32> ptr(dr, &t);
            for (uint64_t tid = (uint64_t)worker_block * blockDim.x + threadIdx.x; tid < n_threads;
                 tid += (uint64_t)n_worker_blocks * blockDim.x)
                for (uint64_t i = 0; i < reqs_per_thread; i++) v += ptr[assignment[tid * reqs_per_thread + i]];
            ptr.fini();
        }
        t.fini();
        atomicAdd(sum, v);
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
    const uint64_t n_elems = arg_u64(argc, argv, "--num_elems", 1ull << 22);
    const uint64_t pages = arg_u64(argc, argv, "--pages", 4096);
    const uint64_t page_size = arg_u64(argc, argv, "--page_size", 4096);
    const uint64_t threads = arg_u64(argc, argv, "--threads", 1ull << 14);
    const uint64_t reqs = arg_u64(argc, argv, "--reqs", 16);
    const uint64_t qd = arg_u64(argc, argv, "--queue_depth", 64);
    const uint64_t nq = arg_u64(argc, argv, "--num_queues", 8);
    const uint64_t seed = arg_u64(argc, argv, "--seed", 11);
    const uint64_t aseed = arg_u64(argc, argv, "--access_seed", 29);
    const uint64_t use_ptr = arg_u64(argc, argv, "--bam_ptr", 0);
    try {
        Controller ctrl("emu:0", 1, 0, qd, nq, n_elems * sizeof(uint64_t));
        bam_ctrl_fill_store(ctrl.h, seed, 0, nullptr);
        std::vector<Controller*> ctrls{ &ctrl };
        page_cache_t h_pc(page_size, pages, 0, ctrl, 64, ctrls);
        const uint64_t total_pages = (n_elems * sizeof(uint64_t) + page_size - 1) / page_size;
        range_t<uint64_t> h_range(0, n_elems, 0, total_pages, 0, page_size, &h_pc, 0);
        std::vector<range_t<uint64_t>*> vr{ &h_range };
        array_t<uint64_t> a(n_elems, 0, vr, 0);

        std::vector<uint64_t> assign(threads * reqs);
        for (uint64_t t = 0; t < threads; t++) {
            bam_pcg32_t g;
            bam_lane_stream(&g, aseed, t);
            for (uint64_t k = 0; k < reqs; k++) assign[t * reqs + k] = bam_uniform_index(&g, n_elems);
        }
        uint64_t* d_assign;
        unsigned long long* d_sum;
        cuda_err_chk(cudaMalloc(&d_assign, assign.size() * 8));
        cuda_err_chk(cudaMalloc(&d_sum, 8));
        cuda_err_chk(cudaMemcpy(d_assign, assign.data(), assign.size() * 8, cudaMemcpyHostToDevice));
        cuda_err_chk(cudaMemset(d_sum, 0, 8));

        Event before;
        cudaError_t e;
        if (use_ptr == 2) e = bam::launch_fused(h_pc.emu(), TlbPtrKernel{ a.d_array_ptr, threads, d_assign, reqs, d_sum });
        else if (use_ptr) e = bam::launch_fused(h_pc.emu(), BamPtrKernel{ a.d_array_ptr, threads, d_assign, reqs, d_sum });
        else e = bam::launch_fused(h_pc.emu(), RandomAccessKernel{ a.d_array_ptr, threads, d_assign, reqs, d_sum });
        Event after;
        cuda_err_chk(e);
        cuda_err_chk(cudaDeviceSynchronize());
        const double us = after - before;
        unsigned long long sum = 0;
        cuda_err_chk(cudaMemcpy(&sum, d_sum, 8, cudaMemcpyDeviceToHost));
        bam_status_out_t st;
        bam_ctrl_status(ctrl.h, &st, 0);
        bam_cache_stats_t cs;
        bam_cache_stats(h_pc.h, &cs, 0);
        uint64_t bad = 0;
        bam_cache_audit(h_pc.h, &bad);
        const double ops = (double)(threads * reqs);
        printf("{\"checksum\": %llu, \"elapsed_us\": %.1f, \"ops\": %.0f, \"ops_per_s\": %.1f, \"status\": %u, \"where\": %u, \"detail\": %llu, "
               "\"hits\": %llu, \"misses\": %llu, \"read_ios\": %llu, \"audit\": %llu}\n",
               sum, us, ops, ops / (us * 1e-6), st.code, st.where, (unsigned long long)st.detail, (unsigned long long)cs.hits, (unsigned long long)cs.misses,
               (unsigned long long)cs.read_ios, (unsigned long long)bad);
        cudaFree(d_assign);
        cudaFree(d_sum);
        ctrl.close();
    } catch (const std::exception& ex) {
        fprintf(stderr, "error: %s\n", ex.what());
        return 1;
    }
    return 0;
}
