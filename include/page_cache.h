/*
 * page_cache.h -- host classes and device API under the names of the reference's
 * include/page_cache.h:
 *   page_cache_t(page_size, n_pages, cudaDevice, ctrl, max_range, ctrls)        (:697-875 there)
 *   range_t<T>(index_start, count, page_start, page_count, page_start_offset,
 *              page_size, cache, cudaDevice, dist)                              (:978-1030)
 *   array_t<T>(n_elems, disk_start_offset, ranges, cudaDevice)                  (:1719-1772)
 *   array_d_t<T>, range_d_t<T>, bam_ptr<T>, tlb<T,n>, bam_ptr_tlb<T,n>, page_cache_d_t (device side)
 * The host classes are thin wrappers over the C ABI (bam_abi.h); the device side is
 * include/bam/*.cuh.  An array takes one or several ranges, and a range may start inside a page
 * (page_start_offset < page_size); the page-walking launchers of the C ABI want a single range
 * that starts on a page boundary.  Compile with nvcc.
 */
#ifndef BAM_COMPAT_PAGE_CACHE_H
#define BAM_COMPAT_PAGE_CACHE_H

#include <cstdint>
#include <cstdio>
#include <stdexcept>
#include <string>
#include <vector>

#include "ctrl.h"
#include "bam/array.cuh"
#include "bam/launch.cuh"
#include "bam/tlb.cuh"

using bam::array_d_t;
using bam::bafs_ptr;
using bam::bam_ptr;
using bam::bam_ptr_tlb;
using bam::read_data;
using bam::write_data;
using bam::access_data;
using bam::access_data_async;
using bam::poll_async;
using bam::tlb;
using bam::range_d_t;

enum data_dist_t { REPLICATE = 0, STRIPE = 1 };

struct page_cache_t {
    bam_cache_t h = nullptr;
    page_cache_d_t pdt;                       /* the device descriptor, by value (page_cache.h:633 there) */
    uint64_t page_size = 0, n_pages = 0;
    Controller* ctrl = nullptr;

    /* `ctrls` lists every controller behind the cache (page_cache.h:714-720 there); `c` is the first of
     * them.  With an empty or one-element list the cache has the single backing controller `c`. */
    page_cache_t(const uint64_t ps, const uint64_t np, const uint32_t /*cudaDevice*/, const Controller& c,
                 const uint64_t /*max_range*/, const std::vector<Controller*>& ctrls)
    {
        int rc;
        if (ctrls.size() > 1) {
            std::vector<bam_ctrl_t> hs;
            for (Controller* k : ctrls) hs.push_back(k->h);
            rc = bam_cache_create_multi(&h, hs.data(), (uint32_t)hs.size(), (uint32_t)ps, np);
        } else
            rc = bam_cache_create(&h, c.h, (uint32_t)ps, np);
        if (rc != 0) throw std::runtime_error(std::string("Failed to create page cache: ") + bam_strerror(rc));
        bam_cache_descriptor(h, &pdt, sizeof pdt);
        page_size = ps; n_pages = np;
        ctrl = ctrls.size() > 1 ? ctrls[0] : const_cast<Controller*>(&c);
    }
    ~page_cache_t() { if (h) bam_cache_destroy(h); }
    page_cache_t(const page_cache_t&) = delete;
    page_cache_t& operator=(const page_cache_t&) = delete;

    void flush_cache() { bam_cache_flush(h, nullptr); cudaDeviceSynchronize(); }
    void print_reset_stats()
    {
        bam_cache_stats_t s;
        bam_cache_stats(h, &s, 1);
        printf("*********************************\n#READ IOs:\t%llu\n", (unsigned long long)s.read_ios);
    }
    /* the descriptor every fused launch needs next to the workload */
    bam_emu_d_t emu() const
    {
        bam_emu_d_t e;
        bam_ctrl_emu_descriptor(ctrl->h, &e, sizeof e);
        return e;
    }
};

template <typename T>
struct range_t {
    uint64_t index_start, count, page_start, page_count, page_start_offset, page_size;
    page_cache_t* cache;
    data_dist_t dist;
    range_t(uint64_t is, uint64_t cnt, uint64_t ps, uint64_t pc, uint64_t pso, uint64_t p_size, page_cache_t* c,
            uint32_t /*cudaDevice*/, data_dist_t d = REPLICATE)
        : index_start(is), count(cnt), page_start(ps), page_count(pc), page_start_offset(pso), page_size(p_size), cache(c),
          dist(d)
    {
        if (pso >= p_size) throw std::runtime_error("range_t: page_start_offset must be smaller than a page");
    }
};

template <typename T>
struct array_t {
    bam_array_t h = nullptr;
    array_d_t<T>* d_array_ptr = nullptr;
    page_cache_t* cache = nullptr;

    array_t(const uint64_t num_elems, const uint64_t disk_start_offset, const std::vector<range_t<T>*>& ranges,
            uint32_t /*cudaDevice*/)
    {
        if (ranges.empty()) throw std::runtime_error("array_t: at least one range is needed");
        cache = ranges[0]->cache;
        (void)disk_start_offset;
        std::vector<bam_range_desc_t> descs;
        for (const range_t<T>* r : ranges) {
            if (r->cache != cache) throw std::runtime_error("array_t: all ranges must sit on one page cache");
            descs.push_back(bam_range_desc_t{ r->index_start, r->count, r->page_start * r->page_size, r->page_start_offset,
                                              (uint32_t)r->dist, 0u });
        }
        int rc = bam_array_create_ranges(&h, cache->h, num_elems, (uint32_t)sizeof(T), descs.data(), (uint32_t)descs.size());
        if (rc != 0) throw std::runtime_error(std::string("Failed to create array: ") + bam_strerror(rc));
        d_array_ptr = static_cast<array_d_t<T>*>(bam_array_device_ptr(h));
    }
    ~array_t() { if (h) bam_array_destroy(h); }
    array_t(const array_t&) = delete;
    array_t& operator=(const array_t&) = delete;

    void print_reset_stats()
    {
        bam_cache_stats_t s;
        bam_cache_stats(cache->h, &s, 1);
        const unsigned long long acc = s.hits + s.misses;
        printf("*********************************\n");
        printf("#READ IOs: %llu\t#Accesses:%llu\t#Misses:%llu\tMiss Rate:%f\t#Hits: %llu\tHit Rate:%f\n",
               (unsigned long long)s.read_ios, acc, (unsigned long long)s.misses, acc ? (double)s.misses / acc : 0.0,
               (unsigned long long)s.hits, acc ? (double)s.hits / acc : 0.0);
        printf("*********************************\n");
    }
};

#endif
