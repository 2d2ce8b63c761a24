/*
 * bam_graph.cu -- graph consumers of bam::array: level-synchronous BFS and label-propagation
 * connected components over a CSR graph whose row offsets AND column indices live in the backing
 * store and are read only through the page cache.
 *
 * Reference kernels: benchmarks/bfs/main.cu:658-689 and benchmarks/cc/main.cu:123-144, :595-617
 * (the "coalesce coarse ptr_pc" variants the published runs use).  There a warp walks one
 * vertex's 16-aligned neighbour list through a bam_ptr and the row offsets stay in plain GPU
 * memory.  Here a warp takes 32 consecutive vertices: their labels are one coalesced load, their
 * offsets one or two cached pages, and each active vertex's neighbour list is consumed page by
 * page -- one pin per 4 KiB page of edges for the whole warp, 256 contiguous bytes per step.
 *
 * One level / sweep = one fused launch (controller blocks + workers), so the host sees the
 * `changed` flag between launches exactly as the reference's drivers do (bfs/main.cu:1577-1736,
 * cc/main.cu:1418-1623).
 */
#include <cuda_runtime.h>

#include <cstddef>
#include <cstring>

#include "bam_abi.h"
#include "bam_synth.h"
#include "bam_fused.cuh"

using namespace bam;

#define BAM_BFS_INF 0xffffffffu

/* ---- scratch of one level / sweep: heavy adjacency lists split into work items ------------------
 * R-MAT degrees are heavily skewed; a hub's list of 10^5 edges walked by one warp page after page
 * would serialise hundreds of page reads.  Lists longer than BAM_HEAVY_EDGES are cut into items of
 * BAM_ITEM_EDGES edges that every warp consumes after its own vertices (no grid barrier: a warp
 * draws a ticket and waits for that item to be published, or for all producers to be done). */
#define BAM_HEAVY_EDGES 2048u
#define BAM_ITEM_EDGES 1024u

struct graph_item_t { uint64_t u; uint64_t begin; uint64_t end; };   /* end != 0 marks the item ready */
struct graph_scratch_t {
    uint32_t n_items, cursor, producers_done, capacity;
    graph_item_t items[1];
};

/* ---- edge weights (SSSP): edge j of the column array carries weight wt[j] (u32 array) --------------
 * A 4 KiB page of column indices holds 512 edges; their weights are 2 KiB, so they sit inside ONE page of
 * the weight array (weight page = column page >> 1 for equal page sizes).  The walkers below are written
 * once for both kinds of graph: Wt is wrange_t for a weighted graph and no_weights_t otherwise, and the
 * edge callback always receives a weight (0 without weights). */
typedef range_d_t<uint32_t> wrange_t;
struct no_weights_t {};

BAM_DEV const range_d_t<uint64_t>& as_u64_range(const wrange_t& w) { return reinterpret_cast<const range_d_t<uint64_t>&>(w); }
template <class Wt> struct has_weights { static constexpr bool value = false; };
template <> struct has_weights<wrange_t> { static constexpr bool value = true; };

/* The whole warp walks cols[begin, end) and calls fn(neighbour, weight) per edge.  Up to BAM_WALK_PAGES
 * column pages are pinned per step in ONE cooperative call (lane k asks for the k-th of them, lanes 16..
 * for the weight pages that go with them), so their reads are in flight together; then the warp consumes
 * them one after the other, 256 contiguous bytes of column indices per step. */
#ifndef BAM_WALK_PAGES
#define BAM_WALK_PAGES 4u
#endif
template <class Wt, class EdgeFn>
BAM_DEV bool warp_walk_edges(const range_d_t<uint64_t>& col, const Wt& wt, uint64_t begin, uint64_t end, uint32_t queue, EdgeFn fn)
{
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t epp_log = col.cache.page_size_log - 3;
    for (uint64_t i = begin; i < end;) {
        const uint64_t p0 = i >> epp_log;
        const uint64_t p_last = (end - 1) >> epp_log;
        const uint32_t np = p_last - p0 + 1 < BAM_WALK_PAGES ? (uint32_t)(p_last - p0 + 1) : BAM_WALK_PAGES;
        bool want = lane < np;
        uint64_t page = p0 + lane;
        uint64_t wp0 = 0;
        uint32_t wshift = 0;
        const range_d_t<uint64_t>* r = &col;
        if constexpr (has_weights<Wt>::value) {
            wshift = (wt.cache.page_size_log - 2) - epp_log;              /* column pages per weight page, log2 */
            wp0 = p0 >> wshift;
            const uint32_t nw = (uint32_t)(((p0 + np - 1) >> wshift) - wp0 + 1);
            if (lane >= 16) { r = &as_u64_range(wt); page = wp0 + (lane - 16); want = lane - 16 < nw; }
        }
        uint32_t slot = range_pin_page(*r, 0xffffffffu, want, page, 1, queue);
        const bool bad = __any_sync(0xffffffffu, want && slot == BAM_SLOT_ERR);
        if (!bad) {
            for (uint32_t k = 0; k < np; k++) {
                const uint32_t sl = __shfl_sync(0xffffffffu, slot, k);
                const uint64_t page_first = (p0 + k) << epp_log;
                const uint64_t lo = page_first > i ? page_first : i;
                uint64_t hi = page_first + (1ull << epp_log);
                if (hi > end) hi = end;
                const uint64_t* base = reinterpret_cast<const uint64_t*>(col.get_cache_page_addr(sl));
                if constexpr (has_weights<Wt>::value) {
                    const uint64_t wp = (p0 + k) >> wshift;
                    const uint32_t wsl = __shfl_sync(0xffffffffu, slot, 16 + (int)(wp - wp0));
                    const uint32_t* wbase = reinterpret_cast<const uint32_t*>(wt.get_cache_page_addr(wsl));
                    const uint64_t wfirst = wp << (wt.cache.page_size_log - 2);
                    for (uint64_t j = lo + lane; j < hi; j += 32) fn(base[j - page_first], wbase[j - wfirst]);
                } else {
                    for (uint64_t j = lo + lane; j < hi; j += 32) fn(base[j - page_first], 0u);
                }
            }
        }
        __syncwarp();
        if (want && slot <= BAM_SLOT_MAX) r->release_page(slot, 1);
        if (bad) return false;
        i = (p0 + np) << epp_log;
    }
    return true;
}

/* Row offsets [s, e) of the 32 consecutive vertices of a chunk (lane <-> vertex v; the whole warp calls it):
 * every lane reads off[v] once -- consecutive elements, mostly one cached page, read without a pin -- and
 * takes its end from the next lane; only the last lane's end is a second read.  Lanes with act == false
 * get s == e == 0.  Indices are clamped to the array (it has one entry per vertex plus one). */
BAM_DEV void chunk_offsets(const range_d_t<uint64_t>& off, uint64_t v, bool act, uint32_t queue, uint64_t& s, uint64_t& e)
{
#ifdef BAM_EXP_OLD_OFFSETS
    s = e = 0;
    if (act) { s = range_read<uint64_t>(off, v, queue); e = range_read<uint64_t>(off, v + 1, queue); }
    __syncwarp();
    return;
#endif
    const uint32_t lane = threadIdx.x & 31u;
    const uint64_t last = off.count - 1;                              /* largest valid index */
    const uint64_t v31 = __shfl_sync(0xffffffffu, v, 31) + 1;
    const uint64_t mine = range_read<uint64_t>(off, v < last ? v : last, queue);
    const uint64_t after = range_read<uint64_t>(off, v31 < last ? v31 : last, queue);
    const uint64_t next = __shfl_down_sync(0xffffffffu, mine, 1);
    s = act ? mine : 0;
    e = act ? (lane == 31 ? after : next) : 0;
}

/* One chunk of 32 consecutive local vertices (lane <-> vertex with row offsets [s, e), act = vertex is in
 * the frontier; s == e == 0 for the others).  Without weights the FIRST edge page of every active vertex is
 * pinned in one cooperative call (lanes that share a page share a pin, and all missing pages are in flight
 * together) and lists that continue on further pages are walked from there; with weights every vertex's
 * list is walked in turn (column and weight pages pinned together); heavy lists become work items.
 * fn(src_lane, neighbour, weight) is called for every edge. */
template <class Wt, class EdgeFn>
BAM_DEV bool chunk_visit(const range_d_t<uint64_t>& col, const Wt& wt, uint64_t s, uint64_t e, uint64_t u_global,
                         bool act, uint32_t queue, graph_scratch_t* scratch, uint64_t& edges, EdgeFn fn)
{
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t epp_log = col.cache.page_size_log - 3;
    const uint64_t deg = e - s;
    edges += deg;
    bool heavy = act && scratch && deg > BAM_HEAVY_EDGES;
    if (heavy) {
        /* items are cut at multiples of BAM_ITEM_EDGES of the edge index (whole pages), so no two items share
         * a page: the warps that draw neighbouring items at the same moment never miss on the same page */
        const uint64_t a0 = (s + BAM_ITEM_EDGES - 1) / BAM_ITEM_EDGES * BAM_ITEM_EDGES;     /* first cut after s */
        const uint32_t n_it = (uint32_t)((e - a0 + BAM_ITEM_EDGES - 1) / BAM_ITEM_EDGES) + (a0 > s ? 1u : 0u);
        const uint32_t base = atom_add_relaxed(&scratch->n_items, n_it);
        /* publish what fits (the scratch is sized so that everything does); anything beyond the
         * capacity is walked by this warp below, and tickets past the capacity are never waited on */
        const uint32_t fit = base >= scratch->capacity ? 0u : (scratch->capacity - base < n_it ? scratch->capacity - base : n_it);
        uint64_t b0 = s;
        for (uint32_t k = 0; k < fit; k++) {
            graph_item_t* it = &scratch->items[base + k];
            uint64_t b1 = (b0 / BAM_ITEM_EDGES + 1) * BAM_ITEM_EDGES;
            if (b1 > e) b1 = e;
            it->u = u_global;
            it->begin = b0;
            __threadfence();
            st_release_gpu(&it->end, b1);
            b0 = b1;
        }
        if (fit < n_it) { s = b0; heavy = false; }
    }
    const bool light = act && !heavy && e > s;
    const uint32_t lm = __ballot_sync(0xffffffffu, light);
    if (lm == 0) return true;
    bool ok = true;
    uint32_t am = lm;
    if constexpr (has_weights<Wt>::value) {
        while (am && ok) {
            const int src = __ffs(am) - 1;
            am &= am - 1;
            const uint64_t vs = __shfl_sync(0xffffffffu, s, src);
            const uint64_t ve = __shfl_sync(0xffffffffu, e, src);
            ok = warp_walk_edges(col, wt, vs, ve, queue, [&](uint64_t nb, uint32_t w) { fn(src, nb, w); });
        }
        __syncwarp();
        return ok;
    } else {
        const uint64_t page0 = s >> epp_log;
        const uint32_t eq = __match_any_sync(0xffffffffu, light ? page0 : (~0ull - lane));
        const uint32_t leader = __ffs(eq) - 1;
        uint32_t slot = range_pin_page(col, 0xffffffffu, light && lane == leader, page0, (uint32_t)__popc(eq), queue);
        slot = __shfl_sync(0xffffffffu, slot, leader);
        if (__any_sync(0xffffffffu, light && slot == BAM_SLOT_ERR)) return false;
        while (am) {
            const int src = __ffs(am) - 1;
            am &= am - 1;
            const uint64_t vs = __shfl_sync(0xffffffffu, s, src);
            const uint64_t ve = __shfl_sync(0xffffffffu, e, src);
            const uint32_t sl = __shfl_sync(0xffffffffu, slot, src);
            const uint64_t page_first = (vs >> epp_log) << epp_log;
            uint64_t first_end = page_first + (1ull << epp_log);
            if (first_end > ve) first_end = ve;
            const uint64_t* base = reinterpret_cast<const uint64_t*>(col.get_cache_page_addr(sl));
            for (uint64_t j = vs + lane; j < first_end; j += 32) fn(src, base[j - page_first], 0u);
            if (first_end < ve) ok = warp_walk_edges(col, wt, first_end, ve, queue, [&](uint64_t nb, uint32_t w) { fn(src, nb, w); }) && ok;
            if (!ok) break;
        }
        __syncwarp();
        if (light && lane == leader && slot != BAM_SLOT_ERR) col.release_page(slot, (uint32_t)__popc(eq));
        return ok;
    }
}

/* After its own chunks a warp helps with the heavy items.  fn(u_global, neighbour, weight) per edge. */
template <class Wt, class EdgeFn>
BAM_DEV void consume_heavy_items(const range_d_t<uint64_t>& col, const Wt& wt, graph_scratch_t* scratch, uint32_t n_warps_total,
                                 uint32_t queue, EdgeFn fn)
{
    if (!scratch) return;
    const uint32_t lane = threadIdx.x & 31u;
    if (lane == 0) { __threadfence(); red_add_release(&scratch->producers_done, 1u); }
    __syncwarp();
    for (;;) {
        uint32_t idx = 0;
        if (lane == 0) idx = atom_add_relaxed(&scratch->cursor, 1u);
        idx = __shfl_sync(0xffffffffu, idx, 0);
        if (idx >= scratch->capacity) return;
        graph_item_t* it = &scratch->items[idx];
        uint64_t end = 0;
        spin_t sp;
        for (;;) {                                         /* the item is published, or it will never be */
            uint32_t done = 0;
            if (lane == 0) {
                end = ld_acquire_gpu(&it->end);
                if (end == 0 && ld_acquire_gpu(&scratch->producers_done) == n_warps_total &&
                    ld_acquire_gpu(&scratch->n_items) <= idx) done = 1;
                if (end == 0 && !done) end = ld_acquire_gpu(&it->end);
            }
            end = __shfl_sync(0xffffffffu, end, 0);
            done = __shfl_sync(0xffffffffu, done, 0);
            if (end != 0) break;
            if (done) return;
            if (__any_sync(0xffffffffu, sp.expired(col.cache.status, BAM_AT_PAGE_BUSY, idx))) return;
        }
        const uint64_t u = it->u, begin = it->begin;
        if (!warp_walk_edges(col, wt, begin, end, queue, [&](uint64_t nb, uint32_t w) { fn(u, nb, w); })) return;
    }
}

/* The sweep of one warp over its chunks of 32 consecutive vertices [c0, c0 + 32), c0 = v_begin + 32 (warp +
 * k n_warps): chunks without an active vertex are skipped, and the row offsets of the warp's next chunk with
 * active vertices are read before the current chunk is processed (the two offset reads are out of the way
 * when its turn comes).  Starting the page reads of the next chunk's first edge pages at that point as well
 * was tried and gave nothing measurable: the traversals are not bound by one warp's chain of waits.
 * active(v) says whether local vertex v takes part
 * (it is called once per vertex and may clear the vertex's flag); fn(c0, src_lane, neighbour, weight) is
 * called for every edge of an active vertex c0 + src_lane.  Ends with the warp's share of the heavy items. */
template <class Wt, class ActiveFn, class EdgeFn>
BAM_DEV void sweep_chunks(const range_d_t<uint64_t>& off, const range_d_t<uint64_t>& col, const Wt& wt, uint64_t v_begin, uint64_t v_end,
                          uint64_t v_base, uint64_t warp, uint64_t nwarps, graph_scratch_t* scratch, uint64_t& edges, ActiveFn active,
                          EdgeFn fn)
{
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t queue = (uint32_t)warp;
    struct chunk_t { uint64_t c0, s, e; bool act; };
    auto advance = [&](uint64_t from, chunk_t& ch) {
        for (uint64_t c0 = from; c0 < v_end; c0 += nwarps * 32) {
            const uint64_t v = c0 + lane;
            const bool act = v < v_end && active(v);
            if (__ballot_sync(0xffffffffu, act) == 0u) continue;
            ch.c0 = c0; ch.act = act;
            chunk_offsets(off, v, act, queue, ch.s, ch.e);
            return true;
        }
        return false;
    };
    chunk_t cur, nxt;
    bool have = advance(v_begin + warp * 32, cur);
    while (have) {
        const bool have_next = advance(cur.c0 + nwarps * 32, nxt);
        const uint64_t c0 = cur.c0;
        const bool ok = chunk_visit(col, wt, cur.s, cur.e, v_base + c0 + lane, cur.act, queue, scratch, edges,
                                    [&](int src, uint64_t nb, uint32_t w) { fn(c0, src, nb, w); });
        if (!ok) break;
        cur = nxt;
        have = have_next;
    }
    consume_heavy_items(col, wt, scratch, (uint32_t)nwarps, queue, [&](uint64_t u, uint64_t nb, uint32_t w) { fn(u - v_base, 0, nb, w); });
}

struct BfsLevelWork {
    range_d_t<uint64_t> off, col;
    uint64_t v_begin, v_end;
    uint64_t v_base;            /* global id of local vertex 0 (labels are indexed by global id) */
    uint32_t level;
    uint32_t* label;
    uint32_t* changed;
    uint64_t* scanned;
    graph_scratch_t* scratch;

    __device__ void operator()(uint32_t vb, uint32_t nvb) const
    {
        const uint32_t lane = threadIdx.x & 31u;
        const uint32_t wpb = blockDim.x >> 5;
        const uint64_t warp = (uint64_t)vb * wpb + (threadIdx.x >> 5);
        const uint64_t nwarps = (uint64_t)nvb * wpb;
        uint64_t edges = 0;
        bool ch = false;
        uint32_t* lab = label;
        const uint32_t next_level = level + 1;
        auto relax = [&](uint64_t nb) {
            if (lab[nb] == BAM_BFS_INF) { lab[nb] = next_level; ch = true; }
        };
        const uint32_t* labc = label;
        const uint64_t vb0 = v_base;
        const uint32_t lv = level;
        sweep_chunks(off, col, no_weights_t{}, v_begin, v_end, v_base, warp, nwarps, scratch, edges,
                     [&](uint64_t v) { return labc[vb0 + v] == lv; },
                     [&](uint64_t, int, uint64_t nb, uint32_t) { relax(nb); });
        __syncwarp();
        if (__any_sync(0xffffffffu, ch) && lane == 0) *changed = 1u;
        warp_sum_to(edges, scanned);
    }
};

struct CcSweepWork {
    range_d_t<uint64_t> off, col;
    uint64_t v_begin, v_end;
    uint64_t v_base;
    unsigned long long* comp;
    const uint8_t* curr_visit;
    uint8_t* next_visit;
    uint32_t* changed;
    uint64_t* scanned;
    graph_scratch_t* scratch;

    __device__ void operator()(uint32_t vb, uint32_t nvb) const
    {
        const uint32_t lane = threadIdx.x & 31u;
        const uint32_t wpb = blockDim.x >> 5;
        const uint64_t warp = (uint64_t)vb * wpb + (threadIdx.x >> 5);
        const uint64_t nwarps = (uint64_t)nvb * wpb;
        uint64_t edges = 0;
        bool ch = false;
        unsigned long long* cp = comp;
        uint8_t* nv = next_visit;
        /* the relaxation of cc_compute: the larger label takes the smaller one */
        auto relax = [&](uint64_t u, uint64_t nb) {
            const unsigned long long cu = *reinterpret_cast<volatile unsigned long long*>(&cp[u]);
            const unsigned long long cn = *reinterpret_cast<volatile unsigned long long*>(&cp[nb]);
            if (cu < cn) { atomicMin(&cp[nb], cu); nv[nb] = 1; ch = true; }
            else if (cn < cu) { atomicMin(&cp[u], cn); nv[u] = 1; ch = true; }
        };
        const uint8_t* cv = curr_visit;
        const uint64_t vb0 = v_base;
        sweep_chunks(off, col, no_weights_t{}, v_begin, v_end, v_base, warp, nwarps, scratch, edges,
                     [&](uint64_t v) { return cv[vb0 + v] != 0; },
                     [&](uint64_t c0, int src, uint64_t nb, uint32_t) { relax(vb0 + c0 + src, nb); });
        __syncwarp();
        if (__any_sync(0xffffffffu, ch) && lane == 0) *changed = 1u;
        warp_sum_to(edges, scanned);
    }
};

/* One relaxation sweep of label-correcting single-source shortest paths (benchmarks/sssp/main.cu:
 * 115-146, 174-202: kernel_*_pc): every vertex flagged in `label` offers cost + weight to its
 * neighbours with atomicMin on new_cost and clears its flag.  The reference samples the vertex's
 * cost once and leaves the loop when it changes; here the current value is read per edge, which
 * offers the same or a better bound (every value new_cost ever holds is the length of a real path). */
struct SsspSweepWork {
    range_d_t<uint64_t> off, col;
    wrange_t wt;
    uint64_t v_begin, v_end;
    uint64_t v_base;            /* global id of local vertex 0 (label and new_cost are indexed by global id) */
    uint8_t* label;
    uint32_t* new_cost;
    uint64_t* scanned;
    graph_scratch_t* scratch;

    __device__ void operator()(uint32_t vb, uint32_t nvb) const
    {
        const uint32_t wpb = blockDim.x >> 5;
        const uint64_t warp = (uint64_t)vb * wpb + (threadIdx.x >> 5);
        const uint64_t nwarps = (uint64_t)nvb * wpb;
        uint64_t edges = 0;
        uint32_t* nc = new_cost;
        auto relax = [&](uint64_t u, uint64_t nb, uint32_t w) {
            const uint32_t cand = *reinterpret_cast<volatile uint32_t*>(&nc[u]) + w;
            if (*reinterpret_cast<volatile uint32_t*>(&nc[nb]) > cand) atomicMin(&nc[nb], cand);
        };
        uint8_t* lb = label;
        const uint64_t vb0 = v_base;
        sweep_chunks(off, col, wt, v_begin, v_end, v_base, warp, nwarps, scratch, edges,
                     [&](uint64_t v) { const bool a = lb[vb0 + v] != 0; if (a) lb[vb0 + v] = 0; return a; },
                     [&](uint64_t c0, int src, uint64_t nb, uint32_t w) { relax(vb0 + c0 + src, nb, w); });
        warp_sum_to(edges, scanned);
    }
};

/* update of benchmarks/sssp/main.cu:282-292: a vertex whose tentative cost fell becomes active */
__global__ void k_sssp_update(uint8_t* label, uint32_t* cost, const uint32_t* new_cost, uint64_t n, uint32_t* changed)
{
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x, nthr = (uint64_t)gridDim.x * blockDim.x;
    bool ch = false;
    for (uint64_t i = tid; i < n; i += nthr)
        if (new_cost[i] < cost[i]) { cost[i] = new_cost[i]; label[i] = 1; ch = true; }
    if (ch) *changed = 1u;
}

__global__ void k_sssp_init(uint8_t* label, uint32_t* cost, uint32_t* new_cost, uint64_t n, uint64_t src)
{
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x, nthr = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = tid; i < n; i += nthr) {
        const bool is = i == src;
        label[i] = is ? 1 : 0;
        cost[i] = new_cost[i] = is ? 0u : BAM_BFS_INF;
    }
}

/* ---- PageRank (benchmarks/pagerank/main.cu:107-115 initialize, :137-160 / :252-274 kernel_*_pc,
 * :412-421 update): push-based delta PageRank.  Every active vertex adds delta[v] to the residual
 * of each neighbour; a vertex whose residual exceeds the tolerance folds it into its value and
 * becomes active with delta = residual * alpha / degree.
 * The reference computes in float with atomicAdd, so its result depends on the order the adds
 * happen to land in.  Here every quantity is a 64-bit fixed-point number with BAM_PR_FRAC_BITS
 * fraction bits and alpha is a ratio of integers: integer adds commute, so the result is
 * bit-identical for every schedule, every grid size and a sequential CPU run. */
struct PrSweepWork {
    range_d_t<uint64_t> off, col;
    uint64_t v_begin, v_end;
    uint64_t v_base;            /* global id of local vertex 0 (label, delta and residual are indexed by global id) */
    uint8_t* label;
    const uint64_t* delta;
    unsigned long long* residual;
    uint64_t* scanned;
    graph_scratch_t* scratch;

    __device__ void operator()(uint32_t vb, uint32_t nvb) const
    {
        const uint32_t wpb = blockDim.x >> 5;
        const uint64_t warp = (uint64_t)vb * wpb + (threadIdx.x >> 5);
        const uint64_t nwarps = (uint64_t)nvb * wpb;
        uint64_t edges = 0;
        unsigned long long* res = residual;
        const uint64_t* dl = delta;
        auto push = [&](uint64_t u, uint64_t nb) { atomicAdd(&res[nb], (unsigned long long)dl[u]); };
        uint8_t* lb = label;
        const uint64_t vb0 = v_base;
        sweep_chunks(off, col, no_weights_t{}, v_begin, v_end, v_base, warp, nwarps, scratch, edges,
                     [&](uint64_t v) { const bool a = lb[vb0 + v] != 0; if (a) lb[vb0 + v] = 0; return a; },
                     [&](uint64_t c0, int src, uint64_t nb, uint32_t) { push(vb0 + c0 + src, nb); });
        warp_sum_to(edges, scanned);
    }
};

/* degree of every vertex, read once through the cache (the reference keeps the row offsets in
 * plain GPU memory for its initialize / update kernels) */
struct DegreeWork {
    range_d_t<uint64_t> off;
    uint64_t n;
    uint32_t* deg;

    __device__ void operator()(uint32_t vb, uint32_t nvb) const
    {
        const uint64_t nthr = (uint64_t)nvb * blockDim.x;
        const uint32_t queue = (uint32_t)(((uint64_t)vb * blockDim.x + threadIdx.x) >> 5);
        for (uint64_t c0 = (uint64_t)vb * blockDim.x + (threadIdx.x & ~31u); c0 < n; c0 += nthr) {
            const uint64_t v = c0 + (threadIdx.x & 31u);
            if (v < n) {
                const uint64_t s = range_read<uint64_t>(off, v, queue);
                const uint64_t e = range_read<uint64_t>(off, v + 1, queue);
                deg[v] = (uint32_t)(e - s);
            }
            __syncwarp();
        }
    }
};

__global__ void k_pr_init(uint8_t* label, uint64_t* delta, uint64_t* residual, uint64_t* value, const uint32_t* deg, uint64_t n,
                          uint64_t alpha_num, uint64_t alpha_den)
{
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x, nthr = (uint64_t)gridDim.x * blockDim.x;
    const uint64_t one = 1ull << BAM_PR_FRAC_BITS;
    const uint64_t base = one - bam_mul_ratio(one, alpha_num, alpha_den);  /* 1 - alpha */
    for (uint64_t i = tid; i < n; i += nthr) {
        value[i] = base;
        delta[i] = deg[i] ? bam_mul_ratio(base, alpha_num, alpha_den) / deg[i] : 0;
        residual[i] = 0;
        label[i] = 1;
    }
}

__global__ void k_pr_update(uint8_t* label, uint64_t* delta, uint64_t* residual, uint64_t* value, const uint32_t* deg, uint64_t n,
                            uint64_t tolerance, uint64_t alpha_num, uint64_t alpha_den, uint32_t* changed)
{
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x, nthr = (uint64_t)gridDim.x * blockDim.x;
    bool ch = false;
    for (uint64_t i = tid; i < n; i += nthr) {
        const uint64_t r = residual[i];
        if (r > tolerance) {
            value[i] += r;
            delta[i] = deg[i] ? bam_mul_ratio(r, alpha_num, alpha_den) / deg[i] : 0;
            residual[i] = 0;
            label[i] = 1;
            ch = true;
        }
    }
    if (ch) *changed = 1u;
}

__global__ void k_bfs_init(uint32_t* label, uint64_t n, uint64_t src)
{
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x, nthr = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = tid; i < n; i += nthr) label[i] = (i == src) ? 0u : BAM_BFS_INF;
}

__global__ void k_cc_init(unsigned long long* comp, uint8_t* curr, uint8_t* next, uint64_t n)
{
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x, nthr = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = tid; i < n; i += nthr) { comp[i] = i; curr[i] = 1; next[i] = 0; }
}

/* R-MAT edge e -> the two directed keys (u<<32|v), (v<<32|u); a self loop gives two ~0 keys
 * (sorted to the end and dropped by the caller). */
__global__ void k_rmat_keys(uint64_t* keys, uint64_t e_begin, uint64_t e_end, uint64_t seed, uint32_t scale, bam_rmat_thresh_t t)
{
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x, nthr = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t e = e_begin + tid; e < e_end; e += nthr) {
        uint64_t u, v;
        bam_rmat_edge(seed, e, scale, t, &u, &v);
        const uint64_t k = 2 * (e - e_begin);
        if (u == v) { keys[k] = ~0ull; keys[k + 1] = ~0ull; }
        else { keys[k] = (u << 32) | v; keys[k + 1] = (v << 32) | u; }
    }
}

/* Clear the level's scratch (header and item flags) on the stream and set its capacity. */
static int prepare_scratch(void* scratch_dev, uint64_t scratch_bytes, cudaStream_t s, graph_scratch_t** out)
{
    *out = nullptr;
    if (!scratch_dev) return BAM_OK;
    if (scratch_bytes < sizeof(graph_scratch_t) + sizeof(graph_item_t)) return BAM_EINVAL;
    const uint64_t cap = (scratch_bytes - offsetof(graph_scratch_t, items)) / sizeof(graph_item_t);
    CK(cudaMemsetAsync(scratch_dev, 0, scratch_bytes, s));
    const uint32_t cap32 = cap > 0x7fffffffu ? 0x7fffffffu : (uint32_t)cap;
    CK(cudaMemcpyAsync((uint8_t*)scratch_dev + offsetof(graph_scratch_t, capacity), &cap32, 4, cudaMemcpyHostToDevice, s));
    *out = static_cast<graph_scratch_t*>(scratch_dev);
    return BAM_OK;
}

extern "C" uint64_t bam_graph_scratch_bytes(uint64_t n_edges)
{
    /* a heavy list of d edges gives at most d / BAM_ITEM_EDGES + 2 items, and there are at most n_edges / BAM_HEAVY_EDGES heavy lists */
    return offsetof(graph_scratch_t, items) + (n_edges / BAM_ITEM_EDGES + 2 * (n_edges / BAM_HEAVY_EDGES) + 1024) * sizeof(graph_item_t);
}

static int check_graph_args(bam_array_t offsets, bam_array_t cols)
{
    if (!offsets || !cols) return BAM_EINVAL;
    if (offsets->elem_bytes != 8 || cols->elem_bytes != 8) return BAM_EINVAL;
    if (offsets->pc != cols->pc) return BAM_EINVAL;
    /* the traversal kernels take each array's one range by value and walk whole pages of it */
    if (offsets->n_ranges != 1 || cols->n_ranges != 1 || offsets->h_range.page_start_offset || cols->h_range.page_start_offset) return BAM_EINVAL;
    return BAM_OK;
}

extern "C" int bam_launch_bfs_level(bam_array_t offsets, bam_array_t cols, uint64_t v_begin, uint64_t v_end, uint64_t v_base,
                                    uint32_t level, uint32_t* label_dev, uint32_t* changed_dev, uint64_t* scanned_dev,
                                    void* scratch_dev, uint64_t scratch_bytes, void* stream)
{
    int rc = check_graph_args(offsets, cols);
    if (rc) return rc;
    if (!label_dev || !changed_dev || v_end > offsets->n_elems - 1 || v_begin > v_end) return BAM_EINVAL;
    bam_ctrl* c = offsets->pc->ctrl;
    CK(cudaSetDevice(c->device));
    BfsLevelWork w;
    w.off = offsets->h_range; w.col = cols->h_range; w.v_begin = v_begin; w.v_end = v_end; w.v_base = v_base; w.level = level;
    w.label = label_dev; w.changed = changed_dev; w.scanned = scanned_dev;
    w.scratch = nullptr;
    rc = prepare_scratch(scratch_dev, scratch_bytes, (cudaStream_t)stream, &w.scratch);
    if (rc) return rc;
    return launch_fused(c, w, (cudaStream_t)stream);
}

extern "C" int bam_launch_cc_sweep(bam_array_t offsets, bam_array_t cols, uint64_t v_begin, uint64_t v_end, uint64_t v_base,
                                   uint64_t* comp_dev, const uint8_t* curr_visit_dev, uint8_t* next_visit_dev,
                                   uint32_t* changed_dev, uint64_t* scanned_dev, void* scratch_dev, uint64_t scratch_bytes,
                                   void* stream)
{
    int rc = check_graph_args(offsets, cols);
    if (rc) return rc;
    if (!comp_dev || !curr_visit_dev || !next_visit_dev || !changed_dev || v_end > offsets->n_elems - 1 || v_begin > v_end) return BAM_EINVAL;
    bam_ctrl* c = offsets->pc->ctrl;
    CK(cudaSetDevice(c->device));
    CcSweepWork w;
    w.off = offsets->h_range; w.col = cols->h_range; w.v_begin = v_begin; w.v_end = v_end; w.v_base = v_base;
    w.comp = reinterpret_cast<unsigned long long*>(comp_dev); w.curr_visit = curr_visit_dev; w.next_visit = next_visit_dev;
    w.changed = changed_dev; w.scanned = scanned_dev;
    w.scratch = nullptr;
    rc = prepare_scratch(scratch_dev, scratch_bytes, (cudaStream_t)stream, &w.scratch);
    if (rc) return rc;
    return launch_fused(c, w, (cudaStream_t)stream);
}

/* Whole traversals on one GPU: the host loops of benchmarks/bfs/main.cu:1577-1736 and
 * benchmarks/cc/main.cu:1418-1623 (launch, read `changed`, repeat). */
extern "C" int bam_bfs_run(bam_array_t offsets, bam_array_t cols, uint64_t n_vertices, uint64_t source,
                           uint32_t* label_dev, uint32_t* n_levels_out, uint64_t* edges_scanned_out)
{
    int rc = check_graph_args(offsets, cols);
    if (rc) return rc;
    if (!label_dev || source >= n_vertices || n_vertices + 1 > offsets->n_elems) return BAM_EINVAL;
    bam_ctrl* c = offsets->pc->ctrl;
    CK(cudaSetDevice(c->device));
    uint32_t* d_changed = nullptr;
    uint64_t* d_scanned = nullptr;
    CK(cudaMalloc(&d_changed, 4));
    cudaError_t e = cudaMalloc(&d_scanned, 8);
    if (e != cudaSuccess) { cudaFree(d_changed); g_last_cuda = e; return BAM_ENOMEM; }
    cudaMemset(d_scanned, 0, 8);
    void* d_scratch = nullptr;
    const uint64_t scratch_bytes = bam_graph_scratch_bytes(cols->n_elems);
    if (cudaMalloc(&d_scratch, scratch_bytes) != cudaSuccess) { (void)cudaGetLastError(); d_scratch = nullptr; }
    k_bfs_init<<<c->num_sms * 4, 256>>>(label_dev, n_vertices, source);
    uint32_t level = 0;
    rc = BAM_OK;
    for (;; level++) {
        cudaMemsetAsync(d_changed, 0, 4, 0);
        rc = bam_launch_bfs_level(offsets, cols, 0, n_vertices, 0, level, label_dev, d_changed, d_scanned, d_scratch, d_scratch ? scratch_bytes : 0, nullptr);
        if (rc) break;
        uint32_t changed = 0;
        e = cudaMemcpy(&changed, d_changed, 4, cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) { g_last_cuda = e; rc = BAM_ECUDA; break; }
        bam_status_t st;
        cudaMemcpy(&st, c->d_status, sizeof st, cudaMemcpyDeviceToHost);
        if (st.code) { rc = (int)st.code; break; }
        if (!changed) break;
    }
    if (n_levels_out) *n_levels_out = level + 1;              /* levels 0..level hold vertices */
    if (edges_scanned_out) cudaMemcpy(edges_scanned_out, d_scanned, 8, cudaMemcpyDeviceToHost);
    cudaFree(d_changed); cudaFree(d_scanned); cudaFree(d_scratch);
    return rc;
}

extern "C" int bam_cc_run(bam_array_t offsets, bam_array_t cols, uint64_t n_vertices, uint64_t* comp_dev,
                          uint32_t* n_sweeps_out, uint64_t* edges_scanned_out)
{
    int rc = check_graph_args(offsets, cols);
    if (rc) return rc;
    if (!comp_dev || n_vertices + 1 > offsets->n_elems) return BAM_EINVAL;
    bam_ctrl* c = offsets->pc->ctrl;
    CK(cudaSetDevice(c->device));
    uint32_t* d_changed = nullptr;
    uint64_t* d_scanned = nullptr;
    uint8_t* d_visit = nullptr;
    cudaError_t e = cudaMalloc(&d_changed, 4);
    if (e == cudaSuccess) e = cudaMalloc(&d_scanned, 8);
    if (e == cudaSuccess) e = cudaMalloc(&d_visit, 2 * n_vertices);
    if (e != cudaSuccess) { cudaFree(d_changed); cudaFree(d_scanned); cudaFree(d_visit); g_last_cuda = e; (void)cudaGetLastError(); return BAM_ENOMEM; }
    cudaMemset(d_scanned, 0, 8);
    void* d_scratch = nullptr;
    const uint64_t scratch_bytes = bam_graph_scratch_bytes(cols->n_elems);
    if (cudaMalloc(&d_scratch, scratch_bytes) != cudaSuccess) { (void)cudaGetLastError(); d_scratch = nullptr; }
    uint8_t* curr = d_visit;
    uint8_t* next = d_visit + n_vertices;
    k_cc_init<<<c->num_sms * 4, 256>>>(reinterpret_cast<unsigned long long*>(comp_dev), curr, next, n_vertices);
    uint32_t sweeps = 0;
    rc = BAM_OK;
    for (;;) {
        cudaMemsetAsync(d_changed, 0, 4, 0);
        rc = bam_launch_cc_sweep(offsets, cols, 0, n_vertices, 0, comp_dev, curr, next, d_changed, d_scanned, d_scratch, d_scratch ? scratch_bytes : 0, nullptr);
        if (rc) break;
        sweeps++;
        uint32_t changed = 0;
        e = cudaMemcpy(&changed, d_changed, 4, cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) { g_last_cuda = e; rc = BAM_ECUDA; break; }
        bam_status_t st;
        cudaMemcpy(&st, c->d_status, sizeof st, cudaMemcpyDeviceToHost);
        if (st.code) { rc = (int)st.code; break; }
        if (!changed) break;
        cudaMemsetAsync(curr, 0, n_vertices, 0);              /* the visited set becomes the next one */
        uint8_t* t = curr; curr = next; next = t;
    }
    if (n_sweeps_out) *n_sweeps_out = sweeps;
    if (edges_scanned_out) cudaMemcpy(edges_scanned_out, d_scanned, 8, cudaMemcpyDeviceToHost);
    cudaFree(d_changed); cudaFree(d_scanned); cudaFree(d_visit); cudaFree(d_scratch);
    return rc;
}

extern "C" int bam_gen_rmat_keys(uint64_t* keys_dev, uint64_t e_begin, uint64_t e_end, uint64_t seed, uint32_t scale,
                                 uint32_t ta, uint32_t tab, uint32_t tabc, void* stream)
{
    if (!keys_dev || e_end < e_begin || scale == 0 || scale > 31) return BAM_EINVAL;
    bam_rmat_thresh_t t = { ta, tab, tabc };
    k_rmat_keys<<<1184, 256, 0, (cudaStream_t)stream>>>(keys_dev, e_begin, e_end, seed, scale, t);
    CK(cudaGetLastError());
    return BAM_OK;
}

extern "C" int bam_ctrl_write_store_from_device(bam_ctrl_t c, uint64_t byte_offset, const void* src_dev, uint64_t bytes, void* stream)
{
    if (!c || !src_dev || byte_offset + bytes > c->store_bytes || byte_offset + bytes < byte_offset) return BAM_EINVAL;
    CK(cudaSetDevice(c->device));
    CK(cudaMemcpyAsync(c->store_host + byte_offset, src_dev, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    return BAM_OK;
}

/* ---- SSSP and PageRank drivers ------------------------------------------------------------------ */

extern "C" int bam_launch_sssp_sweep(bam_array_t offsets, bam_array_t cols, bam_array_t weights, uint64_t v_begin, uint64_t v_end,
                                     uint64_t v_base, uint8_t* label_dev, uint32_t* new_cost_dev, uint64_t* scanned_dev, void* scratch_dev,
                                     uint64_t scratch_bytes, void* stream)
{
    int rc = check_graph_args(offsets, cols);
    if (rc) return rc;
    if (!weights || weights->elem_bytes != 4 || weights->pc != cols->pc || weights->n_elems < cols->n_elems) return BAM_EINVAL;
    if (!label_dev || !new_cost_dev || v_end > offsets->n_elems - 1 || v_begin > v_end) return BAM_EINVAL;
    bam_ctrl* c = offsets->pc->ctrl;
    CK(cudaSetDevice(c->device));
    SsspSweepWork w;
    w.off = offsets->h_range; w.col = cols->h_range;
    static_assert(sizeof(wrange_t) == sizeof(range_d_t<uint64_t>), "range descriptors share one layout");
    memcpy(&w.wt, &weights->h_range, sizeof w.wt);
    w.v_begin = v_begin; w.v_end = v_end; w.v_base = v_base; w.label = label_dev; w.new_cost = new_cost_dev; w.scanned = scanned_dev;
    w.scratch = nullptr;
    rc = prepare_scratch(scratch_dev, scratch_bytes, (cudaStream_t)stream, &w.scratch);
    if (rc) return rc;
    return launch_fused(c, w, (cudaStream_t)stream);
}

/* The host loop of benchmarks/sssp/main.cu:640-720: sweep, update, repeat until nothing changed. */
extern "C" int bam_sssp_run(bam_array_t offsets, bam_array_t cols, bam_array_t weights, uint64_t n_vertices, uint64_t source,
                            uint32_t* cost_dev, uint32_t* n_iters_out, uint64_t* edges_scanned_out)
{
    int rc = check_graph_args(offsets, cols);
    if (rc) return rc;
    if (!weights || !cost_dev || source >= n_vertices || n_vertices + 1 > offsets->n_elems) return BAM_EINVAL;
    bam_ctrl* c = offsets->pc->ctrl;
    CK(cudaSetDevice(c->device));
    uint8_t* d_buf = nullptr;          /* new_cost (4n) | label (n) | changed (4) | scanned (8), 16-byte aligned parts */
    const uint64_t o_label = (4 * n_vertices + 15) / 16 * 16, o_changed = (o_label + n_vertices + 15) / 16 * 16, o_scanned = o_changed + 8;
    cudaError_t e = cudaMalloc(&d_buf, o_scanned + 8);
    if (e != cudaSuccess) { g_last_cuda = e; (void)cudaGetLastError(); return BAM_ENOMEM; }
    uint32_t* d_new = reinterpret_cast<uint32_t*>(d_buf);
    uint8_t* d_label = d_buf + o_label;
    uint32_t* d_changed = reinterpret_cast<uint32_t*>(d_buf + o_changed);
    uint64_t* d_scanned = reinterpret_cast<uint64_t*>(d_buf + o_scanned);
    cudaMemset(d_scanned, 0, 8);
    void* d_scratch = nullptr;
    const uint64_t scratch_bytes = bam_graph_scratch_bytes(cols->n_elems);
    if (cudaMalloc(&d_scratch, scratch_bytes) != cudaSuccess) { (void)cudaGetLastError(); d_scratch = nullptr; }
    k_sssp_init<<<c->num_sms * 4, 256>>>(d_label, cost_dev, d_new, n_vertices, source);
    uint32_t iters = 0;
    rc = BAM_OK;
    for (;;) {
        rc = bam_launch_sssp_sweep(offsets, cols, weights, 0, n_vertices, 0, d_label, d_new, d_scanned, d_scratch,
                                   d_scratch ? scratch_bytes : 0, nullptr);
        if (rc) break;
        iters++;
        cudaMemsetAsync(d_changed, 0, 4, 0);
        k_sssp_update<<<c->num_sms * 4, 256>>>(d_label, cost_dev, d_new, n_vertices, d_changed);
        uint32_t changed = 0;
        e = cudaMemcpy(&changed, d_changed, 4, cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) { g_last_cuda = e; rc = BAM_ECUDA; break; }
        bam_status_t st;
        cudaMemcpy(&st, c->d_status, sizeof st, cudaMemcpyDeviceToHost);
        if (st.code) { rc = (int)st.code; break; }
        if (!changed) break;
    }
    if (n_iters_out) *n_iters_out = iters;
    if (edges_scanned_out) cudaMemcpy(edges_scanned_out, d_scanned, 8, cudaMemcpyDeviceToHost);
    cudaFree(d_buf); cudaFree(d_scratch);
    return rc;
}

extern "C" int bam_launch_pr_sweep(bam_array_t offsets, bam_array_t cols, uint64_t v_begin, uint64_t v_end, uint64_t v_base,
                                   uint8_t* label_dev,
                                   const uint64_t* delta_dev, uint64_t* residual_dev, uint64_t* scanned_dev, void* scratch_dev,
                                   uint64_t scratch_bytes, void* stream)
{
    int rc = check_graph_args(offsets, cols);
    if (rc) return rc;
    if (!label_dev || !delta_dev || !residual_dev || v_end > offsets->n_elems - 1 || v_begin > v_end) return BAM_EINVAL;
    bam_ctrl* c = offsets->pc->ctrl;
    CK(cudaSetDevice(c->device));
    PrSweepWork w;
    w.off = offsets->h_range; w.col = cols->h_range; w.v_begin = v_begin; w.v_end = v_end; w.v_base = v_base;
    w.label = label_dev; w.delta = delta_dev; w.residual = reinterpret_cast<unsigned long long*>(residual_dev); w.scanned = scanned_dev;
    w.scratch = nullptr;
    rc = prepare_scratch(scratch_dev, scratch_bytes, (cudaStream_t)stream, &w.scratch);
    if (rc) return rc;
    return launch_fused(c, w, (cudaStream_t)stream);
}

extern "C" int bam_launch_degrees(bam_array_t offsets, uint64_t n_vertices, uint32_t* deg_dev, void* stream)
{
    if (!offsets || offsets->elem_bytes != 8 || !deg_dev || n_vertices + 1 > offsets->n_elems) return BAM_EINVAL;
    bam_ctrl* c = offsets->pc->ctrl;
    CK(cudaSetDevice(c->device));
    DegreeWork w;
    w.off = offsets->h_range; w.n = n_vertices; w.deg = deg_dev;
    return launch_fused(c, w, (cudaStream_t)stream);
}

/* The host loop of benchmarks/pagerank/main.cu:678-772: initialize, then sweep + update until no
 * residual exceeds the tolerance or max_iters sweeps have run (the reference stops at 100). */
extern "C" int bam_pagerank_run(bam_array_t offsets, bam_array_t cols, uint64_t n_vertices, uint64_t alpha_num, uint64_t alpha_den,
                                uint64_t tolerance_q, uint32_t max_iters, uint64_t* value_dev, uint32_t* n_iters_out,
                                uint64_t* edges_scanned_out)
{
    int rc = check_graph_args(offsets, cols);
    if (rc) return rc;
    if (!value_dev || n_vertices + 1 > offsets->n_elems || alpha_den == 0 || alpha_num >= alpha_den || alpha_den > (1u << 20)) return BAM_EINVAL;
    bam_ctrl* c = offsets->pc->ctrl;
    CK(cudaSetDevice(c->device));
    uint8_t* d_buf = nullptr;          /* delta (8n) | residual (8n) | deg (4n) | label (n) | changed | scanned */
    const uint64_t o_res = 8 * n_vertices, o_deg = 16 * n_vertices, o_label = 20 * n_vertices;
    const uint64_t o_changed = (o_label + n_vertices + 15) / 16 * 16, o_scanned = o_changed + 8;
    cudaError_t e = cudaMalloc(&d_buf, o_scanned + 8);
    if (e != cudaSuccess) { g_last_cuda = e; (void)cudaGetLastError(); return BAM_ENOMEM; }
    uint64_t* d_delta = reinterpret_cast<uint64_t*>(d_buf);
    uint64_t* d_res = reinterpret_cast<uint64_t*>(d_buf + o_res);
    uint32_t* d_deg = reinterpret_cast<uint32_t*>(d_buf + o_deg);
    uint8_t* d_label = d_buf + o_label;
    uint32_t* d_changed = reinterpret_cast<uint32_t*>(d_buf + o_changed);
    uint64_t* d_scanned = reinterpret_cast<uint64_t*>(d_buf + o_scanned);
    cudaMemset(d_scanned, 0, 8);
    void* d_scratch = nullptr;
    const uint64_t scratch_bytes = bam_graph_scratch_bytes(cols->n_elems);
    if (cudaMalloc(&d_scratch, scratch_bytes) != cudaSuccess) { (void)cudaGetLastError(); d_scratch = nullptr; }
    uint32_t iters = 0;
    rc = bam_launch_degrees(offsets, n_vertices, d_deg, nullptr);
    if (rc == BAM_OK) {
        k_pr_init<<<c->num_sms * 4, 256>>>(d_label, d_delta, d_res, value_dev, d_deg, n_vertices, alpha_num, alpha_den);
        while (iters < max_iters) {
            rc = bam_launch_pr_sweep(offsets, cols, 0, n_vertices, 0, d_label, d_delta, d_res, d_scanned, d_scratch,
                                     d_scratch ? scratch_bytes : 0, nullptr);
            if (rc) break;
            iters++;
            cudaMemsetAsync(d_changed, 0, 4, 0);
            k_pr_update<<<c->num_sms * 4, 256>>>(d_label, d_delta, d_res, value_dev, d_deg, n_vertices, tolerance_q, alpha_num, alpha_den, d_changed);
            uint32_t changed = 0;
            e = cudaMemcpy(&changed, d_changed, 4, cudaMemcpyDeviceToHost);
            if (e != cudaSuccess) { g_last_cuda = e; rc = BAM_ECUDA; break; }
            bam_status_t st;
            cudaMemcpy(&st, c->d_status, sizeof st, cudaMemcpyDeviceToHost);
            if (st.code) { rc = (int)st.code; break; }
            if (!changed) break;
        }
    }
    if (n_iters_out) *n_iters_out = iters;
    if (edges_scanned_out) cudaMemcpy(edges_scanned_out, d_scanned, 8, cudaMemcpyDeviceToHost);
    cudaFree(d_buf); cudaFree(d_scratch);
    return rc;
}
