/*
 * bam_oracle.c -- CPU oracle for the BaM storage hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * Nothing the library ships may call into this file: it is the checker (tests, smoke) and
 * the timed host-core baseline (bench), never a fallback for the CUDA path.
 *
 * HOW IT IS PINNED.  The reference repository has no test-suite, golden vectors or fixtures for this
 * path.  The restatement below is pinned by (a) published known-answer vectors of the generators it
 * shares with the device code (SplitMix64, PCG32, CRC-32), (b) independent numpy / zlib / scipy
 * re-computations, and (c) the reference's OWN code for this path, compiled for the host from its
 * sources where they lie (Makefile target `ref`, glue in ref_wire.cpp / ref_pq.cpp / ref_cache.cpp / ref_admin.cpp) and
 * run beside it in the test-suite: command encoding byte for byte, its parallel queue code against the
 * controller below, its cache + array read path against ref_array_read on the same access lists (same
 * checksum, hits, misses and page reads).
 *
 * Two layers:
 *   1. Result oracle (orc_*): pure functions of the seeded inputs -- wrapping 64-bit sums,
 *      page CRC-32s, R-MAT CSR construction, BFS levels, min-vertex CC labels.  Independent
 *      of any cache or queue behaviour; this is what bit-exactness is checked against.
 *   2. Protocol restatement (ref_*): the reference's device algorithms re-expressed for host
 *      threads -- the parallel NVMe queue protocol (include/nvm_parallel_queue.h), the page
 *      cache state machine (include/page_cache.h:1122-1224 acquire_page, :1786-1927
 *      find_slot, :2009-2054 read_data), the command builders (include/nvm_cmd.h:54-88) --
 *      run against a host-thread NVMe controller that serves 4 KiB pages from the backing
 *      store.  Each function cites the reference lines it follows.  This is the "reference's
 *      host-side path" timed as the CPU baseline.
 */
#define _GNU_SOURCE
#include <pthread.h>
#include <unistd.h>
#include <sched.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#include "../include/bam_synth.h"

#define ORC_API __attribute__((visibility("default")))

/* ===================================================================================== */
/* Layer 1: result oracle                                                                */
/* ===================================================================================== */

ORC_API uint64_t orc_splitmix64(uint64_t x) { return bam_splitmix64(x); }

ORC_API void orc_pcg32_stream(uint64_t initstate, uint64_t initseq, uint32_t* out, uint64_t n)
{
    bam_pcg32_t g;
    bam_pcg32_seed(&g, initstate, initseq);
    for (uint64_t i = 0; i < n; i++) out[i] = bam_pcg32_next(&g);
}

ORC_API uint32_t orc_crc32(const uint8_t* p, uint64_t n) { return bam_crc32_update(0, p, n); }

ORC_API uint64_t orc_permute(uint64_t x, uint64_t n, uint64_t seed) { return bam_permute(x, n, seed); }

ORC_API void orc_fill_store(uint64_t* dst, uint64_t seed, uint64_t first_elem, uint64_t n)
{
    for (uint64_t i = 0; i < n; i++) dst[i] = bam_store_elem(seed, first_elem + i);
}

/* Fill only the listed pages of a store (the rest stays as allocated): lets a bounded sample of
 * a large workload run without materialising the whole backing store. */
ORC_API void orc_fill_pages(uint64_t* store, uint64_t seed, uint64_t first_elem, const uint64_t* pages,
                            uint64_t n_pages, uint32_t elems_per_page)
{
    for (uint64_t k = 0; k < n_pages; k++) {
        uint64_t base = pages[k] * elems_per_page;
        for (uint32_t w = 0; w < elems_per_page; w++) store[base + w] = bam_store_elem(seed, first_elem + base + w);
    }
}

/* Indices of lanes [lane_begin, lane_end) of the array random-read workload. */
ORC_API void orc_array_indices(uint64_t access_seed, uint64_t n_elems, uint64_t lane_begin,
                               uint64_t lane_end, uint64_t reqs_per_lane, uint64_t* out)
{
    for (uint64_t l = lane_begin; l < lane_end; l++) {
        bam_pcg32_t g;
        bam_lane_stream(&g, access_seed, l);
        for (uint64_t k = 0; k < reqs_per_lane; k++)
            *out++ = bam_uniform_index(&g, n_elems);
    }
}

/* Wrapping sum of store[idx] over the array random-read workload.  The store is not
 * materialised: element i is recomputed from its definition. */
ORC_API uint64_t orc_array_checksum(uint64_t store_seed, uint64_t n_elems, uint64_t access_seed,
                                    uint64_t lane_begin, uint64_t lane_end, uint64_t reqs_per_lane)
{
    uint64_t sum = 0;
    for (uint64_t l = lane_begin; l < lane_end; l++) {
        bam_pcg32_t g;
        bam_lane_stream(&g, access_seed, l);
        for (uint64_t k = 0; k < reqs_per_lane; k++)
            sum += bam_store_elem(store_seed, bam_uniform_index(&g, n_elems));
    }
    return sum;
}

/* Wrapping sum over an explicit index list (index i addresses element first_elem+i of
 * the global store, i.e. a shard that starts at first_elem). */
ORC_API uint64_t orc_indexed_checksum(uint64_t store_seed, uint64_t first_elem,
                                      const uint64_t* idx, uint64_t n)
{
    uint64_t sum = 0;
    for (uint64_t i = 0; i < n; i++) sum += bam_store_elem(store_seed, first_elem + idx[i]);
    return sum;
}

/* Where page `page` of a range lives when the cache sits in front of n_ctrls controllers:
 * get_backing_page_ and get_backing_ctrl_ (include/page_cache.h:558-582).  dist 0 = REPLICATE
 * (every controller holds the whole range; *ctrl = 0xffffffff, "all"), 1 = STRIPE (pages dealt
 * round-robin).  Returns the backing page on that controller. */
ORC_API uint64_t orc_backing_location(uint64_t page_start, uint64_t page, uint64_t n_ctrls, uint32_t dist, uint32_t* ctrl)
{
    uint64_t backing = page_start;
    if (dist == 1) { backing += page / n_ctrls; *ctrl = (uint32_t)(page % n_ctrls); }
    else { backing += page; *ctrl = 0xffffffffu; }
    return backing;
}

/* CRC-32 of one page of the store (page_bytes/8 little-endian u64 words). */
ORC_API uint32_t orc_page_crc(uint64_t store_seed, uint64_t page, uint32_t page_bytes)
{
    uint32_t words = page_bytes / 8;
    uint32_t crc = ~0u;
    uint64_t first = page * words;
    for (uint32_t w = 0; w < words; w++) crc = bam_crc32_u64(crc, bam_store_elem(store_seed, first + w));
    return ~crc;
}

/* Block random-read workload: page and expected CRC of request r in [r0, r1). */
ORC_API void orc_block_requests(uint64_t store_seed, uint64_t req_seed, uint64_t n_pages,
                                uint32_t page_bytes, uint64_t r0, uint64_t r1,
                                uint64_t* pages_out, uint32_t* crc_out)
{
    for (uint64_t r = r0; r < r1; r++) {
        uint64_t pg = bam_block_request_page(req_seed, r, n_pages);
        if (pages_out) pages_out[r - r0] = pg;
        if (crc_out) crc_out[r - r0] = orc_page_crc(store_seed, pg, page_bytes);
    }
}

/* Skewed (Zipf) scan of one shard: indices of lanes [lane_begin, lane_end). */
ORC_API void orc_zipf_indices(const uint64_t* cdf, uint64_t n_pages, uint32_t elems_per_page,
                              uint64_t perm_seed, uint64_t access_seed, uint64_t lane_begin,
                              uint64_t lane_end, uint64_t reqs_per_lane, uint64_t* out)
{
    for (uint64_t l = lane_begin; l < lane_end; l++) {
        bam_pcg32_t g;
        bam_lane_stream(&g, access_seed, l);
        for (uint64_t k = 0; k < reqs_per_lane; k++)
            *out++ = bam_zipf_access(&g, cdf, n_pages, elems_per_page, perm_seed);
    }
}

/* ---- R-MAT -> undirected, de-duplicated, sorted CSR -------------------------------- */

static void radix_sort_u64(uint64_t* a, uint64_t* tmp, uint64_t n, uint32_t key_bits)
{
    uint64_t* src = a;
    uint64_t* dst = tmp;
    for (uint32_t shift = 0; shift < key_bits; shift += 16) {
        uint64_t* cnt = (uint64_t*)calloc(65537, sizeof(uint64_t));
        for (uint64_t i = 0; i < n; i++) cnt[((src[i] >> shift) & 0xffff) + 1]++;
        for (uint32_t b = 0; b < 65536; b++) cnt[b + 1] += cnt[b];
        for (uint64_t i = 0; i < n; i++) dst[cnt[(src[i] >> shift) & 0xffff]++] = src[i];
        free(cnt);
        uint64_t* t = src; src = dst; dst = t;
    }
    if (src != a) memcpy(a, src, n * sizeof(uint64_t));
}

/* Pass 1 (cols == NULL): returns the number of directed edges after symmetrisation,
 * self-loop removal and de-duplication, and fills offsets[0..n_vertices].
 * Pass 2: also fills cols (adjacency of each vertex ascending).  scale <= 31. */
ORC_API uint64_t orc_rmat_csr(uint64_t seed, uint32_t scale, uint64_t edge_factor,
                              uint32_t ta, uint32_t tab, uint32_t tabc,
                              uint64_t* offsets, uint64_t* cols)
{
    uint64_t n = (uint64_t)1 << scale;
    uint64_t m = edge_factor << scale;
    bam_rmat_thresh_t t = { ta, tab, tabc };
    uint64_t* keys = (uint64_t*)malloc(2 * m * sizeof(uint64_t));
    uint64_t* tmp = (uint64_t*)malloc(2 * m * sizeof(uint64_t));
    uint64_t k = 0;
    for (uint64_t e = 0; e < m; e++) {
        uint64_t u, v;
        bam_rmat_edge(seed, e, scale, t, &u, &v);
        if (u == v) continue;
        keys[k++] = (u << 32) | v;
        keys[k++] = (v << 32) | u;
    }
    radix_sort_u64(keys, tmp, k, 64);
    uint64_t uniq = 0;
    for (uint64_t i = 0; i < k; i++)
        if (i == 0 || keys[i] != keys[i - 1]) keys[uniq++] = keys[i];
    memset(offsets, 0, (n + 1) * sizeof(uint64_t));
    for (uint64_t i = 0; i < uniq; i++) offsets[(keys[i] >> 32) + 1]++;
    for (uint64_t v = 0; v < n; v++) offsets[v + 1] += offsets[v];
    if (cols)
        for (uint64_t i = 0; i < uniq; i++) cols[i] = keys[i] & 0xffffffffu;
    free(keys);
    free(tmp);
    return uniq;
}

/* Highest-degree vertex, ties to the lowest id (the BFS source rule). */
ORC_API uint64_t orc_max_degree_vertex(uint64_t n, const uint64_t* offsets)
{
    uint64_t best = 0, bestdeg = 0;
    for (uint64_t v = 0; v < n; v++) {
        uint64_t d = offsets[v + 1] - offsets[v];
        if (d > bestdeg) { bestdeg = d; best = v; }
    }
    return best;
}

/* Level-synchronous BFS; unreached = 0xFFFFFFFF (benchmarks/bfs/main.cu:1559).  Returns the
 * number of directed edges scanned (sum of degrees of reached vertices). */
ORC_API uint64_t orc_bfs(uint64_t n, const uint64_t* offsets, const uint64_t* cols,
                         uint64_t src, uint32_t* level)
{
    for (uint64_t v = 0; v < n; v++) level[v] = 0xFFFFFFFFu;
    uint64_t* q = (uint64_t*)malloc(n * sizeof(uint64_t));
    uint64_t head = 0, tail = 0, scanned = 0;
    level[src] = 0;
    q[tail++] = src;
    while (head < tail) {
        uint64_t u = q[head++];
        scanned += offsets[u + 1] - offsets[u];
        for (uint64_t e = offsets[u]; e < offsets[u + 1]; e++) {
            uint64_t w = cols[e];
            if (level[w] == 0xFFFFFFFFu) { level[w] = level[u] + 1; q[tail++] = w; }
        }
    }
    free(q);
    return scanned;
}

/* Connected components, label = minimum vertex id of the component, which is the fixed
 * point of the reference's label propagation (benchmarks/cc/main.cu:123-144: labels start
 * as the vertex id and only ever decrease to ids inside the component).  Union-find here,
 * so the oracle does not share the propagation algorithm with the code under test.
 * Returns the number of components. */
static uint64_t uf_find(uint64_t* p, uint64_t x)
{
    while (p[x] != x) { p[x] = p[p[x]]; x = p[x]; }
    return x;
}

ORC_API uint64_t orc_cc(uint64_t n, const uint64_t* offsets, const uint64_t* cols, uint64_t* label)
{
    for (uint64_t v = 0; v < n; v++) label[v] = v;
    for (uint64_t u = 0; u < n; u++)
        for (uint64_t e = offsets[u]; e < offsets[u + 1]; e++) {
            uint64_t a = uf_find(label, u), b = uf_find(label, cols[e]);
            if (a < b) label[b] = a; else if (b < a) label[a] = b;   /* root = min id */
        }
    uint64_t comps = 0;
    for (uint64_t v = 0; v < n; v++) { label[v] = uf_find(label, v); comps += (label[v] == v); }
    return comps;
}

/* Weight of every CSR edge (include/bam_synth.h: bam_edge_weight). */
ORC_API void orc_edge_weights(uint64_t seed, uint64_t n_edges, uint32_t* out)
{
    for (uint64_t j = 0; j < n_edges; j++) out[j] = bam_edge_weight(seed, j);
}

/* Single-source shortest paths: Dijkstra with a binary heap, so the oracle does not share the
 * label-correcting relaxation (benchmarks/sssp/main.cu:115-146 + update :282-292) with the code
 * under test; both end at the unique distances.  Unreachable = 0xFFFFFFFF (MYINFINITY there). */
typedef struct { uint64_t d; uint64_t v; } heap_item_t;

ORC_API void orc_sssp(uint64_t n, const uint64_t* offsets, const uint64_t* cols, const uint32_t* weights,
                      uint64_t src, uint32_t* dist)
{
    uint64_t* d = (uint64_t*)malloc(n * sizeof(uint64_t));
    for (uint64_t v = 0; v < n; v++) d[v] = ~0ull;
    uint64_t cap = 1024, sz = 0;
    heap_item_t* h = (heap_item_t*)malloc(cap * sizeof(heap_item_t));
    d[src] = 0;
    h[sz].d = 0; h[sz].v = src; sz++;
    while (sz) {
        heap_item_t top = h[0];
        heap_item_t last = h[--sz];
        uint64_t i = 0;                                     /* sift the last item down from the root */
        for (;;) {
            uint64_t c = 2 * i + 1;
            if (c >= sz) break;
            if (c + 1 < sz && h[c + 1].d < h[c].d) c++;
            if (h[c].d >= last.d) break;
            h[i] = h[c];
            i = c;
        }
        if (sz) h[i] = last;
        if (top.d != d[top.v]) continue;                    /* a stale entry */
        for (uint64_t e = offsets[top.v]; e < offsets[top.v + 1]; e++) {
            uint64_t nd = top.d + weights[e], w = cols[e];
            if (nd < d[w]) {
                d[w] = nd;
                if (sz == cap) { cap *= 2; h = (heap_item_t*)realloc(h, cap * sizeof(heap_item_t)); }
                uint64_t k = sz++;                          /* sift up */
                while (k && h[(k - 1) / 2].d > nd) { h[k] = h[(k - 1) / 2]; k = (k - 1) / 2; }
                h[k].d = nd; h[k].v = w;
            }
        }
    }
    for (uint64_t v = 0; v < n; v++) dist[v] = d[v] == ~0ull ? 0xFFFFFFFFu : (uint32_t)d[v];
    free(h);
    free(d);
}

/* Push-based delta PageRank (benchmarks/pagerank/main.cu:107-115 initialize, :117-135 kernel,
 * :412-421 update, loop :678-772) in 64-bit fixed point with BAM_PR_FRAC_BITS fraction bits and
 * alpha = alpha_num / alpha_den.  Integer additions commute, so this sequential restatement and
 * any parallel schedule give identical bits.  Returns the number of sweeps. */
ORC_API uint32_t orc_pagerank(uint64_t n, const uint64_t* offsets, const uint64_t* cols, uint64_t alpha_num,
                              uint64_t alpha_den, uint64_t tolerance_q, uint32_t max_iters, uint64_t* value,
                              uint64_t* edges_scanned)
{
    uint64_t* delta = (uint64_t*)malloc(n * sizeof(uint64_t));
    uint64_t* residual = (uint64_t*)calloc(n, sizeof(uint64_t));
    uint8_t* label = (uint8_t*)malloc(n);
    const uint64_t one = 1ull << BAM_PR_FRAC_BITS;
    const uint64_t base = one - bam_mul_ratio(one, alpha_num, alpha_den);
    uint64_t scanned = 0;
    for (uint64_t v = 0; v < n; v++) {
        uint64_t deg = offsets[v + 1] - offsets[v];
        value[v] = base;
        delta[v] = deg ? bam_mul_ratio(base, alpha_num, alpha_den) / deg : 0;
        label[v] = 1;
    }
    uint32_t iters = 0;
    while (iters < max_iters) {
        for (uint64_t v = 0; v < n; v++) {
            if (!label[v]) continue;
            label[v] = 0;
            scanned += offsets[v + 1] - offsets[v];
            for (uint64_t e = offsets[v]; e < offsets[v + 1]; e++) residual[cols[e]] += delta[v];
        }
        iters++;
        int changed = 0;
        for (uint64_t v = 0; v < n; v++) {
            uint64_t r = residual[v];
            if (r > tolerance_q) {
                uint64_t deg = offsets[v + 1] - offsets[v];
                value[v] += r;
                delta[v] = deg ? bam_mul_ratio(r, alpha_num, alpha_den) / deg : 0;
                residual[v] = 0;
                label[v] = 1;
                changed = 1;
            }
        }
        if (!changed) break;
    }
    if (edges_scanned) *edges_scanned = scanned;
    free(delta); free(residual); free(label);
    return iters;
}

/* ===================================================================================== */
/* Layer 2: protocol restatement on host threads                                         */
/* ===================================================================================== */

#define REF_LOCKED 1u
#define REF_UNLOCKED 0u
#define REF_FREE 2u                       /* page_cache.h:  cache slot never assigned   */

/* page state encodings, include/page_cache.h:57-70 */
#define REF_VALID 0x80000000u
#define REF_BUSY 0x40000000u
#define REF_DIRTY 0x20000000u
#define REF_CNT_MASK 0x1fffffffu
#define REF_BUSY_TO_VALID 0xc0000000u
#define REF_NOT_BUSY 0xbfffffffu

#define ld_rlx(p) __atomic_load_n((p), __ATOMIC_RELAXED)
#define ld_acq(p) __atomic_load_n((p), __ATOMIC_ACQUIRE)
#define st_rlx(p, v) __atomic_store_n((p), (v), __ATOMIC_RELAXED)
#define st_rel(p, v) __atomic_store_n((p), (v), __ATOMIC_RELEASE)

typedef struct { uint32_t val; uint8_t pad[28]; } ref_padded_t;   /* nvm_types.h:98-102 */

typedef struct { uint32_t dword[16]; } __attribute__((aligned(64))) ref_cmd_t;  /* nvm_types.h:190-193 */
typedef struct { uint32_t dword[4]; } __attribute__((aligned(16))) ref_cpl_t;   /* nvm_types.h:180-183 */

/* One queue descriptor; fields follow nvm_types.h:123-165. */
typedef struct {
    uint32_t head_lock; uint8_t p0[60];
    uint32_t tail_lock; uint8_t p1[60];
    uint32_t head;      uint8_t p2[60];
    uint32_t tail;      uint8_t p3[60];
    uint32_t in_ticket; uint8_t p4[60];
    uint32_t cid_ticket; uint8_t p5[60];
    ref_padded_t* tickets;
    ref_padded_t* head_mark;
    ref_padded_t* tail_mark;
    ref_padded_t* cid;
    ref_padded_t* pos_locks;
    uint32_t qs, qs_minus_1, qs_log2;
    volatile uint32_t* db;
    void* vaddr;
} ref_queue_t;

typedef struct {
    ref_queue_t sq, cq;
    /* controller-private state of the emulated device for this pair */
    uint32_t dev_sq_head;       /* next SQ entry to fetch (mod qs)                */
    uint32_t dev_cq_tail;       /* next CQ entry to write (virtual, not wrapped)  */
    uint32_t sq_db;             /* SQ tail doorbell register                       */
    uint32_t cq_db;             /* CQ head doorbell register                       */
    uint32_t dev_cq_head_virt;  /* CQ head as last seen, unwrapped                 */
} ref_qp_t;

static void backoff(unsigned* ns)
{
    /* the reference sleeps 8..256 ns; a host thread yields instead once it has spun */
    if (*ns < 256) { *ns *= 2; __builtin_ia32_pause(); } else sched_yield();
}

/* nvm_parallel_queue.h:28-31 */
static uint32_t ref_turn_id(uint32_t ticket, uint32_t qs_log2) { return (ticket >> qs_log2) * 2; }

/* nvm_parallel_queue.h:36-52 : claim a command id from the 65536-entry lock table */
static uint16_t ref_get_cid(ref_queue_t* sq)
{
    for (;;) {
        uint16_t id = (uint16_t)(__atomic_fetch_add(&sq->cid_ticket, 1, __ATOMIC_RELAXED) & 65535u);
        uint32_t old = __atomic_fetch_or(&sq->cid[id].val, REF_LOCKED, __ATOMIC_ACQUIRE);
        if (old != REF_LOCKED) return id;
    }
}

/* nvm_parallel_queue.h:55-57 */
static void ref_put_cid(ref_queue_t* sq, uint16_t id) { st_rel(&sq->cid[id].val, REF_UNLOCKED); }

/* nvm_parallel_queue.h:60-80 : count contiguous submitted slots, never run onto head */
static uint32_t ref_move_tail(ref_queue_t* q, uint32_t cur_tail)
{
    uint32_t count = 0;
    for (;;) {
        if (((cur_tail + count + 1) & q->qs_minus_1) == (ld_rlx(&q->head) & q->qs_minus_1)) break;
        uint32_t pos = (cur_tail + count) & q->qs_minus_1;
        if (__atomic_exchange_n(&q->tail_mark[pos].val, REF_UNLOCKED, __ATOMIC_RELAXED) != REF_LOCKED) break;
        count++;
    }
    return count;
}

/* nvm_parallel_queue.h:168-330 : ticket -> slot/turn, wait for the turn, store the 64-byte
 * command, mark the slot, and let whoever holds tail_lock advance the tail over all
 * contiguous marked slots with one doorbell write. */
static uint16_t ref_sq_enqueue(ref_queue_t* sq, const ref_cmd_t* cmd)
{
    uint32_t ticket = __atomic_fetch_add(&sq->in_ticket, 1, __ATOMIC_RELAXED);
    uint32_t pos = ticket & sq->qs_minus_1;
    uint32_t id = ref_turn_id(ticket, sq->qs_log2);
    unsigned ns = 8;
    while (ld_acq(&sq->tickets[pos].val) != id) backoff(&ns);

    memcpy((ref_cmd_t*)sq->vaddr + pos, cmd, sizeof(ref_cmd_t));
    st_rel(&sq->tail_mark[pos].val, REF_LOCKED);

    ns = 8;
    while (ld_rlx(&sq->tail_mark[pos].val) == REF_LOCKED) {
        if (ld_rlx(&sq->tail_lock) != REF_LOCKED &&
            __atomic_fetch_or(&sq->tail_lock, REF_LOCKED, __ATOMIC_ACQUIRE) != REF_LOCKED) {
            uint32_t cur_tail = ld_rlx(&sq->tail);
            uint32_t moved = ref_move_tail(sq, cur_tail);
            if (moved) {
                uint32_t new_tail = cur_tail + moved;
                /* the reference writes the BAR doorbell with st.mmio.relaxed.sys (:303); the
                 * emulated register is ordinary memory, so a release store publishes the
                 * command bytes to the controller thread */
                st_rel(sq->db, new_tail & sq->qs_minus_1);
                st_rel(&sq->tail, new_tail);
            }
            st_rel(&sq->tail_lock, REF_UNLOCKED);
        }
        if (ld_rlx(&sq->tail_mark[pos].val) == REF_LOCKED) backoff(&ns);
    }
    __atomic_fetch_add(&sq->tickets[pos].val, 1, __ATOMIC_ACQ_REL);    /* odd: in flight */
    return (uint16_t)pos;
}

/* nvm_parallel_queue.h:379-422 : scan the CQ from head for an entry carrying my command id
 * and the phase expected at that position; stop at the first stale entry. */
static uint32_t ref_cq_poll(ref_queue_t* cq, uint16_t search_cid, uint32_t* virt_pos, uint32_t* head_seen)
{
    unsigned ns = 8;
    for (;;) {
        uint32_t head = ld_rlx(&cq->head);
        for (uint32_t i = 0; i < cq->qs_minus_1; i++) {
            uint32_t cur = head + i;
            uint32_t want_phase = (~(cur >> cq->qs_log2)) & 1u;
            uint32_t loc = cur & cq->qs_minus_1;
            uint32_t dw3 = ld_acq(&((ref_cpl_t*)cq->vaddr)[loc].dword[3]);
            uint32_t cid = dw3 & 0xffffu;
            uint32_t phase = (dw3 >> 16) & 1u;
            if (cid == search_cid && phase == want_phase) {
                *head_seen = head;
                *virt_pos = cur;
                return loc;
            }
            if (phase != want_phase) break;
        }
        backoff(&ns);
    }
}

/* nvm_parallel_queue.h:83-123 : advance over contiguous consumed completions; the last one
 * carries the controller's SQ head (DW2[15:0]); every SQ slot the head passed gets its second
 * ticket increment, which opens the slot's next turn. */
static uint32_t ref_move_head_cq(ref_queue_t* cq, uint32_t cur_head, ref_queue_t* sq)
{
    uint32_t count = 0;
    for (;;) {
        uint32_t loc = (cur_head + count) & cq->qs_minus_1;
        if (__atomic_exchange_n(&cq->head_mark[loc].val, REF_UNLOCKED, __ATOMIC_RELAXED) != REF_LOCKED) break;
        count++;
    }
    if (count) {
        uint32_t last = (cur_head + count - 1) & cq->qs_minus_1;
        uint32_t new_sq_head = ld_rlx(&((ref_cpl_t*)cq->vaddr)[last].dword[2]) & 0xffffu;
        uint32_t loc = ld_rlx(&sq->head) & sq->qs_minus_1;
        uint32_t moved = 0;
        for (; loc != new_sq_head; moved++, loc = (loc + 1) & sq->qs_minus_1)
            __atomic_fetch_add(&sq->tickets[loc].val, 1, __ATOMIC_RELEASE);
        if (moved) __atomic_fetch_add(&sq->head, moved, __ATOMIC_ACQ_REL);
    }
    return count;
}

/* nvm_parallel_queue.h:425-535 : per-position lock, mark consumed, head_lock holder sweeps and
 * rings the CQ head doorbell, wait until the head has passed my virtual position. */
static void ref_cq_dequeue(ref_queue_t* cq, uint32_t pos, ref_queue_t* sq, uint32_t virt_pos, uint32_t head_seen)
{
    unsigned ns = 8;
    __atomic_fetch_add(&cq->tail, 1, __ATOMIC_ACQ_REL);
    while (__atomic_fetch_or(&cq->pos_locks[pos].val, 1, __ATOMIC_ACQUIRE) != 0) backoff(&ns);
    st_rel(&cq->head_mark[pos].val, REF_LOCKED);
    ns = 8;
    while (ld_rlx(&cq->head_mark[pos].val) == REF_LOCKED) {
        if (__atomic_fetch_or(&cq->head_lock, REF_LOCKED, __ATOMIC_ACQUIRE) != REF_LOCKED) {
            uint32_t cur_head = ld_rlx(&cq->head);
            uint32_t moved = ref_move_head_cq(cq, cur_head, sq);
            if (moved) {
                uint32_t new_head = cur_head + moved;
                st_rel(cq->db, new_head & cq->qs_minus_1);
                st_rel(&cq->head, new_head);
            }
            st_rel(&cq->head_lock, REF_UNLOCKED);
        }
        if (ld_rlx(&cq->head_mark[pos].val) == REF_LOCKED) backoff(&ns);
    }
    ns = 8;
    for (;;) {   /* :504-532 */
        uint32_t new_head = ld_acq(&cq->head);
        if (new_head > head_seen) { if (virt_pos >= head_seen && virt_pos < new_head) break; }
        else if (new_head < head_seen) { if (virt_pos >= head_seen || virt_pos < new_head) break; }
        backoff(&ns);
    }
    st_rel(&cq->pos_locks[pos].val, 0);
}

/* ---- page cache ---------------------------------------------------------------------- */

typedef struct { uint32_t state; uint32_t offset; uint8_t pad[24]; } ref_data_page_t;       /* page_cache.h:96-102 */
typedef struct { uint32_t take_lock; uint32_t pad0; uint64_t translation; uint8_t pad[16]; } ref_cache_page_t; /* :487-493 */

typedef struct {
    uint8_t* base_addr;
    uint32_t page_size, page_size_log;
    uint64_t n_slots;
    ref_cache_page_t* slots;
    ref_data_page_t* pages;      /* one entry per page of the (single) range */
    uint64_t n_data_pages;
    uint64_t page_ticket;        /* the global clock hand, page_cache.h:1802 */
    ref_qp_t* qps;
    uint32_t n_qps;
    uint32_t n_blocks_per_page;
    uint32_t ns_id;
    /* counters of range_d_t, page_cache.h:904-907 */
    uint64_t access_cnt, miss_cnt, hit_cnt, read_io_cnt;
} ref_cache_t;

/* nvm_cmd.h:54-88 + page_cache.h:2009-2054.  The reference follows each read with
 * enqueue_second (:1961-2007), an extra one-block read that flushes PCIe write ordering for
 * GPUDirect data; the emulated controller publishes its completion after the payload with a
 * release store, so that extra I/O has no counterpart here. */
/* The READ / WRITE command of include/nvm_cmd.h:54-88 (nvm_cmd_header, nvm_cmd_data_ptr,
 * nvm_cmd_rw_blks) as read_data builds it (page_cache.h:2009-2032).  Exported so that tests can
 * compare it with the reference's own builders and with the library's. */
ORC_API void orc_encode_rw(uint16_t cid, uint8_t opcode, uint32_t ns_id, uint64_t prp1, uint64_t prp2, uint64_t start_lba,
                           uint32_t n_blocks, void* out64)
{
    ref_cmd_t cmd;
    memset(&cmd, 0, sizeof cmd);
    cmd.dword[0] = ((uint32_t)cid << 16) | (opcode & 0x7fu);
    cmd.dword[1] = ns_id;
    cmd.dword[6] = (uint32_t)prp1;
    cmd.dword[7] = (uint32_t)(prp1 >> 32);
    cmd.dword[8] = (uint32_t)prp2;
    cmd.dword[9] = (uint32_t)(prp2 >> 32);
    cmd.dword[10] = (uint32_t)start_lba;
    cmd.dword[11] = (uint32_t)(start_lba >> 32);
    cmd.dword[12] = (n_blocks - 1) & 0xffffu;
    memcpy(out64, &cmd, 64);
}

static void ref_read_data(ref_cache_t* pc, ref_qp_t* qp, uint64_t start_lba, uint32_t n_blocks, uint64_t slot)
{
    ref_cmd_t cmd;
    uint16_t cid = ref_get_cid(&qp->sq);
    uint64_t prp1 = (uint64_t)(uintptr_t)(pc->base_addr + slot * pc->page_size);
    orc_encode_rw(cid, 0x02u /* NVM_IO_READ */, pc->ns_id, prp1, 0, start_lba, n_blocks, &cmd);
    ref_sq_enqueue(&qp->sq, &cmd);
    uint32_t virt_pos, head_seen;
    uint32_t cq_pos = ref_cq_poll(&qp->cq, cid, &virt_pos, &head_seen);
    ref_cq_dequeue(&qp->cq, cq_pos, &qp->sq, virt_pos, head_seen);
    ref_put_cid(&qp->sq, cid);
}

/* page_cache.h:1786-1927 : the global clock hand visits slots in order; a FREE slot is taken,
 * an assigned slot is taken if its current page is unpinned and not busy (that page becomes
 * INVALID).  Pages written through the cache would be written back here (:1849-1873); the read
 * path never sets DIRTY. */
static uint32_t ref_find_slot(ref_cache_t* pc, uint64_t page)
{
    for (;;) {
        uint32_t slot = (uint32_t)(__atomic_fetch_add(&pc->page_ticket, 1, __ATOMIC_RELAXED) % pc->n_slots);
        ref_cache_page_t* s = &pc->slots[slot];
        uint32_t v = ld_rlx(&s->take_lock);
        if (v == REF_FREE) {
            if (__atomic_compare_exchange_n(&s->take_lock, &v, REF_LOCKED, 0, __ATOMIC_ACQUIRE, __ATOMIC_RELAXED)) {
                s->translation = page;
                st_rel(&s->take_lock, REF_UNLOCKED);
                return slot;
            }
        } else if (v == REF_UNLOCKED) {
            if (__atomic_compare_exchange_n(&s->take_lock, &v, REF_LOCKED, 0, __ATOMIC_ACQUIRE, __ATOMIC_RELAXED)) {
                uint64_t prev = s->translation;
                int took = 0;
                uint32_t st = ld_rlx(&pc->pages[prev].state);
                if ((st & REF_CNT_MASK) == 0 && (st & REF_BUSY) == 0) {
                    uint32_t old = __atomic_fetch_or(&pc->pages[prev].state, REF_BUSY, __ATOMIC_ACQUIRE);
                    if ((old & REF_BUSY) == 0) {
                        if ((old & REF_CNT_MASK) == 0) {
                            took = 1;
                            __atomic_fetch_and(&pc->pages[prev].state, REF_CNT_MASK, __ATOMIC_RELEASE);
                        } else {
                            __atomic_fetch_and(&pc->pages[prev].state, REF_NOT_BUSY, __ATOMIC_RELEASE);
                        }
                    }
                }
                if (took) s->translation = page;
                st_rel(&s->take_lock, REF_UNLOCKED);
                if (took) return slot;
            }
        }
    }
}

/* page_cache.h:1122-1224 : pin the page; INVALID -> win BUSY, find a slot, read, publish the
 * slot, flip BUSY->VALID; VALID -> hit; BUSY -> back off and look again. */
static uint32_t ref_acquire_page(ref_cache_t* pc, uint64_t page, uint32_t count, uint32_t queue)
{
    __atomic_fetch_add(&pc->access_cnt, count, __ATOMIC_RELAXED);
    ref_data_page_t* dp = &pc->pages[page];
    uint32_t rs = __atomic_fetch_add(&dp->state, count, __ATOMIC_ACQUIRE);
    unsigned ns = 8;
    for (;;) {
        uint32_t st = (rs >> 30) & 3u;
        if (st == 0) {                                        /* NV_NB */
            uint32_t old = __atomic_fetch_or(&dp->state, REF_BUSY, __ATOMIC_ACQUIRE);
            if ((old & REF_BUSY) == 0) {
                if (((old >> 30) & 3u) == 0) {
                    uint32_t slot = ref_find_slot(pc, page);
                    __atomic_fetch_add(&pc->read_io_cnt, 1, __ATOMIC_RELAXED);
                    ref_read_data(pc, &pc->qps[queue], page * pc->n_blocks_per_page, pc->n_blocks_per_page, slot);
                    dp->offset = slot;
                    __atomic_fetch_add(&pc->miss_cnt, count, __ATOMIC_RELAXED);
                    __atomic_fetch_xor(&dp->state, REF_BUSY_TO_VALID, __ATOMIC_RELEASE);
                    return slot;
                }
                __atomic_fetch_and(&dp->state, REF_NOT_BUSY, __ATOMIC_RELEASE);
            }
        } else if (st == 2) {                                 /* V_NB */
            uint32_t slot = dp->offset;
            __atomic_fetch_add(&pc->hit_cnt, count, __ATOMIC_RELAXED);
            return slot;
        }
        backoff(&ns);
        rs = ld_acq(&dp->state);
    }
}

/* page_cache.h:1088-1094 */
static void ref_release_page(ref_cache_t* pc, uint64_t page, uint32_t count)
{
    __atomic_fetch_sub(&pc->pages[page].state, count, __ATOMIC_RELEASE);
}

/* ---- host-thread NVMe controller ------------------------------------------------------
 * Stands in for the SSD the reference talks to.  Behaviour the queue code relies on
 * (include/nvm_parallel_queue.h, src/queue.cpp:12-42): consume SQ entries up to the tail
 * doorbell, execute READ by copying (NLB+1) blocks from SLBA to PRP1, post a 16-byte
 * completion {DW2 = SQHD | SQID<<16, DW3 = CID | phase<<16 | status<<17}, phase starts at 1
 * and flips on each wrap, never overwrite entries the host has not released through the CQ
 * head doorbell. */
typedef struct {
    ref_qp_t* qps;
    uint32_t n_qps, first_qp, stride;
    const uint8_t* store;
    uint64_t store_bytes;
    uint32_t lba_bytes;
    volatile int* stop;
    uint64_t served;
} ref_ctrl_arg_t;

static void* ref_ctrl_thread(void* p)
{
    ref_ctrl_arg_t* a = (ref_ctrl_arg_t*)p;
    unsigned idle = 0;
    while (!ld_acq(a->stop)) {
        int worked = 0;
        for (uint32_t q = a->first_qp; q < a->n_qps; q += a->stride) {
            ref_qp_t* qp = &a->qps[q];
            uint32_t qs = qp->sq.qs, mask = qs - 1;
            uint32_t tail = ld_acq(&qp->sq_db);
            while (qp->dev_sq_head != tail) {
                /* CQ back-pressure: unwrap the head doorbell and keep one slot open */
                uint32_t hdb = ld_acq(&qp->cq_db);
                qp->dev_cq_head_virt += (hdb - (qp->dev_cq_head_virt & mask)) & mask;
                if (qp->dev_cq_tail - qp->dev_cq_head_virt >= qs - 1) break;
                const ref_cmd_t* cmd = (const ref_cmd_t*)qp->sq.vaddr + qp->dev_sq_head;
                uint32_t cid = cmd->dword[0] >> 16;
                uint32_t opc = cmd->dword[0] & 0x7fu;
                uint64_t prp1 = ((uint64_t)cmd->dword[7] << 32) | cmd->dword[6];
                uint64_t slba = ((uint64_t)cmd->dword[11] << 32) | cmd->dword[10];
                uint64_t bytes = (uint64_t)((cmd->dword[12] & 0xffffu) + 1) * a->lba_bytes;
                uint32_t status = 0;
                if (opc != 0x02u) status = 0x01;                          /* invalid opcode   */
                else if (slba * a->lba_bytes + bytes > a->store_bytes) status = 0x80; /* LBA range */
                else memcpy((void*)(uintptr_t)prp1, a->store + slba * a->lba_bytes, bytes);
                qp->dev_sq_head = (qp->dev_sq_head + 1) & mask;
                uint32_t pos = qp->dev_cq_tail & mask;
                uint32_t phase = (~(qp->dev_cq_tail >> qp->cq.qs_log2)) & 1u;
                ref_cpl_t* c = (ref_cpl_t*)qp->cq.vaddr + pos;
                c->dword[0] = 0; c->dword[1] = 0;
                st_rlx(&c->dword[2], qp->dev_sq_head | ((uint32_t)(q + 1) << 16));
                st_rel(&c->dword[3], cid | (phase << 16) | (status << 17));
                qp->dev_cq_tail++;
                a->served++;
                worked = 1;
            }
        }
        if (!worked) { if (++idle > 64) { sched_yield(); idle = 0; } else __builtin_ia32_pause(); }
        else idle = 0;
    }
    return 0;
}

/* The same controller over bare queue memory and doorbell registers (no descriptors of this file):
 * what an NVMe controller sees of a queue pair.  Lets other producers of the wire protocol -- in the
 * tests: the reference's own queue code compiled from its sources -- be served by this controller.
 * READ and WRITE; SQ and CQ may differ in depth. */
typedef struct {
    const ref_cmd_t* sq_mem; ref_cpl_t* cq_mem;
    volatile uint32_t* sq_db; volatile uint32_t* cq_db;
    uint32_t sq_qs, cq_qs, cq_qs_log2; uint16_t sqid;
    uint8_t* store; uint64_t store_bytes; uint32_t lba_bytes;
    volatile int stop;
    uint64_t served;
    pthread_t thread;
} orc_wire_ctrl_t;

static void* orc_wire_ctrl_thread(void* p)
{
    orc_wire_ctrl_t* a = (orc_wire_ctrl_t*)p;
    uint32_t sq_head = 0, cq_tail = 0, cq_head_virt = 0;
    const uint32_t smask = a->sq_qs - 1, cmask = a->cq_qs - 1;
    unsigned idle = 0;
    while (!ld_acq(&a->stop)) {
        uint32_t tail = ld_acq(a->sq_db);
        int worked = 0;
        while (sq_head != tail) {
            uint32_t hdb = ld_acq(a->cq_db);
            cq_head_virt += (hdb - (cq_head_virt & cmask)) & cmask;
            if (cq_tail - cq_head_virt >= a->cq_qs - 1) break;            /* keep one completion slot open */
            const ref_cmd_t* cmd = a->sq_mem + sq_head;
            uint32_t cid = cmd->dword[0] >> 16, opc = cmd->dword[0] & 0x7fu;
            uint64_t prp1 = ((uint64_t)cmd->dword[7] << 32) | cmd->dword[6];
            uint64_t slba = ((uint64_t)cmd->dword[11] << 32) | cmd->dword[10];
            uint64_t bytes = (uint64_t)((cmd->dword[12] & 0xffffu) + 1) * a->lba_bytes;
            uint32_t status = 0;
            if (opc != 0x01u && opc != 0x02u) status = 0x01;                               /* invalid opcode */
            else if (slba * a->lba_bytes + bytes > a->store_bytes) status = 0x80;          /* LBA out of range */
            else if (opc == 0x02u) memcpy((void*)(uintptr_t)prp1, a->store + slba * a->lba_bytes, bytes);
            else memcpy(a->store + slba * a->lba_bytes, (const void*)(uintptr_t)prp1, bytes);
            sq_head = (sq_head + 1) & smask;
            ref_cpl_t* c = a->cq_mem + (cq_tail & cmask);
            uint32_t phase = (~(cq_tail >> a->cq_qs_log2)) & 1u;
            c->dword[0] = 0; c->dword[1] = 0;
            st_rlx(&c->dword[2], sq_head | ((uint32_t)a->sqid << 16));
            st_rel(&c->dword[3], cid | (phase << 16) | (status << 17));
            cq_tail++;
            a->served++;
            worked = 1;
        }
        if (!worked) { if (++idle > 64) { sched_yield(); idle = 0; } else __builtin_ia32_pause(); }
        else idle = 0;
    }
    return 0;
}

ORC_API void* orc_wire_ctrl_start(const void* sq_mem, void* cq_mem, void* sq_db, void* cq_db, uint32_t sq_qs, uint32_t cq_qs,
                                  uint16_t sqid, void* store, uint64_t store_bytes, uint32_t lba_bytes)
{
    orc_wire_ctrl_t* a = (orc_wire_ctrl_t*)calloc(1, sizeof *a);
    if (!a) return 0;
    a->sq_mem = (const ref_cmd_t*)sq_mem; a->cq_mem = (ref_cpl_t*)cq_mem;
    a->sq_db = (volatile uint32_t*)sq_db; a->cq_db = (volatile uint32_t*)cq_db;
    a->sq_qs = sq_qs; a->cq_qs = cq_qs; a->sqid = sqid;
    while ((1u << a->cq_qs_log2) < cq_qs) a->cq_qs_log2++;
    a->store = (uint8_t*)store; a->store_bytes = store_bytes; a->lba_bytes = lba_bytes;
    if (pthread_create(&a->thread, 0, orc_wire_ctrl_thread, a) != 0) { free(a); return 0; }
    return a;
}

ORC_API uint64_t orc_wire_ctrl_stop(void* h)
{
    orc_wire_ctrl_t* a = (orc_wire_ctrl_t*)h;
    __atomic_store_n(&a->stop, 1, __ATOMIC_RELEASE);
    pthread_join(a->thread, 0);
    uint64_t served = a->served;
    free(a);
    return served;
}

/* ---- the device controller's way of sharing ONE queue among several processors, for host threads -------
 * The GPU controller (include/bam/emu_ctrl.cuh) lets several processors serve a queue: a processor takes the
 * queue's lock only to RESERVE a batch (SQ entries [fetch, fetch + n) and the completion slots
 * [cqbase, cqbase + n)), reads the entries out after it has let the lock go, hands them back IN ORDER through
 * the counter sq_decoded, and then executes and completes its commands whenever it gets to them -- so
 * completions of a later batch may be posted before those of an earlier one.  A completion's SQ-head value
 * tells the submitter that every entry below it is free again; the ordered hand-back makes that true at the
 * moment the value is posted.  This model follows the scheme step by step with n_procs threads, stalling at
 * random between the steps so that later batches overtake earlier ones (counted); the tests run the reference's
 * parallel queue code against it on shallow queues, where freed entries are overwritten at once.  What the
 * runs show: the reference's code completes every command exactly once with the right data however the batches
 * overtake one another.  (They would not show a missing hand-back: the reference frees entries only when its
 * completion-queue head moves, which it does in queue order, and completion slots are reserved in SQ order.) */
struct orc_mt_ctrl_s;
typedef struct { struct orc_mt_ctrl_s* c; uint32_t me; } orc_mt_arg_t;
typedef struct orc_mt_ctrl_s {
    orc_wire_ctrl_t base;              /* queue memory, doorbells, media (its thread member is unused)  */
    uint32_t lock;                     /* held for the reservation only                                  */
    uint32_t sq_fetch, cq_tail, cq_head;   /* virtual positions, guarded by lock                          */
    uint32_t sq_decoded;               /* virtual SQ position up to which entries have been read out      */
    uint32_t batch, n_procs;
    uint64_t served_mt, batches, overtaken;    /* overtaken: batches that posted while an earlier one had not finished */
    uint32_t next_seq;                 /* batch sequence numbers, handed out under lock                    */
    uint32_t oldest_open;              /* lowest sequence number that has not finished posting (model bookkeeping) */
    uint32_t done_lock;
    uint8_t done[1024];
    pthread_t threads[16];
    uint32_t seeds[16];
    orc_mt_arg_t args[16];
} orc_mt_ctrl_t;


static void* orc_mt_ctrl_thread(void* p)
{
    orc_mt_arg_t* arg = (orc_mt_arg_t*)p;
    orc_mt_ctrl_t* c = arg->c;
    orc_wire_ctrl_t* a = &c->base;
    uint32_t rnd = c->seeds[arg->me];
    const uint32_t smask = a->sq_qs - 1, cmask = a->cq_qs - 1;
    ref_cmd_t local[32];
    unsigned idle = 0;
    while (!ld_acq(&a->stop)) {
        /* reserve under the lock */
        uint32_t n = 0, fetch = 0, cqbase = 0, seq = 0;
        if (ld_acq(a->sq_db) != (ld_acq(&c->sq_fetch) & smask) && __atomic_exchange_n(&c->lock, 1u, __ATOMIC_ACQUIRE) == 0u) {
            fetch = c->sq_fetch;
            const uint32_t tail = ld_acq(a->sq_db), hdb = ld_acq(a->cq_db);
            c->cq_head += (hdb - c->cq_head) & cmask;
            cqbase = c->cq_tail;
            const uint32_t avail = (tail - fetch) & smask, space = cmask - (cqbase - c->cq_head);
            n = avail < space ? avail : space;
            if (n > c->batch) n = c->batch;
            c->cq_tail = cqbase + n;
            c->sq_fetch = fetch + n;
            if (n) seq = c->next_seq++;
            __atomic_store_n(&c->lock, 0u, __ATOMIC_RELEASE);
        }
        if (n == 0) { if (++idle > 64) { sched_yield(); idle = 0; } else __builtin_ia32_pause(); continue; }
        idle = 0;
        rnd = rnd * 1664525u + 1013904223u;
        if (((rnd >> 16) & 15u) == 0u) usleep(100);                /* let later batches get well ahead */
        else if (rnd & 0x10000u) sched_yield();
        /* read the entries out, outside the lock */
        for (uint32_t i = 0; i < n; i++) local[i] = a->sq_mem[(fetch + i) & smask];
        /* hand them back in order */
        while (ld_acq(&c->sq_decoded) != fetch) { if (ld_acq(&a->stop)) return 0; __builtin_ia32_pause(); }
        st_rel(&c->sq_decoded, fetch + n);
        rnd = rnd * 1664525u + 1013904223u;
        if (rnd & 0x10000u) sched_yield();
        /* execute and complete, last command first (completion slots are the batch's own) */
        if (ld_acq(&c->oldest_open) != seq) __atomic_fetch_add(&c->overtaken, 1, __ATOMIC_RELAXED);
        for (uint32_t k = n; k-- > 0;) {
            const ref_cmd_t* cmd = &local[k];
            uint32_t cid = cmd->dword[0] >> 16, opc = cmd->dword[0] & 0x7fu;
            uint64_t prp1 = ((uint64_t)cmd->dword[7] << 32) | cmd->dword[6];
            uint64_t slba = ((uint64_t)cmd->dword[11] << 32) | cmd->dword[10];
            uint64_t bytes = (uint64_t)((cmd->dword[12] & 0xffffu) + 1) * a->lba_bytes;
            uint32_t status = 0;
            if (opc != 0x01u && opc != 0x02u) status = 0x01;
            else if (slba * a->lba_bytes + bytes > a->store_bytes) status = 0x80;
            else if (opc == 0x02u) memcpy((void*)(uintptr_t)prp1, a->store + slba * a->lba_bytes, bytes);
            else memcpy(a->store + slba * a->lba_bytes, (const void*)(uintptr_t)prp1, bytes);
            const uint32_t slot = cqbase + k;
            ref_cpl_t* e = a->cq_mem + (slot & cmask);
            const uint32_t phase = (~(slot >> a->cq_qs_log2)) & 1u;
            e->dword[0] = 0; e->dword[1] = 0;
            st_rlx(&e->dword[2], ((fetch + n) & smask) | ((uint32_t)a->sqid << 16));
            st_rel(&e->dword[3], cid | (phase << 16) | (status << 17));
        }
        /* bookkeeping of the model only: which batch is the oldest one still being completed */
        while (__atomic_exchange_n(&c->done_lock, 1u, __ATOMIC_ACQUIRE) != 0u) __builtin_ia32_pause();
        c->done[seq & 1023u] = 1;
        while (c->done[c->oldest_open & 1023u]) { c->done[c->oldest_open & 1023u] = 0; st_rel(&c->oldest_open, c->oldest_open + 1); }
        __atomic_store_n(&c->done_lock, 0u, __ATOMIC_RELEASE);
        __atomic_fetch_add(&c->served_mt, n, __ATOMIC_RELAXED);
        __atomic_fetch_add(&c->batches, 1, __ATOMIC_RELAXED);
    }
    return 0;
}

ORC_API void* orc_wire_ctrl_start_mt(const void* sq_mem, void* cq_mem, void* sq_db, void* cq_db, uint32_t sq_qs, uint32_t cq_qs,
                                     uint16_t sqid, void* store, uint64_t store_bytes, uint32_t lba_bytes, uint32_t n_procs, uint32_t batch)
{
    if (n_procs == 0 || n_procs > 16 || batch == 0 || batch > 32) return 0;
    orc_mt_ctrl_t* c = (orc_mt_ctrl_t*)calloc(1, sizeof *c);
    if (!c) return 0;
    orc_wire_ctrl_t* a = &c->base;
    a->sq_mem = (const ref_cmd_t*)sq_mem; a->cq_mem = (ref_cpl_t*)cq_mem;
    a->sq_db = (volatile uint32_t*)sq_db; a->cq_db = (volatile uint32_t*)cq_db;
    a->sq_qs = sq_qs; a->cq_qs = cq_qs; a->sqid = sqid;
    while ((1u << a->cq_qs_log2) < cq_qs) a->cq_qs_log2++;
    a->store = (uint8_t*)store; a->store_bytes = store_bytes; a->lba_bytes = lba_bytes;
    c->batch = batch; c->n_procs = n_procs;
    for (uint32_t i = 0; i < n_procs; i++) {
        c->seeds[i] = 12345u + 977u * i;
        c->args[i].c = c; c->args[i].me = i;
        if (pthread_create(&c->threads[i], 0, orc_mt_ctrl_thread, &c->args[i]) != 0) {
            __atomic_store_n(&a->stop, 1, __ATOMIC_RELEASE);
            for (uint32_t k = 0; k < i; k++) pthread_join(c->threads[k], 0);
            free(c);
            return 0;
        }
    }
    return c;
}

/* Stops the processors; returns the commands served and, through the pointers, the batches taken and how many
 * of them posted their completions while an earlier batch had not finished posting its own. */
ORC_API uint64_t orc_wire_ctrl_stop_mt(void* h, uint64_t* batches, uint64_t* overtaken)
{
    orc_mt_ctrl_t* c = (orc_mt_ctrl_t*)h;
    __atomic_store_n(&c->base.stop, 1, __ATOMIC_RELEASE);
    for (uint32_t i = 0; i < c->n_procs; i++) pthread_join(c->threads[i], 0);
    const uint64_t served = c->served_mt;
    if (batches) *batches = c->batches;
    if (overtaken) *overtaken = c->overtaken;
    free(c);
    return served;
}

static void ref_queue_init(ref_queue_t* q, uint32_t qs, size_t entry_bytes, volatile uint32_t* db, int is_sq)
{
    memset(q, 0, sizeof *q);
    q->qs = qs; q->qs_minus_1 = qs - 1;
    q->qs_log2 = 0; while ((1u << q->qs_log2) < qs) q->qs_log2++;
    q->vaddr = aligned_alloc(4096, ((size_t)qs * entry_bytes + 4095) & ~(size_t)4095);
    memset(q->vaddr, 0, (size_t)qs * entry_bytes);           /* src/queue.cpp:12-42 */
    q->db = db;
    q->tickets = (ref_padded_t*)calloc(qs, sizeof(ref_padded_t));
    q->head_mark = (ref_padded_t*)calloc(qs, sizeof(ref_padded_t));
    q->tail_mark = (ref_padded_t*)calloc(qs, sizeof(ref_padded_t));
    q->pos_locks = (ref_padded_t*)calloc(qs, sizeof(ref_padded_t));
    q->cid = is_sq ? (ref_padded_t*)calloc(65536, sizeof(ref_padded_t)) : 0;
}

static void ref_queue_free(ref_queue_t* q)
{
    free(q->vaddr); free(q->tickets); free(q->head_mark); free(q->tail_mark); free(q->pos_locks); free(q->cid);
}

typedef struct {
    ref_cache_t* pc;
    const uint64_t* idx;       /* explicit index list, or NULL to draw lanes from PCG32 */
    uint64_t n_elems;          /* for the PCG32 path */
    uint64_t access_seed;
    uint64_t lane_begin, lane_end, reqs_per_lane;
    uint32_t worker;
    uint64_t sum;
} ref_worker_arg_t;

/* One host thread plays a contiguous block of reader lanes, one access at a time, exactly as
 * a lone GPU thread would run array_d_t<T>::seq_read (page_cache.h:1541-1574) with a
 * coalescing mask of one lane (the reference's own host stub uses mask = 1, :1552-1554). */
static void* ref_worker_thread(void* p)
{
    ref_worker_arg_t* a = (ref_worker_arg_t*)p;
    ref_cache_t* pc = a->pc;
    uint32_t queue = a->worker % pc->n_qps;                  /* stands in for smid % n_qps, :1341 */
    uint64_t sum = 0;
    uint64_t k = 0;
    for (uint64_t l = a->lane_begin; l < a->lane_end; l++) {
        bam_pcg32_t g;
        bam_lane_stream(&g, a->access_seed, l);
        for (uint64_t r = 0; r < a->reqs_per_lane; r++, k++) {
            uint64_t i = a->idx ? a->idx[l * a->reqs_per_lane + r] : bam_uniform_index(&g, a->n_elems);
            uint64_t byte = i * sizeof(uint64_t);
            uint64_t page = byte >> pc->page_size_log;
            uint64_t sub = byte & (pc->page_size - 1);
            uint32_t slot = ref_acquire_page(pc, page, 1, queue);
            sum += *(const uint64_t*)(pc->base_addr + (uint64_t)slot * pc->page_size + sub);
            ref_release_page(pc, page, 1);
        }
    }
    a->sum = sum;
    return 0;
}

typedef struct {
    uint64_t checksum;
    uint64_t accesses, hits, misses, read_ios;
    double seconds;
    uint32_t worker_threads, ctrl_threads;
} ref_result_t;

static double now_s(void)
{
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return ts.tv_sec + 1e-9 * ts.tv_nsec;
}

/* The reference's array read path on host threads: `workers` reader threads share one page
 * cache and `n_qps` queue pairs of depth `qdepth`; `ctrl_threads` controller threads serve
 * the queues from `store`.  idx == NULL draws the array random-read workload
 * (lanes [lane_begin, lane_end) x reqs_per_lane from PCG32), otherwise idx holds
 * (lane_end-lane_begin)*reqs_per_lane explicit element indices addressed from lane_begin = 0.
 * Only the access loop is timed (set-up excluded, as benchmarks/array/main.cu:164-178). */
ORC_API int ref_array_read(const uint64_t* store, uint64_t n_elems, uint32_t page_size,
                           uint64_t n_slots, uint32_t n_qps, uint32_t qdepth, uint32_t lba_bytes,
                           uint32_t workers, uint32_t ctrl_threads,
                           const uint64_t* idx, uint64_t access_seed,
                           uint64_t lane_begin, uint64_t lane_end, uint64_t reqs_per_lane,
                           ref_result_t* out)
{
    if (!store || !out || workers == 0 || ctrl_threads == 0 || n_qps == 0) return 22;
    if (qdepth < 2 || (qdepth & (qdepth - 1)) || (page_size & (page_size - 1)) || page_size % lba_bytes) return 22;
    ref_cache_t pc;
    memset(&pc, 0, sizeof pc);
    pc.page_size = page_size;
    while ((1u << pc.page_size_log) < page_size) pc.page_size_log++;
    pc.n_slots = n_slots;
    pc.base_addr = (uint8_t*)aligned_alloc(4096, n_slots * (uint64_t)page_size);
    pc.slots = (ref_cache_page_t*)calloc(n_slots, sizeof(ref_cache_page_t));
    for (uint64_t s = 0; s < n_slots; s++) pc.slots[s].take_lock = REF_FREE;     /* page_cache.h:745-748 */
    pc.n_data_pages = (n_elems * 8 + page_size - 1) / page_size;
    pc.pages = (ref_data_page_t*)calloc(pc.n_data_pages, sizeof(ref_data_page_t));
    pc.n_qps = n_qps;
    pc.qps = (ref_qp_t*)aligned_alloc(64, sizeof(ref_qp_t) * n_qps);
    pc.n_blocks_per_page = page_size / lba_bytes;
    pc.ns_id = 1;
    for (uint32_t q = 0; q < n_qps; q++) {
        ref_qp_t* qp = &pc.qps[q];
        memset(qp, 0, sizeof *qp);
        ref_queue_init(&qp->sq, qdepth, sizeof(ref_cmd_t), &qp->sq_db, 1);
        ref_queue_init(&qp->cq, qdepth, sizeof(ref_cpl_t), &qp->cq_db, 0);
    }
    volatile int stop = 0;
    pthread_t* ct = (pthread_t*)calloc(ctrl_threads, sizeof(pthread_t));
    ref_ctrl_arg_t* ca = (ref_ctrl_arg_t*)calloc(ctrl_threads, sizeof(ref_ctrl_arg_t));
    uint32_t n_ct = ctrl_threads < n_qps ? ctrl_threads : n_qps;
    for (uint32_t c = 0; c < n_ct; c++) {
        ca[c] = (ref_ctrl_arg_t){ pc.qps, n_qps, c, n_ct, (const uint8_t*)store, n_elems * 8, lba_bytes, &stop, 0 };
        pthread_create(&ct[c], 0, ref_ctrl_thread, &ca[c]);
    }
    pthread_t* wt = (pthread_t*)calloc(workers, sizeof(pthread_t));
    ref_worker_arg_t* wa = (ref_worker_arg_t*)calloc(workers, sizeof(ref_worker_arg_t));
    uint64_t lanes = lane_end - lane_begin;
    double t0 = now_s();
    for (uint32_t w = 0; w < workers; w++) {
        uint64_t b = lane_begin + lanes * w / workers, e = lane_begin + lanes * (w + 1) / workers;
        wa[w] = (ref_worker_arg_t){ &pc, idx, n_elems, access_seed, b, e, reqs_per_lane, w, 0 };
        pthread_create(&wt[w], 0, ref_worker_thread, &wa[w]);
    }
    uint64_t sum = 0;
    for (uint32_t w = 0; w < workers; w++) { pthread_join(wt[w], 0); sum += wa[w].sum; }
    double t1 = now_s();
    __atomic_store_n(&stop, 1, __ATOMIC_RELEASE);
    for (uint32_t c = 0; c < n_ct; c++) pthread_join(ct[c], 0);

    out->checksum = sum;
    out->accesses = pc.access_cnt; out->hits = pc.hit_cnt; out->misses = pc.miss_cnt; out->read_ios = pc.read_io_cnt;
    out->seconds = t1 - t0;
    out->worker_threads = workers; out->ctrl_threads = n_ct;

    for (uint32_t q = 0; q < n_qps; q++) { ref_queue_free(&pc.qps[q].sq); ref_queue_free(&pc.qps[q].cq); }
    free(pc.qps); free(pc.pages); free(pc.slots); free(pc.base_addr);
    free(ct); free(ca); free(wt); free(wa);
    return 0;
}

/* Raw block reads (the block benchmark shape, benchmarks/block/main.cu:137-200): each request
 * goes straight through read_data into cache slot (request id mod n_slots), bypassing the
 * cache look-up; the page's CRC-32 is taken from the slot right after the completion. */
typedef struct {
    ref_cache_t* pc;
    uint64_t req_seed, n_pages, r0, r1;
    uint32_t worker, n_workers;
    uint32_t* crc_out;
} ref_block_arg_t;

static void* ref_block_thread(void* p)
{
    ref_block_arg_t* a = (ref_block_arg_t*)p;
    ref_cache_t* pc = a->pc;
    uint32_t queue = a->worker % pc->n_qps;
    for (uint64_t r = a->r0; r < a->r1; r++) {
        uint64_t pg = bam_block_request_page(a->req_seed, r, a->n_pages);
        uint64_t slot = a->worker;     /* one private slot per worker: no two requests in flight share it */
        ref_read_data(pc, &pc->qps[queue], pg * pc->n_blocks_per_page, pc->n_blocks_per_page, slot);
        if (a->crc_out)
            a->crc_out[r] = bam_crc32_update(0, pc->base_addr + slot * pc->page_size, pc->page_size);
    }
    return 0;
}

ORC_API int ref_block_read(const uint64_t* store, uint64_t store_bytes, uint32_t page_size,
                           uint32_t n_qps, uint32_t qdepth, uint32_t lba_bytes,
                           uint32_t workers, uint32_t ctrl_threads,
                           uint64_t req_seed, uint64_t n_reqs, uint32_t* crc_out, ref_result_t* out)
{
    if (!store || !out || workers == 0 || ctrl_threads == 0 || n_qps == 0) return 22;
    if (qdepth < 2 || (qdepth & (qdepth - 1)) || page_size % lba_bytes) return 22;
    ref_cache_t pc;
    memset(&pc, 0, sizeof pc);
    pc.page_size = page_size;
    while ((1u << pc.page_size_log) < page_size) pc.page_size_log++;
    pc.n_slots = workers;
    pc.base_addr = (uint8_t*)aligned_alloc(4096, (uint64_t)workers * page_size);
    pc.n_qps = n_qps;
    pc.qps = (ref_qp_t*)aligned_alloc(64, sizeof(ref_qp_t) * n_qps);
    pc.n_blocks_per_page = page_size / lba_bytes;
    pc.ns_id = 1;
    for (uint32_t q = 0; q < n_qps; q++) {
        ref_qp_t* qp = &pc.qps[q];
        memset(qp, 0, sizeof *qp);
        ref_queue_init(&qp->sq, qdepth, sizeof(ref_cmd_t), &qp->sq_db, 1);
        ref_queue_init(&qp->cq, qdepth, sizeof(ref_cpl_t), &qp->cq_db, 0);
    }
    volatile int stop = 0;
    uint32_t n_ct = ctrl_threads < n_qps ? ctrl_threads : n_qps;
    pthread_t* ct = (pthread_t*)calloc(n_ct, sizeof(pthread_t));
    ref_ctrl_arg_t* ca = (ref_ctrl_arg_t*)calloc(n_ct, sizeof(ref_ctrl_arg_t));
    for (uint32_t c = 0; c < n_ct; c++) {
        ca[c] = (ref_ctrl_arg_t){ pc.qps, n_qps, c, n_ct, (const uint8_t*)store, store_bytes, lba_bytes, &stop, 0 };
        pthread_create(&ct[c], 0, ref_ctrl_thread, &ca[c]);
    }
    pthread_t* wt = (pthread_t*)calloc(workers, sizeof(pthread_t));
    ref_block_arg_t* wa = (ref_block_arg_t*)calloc(workers, sizeof(ref_block_arg_t));
    double t0 = now_s();
    for (uint32_t w = 0; w < workers; w++) {
        wa[w] = (ref_block_arg_t){ &pc, req_seed, store_bytes / page_size, n_reqs * w / workers,
                                   n_reqs * (w + 1) / workers, w, workers, crc_out };
        pthread_create(&wt[w], 0, ref_block_thread, &wa[w]);
    }
    for (uint32_t w = 0; w < workers; w++) pthread_join(wt[w], 0);
    double t1 = now_s();
    __atomic_store_n(&stop, 1, __ATOMIC_RELEASE);
    uint64_t served = 0;
    for (uint32_t c = 0; c < n_ct; c++) { pthread_join(ct[c], 0); served += ca[c].served; }
    memset(out, 0, sizeof *out);
    out->accesses = n_reqs; out->read_ios = served; out->misses = n_reqs;
    out->seconds = t1 - t0; out->worker_threads = workers; out->ctrl_threads = n_ct;
    for (uint32_t q = 0; q < n_qps; q++) { ref_queue_free(&pc.qps[q].sq); ref_queue_free(&pc.qps[q].cq); }
    free(pc.qps); free(pc.base_addr); free(ct); free(ca); free(wt); free(wa);
    return 0;
}


/* ---- graph traversals through the restated cache ---------------------------------------------
 * The reference's BFS / CC kernels (benchmarks/bfs/main.cu:658-689, benchmarks/cc/main.cu:123-144,
 * :595-617) on host threads: vertices are handed out in chunks, a thread walks a vertex's neighbour
 * list through a cursor that keeps the current page pinned (bam_ptr, page_cache.h:415-485), labels
 * live in plain memory.  Offsets are read through the cache too, as the GPU build does. */
typedef struct { ref_cache_t* pc; uint64_t page; uint32_t slot; int valid; uint32_t queue; } ref_cursor_t;

static uint64_t ref_cursor_read(ref_cursor_t* c, uint64_t elem)
{
    ref_cache_t* pc = c->pc;
    const uint64_t byte = elem * 8, page = byte >> pc->page_size_log;
    if (!c->valid || c->page != page) {
        if (c->valid) ref_release_page(pc, c->page, 1);
        c->slot = ref_acquire_page(pc, page, 1, c->queue);
        c->page = page; c->valid = 1;
    }
    return *(const uint64_t*)(pc->base_addr + (uint64_t)c->slot * pc->page_size + (byte & (pc->page_size - 1)));
}

static void ref_cursor_done(ref_cursor_t* c) { if (c->valid) { ref_release_page(c->pc, c->page, 1); c->valid = 0; } }

typedef struct {
    ref_cache_t* pc;
    uint64_t n, cols_elem0;
    int mode;                       /* 0 = BFS, 1 = CC */
    uint32_t* level;
    uint64_t* comp;
    uint8_t *curr, *next;
    uint32_t cur_level;
    uint64_t* chunk_cursor;
    int* changed;
    pthread_barrier_t* bar;
    volatile int* finished;
    uint32_t worker, n_workers;
    uint64_t scanned;
    uint32_t iters;
} ref_graph_arg_t;

static void* ref_graph_thread(void* p)
{
    ref_graph_arg_t* a = (ref_graph_arg_t*)p;
    ref_cursor_t co = { a->pc, 0, 0, 0, a->worker % a->pc->n_qps }, ce = co;
    const uint64_t CH = 256;
    for (;;) {
        for (;;) {
            uint64_t v0 = __atomic_fetch_add(a->chunk_cursor, CH, __ATOMIC_RELAXED);
            if (v0 >= a->n) break;
            uint64_t v1 = v0 + CH < a->n ? v0 + CH : a->n;
            for (uint64_t v = v0; v < v1; v++) {
                if (a->mode == 0 ? ld_rlx(&a->level[v]) != a->cur_level : a->curr[v] == 0) continue;
                uint64_t s = ref_cursor_read(&co, v), e = ref_cursor_read(&co, v + 1);
                a->scanned += e - s;
                for (uint64_t i = s; i < e; i++) {
                    uint64_t w = ref_cursor_read(&ce, a->cols_elem0 + i);
                    if (a->mode == 0) {
                        if (ld_rlx(&a->level[w]) == 0xFFFFFFFFu) { st_rlx(&a->level[w], a->cur_level + 1); st_rlx(a->changed, 1); }
                    } else {
                        uint64_t cu = ld_rlx(&a->comp[v]), cw = ld_rlx(&a->comp[w]);
                        if (cu == cw) continue;
                        uint64_t* tgt = cu < cw ? &a->comp[w] : &a->comp[v];
                        uint64_t val = cu < cw ? cu : cw, old = ld_rlx(tgt);
                        while (old > val && !__atomic_compare_exchange_n(tgt, &old, val, 1, __ATOMIC_RELAXED, __ATOMIC_RELAXED)) {}
                        a->next[cu < cw ? w : v] = 1;
                        st_rlx(a->changed, 1);
                    }
                }
            }
        }
        ref_cursor_done(&co); ref_cursor_done(&ce);
        pthread_barrier_wait(a->bar);
        if (a->worker == 0) {                                   /* the host loop between two launches */
            a->iters++;
            if (!*a->changed) *a->finished = 1;
            else {
                *a->changed = 0;
                if (a->mode == 0) { a->cur_level++; }
                else { memset(a->curr, 0, a->n); }
            }
            *a->chunk_cursor = 0;
        }
        pthread_barrier_wait(a->bar);
        if (*a->finished) break;
        if (a->worker != 0) { if (a->mode == 0) a->cur_level++; }
        if (a->mode == 1) { uint8_t* t = a->curr; a->curr = a->next; a->next = t; }
    }
    return 0;
}

/* store = [offsets (n+1 u64, padded to a page) | cols]; mode 0 writes BFS levels (from `source`),
 * mode 1 writes min-vertex labels.  Only the traversal is timed. */
ORC_API int ref_graph_run(const uint64_t* store, uint64_t store_bytes, uint64_t n_vertices, uint64_t cols_byte_offset,
                          int mode, uint64_t source, uint32_t page_size, uint64_t n_slots, uint32_t n_qps, uint32_t qdepth,
                          uint32_t lba_bytes, uint32_t workers, uint32_t ctrl_threads, uint32_t* level_out,
                          uint64_t* comp_out, uint64_t* scanned_out, uint32_t* iters_out, ref_result_t* out)
{
    if (!store || !out || workers == 0 || ctrl_threads == 0 || n_qps == 0 || (mode == 0 ? !level_out : !comp_out)) return 22;
    ref_cache_t pc;
    memset(&pc, 0, sizeof pc);
    pc.page_size = page_size;
    while ((1u << pc.page_size_log) < page_size) pc.page_size_log++;
    pc.n_slots = n_slots;
    pc.base_addr = (uint8_t*)aligned_alloc(4096, n_slots * (uint64_t)page_size);
    pc.slots = (ref_cache_page_t*)calloc(n_slots, sizeof(ref_cache_page_t));
    for (uint64_t s = 0; s < n_slots; s++) pc.slots[s].take_lock = REF_FREE;
    pc.n_data_pages = (store_bytes + page_size - 1) / page_size;
    pc.pages = (ref_data_page_t*)calloc(pc.n_data_pages, sizeof(ref_data_page_t));
    pc.n_qps = n_qps;
    pc.qps = (ref_qp_t*)aligned_alloc(64, sizeof(ref_qp_t) * n_qps);
    pc.n_blocks_per_page = page_size / lba_bytes;
    pc.ns_id = 1;
    for (uint32_t q = 0; q < n_qps; q++) {
        ref_qp_t* qp = &pc.qps[q];
        memset(qp, 0, sizeof *qp);
        ref_queue_init(&qp->sq, qdepth, sizeof(ref_cmd_t), &qp->sq_db, 1);
        ref_queue_init(&qp->cq, qdepth, sizeof(ref_cpl_t), &qp->cq_db, 0);
    }
    volatile int stop = 0;
    uint32_t n_ct = ctrl_threads < n_qps ? ctrl_threads : n_qps;
    pthread_t* ct = (pthread_t*)calloc(n_ct, sizeof(pthread_t));
    ref_ctrl_arg_t* ca = (ref_ctrl_arg_t*)calloc(n_ct, sizeof(ref_ctrl_arg_t));
    for (uint32_t c = 0; c < n_ct; c++) {
        ca[c] = (ref_ctrl_arg_t){ pc.qps, n_qps, c, n_ct, (const uint8_t*)store, store_bytes, lba_bytes, &stop, 0 };
        pthread_create(&ct[c], 0, ref_ctrl_thread, &ca[c]);
    }
    uint8_t* visit = (uint8_t*)malloc(2 * n_vertices);
    if (mode == 0) { for (uint64_t v = 0; v < n_vertices; v++) level_out[v] = 0xFFFFFFFFu; level_out[source] = 0; }
    else { for (uint64_t v = 0; v < n_vertices; v++) comp_out[v] = v; memset(visit, 1, n_vertices); memset(visit + n_vertices, 0, n_vertices); }
    pthread_barrier_t bar;
    pthread_barrier_init(&bar, 0, workers);
    uint64_t chunk_cursor = 0;
    int changed = 0;
    volatile int finished = 0;
    pthread_t* wt = (pthread_t*)calloc(workers, sizeof(pthread_t));
    ref_graph_arg_t* wa = (ref_graph_arg_t*)calloc(workers, sizeof(ref_graph_arg_t));
    double t0 = now_s();
    for (uint32_t w = 0; w < workers; w++) {
        wa[w] = (ref_graph_arg_t){ &pc, n_vertices, cols_byte_offset / 8, mode, level_out, comp_out, visit, visit + n_vertices,
                                   0, &chunk_cursor, &changed, &bar, &finished, w, workers, 0, 0 };
        pthread_create(&wt[w], 0, ref_graph_thread, &wa[w]);
    }
    uint64_t scanned = 0;
    for (uint32_t w = 0; w < workers; w++) { pthread_join(wt[w], 0); scanned += wa[w].scanned; }
    double t1 = now_s();
    __atomic_store_n(&stop, 1, __ATOMIC_RELEASE);
    for (uint32_t c = 0; c < n_ct; c++) pthread_join(ct[c], 0);
    if (scanned_out) *scanned_out = scanned;
    if (iters_out) *iters_out = wa[0].iters;
    memset(out, 0, sizeof *out);
    out->accesses = pc.access_cnt; out->hits = pc.hit_cnt; out->misses = pc.miss_cnt; out->read_ios = pc.read_io_cnt;
    out->seconds = t1 - t0; out->worker_threads = workers; out->ctrl_threads = n_ct;
    pthread_barrier_destroy(&bar);
    for (uint32_t q = 0; q < n_qps; q++) { ref_queue_free(&pc.qps[q].sq); ref_queue_free(&pc.qps[q].cq); }
    free(pc.qps); free(pc.pages); free(pc.slots); free(pc.base_addr); free(ct); free(ca); free(wt); free(wa); free(visit);
    return 0;
}
