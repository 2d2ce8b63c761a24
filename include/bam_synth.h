/*
 * bam_synth.h -- seeded synthetic inputs shared by host (gcc) and device (nvcc) code.
 *
 * Every benchmark input of this library is a pure function of (seed, index), so the
 * backing store, the access streams and the graphs can be regenerated anywhere and
 * the results (checksums, page CRCs, BFS levels, CC labels) compared bit for bit.
 * The reference draws its access patterns from unseeded rand()
 * (benchmarks/array/main.cu:156-158, benchmarks/block/main.cu:323-325), which cannot be
 * reproduced; these generators replace that.
 *
 * Everything here is integer arithmetic: no floating point is evaluated on the device,
 * so host and device agree by construction.  The functions are pinned by published
 * known-answer vectors in the test-suite (splitmix64, PCG32 demo stream, CRC-32 check
 * value), so a transcription error in this file cannot hide behind "both sides agree".
 */
#ifndef BAM_SYNTH_H
#define BAM_SYNTH_H

#include <stdint.h>
#include <stddef.h>

#if defined(__CUDACC__)
#define BAM_HD __host__ __device__ __forceinline__
#else
#define BAM_HD static inline
#endif

/* ---- splitmix64 -------------------------------------------------------------------
 * bam_splitmix64(x) is the value Steele/Lea/Flood's SplitMix64 generator returns from
 * the call that finds its state equal to x (the state is advanced by the golden gamma
 * first).  Backing-store element i is bam_splitmix64(seed ^ i). */
BAM_HD uint64_t bam_splitmix64(uint64_t x)
{
    uint64_t z = x + 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

BAM_HD uint64_t bam_store_elem(uint64_t seed, uint64_t i) { return bam_splitmix64(seed ^ i); }

/* ---- PCG32 (XSH-RR 64/32, O'Neill) ------------------------------------------------ */
typedef struct { uint64_t state; uint64_t inc; } bam_pcg32_t;

BAM_HD uint32_t bam_pcg32_next(bam_pcg32_t* g)
{
    uint64_t old = g->state;
    g->state = old * 6364136223846793005ull + g->inc;
    uint32_t xorshifted = (uint32_t)(((old >> 18u) ^ old) >> 27u);
    uint32_t rot = (uint32_t)(old >> 59u);
    return (xorshifted >> rot) | (xorshifted << ((32u - rot) & 31u));
}

BAM_HD void bam_pcg32_seed(bam_pcg32_t* g, uint64_t initstate, uint64_t initseq)
{
    g->state = 0u;
    g->inc = (initseq << 1u) | 1u;
    (void)bam_pcg32_next(g);
    g->state += initstate;
    (void)bam_pcg32_next(g);
}

/* One 64-bit draw = two consecutive 32-bit draws, first draw in the high half. */
BAM_HD uint64_t bam_pcg32_next64(bam_pcg32_t* g)
{
    uint64_t hi = bam_pcg32_next(g);
    uint64_t lo = bam_pcg32_next(g);
    return (hi << 32) | lo;
}

/* Uniform index in [0, n): the 64-bit draw reduced modulo n (a mask when n is a power
 * of two, which is the case in every stated configuration, so there is no modulo bias
 * there). */
BAM_HD uint64_t bam_uniform_index(bam_pcg32_t* g, uint64_t n)
{
    uint64_t r = bam_pcg32_next64(g);
    return ((n & (n - 1)) == 0) ? (r & (n - 1)) : (r % n);
}

/* Access k of reader lane `lane` in the array random-read workload: the lane owns PCG32
 * stream `lane` seeded with `seed` and draws its indices in order. */
BAM_HD void bam_lane_stream(bam_pcg32_t* g, uint64_t seed, uint64_t lane)
{
    bam_pcg32_seed(g, seed, lane);
}

/* Request r of the block random-read workload: one generator (stream 0) would serialise
 * the requests, so request r owns stream r and its page is that stream's first draw. */
BAM_HD uint64_t bam_block_request_page(uint64_t seed, uint64_t r, uint64_t n_pages)
{
    bam_pcg32_t g;
    bam_pcg32_seed(&g, seed, r);
    return bam_uniform_index(&g, n_pages);
}

/* ---- CRC-32 (IEEE 802.3, reflected, poly 0xEDB88320; equals zlib's crc32) --------- */
BAM_HD uint32_t bam_crc32_update(uint32_t crc, const uint8_t* p, size_t n)
{
    crc = ~crc;
    for (size_t i = 0; i < n; i++) {
        crc ^= p[i];
        for (int k = 0; k < 8; k++) crc = (crc >> 1) ^ (0xEDB88320u & (0u - (crc & 1u)));
    }
    return ~crc;
}

/* Same CRC consumed a 64-bit little-endian word at a time (pages are arrays of u64). */
BAM_HD uint32_t bam_crc32_u64(uint32_t crc_state /* pre-inverted */, uint64_t w)
{
    uint32_t crc = crc_state;
    for (int b = 0; b < 8; b++) {
        crc ^= (uint32_t)(w & 0xffu);
        w >>= 8;
        for (int k = 0; k < 8; k++) crc = (crc >> 1) ^ (0xEDB88320u & (0u - (crc & 1u)));
    }
    return crc;
}

/* ---- bijection on [0, n) used as the Zipf rank -> page permutation ------------------
 * Rounds of (multiply by an odd constant, xor-shift, add key) on k = ceil(log2 n) bits are
 * each invertible modulo 2^k; values that land at or beyond n are walked again (cycle
 * walking), which keeps the map a bijection on [0, n). */
BAM_HD uint32_t bam_ceil_log2_u64(uint64_t n)
{
    uint32_t k = 0;
    while (k < 63 && ((uint64_t)1 << k) < n) k++;
    return k;
}

BAM_HD uint64_t bam_permute_once(uint64_t x, uint32_t k, uint64_t mask, uint64_t key)
{
    uint32_t h = (k + 1) / 2;
    if (h == 0) return x;
    x = (x * 0x9E3779B97F4A7C15ull + key) & mask;
    x ^= x >> h;
    x = (x * 0xD6E8FEB86659FD93ull + (key >> 17)) & mask;
    x ^= x >> h;
    x = (x * 0xC2B2AE3D27D4EB4Full + (key >> 31)) & mask;
    x ^= x >> h;
    return x;
}

BAM_HD uint64_t bam_permute(uint64_t x, uint64_t n, uint64_t seed)
{
    uint32_t k = bam_ceil_log2_u64(n);
    uint64_t mask = (k >= 64) ? ~0ull : (((uint64_t)1 << k) - 1);
    uint64_t key = bam_splitmix64(seed ^ 0x5bd1e995u);
    do { x = bam_permute_once(x, k, mask, key); } while (x >= n);
    return x;
}

/* ---- Zipf rank from a fixed-point CDF table ----------------------------------------
 * cdf[r] = floor(2^64 * P(rank <= r)) clipped to 2^64-1, built once on the host (it needs
 * pow(); the device only does integer compares).  The rank of a 64-bit draw u is the first
 * r with u < cdf[r]; the last entry is forced to 2^64-1 and u == 2^64-1 maps to n-1. */
BAM_HD uint64_t bam_zipf_rank(const uint64_t* cdf, uint64_t n, uint64_t u)
{
    uint64_t lo = 0, hi = n - 1;
    while (lo < hi) {
        uint64_t mid = lo + ((hi - lo) >> 1);
        if (u < cdf[mid]) hi = mid; else lo = mid + 1;
    }
    return lo;
}

/* Access k of the skewed scan of one shard: stream id = lane, draws in order:
 * one 64-bit draw for the rank, one 32-bit draw for the element offset in the page. */
BAM_HD uint64_t bam_zipf_access(bam_pcg32_t* g, const uint64_t* cdf, uint64_t n_pages,
                                uint32_t elems_per_page, uint64_t perm_seed)
{
    uint64_t u = bam_pcg32_next64(g);
    uint64_t rank = bam_zipf_rank(cdf, n_pages, u);
    uint64_t page = bam_permute(rank, n_pages, perm_seed);
    uint32_t off = bam_pcg32_next(g) % elems_per_page;
    return page * elems_per_page + off;
}

/* ---- R-MAT edge generator -----------------------------------------------------------
 * Edge e of a scale-`scale` R-MAT graph: stream e of PCG32 gives one 32-bit draw per level;
 * the draw picks a quadrant by the integer thresholds ta = a*2^32, tab = (a+b)*2^32,
 * tabc = (a+b+c)*2^32 (floor), computed once by the caller. */
typedef struct { uint32_t ta, tab, tabc; } bam_rmat_thresh_t;

BAM_HD void bam_rmat_edge(uint64_t seed, uint64_t e, uint32_t scale, bam_rmat_thresh_t t,
                          uint64_t* src, uint64_t* dst)
{
    bam_pcg32_t g;
    bam_pcg32_seed(&g, seed, e);
    uint64_t u = 0, v = 0;
    for (uint32_t l = 0; l < scale; l++) {
        uint32_t r = bam_pcg32_next(&g);
        uint32_t ubit = (r >= t.tab);                 /* quadrants c,d: lower half  */
        uint32_t vbit = (r >= t.ta && r < t.tab) || (r >= t.tabc); /* b or d: right half */
        u = (u << 1) | ubit;
        v = (v << 1) | vbit;
    }
    *src = u;
    *dst = v;
}

/* ---- edge weights and fixed-point arithmetic of the weighted / ranking traversals ---------------
 * Weight of CSR edge j (its position in the column array): 1..64.  (The reference reads weights
 * from a .val file beside the .bel files, benchmarks/sssp/main.cu:379-431.) */
BAM_HD uint32_t bam_edge_weight(uint64_t seed, uint64_t j)
{
    return 1u + (uint32_t)(bam_splitmix64(seed ^ j) >> 58);
}

/* PageRank quantities are 64-bit fixed-point numbers with this many fraction bits; the damping
 * factor is the ratio alpha_num / alpha_den. */
#define BAM_PR_FRAC_BITS 40

/* floor(x * num / den) without overflow for num < den. */
BAM_HD uint64_t bam_mul_ratio(uint64_t x, uint64_t num, uint64_t den)
{
    return x / den * num + (x % den) * num / den;
}

#endif /* BAM_SYNTH_H */
