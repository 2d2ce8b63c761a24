/*
 * bam/array.cuh -- the array abstraction kernels program against:
 *   range_d_t<T>, array_d_t<T>  (include/page_cache.h:878-1224, :1229-1716 in the reference)
 *   bam_ptr<T>                  (:415-485)  a per-thread cursor that keeps one page pinned
 *   bafs_ptr<T>                 (include/bafs_ptr.h:17-132) a raw-pointer-like façade
 *   bam::array<T>               the name the library's users know the device array by
 *
 * Element index -> (range, page, byte offset) is shift/mask arithmetic.  Lanes of a warp that
 * touch the same page are coalesced with __match_any_sync: the lowest lane of each group pins
 * the page once for the whole group (one fetch-add of the group size), the slot index is
 * broadcast with __shfl_sync, every lane loads its element, and the leader unpins once.
 * Groups are independent: no lane waits for another group between its pin and its unpin, so
 * a warp never holds one page while waiting for another.
 *
 * Element READS of resident pages do not even pin: each lane validates the slot's recycle generation
 * around its load (range_try_read) and only the lanes that could not be served that way -- page
 * absent, being filled or evicted -- go through the coalesced pinning path.  Writes, cursors
 * (bam_ptr) and raw page views keep pinning.
 */
#ifndef BAM_ARRAY_CUH
#define BAM_ARRAY_CUH

#include "cache.cuh"

namespace bam {

template <typename T>
struct range_d_t {
    uint64_t index_start;        /* first element index covered by the range        */
    uint64_t count;              /* one past the last element index (as the reference) */
    uint64_t range_id;
    uint64_t page_start_offset;  /* byte offset of element index_start in its first page */
    uint64_t page_start;         /* first backing page of the range                 */
    uint64_t page_count;
    uint64_t n_elems_per_page;
    uint32_t dist;               /* BAM_DIST_REPLICATE / BAM_DIST_STRIPE over the cache's controllers */
    uint32_t pad_;
    page_cache_d_t cache;

    BAM_DEV uint64_t get_page(size_t i) const { return ((i - index_start) * sizeof(T) + page_start_offset) >> cache.page_size_log; }
    BAM_DEV uint64_t get_subindex(size_t i) const { return ((i - index_start) * sizeof(T) + page_start_offset) & cache.page_size_minus_1; }
    BAM_DEV uint64_t get_global_address(size_t page) const { return (page << cache.n_ranges_bits) | range_id; }
    BAM_DEV uint64_t get_backing_page(size_t page) const { return backing_page_of(page_start, page, cache.n_ctrls, dist); }
    BAM_DEV uint32_t get_backing_ctrl(size_t page) const { return backing_ctrl_of(page, cache.n_ctrls, dist); }
    BAM_DEV uint64_t get_cache_page_addr(uint32_t slot) const { return (uint64_t)(cache.base_addr + (size_t)slot * cache.page_size); }

    /* returns the cache slot (BAM_SLOT_ERR on failure); the page stays pinned `count` times */
    BAM_DEV uint32_t acquire_page(size_t page, uint32_t cnt, bool write, uint32_t queue) const
    {
        return cache_acquire(cache, get_global_address(page), cnt, get_backing_page(page), queue, write, get_backing_ctrl(page));
    }
    /* warp-cooperative form: every lane of `mask` calls it, lanes with want == true pin `page` */
    BAM_DEV uint32_t acquire_page_warp(uint32_t mask, bool want, size_t page, uint32_t cnt, bool write, uint32_t queue) const
    {
        return warp_cache_acquire(mask, want, cache, get_global_address(page), cnt, get_backing_page(page), queue, write,
                                  get_backing_ctrl(page));
    }
    BAM_DEV void release_page(uint32_t slot, uint32_t cnt = 1) const { cache_release(cache, slot, cnt); }
};

/* Pin pages for a warp: every lane of `mask` calls it; each lane with want == true gets the slot
 * of its `page` pinned `cnt` times (one leader may ask on behalf of a group).  The pages are kept
 * by the caller afterwards, so the round is all-or-nothing: if any lane could not claim a slot,
 * the lanes that did get theirs give them back before the warp backs off and tries again --
 * otherwise warps would sit on partial sets of a nearly full cache and wait for each other. */
template <typename T>
BAM_DEV uint32_t range_pin_page(const range_d_t<T>& r, uint32_t mask, bool want, uint64_t page, uint32_t cnt,
                                uint32_t queue, bool write = false)
{
    spin_t sp;
    for (;;) {
        const uint32_t slot = r.acquire_page_warp(mask, want, page, cnt, write, queue);
        if (!__any_sync(mask, want && slot == BAM_SLOT_RETRY)) return slot;
        if (want && slot <= BAM_SLOT_MAX) r.release_page(slot, cnt);
        if (__any_sync(mask, sp.expired(r.cache.status, BAM_AT_FIND_SLOT, page))) return BAM_SLOT_ERR;
        __nanosleep(((get_smid() * 37u + (threadIdx.x >> 5) * 101u) & 255u) * 8u);     /* de-synchronise the warps */
    }
}

template <typename T>
struct array_d_t {
    uint64_t n_elems;
    uint64_t start_offset;
    uint64_t n_ranges;
    range_d_t<T>* d_ranges;

    BAM_DEV int64_t find_range(size_t i) const
    {
        for (int64_t k = 0; k < (int64_t)n_ranges; k++)
            if (d_ranges[k].index_start <= i && d_ranges[k].count > i) return k;
        return -1;
    }

    /* Coalesced pin.  All lanes of `mask` call this together.  Outputs the group mask, its
     * leader and size, and the slot (BAM_SLOT_ERR on failure). */
    BAM_DEV static void coalesce_page(const range_d_t<T>& r, uint32_t mask, uint64_t page, bool write,
                                      uint32_t& eq_mask, uint32_t& leader, uint32_t& cnt, uint32_t& slot)
    {
        const uint64_t gaddr = r.get_global_address(page);
        eq_mask = __match_any_sync(mask, gaddr);
        leader = __ffs(eq_mask) - 1;
        cnt = __popc(eq_mask);
        const uint32_t dirty = __ballot_sync(eq_mask, write) != 0u;
        slot = range_pin_page(r, mask, lane_id() == leader, page, cnt, default_queue(), dirty);
        slot = __shfl_sync(eq_mask, slot, leader);
    }

    BAM_DEV T seq_read(size_t i) const
    {
        const uint32_t mask = __activemask();
        const int64_t ri = find_range(i);
        T v = T();
        /* every active lane takes part in the cooperative acquire; a lane outside every range
         * asks for nothing (and flags the error), lanes of different ranges never share a group
         * because the range id is part of the page's global address */
        const bool valid = ri >= 0;
        const range_d_t<T>& r = d_ranges[valid ? ri : 0];
        /* first without a pin; what that cannot serve goes through the pinning path below */
        const bool fast = valid && range_try_read(r, i, v);
        const uint32_t fm = __ballot_sync(mask, fast);
        if (fm && lane_id() == (uint32_t)(__ffs(fm) - 1)) count_hit(r.cache, __popc(fm));
        if (fm == mask) return v;
        const uint64_t page = valid ? r.get_page(i) : ~0ull;
        const uint64_t key = valid && !fast ? r.get_global_address(page) : ~(uint64_t)lane_id();
        const uint32_t eq = __match_any_sync(mask, key);
        const uint32_t leader = __ffs(eq) - 1;
        const uint32_t cnt = __popc(eq);
        bool pending = valid && !fast;
        spin_t sp;
        for (;;) {
            uint32_t slot = r.acquire_page_warp(mask, pending && lane_id() == leader, valid ? page : 0, cnt, false, default_queue());
            slot = __shfl_sync(eq, slot, leader);
            if (pending && slot != BAM_SLOT_RETRY) {
                if (slot != BAM_SLOT_ERR) v = *reinterpret_cast<const T*>(r.get_cache_page_addr(slot) + r.get_subindex(i));
                __syncwarp(eq);
                if (lane_id() == leader && slot != BAM_SLOT_ERR) r.release_page(slot, cnt);
                pending = false;
            }
            if (!__any_sync(mask, pending)) break;
            if (__any_sync(mask, sp.expired(r.cache.status, BAM_AT_FIND_SLOT, page))) break;
        }
        if (!valid) status_fail(d_ranges[0].cache.status, BAM_ERANGE, BAM_AT_RANGE, i);
        return v;
    }

    BAM_DEV T operator[](size_t i) const { return seq_read(i); }

    /* Shared body of the element updates: pin the page for writing (it becomes DIRTY), apply
     * `op` to the element in the cache, unpin.  Counterpart of seq_write / AtomicAdd
     * (page_cache.h:1577-1609, :1647-1711 in the reference). */
    template <class Op>
    BAM_DEV void update(size_t i, Op op) const
    {
        const uint32_t mask = __activemask();
        const int64_t ri = find_range(i);
        const bool valid = ri >= 0;
        const range_d_t<T>& r = d_ranges[valid ? ri : 0];
        const uint64_t page = valid ? r.get_page(i) : ~0ull;
        const uint64_t key = valid ? r.get_global_address(page) : ~0ull;
        const uint32_t eq = __match_any_sync(mask, key);
        const uint32_t leader = __ffs(eq) - 1;
        const uint32_t cnt = __popc(eq);
        bool pending = valid;
        spin_t sp;
        for (;;) {
            uint32_t slot = r.acquire_page_warp(mask, pending && lane_id() == leader, valid ? page : 0, cnt, true, default_queue());
            slot = __shfl_sync(eq, slot, leader);
            if (pending && slot != BAM_SLOT_RETRY) {
                if (slot != BAM_SLOT_ERR) op(reinterpret_cast<T*>(r.get_cache_page_addr(slot) + r.get_subindex(i)));
                __threadfence();
                __syncwarp(eq);
                if (lane_id() == leader && slot != BAM_SLOT_ERR) r.release_page(slot, cnt);
                pending = false;
            }
            if (!__any_sync(mask, pending)) break;
            if (__any_sync(mask, sp.expired(r.cache.status, BAM_AT_FIND_SLOT, page))) break;
        }
        if (!valid) status_fail(d_ranges[0].cache.status, BAM_ERANGE, BAM_AT_RANGE, i);
    }

    BAM_DEV void seq_write(size_t i, const T val) const { update(i, [val](T* p) { *p = val; }); }
    BAM_DEV void operator()(size_t i, const T val) const { seq_write(i, val); }
    BAM_DEV void AtomicAdd(size_t i, const T val) const
    {
        update(i, [val](T* p) {
            if constexpr (sizeof(T) == 8) atom_add_relaxed(reinterpret_cast<uint64_t*>(p), (uint64_t)val);
            else atomicAdd(p, val);
        });
    }

    /* A pinned view of the page that holds element i (reference: returned_cache_page_t and
     * get_raw / release_raw, page_cache.h:1370-1438): addr points at the first element of the
     * page, size is the number of elements in it, offset the position of element i.  Every lane
     * that calls get_raw(i) calls release_raw(i) with the same i when it is done; lanes of a warp
     * that ask for the same page share one pin.  addr == nullptr after a failure. */
    struct raw_page_t { T* addr; uint32_t size; uint32_t offset; };

    BAM_DEV raw_page_t get_raw(size_t i) const
    {
        raw_page_t ret = { nullptr, 0u, 0u };
        const uint32_t mask = __activemask();
        const int64_t ri = find_range(i);
        const bool valid = ri >= 0;
        const range_d_t<T>& r = d_ranges[valid ? ri : 0];
        const uint64_t page = valid ? r.get_page(i) : ~0ull;
        const uint32_t eq = __match_any_sync(mask, valid ? r.get_global_address(page) : ~0ull);
        const uint32_t leader = __ffs(eq) - 1;
        uint32_t slot = range_pin_page(r, mask, valid && lane_id() == leader, valid ? page : 0, __popc(eq), default_queue());
        slot = __shfl_sync(eq, slot, leader);
        if (!valid) { status_fail(d_ranges[0].cache.status, BAM_ERANGE, BAM_AT_RANGE, i); return ret; }
        if (slot > BAM_SLOT_MAX) return ret;
        ret.addr = reinterpret_cast<T*>(r.get_cache_page_addr(slot));
        ret.size = (uint32_t)(r.cache.page_size / sizeof(T));
        ret.offset = (uint32_t)(r.get_subindex(i) / sizeof(T));
        return ret;
    }

    /* The lanes that call this together must be the lanes that called get_raw together. */
    BAM_DEV void release_raw(size_t i, const raw_page_t& view) const
    {
        const uint32_t mask = __activemask();
        const bool held = view.addr != nullptr;
        const uint32_t eq = __match_any_sync(mask, held ? (uint64_t)(uintptr_t)view.addr : ~0ull);
        if (!held || lane_id() != (uint32_t)(__ffs(eq) - 1)) return;
        const int64_t ri = find_range(i);
        const range_d_t<T>& r = d_ranges[ri >= 0 ? ri : 0];
        const uint32_t slot = (uint32_t)(((uint64_t)(uintptr_t)view.addr - (uint64_t)(uintptr_t)r.cache.base_addr) >> r.cache.page_size_log);
        r.release_page(slot, __popc(eq));
    }

    /* Pin the page of element i and describe it (reference: array_d_t::acquire_page,
     * page_cache.h:1473-1505, what bam_ptr is built on): returns the address of element `start`,
     * the first element of the page; [start, end) are the element indices the page holds; `slot`
     * is what release_page takes. */
    BAM_DEV T* acquire_page(size_t i, uint32_t& slot, size_t& start, size_t& end) const
    {
        raw_page_t v = get_raw(i);
        if (!v.addr) { slot = BAM_SLOT_ERR; start = end = 0; return nullptr; }
        const range_d_t<T>& r = d_ranges[find_range(i)];
        slot = (uint32_t)(((uint64_t)(uintptr_t)v.addr - (uint64_t)(uintptr_t)r.cache.base_addr) >> r.cache.page_size_log);
        start = i - v.offset;
        end = start + v.size;
        return v.addr;
    }
    BAM_DEV void release_page(size_t i, uint32_t slot) const
    {
        const uint32_t mask = __activemask();
        const bool held = slot <= BAM_SLOT_MAX;
        const uint32_t eq = __match_any_sync(mask, held ? (uint64_t)slot : ~0ull);
        if (held && lane_id() == (uint32_t)(__ffs(eq) - 1)) d_ranges[find_range(i)].release_page(slot, __popc(eq));
    }

    /* The whole warp copies `count` elements starting at element i into dest (global or shared
     * memory); all 32 lanes call with the same arguments.  The reference's memcpy
     * (page_cache.h:1256-1316) copies from one page; here the run may cross pages. */
    BAM_DEV void memcpy(uint64_t i, uint64_t count, T* dest) const
    {
        const uint32_t lane = lane_id();
        while (count) {
            const int64_t ri = find_range(i);
            if (ri < 0) { status_fail(d_ranges[0].cache.status, BAM_ERANGE, BAM_AT_RANGE, i); return; }
            const range_d_t<T>& r = d_ranges[ri];
            const uint64_t page = r.get_page(i);
            const uint32_t off = (uint32_t)(r.get_subindex(i) / sizeof(T));
            const uint32_t per_page = (uint32_t)(r.cache.page_size / sizeof(T));
            const uint64_t n = count < per_page - off ? count : per_page - off;
            uint32_t slot = range_pin_page(r, 0xffffffffu, lane == 0, page, 1, default_queue());
            slot = __shfl_sync(0xffffffffu, slot, 0);
            if (slot > BAM_SLOT_MAX) return;
            const T* src = reinterpret_cast<const T*>(r.get_cache_page_addr(slot)) + off;
            if ((((uintptr_t)src | (uintptr_t)dest) & 15u) == 0 && (n * sizeof(T)) % 16 == 0) {
                const uint4* s4 = reinterpret_cast<const uint4*>(src);
                uint4* d4 = reinterpret_cast<uint4*>(dest);
                for (uint64_t k = lane; k < n * sizeof(T) / 16; k += 32) d4[k] = s4[k];
            } else
                for (uint64_t k = lane; k < n; k += 32) dest[k] = src[k];
            __syncwarp();
            if (lane == 0) r.release_page(slot, 1);
            i += n; dest += n; count -= n;
        }
    }
};

/* One element read that pins nothing (cache.cuh: opt_probe / opt_validate); false = not read, take
 * the pinning path.  Per thread, no warp cooperation. */
template <typename T>
BAM_DEV bool range_try_read(const range_d_t<T>& r, size_t i, T& v)
{
    const uint64_t tag = r.get_global_address(r.get_page(i));
    const opt_probe_t pr = opt_probe(r.cache, tag);
    if (pr.slot == BAM_SLOT_NONE) return false;
    v = ld_strong(reinterpret_cast<const T*>(r.get_cache_page_addr(pr.slot) + r.get_subindex(i)));
    BAM_OPT_ORDER();
    return opt_validate(r.cache, tag, pr, opt_dep(v));
}

/* The pinning read, warp-cooperative: every lane of `mask` calls it, lanes with want == true read
 * element i.  Lanes that touch the same page share one pin. */
#ifndef BAM_PINNED_INLINE
#define BAM_PINNED_DEV BAM_DEV_NOINLINE      /* out of line: the miss path's registers stay out of the hit path */
#else
#define BAM_PINNED_DEV BAM_DEV
#endif
template <typename T>
BAM_PINNED_DEV T range_read_pinned(const range_d_t<T>& r, uint32_t mask, bool want, size_t i, uint32_t queue)
{
    const uint64_t page = want ? r.get_page(i) : 0;
    const uint32_t eq = __match_any_sync(mask, want ? page : ~(uint64_t)lane_id());
    const uint32_t leader = __ffs(eq) - 1;
    const uint32_t cnt = __popc(eq);
    T v = T();
    bool pending = want;
    spin_t sp;
    for (;;) {
        uint32_t slot = r.acquire_page_warp(mask, pending && lane_id() == leader, page, cnt, false, queue);
        slot = __shfl_sync(eq, slot, leader);
        if (pending && slot != BAM_SLOT_RETRY) {
            if (slot != BAM_SLOT_ERR) v = *reinterpret_cast<const T*>(r.get_cache_page_addr(slot) + r.get_subindex(i));
            __syncwarp(eq);
            if (lane_id() == leader && slot != BAM_SLOT_ERR) r.release_page(slot, cnt);
            pending = false;
        }
        if (!__any_sync(mask, pending)) break;
        if (__any_sync(mask, sp.expired(r.cache.status, BAM_AT_FIND_SLOT, page))) break;
    }
    return v;
}

/* Same read as array_d_t<T>::seq_read for the common single-range array whose descriptor sits
 * in kernel parameter space (no pointer chasing through global memory per access): first without
 * a pin; the lanes that could not be served that way then pin their pages together. */
template <typename T>
BAM_DEV T range_read(const range_d_t<T>& r, size_t i, uint32_t queue)
{
    const uint32_t mask = __activemask();
    T v = T();
    const bool ok = range_try_read(r, i, v);
    const uint32_t okm = __ballot_sync(mask, ok);
    if (okm && lane_id() == (uint32_t)(__ffs(okm) - 1)) count_hit(r.cache, __popc(okm));
    if (okm != mask) {
        const T x = range_read_pinned(r, mask, !ok, i, queue);
        if (!ok) v = x;
    }
    return v;
}

/* What the batched reader could not serve at once, for one element per lane: every lane of `mask` calls it,
 * lanes with want == true read element i -- first with the full look-up and no pin, then pinned together.
 * Out of line: its registers stay out of the batched loop. */
template <typename T>
struct slow_read_t { T value; uint32_t hit; };          /* hit = 1: served without a page read or a pin */

template <typename T>
BAM_PINNED_DEV slow_read_t<T> range_read_slow(const range_d_t<T>& r, uint32_t mask, bool want, size_t i, uint32_t queue)
{
    slow_read_t<T> out = { T(), 0u };
    if (want && range_try_read(r, i, out.value)) { want = false; out.hit = 1u; }
    if (__any_sync(mask, want)) {
        const T y = range_read_pinned(r, mask, want, i, queue);
        if (want) out.value = y;
    }
    return out;
}

/* N element reads of one thread at once.  The N look-ups, slot records and element loads are issued
 * side by side (straight-line code), so a thread has N independent
 * accesses in flight instead of a chain of dependent ones; reads of the page the thread read last skip
 * the look-up (memo); what cannot be served this way (absent or busy pages, a second candidate in the
 * bucket) is retried with the full look-up and then pinned.
 * n <= N elements are valid; `hits` accumulates the accesses served without a page read. */
template <typename T, int N>
BAM_DEV void range_read_n(const range_d_t<T>& r, const size_t* i, uint32_t n, T* v, uint32_t queue, uint32_t& hits, opt_memo_t& memo)
{
    const uint32_t mask = __activemask();
    uint32_t cand[N];
    opt_probe_t pr[N];
    bool looked_up = false;
#pragma unroll
    for (int b = 0; b < N; b++) {
        const uint64_t tag = r.get_global_address(r.get_page(i[b]));
        const uint64_t h = pt_hash(tag);
        const bool known = tag == memo.tag;
        cand[b] = ((uint32_t)b < n && !known) ? opt_home_candidate(r.cache, (uint32_t)h & r.cache.bucket_mask, (uint32_t)(h >> 56)) : BAM_SLOT_NONE;
        looked_up = looked_up || ((uint32_t)b < n && !known);
    }
#pragma unroll
    for (int b = 0; b < N; b++) {
        const uint64_t tag = r.get_global_address(r.get_page(i[b]));
        pr[b] = opt_probe_record(r.cache, tag, cand[b]);
        if ((uint32_t)b < n && tag == memo.tag) { pr[b].slot = memo.slot; pr[b].gen = memo.gen; }
    }
    if (looked_up) BAM_OPT_ORDER();              /* first samples before the data loads */
#pragma unroll
    for (int b = 0; b < N; b++)
        if (pr[b].slot != BAM_SLOT_NONE) v[b] = ld_strong(reinterpret_cast<const T*>(r.get_cache_page_addr(pr[b].slot) + r.get_subindex(i[b])));
    BAM_OPT_ORDER();                             /* data loads before the validating samples */
    uint32_t dep = 0;
#pragma unroll
    for (int b = 0; b < N; b++)
        if (pr[b].slot != BAM_SLOT_NONE) dep |= opt_dep(v[b]);
    uint32_t need = 0;
    /* one validating sample per slot: neighbours in the batch that read the same slot under the same
     * generation (a run of accesses to one page) share it */
    uint32_t v_slot = BAM_SLOT_NONE, v_gen = 0;
    bool v_ok = false, v_still = false;
#pragma unroll
    for (int b = 0; b < N; b++) {
        const uint64_t tag = r.get_global_address(r.get_page(i[b]));
        bool still = false, ok = false;
        if (pr[b].slot != BAM_SLOT_NONE) {
            if (pr[b].slot == v_slot && pr[b].gen == v_gen) { ok = v_ok; still = v_still; }
            else {
                ok = opt_validate(r.cache, tag, pr[b], dep, &still);
                v_slot = pr[b].slot; v_gen = pr[b].gen; v_ok = ok; v_still = still;
            }
        }
        if (ok) hits++;
        else if ((uint32_t)b < n) need |= 1u << b;
        if (still) { memo.tag = tag; memo.slot = pr[b].slot; memo.gen = pr[b].gen; }
        else if (tag == memo.tag && (uint32_t)b < n) memo.tag = BAM_TAG_NONE;
    }
    if (!__any_sync(mask, need != 0u)) return;
    /* leftovers, one per round, out of line: full look-up without a pin, then the pinning path for the warp */
    while (__any_sync(mask, need != 0u)) {
        const int b = need ? __ffs(need) - 1 : 0;
        size_t ii = i[0];
#pragma unroll
        for (int k = 1; k < N; k++) if (b == k) ii = i[k];
        const slow_read_t<T> x = range_read_slow(r, mask, need != 0u, ii, queue);
        if (need) {
#pragma unroll
            for (int k = 0; k < N; k++) if (b == k) v[k] = x.value;
            hits += x.hit;
            need &= need - 1;
        }
    }
}

/* Per-thread cursor that keeps the page of its last access pinned, so a run of accesses to one
 * page costs one pin/unpin (reference: bam_ptr, page_cache.h:415-485).  p[i] reads the element,
 * p[i] = v writes it (benchmarks/vectoradd/main.cu:103-118 uses both).  Only a real write marks
 * the page dirty; the reference's non-const operator[] marks it on every access (:478-484), which
 * causes spurious write-backs. */
template <typename T>
struct bam_ptr {
    const array_d_t<T>* array = nullptr;
    const range_d_t<T>* range = nullptr;
    uint32_t slot = BAM_SLOT_ERR;
    bool dirty = false;
    size_t start = 0, end = 0;
    T* addr = nullptr;

    struct ref_t {
        bam_ptr* p;
        size_t i;
        BAM_DEV operator T() const { return p->read(i); }
        BAM_DEV ref_t& operator=(const T v) { p->write(i, v); return *this; }
        BAM_DEV ref_t& operator=(const ref_t& o) { p->write(i, (T)o); return *this; }
    };

    BAM_DEV explicit bam_ptr(const array_d_t<T>* a) : array(a) {}
    BAM_DEV ~bam_ptr() { fini(); }

    BAM_DEV void fini()
    {
        if (slot != BAM_SLOT_ERR) {
            const uint32_t mask = __activemask();
            const uint32_t eq = __match_any_sync(mask, ((uint64_t)(uintptr_t)range << 24) ^ slot);
            if (lane_id() == (uint32_t)(__ffs(eq) - 1)) range->release_page(slot, __popc(eq));
            slot = BAM_SLOT_ERR;
            start = end = 0;
            dirty = false;
        }
    }

    BAM_DEV T* update_page(size_t i)
    {
        fini();
        const uint32_t mask = __activemask();
        const int64_t ri = array->find_range(i);
        const bool valid = ri >= 0;
        range = &array->d_ranges[valid ? ri : 0];
        const uint64_t page = valid ? range->get_page(i) : ~0ull;
        const uint64_t key = valid ? range->get_global_address(page) : ~0ull;
        const uint32_t eq = __match_any_sync(mask, key);
        const uint32_t leader = __ffs(eq) - 1;
        slot = range_pin_page(*range, mask, valid && lane_id() == leader, valid ? page : 0, __popc(eq), default_queue());
        slot = __shfl_sync(eq, slot, leader);
        if (!valid) { status_fail(array->d_ranges[0].cache.status, BAM_ERANGE, BAM_AT_RANGE, i); slot = BAM_SLOT_ERR; }
        if (slot == BAM_SLOT_ERR) { addr = nullptr; return nullptr; }
        /* first element index that lives in this page, and one past the last */
        const uint64_t page_byte0 = page << range->cache.page_size_log;
        const uint64_t first_byte = page_byte0 > range->page_start_offset ? page_byte0 - range->page_start_offset : 0;
        start = range->index_start + (first_byte + sizeof(T) - 1) / sizeof(T);
        end = range->index_start + (page_byte0 + range->cache.page_size - range->page_start_offset) / sizeof(T);
        addr = reinterpret_cast<T*>(range->get_cache_page_addr(slot) + range->get_subindex(start));
        return addr;
    }

    BAM_DEV T read(size_t i)
    {
        if (i < start || i >= end) {
            if (update_page(i) == nullptr) return T();
        }
        return addr[i - start];
    }

    BAM_DEV void write(size_t i, const T v)
    {
        if (i < start || i >= end) {
            if (update_page(i) == nullptr) return;
        }
        if (!dirty) { atom_or_relaxed(&range->cache.slots[slot].state, BAM_DIRTY); dirty = true; }
        addr[i - start] = v;
    }

    /* N reads at once: when all N elements lie in the page the cursor holds, their loads are issued
     * back to back (N loads in flight per thread instead of one); otherwise they are read one after
     * the other as read() would.  The reference has no counterpart: its cursor serialises a load
     * behind the use of the previous one. */
    template <int N>
    BAM_DEV void read_n(const size_t* idx, T* out)
    {
        bool here = true;
#pragma unroll
        for (int k = 0; k < N; k++) here = here && idx[k] >= start && idx[k] < end;
        if (here) {
#pragma unroll
            for (int k = 0; k < N; k++) out[k] = addr[idx[k] - start];
        } else {
#pragma unroll 1
            for (int k = 0; k < N; k++) out[k] = read(idx[k]);
        }
    }

    BAM_DEV ref_t operator[](size_t i) { return ref_t{ this, i }; }
};

/* Raw-pointer-like view of an array (reference: include/bafs_ptr.h:17-132). */
template <typename T>
struct bafs_ptr {
    const array_d_t<T>* d = nullptr;
    uint64_t start_idx = 0;

    __host__ __device__ bafs_ptr() {}
    __host__ __device__ bafs_ptr(const array_d_t<T>* a, uint64_t s = 0) : d(a), start_idx(s) {}
    BAM_DEV T operator*() const { return (*d)[start_idx]; }
    BAM_DEV T operator[](uint64_t i) const { return (*d)[start_idx + i]; }
    BAM_DEV void operator()(uint64_t i, const T val) const { (*d)(start_idx + i, val); }
    __host__ __device__ bafs_ptr operator+(uint64_t i) const { return bafs_ptr(d, start_idx + i); }
    __host__ __device__ bafs_ptr operator-(uint64_t i) const { return bafs_ptr(d, start_idx - i); }
    __host__ __device__ bafs_ptr& operator++() { ++start_idx; return *this; }
    __host__ __device__ bafs_ptr operator++(int) { bafs_ptr c(*this); ++start_idx; return c; }
    __host__ __device__ bafs_ptr& operator--() { --start_idx; return *this; }
    __host__ __device__ bafs_ptr operator--(int) { bafs_ptr c(*this); --start_idx; return c; }
    __host__ __device__ bool operator==(const bafs_ptr& o) const { return d == o.d && start_idx == o.start_idx; }
    /* warp-wide copy of `count` elements from element src_idx on (bafs_ptr.h:121-123) */
    BAM_DEV void memcpy_to_array_aligned(uint64_t src_idx, uint64_t count, T* dest) const { d->memcpy(start_idx + src_idx, count, dest); }
    __host__ __device__ bool operator!=(const bafs_ptr& o) const { return !(*this == o); }
};

template <typename T>
using array = array_d_t<T>;

}  // namespace bam
#endif
