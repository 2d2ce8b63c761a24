/*
 * bam/cache.cuh -- the GPU-resident software page cache.
 *
 * Role of the reference's page_cache_d_t + range_d_t<T>::acquire_page + find_slot
 * (include/page_cache.h:1122-1224, :1786-1927), redesigned:
 *
 *  - The page table is HASHED and sized by the cache, not by the backing store.  The
 *    reference keeps one 32-byte state entry per page of the backing store
 *    (page_cache.h:96-102), i.e. 512 MiB of table for a 64 GiB store.  Here a bucket is one
 *    32-byte sector: a control word (insert lock + overflow count) and seven entries of
 *    (8-bit fingerprint | 24-bit slot index).  A look-up is two 128-bit loads of the home
 *    bucket plus one 8-byte tag check; buckets overflow into their successors (linear
 *    probing at bucket granularity, bounded by BAM_MAX_PROBE).
 *  - The 32-bit state word (VALID | BUSY | DIRTY | pin count: the encodings of
 *    page_cache.h:57-62) belongs to the cache slot.  Readers pin with one fetch-add and then
 *    validate the slot's tag; eviction claims a slot with a 32-bit CAS that only succeeds on
 *    an unpinned, non-busy word, so a pinned page can never be recycled and a reader that
 *    raced with a recycle sees a tag mismatch, undoes its pin and looks the page up again.
 *  - Eviction is a clock sweep over the slots (the reference's page_ticket hand, :1802), with up to 16 hands
 *    for a large cache: the SMs are dealt over the hands and every hand sweeps its own residue class of
 *    slots, so the misses of the whole GPU do not meet on one counter.
 *  - Read-only element accesses to resident pages take no pin at all: they validate a recycle
 *    generation around the data load (opt_probe / opt_validate below) and fall back to the pinning
 *    path on any doubt.
 *
 * Slot life cycle:   0 (free) --CAS--> BUSY (filling) --xor--> VALID (+pins)
 *                    VALID,0 pins --CAS--> VALID|BUSY (evicting: tag cleared, entry removed)
 *                    --and--> BUSY (filling for the new page) ...
 */
#ifndef BAM_CACHE_CUH
#define BAM_CACHE_CUH

#include "queue.cuh"

namespace bam {

BAM_DEV uint64_t pt_hash(uint64_t tag)
{
    uint64_t h = tag * 0x9E3779B97F4A7C15ull;
    h ^= h >> 32;
    h *= 0xD6E8FEB86659FD93ull;
    h ^= h >> 29;
    return h;
}

/* Find the slot holding `tag`, or BAM_SLOT_NONE.  Lock-free. */
BAM_DEV uint32_t pt_lookup(const page_cache_d_t& pc, uint64_t tag, uint32_t home, uint32_t fp)
{
    uint32_t b = home;
#pragma unroll 1
    for (uint32_t probe = 0; probe < BAM_MAX_PROBE; probe++) {
        const uint32_t* w = pc.table + (size_t)b * BAM_BUCKET_WORDS;
        const uint4 lo = ld_cg_v4(w);
        const uint4 hi = ld_cg_v4(w + 4);
        const uint32_t e[8] = { lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w };
#pragma unroll
        for (int i = 1; i < 8; i++) {
            if (e[i] != BAM_ENTRY_EMPTY && (e[i] >> 24) == fp) {
                uint32_t s = e[i] & 0xffffffu;
                if (ld_relaxed_gpu(&pc.slots[s].tag) == tag) return s;
            }
        }
        if (probe == 0 && (e[0] & ~BAM_BUCKET_LOCK) == 0u) return BAM_SLOT_NONE;
        b = (b + 1u) & pc.bucket_mask;
    }
    return BAM_SLOT_NONE;
}

#define BAM_PT_OK 0
#define BAM_PT_EXISTS 1
#define BAM_PT_FULL 2
#define BAM_PT_TIMEOUT 3

/* Insert tag -> slot.  Inserts of keys with the same home bucket are serialised by the
 * bucket's lock bit and re-check for the key under the lock, so a page is never present twice. */
BAM_DEV int pt_insert(const page_cache_d_t& pc, uint64_t tag, uint32_t slot, uint32_t home, uint32_t fp)
{
    uint32_t* ctl = pc.table + (size_t)home * BAM_BUCKET_WORDS;
    spin_t sp;
    while (atom_or_acquire(ctl, BAM_BUCKET_LOCK) & BAM_BUCKET_LOCK)
        if (sp.expired(pc.status, BAM_AT_BUCKET_LOCK, home)) return BAM_PT_TIMEOUT;
    int rc = BAM_PT_FULL;
    if (pt_lookup(pc, tag, home, fp) != BAM_SLOT_NONE) {
        rc = BAM_PT_EXISTS;
    } else {
        const uint32_t entry = (fp << 24) | slot;
        uint32_t b = home;
#pragma unroll 1
        for (uint32_t probe = 0; probe < BAM_MAX_PROBE && rc == BAM_PT_FULL; probe++) {
            uint32_t* w = pc.table + (size_t)b * BAM_BUCKET_WORDS;
            if (probe == 1) atom_add_relaxed(ctl, 1u);     /* the key will live outside its home */
            for (int i = 1; i < 8; i++) {
                if (ld_relaxed_gpu(&w[i]) == BAM_ENTRY_EMPTY &&
                    atom_cas_relaxed(&w[i], BAM_ENTRY_EMPTY, entry) == BAM_ENTRY_EMPTY) {
                    rc = BAM_PT_OK;
                    break;
                }
            }
            b = (b + 1u) & pc.bucket_mask;
        }
        if (rc == BAM_PT_FULL && BAM_MAX_PROBE > 1) atom_add_relaxed(ctl, 0xffffffffu);   /* undo the overflow count */
    }
    atom_and_release(ctl, ~BAM_BUCKET_LOCK);
    return rc;
}

/* Remove the entry that maps to `slot` (the caller has claimed the slot). */
BAM_DEV void pt_remove(const page_cache_d_t& pc, uint64_t tag, uint32_t slot)
{
    const uint64_t h = pt_hash(tag);
    const uint32_t home = (uint32_t)h & pc.bucket_mask;
    const uint32_t entry = ((uint32_t)(h >> 56) << 24) | slot;
    uint32_t b = home;
#pragma unroll 1
    for (uint32_t probe = 0; probe < BAM_MAX_PROBE; probe++) {
        uint32_t* w = pc.table + (size_t)b * BAM_BUCKET_WORDS;
        for (int i = 1; i < 8; i++) {
            if (ld_relaxed_gpu(&w[i]) == entry) {
                st_release_gpu(&w[i], BAM_ENTRY_EMPTY);
                if (b != home) atom_add_relaxed(pc.table + (size_t)home * BAM_BUCKET_WORDS, 0xffffffffu);
                return;
            }
        }
        b = (b + 1u) & pc.bucket_mask;
    }
}

BAM_DEV uint64_t slot_bus_addr(const page_cache_d_t& pc, uint32_t slot)
{
    return (uint64_t)(pc.base_addr + (size_t)slot * pc.page_size);
}

/* Clock sweep: returns a slot claimed for the caller (state BUSY, no tag, no table entry), or
 * BAM_SLOT_ERR; with max_tries it gives up after that many probes and returns BAM_SLOT_NONE.
 * Counterpart of page_cache_d_t::find_slot (page_cache.h:1786-1927). */
BAM_DEV uint32_t find_slot(const page_cache_d_t& pc, uint32_t max_tries = 0xffffffffu, uint64_t* dirty_tag = nullptr)
{
    spin_t sp;
    if (dirty_tag) *dirty_tag = BAM_TAG_NONE;
#pragma unroll 1
    for (uint32_t tries = 1;; tries++) {
        if (tries > max_tries) return BAM_SLOT_NONE;          /* caller asked for a bounded attempt */
        /* one hand per group of SMs instead of one counter for the whole GPU (the reference's page_ticket is
         * a single address every miss of every SM hits): hand h visits the slots s = k * n_hands + h in order */
        const uint32_t hand = get_smid() & (pc.n_hands - 1u);
        const uint64_t t = atom_add_relaxed(pc.clock_hand + (size_t)hand * BAM_HAND_STRIDE, 1ull);
        const uint32_t per_hand = (pc.n_slots - hand + pc.n_hands - 1u) / pc.n_hands;       /* slots of this hand (>= 1) */
        const uint32_t s = (uint32_t)(t % per_hand) * pc.n_hands + hand;
        bam_slot_t* sl = &pc.slots[s];
        const uint32_t st = ld_relaxed_gpu(&sl->state);
        if (st == 0u) {
            if (atom_cas_acquire(&sl->state, 0u, BAM_BUSY) == 0u) { BAM_PROF_ADD(pc.status, 12, 1); BAM_PROF_ADD(pc.status, 13, tries); return s; }
        } else if ((st & ~BAM_DIRTY) == BAM_VALID && (!(st & BAM_DIRTY) || dirty_tag)) {
            /* a dirty victim is left alone by a caller that cannot write it back */
            if (atom_cas_acquire(&sl->state, st, st | BAM_BUSY) == st) {
                /* the slot is claimed: readers that hold no pin must learn of it before the tag goes
                 * and long before other data can land here (the releases below order the bump first) */
                red_add_relaxed(&sl->gen, 1u);
                if (st & BAM_DIRTY) {
                    /* the victim must reach the backing store first.  Its tag and table entry stay,
                     * so anyone who wants that page meanwhile finds the slot VALID|BUSY and waits
                     * instead of reading a stale copy from the store; finish_evict() ends it. */
                    *dirty_tag = ld_relaxed_gpu(&sl->tag);
                    return s;
                }
                const uint64_t old = ld_relaxed_gpu(&sl->tag);
                st_relaxed_gpu(&sl->tag, BAM_TAG_NONE);
                pt_remove(pc, old, s);
                atom_and_release(&sl->state, ~(BAM_VALID | BAM_DIRTY));
                BAM_PROF_ADD(pc.status, 11, 1); BAM_PROF_ADD(pc.status, 13, tries);
                return s;
            }
        }
        /* every path that did not claim a slot ends here: the wait is bounded whatever the sweep met */
        if ((tries & 63u) == 0u && sp.expired(pc.status, BAM_AT_FIND_SLOT)) return BAM_SLOT_ERR;
    }
}

/* Second half of the eviction of a dirty victim, after its write-back has completed. */
BAM_DEV void finish_evict(const page_cache_d_t& pc, uint32_t s, uint64_t old_tag)
{
    bam_slot_t* sl = &pc.slots[s];
    st_relaxed_gpu(&sl->tag, BAM_TAG_NONE);
    pt_remove(pc, old_tag, s);
    atom_and_release(&sl->state, ~(BAM_VALID | BAM_DIRTY));
}

/* Where page `page` of a range lives when the cache is backed by n_ctrls controllers
 * (get_backing_page_ / get_backing_ctrl_, page_cache.h:558-582): a replicated range is whole on
 * every controller; a striped range deals its pages round-robin. */
BAM_DEV uint64_t backing_page_of(uint64_t page_start, uint64_t page, uint32_t n_ctrls, uint32_t dist)
{
    return page_start + ((dist == BAM_DIST_STRIPE && n_ctrls > 1) ? page / n_ctrls : page);
}
BAM_DEV uint32_t backing_ctrl_of(uint64_t page, uint32_t n_ctrls, uint32_t dist)
{
    return (dist == BAM_DIST_STRIPE && n_ctrls > 1) ? (uint32_t)(page % n_ctrls) : BAM_ALL_CTRLS;
}

/* Backing page (and controller) of a cached page, from its tag: (page in range << range bits) | range id. */
BAM_DEV uint64_t backing_location_of_tag(const page_cache_d_t& pc, uint64_t tag, uint32_t& ctrl)
{
    const uint32_t rid = (uint32_t)(tag & pc.n_ranges_mask);
    const uint64_t page = tag >> pc.n_ranges_bits;
    const uint32_t dist = pc.n_ctrls > 1 ? ld_relaxed_gpu(&pc.range_dists[rid]) : BAM_DIST_REPLICATE;
    ctrl = backing_ctrl_of(page, pc.n_ctrls, dist);
    return backing_page_of(ld_relaxed_gpu(&pc.range_page_starts[rid]), page, pc.n_ctrls, dist);
}

/* The value callers spread their requests over queues with: the global warp index. */
BAM_DEV uint32_t default_queue() { return (blockIdx.x * blockDim.x + threadIdx.x) >> 5; }

/* The queue pair a request goes to.  `queue` is the caller's spreading value (its global warp
 * index); `ctrl` is the controller that owns the page, or BAM_ALL_CTRLS when any will do (the
 * reference draws from a global counter there, page_cache.h:1150-1152; here the warp index picks
 * the controller and its remaining bits the queue, so all queues of all controllers are used). */
BAM_DEV QueuePair* pick_queue(const page_cache_d_t& pc, uint32_t ctrl, uint32_t queue)
{
    if (pc.n_ctrls <= 1) { Controller* c = pc.d_ctrl; return c->d_qps + (queue % c->n_qps); }
    if (ctrl == BAM_ALL_CTRLS) ctrl = queue % pc.n_ctrls;
    Controller* c = pc.d_ctrls[ctrl];
    return c->d_qps + ((queue / pc.n_ctrls) % c->n_qps);
}

BAM_DEV uint64_t slot_prp2(const page_cache_d_t& pc, uint32_t slot)
{
    if (pc.page_size <= 4096) return 0;
    const uint64_t bus = (uint64_t)(pc.base_addr + (size_t)slot * pc.page_size);
    return (pc.page_size <= 8192) ? bus + 4096 : (uint64_t)(pc.prp_lists + (size_t)slot * pc.prp_list_stride);
}

/* Write cache slot `slot`, which holds the page `tag`, back to its backing store; all lanes of
 * `mask` call it, lanes with wb == true have a page to write.  A replicated page goes to every
 * controller (page_cache.h:1856-1862), a striped page to the one that owns it. */
BAM_DEV int warp_write_back(uint32_t mask, bool wb, const page_cache_d_t& pc, uint64_t tag, uint32_t slot)
{
    const uint32_t queue = default_queue();
    uint32_t ctrl = 0;
    const uint64_t lba = wb ? backing_location_of_tag(pc, tag, ctrl) * pc.n_blocks_per_page : 0;
    const uint64_t bus = wb ? slot_bus_addr(pc, slot) : 0;
    const uint64_t prp2 = wb ? slot_prp2(pc, slot) : 0;
    int rc = BAM_OK;
#pragma unroll 1
    for (uint32_t k = 0; k < pc.n_ctrls; k++) {
        const bool go = wb && (ctrl == BAM_ALL_CTRLS || ctrl == k);
        if (!__any_sync(mask, go)) continue;
        const int r = warp_io(mask, go, pick_queue(pc, k, queue), lba, pc.n_blocks_per_page, bus, prp2, NVM_IO_WRITE);
        if (go && r != BAM_OK) rc = r;
    }
    return rc;
}

/* Raw block I/O between the backing store and cache slot pc_entry, under the reference's names
 * (read_data / write_data / access_data, page_cache.h:2009-2132): one thread, blocking; any number
 * of threads may call concurrently and divergently.  Returns BAM_OK or an error code. */
BAM_DEV int access_data(const page_cache_d_t* pc, QueuePair* qp, uint64_t starting_lba, uint64_t n_blocks,
                        unsigned long long pc_entry, uint8_t opcode)
{
    return access_data_raw(qp, starting_lba, (uint32_t)n_blocks, slot_bus_addr(*pc, (uint32_t)pc_entry), slot_prp2(*pc, (uint32_t)pc_entry), opcode);
}
BAM_DEV int read_data(const page_cache_d_t* pc, QueuePair* qp, uint64_t starting_lba, uint64_t n_blocks, unsigned long long pc_entry)
{
    return access_data(pc, qp, starting_lba, n_blocks, pc_entry, NVM_IO_READ);
}
BAM_DEV int write_data(const page_cache_d_t* pc, QueuePair* qp, uint64_t starting_lba, uint64_t n_blocks, unsigned long long pc_entry)
{
    return access_data(pc, qp, starting_lba, n_blocks, pc_entry, NVM_IO_WRITE);
}
/* The asynchronous pair (access_data_async / poll_async, page_cache.h:1930-1959): submit now, wait
 * later.  A thread must keep fewer commands outstanding than the queue is deep.  *cid identifies
 * the command for poll_async; *sq_pos is the submission slot (informational). */
BAM_DEV int access_data_async(const page_cache_d_t* pc, QueuePair* qp, uint64_t starting_lba, uint64_t n_blocks,
                              unsigned long long pc_entry, uint8_t opcode, uint16_t* cid, uint16_t* sq_pos)
{
    uint32_t c = 0, pos = 0;
    const int rc = access_data_submit(qp, starting_lba, (uint32_t)n_blocks, slot_bus_addr(*pc, (uint32_t)pc_entry),
                                      slot_prp2(*pc, (uint32_t)pc_entry), opcode, &c, &pos);
    *cid = (uint16_t)c;
    *sq_pos = (uint16_t)pos;
    return rc;
}
BAM_DEV int poll_async(QueuePair* qp, uint16_t cid, uint16_t /*sq_pos*/) { return access_data_complete(qp, cid); }

/* ---- reads that pin nothing -------------------------------------------------------------------
 * A read-only access to a resident page needs no pin: look the slot up, sample {state, gen}, read the
 * element, sample {tag, state, gen} again.  The slot held the page during the whole read if it was
 * VALID and not BUSY at the first sample and its generation and tag are unchanged at the second:
 * an eviction bumps the generation right after it claims the slot, before the tag is cleared and long
 * before the fill of another page can write into the slot.  Anything else -- page absent, being filled
 * or evicted, recycled under the reader -- makes the caller fall back to the pinning path.  Two L2
 * atomics per access of the pinning hit path become none.
 *
 * The three steps must be PERFORMED in order: first sample -> data load -> second sample.  All three are
 * strong (L2-coherent) loads.  By default the order comes from dependencies, which cost nothing:
 *   - the data load's address is selected by the outcome of the first sample's check, so it cannot be
 *     issued before that sample has returned;
 *   - the second sample's slot index is computed from the loaded value (opt_dep: 0 for every value but
 *     one reserved bit pattern, which the compiler cannot know), so it cannot be issued before the data
 *     has arrived.  For the reserved pattern the second sample looks at slot 0, the validation fails
 *     and the pinning path serves the read: slower, never wrong.
 * A load that is issued after another has returned is performed after it; the GPU does not speculate.
 * With -DBAM_OPT_USE_FENCES the same order is enforced with fence.acq_rel.gpu between the steps instead
 * (what the PTX memory model spells out; measured 10-35 % slower on all-hit reads). */
#ifdef BAM_OPT_USE_FENCES
#define BAM_OPT_ORDER() fence_acq_rel_gpu()
#else
#define BAM_OPT_ORDER() do {} while (0)
#endif

#define BAM_OPT_RESERVED64 0x7c3a9e1fd25b6048ull
#define BAM_OPT_RESERVED32 0xd25b6048u

/* 0 for every loaded value but one; a true data dependency on the value. */
template <typename T>
BAM_DEV uint32_t opt_dep(const T& v)
{
#ifdef BAM_OPT_USE_FENCES
    return 0u;
#else
    if constexpr (sizeof(T) == 8) return *reinterpret_cast<const uint64_t*>(&v) == BAM_OPT_RESERVED64 ? 1u : 0u;
    else if constexpr (sizeof(T) == 4) return *reinterpret_cast<const uint32_t*>(&v) == BAM_OPT_RESERVED32 ? 1u : 0u;
    else { fence_acq_rel_gpu(); return 0u; }            /* other element sizes: a real fence */
#endif
}

struct opt_probe_t {
    uint32_t slot;      /* BAM_SLOT_NONE: take the pinning path */
    uint32_t gen;
};

/* First half: look-up and first sample.  pr.slot, which the caller's data address is built from, is
 * selected by the sample's check. */
BAM_DEV opt_probe_t opt_probe(const page_cache_d_t& pc, uint64_t tag)
{
    opt_probe_t pr = { BAM_SLOT_NONE, 0u };
    const uint64_t h = pt_hash(tag);
    const uint32_t s = pt_lookup(pc, tag, (uint32_t)h & pc.bucket_mask, (uint32_t)(h >> 56));
    if (s == BAM_SLOT_NONE) return pr;
    const uint64_t sg = ld_relaxed_gpu(reinterpret_cast<const uint64_t*>(&pc.slots[s].state));
    if (((uint32_t)sg & (BAM_VALID | BAM_BUSY)) != BAM_VALID) return pr;
    pr.slot = s;
    pr.gen = (uint32_t)(sg >> 32);
    BAM_OPT_ORDER();
    return pr;
}

/* The same for the common case, as straight-line code so that several probes of one thread overlap:
 * only the home bucket is examined and only its first entry with the right fingerprint; the slot
 * record {tag, state, gen} is one 128-bit load.  Returns BAM_SLOT_NONE whenever the full look-up
 * would have to go on (another candidate, an overflowed bucket). */
BAM_DEV uint32_t opt_home_candidate(const page_cache_d_t& pc, uint32_t home, uint32_t fp)
{
    const uint32_t* w = pc.table + (size_t)home * BAM_BUCKET_WORDS;
    const uint4 lo = ld_cg_v4(w);
    const uint4 hi = ld_cg_v4(w + 4);
    const uint32_t e[8] = { lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w };
    uint32_t cand = BAM_SLOT_NONE;
#pragma unroll
    for (int i = 7; i >= 1; i--)
        if (e[i] != BAM_ENTRY_EMPTY && (e[i] >> 24) == fp) cand = e[i] & 0xffffffu;
    return cand;
}
BAM_DEV opt_probe_t opt_probe_record(const page_cache_d_t& pc, uint64_t tag, uint32_t cand)
{
    opt_probe_t pr = { BAM_SLOT_NONE, 0u };
    if (cand == BAM_SLOT_NONE) return pr;
    const uint4 rec = ld_relaxed_gpu_v4(&pc.slots[cand]);
    if (((((uint64_t)rec.y) << 32) | rec.x) != tag || (rec.z & (BAM_VALID | BAM_BUSY)) != BAM_VALID) return pr;
    pr.slot = cand;
    pr.gen = rec.w;
    return pr;
}

/* Second half, after the data load: true if the data belonged to `tag`.  `dep` is opt_dep() of the
 * loaded value(s).  *still_valid (optional) tells whether this sample can serve as the FIRST sample of
 * the thread's next read of the same page (slot VALID and not BUSY): see opt_memo_t. */
BAM_DEV bool opt_validate(const page_cache_d_t& pc, uint64_t tag, const opt_probe_t& pr, uint32_t dep, bool* still_valid = nullptr)
{
    const uint4 rec = ld_relaxed_gpu_v4(&pc.slots[dep ? 0u : pr.slot]);
    const bool ok = ((((uint64_t)rec.y) << 32) | rec.x) == tag && rec.w == pr.gen;
    if (still_valid) *still_valid = ok && (rec.z & (BAM_VALID | BAM_BUSY)) == BAM_VALID;
    return ok;
}

/* A thread's last translation: the validating sample of one read is a valid first sample for the next
 * read of the same page, so runs of accesses to one page skip the look-up (bucket and slot record) and
 * go straight to the data load and its validation.  Costs four registers; holds no pin, so it never
 * needs releasing and a stale one only costs a failed validation. */
struct opt_memo_t {
    uint64_t tag = BAM_TAG_NONE;
    uint32_t slot = BAM_SLOT_NONE;
    uint32_t gen = 0;
};

BAM_DEV void count_hit(const page_cache_d_t& pc, uint32_t count) { red_add_relaxed(&pc.stats[get_smid() & (BAM_STAT_STRIPES - 1)].hits, (uint64_t)count); }
BAM_DEV void count_miss(const page_cache_d_t& pc, uint32_t count)
{
    bam_stat_stripe_t* s = &pc.stats[get_smid() & (BAM_STAT_STRIPES - 1)];
    red_add_relaxed(&s->misses, (uint64_t)count);
    red_add_relaxed(&s->read_ios, 1ull);
}

/* Pin the page `tag` for `count` lanes and return its slot; on a miss allocate a slot and read
 * backing page `backing_page` through queue pair `queue`.  Returns BAM_SLOT_ERR after an
 * error has been recorded.  Counterpart of range_d_t<T>::acquire_page (page_cache.h:1122-1224). */
BAM_DEV uint32_t cache_acquire(const page_cache_d_t& pc, uint64_t tag, uint32_t count,
                               uint64_t backing_page, uint32_t queue, bool write, uint32_t ctrl = BAM_ALL_CTRLS)
{
    bam_status_t* st = pc.status;
    const uint64_t h = pt_hash(tag);
    const uint32_t home = (uint32_t)h & pc.bucket_mask;
    const uint32_t fp = (uint32_t)(h >> 56);
    spin_t sp;
#pragma unroll 1
    for (;;) {
        const uint32_t s = pt_lookup(pc, tag, home, fp);
        if (s != BAM_SLOT_NONE) {
            bam_slot_t* sl = &pc.slots[s];
            uint32_t old = atom_add_acquire(&sl->state, count);
            for (;;) {
                if (ld_relaxed_gpu(&sl->tag) != tag) break;                 /* recycled under us */
                if ((old & (BAM_VALID | BAM_BUSY)) == BAM_VALID) {
                    if (write && !(old & BAM_DIRTY)) atom_or_relaxed(&sl->state, BAM_DIRTY);
                    count_hit(pc, count);
                    return s;
                }
                if ((old & (BAM_VALID | BAM_BUSY)) == 0u) break;           /* slot was given back */
                if (sp.expired(st, BAM_AT_PAGE_BUSY, tag)) { red_add_relaxed(&sl->state, 0u - count); return BAM_SLOT_ERR; }
                old = ld_acquire_gpu(&sl->state);
            }
            red_add_relaxed(&sl->state, 0u - count);
            if (sp.expired(st, BAM_AT_PAGE_BUSY, tag)) return BAM_SLOT_ERR;
            continue;
        }
        /* miss: claim a slot (a dirty victim is written back first), publish the mapping, fill the slot */
        uint64_t victim_tag = BAM_TAG_NONE;
        const uint32_t v = find_slot(pc, 0xffffffffu, &victim_tag);
        if (v == BAM_SLOT_ERR) return BAM_SLOT_ERR;
        if (victim_tag != BAM_TAG_NONE) {
            uint32_t wctrl = 0;
            const uint64_t wlba = backing_location_of_tag(pc, victim_tag, wctrl) * pc.n_blocks_per_page;
            for (uint32_t k = 0; k < pc.n_ctrls; k++) {
                if (wctrl != BAM_ALL_CTRLS && wctrl != k) continue;
                if (access_data_raw(pick_queue(pc, k, queue), wlba, pc.n_blocks_per_page, slot_bus_addr(pc, v), slot_prp2(pc, v),
                                    NVM_IO_WRITE) != BAM_OK) return BAM_SLOT_ERR;
            }
            finish_evict(pc, v, victim_tag);
        }
        bam_slot_t* sl = &pc.slots[v];
        st_relaxed_gpu(&sl->tag, tag);
        __threadfence();
        const int r = pt_insert(pc, tag, v, home, fp);
        if (r != BAM_PT_OK) {
            st_relaxed_gpu(&sl->tag, BAM_TAG_NONE);
            atom_and_release(&sl->state, ~BAM_BUSY);                        /* give the slot back */
            if (r == BAM_PT_EXISTS) continue;                               /* someone else is filling it */
            if (r == BAM_PT_FULL) status_fail(st, BAM_ENOSPC, BAM_AT_TABLE_FULL, tag);
            return BAM_SLOT_ERR;
        }
        QueuePair* qp = pick_queue(pc, ctrl, queue);
        const uint64_t bus = slot_bus_addr(pc, v);
        const uint64_t mps = 4096;
        uint64_t prp2 = 0;
        if (pc.page_size > mps) prp2 = (pc.page_size <= 2 * mps) ? bus + mps : (uint64_t)(pc.prp_lists + (size_t)v * pc.prp_list_stride);
        const int rc = access_data_raw(qp, backing_page * pc.n_blocks_per_page, pc.n_blocks_per_page, bus, prp2, NVM_IO_READ);
        if (rc != BAM_OK) return BAM_SLOT_ERR;
        count_miss(pc, count);
        atom_add_relaxed(&sl->state, count + (write ? BAM_DIRTY : 0u));
        atom_xor_release(&sl->state, BAM_VALID | BAM_BUSY);                 /* BUSY -> VALID */
        return v;
    }
}

/* Warp-cooperative form of cache_acquire: all lanes of `mask` call it together; lanes with
 * want == true pin their page.  Look-ups and slot claims run per lane without sleeping; the page
 * reads of all missing lanes are then submitted and awaited as one group (warp_io), and lanes
 * that found their page being filled by another warp poll for it in a converged loop, so the
 * warp backs off once for everybody instead of once per lane.  Returns the slot, BAM_SLOT_ERR on
 * failure or when want == false, or BAM_SLOT_RETRY when no slot could be claimed in a bounded
 * sweep: the caller must first release the pages its warp holds (they may be exactly what keeps
 * the cache full) and then call again. */
BAM_DEV uint32_t warp_cache_acquire(uint32_t mask, bool want, const page_cache_d_t& pc, uint64_t tag, uint32_t count,
                                    uint64_t backing_page, uint32_t queue, bool write, uint32_t ctrl = BAM_ALL_CTRLS)
{
    enum { S_DONE = 0, S_LOOKUP = 1, S_WAIT = 2, S_IO = 3, S_WB = 4 };
    uint64_t victim_tag = BAM_TAG_NONE;
    const uint32_t kClaimTries = 64;                     /* clock-sweep probes before giving the turn back */
    bam_status_t* st = pc.status;
    const uint64_t h = pt_hash(tag);
    const uint32_t home = (uint32_t)h & pc.bucket_mask;
    const uint32_t fp = (uint32_t)(h >> 56);
    QueuePair* qp = pick_queue(pc, ctrl, queue);
    uint32_t state = want ? S_LOOKUP : S_DONE;
    uint32_t slot = BAM_SLOT_ERR;
    uint32_t my_hits = 0;                    /* hit counts are summed over the warp: one atomic, not 32 */
    spin_t sp;
#pragma unroll 1
    for (;;) {
        if (state == S_LOOKUP) {
            const uint32_t s = pt_lookup(pc, tag, home, fp);
            if (s != BAM_SLOT_NONE) {
                bam_slot_t* sl = &pc.slots[s];
                const uint32_t old = atom_add_acquire(&sl->state, count);
                if (ld_relaxed_gpu(&sl->tag) != tag || (old & (BAM_VALID | BAM_BUSY)) == 0u) {
                    red_add_relaxed(&sl->state, 0u - count);                   /* recycled or given back */
                } else if ((old & (BAM_VALID | BAM_BUSY)) == BAM_VALID) {
                    if (write && !(old & BAM_DIRTY)) atom_or_relaxed(&sl->state, BAM_DIRTY);
                    my_hits += count;
                    slot = s; state = S_DONE;
                } else {
                    slot = s; state = S_WAIT;                                  /* someone is filling it  */
                }
            } else {
                const uint32_t v = find_slot(pc, kClaimTries, &victim_tag);
                if (v == BAM_SLOT_ERR) { state = S_DONE; }
                else if (v <= BAM_SLOT_MAX && victim_tag != BAM_TAG_NONE) { slot = v; state = S_WB; }
                else if (v == BAM_SLOT_NONE) {
                    /* everything the sweep saw is pinned or busy.  The warp-mates that did get a
                     * slot must not wait for this lane while it waits for slots they hold pinned:
                     * report RETRY, the caller releases its pages and asks again. */
                    slot = BAM_SLOT_RETRY; state = S_DONE;
                } else {
                    bam_slot_t* sl = &pc.slots[v];
                    st_relaxed_gpu(&sl->tag, tag);
                    __threadfence();
                    const int r = pt_insert(pc, tag, v, home, fp);
                    if (r == BAM_PT_OK) { slot = v; state = S_IO; }
                    else {
                        st_relaxed_gpu(&sl->tag, BAM_TAG_NONE);
                        atom_and_release(&sl->state, ~BAM_BUSY);                /* give the slot back     */
                        BAM_PROF_ADD(st, 10, 1);
                        if (r != BAM_PT_EXISTS) {
                            if (r == BAM_PT_FULL) status_fail(st, BAM_ENOSPC, BAM_AT_TABLE_FULL, tag);
                            state = S_DONE;
                        }
                    }
                }
            }
        }
        /* dirty victims are written back as one group; then their slots are free for the new pages */
        if (__any_sync(mask, state == S_WB)) {
            const bool wb = state == S_WB;
            const int rc = warp_write_back(mask, wb, pc, victim_tag, slot);
            if (wb) {
                if (rc == BAM_OK) {
                    finish_evict(pc, slot, victim_tag);
                    bam_slot_t* sl = &pc.slots[slot];
                    st_relaxed_gpu(&sl->tag, tag);
                    __threadfence();
                    const int r = pt_insert(pc, tag, slot, home, fp);
                    if (r == BAM_PT_OK) state = S_IO;
                    else {
                        st_relaxed_gpu(&sl->tag, BAM_TAG_NONE);
                        atom_and_release(&sl->state, ~BAM_BUSY);
                        slot = BAM_SLOT_ERR;
                        if (r == BAM_PT_EXISTS) state = S_LOOKUP;
                        else { if (r == BAM_PT_FULL) status_fail(st, BAM_ENOSPC, BAM_AT_TABLE_FULL, tag); state = S_DONE; }
                    }
                } else { slot = BAM_SLOT_ERR; state = S_DONE; }
                victim_tag = BAM_TAG_NONE;
            }
        }
        /* all page reads of this round go out as one group */
        const bool io = state == S_IO;
        if (__any_sync(mask, io)) {
            const uint64_t bus = io ? slot_bus_addr(pc, slot) : 0;
            const uint64_t prp2 = io ? slot_prp2(pc, slot) : 0;
            const int rc = warp_io(mask, io, qp, backing_page * pc.n_blocks_per_page, pc.n_blocks_per_page, bus, prp2, NVM_IO_READ);
            if (io) {
                if (rc == BAM_OK) {
                    bam_slot_t* sl = &pc.slots[slot];
                    count_miss(pc, count);
                    atom_add_relaxed(&sl->state, count + (write ? BAM_DIRTY : 0u));
                    atom_xor_release(&sl->state, BAM_VALID | BAM_BUSY);         /* BUSY -> VALID          */
                } else slot = BAM_SLOT_ERR;
                state = S_DONE;
            }
        }
        if (state == S_WAIT) {
            bam_slot_t* sl = &pc.slots[slot];
            const uint32_t cur = ld_acquire_gpu(&sl->state);
            if (ld_relaxed_gpu(&sl->tag) != tag || (cur & (BAM_VALID | BAM_BUSY)) == 0u) {
                red_add_relaxed(&sl->state, 0u - count);
                slot = BAM_SLOT_ERR; state = S_LOOKUP;
            } else if ((cur & (BAM_VALID | BAM_BUSY)) == BAM_VALID) {
                if (write && !(cur & BAM_DIRTY)) atom_or_relaxed(&sl->state, BAM_DIRTY);
                my_hits += count;
                state = S_DONE;
            }
        }
        if (!__any_sync(mask, state != S_DONE)) break;
        if (__any_sync(mask, sp.expired(st, BAM_AT_PAGE_BUSY, tag))) {
            if (state == S_WAIT) red_add_relaxed(&pc.slots[slot].state, 0u - count);
            if (state != S_DONE) slot = BAM_SLOT_ERR;
            break;
        }
    }
    const uint32_t warp_hits = __reduce_add_sync(mask, my_hits);
    if (warp_hits && lane_id() == (uint32_t)(__ffs(mask) - 1)) count_hit(pc, warp_hits);
    return slot;
}

BAM_DEV void cache_release(const page_cache_d_t& pc, uint32_t slot, uint32_t count)
{
    red_add_release(&pc.slots[slot].state, 0u - count);
}

}  // namespace bam
#endif
