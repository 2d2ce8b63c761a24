/*
 * bam/tlb.cuh -- a block-level translation buffer in front of the page cache, and the cursor that
 * reads through it (reference: tlb_entry / tlb / bam_ptr_tlb, include/page_cache.h:158-411).
 *
 * A tlb<T, N> is a direct-mapped table of N entries, one per thread block, normally in shared
 * memory.  Entry gid % N remembers which cache slot holds page gid and keeps that page pinned ONCE
 * in the cache on behalf of the whole block; threads that use the page count themselves in the
 * entry's own user count.  A translation that hits costs three shared-memory atomics instead of a
 * hashed look-up and two global atomics.
 *
 * What differs from the reference:
 *  - nobody ever waits for an entry.  The reference holds the entry's lock across the page read
 *    and lets a thread that finds its entry in use by another page spin until the other users
 *    leave (page_cache.h:257-309); users that sit in the same warp, or that the waiter must meet
 *    at a barrier, never leave.  Here the entry lock covers a few loads and stores only, it is
 *    taken with try-lock rounds in which the whole warp stays converged, the page read happens with
 *    no lock held, and a thread whose entry is occupied by another page in use simply keeps the
 *    cache pin it already has ("direct" mode) instead of going through the buffer.
 *  - the warp takes part as a whole (all active lanes call acquire together), like every other
 *    access path of this library.
 *
 * Pin budget: a block keeps up to N pages pinned in its buffer plus one per thread in direct mode,
 * so the cache needs more slots than blocks * N + threads holding a cursor.
 */
#ifndef BAM_TLB_CUH
#define BAM_TLB_CUH

#include "array.cuh"

namespace bam {

#define BAM_TLB_LOCK 0x80000000u
#define BAM_TLB_CNT_MASK 0x7fffffffu
#define BAM_TLB_LOCK_ROUNDS 64         /* try-lock rounds before a lane gives up on its entry */

template <typename T, uint32_t N = 32>
struct tlb {
    struct entry_t {
        uint64_t gid;          /* global address (tag) of the page the entry translates */
        uint32_t state;        /* BAM_TLB_LOCK | users inside this block                */
        uint32_t slot;         /* cache slot of the page, BAM_SLOT_ERR when empty       */
    };
    entry_t entries[N];
    const array_d_t<T>* array;

    /* Every thread of the block calls init before the first access and fini after the last one
     * (both contain a block barrier). */
    BAM_DEV void init(const array_d_t<T>* a)
    {
        for (uint32_t i = threadIdx.x; i < N; i += blockDim.x) {
            entries[i].gid = ~0ull;
            entries[i].state = 0u;
            entries[i].slot = BAM_SLOT_ERR;
        }
        if (threadIdx.x == 0) array = a;
        __syncthreads();
    }

    BAM_DEV void fini()
    {
        __syncthreads();
        for (uint32_t i = threadIdx.x; i < N; i += blockDim.x) {
            const uint32_t s = entries[i].slot;
            if (s <= BAM_SLOT_MAX) cache_release(array->d_ranges[0].cache, s, 1);
            entries[i].slot = BAM_SLOT_ERR;
            entries[i].gid = ~0ull;
            entries[i].state = 0u;
        }
        __syncthreads();
    }

    BAM_DEV entry_t* entry_of(uint64_t gid) { return &entries[gid % N]; }

    /* One try-lock round.  Returns true when the lock was taken. */
    BAM_DEV static bool try_lock(entry_t* e)
    {
        if (atomicOr(&e->state, BAM_TLB_LOCK) & BAM_TLB_LOCK) return false;
        __threadfence_block();
        return true;
    }
    BAM_DEV static void unlock(entry_t* e)
    {
        __threadfence_block();
        atomicAnd(&e->state, ~BAM_TLB_LOCK);
    }

    /* Translate page `page` of range r (global address gid) for the calling warp: all lanes of
     * `mask` call together, lanes with valid == false only take part in the votes.  Returns the
     * cache slot (BAM_SLOT_ERR on failure); via_tlb tells how the lane has to release it. */
    BAM_DEV uint32_t acquire(uint32_t mask, bool valid, const range_d_t<T>& r, uint64_t page, uint64_t gid, bool& via_tlb)
    {
        const uint32_t lane = lane_id();
        const uint32_t eq = __match_any_sync(mask, valid ? gid : ~0ull);
        const uint32_t leader = __ffs(eq) - 1;
        const uint32_t cnt = __popc(eq);
        const bool lead = valid && lane == leader;
        entry_t* e = entry_of(valid ? gid : 0);
        uint32_t slot = BAM_SLOT_ERR;
        bool via = false;

        /* 1. look-up: one leader per distinct page; the warp stays converged over the rounds */
        bool pending = lead;
#pragma unroll 1
        for (uint32_t round = 0; round < BAM_TLB_LOCK_ROUNDS && __any_sync(mask, pending); round++) {
            if (pending && try_lock(e)) {
                const uint32_t s = *(volatile uint32_t*)&e->slot;
                if (s <= BAM_SLOT_MAX && *(volatile uint64_t*)&e->gid == gid) {
                    atomicAdd(&e->state, cnt);
                    slot = s;
                    via = true;
                }
                unlock(e);
                pending = false;
            }
        }
        /* 2. pages not in the buffer are pinned through the cache, all of them in one call */
        const bool miss = lead && !via;
        const uint32_t fresh = range_pin_page(r, mask, miss, page, cnt, default_queue());
        if (miss) slot = fresh;
        /* 3. offer the new translation to the buffer */
        pending = miss && slot <= BAM_SLOT_MAX;
        uint32_t give_back = 0, old_slot = BAM_SLOT_ERR;
#pragma unroll 1
        for (uint32_t round = 0; round < BAM_TLB_LOCK_ROUNDS && __any_sync(mask, pending); round++) {
            if (pending && try_lock(e)) {
                const uint32_t s = *(volatile uint32_t*)&e->slot;
                const uint32_t users = *(volatile uint32_t*)&e->state & BAM_TLB_CNT_MASK;
                if (s <= BAM_SLOT_MAX && *(volatile uint64_t*)&e->gid == gid) {
                    /* another warp of the block installed the same page meanwhile: join it */
                    atomicAdd(&e->state, cnt);
                    give_back = cnt;
                    via = true;
                } else if (s > BAM_SLOT_MAX || users == 0u) {
                    /* empty, or translating a page nobody in the block uses any more: replace it.
                     * The entry keeps one of this group's pins, the rest go back. */
                    old_slot = s;
                    *(volatile uint64_t*)&e->gid = gid;
                    *(volatile uint32_t*)&e->slot = slot;
                    atomicAdd(&e->state, cnt);
                    give_back = cnt - 1;
                    via = true;
                }                                          /* else: in use by another page, stay direct */
                unlock(e);
                pending = false;
            }
        }
        if (give_back) r.release_page(slot, give_back);
        if (old_slot <= BAM_SLOT_MAX) r.release_page(old_slot, 1);
        slot = __shfl_sync(eq, slot, leader);
        via_tlb = __shfl_sync(eq, (int)via, leader) != 0;
        return slot;
    }

    /* Give a translation back: lanes of the calling warp that hold the same page in the same way
     * are counted together.  All lanes of `mask` call; lanes with held == false only vote. */
    BAM_DEV void release(uint32_t mask, bool held, const range_d_t<T>& r, uint64_t gid, uint32_t slot, bool via_tlb)
    {
        const uint64_t key = held ? ((gid << 1) | (via_tlb ? 1u : 0u)) : ~0ull;
        const uint32_t eq = __match_any_sync(mask, key);
        if (!held || lane_id() != (uint32_t)(__ffs(eq) - 1)) return;
        if (via_tlb) {
            __threadfence_block();
            atomicSub(&entry_of(gid)->state, (uint32_t)__popc(eq));
        } else
            r.release_page(slot, __popc(eq));
    }
};

/* Cursor over an array that translates through a block's tlb (reference: bam_ptr_tlb,
 * page_cache.h:337-411).  Reading p[i] gives the element; assigning to p[i] writes it and marks
 * the page dirty (the reference marks the page dirty on every non-const access, :399-406; here
 * only a real write does). */
template <typename T, uint32_t N = 32>
struct bam_ptr_tlb {
    tlb<T, N>* tlb_ = nullptr;
    const array_d_t<T>* array = nullptr;
    const range_d_t<T>* range = nullptr;
    uint64_t gid = 0;
    uint32_t slot = BAM_SLOT_ERR;
    bool via_tlb = false, dirty = false;
    size_t start = 0, end = 0;
    T* addr = nullptr;

    struct ref_t {
        bam_ptr_tlb* p;
        size_t i;
        BAM_DEV operator T() const { return p->read(i); }
        BAM_DEV ref_t& operator=(const T v) { p->write(i, v); return *this; }
        BAM_DEV ref_t& operator=(const ref_t& o) { p->write(i, (T)o); return *this; }
    };

    BAM_DEV bam_ptr_tlb(const array_d_t<T>* a, tlb<T, N>* t) : tlb_(t), array(a) {}
    BAM_DEV ~bam_ptr_tlb() { fini(); }

    /* All lanes of the warp that are still active call fini together (the destructor does). */
    BAM_DEV void fini()
    {
        const uint32_t mask = __activemask();
        const bool held = slot != BAM_SLOT_ERR;
        if (__any_sync(mask, held)) tlb_->release(mask, held, *range_or_first(), gid, slot, via_tlb);
        slot = BAM_SLOT_ERR;
        start = end = 0;
        addr = nullptr;
        dirty = false;
    }

    BAM_DEV const range_d_t<T>* range_or_first() const { return range ? range : &array->d_ranges[0]; }

    BAM_DEV T* update_page(size_t i)
    {
        fini();
        const uint32_t mask = __activemask();
        const int64_t ri = array->find_range(i);
        const bool valid = ri >= 0;
        range = &array->d_ranges[valid ? ri : 0];
        const uint64_t page = valid ? range->get_page(i) : 0;
        gid = valid ? range->get_global_address(page) : ~0ull;
        slot = tlb_->acquire(mask, valid, *range, page, gid, via_tlb);
        if (!valid) { status_fail(range->cache.status, BAM_ERANGE, BAM_AT_RANGE, i); slot = BAM_SLOT_ERR; }
        if (slot > BAM_SLOT_MAX) { slot = BAM_SLOT_ERR; addr = nullptr; return nullptr; }
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

    BAM_DEV ref_t operator[](size_t i) { return ref_t{ this, i }; }
};

}  // namespace bam
#endif
