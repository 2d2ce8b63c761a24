/*
 * bam/sync.cuh -- memory-model primitives and bounded waits for sm_100a device code.
 *
 * The reference synchronises through simt::atomic (libcu++'s predecessor) at device scope and
 * writes doorbells with st.mmio.relaxed.sys (include/nvm_parallel_queue.h:303,481).  Here every
 * cross-thread word is accessed through the explicit PTX below: .gpu scope between threads of
 * one GPU, .sys scope for anything the controller side reads or writes (doorbells, completion
 * entries), so the same device code is correct whether the controller is a set of warps on
 * this GPU or another agent in the system.
 *
 * Every wait in the library goes through bam::spin_t: it backs off with __nanosleep, polls the
 * shared status word, and gives up after bam_status_t::spin_timeout_ns, recording where.  No
 * wait is unbounded (the reference's are: nvm_parallel_queue.h:188,204,287,384; page_cache.h
 * :1133-1222, :1796-1924).
 */
#ifndef BAM_SYNC_CUH
#define BAM_SYNC_CUH

#include <stdint.h>
#include "abi_types.h"

namespace bam {

#define BAM_DEV __device__ __forceinline__
#define BAM_DEV_NOINLINE __device__ __noinline__

/* ---- loads / stores ------------------------------------------------------------------- */
BAM_DEV uint32_t ld_relaxed_gpu(const uint32_t* p) { uint32_t v; asm volatile("ld.relaxed.gpu.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v; }
BAM_DEV uint32_t ld_acquire_gpu(const uint32_t* p) { uint32_t v; asm volatile("ld.acquire.gpu.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v; }
BAM_DEV uint64_t ld_relaxed_gpu(const uint64_t* p) { uint64_t v; asm volatile("ld.relaxed.gpu.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory"); return v; }
BAM_DEV uint64_t ld_acquire_gpu(const uint64_t* p) { uint64_t v; asm volatile("ld.acquire.gpu.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory"); return v; }
BAM_DEV uint32_t ld_relaxed_sys(const uint32_t* p) { uint32_t v; asm volatile("ld.relaxed.sys.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v; }
BAM_DEV uint32_t ld_acquire_sys(const uint32_t* p) { uint32_t v; asm volatile("ld.acquire.sys.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v; }
BAM_DEV uint64_t ld_relaxed_sys(const uint64_t* p) { uint64_t v; asm volatile("ld.relaxed.sys.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory"); return v; }

BAM_DEV void st_relaxed_gpu(uint32_t* p, uint32_t v) { asm volatile("st.relaxed.gpu.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
BAM_DEV void st_release_gpu(uint32_t* p, uint32_t v) { asm volatile("st.release.gpu.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
BAM_DEV void st_relaxed_gpu(uint64_t* p, uint64_t v) { asm volatile("st.relaxed.gpu.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory"); }
BAM_DEV void st_release_gpu(uint64_t* p, uint64_t v) { asm volatile("st.release.gpu.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory"); }
BAM_DEV void st_release_sys(uint32_t* p, uint32_t v) { asm volatile("st.release.sys.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
BAM_DEV void st_release_sys(uint64_t* p, uint64_t v) { asm volatile("st.release.sys.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory"); }

BAM_DEV uint4 ld_relaxed_gpu_v4(const void* p) { uint4 v; asm volatile("ld.relaxed.gpu.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory"); return v; }

/* A strong (L2-coherent) load of one element: the data loads of readers that hold no pin. */
template <typename T>
BAM_DEV T ld_strong(const T* p)
{
    if constexpr (sizeof(T) == 8) { uint64_t v = ld_relaxed_gpu(reinterpret_cast<const uint64_t*>(p)); return *reinterpret_cast<T*>(&v); }
    else if constexpr (sizeof(T) == 4) { uint32_t v = ld_relaxed_gpu(reinterpret_cast<const uint32_t*>(p)); return *reinterpret_cast<T*>(&v); }
    else return *reinterpret_cast<const volatile T*>(p);
}

BAM_DEV void fence_acq_rel_gpu() { asm volatile("fence.acq_rel.gpu;" ::: "memory"); }
BAM_DEV void fence_acq_rel_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }

/* Scope chosen at run time.  Doorbells and completion entries are the words the NVMe controller
 * shares with the GPU threads.  When the controller is another agent of the system (a device on
 * the bus, host threads) they need system scope.  When it is the emulated controller running in
 * the same launch on the same GPU, device scope already contains every thread involved, and it is
 * much cheaper: a system-scope fence has to wait behind the host-link traffic. */
BAM_DEV void st_release_scoped(uint32_t* p, uint32_t v, bool sys) { if (sys) st_release_sys(p, v); else st_release_gpu(p, v); }
BAM_DEV void st_release_scoped(uint64_t* p, uint64_t v, bool sys) { if (sys) st_release_sys(p, v); else st_release_gpu(p, v); }
BAM_DEV void fence_acq_rel_scoped(bool sys) { if (sys) fence_acq_rel_sys(); else fence_acq_rel_gpu(); }

/* ---- read-modify-write ------------------------------------------------------------------ */
BAM_DEV uint32_t atom_add_relaxed(uint32_t* p, uint32_t v) { uint32_t o; asm volatile("atom.relaxed.gpu.add.u32 %0, [%1], %2;" : "=r"(o) : "l"(p), "r"(v) : "memory"); return o; }
BAM_DEV uint32_t atom_add_acquire(uint32_t* p, uint32_t v) { uint32_t o; asm volatile("atom.acquire.gpu.add.u32 %0, [%1], %2;" : "=r"(o) : "l"(p), "r"(v) : "memory"); return o; }
BAM_DEV uint32_t atom_add_acq_rel(uint32_t* p, uint32_t v) { uint32_t o; asm volatile("atom.acq_rel.gpu.add.u32 %0, [%1], %2;" : "=r"(o) : "l"(p), "r"(v) : "memory"); return o; }
BAM_DEV void red_add_release(uint32_t* p, uint32_t v) { asm volatile("red.release.gpu.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
BAM_DEV void red_add_relaxed(uint32_t* p, uint32_t v) { asm volatile("red.relaxed.gpu.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
BAM_DEV void red_add_relaxed(uint64_t* p, uint64_t v) { asm volatile("red.relaxed.gpu.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory"); }
BAM_DEV uint64_t atom_add_relaxed(uint64_t* p, uint64_t v) { uint64_t o; asm volatile("atom.relaxed.gpu.add.u64 %0, [%1], %2;" : "=l"(o) : "l"(p), "l"(v) : "memory"); return o; }
BAM_DEV uint32_t atom_or_acquire(uint32_t* p, uint32_t v) { uint32_t o; asm volatile("atom.acquire.gpu.or.b32 %0, [%1], %2;" : "=r"(o) : "l"(p), "r"(v) : "memory"); return o; }
BAM_DEV uint32_t atom_or_relaxed(uint32_t* p, uint32_t v) { uint32_t o; asm volatile("atom.relaxed.gpu.or.b32 %0, [%1], %2;" : "=r"(o) : "l"(p), "r"(v) : "memory"); return o; }
BAM_DEV uint32_t atom_and_release(uint32_t* p, uint32_t v) { uint32_t o; asm volatile("atom.release.gpu.and.b32 %0, [%1], %2;" : "=r"(o) : "l"(p), "r"(v) : "memory"); return o; }
BAM_DEV uint32_t atom_xor_release(uint32_t* p, uint32_t v) { uint32_t o; asm volatile("atom.release.gpu.xor.b32 %0, [%1], %2;" : "=r"(o) : "l"(p), "r"(v) : "memory"); return o; }
BAM_DEV uint32_t atom_cas_acquire(uint32_t* p, uint32_t cmp, uint32_t v) { uint32_t o; asm volatile("atom.acquire.gpu.cas.b32 %0, [%1], %2, %3;" : "=r"(o) : "l"(p), "r"(cmp), "r"(v) : "memory"); return o; }
BAM_DEV uint32_t atom_cas_relaxed(uint32_t* p, uint32_t cmp, uint32_t v) { uint32_t o; asm volatile("atom.relaxed.gpu.cas.b32 %0, [%1], %2, %3;" : "=r"(o) : "l"(p), "r"(cmp), "r"(v) : "memory"); return o; }
BAM_DEV uint32_t atom_exch_acq_rel(uint32_t* p, uint32_t v) { uint32_t o; asm volatile("atom.acq_rel.gpu.exch.b32 %0, [%1], %2;" : "=r"(o) : "l"(p), "r"(v) : "memory"); return o; }
BAM_DEV uint64_t atom_min_relaxed(uint64_t* p, uint64_t v) { uint64_t o; asm volatile("atom.relaxed.gpu.min.u64 %0, [%1], %2;" : "=l"(o) : "l"(p), "l"(v) : "memory"); return o; }

/* 128-bit loads that bypass L1 (metadata other SMs rewrite) */
BAM_DEV uint4 ld_cg_v4(const void* p) { uint4 v; asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory"); return v; }

/* ---- identification ---------------------------------------------------------------------- */
BAM_DEV uint32_t lane_id() { uint32_t r; asm volatile("mov.u32 %0, %%laneid;" : "=r"(r)); return r; }
BAM_DEV uint32_t get_smid() { uint32_t r; asm volatile("mov.u32 %0, %%smid;" : "=r"(r)); return r; }
BAM_DEV uint64_t global_timer_ns() { uint64_t t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }

/* ---- optional profiling counters (compiled out unless -DBAM_PROFILE) ---------------------------- */
#ifdef BAM_PROFILE
#define BAM_PROF_T0() const long long bam_prof_t0_ = clock64()
#define BAM_PROF_ADD(st, idx, v) red_add_relaxed(&(st)->prof[idx], (uint64_t)(v))
#define BAM_PROF_LAP(st, idx) red_add_relaxed(&(st)->prof[idx], (uint64_t)(clock64() - bam_prof_t0_))
#else
#define BAM_PROF_T0() do {} while (0)
#define BAM_PROF_ADD(st, idx, v) do {} while (0)
#define BAM_PROF_LAP(st, idx) do {} while (0)
#endif

/* ---- status + bounded wait ---------------------------------------------------------------- */
BAM_DEV bool status_bad(const bam_status_t* st) { return ld_relaxed_gpu(&st->code) != 0; }

BAM_DEV void status_fail(bam_status_t* st, uint32_t code, uint32_t where, uint64_t detail)
{
    if (atom_cas_relaxed(&st->code, 0u, code) == 0u) {
        st->where = where;
        st->detail = detail;
        __threadfence();
    }
}

struct spin_t {
    uint32_t ns = 8;
    uint32_t iters = 0;
    uint64_t deadline = 0;

    BAM_DEV void reset() { ns = 8; iters = 0; deadline = 0; }

    /* One back-off step.  Returns true when the caller must stop waiting: either another
     * thread has flagged an error or this wait has outlived the limit (then the time-out is
     * recorded with `where`). */
    BAM_DEV bool expired(bam_status_t* st, uint32_t where, uint64_t detail = 0)
    {
        __nanosleep(ns);
        if (ns < 512) ns <<= 1;
        if (((++iters) & 15u) == 0u) {
            if (status_bad(st)) return true;
            uint64_t now = global_timer_ns();
            if (deadline == 0) deadline = now + st->spin_timeout_ns;
            else if (now > deadline) { status_fail(st, BAM_ETIMEDOUT, where, detail); return true; }
        }
        return false;
    }
};

}  // namespace bam
#endif
