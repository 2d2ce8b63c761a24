"""Host objects mirroring the reference's C++ wrappers over the C ABI.

  Controller  <- struct Controller, include/ctrl.h:39-199 (opens the SSD, creates queue pairs)
  PageCache   <- struct page_cache_t, include/page_cache.h:631-875
  Array       <- range_t<T> + array_t<T>, include/page_cache.h:978-1030, :1719-1772

Device buffers are passed as integer device addresses (e.g. torch.Tensor.data_ptr()).
"""
import ctypes as C
import os

from . import _lib
from ._lib import CacheStats, StatusOut, check

WHERE = {0: "none", 1: "cid", 2: "sq_turn", 3: "sq_doorbell", 4: "cq_wait", 5: "page_busy",
         6: "find_slot", 7: "bucket_lock", 8: "table_full", 9: "nvme_status", 10: "ctrl_cq_full",
         11: "range", 12: "tma", 13: "launch", 14: "sq_order"}

FAULT_NONE, FAULT_DROP_CPL, FAULT_STATUS = 0, 1, 2


def _ptr(x):
    """Accept None, an int device address, or an object with data_ptr()."""
    if x is None:
        return None
    if hasattr(x, "data_ptr"):
        return C.c_void_p(x.data_ptr())
    return C.c_void_p(int(x))


class Controller:
    """Emulated NVMe controller with a pinned host backing store and n I/O queue pairs.

    Same constructor shape as the reference's Controller(path, nvmNamespace, cudaDevice,
    queueDepth, numQueues); `path` is replaced by the size of the emulated namespace.
    """

    def __init__(self, store_bytes, cuda_device=0, queue_depth=1024, num_queues=128, lba_bytes=512,
                 nvm_namespace=1):
        self.lib = _lib.load()
        self.h = C.c_void_p()
        check(self.lib.bam_ctrl_create(C.byref(self.h), cuda_device, store_bytes, lba_bytes, num_queues,
                                       queue_depth), "bam_ctrl_create")
        self.store_bytes, self.device = store_bytes, cuda_device
        self.n_qps, self.queue_depth, self.lba_bytes = num_queues, queue_depth, lba_bytes
        self.ns = nvm_namespace

    def close(self):
        if self.h:
            self.lib.bam_ctrl_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def store_numpy(self, dtype="uint64"):
        """The backing store as a numpy array over the pinned host memory."""
        import numpy as np
        n = self.store_bytes // np.dtype(dtype).itemsize
        buf = (C.c_uint8 * self.store_bytes).from_address(self.lib.bam_ctrl_store_host(self.h))
        return np.frombuffer(buf, dtype=dtype, count=n)

    def fill_store(self, seed, first_elem=0, stream=None):
        check(self.lib.bam_ctrl_fill_store(self.h, seed, first_elem, _ptr(stream)), "bam_ctrl_fill_store")

    def fill_store_striped(self, seed, stripe, n_stripes, first_elem=0, page_bytes=4096, stream=None):
        """Fill this controller's share of a striped store: its page j gets logical page j * n_stripes + stripe."""
        check(self.lib.bam_ctrl_fill_store_striped(self.h, seed, first_elem, page_bytes, stripe, n_stripes, _ptr(stream)),
              "bam_ctrl_fill_store_striped")

    def configure(self, ctrl_blocks=0, batch=0, spin_timeout_ns=0):
        check(self.lib.bam_ctrl_configure(self.h, ctrl_blocks, batch, spin_timeout_ns), "bam_ctrl_configure")

    def set_launch_timeout(self, ns):
        check(self.lib.bam_ctrl_set_launch_timeout(self.h, ns), "bam_ctrl_set_launch_timeout")

    def set_scope(self, system_scope):
        check(self.lib.bam_ctrl_set_scope(self.h, int(system_scope)), "bam_ctrl_set_scope")

    def set_max_grid(self, max_grid):
        check(self.lib.bam_ctrl_set_max_grid(self.h, max_grid), "bam_ctrl_set_max_grid")

    def inject_fault(self, mode, nth=0, status=0):
        check(self.lib.bam_ctrl_inject_fault(self.h, mode, nth, status), "bam_ctrl_inject_fault")

    def status(self, clear=False):
        """Synchronise and return (code, where, detail) of the device status block."""
        st = StatusOut()
        check(self.lib.bam_ctrl_status(self.h, C.byref(st), int(clear)), "bam_ctrl_status")
        return st.code, WHERE.get(st.where, str(st.where)), st.detail

    def check_status(self):
        code, where, detail = self.status()
        if code:
            raise _lib.BamError(code, f"device status (at {where}, detail {detail})")

    def served(self, reset=False):
        v = C.c_uint64()
        check(self.lib.bam_ctrl_served(self.h, C.byref(v), int(reset)), "bam_ctrl_served")
        return v.value

    def profile(self, reset=True):
        """The 32 profiling counters (zeros unless the library was built with -DBAM_PROFILE)."""
        buf = (C.c_uint64 * 32)()
        check(self.lib.bam_ctrl_profile(self.h, buf, int(reset)), "bam_ctrl_profile")
        return list(buf)

    def reset_queues(self):
        check(self.lib.bam_ctrl_reset_queues(self.h), "bam_ctrl_reset_queues")

    def geometry(self):
        g, cb, t = C.c_uint32(), C.c_uint32(), C.c_uint32()
        check(self.lib.bam_launch_geometry(self.h, C.byref(g), C.byref(cb), C.byref(t)), "bam_launch_geometry")
        return g.value, cb.value, t.value


REPLICATE, STRIPE = 0, 1       # data_dist_t (include/page_cache.h:42 in the reference)


def backing_location(page, n_ctrls, dist, page_start=0):
    """(controller, backing page) of page `page` of a range: get_backing_ctrl_ / get_backing_page_
    (include/page_cache.h:558-582 in the reference).  controller is None when any will do."""
    if dist == STRIPE and n_ctrls > 1:
        return page % n_ctrls, page_start + page // n_ctrls
    return None, page_start + page


class PageCache:
    """page_cache_t(page_size, n_pages, gpu, ctrl, max_range, ctrls): `ctrl` is one Controller or
    the list of controllers the cache sits in front of."""

    def __init__(self, ctrl, page_size=4096, n_pages=65536):
        ctrls = list(ctrl) if isinstance(ctrl, (list, tuple)) else [ctrl]
        self.ctrls, self.ctrl = ctrls, ctrls[0]
        self.lib = self.ctrl.lib
        self.h = C.c_void_p()
        if len(ctrls) == 1:
            check(self.lib.bam_cache_create(C.byref(self.h), self.ctrl.h, page_size, n_pages), "bam_cache_create")
        else:
            hs = (C.c_void_p * len(ctrls))(*[c.h for c in ctrls])
            check(self.lib.bam_cache_create_multi(C.byref(self.h), hs, len(ctrls), page_size, n_pages),
                  "bam_cache_create_multi")
        self.page_size, self.n_pages = page_size, n_pages

    def close(self):
        if self.h:
            self.lib.bam_cache_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def stats(self, reset=False):
        s = CacheStats()
        check(self.lib.bam_cache_stats(self.h, C.byref(s), int(reset)), "bam_cache_stats")
        return {"hits": s.hits, "misses": s.misses, "read_ios": s.read_ios, "accesses": s.hits + s.misses}

    def invalidate(self):
        check(self.lib.bam_cache_invalidate(self.h), "bam_cache_invalidate")

    def invalidate_async(self, stream=None):
        check(self.lib.bam_cache_invalidate_async(self.h, _ptr(stream)), "bam_cache_invalidate_async")

    def audit(self):
        v = C.c_uint64()
        check(self.lib.bam_cache_audit(self.h, C.byref(v)), "bam_cache_audit")
        return v.value

    def flush(self, stream=None):
        """Write every dirty page back to the backing store (page_cache_t::flush_cache)."""
        check(self.lib.bam_cache_flush(self.h, _ptr(stream)), "bam_cache_flush")

    def audit_noalloc(self, violations_out, stream=None):
        """Enqueue the allocation-free audit; the count lands in the device u64 `violations_out`."""
        check(self.lib.bam_cache_audit_noalloc(self.h, _ptr(violations_out), _ptr(stream)), "bam_cache_audit_noalloc")

    def bulk_io(self, n_pages, first_store_page, first_slot=0, write=False, stream=None):
        """One NVMe command per cache page between the cache's memory and the store."""
        check(self.lib.bam_launch_bulk_io(self.h, n_pages, first_store_page, first_slot, int(write), _ptr(stream)),
              "bam_launch_bulk_io")

    def load_file(self, path, store_byte_offset=0, file_offset=0, n_bytes=None):
        """Copy a file onto the store through the cache's memory and NVMe WRITE commands, a cache-full at a
        time (the loader of benchmarks/readwrite/main.cu:283-316).  Returns the bytes written; the last
        page is padded with zeros.  Leaves the cache invalidated."""
        import numpy as np
        import torch
        ps = self.page_size
        assert store_byte_offset % ps == 0
        size = os.path.getsize(path) - file_offset if n_bytes is None else n_bytes
        self.invalidate()
        chunk_pages = self.n_pages
        staging = torch.empty(chunk_pages * ps, dtype=torch.uint8).pin_memory()
        done = 0
        with open(path, "rb") as f:
            f.seek(file_offset)
            while done < size:
                n = min(chunk_pages * ps, size - done)
                buf = staging.numpy()
                got = f.readinto(memoryview(buf)[:n])
                assert got == n, "short read"
                pages = (n + ps - 1) // ps
                buf[n:pages * ps] = 0
                check(self.lib.bam_cache_copy(self.h, 0, staging.data_ptr(), pages * ps, 1, None), "bam_cache_copy")
                self.bulk_io(pages, (store_byte_offset + done) // ps, 0, write=True)
                torch.cuda.synchronize()
                self.ctrl.check_status()
                done += n
        self.invalidate()
        return size

    def dump_file(self, path, n_bytes, store_byte_offset=0):
        """The way back: NVMe READ commands into the cache's memory, then out to a file."""
        import torch
        ps = self.page_size
        assert store_byte_offset % ps == 0
        self.invalidate()
        chunk_pages = self.n_pages
        staging = torch.empty(chunk_pages * ps, dtype=torch.uint8).pin_memory()
        done = 0
        with open(path, "wb") as f:
            while done < n_bytes:
                n = min(chunk_pages * ps, n_bytes - done)
                pages = (n + ps - 1) // ps
                self.bulk_io(pages, (store_byte_offset + done) // ps, 0, write=False)
                check(self.lib.bam_cache_copy(self.h, 0, staging.data_ptr(), pages * ps, 0, None), "bam_cache_copy")
                torch.cuda.synchronize()
                self.ctrl.check_status()
                f.write(memoryview(staging.numpy())[:n])
                done += n
        self.invalidate()
        return n_bytes

    def block_read(self, n_reqs, pages=None, req_seed=0, crc_out=None, sum_out=None, stream=None, io_depth=1):
        check(self.lib.bam_launch_block_read_depth(self.h, n_reqs, _ptr(pages), req_seed, io_depth, _ptr(crc_out),
                                                   _ptr(sum_out), _ptr(stream)), "bam_launch_block_read_depth")


class Array:
    """array_t<T>(n_elems, disk_start_offset, {range_t<T>(...)}) for a single range."""

    def __init__(self, cache, n_elems, elem_bytes=8, store_byte_offset=0, dist=REPLICATE):
        self.lib, self.cache = cache.lib, cache
        self.h = C.c_void_p()
        check(self.lib.bam_array_create_dist(C.byref(self.h), cache.h, n_elems, elem_bytes, store_byte_offset, dist),
              "bam_array_create_dist")
        self.n_elems, self.elem_bytes, self.dist = n_elems, elem_bytes, dist

    @classmethod
    def from_ranges(cls, cache, n_elems, ranges, elem_bytes=8):
        """array_t over several range_t: `ranges` is a list of (index_start, index_end, store_byte_offset,
        page_start_offset, dist) -- element index_start of a range lives page_start_offset bytes into the
        backing page at store_byte_offset."""
        a = cls.__new__(cls)
        a.lib, a.cache, a.h = cache.lib, cache, C.c_void_p()
        descs = (_lib.RangeDesc * len(ranges))(*[_lib.RangeDesc(r[0], r[1], r[2], r[3] if len(r) > 3 else 0,
                                                                r[4] if len(r) > 4 else REPLICATE, 0) for r in ranges])
        check(a.lib.bam_array_create_ranges(C.byref(a.h), cache.h, n_elems, elem_bytes, descs, len(ranges)),
              "bam_array_create_ranges")
        a.n_elems, a.elem_bytes, a.dist = n_elems, elem_bytes, None
        return a

    def close(self):
        if self.h:
            self.lib.bam_array_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def d_array_ptr(self):
        return self.lib.bam_array_device_ptr(self.h)

    def read(self, n_lanes, reqs_per_lane, sum_out, idx=None, access_seed=0, stream=None):
        check(self.lib.bam_launch_array_read(self.h, n_lanes, reqs_per_lane, _ptr(idx), access_seed, _ptr(sum_out),
                                             _ptr(stream)), "bam_launch_array_read")

    def write(self, n, idx, val_seed=0, addend=0, stream=None):
        """a[idx[k]] = splitmix64(val_seed ^ idx[k]) (addend == 0) or a[idx[k]] += addend, through the cache."""
        check(self.lib.bam_launch_array_write(self.h, n, _ptr(idx), val_seed, addend, _ptr(stream)), "bam_launch_array_write")

    def thread_acquire(self, first_page, n_pages, first_words, lanes=0x80081, stream=None):
        """The per-thread protocol: the lanes of every warp named by the bit mask `lanes` (default: lanes 0, 7
        and 19) each pin page first_page + k on their own, store its first element in first_words[k] and unpin it."""
        check(self.lib.bam_launch_thread_acquire(self.h, first_page, n_pages, lanes, _ptr(first_words), _ptr(stream)),
              "bam_launch_thread_acquire")

    def pattern_read(self, pattern, n_elems, sum_out, n_warps=0, n_pages_per_warp=1, stride=1, assignment=None, stream=None,
                     impl=0):
        """The pattern / cache benchmark kernels: pattern 0 sequential, 1 sequential by warp, 2 random
        (element indices in `assignment`), 3 random by warp (page indices in `assignment`); impl 0 reads
        through a bam_ptr cursor per thread, impl 1 through array[] (the benchmarks' ORIG type)."""
        check(self.lib.bam_launch_pattern_read_impl(self.h, pattern, impl, n_elems, n_warps, n_pages_per_warp, stride,
                                                    _ptr(assignment), _ptr(sum_out), _ptr(stream)), "bam_launch_pattern_read_impl")

    def page_scan(self, n_pages, sum_out, pages=None, first_page=0, stream=None):
        check(self.lib.bam_launch_page_scan(self.h, n_pages, _ptr(pages), first_page, _ptr(sum_out), _ptr(stream)),
              "bam_launch_page_scan")


def gen_uniform_indices(out, n_lanes, reqs_per_lane, access_seed, n_elems, stream=None):
    """Write the array random-read access stream (bam_synth.h) into a device u64 buffer."""
    lib = _lib.load()
    check(lib.bam_gen_uniform_indices(_ptr(out), n_lanes, reqs_per_lane, access_seed, n_elems, _ptr(stream)),
          "bam_gen_uniform_indices")


def gen_zipf_indices(out, n_lanes, reqs_per_lane, access_seed, cdf, n_pages, elems_per_page, perm_seed, stream=None):
    """Write the skewed-scan access stream (Zipf page popularity) into a device u64 buffer."""
    lib = _lib.load()
    check(lib.bam_gen_zipf_indices(_ptr(out), n_lanes, reqs_per_lane, access_seed, _ptr(cdf), n_pages, elems_per_page,
                                   perm_seed, _ptr(stream)), "bam_gen_zipf_indices")


def zipf_cdf(n_pages, s=0.99):
    """64-bit fixed-point CDF table of Zipf(s) over page ranks 1..n_pages (host, numpy uint64).

    cdf[r] = floor(2^64 * P(rank <= r)); float64 weights, sequential cumulative sum, last entry
    forced to 2^64-1.  Built once on the host: the device only compares integers."""
    import numpy as np
    w = np.arange(1, n_pages + 1, dtype=np.float64) ** (-s)
    c = np.cumsum(w)
    c /= c[-1]
    q = np.minimum(np.floor(c * 18446744073709551616.0), 18446744073709549568.0).astype(np.uint64)
    q[-1] = np.uint64(0xFFFFFFFFFFFFFFFF)
    return q


def shard_pages(n_pages, world_size, rank):
    """Contiguous page-range sharding of a store: returns (first_page, n_local_pages) of `rank`."""
    base, rem = divmod(n_pages, world_size)
    first = rank * base + min(rank, rem)
    return first, base + (1 if rank < rem else 0)


def direct_checksum(idx, n, store_seed, first_elem, sum_out, stream=None):
    """Device-side recomputation of the wrapping sum an index list must read (no cache, no queues)."""
    lib = _lib.load()
    check(lib.bam_direct_checksum(_ptr(idx), n, store_seed, first_elem, _ptr(sum_out), _ptr(stream)),
          "bam_direct_checksum")


def gen_block_pages(out, n_reqs, req_seed, n_pages, stream=None):
    """Write the page of every request of the block random-read workload into a device u64 buffer."""
    lib = _lib.load()
    check(lib.bam_gen_block_pages(_ptr(out), n_reqs, req_seed, n_pages, _ptr(stream)), "bam_gen_block_pages")


def page_sums(pages, n, store_seed, words_per_page, sum_out, stream=None):
    """Device-side recomputation of the wrapping sum of all words of the listed pages."""
    lib = _lib.load()
    check(lib.bam_direct_page_sums(_ptr(pages), n, store_seed, words_per_page, _ptr(sum_out), _ptr(stream)),
          "bam_direct_page_sums")


def bind_to_gpu_numa(cuda_device):
    """Pin the calling process to the CPUs that are local to `cuda_device` (its PCIe root's NUMA
    node), so that the backing store it allocates next -- pinned host memory, placed by first touch --
    sits next to the GPU that will read it.  Returns {"numa_node", "cpus"} or None if the topology
    cannot be read (then nothing is changed)."""
    import os
    try:
        import torch
        p = torch.cuda.get_device_properties(cuda_device)
        dom, bus, dev = getattr(p, "pci_domain_id", 0), p.pci_bus_id, p.pci_device_id
        base = f"/sys/bus/pci/devices/{dom:04x}:{bus:02x}:{dev:02x}.0"
        cpulist = open(os.path.join(base, "local_cpulist")).read().strip()
        node = int(open(os.path.join(base, "numa_node")).read().strip())
        cpus = set()
        for part in cpulist.split(","):
            if "-" in part:
                a, b = part.split("-")
                cpus.update(range(int(a), int(b) + 1))
            elif part:
                cpus.add(int(part))
        allowed = os.sched_getaffinity(0)
        cpus &= allowed
        if not cpus:
            return None
        os.sched_setaffinity(0, cpus)
        return {"numa_node": node, "cpus": len(cpus)}
    except Exception:
        return None


def probe_uplink_groups(n_bytes=128 << 20, shared_below=0.8, max_set=4):
    """Which GPUs of this box share host-link capacity, found by measurement: every visible GPU copies from
    pinned host memory alone; then sets of 2, 3 and 4 GPUs copy at the same time, and the members of a set
    whose rate falls below `shared_below` of their solo rate sit behind one shared link.  Sets larger than
    pairs matter: four GPUs behind one switch whose uplink carries two GPUs' worth of traffic slow down
    only when three of them copy at once.  Returns (groups, solo_gb_per_s): groups is a list of lists of
    device indices.  The PCI tree in sysfs is not used: on virtualised hosts it is flat and says nothing
    about the switches."""
    import itertools
    import torch
    n = torch.cuda.device_count()
    host, dev, streams = [], [], []
    for d in range(n):
        host.append(torch.empty(n_bytes, dtype=torch.uint8).pin_memory())
        dev.append(torch.empty(n_bytes, dtype=torch.uint8, device=f"cuda:{d}"))
        streams.append(torch.cuda.Stream(device=d))

    def run(devs, reps=2):
        best = {d: 0.0 for d in devs}
        for _ in range(reps):
            ev = {}
            for d in devs:
                with torch.cuda.device(d):
                    ev[d] = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            for d in devs:
                with torch.cuda.device(d), torch.cuda.stream(streams[d]):
                    ev[d][0].record(streams[d])
                    dev[d].copy_(host[d], non_blocking=True)
                    ev[d][1].record(streams[d])
            for d in devs:
                streams[d].synchronize()
                best[d] = max(best[d], n_bytes / (ev[d][0].elapsed_time(ev[d][1]) * 1e-3) / 1e9)
        return best

    solo = {}
    for d in range(n):
        solo[d] = run([d], reps=3)[d]
    parent = list(range(n))

    def find(x):
        while parent[x] != x:
            parent[x] = parent[parent[x]]
            x = parent[x]
        return x

    for k in range(2, min(max_set, n) + 1):
        for combo in itertools.combinations(range(n), k):
            if len({find(d) for d in combo}) == 1:
                continue                                  # already known to share
            together = run(list(combo))
            slow = [d for d in combo if together[d] / solo[d] < shared_below]
            for d in slow[1:]:
                parent[find(d)] = find(slow[0])
    groups = {}
    for d in range(n):
        groups.setdefault(find(d), []).append(d)
    del host, dev
    return sorted(groups.values()), [solo[d] for d in range(n)]


def spread_over_uplinks(groups):
    """Device order that deals the GPUs round-robin over the uplink groups: the first len(groups)
    ranks each get an uplink of their own."""
    order, k = [], 0
    while any(k < len(g) for g in groups):
        order += [g[k] for g in groups if k < len(g)]
        k += 1
    return order


def place_rank(world, local_rank, tag):
    """CUDA device for `local_rank` of a `world`-rank job on this box, spreading the ranks over distinct
    host uplinks first.  Matters only when fewer ranks than GPUs run: which GPUs share an uplink decides
    how much host-link bandwidth each rank gets.  Rank 0 measures (probe_uplink_groups) and leaves the
    result in a file in the temporary directory named after `tag` (the job's rendezvous port); the other
    ranks wait for it (bounded).  Returns (device, info); on any failure the identity placement."""
    import json
    import tempfile
    import time
    import torch
    n = torch.cuda.device_count()
    info = {"visible_gpus": n, "placement": "identity"}
    if world >= n or n <= 1 or world == 1:           # a single rank has every link to itself: nothing to measure
        return local_rank % max(1, n), info
    path = os.path.join(tempfile.gettempdir(), f"bam_b200_placement_{tag}.json")
    try:
        if local_rank == 0:
            groups, solo = probe_uplink_groups()
            order = spread_over_uplinks(groups)
            rec = {"groups": groups, "order": order, "solo_gb_per_s": [round(x, 1) for x in solo]}
            tmp = path + f".{os.getpid()}"
            with open(tmp, "w") as f:
                json.dump(rec, f)
            os.replace(tmp, path)
        else:
            t0 = time.time()
            while not os.path.exists(path):
                if time.time() - t0 > 120:
                    raise TimeoutError("placement file never appeared")
                time.sleep(0.05)
            with open(path) as f:
                rec = json.load(f)
        info = {"visible_gpus": n, "placement": "spread over host uplinks (measured)", "uplink_groups": rec["groups"],
                "device_order": rec["order"], "solo_gb_per_s": rec["solo_gb_per_s"]}
        return rec["order"][local_rank], info
    except Exception as e:       # placement is an optimisation: never fail the job over it
        info["placement"] = f"identity ({type(e).__name__}: {e})"
        return local_rank % n, info
