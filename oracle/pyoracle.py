"""ctypes wrapper of oracle/libbam_oracle.so (built from bam_oracle.c by oracle/Makefile).

Test infrastructure only: the checker and the timed host-core baseline, never a fallback.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libbam_oracle.so")
u32, u64, vp = C.c_uint32, C.c_uint64, C.c_void_p


class RefResult(C.Structure):
    _fields_ = [("checksum", u64), ("accesses", u64), ("hits", u64), ("misses", u64), ("read_ios", u64),
                ("seconds", C.c_double), ("worker_threads", u32), ("ctrl_threads", u32)]


def build(force=False):
    src = os.path.join(HERE, "bam_oracle.c")
    hdr = os.path.join(HERE, "..", "include", "bam_synth.h")
    if (force or not os.path.exists(LIB_PATH)
            or os.path.getmtime(LIB_PATH) < max(os.path.getmtime(src), os.path.getmtime(hdr))):
        subprocess.run(["make", "-C", HERE, "-B", "libbam_oracle.so"], check=True, capture_output=True)
    return LIB_PATH


REF_WIRE_PATH = os.path.join(HERE, "_ref", "libref_wire.so")
REF_PQ_PATH = os.path.join(HERE, "_ref", "libref_pq.so")
REF_CACHE_PATH = os.path.join(HERE, "_ref", "libref_cache.so")
REF_ADMIN_PATH = os.path.join(HERE, "_ref", "libref_admin.so")


def _reference_root():
    """Where the reference project lies: $BAM_REFERENCE_ROOT, else a directory `reference` next to this
    repository.  Without either only prebuilt libraries under oracle/_ref are used, and the tests that need
    the reference's code skip with a message that says so."""
    env = os.environ.get("BAM_REFERENCE_ROOT")
    if env:
        return env
    return os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


REFERENCE_ROOT = _reference_root()


def build_ref_wire(force=False):
    """Compile the reference's own wire-format code (oracle/ref_wire.cpp + the reference's sources where
    they lie) into oracle/_ref/libref_wire.so.  Needs the reference project; returns None without it and
    without a prebuilt library."""
    if os.path.isdir(os.path.join(REFERENCE_ROOT, "include")):
        srcs = [os.path.join(HERE, f) for f in ("ref_wire.cpp", "ref_pq.cpp", "ref_cache.cpp", "ref_admin.cpp", "Makefile")]
        srcs.append(os.path.join(HERE, "ref_shim", "simt", "atomic"))
        built = [REF_WIRE_PATH, REF_PQ_PATH, REF_CACHE_PATH, REF_ADMIN_PATH]
        if force or not all(map(os.path.exists, built)) or min(map(os.path.getmtime, built)) < max(map(os.path.getmtime, srcs)):
            subprocess.run(["make", "-C", HERE, "-B", "ref", "REFERENCE=" + REFERENCE_ROOT], check=True, capture_output=True)
    return REF_WIRE_PATH if os.path.exists(REF_WIRE_PATH) else None


_ref_wire = None


def ref_wire():
    """ctypes handle of the reference's wire-format code, or None when it cannot be had."""
    global _ref_wire
    if _ref_wire is None:
        path = build_ref_wire()
        if path is None:
            return None
        L = C.CDLL(path)
        u16, u8 = C.c_uint16, C.c_uint8
        L.refw_queue_new.restype = vp
        L.refw_queue_new.argtypes = [vp, C.c_int, u16, u32, vp, u64]
        L.refw_queue_free.argtypes = [vp]
        L.refw_queue_doorbell_offset.restype = u64
        L.refw_queue_doorbell_offset.argtypes = [vp]
        L.refw_encode_rw.argtypes = [u16, u8, u32, u64, u64, u64, u16, vp]
        L.refw_sq_put_rw.argtypes = [vp, u16, u8, u32, u64, u64, u64, u16]
        L.refw_sq_submit.argtypes = [vp]
        L.refw_cq_take.argtypes = [vp, vp, u64, C.POINTER(u16), C.POINTER(u16), C.POINTER(u16), C.POINTER(u8), C.POINTER(u8),
                                   C.POINTER(C.c_int)]
        L.refw_strerror.restype = C.c_char_p
        L.refw_strerror.argtypes = [C.c_int]
        L.refw_unpack_sct.argtypes = [C.c_int]
        L.refw_unpack_sc.argtypes = [C.c_int]
        L.refw_page_align.restype = u64
        L.refw_page_align.argtypes = [u64, u64]
        L.refw_page_to_block.restype = u64
        L.refw_page_to_block.argtypes = [u64, u64, u64]
        L.refw_sizeof_queue.restype = u32
        L.refw_cmd_data.restype = u64
        L.refw_cmd_data.argtypes = [u64, vp, C.POINTER(u64), u64, u64, C.POINTER(u64), C.POINTER(u32)]
        L.refw_sq_pages.restype = u64
        L.refw_sq_pages.argtypes = [u64, u32]
        L.refw_cq_pages.restype = u64
        L.refw_cq_pages.argtypes = [u64, u32]
        L.refw_default_cid.restype = u32
        L.refw_default_cid.argtypes = [u32, C.c_int, u32]
        L.refw_opcode.restype = u32
        L.refw_opcode.argtypes = [C.c_int, C.c_int, C.c_int]
        _ref_wire = L
    return _ref_wire


_ref_admin = None


def ref_admin():
    """ctypes handle of the reference's admin layer (src/admin.cpp) whose nvm_raw_rpc is bound by the caller
    (refa_bind) to the library under test, or None."""
    global _ref_admin
    if _ref_admin is None:
        build_ref_wire()
        if not os.path.exists(REF_ADMIN_PATH):
            return None
        L = C.CDLL(REF_ADMIN_PATH)
        u16, u8 = C.c_uint16, C.c_uint8
        L.refa_bind.argtypes = [vp, vp]
        L.refa_ctrl_info.argtypes = [vp, vp, vp, u64]
        L.refa_ns_info.argtypes = [vp, vp, u32, vp, u64]
        L.refa_request_num_queues.argtypes = [vp, C.POINTER(u16), C.POINTER(u16)]
        L.refa_get_num_queues.argtypes = [vp, C.POINTER(u16), C.POINTER(u16)]
        L.refa_queue_alloc.restype = vp
        L.refa_queue_free.argtypes = [vp]
        L.refa_queue_qs.restype = u32
        L.refa_queue_qs.argtypes = [vp]
        L.refa_queue_doorbell_offset.restype = u64
        L.refa_queue_doorbell_offset.argtypes = [vp, vp]
        L.refa_cq_create.argtypes = [vp, vp, u16, vp, u64, u64]
        L.refa_sq_create.argtypes = [vp, vp, vp, u16, vp, u64, u64]
        L.refa_cq_delete.argtypes = [vp, vp]
        L.refa_sq_delete.argtypes = [vp, vp, vp]
        L.refa_rw.argtypes = [vp, vp, u8, u32, u64, u64, u16, u64]
        _ref_admin = L
    return _ref_admin


_ref_pq = None


def ref_pq():
    """ctypes handle of the reference's parallel queue protocol compiled for host threads, or None."""
    global _ref_pq
    if _ref_pq is None:
        build_ref_wire()
        if not os.path.exists(REF_PQ_PATH):
            return None
        L = C.CDLL(REF_PQ_PATH)
        u16, u8 = C.c_uint16, C.c_uint8
        L.refpq_pair_new.restype = vp
        L.refpq_pair_new.argtypes = [vp, u16, u32, vp, u64, u32, vp, u64, u32]
        L.refpq_pair_free.argtypes = [vp]
        L.refpq_run.argtypes = [vp, u32, u8, vp, vp, u16, u64, u64]
        L.refpq_state.argtypes = [vp] + [C.POINTER(u32)] * 5
        _ref_pq = L
    return _ref_pq


class RefCacheStats(C.Structure):
    _fields_ = [("checksum", u64), ("accesses", u64), ("misses", u64), ("hits", u64), ("read_ios", u64), ("extra_reads", u64)]


_ref_cache = None


def ref_cache():
    """ctypes handle of the reference's page cache + array read path compiled for host threads, or None."""
    global _ref_cache
    if _ref_cache is None:
        build_ref_wire()
        if not os.path.exists(REF_CACHE_PATH):
            return None
        L = C.CDLL(REF_CACHE_PATH)
        L.refc_new.restype = vp
        L.refc_new.argtypes = [vp, u32, u32, C.POINTER(vp), C.POINTER(vp), u32, u64, u64, u32]
        L.refc_new2.restype = vp
        L.refc_new2.argtypes = [vp, u32, u32, C.POINTER(vp), C.POINTER(vp), u32, u64, u64, u32, vp, u64]
        L.refc_free.argtypes = [vp]
        L.refc_array_read.argtypes = [vp, vp, u64, u32, u64, C.POINTER(RefCacheStats)]
        L.refc_page_state.restype = u32
        L.refc_page_state.argtypes = [vp, u64]
        L.refc_page_slot.restype = u32
        L.refc_page_slot.argtypes = [vp, u64]
        _ref_cache = L
    return _ref_cache


class RefCacheWorld:
    """The reference's array read path (host build) over queue pairs served by the oracle's controller:
    `store` (numpy uint64) is the namespace; reads go through a cache of n_slots pages."""

    def __init__(self, store, n_slots, n_qps=2, qs=16, page_size=4096, lba_bytes=512):
        self.L, self.O = ref_cache(), lib()
        self.store = store
        self.regs = np.zeros(0x2000, dtype=np.uint8)
        self.qmem = np.zeros((2 * n_qps + 1) * 4096, dtype=np.uint8)
        base = (self.qmem.ctypes.data + 4095) // 4096 * 4096
        sq = (vp * n_qps)(*[base + (2 * q + 1) * 4096 for q in range(n_qps)])
        cq = (vp * n_qps)(*[base + (2 * q) * 4096 for q in range(n_qps)])
        assert qs * 64 <= 4096
        self.ctrls = [self.O.orc_wire_ctrl_start(sq[q], cq[q], self.regs.ctypes.data + 0x1000 + 8 * (q + 1),
                                                 self.regs.ctypes.data + 0x1000 + 8 * (q + 1) + 4, qs, qs, q + 1,
                                                 store.ctypes.data, store.nbytes, lba_bytes) for q in range(n_qps)]
        self.h = self.L.refc_new(self.regs.ctypes.data, n_qps, qs, sq, cq, page_size, n_slots, store.nbytes // page_size, lba_bytes)
        assert self.h and all(self.ctrls)

    def read(self, idx, n_threads=1, timeout_ms=60000):
        idx = np.ascontiguousarray(idx, dtype=np.uint64)
        st = RefCacheStats()
        rc = self.L.refc_array_read(self.h, idx.ctypes.data, len(idx), n_threads, timeout_ms, C.byref(st))
        if rc:
            raise RuntimeError(f"the reference's read path stalled ({rc})")
        return st

    def page_state(self, page):
        return self.L.refc_page_state(self.h, page), self.L.refc_page_slot(self.h, page)

    def close(self):
        served = [self.O.orc_wire_ctrl_stop(c) for c in self.ctrls]
        self.L.refc_free(self.h)
        self.ctrls, self.h = [], None
        return served


def encode_rw(cid, opcode, ns_id, prp1, prp2, start_lba, n_blocks):
    """The oracle's restatement of the read/write command encoding (64 bytes)."""
    out = (C.c_uint8 * 64)()
    lib().orc_encode_rw(cid, opcode, ns_id, prp1, prp2, start_lba, n_blocks, out)
    return bytes(out)


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(LIB_PATH)
        L.orc_splitmix64.restype = u64
        L.orc_splitmix64.argtypes = [u64]
        L.orc_pcg32_stream.argtypes = [u64, u64, vp, u64]
        L.orc_crc32.restype = u32
        L.orc_crc32.argtypes = [vp, u64]
        L.orc_permute.restype = u64
        L.orc_permute.argtypes = [u64, u64, u64]
        L.orc_fill_store.argtypes = [vp, u64, u64, u64]
        L.orc_fill_pages.argtypes = [vp, u64, u64, vp, u64, u32]
        L.orc_array_indices.argtypes = [u64, u64, u64, u64, u64, vp]
        L.orc_array_checksum.restype = u64
        L.orc_array_checksum.argtypes = [u64, u64, u64, u64, u64, u64]
        L.orc_indexed_checksum.restype = u64
        L.orc_indexed_checksum.argtypes = [u64, u64, vp, u64]
        L.orc_backing_location.restype = u64
        L.orc_backing_location.argtypes = [u64, u64, u64, u32, C.POINTER(u32)]
        L.orc_wire_ctrl_start.restype = vp
        L.orc_wire_ctrl_start.argtypes = [vp, vp, vp, vp, u32, u32, C.c_uint16, vp, u64, u32]
        L.orc_wire_ctrl_start_mt.restype = vp
        L.orc_wire_ctrl_start_mt.argtypes = [vp, vp, vp, vp, u32, u32, C.c_uint16, vp, u64, u32, u32, u32]
        L.orc_wire_ctrl_stop_mt.restype = u64
        L.orc_wire_ctrl_stop_mt.argtypes = [vp, C.POINTER(u64), C.POINTER(u64)]
        L.orc_wire_ctrl_stop.restype = u64
        L.orc_wire_ctrl_stop.argtypes = [vp]
        L.orc_encode_rw.argtypes = [C.c_uint16, C.c_uint8, u32, u64, u64, u64, u32, vp]
        L.orc_page_crc.restype = u32
        L.orc_page_crc.argtypes = [u64, u64, u32]
        L.orc_block_requests.argtypes = [u64, u64, u64, u32, u64, u64, vp, vp]
        L.orc_zipf_indices.argtypes = [vp, u64, u32, u64, u64, u64, u64, u64, vp]
        L.orc_rmat_csr.restype = u64
        L.orc_rmat_csr.argtypes = [u64, u32, u64, u32, u32, u32, vp, vp]
        L.orc_max_degree_vertex.restype = u64
        L.orc_max_degree_vertex.argtypes = [u64, vp]
        L.orc_bfs.restype = u64
        L.orc_bfs.argtypes = [u64, vp, vp, u64, vp]
        L.orc_cc.restype = u64
        L.orc_cc.argtypes = [u64, vp, vp, vp]
        L.orc_edge_weights.argtypes = [u64, u64, vp]
        L.orc_sssp.argtypes = [u64, vp, vp, vp, u64, vp]
        L.orc_pagerank.restype = u32
        L.orc_pagerank.argtypes = [u64, vp, vp, u64, u64, u64, u32, vp, C.POINTER(u64)]
        L.ref_array_read.restype = C.c_int
        L.ref_array_read.argtypes = [vp, u64, u32, u64, u32, u32, u32, u32, u32, vp, u64, u64, u64, u64,
                                     C.POINTER(RefResult)]
        L.ref_block_read.restype = C.c_int
        L.ref_block_read.argtypes = [vp, u64, u32, u32, u32, u32, u32, u32, u64, u64, vp, C.POINTER(RefResult)]
        L.ref_graph_run.restype = C.c_int
        L.ref_graph_run.argtypes = [vp, u64, u64, u64, C.c_int, u64, u32, u64, u32, u32, u32, u32, u32, vp, vp,
                                    C.POINTER(u64), C.POINTER(u32), C.POINTER(RefResult)]
        _lib = L
    return _lib


def _p(a):
    return a.ctypes.data_as(vp) if a is not None else None


def splitmix64(x):
    return lib().orc_splitmix64(x)


def pcg32_stream(state, seq, n):
    out = np.empty(n, dtype=np.uint32)
    lib().orc_pcg32_stream(state, seq, _p(out), n)
    return out


def crc32(b):
    buf = np.frombuffer(bytes(b), dtype=np.uint8)
    return lib().orc_crc32(_p(buf), len(buf))


def fill_store(seed, first_elem, n, out=None):
    if out is None:
        out = np.empty(n, dtype=np.uint64)
    lib().orc_fill_store(_p(out), seed, first_elem, n)
    return out


def fill_pages(store, seed, first_elem, pages, elems_per_page=512):
    pages = np.ascontiguousarray(pages, dtype=np.uint64)
    lib().orc_fill_pages(_p(store), seed, first_elem, _p(pages), len(pages), elems_per_page)


def array_indices(access_seed, n_elems, lane_begin, lane_end, reqs_per_lane):
    out = np.empty((lane_end - lane_begin) * reqs_per_lane, dtype=np.uint64)
    lib().orc_array_indices(access_seed, n_elems, lane_begin, lane_end, reqs_per_lane, _p(out))
    return out


def array_checksum(store_seed, n_elems, access_seed, lane_begin, lane_end, reqs_per_lane):
    return lib().orc_array_checksum(store_seed, n_elems, access_seed, lane_begin, lane_end, reqs_per_lane)


def indexed_checksum(store_seed, first_elem, idx):
    idx = np.ascontiguousarray(idx, dtype=np.uint64)
    return lib().orc_indexed_checksum(store_seed, first_elem, _p(idx), len(idx))


def backing_location(page_start, page, n_ctrls, dist):
    """(controller or None for "all", backing page) of a range's page behind n_ctrls controllers."""
    ctrl = C.c_uint32()
    backing = lib().orc_backing_location(page_start, page, n_ctrls, dist, C.byref(ctrl))
    return (None if ctrl.value == 0xFFFFFFFF else ctrl.value), backing


def page_crc(store_seed, page, page_bytes=4096):
    return lib().orc_page_crc(store_seed, page, page_bytes)


def block_requests(store_seed, req_seed, n_pages, page_bytes, r0, r1, want_crc=True):
    pages = np.empty(r1 - r0, dtype=np.uint64)
    crc = np.empty(r1 - r0, dtype=np.uint32) if want_crc else None
    lib().orc_block_requests(store_seed, req_seed, n_pages, page_bytes, r0, r1, _p(pages), _p(crc))
    return pages, crc


def zipf_cdf(n_pages, s=0.99):
    """64-bit fixed-point CDF of Zipf(s) over ranks 1..n_pages (rank r has weight r^-s).
    Built in float64 with a sequential cumulative sum; the last entry is forced to 2^64-1."""
    w = np.arange(1, n_pages + 1, dtype=np.float64) ** (-s)
    c = np.cumsum(w)
    c /= c[-1]
    q = np.minimum(np.floor(c * 18446744073709551616.0), 18446744073709549568.0).astype(np.uint64)
    q[-1] = np.uint64(0xFFFFFFFFFFFFFFFF)
    return q


def zipf_indices(cdf, n_pages, elems_per_page, perm_seed, access_seed, lane_begin, lane_end, reqs_per_lane):
    out = np.empty((lane_end - lane_begin) * reqs_per_lane, dtype=np.uint64)
    lib().orc_zipf_indices(_p(cdf), n_pages, elems_per_page, perm_seed, access_seed, lane_begin, lane_end,
                           reqs_per_lane, _p(out))
    return out


def rmat_thresholds(a=0.57, b=0.19, c=0.19):
    """Integer quadrant thresholds floor(p * 2^32) for the R-MAT generator."""
    ta = int(a * 4294967296.0)
    tab = int((a + b) * 4294967296.0)
    tabc = int((a + b + c) * 4294967296.0)
    return ta, tab, tabc


def rmat_csr(seed, scale, edge_factor=16, thresholds=None):
    ta, tab, tabc = thresholds or rmat_thresholds()
    n = 1 << scale
    offsets = np.empty(n + 1, dtype=np.uint64)
    m = lib().orc_rmat_csr(seed, scale, edge_factor, ta, tab, tabc, _p(offsets), None)
    cols = np.empty(m, dtype=np.uint64)
    m2 = lib().orc_rmat_csr(seed, scale, edge_factor, ta, tab, tabc, _p(offsets), _p(cols))
    assert m == m2
    return offsets, cols


def max_degree_vertex(offsets):
    return lib().orc_max_degree_vertex(len(offsets) - 1, _p(offsets))


def bfs(offsets, cols, src):
    n = len(offsets) - 1
    level = np.empty(n, dtype=np.uint32)
    scanned = lib().orc_bfs(n, _p(offsets), _p(cols), src, _p(level))
    return level, scanned


def cc(offsets, cols):
    n = len(offsets) - 1
    label = np.empty(n, dtype=np.uint64)
    comps = lib().orc_cc(n, _p(offsets), _p(cols), _p(label))
    return label, comps


PR_FRAC_BITS = 40


def edge_weights(seed, n_edges):
    out = np.empty(n_edges, dtype=np.uint32)
    lib().orc_edge_weights(seed, n_edges, _p(out))
    return out


def sssp(offsets, cols, weights, src):
    """Dijkstra distances (uint32, 0xFFFFFFFF = unreachable)."""
    n = len(offsets) - 1
    dist = np.empty(n, dtype=np.uint32)
    weights = np.ascontiguousarray(weights, dtype=np.uint32)
    lib().orc_sssp(n, _p(offsets), _p(cols), _p(weights), src, _p(dist))
    return dist


def pagerank(offsets, cols, alpha=(85, 100), tolerance_q=None, max_iters=100):
    """Fixed-point delta PageRank; returns (values uint64 with PR_FRAC_BITS fraction bits, sweeps, edges scanned)."""
    n = len(offsets) - 1
    if tolerance_q is None:
        tolerance_q = (1 << PR_FRAC_BITS) // 1000
    value = np.empty(n, dtype=np.uint64)
    scanned = u64()
    iters = lib().orc_pagerank(n, _p(offsets), _p(cols), alpha[0], alpha[1], tolerance_q, max_iters, _p(value),
                               C.byref(scanned))
    return value, iters, scanned.value


def ref_array_read(store, page_size, n_slots, n_qps, qdepth, lba_bytes, workers, ctrl_threads,
                   idx=None, access_seed=0, lane_begin=0, lane_end=0, reqs_per_lane=0):
    """The reference's array read path restated on host threads; returns a RefResult."""
    r = RefResult()
    if idx is not None:
        idx = np.ascontiguousarray(idx, dtype=np.uint64)
    rc = lib().ref_array_read(_p(store), len(store), page_size, n_slots, n_qps, qdepth, lba_bytes, workers,
                              ctrl_threads, _p(idx), access_seed, lane_begin, lane_end, reqs_per_lane, C.byref(r))
    if rc:
        raise RuntimeError(f"ref_array_read failed: {rc}")
    return r


def ref_block_read(store, page_size, n_qps, qdepth, lba_bytes, workers, ctrl_threads, req_seed, n_reqs,
                   want_crc=True):
    r = RefResult()
    crc = np.zeros(n_reqs, dtype=np.uint32) if want_crc else None
    rc = lib().ref_block_read(_p(store), store.nbytes, page_size, n_qps, qdepth, lba_bytes, workers, ctrl_threads,
                              req_seed, n_reqs, _p(crc), C.byref(r))
    if rc:
        raise RuntimeError(f"ref_block_read failed: {rc}")
    return r, crc


def csr_store(offsets, cols, page_size=4096):
    """The backing-store image of a CSR graph: offsets (padded to a page) followed by cols."""
    pad = lambda b: (b + page_size - 1) // page_size * page_size  # noqa: E731
    off_bytes = pad(len(offsets) * 8)
    store = np.zeros((off_bytes + pad(max(1, len(cols)) * 8)) // 8, dtype=np.uint64)
    store[:len(offsets)] = offsets
    store[off_bytes // 8:off_bytes // 8 + len(cols)] = cols
    return store, off_bytes


def ref_graph_run(store, n_vertices, cols_byte_offset, mode, source, n_slots, n_qps, qdepth, workers, ctrl_threads,
                  page_size=4096, lba_bytes=512):
    """BFS (mode 0) or CC (mode 1) through the CPU restatement of the reference's cache and queues.
    Returns (levels or labels, edges scanned, iterations, RefResult)."""
    r = RefResult()
    level = np.empty(n_vertices, dtype=np.uint32) if mode == 0 else None
    comp = np.empty(n_vertices, dtype=np.uint64) if mode == 1 else None
    scanned, iters = u64(), u32()
    rc = lib().ref_graph_run(_p(store), store.nbytes, n_vertices, cols_byte_offset, mode, source, page_size, n_slots,
                             n_qps, qdepth, lba_bytes, workers, ctrl_threads, _p(level), _p(comp), C.byref(scanned),
                             C.byref(iters), C.byref(r))
    if rc:
        raise RuntimeError(f"ref_graph_run failed: {rc}")
    return (level if mode == 0 else comp), scanned.value, iters.value, r
