"""Graph consumers: CSR graphs in the backing store, BFS and connected components through
bam::array (host mirror of the drivers in the reference's benchmarks/bfs and benchmarks/cc).

The CSR is built on the GPU from the seeded R-MAT generator of include/bam_synth.h (torch sort /
unique are plumbing here, exactly like reading a .bel file would be); row offsets and column
indices are then written to the controller's backing store, offsets first, each page aligned, and
from then on are read only through the page cache."""
import ctypes as C

import numpy as np

from . import _lib
from ._lib import BamError, check
from .host import Array, Controller, PageCache, _ptr


def rmat_thresholds(a=0.57, b=0.19, c=0.19):
    """Integer quadrant thresholds floor(p * 2^32) of the R-MAT generator."""
    return int(a * 4294967296.0), int((a + b) * 4294967296.0), int((a + b + c) * 4294967296.0)


def build_rmat_csr(seed, scale, edge_factor=16, device="cuda", thresholds=None, chunk_edges=1 << 25):
    """Undirected, de-duplicated, sorted CSR of the seeded R-MAT graph, on the device.

    Returns (offsets[n+1], cols[m]) as int64 tensors (the u64 values fit: scale <= 31)."""
    import torch
    lib = _lib.load()
    ta, tab, tabc = thresholds or rmat_thresholds()
    n, m = 1 << scale, edge_factor << scale
    parts = []
    for e0 in range(0, m, chunk_edges):
        e1 = min(m, e0 + chunk_edges)
        k = torch.empty(2 * (e1 - e0), dtype=torch.int64, device=device)
        check(lib.bam_gen_rmat_keys(_ptr(k), e0, e1, seed, scale, ta, tab, tabc, None), "bam_gen_rmat_keys")
        k = torch.unique(k)                      # sorted, duplicates within the chunk removed
        parts.append(k)
    keys = torch.unique(torch.cat(parts)) if len(parts) > 1 else parts[0]
    del parts
    if keys.numel() and int(keys[0].item()) == -1:      # self loops were written as ~0
        keys = keys[1:]
    src = keys >> 32
    cols = keys & 0xFFFFFFFF
    counts = torch.bincount(src, minlength=n)
    offsets = torch.zeros(n + 1, dtype=torch.int64, device=device)
    torch.cumsum(counts, 0, out=offsets[1:])
    return offsets, cols


def write_bel(path, values):
    """Write a `.bel.*` file as the reference's converter does (benchmarks/bam_data_conversion.py:26-35):
    a 16-byte header {count: u64, type size: u64} followed by the values as little-endian int64."""
    a = np.ascontiguousarray(values, dtype="<i8")
    with open(path, "wb") as f:
        f.write(np.array([a.size, 8], dtype="<u8").tobytes())
        f.write(a.tobytes())


def read_bel(path):
    """Read a `.bel.col` (row offsets) / `.bel.dst` (column indices) file: 16-byte header, then
    int64 values (the layout benchmarks/bfs/main.cu:1244-1281 reads)."""
    with open(path, "rb") as f:
        hdr = np.frombuffer(f.read(16), dtype="<u8")
        count = int(hdr[0])
        data = np.frombuffer(f.read(count * 8), dtype="<i8")
    if data.size != count:
        raise ValueError(f"{path}: header announces {count} values, file holds {data.size}")
    return data


def load_bel_graph(prefix, device="cuda"):
    """CSR (offsets, cols) tensors from `<prefix>.bel.col` and `<prefix>.bel.dst`."""
    import torch
    off = torch.from_numpy(read_bel(prefix + ".bel.col").copy()).to(device)
    cols = torch.from_numpy(read_bel(prefix + ".bel.dst").copy()).to(device)
    return off, cols


PR_FRAC_BITS = 40     # fraction bits of the fixed-point PageRank values (BAM_PR_FRAC_BITS)


class CsrGraph:
    """A CSR graph stored behind an emulated NVMe controller and read through a page cache."""

    def __init__(self, offsets, cols, cache_pages, cuda_device=0, queue_depth=1024, num_queues=128, page_size=4096,
                 ctrl_blocks=0, weights=None):
        """`weights` (optional, int32 tensor, one per edge) is stored behind the column indices as a
        third array of u32 elements (the .val file of the reference's weighted benchmarks)."""
        import torch
        self.n = offsets.numel() - 1
        self.m = cols.numel()
        pad = lambda b: (b + page_size - 1) // page_size * page_size  # noqa: E731
        self.off_bytes = pad((self.n + 1) * 8)
        self.col_bytes = pad(max(1, self.m) * 8)
        self.wt_bytes = pad(max(1, self.m) * 4) if weights is not None else 0
        self.ctrl = Controller(self.off_bytes + self.col_bytes + self.wt_bytes, cuda_device, queue_depth=queue_depth,
                               num_queues=num_queues)
        if ctrl_blocks:
            self.ctrl.configure(ctrl_blocks=ctrl_blocks)
        lib = self.ctrl.lib
        check(lib.bam_ctrl_write_store_from_device(self.ctrl.h, 0, _ptr(offsets), (self.n + 1) * 8, None), "write offsets")
        if self.m:
            check(lib.bam_ctrl_write_store_from_device(self.ctrl.h, self.off_bytes, _ptr(cols), self.m * 8, None), "write cols")
            if weights is not None:
                assert weights.numel() == self.m and weights.element_size() == 4
                check(lib.bam_ctrl_write_store_from_device(self.ctrl.h, self.off_bytes + self.col_bytes, _ptr(weights),
                                                           self.m * 4, None), "write weights")
        torch.cuda.synchronize()
        self.cache = PageCache(self.ctrl, page_size, cache_pages)
        self._owns = True
        self._bind(cuda_device, weighted=weights is not None)

    @classmethod
    def over_cache(cls, cache, n_vertices, n_edges, off_bytes, dist=0, cuda_device=0):
        """A graph whose store image (offsets padded to `off_bytes`, then the edges) is already on the
        media behind `cache` -- one controller or several, laid out as `dist` says."""
        g = cls.__new__(cls)
        g.n, g.m, g.off_bytes, g.col_bytes = n_vertices, n_edges, off_bytes, 0
        g.ctrl, g.cache, g._owns = cache.ctrl, cache, False
        g._bind(cuda_device, dist)
        return g

    def _bind(self, cuda_device, dist=0, weighted=False):
        import torch
        self.offsets = Array(self.cache, self.n + 1, 8, 0, dist)
        self.cols = Array(self.cache, max(1, self.m), 8, self.off_bytes, dist)
        self.weights = Array(self.cache, max(1, self.m), 4, self.off_bytes + self.col_bytes, dist) if weighted else None
        self.device = cuda_device
        # per-level scratch for the work items of hub vertices
        self.scratch_bytes = self.ctrl.lib.bam_graph_scratch_bytes(max(1, self.m))
        self.scratch = torch.empty(self.scratch_bytes, dtype=torch.uint8, device=f"cuda:{cuda_device}")

    def close(self):
        if self.weights is not None:
            self.weights.close()
        self.cols.close(); self.offsets.close()
        if self._owns:
            self.cache.close(); self.ctrl.close()

    def sssp(self, source):
        """Single-source shortest paths over the edge weights; returns (u32 distances as an int32
        tensor, 0xFFFFFFFF = unreachable; sweeps; edges_scanned)."""
        import torch
        if self.weights is None:
            raise ValueError("the graph has no weights")
        cost = torch.empty(self.n, dtype=torch.int32, device=f"cuda:{self.device}")
        ni, sc = C.c_uint32(), C.c_uint64()
        check(self.ctrl.lib.bam_sssp_run(self.offsets.h, self.cols.h, self.weights.h, self.n, source, _ptr(cost),
                                         C.byref(ni), C.byref(sc)), "bam_sssp_run")
        return cost, ni.value, sc.value

    def pagerank(self, alpha=(85, 100), tolerance_q=None, max_iters=100):
        """Delta PageRank in 64-bit fixed point (PR_FRAC_BITS fraction bits); returns (ranks as an int64
        tensor of fixed-point values, sweeps, edges_scanned).  tolerance_q defaults to 0.001."""
        import torch
        if tolerance_q is None:
            tolerance_q = (1 << PR_FRAC_BITS) // 1000
        value = torch.empty(self.n, dtype=torch.int64, device=f"cuda:{self.device}")
        ni, sc = C.c_uint32(), C.c_uint64()
        check(self.ctrl.lib.bam_pagerank_run(self.offsets.h, self.cols.h, self.n, alpha[0], alpha[1], tolerance_q, max_iters,
                                             _ptr(value), C.byref(ni), C.byref(sc)), "bam_pagerank_run")
        return value, ni.value, sc.value

    def bfs(self, source):
        """Level-synchronous BFS from `source`; returns (levels uint32 tensor as int32 bits, n_levels, edges_scanned)."""
        import torch
        label = torch.empty(self.n, dtype=torch.int32, device=f"cuda:{self.device}")
        nl, sc = C.c_uint32(), C.c_uint64()
        check(self.ctrl.lib.bam_bfs_run(self.offsets.h, self.cols.h, self.n, source, _ptr(label), C.byref(nl), C.byref(sc)),
              "bam_bfs_run")
        return label, nl.value, sc.value

    def cc(self):
        """Connected components by label propagation; returns (labels int64 tensor, sweeps, edges_scanned)."""
        import torch
        comp = torch.empty(self.n, dtype=torch.int64, device=f"cuda:{self.device}")
        ns, sc = C.c_uint32(), C.c_uint64()
        check(self.ctrl.lib.bam_cc_run(self.offsets.h, self.cols.h, self.n, _ptr(comp), C.byref(ns), C.byref(sc)),
              "bam_cc_run")
        return comp, ns.value, sc.value

    def bfs_level(self, v_begin, v_end, level, label, changed, scanned=None, v_base=0, stream=None):
        check(self.ctrl.lib.bam_launch_bfs_level(self.offsets.h, self.cols.h, v_begin, v_end, v_base, level, _ptr(label),
                                                 _ptr(changed), _ptr(scanned), _ptr(self.scratch), self.scratch_bytes,
                                                 _ptr(stream)), "bam_launch_bfs_level")

    def cc_sweep(self, v_begin, v_end, comp, curr_visit, next_visit, changed, scanned=None, v_base=0, stream=None):
        check(self.ctrl.lib.bam_launch_cc_sweep(self.offsets.h, self.cols.h, v_begin, v_end, v_base, _ptr(comp),
                                                _ptr(curr_visit), _ptr(next_visit), _ptr(changed), _ptr(scanned),
                                                _ptr(self.scratch), self.scratch_bytes, _ptr(stream)), "bam_launch_cc_sweep")

    # exchange steps of the sharded traversals (bam_exchange.cu); hdr = int64[2], hdrs = int64[2 * world]
    def frontier_compact(self, label, level_value, out, hdr, stream=None):
        check(self.ctrl.lib.bam_launch_frontier_compact(self.cache.h, _ptr(label), label.numel(), level_value, _ptr(out),
                                                        out.numel(), _ptr(hdr), _ptr(stream)), "bam_launch_frontier_compact")

    def frontier_apply(self, label, level_value, recv, stride, hdrs, world, rank, stream=None):
        check(self.ctrl.lib.bam_launch_frontier_apply(_ptr(label), label.numel(), level_value, _ptr(recv), stride, _ptr(hdrs),
                                                      world, rank, _ptr(stream)), "bam_launch_frontier_apply")

    def cc_compact(self, comp, next_visit, out, hdr, stream=None):
        check(self.ctrl.lib.bam_launch_cc_compact(self.cache.h, _ptr(comp), _ptr(next_visit), comp.numel(), _ptr(out),
                                                  out.numel(), _ptr(hdr), _ptr(stream)), "bam_launch_cc_compact")

    def cc_apply(self, comp, next_visit, own_begin, own_end, recv, stride, hdrs, world, rank, stream=None):
        check(self.ctrl.lib.bam_launch_cc_apply(_ptr(comp), _ptr(next_visit), comp.numel(), own_begin, own_end, _ptr(recv),
                                                stride, _ptr(hdrs), world, rank, _ptr(stream)), "bam_launch_cc_apply")

    def cc_dense_flag(self, comp, before_own, next_visit, own_begin, own_end, stream=None):
        check(self.ctrl.lib.bam_launch_cc_dense_flag(_ptr(comp), _ptr(before_own), _ptr(next_visit), own_begin, own_end,
                                                     _ptr(stream)), "bam_launch_cc_dense_flag")

    def sssp_sweep(self, v_begin, v_end, label, new_cost, scanned=None, v_base=0, stream=None):
        check(self.ctrl.lib.bam_launch_sssp_sweep(self.offsets.h, self.cols.h, self.weights.h, v_begin, v_end, v_base,
                                                  _ptr(label), _ptr(new_cost), _ptr(scanned), _ptr(self.scratch),
                                                  self.scratch_bytes, _ptr(stream)), "bam_launch_sssp_sweep")

    def pr_sweep(self, v_begin, v_end, label, delta, residual, scanned=None, v_base=0, stream=None):
        check(self.ctrl.lib.bam_launch_pr_sweep(self.offsets.h, self.cols.h, v_begin, v_end, v_base, _ptr(label), _ptr(delta),
                                                _ptr(residual), _ptr(scanned), _ptr(self.scratch), self.scratch_bytes,
                                                _ptr(stream)), "bam_launch_pr_sweep")


# ---- multi-GPU traversals: vertex-range sharding, replicated labels, all-gather exchange -------------

def shard_vertices(n, world_size, rank):
    """Contiguous vertex range [v0, v1) of `rank`."""
    base, rem = divmod(n, world_size)
    v0 = rank * base + min(rank, rem)
    return v0, v0 + base + (1 if rank < rem else 0)


def shard_vertices_by_edges(offsets, world_size, rank):
    """Contiguous vertex range [v0, v1) of `rank` such that every rank owns about the same number of
    edges (R-MAT degrees are so skewed that equal vertex counts would give very unequal shards).
    `offsets` is the CSR row-offset tensor; the cut points are the same on every rank."""
    import torch
    n = offsets.numel() - 1
    m = int(offsets[-1].item())
    targets = torch.tensor([m * r // world_size for r in range(world_size + 1)], dtype=offsets.dtype, device=offsets.device)
    cuts = torch.searchsorted(offsets, targets, right=False).clamp_(0, n)
    cuts[0], cuts[-1] = 0, n
    cuts = torch.cummax(cuts, 0).values
    return int(cuts[rank].item()), int(cuts[rank + 1].item())


def gather_headers(hdr, hdrs, group=None):
    """All-gather the 16-byte headers {entries, status} of every rank's send buffer and bring them to the
    host: the ONE device-to-host read of a level / sweep.  Returns (counts, statuses) as lists."""
    import torch.distributed as dist
    dist.all_gather_into_tensor(hdrs, hdr, group=group)
    h = hdrs.tolist()
    return h[0::2], h[1::2]


def raise_on_rank_failure(statuses):
    """Every rank sees every rank's status code in the gathered headers, so all of them stop together."""
    bad = [(r, c) for r, c in enumerate(statuses) if c]
    if bad:
        r, c = bad[0]
        raise BamError(int(c), f"rank {r} reported a device-side failure during the traversal")


def allreduce_min_u32(t, group=None):
    """Element-wise minimum over ranks of a tensor that holds u32 values in int32 storage
    (0xFFFFFFFF = unreachable must compare as the largest value): flipping the sign bit maps the
    unsigned order onto the signed one.  In place; returns t."""
    import torch.distributed as dist
    t ^= -2147483648
    dist.all_reduce(t, op=dist.ReduceOp.MIN, group=group)
    t ^= -2147483648
    return t


def u32_less(a, b):
    """a < b for u32 values held in int32 tensors."""
    return (a ^ -2147483648) < (b ^ -2147483648)


class DistCsrGraph:
    """One rank's shard (a contiguous vertex range and its adjacency lists) of a CSR graph; BFS and
    CC run level by level with the frontier / the changed labels exchanged by all-gather (compaction and
    apply kernels of bam_exchange.cu around the collective; no per-level allocation)."""

    def __init__(self, offsets, cols, rank, world_size, cache_pages, cuda_device=0, group=None, weights=None, **kw):
        self.n = offsets.numel() - 1
        self.rank, self.world, self.group = rank, world_size, group
        self.v0, self.v1 = shard_vertices_by_edges(offsets, world_size, rank)
        e0, e1 = int(offsets[self.v0].item()), int(offsets[self.v1].item())
        loc_off = (offsets[self.v0:self.v1 + 1] - e0).contiguous()
        loc_cols = cols[e0:e1].contiguous()
        loc_w = weights[e0:e1].contiguous() if weights is not None else None
        self.local = CsrGraph(loc_off, loc_cols, cache_pages, cuda_device=cuda_device, weights=loc_w, **kw)
        self.device = cuda_device
        self.degree = (offsets[1:] - offsets[:-1]).contiguous()       # replicated, like the labels

    def sssp(self, source):
        """Label-correcting SSSP: every rank relaxes the edges of its own vertices into its copy of
        the tentative costs, the copies are combined with an element-wise minimum (all-reduce), and
        the update step runs replicated.  Returns (u32 distances in an int32 tensor, sweeps, edges
        this rank scanned)."""
        import torch
        dev = self.torch_device
        cost = torch.full((self.n,), -1, dtype=torch.int32, device=dev)       # 0xFFFFFFFF
        cost[source] = 0
        new = cost.clone()
        label = torch.zeros(self.n, dtype=torch.uint8, device=dev)
        label[source] = 1
        scanned = torch.zeros(1, dtype=torch.int64, device=dev)
        sweeps = 0
        while True:
            self.local.sssp_sweep(0, self.v1 - self.v0, label, new, scanned, v_base=self.v0)
            self.local.ctrl.check_status()
            sweeps += 1
            allreduce_min_u32(new, self.group)
            better = u32_less(new, cost)
            if not bool(better.any()):
                break
            cost = torch.where(better, new, cost)
            label = better.to(torch.uint8)
        return cost, sweeps, int(scanned.item())

    def pagerank(self, alpha=(85, 100), tolerance_q=None, max_iters=100):
        """Fixed-point delta PageRank: every rank pushes the deltas of its own active vertices into a
        zeroed buffer, the buffers are summed over ranks (all-reduce) and added to the replicated
        residuals; the update step runs replicated.  Integer sums: the result does not depend on the
        number of ranks.  Returns (ranks as int64 fixed-point values, sweeps, edges this rank scanned)."""
        import torch
        import torch.distributed as dist
        dev = self.torch_device
        num, den = alpha
        one = 1 << PR_FRAC_BITS
        if tolerance_q is None:
            tolerance_q = one // 1000
        ratio = lambda x: x // den * num + (x % den) * num // den  # noqa: E731
        deg = self.degree
        degc = deg.clamp(min=1)
        zero = torch.zeros(self.n, dtype=torch.int64, device=dev)
        base = one - ratio(one)
        value = torch.full((self.n,), base, dtype=torch.int64, device=dev)
        delta = torch.where(deg > 0, torch.full_like(value, ratio(base)) // degc, zero)
        residual = zero.clone()
        label = torch.ones(self.n, dtype=torch.uint8, device=dev)
        scanned = torch.zeros(1, dtype=torch.int64, device=dev)
        sweeps = 0
        while sweeps < max_iters:
            push = torch.zeros(self.n, dtype=torch.int64, device=dev)
            self.local.pr_sweep(0, self.v1 - self.v0, label, delta, push, scanned, v_base=self.v0)
            self.local.ctrl.check_status()
            sweeps += 1
            dist.all_reduce(push, op=dist.ReduceOp.SUM, group=self.group)
            residual += push
            act = residual > tolerance_q
            if not bool(act.any()):
                break
            value = torch.where(act, value + residual, value)
            delta = torch.where(act, torch.where(deg > 0, ratio(residual) // degc, zero), delta)
            residual = torch.where(act, zero, residual)
            label = act.to(torch.uint8)
        return value, sweeps, int(scanned.item())

    @property
    def torch_device(self):
        return "cpu" if self.device is None else f"cuda:{self.device}"

    def close(self):
        self.local.close()

    def _buffers(self, kind):
        """Persistent exchange buffers, allocated at the first traversal of a kind: the send buffer the
        compaction kernel fills (and the collective reads in place), the receive buffer, the headers."""
        import torch
        buf = getattr(self, "_xbuf", None)
        if buf is None:
            buf = self._xbuf = {}
        if kind not in buf:
            dev, n, w = self.torch_device, self.n, self.world
            d = {"hdr": torch.zeros(2, dtype=torch.int64, device=dev), "hdrs": torch.zeros(2 * w, dtype=torch.int64, device=dev)}
            if kind == "bfs":
                d["send"] = torch.empty(n, dtype=torch.int32, device=dev)
                d["recv"] = torch.empty(n * w, dtype=torch.int32, device=dev)
            else:
                d["sparse_cap"] = max(1, int(n * self.CC_DENSE_FRACTION))
                d["send"] = torch.empty(n, dtype=torch.int64, device=dev)
                d["recv"] = torch.empty(min(n, d["sparse_cap"]) * w, dtype=torch.int64, device=dev)
                d["before"] = torch.empty(self.v1 - self.v0, dtype=torch.int64, device=dev)
            buf[kind] = d
        return buf[kind]

    # a sweep that changed more than CC_DENSE_FRACTION * n labels, summed over the ranks, is exchanged as
    # one element-wise MIN all-reduce of the replicas instead of (vertex, label) lists
    CC_DENSE_FRACTION = 0.25

    def bfs(self, source):
        """Level-synchronous BFS over the sharded graph.  Per level: the rank's fused level launch, the
        compaction of what it labelled into the send buffer, one all-gather of the headers (the only
        device-to-host read of the level: sizes, termination, failures), one all-gather of the frontier
        sized to the largest contribution, and the apply kernel.  Returns (levels, n_levels, edges this
        rank scanned)."""
        import torch
        import torch.distributed as dist
        dev = self.torch_device
        b = self._buffers("bfs")
        label = torch.full((self.n,), -1, dtype=torch.int32, device=dev)      # 0xFFFFFFFF
        label[source] = 0
        changed = torch.zeros(1, dtype=torch.int32, device=dev)
        scanned = torch.zeros(1, dtype=torch.int64, device=dev)
        level = 0
        while True:
            self.local.bfs_level(0, self.v1 - self.v0, level, label, changed, scanned, v_base=self.v0)
            self.local.frontier_compact(label, level + 1, b["send"], b["hdr"])
            counts, statuses = gather_headers(b["hdr"], b["hdrs"], self.group)
            raise_on_rank_failure(statuses)
            if sum(counts) == 0:
                break
            mx = max(counts)
            dist.all_gather_into_tensor(b["recv"][:mx * self.world], b["send"][:mx], group=self.group)
            self.local.frontier_apply(label, level + 1, b["recv"], mx, b["hdrs"], self.world, self.rank)
            level += 1
        return label, level + 1, int(scanned.item())

    def cc(self):
        """Label-propagation CC over the sharded graph.  Per sweep: the rank's fused sweep launch, the
        compaction of (vertex, label) for every label it lowered, one all-gather of the headers, then
        either the all-gather of the pairs + apply kernel, or -- when most labels changed -- one MIN
        all-reduce of the replicas + the kernel that flags the owned vertices whose label fell.
        Returns (labels, sweeps, edges this rank scanned)."""
        import torch
        import torch.distributed as dist
        dev = self.torch_device
        b = self._buffers("cc")
        comp = torch.arange(self.n, dtype=torch.int64, device=dev)
        curr = torch.ones(self.n, dtype=torch.uint8, device=dev)
        nxt = torch.zeros(self.n, dtype=torch.uint8, device=dev)
        changed = torch.zeros(1, dtype=torch.int32, device=dev)
        scanned = torch.zeros(1, dtype=torch.int64, device=dev)
        sweeps = 0
        self.cc_dense_sweeps = 0
        while True:
            self.local.cc_sweep(0, self.v1 - self.v0, comp, curr, nxt, changed, scanned, v_base=self.v0)
            sweeps += 1
            self.local.cc_compact(comp, nxt, b["send"], b["hdr"])
            counts, statuses = gather_headers(b["hdr"], b["hdrs"], self.group)
            raise_on_rank_failure(statuses)
            total = sum(counts)
            if total == 0:
                break
            if total > b["sparse_cap"]:
                b["before"].copy_(comp[self.v0:self.v1])
                dist.all_reduce(comp, op=dist.ReduceOp.MIN, group=self.group)
                self.local.cc_dense_flag(comp, b["before"], nxt, self.v0, self.v1)
                self.cc_dense_sweeps += 1
            else:
                mx = max(counts)
                dist.all_gather_into_tensor(b["recv"][:mx * self.world], b["send"][:mx], group=self.group)
                self.local.cc_apply(comp, nxt, self.v0, self.v1, b["recv"], mx, b["hdrs"], self.world, self.rank)
            curr.zero_()
            curr, nxt = nxt, curr
        return comp, sweeps, int(scanned.item())
