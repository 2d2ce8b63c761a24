"""world_size-2 gloo test (CPU) of the multi-GPU sharding logic: the store is sharded by page
range, every rank scans only its shard, and the wrapping sum of the per-rank checksums equals
the single-rank checksum of the whole store's access stream.  No data-path collective exists;
the only exchange is the final reduction."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    from oracle import pyoracle as orc
    import bam_b200
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    n_pages_total, lanes, reqs, seed = 1 << 10, 128, 8, 9
    first_page, n_local = bam_b200.shard_pages(n_pages_total, world, rank)
    cdf = bam_b200.zipf_cdf(n_local)
    idx = orc.zipf_indices(cdf, n_local, 512, 17 + rank, 23 + rank, 0, lanes, reqs)     # indices inside the shard
    local = orc.indexed_checksum(seed, first_page * 512, idx)
    # int64 carries the u64 bit pattern; wrapping addition is the same in both
    t = torch.tensor([np.uint64(local).astype(np.int64)], dtype=torch.int64)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    glob_idx = idx + np.uint64(first_page * 512)
    q.put((rank, int(t.item()) & ((1 << 64) - 1), local, glob_idx))
    dist.barrier()
    dist.destroy_process_group()


def test_sharded_checksum_reduces_to_global():
    world, port = 2, 29571
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    sys.path.insert(0, ROOT)
    from oracle import pyoracle as orc
    total = sum(r[2] for r in res) & ((1 << 64) - 1)
    assert all(r[1] == total for r in res)                      # every rank holds the reduced sum
    all_idx = np.concatenate([r[3] for r in sorted(res, key=lambda r: r[0])])
    assert orc.indexed_checksum(9, 0, all_idx) == total         # equals the unsharded computation


def _graph_worker(rank, world, port, q):
    """Distributed BFS and CC: the product's host loops (DistCsrGraph.bfs / .cc: persistent buffers,
    header all-gather, sized payload all-gather, sparse or dense CC exchange, termination) over gloo;
    the level / sweep kernel and the compaction / apply kernels are played by numpy on the rank's
    vertex range (the CUDA kernels themselves are covered by the GPU tests)."""
    sys.path.insert(0, ROOT)
    from oracle import pyoracle as orc
    import bam_b200
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    off, cols = orc.rmat_csr(2, 10, 16)
    n = len(off) - 1
    g = bam_b200.DistCsrGraph.__new__(bam_b200.DistCsrGraph)
    g.n, g.rank, g.world, g.group, g.device = n, rank, world, None, None
    g.v0, g.v1 = bam_b200.shard_vertices(n, world, rank)
    g.local = _HostShard(off, cols, None)
    src = int(orc.max_degree_vertex(off))
    label, n_levels, _ = g.bfs(src)
    out = [rank, label.numpy().view(np.uint32).copy(), n_levels]
    for fraction in (0.25, float(world)):        # the default mix of dense and sparse sweeps, then sparse only
        g.CC_DENSE_FRACTION = fraction
        g._xbuf.pop("cc", None)
        comp, sweeps, _ = g.cc()
        out += [comp.numpy().view(np.uint64).copy(), sweeps, g.cc_dense_sweeps]
    q.put(tuple(out))
    dist.barrier()
    dist.destroy_process_group()


def test_distributed_bfs_cc_exchange_matches_oracle():
    world, port = 2, 29573
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_graph_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    sys.path.insert(0, ROOT)
    from oracle import pyoracle as orc
    off, cols = orc.rmat_csr(2, 10, 16)
    want_lv, _ = orc.bfs(off, cols, orc.max_degree_vertex(off))
    want_lab, _ = orc.cc(off, cols)
    for _, lv, n_levels, lab_a, sweeps_a, dense_a, lab_b, sweeps_b, dense_b in res:    # every replica ends bit-identical to the oracle
        assert (lv == want_lv).all() and (lab_a == want_lab).all() and (lab_b == want_lab).all()
        assert n_levels == int(want_lv[want_lv != 0xFFFFFFFF].max()) + 1 and sweeps_a >= 1 and sweeps_b >= 1
        assert dense_a >= 1 and dense_a < sweeps_a          # the first sweep changes most labels, the last ones few
        assert dense_b == 0


class _HostShard:
    """Stands in for the rank's CsrGraph: the sweeps of the CUDA kernels restated with numpy on the
    rank's rows (local vertex v = global vertex v_base + v)."""

    class _Ctrl:
        def check_status(self):
            pass

    def __init__(self, off, cols, wts):
        self.off, self.cols, self.wts, self.ctrl = off.astype(np.int64), cols.astype(np.int64), wts, self._Ctrl()

    def bfs_level(self, v_begin, v_end, level, label, changed, scanned, v_base=0):
        lab = label.numpy()
        for u in np.flatnonzero(lab[v_base + v_begin:v_base + v_end] == level) + v_base + v_begin:
            nb = self.cols[self.off[u]:self.off[u + 1]]
            lab[nb[lab[nb] == -1]] = level + 1

    def cc_sweep(self, v_begin, v_end, comp, curr_visit, next_visit, changed, scanned, v_base=0):
        c, nv = comp.numpy(), next_visit.numpy()
        for u in np.flatnonzero(curr_visit.numpy()[v_base + v_begin:v_base + v_end]) + v_base + v_begin:
            for w in self.cols[self.off[u]:self.off[u + 1]]:
                if c[u] < c[w]:
                    c[w] = c[u]; nv[w] = 1
                elif c[w] < c[u]:
                    c[u] = c[w]; nv[u] = 1

    # the exchange kernels of bam_exchange.cu, restated
    def frontier_compact(self, label, level_value, out, hdr):
        idx = np.flatnonzero(label.numpy() == level_value)
        out.numpy()[:len(idx)] = idx
        hdr[0], hdr[1] = len(idx), 0

    def frontier_apply(self, label, level_value, recv, stride, hdrs, world, rank):
        lab, h = label.numpy(), hdrs.tolist()
        for r in range(world):
            if r != rank:
                v = recv.numpy()[r * stride:r * stride + h[2 * r]]
                lab[v[lab[v] == -1]] = level_value

    def cc_compact(self, comp, next_visit, out, hdr):
        idx = np.flatnonzero(next_visit.numpy())
        out.numpy()[:len(idx)] = (idx.astype(np.int64) << 32) | comp.numpy()[idx]
        hdr[0], hdr[1] = len(idx), 0

    def cc_apply(self, comp, next_visit, own_begin, own_end, recv, stride, hdrs, world, rank):
        c, nv, h = comp.numpy(), next_visit.numpy(), hdrs.tolist()
        for r in range(world):
            if r == rank:
                continue
            for e in recv.numpy()[r * stride:r * stride + h[2 * r]]:
                v, lab = int(e) >> 32, int(e) & 0xFFFFFFFF
                if lab < c[v]:
                    c[v] = lab
                    if own_begin <= v < own_end:
                        nv[v] = 1

    def cc_dense_flag(self, comp, before_own, next_visit, own_begin, own_end):
        next_visit.numpy()[own_begin:own_end][comp.numpy()[own_begin:own_end] < before_own.numpy()] = 1

    def sssp_sweep(self, v_begin, v_end, label, new_cost, scanned, v_base=0):
        lab, nc = label.numpy(), new_cost.numpy().view(np.uint32)
        for v in range(v_begin, v_end):
            u = v_base + v
            if lab[u]:
                lab[u] = 0
                e0, e1 = self.off[u], self.off[u + 1]
                scanned += int(e1 - e0)
                cand = nc[u] + self.wts[e0:e1]
                np.minimum.at(nc, self.cols[e0:e1], cand)

    def pr_sweep(self, v_begin, v_end, label, delta, residual, scanned, v_base=0):
        lab, dl, res = label.numpy(), delta.numpy(), residual.numpy()
        for v in range(v_begin, v_end):
            u = v_base + v
            if lab[u]:
                lab[u] = 0
                e0, e1 = self.off[u], self.off[u + 1]
                scanned += int(e1 - e0)
                np.add.at(res, self.cols[e0:e1], dl[u])


def _rank_worker(rank, world, port, q):
    """Distributed SSSP and PageRank: the product's host loops and exchanges (DistCsrGraph.sssp /
    .pagerank) over gloo, with the per-sweep kernel played by numpy."""
    sys.path.insert(0, ROOT)
    from oracle import pyoracle as orc
    import bam_b200
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    off, cols = orc.rmat_csr(2, 9, 16)
    wts = orc.edge_weights(55, len(cols))
    n = len(off) - 1
    g = bam_b200.DistCsrGraph.__new__(bam_b200.DistCsrGraph)
    g.n, g.rank, g.world, g.group, g.device = n, rank, world, None, None
    t_off = torch.from_numpy(off.view(np.int64))
    g.v0, g.v1 = bam_b200.shard_vertices_by_edges(t_off, world, rank)
    g.degree = (t_off[1:] - t_off[:-1]).contiguous()
    g.local = _HostShard(off, cols, wts)
    src = int(orc.max_degree_vertex(off))
    cost, sweeps, _ = g.sssp(src)
    value, pr_sweeps, _ = g.pagerank()
    # the unsigned minimum must treat 0xFFFFFFFF as the largest value
    t = torch.tensor([-1, 5, -2147483648] if rank == 0 else [7, -1, 3], dtype=torch.int32)
    bam_b200.allreduce_min_u32(t)
    q.put((rank, cost.numpy().view(np.uint32).copy(), sweeps, value.numpy().view(np.uint64).copy(), pr_sweeps, t.tolist()))
    dist.barrier()
    dist.destroy_process_group()


def test_distributed_sssp_pagerank_match_oracle():
    world, port = 2, 29577
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    sys.path.insert(0, ROOT)
    from oracle import pyoracle as orc
    off, cols = orc.rmat_csr(2, 9, 16)
    wts = orc.edge_weights(55, len(cols))
    want = orc.sssp(off, cols, wts, int(orc.max_degree_vertex(off)))
    want_rank, want_sweeps, _ = orc.pagerank(off, cols)
    for _, cost, sweeps, value, pr_sweeps, t in res:
        assert (cost == want).all() and sweeps >= 2
        assert (value == want_rank).all() and pr_sweeps == want_sweeps
        assert t == [7, 5, 3]

