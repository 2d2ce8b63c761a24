"""GPU parity tests of the weighted and ranking consumers: single-source shortest paths (bit-exact
against the oracle's Dijkstra) and fixed-point PageRank (bit-exact against the oracle's sequential
sweeps), with offsets, edges and weights read only through bam::array."""
import hashlib
import json
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
GOLDEN = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "golden.json")))


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def weights_tensor(cuda, orc, seed, m):
    return cuda.from_numpy(orc.edge_weights(seed, m).view(np.int32)).cuda()


@pytest.mark.parametrize("gi", [0, 1, 2])
def test_sssp_pagerank_golden(cuda, bam, orc, gi):
    g = GOLDEN["graphs"][gi]
    off, cols = bam.build_rmat_csr(g["seed"], g["scale"], g["edge_factor"])
    gr = bam.CsrGraph(off, cols, cache_pages=2048, queue_depth=64, num_queues=8,
                      weights=weights_tensor(cuda, orc, g["weight_seed"], cols.numel()))
    dist, sweeps, scanned = gr.sssp(g["source"])
    assert gr.ctrl.status() == (0, "none", 0) and gr.cache.audit() == 0
    d = dist.cpu().numpy().view(np.uint32)
    assert sha(d) == g["dist_sha256"] and int(d[d != 0xFFFFFFFF].max()) == g["max_dist"]
    assert sweeps >= 2 and scanned >= g["edges_scanned"]
    rank, pr_sweeps, pr_scanned = gr.pagerank()
    assert gr.ctrl.status() == (0, "none", 0) and gr.cache.audit() == 0
    r = rank.cpu().numpy().view(np.uint64)
    assert sha(r) == g["rank_sha256"]
    assert pr_sweeps == g["pr_sweeps"] and pr_scanned == g["pr_edges_scanned"]
    assert int(r.sum(dtype=np.uint64)) == g["rank_sum_q40"]
    gr.close()


def test_sssp_pagerank_scale15_small_cache(cuda, bam, orc):
    """A graph several times larger than the cache (evictions all the time), hubs cut into work items."""
    scale, seed = 15, 12
    off_o, cols_o = orc.rmat_csr(seed, scale, 16)
    off, cols = bam.build_rmat_csr(seed, scale, 16)
    wts = orc.edge_weights(77, len(cols_o))
    n_pages = (len(cols_o) * 12 + len(off_o) * 8) // 4096
    gr = bam.CsrGraph(off, cols, cache_pages=max(20000, n_pages // 3), queue_depth=256, num_queues=32,
                      weights=cuda.from_numpy(wts.view(np.int32)).cuda())
    src = orc.max_degree_vertex(off_o)
    assert off_o[src + 1] - off_o[src] > 2048                   # the source is a heavy vertex
    want = orc.sssp(off_o, cols_o, wts, src)
    dist, sweeps, _ = gr.sssp(src)
    assert gr.ctrl.status() == (0, "none", 0) and gr.cache.audit() == 0
    d = dist.cpu().numpy().view(np.uint32)
    assert (d == want).all()
    # triangle inequality over every edge out of a reached vertex: dist[v] <= dist[u] + w(u, v)
    srcs = np.repeat(np.arange(len(off_o) - 1), np.diff(off_o.astype(np.int64)))
    reach = d[srcs] != 0xFFFFFFFF
    assert (d[cols_o.astype(np.int64)][reach].astype(np.int64) <= d[srcs][reach].astype(np.int64) + wts[reach]).all()
    assert d[src] == 0
    # a second source, from a cache that already holds part of the graph
    want2 = orc.sssp(off_o, cols_o, wts, 1)
    d2, _, _ = gr.sssp(1)
    assert (d2.cpu().numpy().view(np.uint32) == want2).all()
    want_rank, want_sweeps, want_scanned = orc.pagerank(off_o, cols_o)
    rank, pr_sweeps, pr_scanned = gr.pagerank()
    assert gr.ctrl.status() == (0, "none", 0) and gr.cache.audit() == 0
    assert (rank.cpu().numpy().view(np.uint64) == want_rank).all()
    assert pr_sweeps == want_sweeps and pr_scanned == want_scanned
    # a different damping factor and a tight tolerance, cut off by max_iters
    want_rank, want_sweeps, _ = orc.pagerank(off_o, cols_o, alpha=(1, 2), tolerance_q=1 << 10, max_iters=7)
    rank, pr_sweeps, _ = gr.pagerank(alpha=(1, 2), tolerance_q=1 << 10, max_iters=7)
    assert pr_sweeps == want_sweeps == 7 and (rank.cpu().numpy().view(np.uint64) == want_rank).all()
    gr.close()


def test_sssp_edge_cases(cuda, bam, orc):
    # path 0 -> 1 -> 2 with a costly shortcut 0 -> 2, an unreachable vertex 3, an isolated source 4
    off = np.array([0, 2, 3, 3, 3, 3], dtype=np.uint64)
    cols = np.array([1, 2, 2], dtype=np.uint64)
    wts = np.array([5, 100, 7], dtype=np.uint32)
    gr = bam.CsrGraph(cuda.from_numpy(off.view(np.int64)).cuda(), cuda.from_numpy(cols.view(np.int64)).cuda(), cache_pages=64,
                      queue_depth=16, num_queues=2, weights=cuda.from_numpy(wts.view(np.int32)).cuda())
    d, sweeps, _ = gr.sssp(0)
    assert d.cpu().numpy().view(np.uint32).tolist() == [0, 5, 12, 0xFFFFFFFF, 0xFFFFFFFF] and sweeps == 3
    assert (d.cpu().numpy().view(np.uint32) == orc.sssp(off, cols, wts, 0)).all()
    d, sweeps, scanned = gr.sssp(4)
    assert d.cpu().numpy().view(np.uint32).tolist() == [0xFFFFFFFF] * 4 + [0] and sweeps == 1 and scanned == 0
    rank, pr_sweeps, _ = gr.pagerank()
    want, want_sweeps, _ = orc.pagerank(off, cols)
    assert (rank.cpu().numpy().view(np.uint64) == want).all() and pr_sweeps == want_sweeps
    assert gr.ctrl.status() == (0, "none", 0) and gr.cache.audit() == 0
    gr.close()
