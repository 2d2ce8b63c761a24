"""GPU parity tests of the graph consumers: BFS levels and CC labels, bit-exact against the CPU
oracle and the committed golden fixtures, with offsets and edges read only through bam::array."""
import hashlib
import json
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
GOLDEN = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "golden.json")))


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


@pytest.mark.parametrize("gi", [0, 1, 2])
def test_rmat_csr_bfs_cc_golden(cuda, bam, gi):
    g = GOLDEN["graphs"][gi]
    off, cols = bam.build_rmat_csr(g["seed"], g["scale"], g["edge_factor"])
    assert sha(off.cpu().numpy().view(np.uint64)) == g["offsets_sha256"]
    assert sha(cols.cpu().numpy().view(np.uint64)) == g["cols_sha256"]
    gr = bam.CsrGraph(off, cols, cache_pages=2048, queue_depth=64, num_queues=8)
    levels, n_levels, scanned = gr.bfs(g["source"])
    assert gr.ctrl.status() == (0, "none", 0) and gr.cache.audit() == 0
    lv = levels.cpu().numpy().view(np.uint32)
    assert sha(lv) == g["levels_sha256"]
    assert scanned == g["edges_scanned"] and n_levels == g["max_level"] + 1
    labels, sweeps, _ = gr.cc()
    assert gr.ctrl.status() == (0, "none", 0) and gr.cache.audit() == 0
    assert sha(labels.cpu().numpy().view(np.uint64)) == g["labels_sha256"]
    assert sweeps >= 1
    gr.close()


def test_bfs_cc_scale16_vs_oracle_small_cache(cuda, bam, orc):
    """A graph several times larger than the cache: edges are re-read through evictions."""
    scale, seed = 16, 5
    off_o, cols_o = orc.rmat_csr(seed, scale, 16)
    off, cols = bam.build_rmat_csr(seed, scale, 16)
    assert (off.cpu().numpy().view(np.uint64) == off_o).all() and (cols.cpu().numpy().view(np.uint64) == cols_o).all()
    n_pages = (len(cols_o) * 8 + len(off_o) * 8) // 4096
    gr = bam.CsrGraph(off, cols, cache_pages=max(15000, n_pages // 4), queue_depth=256, num_queues=32)
    src = orc.max_degree_vertex(off_o)
    want_lv, want_scanned = orc.bfs(off_o, cols_o, src)
    levels, n_levels, scanned = gr.bfs(src)
    assert gr.ctrl.status() == (0, "none", 0)
    lv = levels.cpu().numpy().view(np.uint32)
    assert (lv == want_lv).all() and scanned == want_scanned
    # structural invariants of any BFS: source at 0, every edge spans at most one level
    assert lv[src] == 0
    srcs = np.repeat(np.arange(len(off_o) - 1), np.diff(off_o.astype(np.int64)))
    reach = lv[srcs] != 0xFFFFFFFF
    assert (np.abs(lv[srcs][reach].astype(np.int64) - lv[cols_o.astype(np.int64)][reach].astype(np.int64)) <= 1).all()
    want_lab, comps = orc.cc(off_o, cols_o)
    labels, sweeps, _ = gr.cc()
    assert gr.ctrl.status() == (0, "none", 0) and gr.cache.audit() == 0
    lab = labels.cpu().numpy().view(np.uint64)
    assert (lab == want_lab).all()
    assert (lab <= np.arange(len(lab), dtype=np.uint64)).all() and (lab[lab.astype(np.int64)] == lab).all()
    assert len(np.unique(lab)) == comps
    st = gr.cache.stats()
    assert st["read_ios"] > n_pages // 2
    gr.close()


def test_bfs_isolated_source_and_tiny_graph(cuda, bam, orc):
    import torch
    # 6 vertices: path 0-1-2, edge 3-4, vertex 5 isolated
    off = torch.tensor([0, 1, 3, 4, 5, 6, 6], dtype=torch.int64, device="cuda")
    cols = torch.tensor([1, 0, 2, 1, 4, 3], dtype=torch.int64, device="cuda")
    gr = bam.CsrGraph(off, cols, cache_pages=8, queue_depth=4, num_queues=1, ctrl_blocks=1)
    gr.ctrl.set_max_grid(3)
    lv, n_levels, scanned = gr.bfs(5)                       # isolated source: one level, nothing scanned
    assert lv.cpu().numpy().view(np.uint32).tolist() == [0xFFFFFFFF] * 5 + [0] and n_levels == 1 and scanned == 0
    lv, n_levels, scanned = gr.bfs(0)
    assert lv.cpu().numpy().view(np.uint32).tolist() == [0, 1, 2, 0xFFFFFFFF, 0xFFFFFFFF, 0xFFFFFFFF]
    assert n_levels == 3 and scanned == 4
    lab, _, _ = gr.cc()
    assert lab.cpu().numpy().tolist() == [0, 0, 0, 3, 3, 5]
    assert gr.ctrl.status() == (0, "none", 0)
    gr.close()
