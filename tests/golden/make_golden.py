"""Regenerates tests/golden/golden.json from the CPU oracle.

The reference repository has no golden vectors for this path (no test-suite at all), and
neither its host library nor its kernels can run without /dev/libnvm* and a raw SSD, so these
fixtures come from the oracle, which is itself pinned by published known-answer vectors, by
independent numpy / scipy re-computations and by the reference's own code compiled for the host
(see tests/test_oracle.py).  Run from the repository root:  python tests/golden/make_golden.py
"""
import hashlib
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import pyoracle as orc  # noqa: E402


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def main():
    g = {}
    g["array_checksum"] = [
        {"store_seed": ss, "n_elems": n, "access_seed": a, "lanes": l, "reqs": r,
         "checksum": orc.array_checksum(ss, n, a, 0, l, r)}
        for (ss, n, a, l, r) in [(11, 1 << 16, 29, 512, 8), (7, 1 << 20, 99, 4096, 16), (1, 1 << 22, 2, 1 << 14, 64),
                                 (0xDEADBEEF, (1 << 20) + 12345, 5, 1000, 7), (3, 1 << 27, 4, 1 << 12, 64)]]
    g["page_crc"] = [{"store_seed": s, "page": p, "page_bytes": b, "crc": orc.page_crc(s, p, b)}
                     for (s, p, b) in [(11, 0, 4096), (11, 1, 4096), (11, 123456, 4096), (5, 7, 512), (5, 3, 8192)]]
    pages, crcs = orc.block_requests(11, 77, 1 << 13, 4096, 0, 256)
    g["block_requests"] = {"store_seed": 11, "req_seed": 77, "n_pages": 1 << 13, "page_bytes": 4096,
                           "pages_sha256": sha(pages), "crc_sha256": sha(crcs), "first_pages": pages[:8].tolist(),
                           "first_crcs": crcs[:8].tolist()}
    cdf = orc.zipf_cdf(1 << 12)
    idx = orc.zipf_indices(cdf, 1 << 12, 512, 17, 23, 0, 64, 16)
    g["zipf"] = {"n_pages": 1 << 12, "s": 0.99, "perm_seed": 17, "access_seed": 23, "lanes": 64, "reqs": 16,
                 "cdf_sha256": sha(cdf), "idx_sha256": sha(idx), "first_idx": idx[:8].tolist(),
                 "checksum": orc.indexed_checksum(9, 0, idx)}
    graphs = []
    for scale, seed in [(8, 1), (10, 2), (12, 3)]:
        off, cols = orc.rmat_csr(seed, scale, 16)
        src = orc.max_degree_vertex(off)
        lvl, scanned = orc.bfs(off, cols, src)
        lab, comps = orc.cc(off, cols)
        wts = orc.edge_weights(seed + 100, len(cols))
        dist = orc.sssp(off, cols, wts, src)
        rank, pr_iters, pr_scanned = orc.pagerank(off, cols)
        graphs.append({"weight_seed": seed + 100, "weights_sha256": sha(wts), "dist_sha256": sha(dist),
                       "max_dist": int(dist[dist != 0xFFFFFFFF].max()),
                       "rank_sha256": sha(rank), "pr_sweeps": int(pr_iters), "pr_edges_scanned": int(pr_scanned),
                       "rank_sum_q40": int(rank.sum(dtype=np.uint64)),"scale": scale, "seed": seed, "edge_factor": 16, "directed_edges": int(len(cols)),
                       "offsets_sha256": sha(off), "cols_sha256": sha(cols), "source": int(src),
                       "levels_sha256": sha(lvl), "max_level": int(lvl[lvl != 0xFFFFFFFF].max()),
                       "reached": int((lvl != 0xFFFFFFFF).sum()), "edges_scanned": int(scanned),
                       "labels_sha256": sha(lab), "components": int(comps)})
    g["graphs"] = graphs
    with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden.json"), "w") as f:
        json.dump(g, f, indent=1)
    print("wrote golden.json")


if __name__ == "__main__":
    main()
