"""Multi-GPU tests (need at least two GPUs; skipped otherwise): sharded array scan with the NCCL
reduction of the checksums, BFS / CC sharded by vertex range with the all-gather exchange, SSSP /
PageRank with the all-reduce exchange.
Results must be bit-identical to the single-rank oracle on every rank."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    import bam_b200
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    # --- sharded skewed scan ---
    n_pages_total, lanes, reqs, seed = 1 << 14, 1 << 12, 16, 9
    first, n_local = bam_b200.shard_pages(n_pages_total, world, rank)
    ctrl = bam_b200.Controller(n_local * 4096, rank, queue_depth=64, num_queues=8)
    ctrl.fill_store(seed, first_elem=first * 512)
    cache = bam_b200.PageCache(ctrl, 4096, n_local // 4)
    arr = bam_b200.Array(cache, n_local * 512)
    cdf = bam_b200.zipf_cdf(n_local)
    d_cdf = torch.from_numpy(cdf.view(np.int64)).to(dev)
    d_idx = torch.zeros(lanes * reqs, dtype=torch.int64, device=dev)
    bam_b200.gen_zipf_indices(d_idx, lanes, reqs, 23 + rank, d_cdf, n_local, 512, 17 + rank)
    out = torch.zeros(1, dtype=torch.int64, device=dev)
    arr.read(lanes, reqs, out, idx=d_idx)
    ctrl.check_status()
    local_sum = int(out.item())
    dist.all_reduce(out, op=dist.ReduceOp.SUM)
    scan = (rank, local_sum & ((1 << 64) - 1), int(out.item()) & ((1 << 64) - 1),
            (d_idx + first * 512).cpu().numpy().view(np.uint64))
    arr.close(); cache.close(); ctrl.close()
    # --- sharded BFS / CC ---
    off, cols = bam_b200.build_rmat_csr(3, 12, 16, device=dev)
    src = int(torch.argmax(off[1:] - off[:-1]).item())
    g = bam_b200.DistCsrGraph(off, cols, rank, world, cache_pages=1024, cuda_device=rank, queue_depth=64, num_queues=8)
    lv, n_levels, scanned = g.bfs(src)
    lab, sweeps, _ = g.cc()
    audit = g.local.cache.audit()
    g.close()
    # --- sharded SSSP / PageRank (dense exchange: all-reduce min / sum) ---
    from oracle import pyoracle as orc
    wts = torch.from_numpy(orc.edge_weights(41, cols.numel()).view(np.int32)).to(dev)
    gw = bam_b200.DistCsrGraph(off, cols, rank, world, cache_pages=1024, cuda_device=rank, queue_depth=64, num_queues=8,
                               weights=wts)
    dist_, s_sweeps, _ = gw.sssp(src)
    rank_, pr_sweeps, _ = gw.pagerank()
    audit += gw.local.cache.audit()
    q.put((scan, lv.cpu().numpy().view(np.uint32), lab.cpu().numpy().view(np.uint64), n_levels, scanned, audit,
           dist_.cpu().numpy().view(np.uint32), rank_.cpu().numpy().view(np.uint64), pr_sweeps))
    gw.close()
    dist.barrier()
    dist.destroy_process_group()


def test_two_gpu_scan_bfs_cc():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    sys.path.insert(0, ROOT)
    from oracle import pyoracle as orc
    world, port = 2, 29581
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=600) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    # scan: every rank's local sum equals the oracle on its shard, the reduction equals the global oracle
    total = 0
    for (rank, local_sum, reduced, gidx), *_ in res:
        assert local_sum == orc.indexed_checksum(9, 0, gidx)
        total = (total + local_sum) & ((1 << 64) - 1)
    assert all(r[0][2] == total for r in res)
    off, cols = orc.rmat_csr(3, 12, 16)
    want_lv, want_scanned = orc.bfs(off, cols, orc.max_degree_vertex(off))
    want_lab, _ = orc.cc(off, cols)
    want_dist = orc.sssp(off, cols, orc.edge_weights(41, len(cols)), orc.max_degree_vertex(off))
    want_rank, want_pr_sweeps, _ = orc.pagerank(off, cols)
    for _, lv, lab, n_levels, scanned, audit, dist_, rank_, pr_sweeps in res:
        assert (lv == want_lv).all() and (lab == want_lab).all() and audit == 0
        assert (dist_ == want_dist).all() and (rank_ == want_rank).all() and pr_sweeps == want_pr_sweeps
    assert sum(r[4] for r in res) == want_scanned
