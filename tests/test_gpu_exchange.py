"""The exchange kernels of the sharded traversals (bam_launch_frontier_compact / _apply,
bam_launch_cc_compact / _apply / _dense_flag) on ONE GPU: the ranks of a 3-way sharded graph are run
one after the other in this process, each with its own shard (store, cache, queues) and its own
replica of the labels, and the collectives between the kernels are played by plain copies.  None of
these kernels waits for another, so running the ranks in turn is the same computation.
BFS levels and CC labels of every replica must equal the oracle's bit for bit."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

WORLD = 3


def _shards(bam, torch, scale, seed):
    off, cols = bam.build_rmat_csr(seed, scale, 16, device="cuda")
    shards = [bam.DistCsrGraph(off, cols, r, WORLD, cache_pages=512, cuda_device=0, queue_depth=64, num_queues=8)
              for r in range(WORLD)]
    return off, cols, shards


def _gather(torch, bufs, key, mx):
    """What all_gather_into_tensor does: every rank's first mx entries, rank after rank, in every recv buffer."""
    for b in bufs:
        for r, src in enumerate(bufs):
            b["recv"][r * mx:(r + 1) * mx].copy_(src[key][:mx])


def _headers(torch, bufs):
    hdrs = torch.cat([b["hdr"] for b in bufs])
    for b in bufs:
        b["hdrs"].copy_(hdrs)
    h = hdrs.tolist()
    return h[0::2], h[1::2]


def test_sharded_bfs_through_exchange_kernels(bam, cuda, orc):
    torch = cuda
    off, cols, shards = _shards(bam, torch, 12, 3)
    n = off.numel() - 1
    src = int(torch.argmax(off[1:] - off[:-1]).item())
    bufs = [g._buffers("bfs") for g in shards]
    labels = [torch.full((n,), -1, dtype=torch.int32, device="cuda") for _ in shards]
    for lab in labels:
        lab[src] = 0
    changed = torch.zeros(1, dtype=torch.int32, device="cuda")
    scanned = torch.zeros(1, dtype=torch.int64, device="cuda")
    level = 0
    while True:
        for g, lab, b in zip(shards, labels, bufs):
            g.local.bfs_level(0, g.v1 - g.v0, level, lab, changed, scanned, v_base=g.v0)
            g.local.frontier_compact(lab, level + 1, b["send"], b["hdr"])
        counts, statuses = _headers(torch, bufs)
        assert not any(statuses)
        if sum(counts) == 0:
            break
        mx = max(counts)
        _gather(torch, bufs, "send", mx)
        for g, lab, b in zip(shards, labels, bufs):
            g.local.frontier_apply(lab, level + 1, b["recv"], mx, b["hdrs"], WORLD, g.rank)
        level += 1
        assert level < 64
    torch.cuda.synchronize()
    o, c = orc.rmat_csr(3, 12, 16)
    want, want_scanned = orc.bfs(o, c, orc.max_degree_vertex(o))
    for g, lab in zip(shards, labels):
        g.local.ctrl.check_status()
        assert (lab.cpu().numpy().view(np.uint32) == want).all()
        assert g.local.cache.audit() == 0
    assert int(scanned.item()) == want_scanned and level + 1 == int(want[want != 0xFFFFFFFF].max()) + 1
    for g in shards:
        g.close()


@pytest.mark.parametrize("dense_fraction", [0.25, 3.0])
def test_sharded_cc_through_exchange_kernels(bam, cuda, orc, dense_fraction):
    """dense_fraction 0.25: the first sweeps go through the MIN reduction + flag kernel, the last through
    (vertex, label) pairs; 3.0 (= the number of ranks): pairs only."""
    torch = cuda
    off, cols, shards = _shards(bam, torch, 12, 5)
    n = off.numel() - 1
    for g in shards:
        g.CC_DENSE_FRACTION = dense_fraction
    bufs = [g._buffers("cc") for g in shards]
    comps = [torch.arange(n, dtype=torch.int64, device="cuda") for _ in shards]
    curr = [torch.ones(n, dtype=torch.uint8, device="cuda") for _ in shards]
    nxt = [torch.zeros(n, dtype=torch.uint8, device="cuda") for _ in shards]
    changed = torch.zeros(1, dtype=torch.int32, device="cuda")
    scanned = torch.zeros(1, dtype=torch.int64, device="cuda")
    sweeps = dense = 0
    while True:
        for k, g in enumerate(shards):
            g.local.cc_sweep(0, g.v1 - g.v0, comps[k], curr[k], nxt[k], changed, scanned, v_base=g.v0)
            g.local.cc_compact(comps[k], nxt[k], bufs[k]["send"], bufs[k]["hdr"])
        sweeps += 1
        counts, statuses = _headers(torch, bufs)
        assert not any(statuses)
        total = sum(counts)
        # the header counts the flagged vertices, and every pair carries its vertex's current label
        for k in range(WORLD):
            flagged = torch.nonzero(nxt[k]).flatten()
            assert counts[k] == flagged.numel()
            pairs = bufs[k]["send"][:counts[k]]
            assert bool((torch.sort(pairs >> 32).values == flagged).all())
            assert bool(((pairs & 0xFFFFFFFF) == comps[k][pairs >> 32]).all())
        if total == 0:
            break
        if total > bufs[0]["sparse_cap"]:
            for k, g in enumerate(shards):
                bufs[k]["before"].copy_(comps[k][g.v0:g.v1])
            low = torch.stack(comps).min(dim=0).values                   # the MIN all-reduce
            for k, g in enumerate(shards):
                comps[k].copy_(low)
                g.local.cc_dense_flag(comps[k], bufs[k]["before"], nxt[k], g.v0, g.v1)
            dense += 1
        else:
            mx = max(counts)
            _gather(torch, bufs, "send", mx)
            for k, g in enumerate(shards):
                g.local.cc_apply(comps[k], nxt[k], g.v0, g.v1, bufs[k]["recv"], mx, bufs[k]["hdrs"], WORLD, g.rank)
        for k in range(WORLD):
            curr[k].zero_()
            curr[k], nxt[k] = nxt[k], curr[k]
        assert sweeps < 64
    torch.cuda.synchronize()
    o, c = orc.rmat_csr(5, 12, 16)
    want, _ = orc.cc(o, c)
    for g, comp in zip(shards, comps):
        g.local.ctrl.check_status()
        assert (comp.cpu().numpy().view(np.uint64) == want).all()
        assert g.local.cache.audit() == 0
    assert (dense >= 1 and dense < sweeps) if dense_fraction < 1 else dense == 0
    for g in shards:
        g.close()


def test_exchange_headers_carry_the_status_and_reject_bad_arguments(bam, cuda):
    """The compaction kernel copies the status code of its cache's controller into the header (here: a code
    left by an injected NVMe error status), which is how every rank learns that one of them failed."""
    import ctypes as C
    torch = cuda
    ctrl = bam.Controller(1 << 22, 0, queue_depth=64, num_queues=1)
    ctrl.configure(ctrl_blocks=1, spin_timeout_ns=200_000_000)
    ctrl.set_max_grid(3)
    ctrl.fill_store(1)
    cache = bam.PageCache(ctrl, 4096, 1 << 10)
    arr = bam.Array(cache, 1 << 19)
    lib = ctrl.lib
    label = torch.full((1000,), -1, dtype=torch.int32, device="cuda")
    label[5], label[77], label[999] = 4, 4, 4
    out = torch.zeros(1000, dtype=torch.int32, device="cuda")
    hdr = torch.zeros(2, dtype=torch.int64, device="cuda")
    p = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
    assert lib.bam_launch_frontier_compact(cache.h, p(label), 1000, 4, p(out), 1000, p(hdr), None) == 0
    assert hdr.tolist() == [3, 0] and sorted(out[:3].tolist()) == [5, 77, 999]
    ctrl.inject_fault(bam.host.FAULT_STATUS, nth=3, status=0x281)
    s = torch.zeros(1, dtype=torch.int64, device="cuda")
    arr.read(256, 4, s, access_seed=3)
    assert lib.bam_launch_frontier_compact(cache.h, p(label), 1000, 4, p(out), 1000, p(hdr), None) == 0
    assert hdr.tolist()[0] == 3 and hdr.tolist()[1] != 0
    with pytest.raises(bam.BamError):
        bam.raise_on_rank_failure([0, hdr.tolist()[1]])
    code, where, _ = ctrl.status(clear=True)
    assert code != 0 and where == "nvme_status"
    assert lib.bam_launch_frontier_compact(cache.h, None, 1000, 4, p(out), 1000, p(hdr), None) == 22
    assert lib.bam_launch_frontier_apply(p(label), 1000, 4, p(out), 10, p(hdr), 2, 2, None) == 22      # rank outside the world
    assert lib.bam_launch_cc_compact(cache.h, p(hdr), p(out), (1 << 32) + 1, p(hdr), 1, p(hdr), None) == 22
    ctrl.inject_fault(bam.host.FAULT_NONE)
    ctrl.reset_queues()
    arr.close(); cache.close(); ctrl.close()
