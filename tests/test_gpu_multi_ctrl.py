"""GPU tests of a page cache in front of several controllers: replicated and striped ranges
(data_dist_t, include/page_cache.h:42, :558-582 of the reference), reads, write-back, flush,
fault reporting and graph traversal.  Expected values come from the oracle and from numpy."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
SEC = 1_000_000_000
M64 = (1 << 64) - 1


def np_splitmix64(x):
    x = x + np.uint64(0x9E3779B97F4A7C15)
    z = (x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def make_ctrls(bam, n, store_bytes, **kw):
    ctrls = [bam.Controller(store_bytes, 0, **kw) for _ in range(n)]
    for c in ctrls:
        c.configure(spin_timeout_ns=5 * SEC)
    return ctrls


def scatter_striped(ctrls, logical, page_words=512):
    """Deal the pages of the logical store round-robin onto the controllers' media."""
    n = len(ctrls)
    pages = logical.reshape(-1, page_words)
    for k, c in enumerate(ctrls):
        mine = pages[k::n]
        c.store_numpy()[: mine.size] = mine.reshape(-1)


def gather_striped(ctrls, n_pages, page_words=512):
    n = len(ctrls)
    out = np.empty((n_pages, page_words), dtype=np.uint64)
    for k, c in enumerate(ctrls):
        cnt = len(range(k, n_pages, n))
        out[k::n] = c.store_numpy()[: cnt * page_words].reshape(cnt, page_words)
    return out.reshape(-1)


@pytest.mark.parametrize("n_ctrls", [2, 3])
def test_replicated_read_uses_every_controller(cuda, bam, orc, n_ctrls):
    n_elems, seed, aseed = 1 << 20, 21, 5                    # 2048 pages
    ctrls = make_ctrls(bam, n_ctrls, n_elems * 8, queue_depth=64, num_queues=8)
    for c in ctrls:
        c.fill_store(seed)
    cache = bam.PageCache(ctrls, 4096, 512)
    arr = bam.Array(cache, n_elems, dist=bam.REPLICATE)
    out = cuda.zeros(1, dtype=cuda.int64, device="cuda")
    n_lanes, per_lane = 1 << 13, 16
    arr.read(n_lanes, per_lane, out, access_seed=aseed)
    for c in ctrls:
        assert c.status() == (0, "none", 0)
    assert cache.audit() == 0
    assert (int(out.item()) & M64) == orc.array_checksum(seed, n_elems, aseed, 0, n_lanes, per_lane)
    st = cache.stats()
    served = [c.served(reset=True) for c in ctrls]
    assert sum(served) == st["read_ios"] and st["read_ios"] > 0
    assert min(served) > st["read_ios"] // (4 * n_ctrls)       # the load is spread over all of them
    arr.close(); cache.close()
    # after the cache is gone every controller works on its own again
    c1 = bam.PageCache(ctrls[1], 4096, 512)
    a1 = bam.Array(c1, n_elems)
    out.zero_()
    a1.read(n_lanes, per_lane, out, access_seed=aseed)
    assert ctrls[1].status() == (0, "none", 0)
    assert (int(out.item()) & M64) == orc.array_checksum(seed, n_elems, aseed, 0, n_lanes, per_lane)
    assert ctrls[1].served() == c1.stats()["read_ios"] and ctrls[0].served() == 0
    a1.close(); c1.close()
    for c in ctrls:
        c.close()


@pytest.mark.parametrize("n_ctrls,slots", [(2, 4096), (3, 300), (4, 128)])
def test_striped_read_matches_oracle(cuda, bam, orc, n_ctrls, slots):
    n_pages = 2050                                            # not a multiple of 3 or 4: ragged last stripe
    n_elems, seed, aseed = n_pages * 512, 8, 13
    per_ctrl_pages = (n_pages + n_ctrls - 1) // n_ctrls
    ctrls = make_ctrls(bam, n_ctrls, per_ctrl_pages * 4096, queue_depth=32, num_queues=4)
    logical = orc.fill_store(seed, 0, n_elems)
    scatter_striped(ctrls, logical)
    cache = bam.PageCache(ctrls, 4096, slots)
    arr = bam.Array(cache, n_elems, dist=bam.STRIPE)
    out = cuda.zeros(1, dtype=cuda.int64, device="cuda")
    n_lanes, per_lane = 1 << 12, 8
    arr.read(n_lanes, per_lane, out, access_seed=aseed)
    assert ctrls[0].status() == (0, "none", 0) and ctrls[-1].status() == (0, "none", 0)
    assert cache.audit() == 0
    assert (int(out.item()) & M64) == orc.array_checksum(seed, n_elems, aseed, 0, n_lanes, per_lane)
    # every controller served at least the distinct pages it owns (more only through re-reads after
    # evictions), and together they served exactly the cache's page reads
    idx = orc.array_indices(aseed, n_elems, 0, n_lanes, per_lane)
    pages = np.unique(idx // np.uint64(512))
    served = [c.served() for c in ctrls]
    for k in range(n_ctrls):
        assert served[k] >= int((pages % np.uint64(n_ctrls) == k).sum())
    assert sum(served) == cache.stats()["read_ios"]
    p0 = int(pages[0])
    assert orc.backing_location(0, p0, n_ctrls, 1) == bam.backing_location(p0, n_ctrls, bam.STRIPE)
    arr.close(); cache.close()
    for c in ctrls:
        c.close()


def test_striped_fill_matches_scatter(cuda, bam, orc):
    n_ctrls, n_pages, seed, first = 3, 96, 5, 512 * 7
    ctrls = make_ctrls(bam, n_ctrls, n_pages // n_ctrls * 4096, queue_depth=16, num_queues=1)
    for k, c in enumerate(ctrls):
        c.fill_store_striped(seed, k, n_ctrls, first_elem=first)
    cuda.cuda.synchronize()
    assert (gather_striped(ctrls, n_pages) == orc.fill_store(seed, first, n_pages * 512)).all()
    for c in ctrls:
        c.close()


@pytest.mark.parametrize("dist_name", ["stripe", "replicate"])
def test_write_back_reaches_the_right_controllers(cuda, bam, orc, dist_name):
    n_ctrls, n_pages, seed, vseed = 3, 510, 31, 99
    n_elems = n_pages * 512
    dist = bam.STRIPE if dist_name == "stripe" else bam.REPLICATE
    per_ctrl = (n_pages // n_ctrls if dist == bam.STRIPE else n_pages) * 4096
    ctrls = make_ctrls(bam, n_ctrls, per_ctrl, queue_depth=64, num_queues=4)
    ctrls[0].configure(ctrl_blocks=2)                        # the first controller sets the launch geometry
    ctrls[0].set_max_grid(4)
    logical = orc.fill_store(seed, 0, n_elems)
    if dist == bam.STRIPE:
        scatter_striped(ctrls, logical)
    else:
        for c in ctrls:
            c.store_numpy()[:] = logical
    cache = bam.PageCache(ctrls, 4096, 96)                    # dirty pages are evicted all the time
    arr = bam.Array(cache, n_elems, dist=dist)
    rng = np.random.default_rng(17)
    idx = rng.integers(0, n_elems, 20000, dtype=np.uint64)
    d_idx = cuda.from_numpy(idx.view(np.int64)).cuda()
    arr.write(len(idx), d_idx, val_seed=vseed)
    assert ctrls[0].status() == (0, "none", 0)
    cache.flush()
    assert ctrls[0].status() == (0, "none", 0) and cache.audit() == 0
    want = logical.copy()
    with np.errstate(over="ignore"):
        want[idx.astype(np.int64)] = np_splitmix64(np.uint64(vseed) ^ idx)
    if dist == bam.STRIPE:
        assert (gather_striped(ctrls, n_pages) == want).all()
    else:
        for c in ctrls:
            assert (c.store_numpy() == want).all()            # every replica got every write-back
    out = cuda.zeros(1, dtype=cuda.int64, device="cuda")
    arr.read(len(idx), 1, out, idx=d_idx)
    assert (int(out.item()) & M64) == int(want[idx.astype(np.int64)].sum(dtype=np.uint64))
    arr.close(); cache.close()
    for c in ctrls:
        c.close()


def test_fault_on_second_controller_is_reported_to_the_group(cuda, bam, orc):
    n_elems, seed = 1 << 18, 4
    ctrls = make_ctrls(bam, 2, n_elems * 8 // 2, queue_depth=64, num_queues=4)
    for c in ctrls:
        c.configure(spin_timeout_ns=SEC // 2)
    scatter_striped(ctrls, orc.fill_store(seed, 0, n_elems))
    cache = bam.PageCache(ctrls, 4096, 1024)
    arr = bam.Array(cache, n_elems, dist=bam.STRIPE)
    ctrls[1].inject_fault(2, nth=5, status=0x281)              # BAM_FAULT_STATUS
    out = cuda.zeros(1, dtype=cuda.int64, device="cuda")
    arr.read(1 << 10, 8, out, access_seed=3)
    # whichever member is asked, the group's status block answers
    code0, where0, detail0 = ctrls[0].status()
    assert ctrls[1].status() == (code0, where0, detail0)
    assert code0 != 0 and where0 == "nvme_status" and detail0 == 0x281
    ctrls[0].status(clear=True)
    ctrls[1].inject_fault(0)
    for c in ctrls:
        c.reset_queues()
    cache.invalidate()
    out.zero_()
    arr.read(1 << 10, 8, out, access_seed=3)
    assert ctrls[1].status() == (0, "none", 0) and cache.audit() == 0
    assert (int(out.item()) & M64) == orc.array_checksum(seed, n_elems, 3, 0, 1 << 10, 8)
    arr.close(); cache.close()
    for c in ctrls:
        c.close()


def test_bfs_and_cc_over_striped_graph(cuda, bam, orc):
    scale, seed, n_ctrls = 12, 5, 3
    offsets, cols = orc.rmat_csr(seed, scale)
    store, off_bytes = orc.csr_store(offsets, cols)           # offsets first, page aligned, then the edges
    n_pages = (store.nbytes + 4095) // 4096
    n_pages += (-n_pages) % n_ctrls
    logical = np.zeros(n_pages * 512, dtype=np.uint64)
    logical[: store.size] = store
    ctrls = make_ctrls(bam, n_ctrls, n_pages // n_ctrls * 4096, queue_depth=64, num_queues=8)
    cache = bam.PageCache(ctrls, 4096, 256)
    n = len(offsets) - 1
    # offsets and edges are two arrays = two ranges, each striped from its own first page: on every
    # controller its share of the offset pages comes first, then its share of the edge pages
    off_pages = off_bytes // 4096
    assert off_pages % n_ctrls == 0
    for k, c in enumerate(ctrls):
        media = c.store_numpy()
        o = logical[: off_pages * 512].reshape(-1, 512)[k::n_ctrls]
        e = logical[off_pages * 512:].reshape(-1, 512)[k::n_ctrls]
        media[: o.size] = o.reshape(-1)
        media[o.size: o.size + e.size] = e.reshape(-1)
    g = bam.CsrGraph.over_cache(cache, n, len(cols), off_bytes // n_ctrls, dist=bam.STRIPE)
    src = orc.max_degree_vertex(offsets)
    levels, _, scanned = g.bfs(src)
    assert ctrls[0].status() == (0, "none", 0) and cache.audit() == 0
    want, want_scanned = orc.bfs(offsets, cols, src)
    assert (levels.cpu().numpy().view(np.uint32) == want).all() and scanned == want_scanned
    assert all(c.served() > 0 for c in ctrls)
    comp, _, _ = g.cc()
    want_cc, _ = orc.cc(offsets, cols)
    assert ctrls[0].status() == (0, "none", 0) and cache.audit() == 0
    assert (comp.cpu().numpy().view(np.uint64) == want_cc).all()
    g.close(); cache.close()
    for c in ctrls:
        c.close()
