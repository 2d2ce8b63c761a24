"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle.

Bit-exact everywhere (integer work): wrapping 64-bit sums, page CRC-32s.  Small cases compare
with the oracle directly and with the committed golden fixtures; queue depths of 2..8 and caches
of a few pages force every wrap-around (phase bit, tickets, clock hand) and constant eviction.
After every launch the device status must be clean and the cache audit must find no leaked pin,
no BUSY bit and a consistent page table."""
import json
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
GOLDEN = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "golden.json")))
M64 = (1 << 64) - 1
SEC = 1_000_000_000


def u64(t):
    return int(t.item()) & M64


def make(bam, n_elems, slots, nq, depth, max_grid=0, ctrl_blocks=0, page=4096, lba=512, seed=11):
    ctrl = bam.Controller(n_elems * 8, 0, queue_depth=depth, num_queues=nq, lba_bytes=lba)
    ctrl.configure(ctrl_blocks=ctrl_blocks, spin_timeout_ns=5 * SEC)
    ctrl.set_launch_timeout(60 * SEC)
    if max_grid:
        ctrl.set_max_grid(max_grid)
    ctrl.fill_store(seed)
    cache = bam.PageCache(ctrl, page, slots)
    arr = bam.Array(cache, n_elems)
    return ctrl, cache, arr


def finish(ctrl, cache):
    assert ctrl.status() == (0, "none", 0)
    assert cache.audit() == 0


def test_store_fill_matches_oracle(cuda, bam, orc):
    ctrl = bam.Controller(1 << 20, 0, queue_depth=4, num_queues=1)
    ctrl.fill_store(0xC0FFEE, first_elem=1000)
    cuda.cuda.synchronize()
    assert (ctrl.store_numpy() == orc.fill_store(0xC0FFEE, 1000, (1 << 20) // 8)).all()
    ctrl.close()


@pytest.mark.parametrize("slots,nq,depth,max_grid,ctrl_blocks,lanes,reqs", [
    (64, 1, 2, 2, 1, 64, 8),        # depth 2: one command in flight, wraps every command
    (64, 1, 4, 3, 1, 512, 8),       # 128-page store in 64 slots: constant eviction
    (96, 2, 8, 3, 1, 777, 5),       # ragged lane count, two queues
    (4096, 8, 64, 0, 0, 1 << 14, 16),   # full grid, cache smaller than the store
])
def test_array_read_small(cuda, bam, orc, slots, nq, depth, max_grid, ctrl_blocks, lanes, reqs):
    n_elems, seed, aseed = 1 << 16 if slots < 1000 else 1 << 22, 11, 29
    ctrl, cache, arr = make(bam, n_elems, slots, nq, depth, max_grid, ctrl_blocks, seed=seed)
    out = cuda.zeros(1, dtype=cuda.int64, device="cuda")
    arr.read(lanes, reqs, out, access_seed=aseed)
    finish(ctrl, cache)
    assert u64(out) == orc.array_checksum(seed, n_elems, aseed, 0, lanes, reqs)
    st = cache.stats()
    assert st["accesses"] == lanes * reqs
    idx = orc.array_indices(aseed, n_elems, 0, lanes, reqs)
    assert st["read_ios"] >= len(np.unique(idx // 512)) if slots >= 1000 else st["read_ios"] > 0
    assert ctrl.served() == st["read_ios"]
    # second pass over the same stream: same sum again (cache state differs, result must not)
    out.zero_()
    arr.read(lanes, reqs, out, access_seed=aseed)
    finish(ctrl, cache)
    assert u64(out) == orc.array_checksum(seed, n_elems, aseed, 0, lanes, reqs)
    arr.close(); cache.close(); ctrl.close()


def test_array_read_golden(cuda, bam):
    for c in GOLDEN["array_checksum"][:4]:
        n = c["n_elems"]
        ctrl, cache, arr = make(bam, (n + 511) // 512 * 512, 2048, 4, 64, seed=c["store_seed"])
        arr.close()
        arr = bam.Array(cache, n)
        out = cuda.zeros(1, dtype=cuda.int64, device="cuda")
        arr.read(c["lanes"], c["reqs"], out, access_seed=c["access_seed"])
        finish(ctrl, cache)
        assert u64(out) == c["checksum"]
        arr.close(); cache.close(); ctrl.close()


def test_array_read_explicit_indices_edge_cases(cuda, bam, orc):
    n_elems, seed = 1 << 16, 3
    ctrl, cache, arr = make(bam, n_elems, 256, 2, 16, seed=seed)
    out = cuda.zeros(1, dtype=cuda.int64, device="cuda")
    cases = {
        "all_same": np.full(4096, 12345, dtype=np.uint64),                     # one page, maximal coalescing
        "first_last": np.array([0, n_elems - 1] * 100, dtype=np.uint64),
        "page_edges": np.array([511, 512, 1023, 1024, 0, 65535] * 50, dtype=np.uint64),
        "sequential": np.arange(8192, dtype=np.uint64),                        # 32 lanes share pages
        "single": np.array([777], dtype=np.uint64),
    }
    for name, idx in cases.items():
        d_idx = cuda.from_numpy(idx.view(np.int64)).cuda()
        out.zero_()
        arr.read(len(idx), 1, out, idx=d_idx)
        finish(ctrl, cache)
        assert u64(out) == orc.indexed_checksum(seed, 0, idx), name
    # empty input: no work, no error
    out.zero_()
    arr.read(0, 64, out, access_seed=1)
    finish(ctrl, cache)
    assert u64(out) == 0
    arr.close(); cache.close(); ctrl.close()


def test_generated_index_streams_match_oracle(cuda, bam, orc):
    n_elems, lanes, reqs = 1 << 20, 300, 9
    d = cuda.zeros(lanes * reqs, dtype=cuda.int64, device="cuda")
    bam.gen_uniform_indices(d, lanes, reqs, 99, n_elems)
    assert (d.cpu().numpy().view(np.uint64) == orc.array_indices(99, n_elems, 0, lanes, reqs)).all()
    z = GOLDEN["zipf"]
    cdf = bam.zipf_cdf(z["n_pages"], z["s"])
    assert (cdf == orc.zipf_cdf(z["n_pages"], z["s"])).all()
    d_cdf = cuda.from_numpy(cdf.view(np.int64)).cuda()
    d = cuda.zeros(z["lanes"] * z["reqs"], dtype=cuda.int64, device="cuda")
    bam.gen_zipf_indices(d, z["lanes"], z["reqs"], z["access_seed"], d_cdf, z["n_pages"], 512, z["perm_seed"])
    got = d.cpu().numpy().view(np.uint64)
    assert got[:8].tolist() == z["first_idx"]
    assert (got == orc.zipf_indices(cdf, z["n_pages"], 512, z["perm_seed"], z["access_seed"], 0, z["lanes"], z["reqs"])).all()


def test_zipf_scan_through_cache(cuda, bam, orc):
    """The skewed multi-GPU scan on one shard: Zipf page popularity, shard offset in the store."""
    n_pages, lanes, reqs, seed = 1 << 12, 1 << 12, 16, 9
    first_elem = 5 * n_pages * 512                                  # this shard starts 5 shards in
    ctrl = bam.Controller(n_pages * 4096, 0, queue_depth=64, num_queues=8)
    ctrl.configure(spin_timeout_ns=5 * SEC)
    ctrl.fill_store(seed, first_elem=first_elem)
    cache = bam.PageCache(ctrl, 4096, n_pages // 4)
    arr = bam.Array(cache, n_pages * 512)
    cdf = bam.zipf_cdf(n_pages)
    d_cdf = cuda.from_numpy(cdf.view(np.int64)).cuda()
    d_idx = cuda.zeros(lanes * reqs, dtype=cuda.int64, device="cuda")
    bam.gen_zipf_indices(d_idx, lanes, reqs, 23, d_cdf, n_pages, 512, 17)
    out = cuda.zeros(1, dtype=cuda.int64, device="cuda")
    arr.read(lanes, reqs, out, idx=d_idx)
    finish(ctrl, cache)
    idx = orc.zipf_indices(cdf, n_pages, 512, 17, 23, 0, lanes, reqs)
    assert u64(out) == orc.indexed_checksum(seed, first_elem, idx)
    st = cache.stats()
    assert st["accesses"] == lanes * reqs and st["hits"] > st["misses"]      # skew -> mostly hits
    arr.close(); cache.close(); ctrl.close()


@pytest.mark.parametrize("nq,depth,lba", [(1, 2, 512), (1, 64, 4096), (16, 256, 512), (128, 1024, 512)])
def test_block_read_crc(cuda, bam, orc, nq, depth, lba):
    seed, n_store_pages = 11, 1 << 13
    ctrl = bam.Controller(n_store_pages * 4096, 0, queue_depth=depth, num_queues=nq, lba_bytes=lba)
    ctrl.configure(spin_timeout_ns=5 * SEC)
    ctrl.set_launch_timeout(60 * SEC)
    if depth <= 2:
        ctrl.configure(ctrl_blocks=1)
        ctrl.set_max_grid(3)
    ctrl.fill_store(seed)
    g, cb, th = ctrl.geometry()
    cache = bam.PageCache(ctrl, 4096, g * th)
    n_reqs = 1 << 12 if depth <= 2 else 1 << 15
    crc = cuda.zeros(n_reqs, dtype=cuda.int32, device="cuda")
    out = cuda.zeros(1, dtype=cuda.int64, device="cuda")
    cache.block_read(n_reqs, req_seed=77, crc_out=crc, sum_out=out)
    assert ctrl.status() == (0, "none", 0)
    pages, want = orc.block_requests(seed, 77, n_store_pages, 4096, 0, n_reqs)
    assert (crc.cpu().numpy().view(np.uint32) == want).all()
    b = GOLDEN["block_requests"]
    assert crc[:8].cpu().numpy().view(np.uint32).tolist() == b["first_crcs"]
    # wrapping sum of every word of every page read
    words = orc.fill_store(seed, 0, n_store_pages * 512).reshape(n_store_pages, 512)
    page_sums = words.sum(axis=1, dtype=np.uint64)
    assert u64(out) == int(page_sums[pages.astype(np.int64)].sum(dtype=np.uint64))
    assert ctrl.served() == n_reqs
    cache.close(); ctrl.close()


def test_block_read_explicit_pages(cuda, bam, orc):
    seed, n_store_pages = 5, 256
    ctrl = bam.Controller(n_store_pages * 4096, 0, queue_depth=8, num_queues=3)
    ctrl.configure(spin_timeout_ns=5 * SEC)
    ctrl.fill_store(seed)
    g, cb, th = ctrl.geometry()
    cache = bam.PageCache(ctrl, 4096, g * th)
    pages = np.array([0, 255, 255, 0, 17] * 100, dtype=np.uint64)           # first, last, repeats
    crc = cuda.zeros(len(pages), dtype=cuda.int32, device="cuda")
    cache.block_read(len(pages), pages=cuda.from_numpy(pages.view(np.int64)).cuda(), crc_out=crc)
    assert ctrl.status() == (0, "none", 0)
    want = np.array([orc.page_crc(seed, int(p), 4096) for p in pages], dtype=np.uint32)
    assert (crc.cpu().numpy().view(np.uint32) == want).all()
    cache.close(); ctrl.close()


def test_page_scan_cold_and_warm(cuda, bam, orc):
    n_elems, seed = 1 << 20, 13
    ctrl, cache, arr = make(bam, n_elems, 4096, 8, 64, seed=seed)       # 2048 pages, all fit
    want = int(orc.fill_store(seed, 0, n_elems).sum(dtype=np.uint64))
    out = cuda.zeros(1, dtype=cuda.int64, device="cuda")
    for expect_hits in (0, 2048):
        out.zero_()
        arr.page_scan(2048, out)
        finish(ctrl, cache)
        assert u64(out) == want
        st = cache.stats(reset=True)
        assert st["hits"] == expect_hits and st["misses"] == 2048 - expect_hits
    # explicit page list with repeats, cache smaller than the list's footprint
    cache.invalidate()
    pages = np.array([5, 5, 2047, 0, 1000] * 64, dtype=np.uint64)
    out.zero_()
    arr.page_scan(len(pages), out, pages=cuda.from_numpy(pages.view(np.int64)).cuda())
    finish(ctrl, cache)
    words = orc.fill_store(seed, 0, n_elems).reshape(2048, 512).sum(axis=1, dtype=np.uint64)
    assert u64(out) == int(words[pages.astype(np.int64)].sum(dtype=np.uint64))
    arr.close(); cache.close(); ctrl.close()


def test_large_page_prp2_and_prp_list(cuda, bam, orc):
    """8 KiB pages use PRP2 as a second pointer, larger pages a PRP list (3 entries for 16 KiB, 15 for
    64 KiB: the lists of 64 slots span more than one list page without any crossing a page end)."""
    n_elems, seed = 1 << 18, 21
    for page in (8192, 16384, 65536):
        ctrl, cache, arr = make(bam, n_elems, 64, 2, 16, page=page, seed=seed)
        out = cuda.zeros(1, dtype=cuda.int64, device="cuda")
        arr.read(2048, 8, out, access_seed=4)
        finish(ctrl, cache)
        assert u64(out) == orc.array_checksum(seed, n_elems, 4, 0, 2048, 8)
        arr.close(); cache.close(); ctrl.close()


def test_dropped_completion_times_out_cleanly(cuda, bam):
    """Failure detection without a GPU fault: the controller swallows one completion (host-side
    injection); the waiter's bounded wait runs out, the launch drains and reports where."""
    ctrl, cache, arr = make(bam, 1 << 16, 64, 1, 8, max_grid=3, ctrl_blocks=1)
    ctrl.configure(spin_timeout_ns=SEC // 5)
    ctrl.inject_fault(1, nth=5)                         # BAM_FAULT_DROP_CPL
    out = cuda.zeros(1, dtype=cuda.int64, device="cuda")
    arr.read(256, 4, out, access_seed=1)
    code, where, _ = ctrl.status(clear=True)
    assert code == 110 and where in ("cq_wait", "sq_turn", "sq_doorbell", "page_busy", "cid")
    # the context is still usable: reset the queues and the cache, run again cleanly
    ctrl.inject_fault(0)
    ctrl.reset_queues()
    cache.invalidate()
    out.zero_()
    arr.read(256, 4, out, access_seed=1)
    assert ctrl.status() == (0, "none", 0)
    arr.close(); cache.close(); ctrl.close()


def test_nvme_error_status_is_reported(cuda, bam):
    ctrl, cache, arr = make(bam, 1 << 16, 64, 1, 8, max_grid=3, ctrl_blocks=1)
    ctrl.configure(spin_timeout_ns=SEC // 5)
    ctrl.inject_fault(2, nth=3, status=0x281)           # BAM_FAULT_STATUS: SCT 2, SC 0x81
    out = cuda.zeros(1, dtype=cuda.int64, device="cuda")
    arr.read(256, 4, out, access_seed=1)
    code, where, detail = ctrl.status(clear=True)
    assert code == 5 and where == "nvme_status" and detail == 0x281
    arr.close(); cache.close(); ctrl.close()


def test_out_of_range_lba_gets_nvme_status(cuda, bam):
    """A request beyond the namespace completes with LBA Out of Range instead of touching memory."""
    ctrl = bam.Controller(64 * 4096, 0, queue_depth=8, num_queues=1)
    ctrl.configure(ctrl_blocks=1, spin_timeout_ns=SEC // 5)
    ctrl.set_max_grid(2)
    ctrl.fill_store(1)
    g, cb, th = ctrl.geometry()
    cache = bam.PageCache(ctrl, 4096, g * th)
    pages = np.array([3, 64, 5], dtype=np.uint64)       # page 64 is one past the end
    cache.block_read(3, pages=cuda.from_numpy(pages.view(np.int64)).cuda())
    code, where, detail = ctrl.status(clear=True)
    assert code == 5 and where == "nvme_status" and detail == 0x80
    cache.close(); ctrl.close()


def test_config1_shape_reduced_lanes(cuda, bam, orc):
    """Array random-read configuration (1 GiB store, 256 MiB cache, 1 queue pair x 1024) on a
    reduced lane count; the oracle needs no store, so the full 2^27-element range is covered."""
    c = GOLDEN["array_checksum"][4]
    ctrl, cache, arr = make(bam, c["n_elems"], 65536, 1, 1024, seed=c["store_seed"])
    out = cuda.zeros(1, dtype=cuda.int64, device="cuda")
    arr.read(c["lanes"], c["reqs"], out, access_seed=c["access_seed"])
    finish(ctrl, cache)
    assert u64(out) == c["checksum"]
    arr.close(); cache.close(); ctrl.close()


def test_system_scope_queues(cuda, bam, orc):
    """Doorbells and completion entries synchronised at system scope (what a controller outside the
    GPU needs) give the same results as the default device scope."""
    n_elems, seed, aseed = 1 << 20, 11, 29
    ctrl, cache, arr = make(bam, n_elems, 1024, 4, 64, seed=seed)
    ctrl.set_scope(1)
    out = cuda.zeros(1, dtype=cuda.int64, device="cuda")
    arr.read(1 << 13, 8, out, access_seed=aseed)
    finish(ctrl, cache)
    assert u64(out) == orc.array_checksum(seed, n_elems, aseed, 0, 1 << 13, 8)
    ctrl.set_scope(0)
    out.zero_()
    arr.read(1 << 13, 8, out, access_seed=aseed + 1)
    finish(ctrl, cache)
    assert u64(out) == orc.array_checksum(seed, n_elems, aseed + 1, 0, 1 << 13, 8)
    arr.close(); cache.close(); ctrl.close()


def test_bel_files_to_bfs(cuda, bam, orc, tmp_path):
    """A graph loaded from the reference's .bel files gives the oracle's BFS levels."""
    off, cols = orc.rmat_csr(4, 9, 8)
    prefix = str(tmp_path / "rmat9")
    bam.write_bel(prefix + ".bel.col", off.astype(np.int64))
    bam.write_bel(prefix + ".bel.dst", cols.astype(np.int64))
    d_off, d_cols = bam.load_bel_graph(prefix)
    gr = bam.CsrGraph(d_off, d_cols, cache_pages=64, queue_depth=16, num_queues=2)
    src = orc.max_degree_vertex(off)
    lv, _, _ = gr.bfs(src)
    want, _ = orc.bfs(off, cols, src)
    assert (lv.cpu().numpy().view(np.uint32) == want).all() and gr.ctrl.status() == (0, "none", 0)
    gr.close()


@pytest.mark.parametrize("io_depth", [2, 4])
def test_block_read_with_several_requests_in_flight_per_thread(cuda, bam, orc, io_depth):
    """The iodepth-block shape: each thread submits io_depth reads, then waits for each."""
    seed, n_store_pages = 11, 1 << 13
    ctrl = bam.Controller(n_store_pages * 4096, 0, queue_depth=1024, num_queues=16)
    ctrl.configure(spin_timeout_ns=5 * SEC)
    ctrl.fill_store(seed)
    g, cb, th = ctrl.geometry()
    cache = bam.PageCache(ctrl, 4096, g * th * io_depth)
    n_reqs = (1 << 15) + 77                                  # ragged tail
    crc = cuda.zeros(n_reqs, dtype=cuda.int32, device="cuda")
    cache.block_read(n_reqs, req_seed=77, crc_out=crc, io_depth=io_depth)
    assert ctrl.status() == (0, "none", 0)
    _, want = orc.block_requests(seed, 77, n_store_pages, 4096, 0, n_reqs)
    assert (crc.cpu().numpy().view(np.uint32) == want).all() and ctrl.served() == n_reqs
    cache.close(); ctrl.close()


def test_randomised_configurations(cuda, bam, orc):
    """Seeded random geometry: store size, cache size (from a handful of slots to everything),
    queue count and depth, lane count and reads per lane -- the checksum must always equal the
    oracle's and the cache must audit clean."""
    rng = np.random.default_rng(20261125)
    out = cuda.zeros(1, dtype=cuda.int64, device="cuda")
    for case in range(10):
        n_pages = int(rng.integers(64, 4096))
        n_elems = n_pages * 512 - int(rng.integers(0, 511))            # ragged last page
        slots = int(rng.choice([n_pages // 8 + 40, n_pages // 2 + 40, n_pages + 64]))
        nq = int(rng.choice([1, 2, 3, 8, 32]))
        depth = int(rng.choice([4, 16, 64, 256, 1024]))
        lanes = int(rng.integers(1, 20000))
        reqs = int(rng.integers(1, 12))
        seed, aseed = int(rng.integers(1, 1 << 30)), int(rng.integers(1, 1 << 30))
        ctrl = bam.Controller(n_pages * 4096, 0, queue_depth=depth, num_queues=nq)
        ctrl.configure(spin_timeout_ns=5 * SEC)
        ctrl.set_launch_timeout(60 * SEC)
        # a resident warp can hold 32 pages while it waits for more: keep warps x 32 below the slots
        ctrl.configure(ctrl_blocks=2)
        ctrl.set_max_grid(2 + max(1, min(400, slots // 32 // 8)))
        ctrl.fill_store(seed)
        cache = bam.PageCache(ctrl, 4096, slots)
        arr = bam.Array(cache, n_elems)
        out.zero_()
        arr.read(lanes, reqs, out, access_seed=aseed)
        what = f"case {case}: pages {n_pages} slots {slots} queues {nq}x{depth} lanes {lanes}x{reqs}"
        assert ctrl.status() == (0, "none", 0), what
        assert cache.audit() == 0, what
        assert u64(out) == orc.array_checksum(seed, n_elems, aseed, 0, lanes, reqs), what
        arr.close(); cache.close(); ctrl.close()


@pytest.mark.parametrize("slots", [1 << 15, 1 << 17])       # fewer slots than pages (evictions) / everything fits
def test_pattern_reads_through_cursors(cuda, bam, orc, slots):
    """The pattern benchmark's bam_ptr kernels: sequential, sequential by warp (in order and
    interleaved), random elements, random whole pages -- every sum against the oracle."""
    n_pages, seed = 1 << 16, 31
    n_elems = n_pages * 512 - 100                              # ragged last page
    ctrl = bam.Controller(n_pages * 4096, 0, queue_depth=256, num_queues=32)
    ctrl.configure(spin_timeout_ns=5 * SEC)
    # a cursor keeps its page pinned: with the smaller cache run fewer threads than there are slots
    if slots < (1 << 17):
        ctrl.set_max_grid(48 + 64)
    ctrl.fill_store(seed)
    cache = bam.PageCache(ctrl, 4096, slots)
    arr = bam.Array(cache, n_elems)
    store = orc.fill_store(seed, 0, n_elems)
    out = cuda.zeros(1, dtype=cuda.int64, device="cuda")

    def total(a):
        return int(a.sum(dtype=np.uint64))

    def run(*args, **kw):
        out.zero_()
        arr.pattern_read(*args, out, **kw)
        assert ctrl.status() == (0, "none", 0) and cache.audit() == 0
        return int(out.item()) & M64

    assert run(0, n_elems) == total(store)                                     # sequential, everything
    assert run(0, 12345) == total(store[:12345])                               # sequential, a ragged prefix
    assert run(1, n_elems, n_warps=n_pages, n_pages_per_warp=1) == total(store)
    assert run(1, n_elems, n_warps=n_pages // 4, n_pages_per_warp=4, stride=8) == total(store)
    rng = np.random.default_rng(2)
    idx = rng.integers(0, n_elems, 1 << 18, dtype=np.uint64)
    d_idx = cuda.from_numpy(idx.view(np.int64)).cuda()
    assert run(2, len(idx), assignment=d_idx) == total(store[idx.astype(np.int64)])
    pages = rng.integers(0, n_pages - 1, 3000, dtype=np.uint64)               # whole pages, with repeats
    d_pages = cuda.from_numpy(pages.view(np.int64)).cuda()
    want = total(store[: (n_pages - 1) * 512].reshape(-1, 512)[pages.astype(np.int64)])
    assert run(3, n_elems, n_warps=1000, n_pages_per_warp=3, assignment=d_pages) == want
    arr.close(); cache.close(); ctrl.close()

