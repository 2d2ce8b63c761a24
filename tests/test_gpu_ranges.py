"""Arrays of several ranges and ranges that start inside a page (bam_array_create_ranges: array_t over a
vector of range_t with a page_start_offset, include/page_cache.h:985-1030, :1318-1329, :1754-1772 in the
reference; the shape benchmarks/bfs/main.cu:1481-1484 builds for an edge list at a file offset), and the race
the pin-free read path must survive: element reads of hot pages while reads of a second range force their
eviction from a cache of a few dozen slots.  Every result is compared bit for bit with what the backing
store holds (numpy over the store's host memory) or with the CPU oracle."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
M64 = (1 << 64) - 1
SEC = 1_000_000_000
PAGE = 4096


def _world(bam, store_pages, slots, max_grid=3, ctrl_blocks=1, nq=2, depth=16, seed=21):
    ctrl = bam.Controller(store_pages * PAGE, 0, queue_depth=depth, num_queues=nq)
    ctrl.configure(ctrl_blocks=ctrl_blocks, spin_timeout_ns=5 * SEC)
    ctrl.set_launch_timeout(60 * SEC)
    if max_grid:
        ctrl.set_max_grid(max_grid)
    ctrl.fill_store(seed)
    return ctrl, bam.PageCache(ctrl, PAGE, slots)


def _expected(store, ranges, idx):
    """Values the store holds for the element indices idx of an array made of `ranges`."""
    out = np.zeros(len(idx), dtype=np.uint64)
    for i0, i1, off, pso in ranges:
        m = (idx >= i0) & (idx < i1)
        out[m] = store[(off + pso) // 8 + (idx[m] - i0)]
    return out


def test_two_ranges_second_one_starts_mid_page(cuda, bam):
    torch = cuda
    ctrl, cache = _world(bam, 256, 64)
    torch.cuda.synchronize()
    store = ctrl.store_numpy()
    # range 0: indices [0, 3000) from store page 0; range 1: indices [3000, 23000), element 3000 lives 520 bytes
    # into store page 16 (so every page of range 1 holds elements that straddle the usual 512-element grid)
    ranges = [(0, 3000, 0, 0), (3000, 23000, 16 * PAGE, 520)]
    arr = bam.Array.from_ranges(cache, 23000, ranges)
    rng = np.random.default_rng(5)
    idx = rng.integers(0, 23000, size=256 * 16, dtype=np.uint64)
    idx[:8] = [0, 2999, 3000, 3001, 3000 + 446, 3000 + 447, 3000 + 448, 22999]      # range and page borders
    d_idx = torch.from_numpy(idx.view(np.int64)).cuda()
    out = torch.zeros(1, dtype=torch.int64, device="cuda")
    arr.read(256, 16, out, idx=d_idx)
    assert ctrl.status() == (0, "none", 0) and cache.audit() == 0
    want = int(_expected(store, ranges, idx).sum(dtype=np.uint64))
    assert int(out.item()) & M64 == want
    st = cache.stats(reset=True)
    assert st["accesses"] == len(idx) and st["read_ios"] >= 46         # 6 pages of range 0 + 40 of range 1
    # the cursor form over the same array (bam_ptr computes the element span of a page from the offset)
    out.zero_()
    arr.pattern_read(0, 23000, out)
    assert ctrl.status() == (0, "none", 0) and cache.audit() == 0
    assert int(out.item()) & M64 == int(_expected(store, ranges, np.arange(23000, dtype=np.uint64)).sum(dtype=np.uint64))
    # writes through both ranges reach the right bytes of the store
    widx = np.unique(rng.integers(0, 23000, size=2000, dtype=np.uint64))
    arr.write(len(widx), torch.from_numpy(widx.view(np.int64)).cuda(), val_seed=77)
    cache.flush()
    assert ctrl.status() == (0, "none", 0) and cache.audit() == 0
    torch.cuda.synchronize()
    x = (widx ^ np.uint64(77)) + np.uint64(0x9E3779B97F4A7C15)                           # splitmix64(val_seed ^ i)
    x = (x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    x = (x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    x = x ^ (x >> np.uint64(31))
    assert (_expected(ctrl.store_numpy(), ranges, widx) == x).all()
    # an index outside every range is reported, not read
    bad = torch.tensor([5, 23000 + 5], dtype=torch.int64, device="cuda")
    arr2 = bam.Array.from_ranges(cache, 30000, [(0, 3000, 0, 0), (3000, 23000, 16 * PAGE, 520)])
    arr2.read(2, 1, out, idx=bad)
    code, where, detail = ctrl.status(clear=True)
    assert code == 34 and where == "range" and detail == 23005
    arr2.close(); arr.close(); cache.close(); ctrl.close()


def test_range_arguments_are_checked(cuda, bam):
    ctrl, cache = _world(bam, 64, 64)
    bad = [
        [(0, 100, 0, 0), (50, 200, 8 * PAGE, 0)],        # overlapping index ranges
        [(0, 100, 100, 0)],                               # store offset not page aligned
        [(0, 100, 0, PAGE)],                              # offset not inside the first page
        [(0, 100, 0, 12)],                                # offset not a multiple of the element size
        [(0, 100, 63 * PAGE, 4000)],                      # runs past the end of the store
        [(10, 10, 0, 0)],                                 # empty range
    ]
    for ranges in bad:
        with pytest.raises(bam.BamError) as e:
            bam.Array.from_ranges(cache, 1000, ranges)
        assert e.value.code == 22
    # page-walking launchers refuse what they cannot walk
    arr = bam.Array.from_ranges(cache, 1000, [(0, 1000, 0, 8)])
    out = cuda.zeros(1, dtype=cuda.int64, device="cuda")
    with pytest.raises(bam.BamError):
        arr.page_scan(1, out)
    arr.close(); cache.close(); ctrl.close()


@pytest.mark.parametrize("slots,max_grid", [(64, 3), (96, 4)])
def test_hot_reads_survive_constant_eviction(cuda, bam, slots, max_grid):
    """Range 0: 16 hot pages, read over and over (mostly without a pin).  Range 1: 2048 pages read once each,
    which recycles every slot of the small cache many times while the hot reads are in flight.  A read that
    validated against a recycled slot would return another page's data and break the sum."""
    torch = cuda
    ctrl, cache = _world(bam, 16 + 2048, slots, max_grid=max_grid, nq=4, depth=64)
    torch.cuda.synchronize()
    store = ctrl.store_numpy()
    hot_elems, cold_elems = 16 * 512, 2048 * 512
    ranges = [(0, hot_elems, 0, 0), (hot_elems, hot_elems + cold_elems, 16 * PAGE, 0)]
    arr = bam.Array.from_ranges(cache, hot_elems + cold_elems, ranges)
    single = bam.Array(cache, hot_elems + cold_elems)                       # the same bytes as one range (batched reader)
    rng = np.random.default_rng(slots)
    lanes, reqs = 1 << 12, 32
    idx = rng.integers(0, hot_elems, size=lanes * reqs, dtype=np.uint64)
    cold = rng.permutation(2048).astype(np.uint64) * np.uint64(512) + rng.integers(0, 512, size=2048, dtype=np.uint64)
    pos = rng.choice(lanes * reqs, size=8 * 2048, replace=False)
    idx[pos] = np.uint64(hot_elems) + np.tile(cold, 8)                      # one access in 8 streams through range 1
    d_idx = torch.from_numpy(idx.view(np.int64)).cuda()
    want = int(_expected(store, ranges, idx).sum(dtype=np.uint64))
    out = torch.zeros(1, dtype=torch.int64, device="cuda")
    for a in (arr, single, arr, single):
        out.zero_()
        cache.stats(reset=True)
        a.read(lanes, reqs, out, idx=d_idx)
        assert ctrl.status() == (0, "none", 0) and cache.audit() == 0
        assert int(out.item()) & M64 == want
        st = cache.stats()
        assert st["accesses"] == lanes * reqs
        assert st["read_ios"] > 4 * slots and st["hits"] > lanes * reqs // 2      # constant recycling, yet mostly hits
    single.close(); arr.close(); cache.close(); ctrl.close()
