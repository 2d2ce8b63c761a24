"""GPU tests of the write path: element writes and atomic adds through the cache, write-back of
dirty pages on eviction, flush.  The expected backing store is computed with numpy."""
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


@pytest.mark.parametrize("slots", [4096, 96])          # everything fits / constant eviction of dirty pages
def test_write_flush_store_matches_numpy(cuda, bam, orc, slots):
    n_elems, seed, vseed = 1 << 18, 11, 77                # 512 pages
    ctrl = bam.Controller(n_elems * 8, 0, queue_depth=64, num_queues=4)
    ctrl.configure(spin_timeout_ns=5 * SEC)
    if slots < 1000:
        ctrl.configure(ctrl_blocks=2)
        ctrl.set_max_grid(4)
    ctrl.fill_store(seed)
    cache = bam.PageCache(ctrl, 4096, slots)
    arr = bam.Array(cache, n_elems)
    rng = np.random.default_rng(5)
    idx = rng.integers(0, n_elems, 20000, dtype=np.uint64)
    idx[:64] = np.arange(64)                              # a run inside one page, coalesced by the warp
    d_idx = cuda.from_numpy(idx.view(np.int64)).cuda()
    arr.write(len(idx), d_idx, val_seed=vseed)
    assert ctrl.status() == (0, "none", 0)
    cache.flush()
    assert ctrl.status() == (0, "none", 0) and cache.audit() == 0
    want = orc.fill_store(seed, 0, n_elems)
    with np.errstate(over="ignore"):
        want[idx.astype(np.int64)] = np_splitmix64(np.uint64(vseed) ^ idx)
    assert (ctrl.store_numpy() == want).all()
    # reads through the cache see the written values too
    out = cuda.zeros(1, dtype=cuda.int64, device="cuda")
    arr.read(len(idx), 1, out, idx=d_idx)
    assert ctrl.status() == (0, "none", 0)
    assert (int(out.item()) & M64) == int(want[idx.astype(np.int64)].sum(dtype=np.uint64))
    arr.close(); cache.close(); ctrl.close()


def test_atomic_add_through_cache(cuda, bam, orc):
    n_elems, seed = 1 << 16, 3
    ctrl = bam.Controller(n_elems * 8, 0, queue_depth=16, num_queues=2)
    ctrl.configure(ctrl_blocks=2, spin_timeout_ns=5 * SEC)
    ctrl.set_max_grid(6)
    ctrl.fill_store(seed)
    cache = bam.PageCache(ctrl, 4096, 64)                 # 128 pages in 64 slots
    arr = bam.Array(cache, n_elems)
    rng = np.random.default_rng(9)
    idx = rng.integers(0, n_elems, 30000, dtype=np.uint64)
    idx[:5000] = 4242                                     # a hot element: 5000 adds land on it
    d_idx = cuda.from_numpy(idx.view(np.int64)).cuda()
    arr.write(len(idx), d_idx, addend=0x100000001)
    assert ctrl.status() == (0, "none", 0)
    cache.flush()
    assert ctrl.status() == (0, "none", 0) and cache.audit() == 0
    want = orc.fill_store(seed, 0, n_elems)
    with np.errstate(over="ignore"):
        np.add.at(want, idx.astype(np.int64), np.uint64(0x100000001))
    assert (ctrl.store_numpy() == want).all()
    arr.close(); cache.close(); ctrl.close()


def test_file_round_trip_through_the_store(cuda, bam, orc, tmp_path):
    """The reference's read-write check (benchmarks/readwrite/main.cu:392-468: file -> SSD -> file, compared
    element by element): a file is loaded onto the store with NVMe WRITE commands, a cache-full at a time,
    read back with NVMe READ commands and compared; the store holds it where it was put, a .bel graph
    loaded this way traverses like the generated one."""
    rng = np.random.default_rng(8)
    blob = rng.integers(0, 256, 3 * 1024 * 1024 + 1234, dtype=np.uint8)         # ragged last page
    src, back = tmp_path / "in.bin", tmp_path / "out.bin"
    blob.tofile(src)
    ctrl = bam.Controller(8 << 20, 0, queue_depth=64, num_queues=8)
    ctrl.configure(spin_timeout_ns=5 * SEC)
    ctrl.store_numpy()[:] = np.uint64(0x5555555555555555)
    cache = bam.PageCache(ctrl, 4096, 200)                    # the file needs four cache-fulls
    off = 1 << 20
    assert cache.load_file(str(src), store_byte_offset=off) == blob.size
    assert ctrl.status() == (0, "none", 0) and cache.audit() == 0
    media = ctrl.store_numpy(dtype="uint8")
    assert (media[off: off + blob.size] == blob).all()
    assert (media[:off] == 0x55).all()                        # nothing before the target
    pad_end = off + (blob.size + 4095) // 4096 * 4096
    assert (media[off + blob.size: pad_end] == 0).all() and (media[pad_end:] == 0x55).all()
    assert cache.dump_file(str(back), blob.size, store_byte_offset=off) == blob.size
    assert (np.fromfile(back, dtype=np.uint8) == blob).all()
    cache.close(); ctrl.close()



def test_per_thread_acquire_writes_back_dirty_victims(cuda, bam, orc):
    """range_d_t::acquire_page as a diverged caller uses it (every lane on its own) on a cache whose every slot
    holds a dirty page: each miss has to claim a dirty victim and write it back itself.  Waits are short
    (5 s), so a miss that found no way forward would come back as a time-out at find_slot, not hold the launch."""
    torch = cuda
    pages, slots, seed, vseed = 256, 64, 13, 91
    ctrl = bam.Controller(pages * 4096, 0, queue_depth=16, num_queues=2)
    ctrl.configure(ctrl_blocks=2, spin_timeout_ns=5 * SEC)
    ctrl.set_launch_timeout(60 * SEC)
    ctrl.set_max_grid(4)                                  # two worker blocks: 16 warps x 3 lanes pin one page each at a time
    ctrl.fill_store(seed)
    cache = bam.PageCache(ctrl, 4096, slots)
    arr = bam.Array(cache, pages * 512)
    torch.cuda.synchronize()
    before = ctrl.store_numpy().copy()
    # element 1 of each of the first 128 pages is written: 128 dirty pages go through 64 slots, the last 64 stay
    idx = np.arange(128, dtype=np.uint64) * np.uint64(512) + np.uint64(1)
    d_idx = torch.from_numpy(idx.view(np.int64)).cuda()
    arr.write(len(idx), d_idx, val_seed=vseed)
    assert ctrl.status() == (0, "none", 0) and cache.audit() == 0
    with np.errstate(over="ignore"):
        new = np_splitmix64(np.uint64(vseed) ^ idx)
    only_cached = int((ctrl.store_numpy()[idx.astype(np.int64)] != new).sum())
    assert only_cached >= 32                              # these pages live only in the cache, dirty
    # 128 clean pages, pinned by lanes 0, 7 and 19 of every warp, each for itself
    first_words = torch.zeros(128, dtype=torch.int64, device="cuda")
    cache.stats(reset=True)
    arr.thread_acquire(128, 128, first_words)
    assert ctrl.status() == (0, "none", 0) and cache.audit() == 0
    got = first_words.cpu().numpy().view(np.uint64)
    assert (got == before[(128 + np.arange(128)) * 512]).all()
    # 128 misses went through 64 slots: every dirty page has reached the store by now, without a flush
    after = ctrl.store_numpy()
    assert (after[idx.astype(np.int64)] == new).all()
    want = before.copy()
    want[idx.astype(np.int64)] = new
    assert (after == want).all()
    st = cache.stats()
    assert st["misses"] == 128 and st["read_ios"] == 128 and st["hits"] == 0
    # argument checks
    with pytest.raises(bam.BamError):
        arr.thread_acquire(200, 128, first_words)         # runs past the last page of the range
    with pytest.raises(bam.BamError):
        arr.thread_acquire(0, 16, first_words, lanes=0)
    arr.close(); cache.close(); ctrl.close()
