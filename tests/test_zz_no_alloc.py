"""GPU test of bam_cache_audit_noalloc, the audit for callers that cannot allocate device memory
or stall the device (a monitor thread beside running streams, a process with a single owning
allocator, a path where allocation calls are forbidden).  It must return exactly what
bam_cache_audit returns -- on a clean cache and on one a failed launch left inconsistent -- on
two calls in a row, because the fixed scratch it uses still holds the previous call's data.
Collected last on purpose: a run that stops at the first failure has then run everything else."""
import ctypes as C

import pytest

pytestmark = pytest.mark.gpu
SEC = 1_000_000_000


def both_audits(cuda, cache):
    out = cuda.full((1,), -1, dtype=cuda.int64, device="cuda")
    want = cache.audit()                                   # allocating entry point
    got = []
    for _ in range(2):                                     # two calls in a row share the scratch
        out.fill_(-1)
        cache.audit_noalloc(out, stream=cuda.cuda.current_stream().cuda_stream)
        cuda.cuda.synchronize()
        got.append(int(out.item()))
    return want, got


def test_noalloc_audit_matches_allocating_audit(cuda, bam, orc):
    n_elems, seed = 1 << 18, 11
    ctrl = bam.Controller(n_elems * 8, 0, queue_depth=8, num_queues=2)
    ctrl.configure(ctrl_blocks=1, spin_timeout_ns=SEC // 5)
    ctrl.set_launch_timeout(30 * SEC)
    ctrl.set_max_grid(4)
    ctrl.fill_store(seed)
    cache = bam.PageCache(ctrl, 4096, 20000)               # three audit blocks, ragged last one
    arr = bam.Array(cache, n_elems)
    # empty cache, then a cache with resident pages: both audits say "clean"
    want, got = both_audits(cuda, cache)
    assert want == 0 and got == [0, 0]
    out = cuda.zeros(1, dtype=cuda.int64, device="cuda")
    arr.read(512, 8, out, access_seed=29)
    assert ctrl.status() == (0, "none", 0)
    assert (int(out.item()) & ((1 << 64) - 1)) == orc.array_checksum(seed, n_elems, 29, 0, 512, 8)
    want, got = both_audits(cuda, cache)
    assert want == 0 and got == [0, 0]
    # a launch that timed out (dropped completion, injected on the controller side) leaves BUSY
    # slots and pins behind: both audits must count the same violations, twice
    cache.invalidate()                                     # every page misses again
    ctrl.inject_fault(1, nth=3)
    arr.read(512, 8, out, access_seed=31)
    code, _, _ = ctrl.status(clear=True)
    assert code == 110
    want, got = both_audits(cuda, cache)
    assert want > 0 and got == [want, want]
    arr.close(); cache.close(); ctrl.close()


def test_noalloc_audit_rejects_bad_arguments(cuda, bam):
    lib = bam.load()
    assert lib.bam_cache_audit_noalloc(None, None, None) == 22
    # the size check needs a real cache of one slot more than the scratch covers: about 4.5 GB of device
    # memory.  On a GPU that other jobs have filled, that part is skipped rather than failed.
    free_bytes, _ = cuda.cuda.mem_get_info()
    if free_bytes < 6 << 30:
        pytest.skip("less than 6 GB of device memory free: the oversize cache cannot be built")
    ctrl = bam.Controller(1 << 20, 0, queue_depth=8, num_queues=1)
    try:
        cache = bam.PageCache(ctrl, 512, 8_380_417)
    except bam.BamError as e:
        ctrl.close()
        if e.code == 12:
            pytest.skip("the oversize cache could not be allocated")
        raise
    out = cuda.zeros(1, dtype=cuda.int64, device="cuda")
    rc = lib.bam_cache_audit_noalloc(cache.h, C.c_void_p(out.data_ptr()), None)
    assert rc == 7 and b"limit" in lib.bam_strerror(rc)
    cache.close(); ctrl.close()
