"""GPU test of the C++ drop-in layer: tests/cpp/array_bench.cu is the reference's array benchmark
written with Controller / page_cache_t / range_t / array_t on the host and array_d_t<T>::operator[]
and bam_ptr<T> in a user kernel.  Its checksum must equal the oracle's."""
import json
import subprocess

import pytest

pytestmark = pytest.mark.gpu


def run(exe, *args):
    out = subprocess.run([exe, *map(str, args)], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    return json.loads(out.stdout.strip().splitlines()[-1])


@pytest.mark.parametrize("use_ptr", [0, 1])
def test_cpp_array_bench_matches_oracle(cuda, bam, orc, use_ptr):
    from bam_b200 import _build
    exe = _build.build_cpp_bench()
    # a bam_ptr keeps one page pinned per thread, so (as with the reference) the cache needs more
    # slots than threads that hold a cursor; operator[] has no such requirement
    n_elems, threads, reqs, seed, aseed = 1 << 22, 1 << 13, 16, 11, 29
    pages = 16384 if use_ptr else 2048
    r = run(exe, "--num_elems", n_elems, "--pages", pages, "--threads", threads, "--reqs", reqs, "--seed", seed,
            "--access_seed", aseed, "--queue_depth", 64, "--num_queues", 8, "--bam_ptr", use_ptr)
    assert r["status"] == 0 and r["audit"] == 0
    assert r["checksum"] == orc.array_checksum(seed, n_elems, aseed, 0, threads, reqs)
    assert r["hits"] + r["misses"] == threads * reqs if not use_ptr else r["read_ios"] > 0
