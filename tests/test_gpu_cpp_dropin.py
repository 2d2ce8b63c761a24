"""GPU test of the C++ drop-in layer: tests/cpp/array_bench.cu is the reference's array benchmark
written with Controller / page_cache_t / range_t / array_t on the host and array_d_t<T>::operator[]
and bam_ptr<T> / bam_ptr_tlb<T> in a user kernel; its checksum must equal the oracle's.
tests/cpp/vectoradd_bench.cu is the reference's vector add (C[i] = A[i] + B[i] through three cursors),
checked on the host after a flush."""
import json
import subprocess

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def run(exe, *args):
    out = subprocess.run([exe, *map(str, args)], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    return json.loads(out.stdout.strip().splitlines()[-1])


@pytest.mark.parametrize("use_ptr", [0, 1, 2])
def test_cpp_array_bench_matches_oracle(cuda, bam, orc, use_ptr):
    from bam_b200 import _build
    exe = _build.build_cpp_bench()
    # a bam_ptr keeps one page pinned per thread, so (as with the reference) the cache needs more
    # slots than threads that hold a cursor; operator[] has no such requirement
    n_elems, threads, reqs, seed, aseed = 1 << 22, 1 << 13, 16, 11, 29
    # (with a tlb also 32 per block)
    pages = {0: 2048, 1: 16384, 2: 32768}[use_ptr]
    r = run(exe, "--num_elems", n_elems, "--pages", pages, "--threads", threads, "--reqs", reqs, "--seed", seed,
            "--access_seed", aseed, "--queue_depth", 64, "--num_queues", 8, "--bam_ptr", use_ptr)
    assert r["status"] == 0 and r["audit"] == 0
    assert r["checksum"] == orc.array_checksum(seed, n_elems, aseed, 0, threads, reqs)
    assert r["hits"] + r["misses"] == threads * reqs if not use_ptr else r["read_ios"] > 0


@pytest.mark.parametrize("use_tlb", [0, 1])
def test_cpp_vectoradd_writes_through_cursors(cuda, bam, orc, use_tlb):
    from bam_b200 import _build
    exe = _build.build_cpp_bench(name="vectoradd_bench")
    n_elems, seed = (1 << 20) + 77, 7                       # ragged last page and last warp
    r = run(exe, "--num_elems", n_elems, "--pages", 1 << 16, "--seed", seed, "--tlb", use_tlb)
    assert r["status"] == 0 and r["flush_status"] == 0 and r["audit"] == 0
    assert r["mismatches"] == 0
    a = orc.fill_store(seed, 0, n_elems)
    b = orc.fill_store(seed + 1, 0, n_elems)
    with np.errstate(over="ignore"):
        assert r["checksum"] == int((a + b).sum(dtype=np.uint64))
    assert r["read_ios"] >= 2 * (n_elems * 8 // 4096)       # A and B came in through the controller


def test_cpp_device_api(cuda, bam):
    """get_raw / release_raw, acquire_page / release_page, memcpy, bafs_ptr::memcpy_to_array_aligned,
    read_data / write_data and the asynchronous pair, each checked on the host by the program."""
    from bam_b200 import _build
    exe = _build.build_cpp_bench(name="device_api_bench")
    r = run(exe)
    assert r == {"bad_get_raw": 0, "bad_acquire_page": 0, "bad_bafs_ptr_ops": 0, "bad_memcpy": 0, "bad_raw_io": 0, "bad_async": 0,
                 "status": 0, "where": 0, "audit": 0}


def test_cpp_host_libnvm_io(cuda, bam):
    """tests/cpp/host_io_bench.cu: a host program written against the reference's libnvm names
    (nvm_ctrl / nvm_dma / nvm_aq / nvm_admin / nvm_queue) submits NVMe READ and WRITE commands from the
    host through a queue pair in host memory; the emulated controller serves them."""
    from bam_b200 import _build
    exe = _build.build_cpp_bench(name="host_io_bench")
    r = run(exe)
    assert (r["page_size"], r["max_entries"], r["sq_entry"], r["cq_entry"], r["lba"]) == (4096, 1024, 64, 16, 512)
    assert r["ns_blocks"] == (64 << 20) // 512 and r["queues"] == [4, 4]
    assert (r["sq_depth"], r["cq_depth"]) == (64, 256)        # the page-sized defaults of sq_create / cq_create
    assert r["bad_read"] == r["bad_write"] == r["bad_neighbours"] == r["bad_device_read"] == r["bad_status"] == 0
    assert r["oob_status"] == 0x80 and r["oob_cid"] == 7      # LBA out of range, generic status code type
    # transfers of 2, 37 and 21 pages: second pointer, a PRP list, a list continued in a second list page
    assert r["bad_multi"] == 0 and (r["st_two"], r["st_list"], r["st_chain"]) == (0, 0, 0)
    # a list in memory the controller was never given: data transfer error, as a packed status and as text
    assert r["st_foreign"] == -0x04 and "transfer" in r["foreign_text"]
    # nvm_raw_ctrl_init over the register window, nvm_ctrl_from_dma / _from_aq_ref, nvm_dma_remap outliving its original
    assert r["bad_handles"] == 0
    # nvm_raw_rpc: identify (into host and into GPU memory), features, refused opcodes / queue ids / memory, log pages
    assert r["bad_admin"] == 0



def test_grid_cap_travels_in_the_launch_descriptor(cuda, bam):
    """bam_ctrl_set_max_grid reaches user kernels launched through the device headers: bam::launch_fused takes
    the cap from the descriptor bam_ctrl_emu_descriptor hands out (include/bam/launch.cuh)."""
    import ctypes as C
    ctrl = bam.Controller(1 << 20, 0, queue_depth=16, num_queues=2)
    buf = (C.c_uint8 * 256)()

    def max_grid():
        assert ctrl.lib.bam_ctrl_emu_descriptor(ctrl.h, buf, 256) == 0
        # qps (8), six 32-bit fields, three pointers, n_windows, procs_per_queue, then max_grid
        return int.from_bytes(bytes(buf[64:68]), "little")

    assert max_grid() == 0
    ctrl.set_max_grid(5)
    assert max_grid() == 5
    ctrl.set_max_grid(0)
    assert max_grid() == 0
    assert ctrl.lib.bam_ctrl_emu_descriptor(ctrl.h, buf, 16) != 0       # a buffer too small for the descriptor
    ctrl.close()
