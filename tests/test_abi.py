"""CPU tests of the C-ABI boundary: the library loads, exports every symbol the header declares,
the ctypes table covers the header, arguments are validated, and without a GPU the product path
fails loudly instead of falling back to anything."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    src = open(os.path.join(ROOT, "include", "bam_abi.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    names = re.findall(r"\b(bam_[a-z0-9_]+)\s*\(", src)
    return sorted(set(names))


def test_header_symbols_are_exported(bam):
    from bam_b200 import _lib
    lib = C.CDLL(_lib.LIB_PATH)
    names = declared_functions()
    assert len(names) >= 30
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/bam_abi.h but not exported"


def test_host_libnvm_symbols_are_exported(bam):
    """Every function include/nvm_host_api.h declares (and does not define inline) is exported."""
    from bam_b200 import _lib
    lib = C.CDLL(_lib.LIB_PATH)
    src = open(os.path.join(ROOT, "include", "nvm_host_api.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    src = src[: src.index("static inline")]                 # the classic queue functions are header-only
    names = sorted(set(re.findall(r"\b(nvm_[a-z0-9_]+)\s*\(", src)))
    names += ["nvm_queue_clear", "nvm_queue_reset", "nvm_cq_dequeue_block", "nvm_strerror"]
    for n in ("nvm_raw_ctrl_init", "nvm_raw_ctrl_reset", "nvm_dma_remap", "nvm_ctrl_from_dma", "nvm_ctrl_from_aq_ref", "nvm_rpc_unbind"):
        assert n in names, n
    assert len(names) >= 32
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/nvm_host_api.h but not exported"
    ctrl = C.c_void_p()
    assert lib.nvm_ctrl_init(C.byref(ctrl), 3) == 19        # ENODEV: there is no kernel module behind a descriptor
    assert lib.nvm_emu_ctrl_init(C.byref(ctrl), None) == 22
    buf = (C.c_uint8 * 0x2000)()
    assert lib.nvm_raw_ctrl_init(C.byref(ctrl), buf, 0x2000) == 19 and not ctrl.value     # not the register window of any controller
    assert lib.nvm_raw_ctrl_init(C.byref(ctrl), buf, 0x1000) == 22                         # smaller than the registers
    assert lib.nvm_dma_remap(C.byref(ctrl), None) == 22
    lib.nvm_strerror.restype = C.c_char_p
    assert lib.nvm_strerror(-0x80) == b"NVMe: LBA out of range" and lib.nvm_strerror(0) == b"success"
    assert lib.nvm_strerror(-0x281) == b"NVMe: unrecovered read error" and lib.nvm_strerror(22) == b"invalid argument"


def test_ctypes_table_covers_header(bam):
    from bam_b200 import _lib
    assert sorted(_lib.SIGNATURES) == declared_functions()


def test_no_oracle_in_product():
    """Nothing under bam_b200/ or include/ may reference the oracle."""
    for base in ("bam_b200", "include"):
        for d, _, files in os.walk(os.path.join(ROOT, base)):
            for f in files:
                if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                    assert "oracle" not in open(os.path.join(d, f), errors="ignore").read().lower(), f


def test_argument_validation(bam):
    lib = bam.load()
    h = C.c_void_p()
    EINVAL = 22
    assert lib.bam_ctrl_create(None, 0, 1 << 20, 512, 1, 64) == EINVAL
    assert lib.bam_ctrl_create(C.byref(h), 0, 1 << 20, 513, 1, 64) == EINVAL      # block size
    assert lib.bam_ctrl_create(C.byref(h), 0, 1 << 20, 512, 0, 64) == EINVAL      # no queues
    assert lib.bam_ctrl_create(C.byref(h), 0, 1 << 20, 512, 1, 48) == EINVAL      # depth not 2^k
    assert lib.bam_ctrl_create(C.byref(h), 0, 1 << 20, 512, 1, 2048) == EINVAL    # depth > 1024
    assert lib.bam_ctrl_create(C.byref(h), 0, 1000, 512, 1, 64) == EINVAL         # store not page multiple
    assert lib.bam_cache_create(C.byref(h), None, 4096, 16) == EINVAL
    assert lib.bam_array_create(C.byref(h), None, 16, 8, 0) == EINVAL
    assert lib.bam_launch_array_read(None, 1, 1, None, 0, None, None) == EINVAL
    assert lib.bam_launch_block_read(None, 1, None, 0, None, None, None) == EINVAL
    assert lib.bam_ctrl_status(None, None, 0) == EINVAL
    assert b"invalid" in lib.bam_strerror(EINVAL)


def test_fails_loudly_without_gpu(bam):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(bam.BamError) as e:
        bam.Controller(1 << 20, 0, queue_depth=64, num_queues=1)
    assert e.value.code == 1000            # BAM_ECUDA: no fallback path exists


def test_shard_pages(bam):
    for n, w in [(10, 3), (1 << 24, 8), (7, 8), (16, 1)]:
        spans = [bam.shard_pages(n, w, r) for r in range(w)]
        assert spans[0][0] == 0 and sum(c for _, c in spans) == n
        for (a, ca), (b, _) in zip(spans, spans[1:]):
            assert a + ca == b


def test_bel_file_round_trip(bam, tmp_path):
    """The reference's on-disk CSR format (.bel.col / .bel.dst: 16-byte header {count, 8} + int64)."""
    import numpy as np
    off = np.array([0, 2, 3, 3, 6], dtype=np.int64)
    dst = np.array([1, 3, 0, 0, 1, 2], dtype=np.int64)
    prefix = str(tmp_path / "g")
    bam.write_bel(prefix + ".bel.col", off)
    bam.write_bel(prefix + ".bel.dst", dst)
    raw = open(prefix + ".bel.col", "rb").read()
    assert len(raw) == 16 + 8 * len(off) and np.frombuffer(raw[:16], dtype="<u8").tolist() == [len(off), 8]
    assert (bam.read_bel(prefix + ".bel.col") == off).all() and (bam.read_bel(prefix + ".bel.dst") == dst).all()
    open(prefix + ".bad", "wb").write(raw[:-8])
    import pytest
    with pytest.raises(ValueError):
        bam.read_bel(prefix + ".bad")


def test_reference_include_list_compiles(tmp_path):
    """tests/cpp/include_compat.cu includes the headers a benchmark of the reference includes, under
    the reference's names, and touches the types they must provide (compile only, no GPU)."""
    import shutil
    import subprocess
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not available")
    src = os.path.join(ROOT, "tests", "cpp", "include_compat.cu")
    res = subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-I" + os.path.join(ROOT, "include"),
                          "-c", src, "-o", str(tmp_path / "include_compat.o")], capture_output=True, text=True)
    assert res.returncode == 0, res.stderr

