"""GPU interoperability test with the REFERENCE's own host code: its classic queue functions
(nvm_sq_enqueue, nvm_sq_submit, nvm_cq_dequeue_block, nvm_sq_update, nvm_cq_update), its queue set-up
(nvm_queue_clear, doorbell offsets of src/regs.h) and its command builders -- compiled from the
reference's sources into oracle/_ref/libref_wire.so -- submit NVMe READ / WRITE commands that the
emulated controller of this library serves.  What moves must equal the media, byte for byte, and every
completion must carry what the reference's accessors expect."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
u8, u16, u32, u64, vp = C.c_uint8, C.c_uint16, C.c_uint32, C.c_uint64, C.c_void_p
PAGE = 4096


class NvmCtrl(C.Structure):                       # nvm_ctrl_t (include/bam/abi_types.h)
    _fields_ = [("page_size", C.c_size_t), ("dstrd", u8), ("timeout", u64), ("max_qs", u32), ("mm_size", C.c_size_t),
                ("mm_ptr", vp)]


class NvmDma(C.Structure):                        # nvm_dma_t without its trailing ioaddrs[]
    _fields_ = [("vaddr", vp), ("local", C.c_int8), ("contiguous", C.c_int8), ("page_size", C.c_size_t),
                ("n_ioaddrs", C.c_size_t)]


def ioaddrs(dma_ptr, n):
    return (u64 * n).from_address(dma_ptr.value + C.sizeof(NvmDma))


def test_reference_host_queue_code_drives_the_emulated_controller(cuda, bam, orc):
    ref = orc.ref_wire()
    if ref is None:
        pytest.skip("the reference's wire-format code is not built (needs the reference project)")
    lib = bam.load()
    for name, args in (("nvm_emu_ctrl_init", [C.POINTER(vp), vp]), ("nvm_aq_create", [C.POINTER(vp), vp, vp]),
                       ("nvm_dma_create", [C.POINTER(vp), vp, C.c_size_t]), ("nvm_admin_cq_create", [vp, vp, u16, vp, C.c_size_t, C.c_size_t]),
                       ("nvm_admin_sq_create", [vp, vp, vp, u16, vp, C.c_size_t, C.c_size_t]), ("nvm_admin_sq_delete", [vp, vp, vp]),
                       ("nvm_admin_cq_delete", [vp, vp])):
        getattr(lib, name).argtypes = args
        getattr(lib, name).restype = C.c_int
    for name in ("nvm_dma_unmap", "nvm_aq_destroy", "nvm_ctrl_free"):
        getattr(lib, name).argtypes = [vp]
        getattr(lib, name).restype = None

    n_media_pages, seed = 4096, 77
    emu = bam.Controller(n_media_pages * PAGE, 0, queue_depth=64, num_queues=1)
    emu.set_launch_timeout(60 * 1_000_000_000)               # the service kernel leaves after a minute at most
    media = emu.store_numpy()
    media[:] = orc.fill_store(seed, 0, n_media_pages * 512)

    nctrl, aq, qmem, buf = vp(), vp(), vp(), vp()
    assert lib.nvm_emu_ctrl_init(C.byref(nctrl), emu.h) == 0
    ctrl = NvmCtrl.from_address(nctrl.value)
    assert (ctrl.page_size, ctrl.dstrd, ctrl.max_qs) == (4096, 0, 1024) and ctrl.mm_ptr
    assert lib.nvm_aq_create(C.byref(aq), nctrl, None) == 0
    assert lib.nvm_dma_create(C.byref(qmem), nctrl, 2 * PAGE) == 0
    n_buf = 200
    assert lib.nvm_dma_create(C.byref(buf), nctrl, n_buf * PAGE) == 0
    qd, bd = NvmDma.from_address(qmem.value), NvmDma.from_address(buf.value)
    q_io, b_io = ioaddrs(qmem, 2), ioaddrs(buf, n_buf)
    # this library's side: register the queue memory with the command processor (starts the service)
    my_cq = np.zeros(4096, dtype=np.uint8)
    my_sq = np.zeros(4096, dtype=np.uint8)
    assert lib.nvm_admin_cq_create(aq, my_cq.ctypes.data, 1, qmem, 0, 0) == 0
    assert lib.nvm_admin_sq_create(aq, my_sq.ctypes.data, my_cq.ctypes.data, 1, qmem, 1, 0) == 0
    # the reference's side: its own queue descriptors over the same memory and register window
    rcq = ref.refw_queue_new(ctrl.mm_ptr, 1, 1, 256, qd.vaddr, q_io[0])
    rsq = ref.refw_queue_new(ctrl.mm_ptr, 0, 1, 64, qd.vaddr + PAGE, q_io[1])
    assert rcq and rsq
    assert ref.refw_queue_doorbell_offset(rsq) == 0x1000 + 2 * 4 and ref.refw_queue_doorbell_offset(rcq) == 0x1000 + 3 * 4

    cid, sqhd, sqid, sct, sc, packed = u16(), u16(), u16(), u8(), u8(), C.c_int()

    def service_state():
        run, code, where, served = u32(), u32(), u32(), u64()
        lib.nvm_emu_service_status.argtypes = [vp] + [vp] * 4
        rc = lib.nvm_emu_service_status(nctrl, C.byref(run), C.byref(code), C.byref(where), C.byref(served))
        sq_db = u32.from_address(ctrl.mm_ptr + 0x1008).value
        return f"service: rc {rc} running {run.value} code {code.value} where {where.value} served {served.value}, SQ doorbell {sq_db}"

    def transfer(opcode, first_media_page, n):
        sent = done = 0
        seen = []
        while done < n:
            while sent < n and ref.refw_sq_put_rw(rsq, 1000 + sent, opcode, 1, b_io[sent], 0, (first_media_page + sent) * 8, 8) == 0:
                sent += 1
            ref.refw_sq_submit(rsq)
            assert ref.refw_cq_take(rcq, rsq, 5000, C.byref(cid), C.byref(sqhd), C.byref(sqid), C.byref(sct), C.byref(sc),
                                    C.byref(packed)) == 0, "the controller did not answer; " + service_state()
            assert (sqid.value, sct.value, sc.value, packed.value) == (1, 0, 0, 0) and sqhd.value < 64
            seen.append(cid.value)
            done += 1
        assert sorted(seen) == list(range(1000, 1000 + n))     # every command completed exactly once
        assert sent == n

    data = np.frombuffer((C.c_uint8 * (n_buf * PAGE)).from_address(bd.vaddr), dtype=np.uint64)
    # READ 200 pages (several wraps of the 64-entry SQ) and compare with the media
    transfer(2, 300, n_buf)
    assert (data == media[300 * 512: (300 + n_buf) * 512]).all()
    # WRITE them somewhere else, READ that back
    data[:] = orc.fill_store(seed + 1, 0, n_buf * 512)
    transfer(1, 2000, n_buf)
    assert (media[2000 * 512: (2000 + n_buf) * 512] == orc.fill_store(seed + 1, 0, n_buf * 512)).all()
    assert media[2000 * 512 - 1] == orc.fill_store(seed, 2000 * 512 - 1, 1)[0]            # neighbours untouched
    data[:] = 0
    transfer(2, 2000, n_buf)
    assert (data == orc.fill_store(seed + 1, 0, n_buf * 512)).all()
    # a read beyond the namespace: generic status "LBA out of range", which the reference packs as -0x80
    assert ref.refw_sq_put_rw(rsq, 7, 2, 1, b_io[0], 0, n_media_pages * 8, 8) == 0
    ref.refw_sq_submit(rsq)
    assert ref.refw_cq_take(rcq, rsq, 5000, C.byref(cid), C.byref(sqhd), C.byref(sqid), C.byref(sct), C.byref(sc), C.byref(packed)) == 0
    assert (cid.value, sct.value, sc.value, packed.value) == (7, 0, 0x80, -0x80)
    assert b"range" in ref.refw_strerror(packed.value).lower()
    # a data pointer outside every DMA mapping is refused (data transfer error), not followed
    assert ref.refw_sq_put_rw(rsq, 8, 2, 1, 0x10000, 0, 0, 8) == 0
    ref.refw_sq_submit(rsq)
    assert ref.refw_cq_take(rcq, rsq, 5000, C.byref(cid), C.byref(sqhd), C.byref(sqid), C.byref(sct), C.byref(sc), C.byref(packed)) == 0
    assert (cid.value, sct.value, sc.value) == (8, 0, 0x04)
    # so is a page-crossing transfer whose second pointer is missing
    assert ref.refw_sq_put_rw(rsq, 9, 2, 1, b_io[0] + 512, 0, 0, 8) == 0
    ref.refw_sq_submit(rsq)
    assert ref.refw_cq_take(rcq, rsq, 5000, C.byref(cid), C.byref(sqhd), C.byref(sqid), C.byref(sct), C.byref(sc), C.byref(packed)) == 0
    assert (cid.value, sc.value) == (9, 0x04)

    ref.refw_queue_free(rsq); ref.refw_queue_free(rcq)
    assert lib.nvm_admin_sq_delete(aq, my_sq.ctypes.data, my_cq.ctypes.data) == 0
    assert lib.nvm_admin_cq_delete(aq, my_cq.ctypes.data) == 0
    del data
    lib.nvm_dma_unmap(buf); lib.nvm_dma_unmap(qmem)
    lib.nvm_aq_destroy(aq)
    lib.nvm_ctrl_free(nctrl)
    emu.close()


def test_reference_parallel_queue_code_drives_the_emulated_controller(cuda, bam, orc):
    """The protocol the reference's GPU threads run -- get_cid, sq_enqueue with ticketed slots and batched
    doorbells, cq_poll by command id and phase, cq_dequeue with SQ-head propagation, put_cid
    (include/nvm_parallel_queue.h, compiled for the host into oracle/_ref/libref_pq.so) -- executed by 16 host
    threads sharing one queue pair, against the emulated controller on the GPU."""
    pq = orc.ref_pq()
    if pq is None:
        pytest.skip("the reference's queue code is not built (needs the reference project)")
    lib = bam.load()
    for name, args in (("nvm_emu_ctrl_init", [C.POINTER(vp), vp]), ("nvm_aq_create", [C.POINTER(vp), vp, vp]),
                       ("nvm_dma_create", [C.POINTER(vp), vp, C.c_size_t]), ("nvm_admin_cq_create", [vp, vp, u16, vp, C.c_size_t, C.c_size_t]),
                       ("nvm_admin_sq_create", [vp, vp, vp, u16, vp, C.c_size_t, C.c_size_t]), ("nvm_admin_sq_delete", [vp, vp, vp]),
                       ("nvm_admin_cq_delete", [vp, vp])):
        getattr(lib, name).argtypes = args
        getattr(lib, name).restype = C.c_int
    for name in ("nvm_dma_unmap", "nvm_aq_destroy", "nvm_ctrl_free"):
        getattr(lib, name).argtypes = [vp]
        getattr(lib, name).restype = None
    n_media_pages, seed, qs = 8192, 91, 64
    emu = bam.Controller(n_media_pages * PAGE, 0, queue_depth=64, num_queues=1)
    emu.set_launch_timeout(60 * 1_000_000_000)
    media = emu.store_numpy()
    media[:] = orc.fill_store(seed, 0, n_media_pages * 512)
    nctrl, aq, qmem, buf = vp(), vp(), vp(), vp()
    assert lib.nvm_emu_ctrl_init(C.byref(nctrl), emu.h) == 0
    ctrl = NvmCtrl.from_address(nctrl.value)
    assert lib.nvm_aq_create(C.byref(aq), nctrl, None) == 0
    assert lib.nvm_dma_create(C.byref(qmem), nctrl, 2 * PAGE) == 0
    n_req = 3000
    assert lib.nvm_dma_create(C.byref(buf), nctrl, n_req * PAGE) == 0
    qd, bd = NvmDma.from_address(qmem.value), NvmDma.from_address(buf.value)
    q_io, b_io = ioaddrs(qmem, 2), ioaddrs(buf, n_req)
    my_cq, my_sq = np.zeros(4096, dtype=np.uint8), np.zeros(4096, dtype=np.uint8)
    assert lib.nvm_admin_cq_create(aq, my_cq.ctypes.data, 1, qmem, 0, qs) == 0
    assert lib.nvm_admin_sq_create(aq, my_sq.ctypes.data, my_cq.ctypes.data, 1, qmem, 1, qs) == 0
    pair = pq.refpq_pair_new(ctrl.mm_ptr, 1, qs, qd.vaddr + PAGE, q_io[1], qs, qd.vaddr, q_io[0], 1)
    assert pair
    rng = np.random.default_rng(3)
    pages = rng.integers(0, n_media_pages, n_req, dtype=np.uint64)
    lbas = np.ascontiguousarray(pages * np.uint64(8))
    prps = np.ascontiguousarray(np.array(b_io[:n_req], dtype=np.uint64))
    data = np.frombuffer((C.c_uint8 * (n_req * PAGE)).from_address(bd.vaddr), dtype=np.uint64).reshape(n_req, 512)
    # 3000 random page reads by 16 threads through a 64-entry queue pair: dozens of wraps, batched doorbells
    assert pq.refpq_run(pair, 16, 2, lbas.ctypes.data, prps.ctypes.data, 8, n_req, 30000) == 0, "the protocol stalled"
    assert (data == media.reshape(-1, 512)[pages.astype(np.int64)]).all()
    sq_head, sq_tail, cq_head, cq_tail, in_ticket = (u32() for _ in range(5))
    pq.refpq_state(pair, *(C.byref(x) for x in (sq_head, sq_tail, cq_head, cq_tail, in_ticket)))
    # the reference's own view afterwards: every ticket was published, every completion consumed, SQ head caught up
    assert in_ticket.value == n_req and sq_tail.value == n_req and cq_head.value == n_req
    assert sq_head.value == n_req
    # writes: distinct target pages, then read them back through the same code
    targets = rng.permutation(n_media_pages)[:n_req].astype(np.uint64)
    data[:] = orc.fill_store(seed + 5, 0, n_req * 512).reshape(n_req, 512)
    want = data.copy()
    wl = np.ascontiguousarray(targets * np.uint64(8))
    assert pq.refpq_run(pair, 16, 1, wl.ctypes.data, prps.ctypes.data, 8, n_req, 30000) == 0
    assert (media.reshape(-1, 512)[targets.astype(np.int64)] == want).all()
    data[:] = 0
    assert pq.refpq_run(pair, 7, 2, wl.ctypes.data, prps.ctypes.data, 8, n_req, 30000) == 0
    assert (data == want).all()
    pq.refpq_pair_free(pair)
    assert lib.nvm_admin_sq_delete(aq, my_sq.ctypes.data, my_cq.ctypes.data) == 0
    assert lib.nvm_admin_cq_delete(aq, my_cq.ctypes.data) == 0
    del data
    lib.nvm_dma_unmap(buf); lib.nvm_dma_unmap(qmem)
    lib.nvm_aq_destroy(aq)
    lib.nvm_ctrl_free(nctrl)
    emu.close()


def test_reference_array_read_path_end_to_end_on_the_emulated_controller(cuda, bam, orc):
    """The reference's whole read path -- array_d_t::seq_read, its page cache (acquire_page, find_slot with
    evictions), read_data with enqueue_second, its parallel queues -- compiled for host threads
    (oracle/_ref/libref_cache.so), with its cache memory and queue pairs in DMA-mapped host memory, served by
    the emulated controller on the GPU: 8 threads, a cache a fraction of the data, the result oracle's sum."""
    rc_lib = orc.ref_cache()
    if rc_lib is None:
        pytest.skip("the reference's cache code is not built (needs the reference project)")
    lib = bam.load()
    for name, args in (("nvm_emu_ctrl_init", [C.POINTER(vp), vp]), ("nvm_aq_create", [C.POINTER(vp), vp, vp]),
                       ("nvm_dma_create", [C.POINTER(vp), vp, C.c_size_t]), ("nvm_admin_cq_create", [vp, vp, u16, vp, C.c_size_t, C.c_size_t]),
                       ("nvm_admin_sq_create", [vp, vp, vp, u16, vp, C.c_size_t, C.c_size_t]), ("nvm_admin_sq_delete", [vp, vp, vp]),
                       ("nvm_admin_cq_delete", [vp, vp])):
        getattr(lib, name).argtypes = args
        getattr(lib, name).restype = C.c_int
    for name in ("nvm_dma_unmap", "nvm_aq_destroy", "nvm_ctrl_free"):
        getattr(lib, name).argtypes = [vp]
        getattr(lib, name).restype = None
    n_media_pages, seed, n_qps, qs, n_slots = 2048, 57, 3, 16, 96
    emu = bam.Controller(n_media_pages * PAGE, 0, queue_depth=64, num_queues=1)
    emu.set_launch_timeout(60 * 1_000_000_000)
    emu.store_numpy()[:] = orc.fill_store(seed, 0, n_media_pages * 512)
    nctrl, aq, qmem, cmem = vp(), vp(), vp(), vp()
    assert lib.nvm_emu_ctrl_init(C.byref(nctrl), emu.h) == 0
    ctrl = NvmCtrl.from_address(nctrl.value)
    assert lib.nvm_aq_create(C.byref(aq), nctrl, None) == 0
    assert lib.nvm_dma_create(C.byref(qmem), nctrl, 2 * n_qps * PAGE) == 0
    assert lib.nvm_dma_create(C.byref(cmem), nctrl, n_slots * PAGE) == 0          # the reference's cache lives in DMA memory
    qd, cd = NvmDma.from_address(qmem.value), NvmDma.from_address(cmem.value)
    q_io, c_io = ioaddrs(qmem, 2 * n_qps), ioaddrs(cmem, n_slots)
    mine = [(np.zeros(4096, dtype=np.uint8), np.zeros(4096, dtype=np.uint8)) for _ in range(n_qps)]
    for q, (my_cq, my_sq) in enumerate(mine):                                     # page 2q: CQ q+1, page 2q+1: SQ q+1
        assert lib.nvm_admin_cq_create(aq, my_cq.ctypes.data, q + 1, qmem, 2 * q, qs) == 0
        assert lib.nvm_admin_sq_create(aq, my_sq.ctypes.data, my_cq.ctypes.data, q + 1, qmem, 2 * q + 1, qs) == 0
    sq = (vp * n_qps)(*[qd.vaddr + (2 * q + 1) * PAGE for q in range(n_qps)])
    cq = (vp * n_qps)(*[qd.vaddr + (2 * q) * PAGE for q in range(n_qps)])
    world = rc_lib.refc_new2(ctrl.mm_ptr, n_qps, qs, sq, cq, PAGE, n_slots, n_media_pages, 512, cd.vaddr, c_io[0])
    assert world
    idx = np.random.default_rng(6).integers(0, n_media_pages * 512, 12000, dtype=np.uint64)
    st = orc.RefCacheStats()
    assert rc_lib.refc_array_read(world, idx.ctypes.data, len(idx), 8, 60000, C.byref(st)) == 0, "the read path stalled"
    assert st.checksum == orc.indexed_checksum(seed, 0, idx)
    assert st.accesses == len(idx) and st.hits + st.misses == len(idx) and st.read_ios == st.misses and st.misses > n_slots
    rc_lib.refc_free(world)
    for my_cq, my_sq in mine:
        assert lib.nvm_admin_sq_delete(aq, my_sq.ctypes.data, my_cq.ctypes.data) == 0
        assert lib.nvm_admin_cq_delete(aq, my_cq.ctypes.data) == 0
    lib.nvm_dma_unmap(cmem); lib.nvm_dma_unmap(qmem)
    lib.nvm_aq_destroy(aq)
    lib.nvm_ctrl_free(nctrl)
    emu.close()


def test_device_command_encoding_equals_the_reference_builders(cuda, bam, orc):
    """The register-built command of the device submission paths, run in a kernel, against the reference's
    nvm_cmd_header / nvm_cmd_data_ptr / nvm_cmd_rw_blks."""
    ref = orc.ref_wire()
    if ref is None:
        pytest.skip("the reference's wire-format code is not built (needs the reference project)")
    lib = bam.load()
    rng = np.random.default_rng(5)
    for _ in range(40):
        cidv, opc, ns = int(rng.integers(0, 1 << 16)), int(rng.choice([1, 2])), int(rng.integers(1, 1 << 32))
        prp1, prp2, lba = (int(x) for x in rng.integers(0, 1 << 63, 3, dtype=np.uint64))
        nb = int(rng.integers(1, 1 << 16))
        want, got = (C.c_uint8 * 64)(), (C.c_uint8 * 64)()
        ref.refw_encode_rw(cidv, opc, ns, prp1, prp2, lba, nb, want)
        assert lib.bam_encode_rw_command(got, cidv, opc, ns, prp1, prp2, lba, nb, 1) == 0
        assert bytes(got) == bytes(want)


class NvmCtrlInfo(C.Structure):                   # struct nvm_ctrl_info (include/nvm_types.h:198-216 of the reference)
    _fields_ = [("nvme_version", u32), ("page_size", C.c_size_t), ("db_stride", C.c_size_t), ("timeout", u64), ("contiguous", C.c_int),
                ("max_entries", u16), ("pci_vendor", u8 * 4), ("serial_no", C.c_char * 20), ("model_no", C.c_char * 40),
                ("firmware", C.c_char * 8), ("max_data_size", C.c_size_t), ("max_data_pages", C.c_size_t), ("cq_entry_size", C.c_size_t),
                ("sq_entry_size", C.c_size_t), ("max_out_cmds", C.c_size_t), ("max_n_ns", C.c_size_t)]


class NvmNsInfo(C.Structure):                     # struct nvm_ns_info (:225-233 there)
    _fields_ = [("ns_id", u32), ("size", C.c_size_t), ("capacity", C.c_size_t), ("utilization", C.c_size_t),
                ("lba_data_size", C.c_size_t), ("metadata_size", C.c_size_t)]


def test_reference_admin_layer_over_the_pass_through(cuda, bam, orc):
    """The reference's whole host stack above nvm_raw_rpc -- src/admin.cpp building the admin commands and parsing
    the identify pages, src/queue.cpp setting the queue descriptors up, include/nvm_queue.h driving them --
    compiled from the reference's sources (oracle/_ref/libref_admin.so), with nvm_raw_rpc bound to this
    library: the emulated controller executes the admin commands and then serves the queue pair the
    reference's code created."""
    ra = orc.ref_admin()
    if ra is None:
        pytest.skip("the reference's admin layer is not built (needs the reference project)")
    lib = bam.load()
    for name, args in (("nvm_emu_ctrl_init", [C.POINTER(vp), vp]), ("nvm_aq_create", [C.POINTER(vp), vp, vp]),
                       ("nvm_dma_create", [C.POINTER(vp), vp, C.c_size_t]), ("nvm_admin_ctrl_info", [vp, vp, vp, u64]),
                       ("nvm_admin_ns_info", [vp, vp, u32, vp, u64]), ("nvm_admin_get_num_queues", [vp, C.POINTER(u16), C.POINTER(u16)])):
        getattr(lib, name).argtypes = args
        getattr(lib, name).restype = C.c_int
    for name in ("nvm_dma_unmap", "nvm_aq_destroy", "nvm_ctrl_free"):
        getattr(lib, name).argtypes = [vp]
        getattr(lib, name).restype = None
    ra.refa_bind(C.cast(lib.nvm_raw_rpc, vp), C.cast(lib.nvm_ctrl_from_aq_ref, vp))

    n_media_pages, seed = 2048, 91
    emu = bam.Controller(n_media_pages * PAGE, 0, queue_depth=64, num_queues=1)
    emu.set_launch_timeout(60 * 1_000_000_000)               # the service kernel leaves after a minute at most
    media = emu.store_numpy()
    media[:] = orc.fill_store(seed, 0, n_media_pages * 512)
    nctrl, aq, qmem, buf = vp(), vp(), vp(), vp()
    assert lib.nvm_emu_ctrl_init(C.byref(nctrl), emu.h) == 0
    ctrl = NvmCtrl.from_address(nctrl.value)
    assert lib.nvm_aq_create(C.byref(aq), nctrl, None) == 0
    assert lib.nvm_dma_create(C.byref(qmem), nctrl, 2 * PAGE) == 0
    assert lib.nvm_dma_create(C.byref(buf), nctrl, 4 * PAGE) == 0
    bd = NvmDma.from_address(buf.value)
    b_io = ioaddrs(buf, 4)

    # identify: the reference's parse of the pages the controller returns == this library's own answer
    theirs, mine = NvmCtrlInfo(), NvmCtrlInfo()
    assert ra.refa_ctrl_info(aq, C.byref(theirs), bd.vaddr, b_io[0]) == 0
    assert lib.nvm_admin_ctrl_info(aq, C.byref(mine), bd.vaddr + PAGE, b_io[1]) == 0
    assert bytes(theirs) == bytes(mine)
    assert (theirs.nvme_version, theirs.page_size, theirs.max_entries, theirs.timeout, theirs.contiguous) == (0x00010400, 4096, 1024, 5000, 1)
    assert (theirs.max_data_size, theirs.sq_entry_size, theirs.cq_entry_size, theirs.max_n_ns) == (1 << 20, 64, 16, 1)
    assert theirs.serial_no.startswith(b"BAMB200EMU")
    ns_theirs, ns_mine = NvmNsInfo(), NvmNsInfo()
    assert ra.refa_ns_info(aq, C.byref(ns_theirs), 1, bd.vaddr, b_io[0]) == 0
    assert lib.nvm_admin_ns_info(aq, C.byref(ns_mine), 1, bd.vaddr + PAGE, b_io[1]) == 0
    assert bytes(ns_theirs) == bytes(ns_mine)
    assert (ns_theirs.size, ns_theirs.lba_data_size, ns_theirs.metadata_size) == (n_media_pages * 8, 512, 0)
    assert ra.refa_ns_info(aq, C.byref(ns_theirs), 3, bd.vaddr, b_io[0]) == -0x00b          # invalid namespace, as a packed status

    # number of queues: set by the reference's code (3 completion, 5 submission queues), read back by both.  The
    # controller answers as the NVMe specification lays the result out (completion queues in the upper half);
    # the reference reads the halves the other way round (src/admin.cpp:466-467, 503-504), on any controller
    ncq, nsq = u16(3), u16(5)
    assert ra.refa_request_num_queues(aq, C.byref(ncq), C.byref(nsq)) == 0 and (ncq.value, nsq.value) == (5, 3)
    ncq2, nsq2 = u16(), u16()
    assert lib.nvm_admin_get_num_queues(aq, C.byref(ncq2), C.byref(nsq2)) == 0 and (ncq2.value, nsq2.value) == (3, 5)

    # a queue pair created by the reference's code (its descriptors, its commands), page-sized defaults
    rcq, rsq, extra = ra.refa_queue_alloc(), ra.refa_queue_alloc(), ra.refa_queue_alloc()
    assert ra.refa_cq_create(aq, extra, 9, qmem, 0, 0) == -0x101                              # queue 9 was never granted
    assert ra.refa_cq_create(aq, rcq, 1, qmem, 0, 0) == 0 and ra.refa_queue_qs(rcq) == 256
    assert ra.refa_sq_create(aq, rsq, rcq, 1, qmem, 1, 0) == 0 and ra.refa_queue_qs(rsq) == 64
    assert ra.refa_queue_doorbell_offset(rsq, ctrl.mm_ptr) == 0x1008 and ra.refa_queue_doorbell_offset(rcq, ctrl.mm_ptr) == 0x100c
    assert ra.refa_cq_delete(aq, rcq) == -0x10c                                               # its submission queue still exists
    data = np.frombuffer((C.c_uint8 * (4 * PAGE)).from_address(bd.vaddr), dtype=np.uint64)
    for k in range(150):                                                                      # more than two wraps of the 64-entry SQ
        page = (k * 37) % n_media_pages
        assert ra.refa_rw(rsq, rcq, 2, 1, b_io[k & 3], page * 8, 8, 5000) == 0, k
        assert (data[(k & 3) * 512:(k & 3) * 512 + 512] == media[page * 512:(page + 1) * 512]).all(), k
    data[:512] = orc.fill_store(seed + 1, 0, 512)
    assert ra.refa_rw(rsq, rcq, 1, 1, b_io[0], 700 * 8, 8, 5000) == 0                         # WRITE
    assert (media[700 * 512:701 * 512] == orc.fill_store(seed + 1, 0, 512)).all()
    assert ra.refa_rw(rsq, rcq, 2, 1, b_io[0], n_media_pages * 8, 8, 5000) == -0x80           # LBA out of range
    assert ra.refa_sq_delete(aq, rsq, rcq) == 0 and ra.refa_cq_delete(aq, rcq) == 0
    del data
    for q in (rcq, rsq, extra):
        ra.refa_queue_free(q)
    lib.nvm_dma_unmap(buf); lib.nvm_dma_unmap(qmem)
    lib.nvm_aq_destroy(aq)
    lib.nvm_ctrl_free(nctrl)
    emu.close()
