"""CPU tests of the oracle: pins it against published known-answer vectors and against
independent re-computations (numpy, zlib, scipy), then against the committed golden fixtures.

The reference has no golden vectors for this path, so these pins are what anchors parity."""
import hashlib
import json
import os
import zlib

import ctypes as C

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "golden.json")))
M64 = (1 << 64) - 1


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def np_splitmix64(x):
    """Independent numpy SplitMix64 output function (state already advanced by the caller? no:
    adds the golden gamma first, like the generator)."""
    x = (np.asarray(x, dtype=np.uint64) + np.uint64(0x9E3779B97F4A7C15))
    z = (x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def py_pcg32(initstate, initseq, n):
    """Pure-Python PCG32 (XSH-RR), written from the published description."""
    mult = 6364136223846793005
    inc = ((initseq << 1) | 1) & M64
    state = 0

    def step():
        nonlocal state
        old = state
        state = (old * mult + inc) & M64
        xs = (((old >> 18) ^ old) >> 27) & 0xFFFFFFFF
        rot = old >> 59
        return ((xs >> rot) | (xs << ((-rot) & 31))) & 0xFFFFFFFF

    step()
    state = (state + initstate) & M64
    step()
    return [step() for _ in range(n)]


def test_splitmix64_known_answers(orc):
    # first outputs of SplitMix64 seeded with 1234567 (the generator's published test vector)
    want = [6457827717110365317, 3203168211198807973, 9817491932198370423, 4593380528125082431, 16408922859458223821]
    state = 1234567
    for w in want:
        assert orc.splitmix64(state) == w
        state = (state + 0x9E3779B97F4A7C15) & M64


def test_splitmix64_matches_numpy(orc):
    seed = 0xC0FFEE
    got = orc.fill_store(seed, 1000, 4096)
    with np.errstate(over="ignore"):
        want = np_splitmix64(np.uint64(seed) ^ np.arange(1000, 1000 + 4096, dtype=np.uint64))
    assert (got == want).all()


def test_pcg32_demo_vector(orc):
    # pcg32-demo: seed (42, 54) -> first six outputs
    want = [0xA15C02B7, 0x7B47F409, 0xBA1D3330, 0x83D2F293, 0xBFA4784B, 0xCBED606E]
    assert orc.pcg32_stream(42, 54, 6).tolist() == want
    assert py_pcg32(42, 54, 6) == want


@pytest.mark.parametrize("state,seq", [(0, 0), (29, 511), (0xDEADBEEF, 1 << 40)])
def test_pcg32_matches_python(orc, state, seq):
    assert orc.pcg32_stream(state, seq, 32).tolist() == py_pcg32(state, seq, 32)


def test_crc32_check_value_and_zlib(orc):
    assert orc.crc32(b"123456789") == 0xCBF43926
    rng = np.random.default_rng(1)
    for n in (0, 1, 15, 16, 4096):
        b = rng.integers(0, 256, n, dtype=np.uint8).tobytes()
        assert orc.crc32(b) == zlib.crc32(b)


def test_page_crc_matches_zlib(orc):
    for seed, page, nbytes in [(11, 0, 4096), (11, 77, 4096), (5, 3, 512), (5, 3, 8192)]:
        words = orc.fill_store(seed, page * (nbytes // 8), nbytes // 8)
        assert orc.page_crc(seed, page, nbytes) == zlib.crc32(words.tobytes())


def test_array_indices_and_checksum(orc):
    n_elems, seed, aseed, lanes, reqs = 1 << 20, 7, 99, 300, 9
    idx = orc.array_indices(aseed, n_elems, 0, lanes, reqs)
    # independent: lane l draws (hi, lo) pairs from PCG32 stream l
    for l in (0, 1, 299):
        d = py_pcg32(aseed, l, 2 * reqs)
        want = [(((d[2 * k] << 32) | d[2 * k + 1]) & (n_elems - 1)) for k in range(reqs)]
        assert idx[l * reqs:(l + 1) * reqs].tolist() == want
    store = orc.fill_store(seed, 0, n_elems)
    want = int(store[idx].sum(dtype=np.uint64))
    assert orc.array_checksum(seed, n_elems, aseed, 0, lanes, reqs) == want
    assert orc.indexed_checksum(seed, 0, idx) == want
    # non power of two: modulo rule
    idx2 = orc.array_indices(aseed, 1000003, 5, 6, 4)
    d = py_pcg32(aseed, 5, 8)
    assert idx2.tolist() == [(((d[2 * k] << 32) | d[2 * k + 1]) % 1000003) for k in range(4)]


def test_lane_split_is_additive(orc):
    a = orc.array_checksum(3, 1 << 18, 4, 0, 100, 5)
    b = orc.array_checksum(3, 1 << 18, 4, 100, 257, 5)
    assert (a + b) & M64 == orc.array_checksum(3, 1 << 18, 4, 0, 257, 5)


@pytest.mark.parametrize("n", [1, 2, 7, 64, 1000, 4096, 100003])
def test_permutation_is_bijection(orc, n):
    out = np.array([orc.lib().orc_permute(x, n, 17) for x in range(n)], dtype=np.uint64)
    assert sorted(out.tolist()) == list(range(n))


def test_zipf_cdf_and_ranks(orc):
    n = 1 << 10
    cdf = orc.zipf_cdf(n)
    assert (np.diff(cdf.astype(np.float64)) >= 0).all() and cdf[-1] == np.uint64(M64)
    idx = orc.zipf_indices(cdf, n, 512, 17, 23, 0, 256, 64)
    pages = idx // 512
    assert pages.max() < n and (idx % 512).max() < 512
    # the most popular rank maps to permute(0); it must be the most frequent page
    top = orc.lib().orc_permute(0, n, 17)
    counts = np.bincount(pages.astype(np.int64), minlength=n)
    assert counts.argmax() == top
    # rank-1 probability ~ 1/H(n, 0.99)
    p1 = 1.0 / (np.arange(1, n + 1, dtype=np.float64) ** -0.99).sum()
    assert abs(counts[top] / len(idx) - p1) < 0.02


def _scipy_graph(off, cols):
    import scipy.sparse as sp
    n = len(off) - 1
    return sp.csr_matrix((np.ones(len(cols), dtype=np.int8), cols.astype(np.int64), off.astype(np.int64)), shape=(n, n))


@pytest.mark.parametrize("scale,seed", [(8, 1), (10, 2)])
def test_rmat_csr_properties_and_scipy(orc, scale, seed):
    from scipy.sparse import csgraph
    off, cols = orc.rmat_csr(seed, scale, 16)
    n = 1 << scale
    assert off[0] == 0 and off[-1] == len(cols) and (np.diff(off.astype(np.int64)) >= 0).all()
    src_of = np.repeat(np.arange(n, dtype=np.uint64), np.diff(off.astype(np.int64)))
    assert (src_of != cols).all()                                   # no self loops
    key = (src_of << np.uint64(32)) | cols
    assert (np.diff(key.astype(np.int64)) > 0).all()                # sorted, no duplicates
    rev = np.sort((cols << np.uint64(32)) | src_of)
    assert (rev == key).all()                                       # symmetric
    # independent regeneration of the edge list from the published R-MAT recursion
    ta, tab, tabc = orc.rmat_thresholds()
    edges = set()
    for e in range(0, 16 << scale, 997):                            # a sample of the generated edges
        d = py_pcg32(seed, e, scale)
        u = v = 0
        for r in d:
            u = (u << 1) | (1 if r >= tab else 0)
            v = (v << 1) | (1 if (ta <= r < tab) or r >= tabc else 0)
        if u != v:
            edges.add((u, v))
    for (u, v) in edges:
        assert v in cols[off[u]:off[u + 1]] and u in cols[off[v]:off[v + 1]]
    g = _scipy_graph(off, cols)
    src = orc.max_degree_vertex(off)
    deg = np.diff(off.astype(np.int64))
    assert src == int(np.flatnonzero(deg == deg.max())[0])
    lvl, scanned = orc.bfs(off, cols, src)
    dist = csgraph.shortest_path(g, unweighted=True, indices=src)
    want = np.where(np.isinf(dist), 0xFFFFFFFF, dist).astype(np.uint32)
    assert (lvl == want).all()
    assert scanned == int(deg[lvl != 0xFFFFFFFF].sum())
    lab, comps = orc.cc(off, cols)
    ncomp, sl = csgraph.connected_components(g, directed=False)
    assert comps == ncomp
    mins = np.full(ncomp, n, dtype=np.int64)
    np.minimum.at(mins, sl, np.arange(n))
    assert (lab == mins[sl].astype(np.uint64)).all()                # canonical min-vertex label


def test_protocol_restatement_matches_result_oracle(orc):
    """The host-thread restatement of the reference's queue + cache protocol returns the same
    checksum as the pure result oracle, with evictions, queue wrap-around and a shared queue."""
    n_elems, seed, aseed = 1 << 18, 7, 99
    store = orc.fill_store(seed, 0, n_elems)
    for (slots, nq, depth, workers, lanes, reqs) in [(64, 1, 4, 3, 256, 8), (128, 2, 8, 4, 512, 8), (1024, 3, 64, 6, 2048, 4)]:
        r = orc.ref_array_read(store, 4096, slots, nq, depth, 512, workers, 2, access_seed=aseed,
                               lane_begin=0, lane_end=lanes, reqs_per_lane=reqs)
        assert r.checksum == orc.array_checksum(seed, n_elems, aseed, 0, lanes, reqs)
        assert r.accesses == lanes * reqs and r.hits + r.misses == r.accesses and r.read_ios == r.misses
        assert r.read_ios >= min(len(np.unique(orc.array_indices(aseed, n_elems, 0, lanes, reqs) // 512)), 1)


def test_protocol_restatement_block_read(orc):
    seed = 5
    store = orc.fill_store(seed, 0, 1 << 16)                       # 128 pages
    r, crc = orc.ref_block_read(store, 4096, 2, 4, 512, 3, 1, 78, 600)
    pages, want = orc.block_requests(seed, 78, 128, 4096, 0, 600)
    assert (crc == want).all() and r.read_ios == 600


def test_golden_fixtures(orc):
    for c in GOLDEN["array_checksum"]:
        assert orc.array_checksum(c["store_seed"], c["n_elems"], c["access_seed"], 0, c["lanes"], c["reqs"]) == c["checksum"]
    for c in GOLDEN["page_crc"]:
        assert orc.page_crc(c["store_seed"], c["page"], c["page_bytes"]) == c["crc"]
    b = GOLDEN["block_requests"]
    pages, crcs = orc.block_requests(b["store_seed"], b["req_seed"], b["n_pages"], b["page_bytes"], 0, 256)
    assert sha(pages) == b["pages_sha256"] and sha(crcs) == b["crc_sha256"]
    z = GOLDEN["zipf"]
    cdf = orc.zipf_cdf(z["n_pages"], z["s"])
    assert sha(cdf) == z["cdf_sha256"]
    idx = orc.zipf_indices(cdf, z["n_pages"], 512, z["perm_seed"], z["access_seed"], 0, z["lanes"], z["reqs"])
    assert sha(idx) == z["idx_sha256"] and orc.indexed_checksum(9, 0, idx) == z["checksum"]
    for gph in GOLDEN["graphs"]:
        off, cols = orc.rmat_csr(gph["seed"], gph["scale"], gph["edge_factor"])
        assert sha(off) == gph["offsets_sha256"] and sha(cols) == gph["cols_sha256"]
        lvl, scanned = orc.bfs(off, cols, gph["source"])
        lab, comps = orc.cc(off, cols)
        assert sha(lvl) == gph["levels_sha256"] and sha(lab) == gph["labels_sha256"]
        assert comps == gph["components"] and scanned == gph["edges_scanned"]
        wts = orc.edge_weights(gph["weight_seed"], len(cols))
        dist = orc.sssp(off, cols, wts, gph["source"])
        assert sha(wts) == gph["weights_sha256"] and sha(dist) == gph["dist_sha256"]
        rank, sweeps, pr_scanned = orc.pagerank(off, cols)
        assert sha(rank) == gph["rank_sha256"] and sweeps == gph["pr_sweeps"] and pr_scanned == gph["pr_edges_scanned"]


def test_protocol_restatement_graph_traversals(orc):
    """BFS and CC through the host-thread restatement of cache + queues equal the result oracle."""
    off, cols = orc.rmat_csr(2, 10, 16)
    store, off_bytes = orc.csr_store(off, cols)
    n = len(off) - 1
    src = orc.max_degree_vertex(off)
    want_lv, want_sc = orc.bfs(off, cols, src)
    lv, scanned, iters, r = orc.ref_graph_run(store, n, off_bytes, 0, src, 16, 2, 8, 4, 1)      # 16 slots: evictions
    assert (lv == want_lv).all() and scanned == want_sc and r.read_ios > 0
    assert iters == int(want_lv[want_lv != 0xFFFFFFFF].max()) + 1
    want_lab, _ = orc.cc(off, cols)
    lab, _, sweeps, _ = orc.ref_graph_run(store, n, off_bytes, 1, 0, 64, 2, 8, 4, 1)
    assert (lab == want_lab).all() and sweeps >= 1


def test_backing_location_of_replicated_and_striped_ranges(orc):
    """The page -> (controller, backing page) map of include/page_cache.h:558-582: the oracle's C
    restatement, the host mirror and a direct statement of the rule agree."""
    import bam_b200
    rng = np.random.default_rng(3)
    for n_ctrls in (1, 2, 3, 8):
        for page in [0, 1, n_ctrls - 1, n_ctrls, 12345] + rng.integers(0, 1 << 40, 20).tolist():
            for start in (0, 77):
                assert orc.backing_location(start, page, n_ctrls, 0) == (None, start + page)
                assert bam_b200.backing_location(page, n_ctrls, bam_b200.REPLICATE, start) == (None, start + page)
                want = (page % n_ctrls, start + page // n_ctrls)
                assert orc.backing_location(start, page, n_ctrls, 1) == want
                if n_ctrls > 1:
                    assert bam_b200.backing_location(page, n_ctrls, bam_b200.STRIPE, start) == want
    # striping is a bijection between a range's pages and (controller, backing page) pairs
    n_ctrls, n_pages = 3, 1000
    seen = {orc.backing_location(5, p, n_ctrls, 1) for p in range(n_pages)}
    assert len(seen) == n_pages and max(b for _, b in seen) == 5 + (n_pages - 1) // n_ctrls


def test_sssp_oracle_matches_scipy(orc):
    sp = pytest.importorskip("scipy.sparse")
    from scipy.sparse.csgraph import dijkstra
    off, cols = orc.rmat_csr(4, 10, 8)
    n = len(off) - 1
    wts = orc.edge_weights(9, len(cols))
    assert wts.min() >= 1 and wts.max() <= 64 and len(np.unique(wts)) == 64
    m = sp.csr_matrix((wts.astype(np.float64), cols.astype(np.int64), off.astype(np.int64)), shape=(n, n))
    for src in (0, int(orc.max_degree_vertex(off))):
        want = dijkstra(m, directed=True, indices=src)
        got = orc.sssp(off, cols, wts, src)
        reach = np.isfinite(want)
        assert (got[~reach] == 0xFFFFFFFF).all() and (got[reach] == want[reach].astype(np.uint32)).all()


def test_pagerank_oracle_against_linear_solve(orc):
    """The fixed-point delta PageRank ends within its tolerance of the solution of
    x = (1 - alpha) + alpha * sum_{u -> v} x_u / deg_u (no redistribution of dangling mass, as in
    benchmarks/pagerank/main.cu), and its sweeps are order independent."""
    off, cols = orc.rmat_csr(6, 9, 8)
    n = len(off) - 1
    deg = np.diff(off).astype(np.float64)
    P = np.zeros((n, n))
    src = np.repeat(np.arange(n), np.diff(off).astype(np.int64))
    np.add.at(P, (cols.astype(np.int64), src), 1.0 / deg[src])
    alpha = 0.85
    x = np.linalg.solve(np.eye(n) - alpha * P, np.full(n, 1 - alpha))
    rank, sweeps, scanned = orc.pagerank(off, cols)
    v = rank.astype(np.float64) / float(1 << orc.PR_FRAC_BITS)
    assert 1 < sweeps < 100 and scanned >= len(cols)
    assert np.abs(v - x).sum() / x.sum() < 0.01
    assert (np.abs(v - x) / x).max() < 0.02
    # a tighter tolerance gets closer
    rank2, sweeps2, _ = orc.pagerank(off, cols, tolerance_q=(1 << orc.PR_FRAC_BITS) // 1000000)
    v2 = rank2.astype(np.float64) / float(1 << orc.PR_FRAC_BITS)
    assert sweeps2 >= sweeps and np.abs(v2 - x).sum() / x.sum() < 1e-4


def test_command_encoding_against_the_reference_builders(orc, bam):
    """The reference's own nvm_cmd_header / nvm_cmd_data_ptr / nvm_cmd_rw_blks (compiled from its sources
    into oracle/_ref/libref_wire.so), the oracle's restatement and the library's host-side builders give
    the same 64 bytes; so do the reference's status packing and page arithmetic."""
    ref = orc.ref_wire()
    if ref is None:
        pytest.skip("the reference's wire-format code is not built (needs the reference project)")
    lib = bam.load()
    rng = np.random.default_rng(11)
    for _ in range(300):
        cid = int(rng.integers(0, 1 << 16))
        opc = int(rng.choice([1, 2]))
        ns = int(rng.integers(1, 1 << 32))
        prp1, prp2, lba = (int(x) for x in rng.integers(0, 1 << 63, 3, dtype=np.uint64))
        nb = int(rng.integers(1, 1 << 16))
        want = (C.c_uint8 * 64)()
        ref.refw_encode_rw(cid, opc, ns, prp1, prp2, lba, nb, want)
        assert orc.encode_rw(cid, opc, ns, prp1, prp2, lba, nb) == bytes(want)
        got = (C.c_uint8 * 64)()
        assert lib.bam_encode_rw_command(got, cid, opc, ns, prp1, prp2, lba, nb, 0) == 0
        assert bytes(got) == bytes(want)
    # -(SCT << 8 | SC) packing and the strings behind it
    assert ref.refw_unpack_sct(-0x281) == 2 and ref.refw_unpack_sc(-0x281) == 0x81
    assert b"LBA out of range" in ref.refw_strerror(-0x80) or b"range" in ref.refw_strerror(-0x80).lower()
    assert ref.refw_page_align(4097, 4096) == 8192 and ref.refw_page_to_block(4096, 512, 3) == 24
    assert ref.refw_sizeof_queue() > 0


def test_prp_list_helpers_against_the_reference(orc, bam, tmp_path):
    """nvm_cmd_data / nvm_prp_list / nvm_prp_list_chain, the queue sizing macros, NVM_DEFAULT_CID, the
    opcode packing and the status strings of the library's headers against the reference's own (its
    include/nvm_cmd.h:113-216 and nvm_util.h:186-227 compiled into oracle/_ref/libref_wire.so): same data
    pointer, same list pages, same number of addresses consumed."""
    import shutil
    import subprocess
    ref = orc.ref_wire()
    if ref is None:
        pytest.skip("the reference's wire-format code is not built (needs the reference project)")
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not available")
    from bam_b200 import _lib
    exe = str(tmp_path / "include_compat")
    res = subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-I" + os.path.join(ROOT, "include"),
                          os.path.join(ROOT, "tests", "cpp", "include_compat.cu"), "-o", exe, "-L" + os.path.dirname(_lib.LIB_PATH),
                          "-lbam_b200", "-Xlinker", "-rpath=" + os.path.dirname(_lib.LIB_PATH)], capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    # the program's own host-side checks (macros, entry fields, status packing, list building)
    out = subprocess.run([exe], capture_output=True, text=True)
    assert out.returncode == 0 and json.loads(out.stdout.strip().splitlines()[-1]) == {"bad": 0}, out.stdout + out.stderr
    for n_lists, n_pages in [(0, 1), (0, 2), (0, 5), (1, 1), (1, 2), (1, 3), (1, 17), (1, 256), (1, 512), (1, 513), (2, 513), (2, 514), (2, 601),
                             (3, 1100), (4, 1535)]:
        got = json.loads(subprocess.run([exe, "--prp", str(n_lists), str(n_pages)], capture_output=True, text=True, check=True).stdout)
        mem = np.full(max(n_lists, 1) * 512, 0xFFFFFFFFFFFFFFFF, dtype=np.uint64)
        list_io = (C.c_uint64 * max(n_lists, 1))(*[0xa000 + l * 0x1000 for l in range(max(n_lists, 1))])
        addrs = (C.c_uint64 * (n_pages + 1))(*[0x100000 + i * 4096 for i in range(n_pages + 1)])
        dptr = (C.c_uint32 * 4)()
        used = ref.refw_cmd_data(n_lists, mem.ctypes.data, list_io, 4096, n_pages, addrs, dptr)
        assert got["used"] == used and got["dptr"] == list(dptr), (n_lists, n_pages)
        for l in range(n_lists):
            assert got["lists"][l] == mem[l * 512:(l + 1) * 512].tolist(), (n_lists, n_pages, l)
    lib = bam.load()
    for qs in (1, 2, 64, 65, 256, 257, 1024):
        assert ref.refw_sq_pages(4096, qs) == ((qs - 1) & 0xFFFF) * 64 // 4096 + 1
        assert ref.refw_cq_pages(4096, qs) == ((qs - 1) & 0xFFFF) * 16 // 4096 + 1
    assert ref.refw_default_cid(5, 1, 64) == 5 and ref.refw_default_cid(5, 0, 64) == 69
    assert [ref.refw_opcode(0, 0, 2), ref.refw_opcode(0, 0, 1), ref.refw_opcode(0, 2, 0), ref.refw_opcode(0, 1, 2)] == [2, 1, 8, 6]
    # status text: same subject as the reference's table for the statuses the emulated controller can return
    lib.nvm_strerror.restype = C.c_char_p
    lib.nvm_strerror.argtypes = [C.c_int]
    for status, word in [(-0x80, b"range"), (-0x01, b"opcode"), (-0x02, b"field"), (-0x04, b"transfer"), (-0x13, b"offset"), (-0x101, b"queue")]:
        assert word in lib.nvm_strerror(status).lower() and word in ref.refw_strerror(status).lower(), status
    assert lib.nvm_strerror(0) == b"success" and lib.nvm_strerror(2) == ref.refw_strerror(2)       # an errno both pass to strerror()


def test_reference_parallel_queue_code_against_the_oracle_controller(orc):
    """The reference's parallel queue protocol (get_cid, sq_enqueue, cq_poll, cq_dequeue, put_cid of
    include/nvm_parallel_queue.h, compiled for host threads into oracle/_ref/libref_pq.so) runs against the
    oracle's NVMe controller over bare queue memory: the controller the CPU baseline uses speaks the
    protocol the reference's code expects."""
    pq = orc.ref_pq()
    if pq is None:
        pytest.skip("the reference's queue code is not built (needs the reference project)")
    L = orc.lib()
    qs, n_pages, n_req, seed = 16, 512, 2000, 13
    regs = np.zeros(0x2000, dtype=np.uint8)
    qmem = np.zeros(3 * 4096, dtype=np.uint8)
    base = (qmem.ctypes.data + 4095) // 4096 * 4096            # page 0: CQ, page 1: SQ
    media = orc.fill_store(seed, 0, n_pages * 512)
    bufs = np.zeros((n_req, 512), dtype=np.uint64)
    ctrl = L.orc_wire_ctrl_start(base + 4096, base, regs.ctypes.data + 0x1000 + 8, regs.ctypes.data + 0x1000 + 12, qs, qs, 1,
                                 media.ctypes.data, media.nbytes, 512)
    assert ctrl
    pair = pq.refpq_pair_new(regs.ctypes.data, 1, qs, base + 4096, base + 4096, qs, base, base, 1)
    assert pair
    rng = np.random.default_rng(1)
    pages = rng.integers(0, n_pages, n_req, dtype=np.uint64)
    lbas = np.ascontiguousarray(pages * np.uint64(8))
    prps = np.ascontiguousarray(bufs.ctypes.data + np.arange(n_req, dtype=np.uint64) * np.uint64(4096))
    try:
        assert pq.refpq_run(pair, 6, 2, lbas.ctypes.data, prps.ctypes.data, 8, n_req, 60000) == 0, "the protocol stalled"
        assert (bufs == media.reshape(-1, 512)[pages.astype(np.int64)]).all()
        state = [C.c_uint32() for _ in range(5)]
        pq.refpq_state(pair, *(C.byref(x) for x in state))
        sq_head, sq_tail, cq_head, cq_tail, in_ticket = (x.value for x in state)
        assert in_ticket == n_req and sq_tail == n_req and cq_head == n_req and sq_head == n_req
    finally:
        served = L.orc_wire_ctrl_stop(ctrl)
    assert served == n_req
    pq.refpq_pair_free(pair)


@pytest.mark.parametrize("n_slots,n_qps,qs", [(8, 1, 4), (32, 2, 16), (300, 2, 64)])
def test_restated_cache_against_the_reference_cache_code(orc, n_slots, n_qps, qs):
    """The reference's own array read path -- array_d_t::seq_read, coalesce_page, acquire_page, find_slot,
    read_data, over its parallel queues (include/page_cache.h and nvm_parallel_queue.h compiled for host
    threads into oracle/_ref/libref_cache.so) -- and the restatement in bam_oracle.c read the same access
    list through a cache with constant eviction: same checksum, and -- one thread, so the clock sweep is
    deterministic -- the same hits, misses and page reads."""
    if orc.ref_cache() is None:
        pytest.skip("the reference's cache code is not built (needs the reference project)")
    n_pages, seed = 256, 5
    store = orc.fill_store(seed, 0, n_pages * 512)
    rng = np.random.default_rng(n_slots)
    # a skewed list: a hot set that fits, a cold tail that evicts
    hot = rng.integers(0, 6 * 512, 3000, dtype=np.uint64)
    cold = rng.integers(0, n_pages * 512, 3000, dtype=np.uint64)
    idx = np.where(rng.random(3000) < 0.5, hot, cold).astype(np.uint64)
    world = orc.RefCacheWorld(store, n_slots=n_slots, n_qps=n_qps, qs=qs)
    try:
        ref = world.read(idx, n_threads=1)
    finally:
        served = world.close()
    port = orc.ref_array_read(store, 4096, n_slots, n_qps, qs, 512, 1, 1, idx=idx, lane_begin=0, lane_end=len(idx), reqs_per_lane=1)
    want = orc.indexed_checksum(seed, 0, idx)
    assert ref.checksum == want == port.checksum
    assert (ref.accesses, ref.hits, ref.misses, ref.read_ios) == (port.accesses, port.hits, port.misses, port.read_ios)
    assert ref.accesses == len(idx) and ref.hits + ref.misses == len(idx) and ref.read_ios == ref.misses
    assert 0 < ref.hits < len(idx)
    # the reference follows every page read with a second one-block read (enqueue_second, page_cache.h:1961-2007),
    # which neither the restatement nor the library issue: its controller served both
    assert ref.extra_reads == ref.misses and sum(served) == ref.read_ios + ref.extra_reads


def test_reference_cache_code_with_concurrent_threads(orc):
    """Six host threads share the reference's cache and queue pairs (races on pages, slots and queue slots
    are real): the sum of everything read still equals the result oracle, and the counters add up."""
    if orc.ref_cache() is None:
        pytest.skip("the reference's cache code is not built (needs the reference project)")
    n_pages, seed = 512, 9
    store = orc.fill_store(seed, 0, n_pages * 512)
    idx = np.random.default_rng(4).integers(0, n_pages * 512, 20000, dtype=np.uint64)
    world = orc.RefCacheWorld(store, n_slots=64, n_qps=3, qs=16)
    try:
        ref = world.read(idx, n_threads=6)
    finally:
        served = world.close()
    assert ref.checksum == orc.indexed_checksum(seed, 0, idx)
    assert ref.accesses == len(idx) and ref.hits + ref.misses == len(idx) and ref.read_ios == ref.misses
    assert all(s > 0 for s in served)                       # thread number mod 3 picks the queue pair, as smid does



def test_reference_admin_layer_parses_the_identify_pages(orc, bam):
    """The reference's admin layer (src/admin.cpp compiled into oracle/_ref/libref_admin.so) over a controller
    played by a Python callback: its IDENTIFY commands are answered with the pages the emulated controller
    returns (bam_identify_page, which needs no GPU), its register reads go to a window laid out as the
    library lays its own out; what it parses must be the configuration."""
    ra = orc.ref_admin()
    if ra is None:
        pytest.skip("the reference's admin layer is not built (needs the reference project)")
    lib = bam.load()
    u8, u16, u32, u64, vp = C.c_uint8, C.c_uint16, C.c_uint32, C.c_uint64, C.c_void_p

    class NvmCtrl(C.Structure):
        _fields_ = [("page_size", C.c_size_t), ("dstrd", u8), ("timeout", u64), ("max_qs", u32), ("mm_size", C.c_size_t), ("mm_ptr", vp)]

    class CtrlInfo(C.Structure):
        _fields_ = [("nvme_version", u32), ("page_size", C.c_size_t), ("db_stride", C.c_size_t), ("timeout", u64), ("contiguous", C.c_int),
                    ("max_entries", u16), ("pci_vendor", u8 * 4), ("serial_no", C.c_char * 20), ("model_no", C.c_char * 40),
                    ("firmware", C.c_char * 8), ("max_data_size", C.c_size_t), ("max_data_pages", C.c_size_t), ("cq_entry_size", C.c_size_t),
                    ("sq_entry_size", C.c_size_t), ("max_out_cmds", C.c_size_t), ("max_n_ns", C.c_size_t)]

    class NsInfo(C.Structure):
        _fields_ = [("ns_id", u32), ("size", C.c_size_t), ("capacity", C.c_size_t), ("utilization", C.c_size_t),
                    ("lba_data_size", C.c_size_t), ("metadata_size", C.c_size_t)]

    regs = np.zeros(0x2000, dtype=np.uint8)                     # CAP: MQES 1023, CQR, TO 10 x 500 ms, DSTRD 0, NVM command set; VS 1.4
    regs[:8].view(np.uint64)[0] = 1023 | (1 << 16) | (10 << 24) | (1 << 37)
    regs[8:12].view(np.uint32)[0] = 0x00010400
    ctrl = NvmCtrl(4096, 0, 5000, 1024, 0x2000, regs.ctypes.data)
    granted = {"cq": 64, "sq": 64}
    seen = []

    for store_bytes, lba in ((1 << 30, 512), (3 << 28, 4096)):
        def rpc(ref, cmd, cpl, store_bytes=store_bytes, lba=lba):
            dw = (u32 * 16).from_address(cmd)
            out = (u32 * 4).from_address(cpl)
            opcode, prp1 = dw[0] & 0xff, dw[6] | (dw[7] << 32)
            seen.append(opcode)
            if opcode == 0x06:
                if (dw[10] & 0xff) == 0 and dw[1] != 1:
                    return -0x00b
                return lib.bam_identify_page(dw[10] & 0xff, store_bytes, lba, prp1)
            if opcode in (0x09, 0x0a) and (dw[10] & 0xff) == 0x07:
                if opcode == 0x09:
                    granted["sq"], granted["cq"] = (dw[11] & 0xffff) + 1, (dw[11] >> 16) + 1
                out[0] = ((granted["cq"] - 1) << 16) | (granted["sq"] - 1)
                return 0
            return -0x001

        rpc_cb = C.CFUNCTYPE(C.c_int, vp, vp, vp)(rpc)
        from_cb = C.CFUNCTYPE(vp, vp)(lambda ref: C.addressof(ctrl))
        ra.refa_bind(C.cast(rpc_cb, vp), C.cast(from_cb, vp))
        page = np.zeros(4096, dtype=np.uint8)
        info = CtrlInfo()
        assert ra.refa_ctrl_info(None, C.byref(info), page.ctypes.data, page.ctypes.data) == 0
        assert (info.nvme_version, info.page_size, info.db_stride, info.timeout, info.contiguous, info.max_entries) == (0x00010400, 4096, 1, 5000, 1, 1024)
        assert (info.max_data_size, info.max_data_pages, info.sq_entry_size, info.cq_entry_size, info.max_out_cmds, info.max_n_ns) == \
               (1 << 20, 256, 64, 16, 0xFFFF, 1)
        assert info.serial_no == b"BAMB200EMU0000000001" and info.model_no.startswith(b"emulated NVMe controller") and info.firmware == b"1.0     "
        ns = NsInfo()
        assert ra.refa_ns_info(None, C.byref(ns), 1, page.ctypes.data, page.ctypes.data) == 0
        assert (ns.ns_id, ns.size, ns.capacity, ns.utilization, ns.lba_data_size, ns.metadata_size) == \
               (1, store_bytes // lba, store_bytes // lba, store_bytes // lba, lba, 0)
        assert ra.refa_ns_info(None, C.byref(ns), 2, page.ctypes.data, page.ctypes.data) == -0x00b
        # the number-of-queues feature: the command carries completion queues in the upper half (as the
        # specification says), the reference reads the answer's halves the other way round
        ncq, nsq = u16(3), u16(5)
        assert ra.refa_request_num_queues(None, C.byref(ncq), C.byref(nsq)) == 0
        assert (granted["cq"], granted["sq"]) == (3, 5) and (ncq.value, nsq.value) == (5, 3)
    assert seen.count(0x06) == 6 and seen.count(0x09) == 2
    assert lib.bam_identify_page(2, 1 << 30, 512, page.ctypes.data) == 22 and lib.bam_identify_page(0, 1 << 30, 500, page.ctypes.data) == 22


@pytest.mark.parametrize("qs,n_procs,batch", [(16, 4, 4), (16, 6, 2), (64, 4, 8), (8, 3, 2)])
def test_reference_parallel_queue_code_against_several_processors_per_queue(orc, qs, n_procs, batch):
    """The scheme by which the GPU controller lets several processors serve ONE queue -- reserve a batch under
    the queue's lock, read the entries out after the lock has gone, hand them back in order, complete whenever
    ready, so that later batches overtake earlier ones -- restated for host threads (orc_wire_ctrl_start_mt)
    under the reference's parallel queue code (oracle/_ref/libref_pq.so) on shallow queues: every command
    completes exactly once with the right data, the reference's counters end at the request count, and a good
    part of the batches did post out of order."""
    pq = orc.ref_pq()
    if pq is None:
        pytest.skip("the reference's queue code is not built (needs the reference project)")
    L = orc.lib()
    n_pages, n_req, seed = 512, 6000, 17
    regs = np.zeros(0x2000, dtype=np.uint8)
    qmem = np.zeros(3 * 4096, dtype=np.uint8)
    base = (qmem.ctypes.data + 4095) // 4096 * 4096            # page 0: CQ, page 1: SQ
    media = orc.fill_store(seed, 0, n_pages * 512)
    bufs = np.zeros((n_req, 512), dtype=np.uint64)
    ctrl = L.orc_wire_ctrl_start_mt(base + 4096, base, regs.ctypes.data + 0x1000 + 8, regs.ctypes.data + 0x1000 + 12, qs, qs, 1,
                                    media.ctypes.data, media.nbytes, 512, n_procs, batch)
    assert ctrl
    pair = pq.refpq_pair_new(regs.ctypes.data, 1, qs, base + 4096, base + 4096, qs, base, base, 1)
    assert pair
    pages = np.random.default_rng(qs + n_procs).integers(0, n_pages, n_req, dtype=np.uint64)
    lbas = np.ascontiguousarray(pages * np.uint64(8))
    prps = np.ascontiguousarray(bufs.ctypes.data + np.arange(n_req, dtype=np.uint64) * np.uint64(4096))
    batches, overtaken = C.c_uint64(), C.c_uint64()
    try:
        assert pq.refpq_run(pair, 6, 2, lbas.ctypes.data, prps.ctypes.data, 8, n_req, 60000) == 0, "the protocol stalled"
        assert (bufs == media.reshape(-1, 512)[pages.astype(np.int64)]).all()
        state = [C.c_uint32() for _ in range(5)]
        pq.refpq_state(pair, *(C.byref(x) for x in state))
        sq_head, sq_tail, cq_head, cq_tail, in_ticket = (x.value for x in state)
        assert in_ticket == n_req and sq_tail == n_req and cq_head == n_req and sq_head == n_req
    finally:
        served = L.orc_wire_ctrl_stop_mt(ctrl, C.byref(batches), C.byref(overtaken))
    assert served == n_req and batches.value >= n_req // batch
    assert overtaken.value > batches.value // 20                 # the interleavings the model is there for did occur
    pq.refpq_pair_free(pair)
