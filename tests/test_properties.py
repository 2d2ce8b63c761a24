"""Property tests (hypothesis) of the host-side index arithmetic: sharding, striping, permutations,
page arithmetic -- the pieces every larger test relies on."""
import numpy as np
from hypothesis import given, settings
from hypothesis import strategies as st


@given(n=st.integers(0, 1 << 40), world=st.integers(1, 64))
def test_shard_pages_partitions_the_store(bam, n, world):
    cuts = [bam.shard_pages(n, world, r) for r in range(world)]
    assert cuts[0][0] == 0 and sum(c for _, c in cuts) == n
    for (f0, c0), (f1, _) in zip(cuts, cuts[1:]):
        assert f0 + c0 == f1                                   # contiguous, in rank order
    sizes = [c for _, c in cuts]
    assert max(sizes) - min(sizes) <= 1                        # balanced


@given(n=st.integers(1, 1 << 30), world=st.integers(1, 16))
def test_shard_vertices_partitions(bam, n, world):
    cuts = [bam.shard_vertices(n, world, r) for r in range(world)]
    assert cuts[0][0] == 0 and cuts[-1][1] == n
    assert all(a[1] == b[0] for a, b in zip(cuts, cuts[1:]))


@given(page=st.integers(0, 1 << 50), n_ctrls=st.integers(1, 16), start=st.integers(0, 1 << 30))
def test_striping_is_invertible(bam, orc, page, n_ctrls, start):
    ctrl, backing = bam.backing_location(page, n_ctrls, bam.STRIPE, start)
    if n_ctrls == 1:
        assert (ctrl, backing) == (None, start + page)
    else:
        assert 0 <= ctrl < n_ctrls and (backing - start) * n_ctrls + ctrl == page
        assert orc.backing_location(start, page, n_ctrls, 1) == (ctrl, backing)
    assert bam.backing_location(page, n_ctrls, bam.REPLICATE, start) == (None, start + page)


@settings(max_examples=30, deadline=None)
@given(n=st.integers(1, 5000), seed=st.integers(0, (1 << 64) - 1))
def test_permutation_is_a_bijection_for_any_size(orc, n, seed):
    L = orc.lib()
    out = {L.orc_permute(i, n, seed) for i in range(n)}
    assert out == set(range(n))


@given(size=st.integers(0, 1 << 50), log2=st.integers(9, 20))
def test_page_rounding(orc, size, log2):
    ref = orc.ref_wire()
    page = 1 << log2
    want = (size + page - 1) // page * page
    if ref is not None:                                        # the reference's NVM_PAGE_ALIGN agrees
        assert ref.refw_page_align(size, page) == want
    assert (want - size) < page and want % page == 0


@settings(max_examples=25, deadline=None)
@given(seed=st.integers(0, (1 << 63) - 1), scale=st.integers(3, 9), ef=st.integers(1, 8))
def test_rmat_csr_is_a_simple_symmetric_graph(orc, seed, scale, ef):
    off, cols = orc.rmat_csr(seed, scale, ef)
    n = 1 << scale
    assert off[0] == 0 and off[-1] == len(cols) and (np.diff(off.astype(np.int64)) >= 0).all()
    src = np.repeat(np.arange(n, dtype=np.uint64), np.diff(off.astype(np.int64)))
    assert (src != cols).all()                                 # no self loops
    keys = src * np.uint64(n) + cols
    assert len(np.unique(keys)) == len(keys)                   # no duplicates
    assert set(keys.tolist()) == set((cols * np.uint64(n) + src).tolist())     # symmetric
    for v in range(n):                                         # adjacency lists sorted
        row = cols[off[v]:off[v + 1]]
        assert (np.diff(row.astype(np.int64)) > 0).all()


def test_ranks_are_dealt_over_uplink_groups():
    """Placement of fewer ranks than GPUs: one GPU of every uplink group first, then the second of each."""
    import bam_b200
    assert bam_b200.spread_over_uplinks([[0, 1], [2, 3], [4, 5], [6, 7]]) == [0, 2, 4, 6, 1, 3, 5, 7]
    assert bam_b200.spread_over_uplinks([[0, 2], [1, 3], [4, 6], [5, 7]])[:4] == [0, 1, 4, 5]
    assert bam_b200.spread_over_uplinks([[0, 1, 2], [3]]) == [0, 3, 1, 2]
    assert bam_b200.spread_over_uplinks([[0], [1], [2], [3]]) == [0, 1, 2, 3]
    order = bam_b200.spread_over_uplinks([[3, 5, 6], [0, 7], [1, 2, 4]])
    assert sorted(order) == list(range(8)) and {order[0], order[1], order[2]} == {3, 0, 1}
    # as many ranks as GPUs (or no GPU at all): nothing to choose, nothing is measured
    dev, info = bam_b200.place_rank(8, 3, "test")
    assert info["placement"] == "identity"
