"""bam_b200 -- B200-native GPU storage hot path (page cache + parallel NVMe queues).

Host-side mirror of the reference's C++ host objects (Controller, page_cache_t, range_t /
array_t) over the C ABI of libbam_b200.so.  The CUDA library is mandatory.
"""
from ._lib import BamError, CacheStats, StatusOut, load  # noqa: F401
from .host import (REPLICATE, STRIPE, Array, Controller, PageCache, backing_location, bind_to_gpu_numa, gen_uniform_indices, gen_zipf_indices,  # noqa: F401
                   direct_checksum, gen_block_pages, page_sums, place_rank, probe_uplink_groups, shard_pages, spread_over_uplinks, zipf_cdf)
from .graph import (CsrGraph, DistCsrGraph, build_rmat_csr, load_bel_graph, read_bel, write_bel, allreduce_min_u32, u32_less, gather_headers, raise_on_rank_failure,  # noqa: F401,E402
                    rmat_thresholds, shard_vertices, shard_vertices_by_edges)
