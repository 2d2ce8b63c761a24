"""ctypes binding of libbam_b200.so (the C ABI declared in include/bam_abi.h).

The library is the product: if it is missing this module raises, there is no fallback.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# BAM_B200_LIB selects another build of the same library (e.g. one compiled with -DBAM_PROFILE)
LIB_PATH = os.environ.get("BAM_B200_LIB") or os.path.join(HERE, "libbam_b200.so")

u32, u64, vp, ci = C.c_uint32, C.c_uint64, C.c_void_p, C.c_int


class CacheStats(C.Structure):
    _fields_ = [("hits", u64), ("misses", u64), ("read_ios", u64)]


class RangeDesc(C.Structure):
    _fields_ = [("index_start", u64), ("index_end", u64), ("store_byte_offset", u64), ("page_start_offset", u64),
                ("dist", u32), ("reserved", u32)]


class StatusOut(C.Structure):
    _fields_ = [("code", u32), ("where", u32), ("detail", u64)]


# name -> (restype, argtypes); mirrors include/bam_abi.h one to one
SIGNATURES = {
    "bam_version": (C.c_char_p, []),
    "bam_strerror": (C.c_char_p, [ci]),
    "bam_ctrl_create": (ci, [C.POINTER(vp), ci, u64, u32, u32, u32]),
    "bam_ctrl_destroy": (ci, [vp]),
    "bam_ctrl_store_host": (vp, [vp]),
    "bam_ctrl_store_bytes": (u64, [vp]),
    "bam_ctrl_fill_store": (ci, [vp, u64, u64, vp]),
    "bam_ctrl_fill_store_striped": (ci, [vp, u64, u64, u32, u32, u32, vp]),
    "bam_ctrl_write_store": (ci, [vp, u64, vp, u64]),
    "bam_ctrl_configure": (ci, [vp, u32, u32, u64]),
    "bam_ctrl_set_scope": (ci, [vp, ci]),
    "bam_ctrl_set_max_grid": (ci, [vp, u32]),
    "bam_ctrl_set_launch_timeout": (ci, [vp, u64]),
    "bam_ctrl_inject_fault": (ci, [vp, u32, u64, u32]),
    "bam_ctrl_status": (ci, [vp, C.POINTER(StatusOut), ci]),
    "bam_ctrl_profile": (ci, [vp, C.POINTER(u64), ci]),
    "bam_ctrl_served": (ci, [vp, C.POINTER(u64), ci]),
    "bam_ctrl_reset_queues": (ci, [vp]),
    "bam_ctrl_device_controller": (vp, [vp]),
    "bam_ctrl_emu_descriptor": (ci, [vp, vp, C.c_size_t]),
    "bam_cache_create": (ci, [C.POINTER(vp), vp, u32, u64]),
    "bam_cache_create_multi": (ci, [C.POINTER(vp), C.POINTER(vp), u32, u32, u64]),
    "bam_cache_destroy": (ci, [vp]),
    "bam_cache_stats": (ci, [vp, C.POINTER(CacheStats), ci]),
    "bam_cache_invalidate": (ci, [vp]),
    "bam_cache_invalidate_async": (ci, [vp, vp]),
    "bam_cache_audit": (ci, [vp, C.POINTER(u64)]),
    "bam_cache_audit_noalloc": (ci, [vp, vp, vp]),
    "bam_cache_descriptor": (ci, [vp, vp, C.c_size_t]),
    "bam_array_create": (ci, [C.POINTER(vp), vp, u64, u32, u64]),
    "bam_array_create_dist": (ci, [C.POINTER(vp), vp, u64, u32, u64, u32]),
    "bam_array_create_ranges": (ci, [C.POINTER(vp), vp, u64, u32, C.POINTER(RangeDesc), u32]),
    "bam_array_destroy": (ci, [vp]),
    "bam_array_device_ptr": (vp, [vp]),
    "bam_launch_block_read": (ci, [vp, u64, vp, u64, vp, vp, vp]),
    "bam_launch_block_read_depth": (ci, [vp, u64, vp, u64, u32, vp, vp, vp]),
    "bam_launch_array_read": (ci, [vp, u64, u64, vp, u64, vp, vp]),
    "bam_launch_frontier_compact": (ci, [vp, vp, u64, u32, vp, u64, vp, vp]),
    "bam_launch_frontier_apply": (ci, [vp, u64, u32, vp, u64, vp, u32, u32, vp]),
    "bam_launch_cc_compact": (ci, [vp, vp, vp, u64, vp, u64, vp, vp]),
    "bam_launch_cc_apply": (ci, [vp, vp, u64, u64, u64, vp, u64, vp, u32, u32, vp]),
    "bam_launch_cc_dense_flag": (ci, [vp, vp, vp, u64, u64, vp]),
    "bam_launch_array_write": (ci, [vp, u64, vp, u64, u64, vp]),
    "bam_launch_thread_acquire": (ci, [vp, u64, u64, u32, vp, vp]),
    "bam_launch_pattern_read": (ci, [vp, u32, u64, u64, u64, u64, vp, vp, vp]),
    "bam_launch_pattern_read_impl": (ci, [vp, u32, u32, u64, u64, u64, u64, vp, vp, vp]),
    "bam_launch_bulk_io": (ci, [vp, u64, u64, u64, ci, vp]),
    "bam_cache_copy": (ci, [vp, u64, vp, u64, ci, vp]),
    "bam_cache_flush": (ci, [vp, vp]),
    "bam_launch_page_scan": (ci, [vp, u64, vp, u64, vp, vp]),
    "bam_launch_bfs_level": (ci, [vp, vp, u64, u64, u64, u32, vp, vp, vp, vp, u64, vp]),
    "bam_graph_scratch_bytes": (u64, [u64]),
    "bam_launch_cc_sweep": (ci, [vp, vp, u64, u64, u64, vp, vp, vp, vp, vp, vp, u64, vp]),
    "bam_bfs_run": (ci, [vp, vp, u64, u64, vp, C.POINTER(u32), C.POINTER(u64)]),
    "bam_cc_run": (ci, [vp, vp, u64, vp, C.POINTER(u32), C.POINTER(u64)]),
    "bam_launch_sssp_sweep": (ci, [vp, vp, vp, u64, u64, u64, vp, vp, vp, vp, u64, vp]),
    "bam_sssp_run": (ci, [vp, vp, vp, u64, u64, vp, C.POINTER(u32), C.POINTER(u64)]),
    "bam_launch_pr_sweep": (ci, [vp, vp, u64, u64, u64, vp, vp, vp, vp, vp, u64, vp]),
    "bam_launch_degrees": (ci, [vp, u64, vp, vp]),
    "bam_pagerank_run": (ci, [vp, vp, u64, u64, u64, u64, u32, vp, C.POINTER(u32), C.POINTER(u64)]),
    "bam_gen_rmat_keys": (ci, [vp, u64, u64, u64, u32, u32, u32, u32, vp]),
    "bam_ctrl_write_store_from_device": (ci, [vp, u64, vp, u64, vp]),
    "bam_gen_uniform_indices": (ci, [vp, u64, u64, u64, u64, vp]),
    "bam_gen_zipf_indices": (ci, [vp, u64, u64, u64, vp, u64, u32, u64, vp]),
    "bam_gen_block_pages": (ci, [vp, u64, u64, u64, vp]),
    "bam_direct_page_sums": (ci, [vp, u64, u64, u32, vp, vp]),
    "bam_direct_checksum": (ci, [vp, u64, u64, u64, vp, vp]),
    "bam_identify_page": (ci, [u32, u64, u32, vp]),
    "bam_encode_rw_command": (ci, [vp, C.c_uint16, C.c_uint8, u32, u64, u64, u64, C.c_uint16, ci]),
    "bam_launch_geometry": (ci, [vp, C.POINTER(u32), C.POINTER(u32), C.POINTER(u32)]),
}

_lib = None


def load():
    """Load the shared library and declare every entry point.  Raises if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            "libbam_b200.so is not built (run `python -c 'import __graft_entry__ as g; g.build()'`); "
            "bam_b200 has no CPU fallback")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


class BamError(RuntimeError):
    def __init__(self, code, what):
        self.code = code
        msg = load().bam_strerror(code).decode()
        super().__init__(f"{what}: {msg} (code {code})")


def check(code, what):
    if code != 0:
        raise BamError(code, what)
