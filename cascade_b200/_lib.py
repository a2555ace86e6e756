"""ctypes loader of the device library. There is no CPU fallback: a missing library is an error."""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libcascade_b200.so")

c_u64 = ctypes.c_uint64
c_u32 = ctypes.c_uint32
c_vp = ctypes.c_void_p
c_int = ctypes.c_int


class BuildStats(ctypes.Structure):
    _fields_ = [
        ("n", c_u64), ("partitions", c_u32), ("generations", c_u32), ("max_partition", c_u64),
        ("active_after_gen0", c_u64), ("sort_passes", c_u64), ("sort_records", c_u64), ("kernel_launches", c_u64),
        ("peer_bytes", c_u64),
        ("ms_partition", ctypes.c_double), ("ms_gen0", ctypes.c_double), ("ms_doubling", ctypes.c_double),
        ("ms_output", ctypes.c_double), ("ms_total", ctypes.c_double), ("ms_sort_passes", ctypes.c_double),
        ("active_per_gen", c_u64 * 48), ("peer_bytes_per_gen", c_u64 * 49),
        ("host_parts", c_u32), ("file_parts", c_u32), ("file_bytes_read", c_u64), ("file_bytes_written", c_u64),
    ]


class TierOptions(ctypes.Structure):
    _fields_ = [("part_suffixes", c_u64), ("host_list_bytes", c_u64), ("scratch_dir", ctypes.c_char_p), ("output_path", ctypes.c_char_p)]


ALLGATHER_FN = ctypes.CFUNCTYPE(c_int, c_vp, c_vp, c_vp, c_u64)


class Comm(ctypes.Structure):
    _fields_ = [("rank", c_u32), ("world", c_u32), ("policy", c_u32), ("allgather", ALLGATHER_FN), ("user", c_vp)]


class Part(ctypes.Structure):
    _fields_ = [("lanes", c_vp), ("ranks", c_vp), ("count", c_u64), ("part", c_u32)]


class PartResult(ctypes.Structure):
    _fields_ = [("lanes", c_vp), ("ranks", c_vp), ("active", c_u64), ("messages", c_u64)]


class QueryPlacement(ctypes.Structure):
    _fields_ = [("plan", c_u32), ("key_words", c_u32), ("stride", c_u64), ("table_bytes", c_u64), ("device_bytes", c_u64), ("host_bytes", c_u64),
                ("device_budget", c_u64), ("host_budget", c_u64), ("device_margin", c_u64), ("host_margin", c_u64),
                ("chunk_queries", c_u64), ("chunk_symbols", c_u64), ("why", ctypes.c_char * 512)]


class Index(ctypes.Structure):
    _fields_ = [("text", c_vp), ("sa40", c_vp), ("table", c_vp), ("n", c_u64), ("stride", c_u64), ("sa_entries", c_u64), ("sa_first", c_u64)]


_SIGS = {
    "csa_ctx_create": (c_int, [c_int, ctypes.POINTER(c_vp)]),
    "csa_ctx_destroy": (None, [c_vp]),
    "csa_sync": (c_int, [c_vp, ctypes.POINTER(c_u64)]),
    "csa_last_error": (ctypes.c_char_p, [c_vp]),
    "csa_ctx_stream": (c_vp, [c_vp]),
    "csa_kernel_launches": (c_u64, [c_vp]),
    "csa_reset_counters": (None, [c_vp]),
    "csa_version": (ctypes.c_char_p, []),
    "csa_sort_workspace_bytes": (ctypes.c_size_t, [c_u64]),
    "csa_sort_pairs": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_u32, c_u64, c_int, c_int, c_vp, ctypes.c_size_t, ctypes.POINTER(c_int)]),
    "csa_sort_segments_workspace_bytes": (ctypes.c_size_t, [c_u64, c_u32]),
    "csa_sort_segments": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_u32, c_int, c_int, c_vp, ctypes.c_size_t, ctypes.POINTER(c_int)]),
    "csa_sort_pairs_static": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_u64, c_int, c_int, ctypes.POINTER(c_int)]),
    "csa_debug_set": (c_int, [c_int, c_u64]),
    "csa_set_pass_timing": (c_int, [c_vp, c_int]),
    "csa_get_pass_timing": (c_int, [c_vp, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(c_u64), ctypes.POINTER(c_u64), ctypes.POINTER(c_u64)]),
    "csa_sample_kgrams": (c_int, [c_vp, c_vp, c_u64, c_u64, c_u64, c_vp]),
    "csa_select_pivots": (c_int, [c_vp, c_u64, c_u32, c_vp, ctypes.POINTER(c_u32)]),
    "csa_select_pivots_dev": (c_int, [c_vp, c_vp, c_u64, c_u32, c_vp, ctypes.POINTER(c_u32)]),
    "csa_partition_ids": (c_int, [c_vp, c_vp, c_u64, c_u64, c_u64, c_vp, c_u32, c_vp, c_vp]),
    "csa_scatter_by_pid": (c_int, [c_vp, c_vp, c_u64, c_u64, c_u32, c_vp, c_vp]),
    "csa_build_device_bytes": (ctypes.c_size_t, [c_u64, c_u32]),
    "csa_build_sa": (c_int, [c_vp, c_vp, c_u64, c_u32, c_u64, c_vp, ctypes.POINTER(BuildStats)]),
    "csa_build_sa_host": (c_int, [c_vp, c_vp, c_u64, c_u32, c_u64, c_vp, ctypes.POINTER(BuildStats)]),
    "csa_text_from_u8": (c_int, [c_vp, c_vp, c_u64, c_vp]),
    "csa_text_from_u32": (c_int, [c_vp, c_vp, c_u64, c_vp, c_vp, ctypes.POINTER(c_u32)]),
    "csa_store_create": (c_int, [c_vp, c_vp, c_u64, c_vp, c_vp, c_u32, c_vp, ctypes.POINTER(c_vp)]),
    "csa_store_use_outbox": (c_int, [c_vp, c_vp, c_vp, c_vp, c_u64]),
    "csa_store_outbox_count": (c_u64, [c_vp]),
    "csa_store_apply_messages": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_u64]),
    "csa_install_pivots": (c_int, [c_vp, c_vp, c_u32]),
    "csa_part_sizes": (c_int, [c_vp, c_vp, c_u64, c_u64, c_u32, c_vp]),
    "csa_scatter_lanes": (c_int, [c_vp, c_vp, c_u64, c_u64, c_vp, c_vp, c_vp]),
    "csa_store_drop_partition_ids": (None, [c_vp]),
    "csa_store_destroy": (None, [c_vp]),
    "csa_store_reserve_messages": (c_int, [c_vp, c_vp, c_u64]),
    "csa_part_workspace_bytes": (ctypes.c_size_t, [c_u64]),
    "csa_rank_gen0": (c_int, [c_vp, c_vp, ctypes.POINTER(Part), ctypes.POINTER(PartResult)]),
    "csa_rank_gen": (c_int, [c_vp, c_vp, ctypes.POINTER(Part), c_u64, ctypes.POINTER(PartResult)]),
    "csa_scatter_lanes_keys": (c_int, [c_vp, c_vp, c_vp, c_vp, c_u64, c_u64, c_vp, c_vp, c_vp, c_vp]),
    "csa_rank_gen0_keys": (c_int, [c_vp, c_vp, ctypes.POINTER(Part), c_vp, ctypes.POINTER(PartResult)]),
    "csa_part_positions": (c_int, [c_vp, c_vp, c_vp, c_u64, c_u64, c_vp]),
    "csa_rank_gen_ranks": (c_int, [c_vp, c_vp, ctypes.POINTER(Part), c_vp, ctypes.POINTER(PartResult)]),
    "csa_bucket_by_owner": (c_int, [c_vp, c_vp, c_vp, c_u64, c_u64, c_u32, c_vp, c_vp, c_vp, c_vp]),
    "csa_order_by_address": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_u64, c_int, c_int, c_u64, c_u32, c_int, c_vp, c_vp, ctypes.c_size_t, ctypes.POINTER(c_int)]),
    "csa_rank_shard_read": (c_int, [c_vp, c_vp, c_u64, c_u64, c_vp, c_u64, c_vp]),
    "csa_rank_shard_apply": (c_int, [c_vp, c_vp, c_u64, c_u64, c_vp, c_vp, c_u64]),
    "csa_unbucket": (c_int, [c_vp, c_vp, c_vp, c_u64, c_vp]),
    "csa_outbox_positions": (c_int, [c_vp, c_vp, c_vp, c_u64, c_vp]),
    "csa_exchange_messages": (c_int, [c_vp, c_vp, ctypes.POINTER(c_u64)]),
    "csa_rank_order": (c_int, [c_vp, c_vp, c_vp, c_u64, c_vp]),
    "csa_build_sa_streamed": (c_int, [c_vp, c_vp, c_u64, c_u32, c_u64, c_vp, c_u64, ctypes.POINTER(BuildStats)]),
    "csa_build_sa_tiered": (c_int, [c_vp, c_vp, c_u64, c_u32, c_u64, c_vp, ctypes.POINTER(TierOptions), ctypes.POINTER(BuildStats)]),
    "csa_validate_workspace_bytes": (ctypes.c_size_t, [c_u64]),
    "csa_validate_sa": (c_int, [c_vp, c_vp, c_u64, c_vp, c_vp, ctypes.c_size_t, c_vp]),
    "csa_comm_open_shm": (c_int, [ctypes.c_char_p, c_u32, c_u32, c_u32, c_vp]),
    "csa_comm_shm_set_timeout": (c_int, [c_vp, ctypes.c_double]),
    "csa_comm_close_shm": (None, [c_vp, c_int]),
    "csa_plan_shards": (c_int, [c_vp, c_u32, c_u32, c_u32, c_vp, c_vp, c_vp, c_vp, c_vp]),
    "csa_build_sa_multi": (c_int, [c_vp, c_vp, c_vp, c_u64, c_u32, c_u64, c_vp, c_u64, c_vp, c_vp, ctypes.POINTER(c_u32), ctypes.POINTER(BuildStats)]),
    "csa_table_build": (c_int, [c_vp, c_vp, c_u64, c_vp, c_u64, c_vp]),
    "csa_table_build_slice": (c_int, [c_vp, c_vp, c_u64, c_vp, c_u64, c_u64, c_vp]),
    "csa_locate_window": (c_int, [c_vp, ctypes.POINTER(Index), c_vp, c_u64, c_u32, c_vp]),
    "csa_locate_window_packed": (c_int, [c_vp, ctypes.POINTER(Index), c_vp, c_u64, c_u32, c_vp, c_vp, c_vp, c_vp]),
    "csa_find": (c_int, [c_vp, ctypes.POINTER(Index), c_vp, c_vp, c_u64, c_vp]),
    "csa_locate": (c_int, [c_vp, ctypes.POINTER(Index), c_vp, c_u64, c_u32, c_vp, c_vp]),
    "csa_certify": (c_int, [c_vp, ctypes.POINTER(Index), c_vp, c_vp, c_u64, c_vp, c_vp]),
    "csa_query_host": (c_int, [c_vp, ctypes.POINTER(Index), c_vp, c_vp, c_u64, c_u32, c_vp, c_vp, c_vp, c_vp, c_u64, ctypes.POINTER(c_u64)]),
    "csa_query_plan": (c_int, [c_u64, c_u64, c_u64, c_u64, c_int, ctypes.POINTER(QueryPlacement)]),
    "csa_gen_corpus_dev": (c_int, [c_vp, c_vp, c_u64, c_u64, c_u32, c_vp, c_u32]),
    "csa_gen_corpus_dev_window": (c_int, [c_vp, c_vp, c_u64, c_u64, c_u64, c_u32, c_vp, c_u32]),
    "csa_gen_queries_host": (c_int, [c_int, c_vp, c_u64, c_u64, c_vp, c_u32, c_u64, c_u64, c_vp, c_vp, c_u64]),
    "csa_counts_hash": (c_u64, [c_vp, c_u64]),
    "csa_gen_corpus_host": (c_int, [c_vp, c_u64, c_u64, c_u64, c_u32, c_vp, c_u32]),
}

_lib = None


def exported_names():
    """Names of the entry points that include/cascade_b200.h declares."""
    return sorted(_SIGS)


def lib():
    """Returns the loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m cascade_b200.build` (there is no CPU fallback)")
        L = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in _SIGS.items():
            f = getattr(L, name)
            f.restype = res
            f.argtypes = args
        _lib = L
    return _lib
