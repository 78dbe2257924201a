"""ctypes binding of libdoksparse.so (C ABI: include/doksparse.h).

The library is built in-tree by `doksparse_b200.build.build()` (nvcc, sm_100a).  There is no CPU or
PyTorch fallback: if the shared object is missing, importing this module's `lib()` raises.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "csrc", "libdoksparse.so")

MAX_KEY_SIZE = 8
MAX_VALUE_BYTES = 248
MAX_SELECTOR_NDIM = 8
MAX_SHARDS = 64
N_COUNTERS = 8
MAX_EPOCH = (1 << 30) - 1
CNT_CLAIMED_EMPTY, CNT_REUSED_REMOVED, CNT_FAILED, CNT_HITS, CNT_DUPLICATES, CNT_PROBES = range(6)

DTYPE_CODES = {
    torch.int8: 0, torch.uint8: 1, torch.int16: 2, torch.int32: 3, torch.int64: 4,
    torch.float16: 5, torch.bfloat16: 6, torch.float32: 7, torch.float64: 8,
}
FLOAT_DTYPES = (torch.float16, torch.bfloat16, torch.float32, torch.float64)


class HashParams(ctypes.Structure):
    _fields_ = [
        ("key_size", ctypes.c_int32), ("key_dtype", ctypes.c_int32),
        ("alpha2", ctypes.c_int64 * MAX_KEY_SIZE), ("beta2", ctypes.c_int64 * MAX_KEY_SIZE),
        ("prime2", ctypes.c_int64 * MAX_KEY_SIZE),
        ("alpha1", ctypes.c_int64 * MAX_KEY_SIZE), ("beta1", ctypes.c_int64 * MAX_KEY_SIZE),
        ("prime1", ctypes.c_int64 * MAX_KEY_SIZE), ("key_perm", ctypes.c_int32 * MAX_KEY_SIZE),
    ]


class Table(ctypes.Structure):
    _fields_ = [
        ("slots", ctypes.c_void_p), ("stamp", ctypes.c_void_p), ("n_buckets", ctypes.c_int64),
        ("slot_bytes", ctypes.c_int32), ("value_bytes", ctypes.c_int32), ("key_bytes", ctypes.c_int32),
        ("reserved", ctypes.c_int32),
    ]


class LayoutInfo(ctypes.Structure):
    _fields_ = [
        ("slot_bytes", ctypes.c_int32), ("slots_per_group", ctypes.c_int32), ("value_offset", ctypes.c_int32),
        ("key_offset", ctypes.c_int32), ("stamp_offset", ctypes.c_int32), ("reserved", ctypes.c_int32),
        ("n_slots", ctypes.c_int64), ("total_bytes", ctypes.c_int64),
    ]


class Selectors(ctypes.Structure):
    _fields_ = [
        ("ndim", ctypes.c_int32), ("selector_ndim", ctypes.c_int32),
        ("sizes", ctypes.c_int64 * MAX_SELECTOR_NDIM),
        ("ptr", ctypes.c_void_p * MAX_KEY_SIZE),
        ("strides", (ctypes.c_int64 * MAX_SELECTOR_NDIM) * MAX_KEY_SIZE),
    ]


class DokError(RuntimeError):
    pass


_STATUS = {1: "DOK_BAD_ARG", 2: "DOK_CUDA_ERROR", 3: "DOK_TOO_LARGE"}
_lib = None


def _declare(lib):
    P, I64, I = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
    TP, HP, SP = ctypes.POINTER(Table), ctypes.POINTER(HashParams), ctypes.POINTER(Selectors)
    sig = {
        "dok_version": ([], I),
        "dok_last_cuda_error": ([], I),
        "dok_launch_count": ([], I64),
        "dok_table_layout": ([I, I, I64, ctypes.POINTER(LayoutInfo)], I),
        "dok_map_init": ([TP, P], I),
        "dok_map_uuid": ([TP, HP, P, I64, P, P, P], I),
        "dok_map_get": ([TP, HP, P, I64, P, P, P, P, P], I),
        "dok_map_get_probe_stats": ([TP, HP, P, I64, P, P, P, P], I),
        "dok_map_set_unique": ([TP, HP, P, P, I64, P, P, P], I),
        "dok_map_set": ([TP, HP, P, P, I64, P, I64, P, P, P], I),
        "dok_map_remove": ([TP, HP, P, I64, P, P, P], I),
        "dok_map_count_exists": ([TP, HP, P, I64, P, P, P], I),
        "dok_map_count_new": ([TP, HP, P, I64, P, I64, P, P], I),
        "dok_static_scratch_max_rows": ([], I64),
        "dok_map_count_new_static": ([TP, HP, P, I64, P, P], I),
        "dok_map_get_sliced": ([TP, HP, P, I64, I64, P, P, P, P, P, P, P], I),
        "dok_map_set_sliced": ([TP, HP, P, P, I64, I64, P, P, P, I64, I, P, P], I),
        "dok_map_remove_sliced": ([TP, HP, P, I64, I64, P, P, P, P, P], I),
        "dok_set_window_bytes": ([I64, I64], I),
        "dok_table_passes": ([TP], I),
        "dok_compact_tiles": ([I64], I64),
        "dok_map_compact_count": ([TP, P, P], I),
        "dok_map_compact_scatter": ([TP, HP, P, P, I, P, P, P], I),
        "dok_dok_get": ([TP, HP, SP, P, P, P, P, P], I),
        "dok_dok_count_exists": ([TP, HP, SP, P, P], I),
        "dok_dok_zero_items": ([TP, HP, SP, P, P], I),
        "dok_dok_gather_insert": ([TP, HP, SP, TP, HP, P, P], I),
        "dok_dok_set_dense": ([TP, HP, SP, P, P, P, I64, P, P], I),
        "dok_dense_count_nonzero": ([P, I64, I, I, P, P], I),
        "dok_dense_insert_nonzero": ([TP, HP, P, P, I64, I, P, P], I),
        "dok_partition_tiles": ([I64], I64),
        "dok_partition_offset_words": ([I64, I], I64),
        "dok_shard_partition_count": ([HP, P, I64, I, P, P, P, P], I),
        "dok_partition_capacity": ([I64, I], I64),
        "dok_shard_partition_scatter": ([P, I, P, I, I64, I, P, P, P, P, P, P, P], I),
        "dok_shard_unpermute": ([P, P, P, I, I64, P, P, P, P], I),
        "dok_words_to_pinned": ([P, P, I, P], I),
        "dok_dok_rekey_insert": ([TP, HP, P, TP, HP, P, P, P], I),
        "dok_map_reinsert": ([TP, TP, HP, P, P], I),
        "dok_shard_partition_scatter_peer": ([P, I, P, I, I64, I, P, P, P, P, P, P, P, P], I),
        "dok_shard_partition_check_slices": ([P, I, I64, I, P, P], I),
        "dok_shard_partition_scatter_sliced": ([P, I, P, I, I64, I, P, P, P, P, P, P, I64, P, P, P], I),
        "dok_copy_counted": ([P, P, I, P, P, I, I64, P, P, P], I),
        "dok_shard_token_prepare": ([P, I64, P, P], I),
        "dok_set_routing_blocks": ([I], I),
        "dok_shard_token_finish": ([P, P, P], I),
        "dok_peer_alloc": ([I64, P], I),
        "dok_peer_free": ([P], I),
        "dok_peer_export": ([P, P], I),
        "dok_peer_open": ([P, P], I),
        "dok_peer_close": ([P], I),
        "dok_shard_owner": ([HP, P, I64, I, P, P], I),
        "dok_diag_random_reads": ([P, I64, I64, ctypes.c_uint64, P, P], I),
        "dok_diag_random_requests": ([P, I64, I64, I, I, ctypes.c_uint64, P, P], I),
    }
    for name, (argtypes, restype) in sig.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = restype
    return sig


EXPORTED = None


def lib():
    """The loaded shared library.  Raises if it has not been built: there is no fallback path."""
    global _lib, EXPORTED
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise DokError(
                f"{LIB_PATH} is missing: build it with `python -c 'import doksparse_b200.build as b; b.build()'` "
                "(nvcc, sm_100a). doksparse_b200 has no CPU or PyTorch fallback.")
        loaded = ctypes.CDLL(LIB_PATH)
        EXPORTED = sorted(_declare(loaded))
        _lib = loaded
    return _lib


def check(status, what):
    if status != 0:
        extra = f" (cudaError {lib().dok_last_cuda_error()})" if status == 2 else ""
        raise DokError(f"{what} failed: {_STATUS.get(status, status)}{extra}")


def stream_ptr(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())
