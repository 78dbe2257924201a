"""The C-ABI library loads without a GPU and exports every function include/doksparse.h declares
(no compute calls here)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "doksparse.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dok_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    names = declared_functions()
    for must in ("dok_map_get", "dok_map_set", "dok_map_set_unique", "dok_map_remove", "dok_map_compact_scatter",
                 "dok_dok_get", "dok_dok_set_dense", "dok_dense_insert_nonzero", "dok_shard_partition_scatter"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from doksparse_b200 import _lib
    if not os.path.exists(_lib.LIB_PATH):
        from doksparse_b200.build import build
        build()
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} is declared in include/doksparse.h but not exported"
    assert _lib.lib().dok_version() >= 1
    assert set(_lib.EXPORTED) == set(declared_functions())


def test_bucket_geometry():
    from doksparse_b200 import _lib
    lib = _lib.lib()
    assert lib.dok_bucket_bytes(4) == 16 and lib.dok_bucket_bytes(8) == 16
    assert lib.dok_bucket_bytes(16) == 32 and lib.dok_bucket_bytes(40) == 48
    assert lib.dok_bucket_bytes(0) == -1 and lib.dok_bucket_bytes(249) == -1
    assert lib.dok_compact_tiles(1) == 1 and lib.dok_compact_tiles(2049) == 2
    assert ctypes.sizeof(_lib.HashParams) == 8 + 6 * 64 + 32
    assert ctypes.sizeof(_lib.Table) == 40


def test_no_cpu_fallback():
    import torch
    from doksparse_b200 import CudaClosedHashmap, _lib
    with pytest.raises(_lib.DokError):
        CudaClosedHashmap(device="cpu")
    if not torch.cuda.is_available():
        with pytest.raises(Exception):
            CudaClosedHashmap()     # needs a CUDA device; nothing silently runs on the host
