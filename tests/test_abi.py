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


def declared_parameter_counts():
    """function name -> number of parameters of its prototype in include/doksparse.h"""
    text = open(os.path.join(ROOT, "include", "doksparse.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    counts = {}
    for name, params in re.findall(r"\b(dok_[a-z0-9_]+)\s*\(([^)]*)\)\s*;", text):
        params = params.strip()
        counts[name] = 0 if params in ("", "void") else params.count(",") + 1
    return counts


def test_python_bindings_match_the_header_arity():
    """A prototype that gains or loses a parameter in the header must change in the ctypes table too: with a stale
    argtypes list ctypes would pass garbage for the missing argument without any complaint."""
    from doksparse_b200 import _lib
    lib = _lib.lib()
    counts = declared_parameter_counts()
    assert set(counts) == set(declared_functions())
    for name, n in counts.items():
        argtypes = getattr(lib, name).argtypes
        assert argtypes is not None and len(argtypes) == n, f"{name}: header has {n} parameters, _lib.py declares {argtypes}"


def test_slot_geometry():
    from doksparse_b200 import _lib
    lib = _lib.lib()

    def layout(vb, kb, nb):
        out = _lib.LayoutInfo()
        assert lib.dok_table_layout(vb, kb, nb, ctypes.byref(out)) == 0
        return out

    a = layout(8, 8, 1000)           # int64 -> float32[2]: tag + value + key + stamp fill a 32-byte slot
    assert (a.slot_bytes, a.slots_per_group, a.value_offset, a.key_offset, a.stamp_offset) == (32, 4, 8, 16, 24)
    assert (a.n_slots, a.total_bytes) == (1000, 32000)
    b = layout(4, 16, 1001)          # 2-D DOK float32: 32-byte slot, no room for the stamp, 4 slots per group
    assert (b.slot_bytes, b.value_offset, b.key_offset, b.stamp_offset, b.n_slots) == (32, 8, 16, -1, 1004)
    c = layout(40, 12, 7)            # float32[3] -> int64[5]: 64-byte slot, 2 per group
    assert (c.slot_bytes, c.slots_per_group, c.key_offset, c.stamp_offset, c.n_slots) == (64, 2, 48, -1, 8)
    d = layout(4, 32, 10)            # 4-D DOK float32: 64-byte slot with the stamp inside
    assert (d.slot_bytes, d.value_offset, d.key_offset, d.stamp_offset) == (64, 8, 16, 48)
    e = layout(248, 64, 5)           # widest supported row: slots span several lines, probed one by one
    assert (e.slot_bytes, e.slots_per_group, e.stamp_offset, e.n_slots) == (384, 1, 320, 5)
    out = _lib.LayoutInfo()
    assert lib.dok_table_layout(0, 8, 10, ctypes.byref(out)) != 0 and lib.dok_table_layout(249, 8, 10, ctypes.byref(out)) != 0
    assert lib.dok_compact_tiles(1) == 1 and lib.dok_compact_tiles(2049) == 2
    assert ctypes.sizeof(_lib.HashParams) == 8 + 6 * 64 + 32
    assert ctypes.sizeof(_lib.Table) == 40 and ctypes.sizeof(_lib.LayoutInfo) == 40


def test_no_cpu_fallback():
    import torch
    from doksparse_b200 import CudaClosedHashmap, _lib
    with pytest.raises(_lib.DokError):
        CudaClosedHashmap(device="cpu")
    if not torch.cuda.is_available():
        with pytest.raises(Exception):
            CudaClosedHashmap()     # needs a CUDA device; nothing silently runs on the host
