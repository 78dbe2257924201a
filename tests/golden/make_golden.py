"""Generates the committed fixtures of tests/golden/ from the REFERENCE itself.  Run in a container that has
the reference checkout (it is not needed to run the tests):

    make -C oracle ref && python tests/golden/make_golden.py

map_streams.npz   : seeded operation streams replayed on the reference's own kernel text compiled for the host
                    (oracle/_ref): per case the hash parameters, the inputs of every step and what the reference
                    returned (flags, values) plus the sorted live items after every mutation.
selectors.json    : what SparseDOKTensor._handle_selectors of the reference returns (shapes, index values,
                    scalar positions, or the exception type) for a list of selector expressions.  The method's
                    source is extracted from the reference file with `ast` and run on CPU against a stub object,
                    because the reference package cannot be imported without CuPy.
"""
import ast
import json
import os
import sys
import textwrap

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import port, ref  # noqa: E402

REFERENCE = os.environ.get("REFERENCE", "/root/reference")

CASES = [
    # name, key dtype, key size, value dtype, value size, n_buckets, key_perm, key range
    ("i64x1_f32x2", np.int64, 1, np.float32, 2, 211, None, (-10 ** 12, 10 ** 12)),
    ("i64x2_f32x1", np.int64, 2, np.float32, 1, 256, [1, 0], (0, 300)),
    ("i64x4_f32x1", np.int64, 4, np.float32, 1, 128, [2, 0, 3, 1], (0, 12)),
    ("f32x3_i64x5", np.float32, 3, np.int64, 5, 128, None, (-40, 40)),
    ("i32x2_f32x3", np.int32, 2, np.float32, 3, 97, None, (-2 ** 31, 2 ** 31 - 1)),
    ("i16x3_i32x2", np.int16, 3, np.int32, 2, 64, None, (-2 ** 15, 2 ** 15 - 1)),
    ("f64x2_f32x1", np.float64, 2, np.float32, 1, 64, None, (-1e6, 1e6)),
]


def draw_keys(rng, n, dtype, ks, lo, hi):
    if np.issubdtype(dtype, np.floating):
        return rng.uniform(lo, hi, size=(n, ks)).astype(dtype)
    return rng.integers(lo, hi, size=(n, ks), endpoint=False).astype(dtype)


def draw_values(rng, n, dtype, vs):
    if np.issubdtype(dtype, np.floating):
        return rng.standard_normal((n, vs)).astype(dtype)
    return rng.integers(-2 ** 40, 2 ** 40, size=(n, vs)).astype(dtype) if dtype == np.int64 else \
        rng.integers(-2 ** 31, 2 ** 31, size=(n, vs)).astype(dtype)


def live_items(r):
    live = (r.all_uuids != -1) & (r.all_uuids != -3)
    perm = r.params["key_perm"]
    return port.sort_items(r.all_keys[live][:, perm], r.all_values[live], r.all_uuids[live])


def map_streams():
    out = {}
    for case_no, (name, kd, ks, vd, vs, nb, perm, (lo, hi)) in enumerate(CASES):
        np.random.seed(100 + case_no)
        params = port.draw_hash_parameters(nb, ks)
        params["key_perm"] = np.arange(ks) if perm is None else np.asarray(perm)
        r = ref.RefMap(nb, kd, ks, vd, vs, params)
        rng = np.random.default_rng(200 + case_no)
        for k, v in params.items():
            out[f"{name}/param/{k}"] = np.asarray(v, dtype=np.int64)
        out[f"{name}/meta"] = np.asarray([nb, ks, vs], dtype=np.int64)
        pool = draw_keys(rng, nb, kd, ks, lo, hi)
        for step in range(5):
            n = int(nb * 0.22)
            keys = pool[rng.permutation(nb)[:n]] if step % 2 else draw_keys(rng, n, kd, ks, lo, hi)
            # unique rows only: concurrent duplicates are undefined in the reference
            keys = np.unique(keys, axis=0)
            keys = keys[rng.permutation(len(keys))]
            vals = draw_values(rng, len(keys), vd, vs)
            stored = r.set(keys, vals)
            q = np.concatenate([keys[: len(keys) // 2], draw_keys(rng, n, kd, ks, lo, hi), pool[:8]])
            gv, gf = r.get(q, fallback=7)
            dele = np.unique(q[rng.permutation(len(q))[: len(q) // 3]], axis=0)
            removed = r.remove(dele)
            ik, iv, iu = live_items(r)
            for key, arr in dict(set_keys=keys, set_values=vals, set_stored=stored, get_keys=q, get_values=gv,
                                 get_found=gf, remove_keys=dele, remove_flags=removed, items_keys=ik, items_values=iv,
                                 items_uuid=iu).items():
                out[f"{name}/step{step}/{key}"] = arr
    np.savez_compressed(os.path.join(HERE, "map_streams.npz"), **out)
    print("map_streams.npz:", len(out), "arrays")


# ---- selectors ----------------------------------------------------------------------------------------------

SELECTOR_CASES = [
    # (tensor shape, python expression of the selector; `T` = torch.tensor, `np` = numpy)
    ((10,), "[3, 6, 9]"),
    ((10,), "T([[1, 2], [3, 4]])"),
    ((10,), "T([True, False] * 5)"),
    ((10,), "slice(0, 5)"),
    ((10,), "slice(None, None)"),
    ((10,), "slice(7, 100)"),
    ((10,), "slice(8, 3)"),
    ((10,), "T(4)"),
    ((6, 7), "(T([0, 1, 2]), T([3, 4, 5]))"),
    ((6, 7), "(T([[0], [1]]), T([3, 4, 5]))"),
    ((6, 7), "(slice(1, 4), T([3, 4, 5]))"),
    ((6, 7), "(T([3, 4, 5]), slice(1, 4))"),
    ((6, 7), "(2, slice(None))"),
    ((6, 7), "(slice(None), 2)"),
    ((6, 7), "(T([1, 2]),)"),
    ((6, 7), "T([[True] * 7] * 3 + [[False] * 7] * 3)"),
    ((6, 7), "(3, 5)"),
    ((5, 6, 7), "(T([[1], [2]]), slice(0, 3), T([0, 1, 2, 3]))"),
    ((5, 6, 7), "(slice(0, 2), T([1, 2, 3]), slice(2, 4))"),
    ((5, 6, 7), "(slice(0, 2), slice(1, 3), T([1, 2, 3]))"),
    ((5, 6, 7), "(1, slice(0, 2), [1, 2, 3])"),
    ((5, 6, 7), "(slice(0, 2),)"),
    ((13, 11, 7, 3), "(5, slice(None, 4), [3, 5, 6], T([True, False, True]))"),
    ((13, 11, 7, 3), "(T([5, 6])[:, None, None], slice(None, 4), T([3, 5, 6])[None, :, None], T([True, False, True]))"),
    ((13, 11, 7, 3), "(T([[1, 2]]), T([[3], [4]]))"),
    ((4, 4), "(T([1, 2, 3]), T([1, 2]))"),
    ((4, 4), "'abc'"),
    ((4, 4), "(1.5,)"),
]


def load_reference_handle_selectors():
    path = os.path.join(REFERENCE, "sparse_dok", "components", "sparse_dok_tensor.py")
    tree = ast.parse(open(path).read())
    for node in ast.walk(tree):
        if isinstance(node, ast.FunctionDef) and node.name == "_handle_selectors":
            src = textwrap.dedent(ast.get_source_segment(open(path).read(), node))
            scope = {"torch": torch, "np": np, "Tensor": torch.Tensor}
            exec(src, scope)
            return scope["_handle_selectors"]
    raise RuntimeError("_handle_selectors not found")


class Stub:
    def __init__(self, shape):
        self.shape = torch.Size(shape)
        self.ndim = len(shape)
        self.device = torch.device("cpu")


def selectors():
    fn = load_reference_handle_selectors()
    T = torch.tensor
    records = []
    for shape, expr in SELECTOR_CASES:
        sel = eval(expr, {"T": T, "np": np, "slice": slice})
        rec = {"shape": list(shape), "expr": expr}
        try:
            out, scalars = fn(Stub(shape), sel)
            rec["result_shape"] = list(out[0].shape)
            rec["scalars"] = list(scalars)
            rec["indices"] = [o.reshape(-1).tolist() for o in out]
        except Exception as e:  # the exception type is part of the fixture
            rec["raises"] = type(e).__name__
        records.append(rec)
    with open(os.path.join(HERE, "selectors.json"), "w") as f:
        json.dump(records, f, indent=0)
    print("selectors.json:", len(records), "cases,", sum("raises" in r for r in records), "raise")


if __name__ == "__main__":
    map_streams()
    selectors()
