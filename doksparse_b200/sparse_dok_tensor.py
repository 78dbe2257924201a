"""SparseDOKTensor: the reference's dictionary-of-keys sparse tensor
(sparse_dok/components/sparse_dok_tensor.py) on top of the CUDA hash map of this package.

Same constructor, classmethods, indexing / assignment / conversion methods and bookkeeping as the
reference.  The hot paths do not materialise an int64[n, ndim] key matrix: `__getitem__`,
`__setitem__` and `from_dense` hand the broadcast selector views (or the dense tensor) to fused kernels
that form each key on the fly, and `to_sparse_coo` compacts indices and values in one pass.
"""
import ctypes
import math

import numpy as np
import torch
from torch import Tensor

from . import _lib as L
from . import util
from .cuda_closed_hashmap import CudaClosedHashmap
from .selectors import normalise_selectors
from .util import next_power_of_2, str2dtype


def _selectors_struct(selectors):
    """Packs broadcast index tensors (views of one common shape) into a dok_selectors struct."""
    s = L.Selectors()
    shape = tuple(selectors[0].shape)
    if len(shape) > L.MAX_SELECTOR_NDIM:
        raise L.DokError(f"selector shapes may have at most {L.MAX_SELECTOR_NDIM} dims, got {len(shape)}")
    s.ndim = len(selectors)
    s.selector_ndim = len(shape)
    for j, extent in enumerate(shape):
        s.sizes[j] = extent
    for d, sel in enumerate(selectors):
        assert sel.dtype == torch.long and tuple(sel.shape) == shape
        s.ptr[d] = sel.data_ptr()
        for j, st in enumerate(sel.stride()):
            s.strides[d][j] = st
    return s


class SparseDOKTensor(object):
    def __init__(self, size, indices=None, values=None, device=None, dtype=None, storage=None):
        assert isinstance(size, (list, tuple))
        self._size = torch.Size(size)

        if storage is None:
            self.device = torch.device("cuda:0") if device is None else torch.device(device)
        else:
            assert isinstance(storage, CudaClosedHashmap)
            self.device = storage.device

        if storage is not None and storage._keys is not None:
            assert len(storage.key_shape) == 1 and storage.key_shape[0] == self.ndim
            self._dtype = storage.value_type
        elif dtype is None:
            self._dtype = torch.float32 if values is None else values.dtype
        else:
            self._dtype = str2dtype(dtype)

        if indices is None:
            self._hashmap = CudaClosedHashmap(n_buckets=32, device=self.device) if storage is None else storage
        else:
            assert values is not None
            assert len(indices.shape) == 2
            assert len(values.shape) == 1
            assert indices.shape[1] == values.shape[0]
            assert indices.shape[0] == self.ndim
            if storage is None:
                self._hashmap = CudaClosedHashmap(n_buckets=next_power_of_2(values.shape[0]), device=self.device)
            else:
                self._hashmap = storage
            self._hashmap.set(indices.T.to(self.device), values.to(device=self.device, dtype=self.dtype)[:, None])

    # ------------------------------------------------------------------ constructors
    @classmethod
    def from_sparse_coo(cls, tensor):
        assert isinstance(tensor, Tensor)
        assert tensor.layout == torch.sparse_coo
        tensor = tensor.coalesce()
        return cls(size=tuple(tensor.shape), indices=tensor._indices(), values=tensor._values(), device=tensor.device)

    @classmethod
    def from_dense(cls, tensor):
        """Same result as the reference's `from_sparse_coo(tensor.to_sparse())` (sparse_dok_tensor.py:86-90): a map of
        next_power_of_2(nnz) buckets (grown like `set` would grow it) holding every non-zero element.  The dense
        tensor is scanned twice (count, insert); no COO index tensor is built."""
        assert isinstance(tensor, Tensor)
        assert tensor.layout == torch.strided
        if tensor.ndim == 0 or tensor.ndim > L.MAX_KEY_SIZE or tensor.dtype == torch.bool or tensor.is_complex() \
                or tensor.device.type != "cuda":
            return cls.from_sparse_coo(tensor.to_sparse())
        lib = L.lib()
        dense = tensor.contiguous()
        device = dense.device
        es = dense.element_size()
        is_float = int(dense.dtype.is_floating_point)
        with torch.cuda.device(device):
            st = L.stream_ptr(device)
            count = torch.zeros(1, device=device, dtype=torch.long)
            L.check(lib.dok_dense_count_nonzero(L.ptr(dense), dense.numel(), es, is_float, L.ptr(count), st),
                    "dok_dense_count_nonzero")
            nnz = int(count.item())
        new = cls(size=tuple(dense.shape), device=device, dtype=dense.dtype)
        hashmap = CudaClosedHashmap(n_buckets=next_power_of_2(nnz), device=device)
        new._hashmap = hashmap
        hashmap._begin_bulk_insert((dense.ndim,), torch.long, (1,), dense.dtype, nnz)
        if nnz:
            sizes = (ctypes.c_int64 * dense.ndim)(*dense.shape)
            cnt = hashmap._counters()
            with torch.cuda.device(device):
                L.check(lib.dok_dense_insert_nonzero(hashmap._c_table(), hashmap._c_hash(), L.ptr(dense), sizes,
                                                     dense.numel(), is_float, L.ptr(cnt), L.stream_ptr(device)),
                        "dok_dense_insert_nonzero")
        return new

    @classmethod
    def from_storage(cls, storage: CudaClosedHashmap, size=None):
        assert isinstance(storage, CudaClosedHashmap)
        assert storage.value_shape == (1,)
        assert len(storage.key_shape) == 1
        ndims = storage.key_shape[0]
        if size is None:
            size = tuple(storage.keys().max(dim=0).values.cpu().tolist())
        else:
            assert len(size) == ndims
            assert all(i >= 0 for i in size)
        return cls(size=tuple(size), storage=storage)

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        if kwargs is None:
            kwargs = {}
        args = [arg.to_sparse_coo() if isinstance(arg, cls) else arg for arg in args]
        kwargs = {key: (arg.to_sparse_coo() if isinstance(arg, cls) else arg) for key, arg in kwargs.items()}
        return func(*args, **kwargs)

    # ------------------------------------------------------------------ properties
    @property
    def is_sparse(self):
        return True

    def _is_coalesced(self):
        return False

    def is_coalesced(self):
        return False

    def size(self):
        return self._size

    @property
    def shape(self):
        return self.size()

    def _stride(self, dim=None):
        stride = util.shape_to_stride(self.shape)
        return stride if dim is None else stride[dim]

    @property
    def dtype(self):
        return self._dtype

    @property
    def ndim(self):
        return len(self.shape)

    def _nnz(self):
        return self._hashmap.n_elements

    @property
    def sparsity(self):
        return 1 - self._nnz() / float(np.prod(self.shape))

    def storage(self):
        return self._hashmap

    def clone(self, deepclone=True):
        new = SparseDOKTensor(size=tuple(self._size), indices=None, values=None, device=self.device, dtype=self.dtype)
        new._hashmap = self._hashmap.clone(deepclone=deepclone)
        return new

    def resize(self, *new_size):
        new_size = new_size + (self.ndim - len(new_size)) * (-1,)
        assert len(new_size) == self.ndim
        self._size = torch.Size([self.shape[i] if new_size[i] == -1 else new_size[i] for i in range(self.ndim)])

    # ------------------------------------------------------------------ conversion
    def _indices(self):
        return self._hashmap._keys

    def _values(self):
        return self._hashmap._values

    def indices(self):
        if self._hashmap._keys is None:
            return torch.empty(self.ndim, 0, device=self.device, dtype=torch.long)
        return self._hashmap.items(values=False, uuid=False, transposed_keys=True)[0]

    def values(self):
        if self._hashmap._values is None:
            return torch.empty(0, device=self.device, dtype=self.dtype)
        return self._hashmap.items(keys=False, uuid=False)[1].flatten()

    def set_values(self, selectors, new_values):
        self._hashmap.set_values(selectors=selectors, new_values=new_values[:, None])

    def to_sparse_coo(self):
        """Uncoalesced COO in slot order (sparse_dok_tensor.py:195-203); indices and values come from ONE pass."""
        if self._hashmap._keys is None:
            indices, values = self.indices(), self.values()
        else:
            indices, values, _ = self._hashmap.items(uuid=False, transposed_keys=True)
            values = values.flatten()
        return torch.sparse_coo_tensor(indices=indices, values=values, size=tuple(self.shape), device=self.device)

    @property
    def _as_sparse_coo_tensor(self):
        return self.to_sparse_coo()

    def to_sparse_csr(self):
        return self.to_sparse_coo().to_sparse_csr()

    def to_dense(self):
        return self.to_sparse_coo().to_dense()

    # ------------------------------------------------------------------ indexing
    def _handle_selectors(self, selectors, return_slice_as_tensor=True):
        return normalise_selectors(selectors, self.shape, self.device)

    def __getitem__(self, selectors):
        """Dense gather with zero fill (sparse_dok_tensor.py:302-315)."""
        selectors, scalar_positions = self._handle_selectors(selectors)
        shape = tuple(selectors[0].shape)
        values = torch.empty(shape, device=self.device, dtype=self.dtype)
        hashmap = self._hashmap
        if hashmap._values is None:
            values.zero_()
        elif values.numel():
            sel = _selectors_struct(selectors)
            with torch.cuda.device(self.device):
                L.check(L.lib().dok_dok_get(hashmap._c_table(), hashmap._c_hash(), ctypes.byref(sel), L.ptr(values), None,
                                            None, None, L.stream_ptr(self.device)), "dok_dok_get")
        for i in reversed(scalar_positions):
            if i < values.ndim and values.shape[i] == 1:
                values = values.squeeze(i)
        return values

    def __spgetitem__(self, selectors):
        """Sparse gather (sparse_dok_tensor.py:342-350 -> get_items, sparse_dok_tensor_impl.py:148-232; kernels
        sparse_dok_tensor_impl.cu:110-268): a SparseDOKTensor of the selection's broadcast shape that holds the selected
        positions which are stored, keyed by their position in the selection.  Two fused kernels over the selectors,
        like the reference: a count of the hits (it sizes the new map: int(2 * hits) buckets), then lookup and insert
        into the new map in one kernel.  A selection without a hit gives an empty tensor (the reference builds a
        0-bucket map)."""
        selectors, _ = self._handle_selectors(selectors)
        shape = tuple(selectors[0].shape)
        hashmap = self._hashmap
        n_sel = int(selectors[0].numel())
        if hashmap._values is None or n_sel == 0:
            return SparseDOKTensor(size=shape, device=self.device, dtype=self.dtype)
        sel = _selectors_struct(selectors)
        lib = L.lib()
        # pass 1: how many selected positions are stored (sizes the new map like the reference: int(2 * hits) buckets)
        cnt = hashmap._counters()
        with torch.cuda.device(self.device):
            L.check(lib.dok_dok_count_exists(hashmap._c_table(), hashmap._c_hash(), ctypes.byref(sel), L.ptr(cnt),
                                             L.stream_ptr(self.device)), "dok_dok_count_exists")
        n = int(cnt[L.CNT_HITS].item())
        if not shape:
            shape = (1,)                                       # all selectors scalar: a one-element selection
        if n == 0:
            return SparseDOKTensor(size=shape, device=self.device, dtype=self.dtype)
        out = CudaClosedHashmap(n_buckets=int(n * 2.0), device=self.device)
        out._begin_bulk_insert((len(shape),), torch.long, (1,), self.dtype, n)
        # pass 2: lookup and insert in ONE kernel (positions in the selection are the new keys)
        cnt = hashmap._counters()
        with torch.cuda.device(self.device):
            rc = lib.dok_dok_gather_insert(hashmap._c_table(), hashmap._c_hash(), ctypes.byref(sel), out._c_table(),
                                           out._c_hash(), L.ptr(cnt), L.stream_ptr(self.device))
        if rc == 3:                                            # a table served in passes: lookup, then insert
            values = torch.empty(n_sel, device=self.device, dtype=self.dtype)
            found = torch.empty(n_sel, device=self.device, dtype=torch.bool)
            with torch.cuda.device(self.device):
                L.check(lib.dok_dok_get(hashmap._c_table(), hashmap._c_hash(), ctypes.byref(sel), L.ptr(values),
                                        L.ptr(found), None, None, L.stream_ptr(self.device)), "dok_dok_get")
            hits = found.nonzero().flatten()
            keys = torch.stack(torch.unravel_index(hits, shape), dim=1)
            out.set_rows(keys.contiguous(), values[hits][:, None].contiguous(), assume_unique=True)
            out._n_elements.fill_(n)
        else:
            L.check(rc, "dok_dok_gather_insert")
        return SparseDOKTensor.from_storage(out, size=shape)

    def _set_items_sparse(self, src, selectors):
        """Assignment of a sparse source of the selection's shape (set_items_sparse, sparse_dok_tensor_impl.py:234-340):
        every selected position that is stored is removed, the table is rebuilt with
        ceil((n_elements + nnz(src)) * rehash_factor * 2) buckets -- unconditionally, as in the reference -- and the
        stored elements of the source are inserted at the positions the selectors map them to; n_elements grows by
        nnz(src).  Equal destination positions: the last source element wins (the reference's kernel races)."""
        hashmap = self._hashmap
        if isinstance(src, SparseDOKTensor):
            if src._hashmap._values is None:
                src_indices = torch.zeros(len(src.shape), 0, device=self.device, dtype=torch.long)
                src_values = torch.zeros(0, device=self.device, dtype=self.dtype)
            else:
                src_indices, src_values = src.indices(), src.values()
        else:
            src = src if src.layout == torch.sparse_coo else src.to_sparse_coo()
            src_indices, src_values = src._indices(), src._values()
        assert selectors[0].ndim == src_indices.shape[0]
        src_indices = src_indices.to(self.device)
        src_values = src_values.to(device=self.device, dtype=self.dtype)
        first = (0,) * selectors[0].ndim
        if hashmap._keys is None:            # the reference seeds an empty map with a zero at the first position (:236-239)
            first_key = torch.stack([s[first] for s in selectors], dim=0)[None]
            hashmap.set(first_key, torch.zeros(1, 1, device=self.device, dtype=self.dtype))
        if selectors[0].numel():
            cnt = hashmap._counters()
            sel = _selectors_struct(selectors)
            with torch.cuda.device(self.device):
                L.check(L.lib().dok_dok_zero_items(hashmap._c_table(), hashmap._c_hash(), ctypes.byref(sel), L.ptr(cnt),
                                                   L.stream_ptr(self.device)), "dok_dok_zero_items")
            hashmap._n_elements -= cnt[L.CNT_HITS]
            hashmap._after_mutation(0)
        n_src = int(src_values.shape[0])
        hashmap.rehash(math.ceil((hashmap.n_elements + n_src) * hashmap._rehash_factor * 2))
        if n_src:
            where = tuple(src_indices[d] for d in range(src_indices.shape[0]))
            dest_keys = torch.stack([s[where] for s in selectors], dim=1).contiguous()
            hashmap = self._hashmap
            before = hashmap.n_elements
            hashmap.set(dest_keys, src_values[:, None].contiguous())
            # the reference adds nnz(src) whatever was new (:340)
            hashmap._n_elements += n_src - (hashmap.n_elements - before)
            hashmap._after_mutation(n_src)

    def __setitem__(self, selectors, values):
        """Dense assignment (sparse_dok_tensor.py:317-327 -> sparse_dok_tensor_impl.py:412-474).  A Python scalar is
        treated like a 0-dim tensor, as the reference's README documents."""
        selectors, _ = self._handle_selectors(selectors)
        shape = selectors[0].shape
        if isinstance(values, SparseDOKTensor) or (isinstance(values, Tensor) and values.is_sparse):
            assert tuple(values.shape) == tuple(shape), f"expecting the value shape to be {tuple(shape)}, got {tuple(values.shape)} instead"
            self._set_items_sparse(values, selectors)
            return
        if not isinstance(values, Tensor):
            values = torch.tensor(values, device=self.device, dtype=self.dtype)
        values = torch.broadcast_to(values.to(device=self.device, dtype=self.dtype), shape)
        self._set_items_dense(values, selectors)

    def _count_existing(self, selectors):
        hashmap = self._hashmap
        cnt = hashmap._counters()
        sel = _selectors_struct(selectors)
        with torch.cuda.device(self.device):
            L.check(L.lib().dok_dok_count_exists(hashmap._c_table(), hashmap._c_hash(), ctypes.byref(sel), L.ptr(cnt),
                                                 L.stream_ptr(self.device)), "dok_dok_count_exists")
        return cnt[L.CNT_HITS]

    def count_items(self, selectors):
        """Number of selected positions that are stored (sparse_dok_tensor_impl.py:56-108)."""
        selectors, _ = self._handle_selectors(selectors)
        if self._hashmap._values is None or selectors[0].numel() == 0:
            return 0
        return int(self._count_existing(selectors).item())

    def _set_items_dense(self, src, selectors):
        hashmap = self._hashmap
        n_sel = int(selectors[0].numel())
        if n_sel == 0:
            return
        first = (0,) * selectors[0].ndim
        if hashmap._keys is None:
            # the reference seeds an empty map with the first element before counting (:413-416)
            first_key = torch.stack([s[first] for s in selectors], dim=0)[None]
            hashmap.set(first_key, src[first].reshape(1, 1))
        n_existing = self._count_existing(selectors)          # device scalar, no sync
        # rehash decision of the reference (:461-462) depends on n_elements and the batch size only
        if hashmap._element_bound() + n_sel > hashmap.n_buckets * hashmap._rehash_threshold:
            n_elements = hashmap.n_elements
            if n_elements + n_sel > hashmap.n_buckets * hashmap._rehash_threshold:
                hashmap.rehash(math.ceil((n_elements + n_sel) * hashmap._rehash_factor))
        sel = _selectors_struct(selectors)
        src_strides = (ctypes.c_int64 * L.MAX_SELECTOR_NDIM)(*src.stride())
        epoch = hashmap._next_epoch()
        scratch = torch.empty(n_sel + 1, device=self.device, dtype=torch.long)
        with torch.cuda.device(self.device):
            L.check(L.lib().dok_dok_set_dense(hashmap._c_table(), hashmap._c_hash(), ctypes.byref(sel), L.ptr(src),
                                              src_strides, L.ptr(scratch), epoch, None, L.stream_ptr(self.device)),
                    "dok_dok_set_dense")
        hashmap._n_elements += n_sel - n_existing             # duplicates over-count, like the reference (:474)
        hashmap._after_mutation(n_sel)

    def zero_items(self, selectors):
        """Removes the selected positions that are stored; returns how many (sparse_dok_tensor_impl.py:110-146)."""
        selectors, _ = self._handle_selectors(selectors)
        hashmap = self._hashmap
        if hashmap._values is None or selectors[0].numel() == 0:
            return 0
        cnt = hashmap._counters()
        sel = _selectors_struct(selectors)
        with torch.cuda.device(self.device):
            L.check(L.lib().dok_dok_zero_items(hashmap._c_table(), hashmap._c_hash(), ctypes.byref(sel), L.ptr(cnt),
                                               L.stream_ptr(self.device)), "dok_dok_zero_items")
        hashmap._n_elements -= cnt[L.CNT_HITS]
        hashmap._after_mutation(0)
        return int(cnt[L.CNT_HITS].item())

    # ------------------------------------------------------------------ views and reshapes
    def permute_(self, *ordering):
        self._hashmap.key_perm = ordering
        self._size = torch.Size(self._size[i] for i in ordering)
        return self

    def permute(self, *ordering):
        new = self.clone(False)
        new._hashmap.key_perm = ordering
        new._size = torch.Size(new._size[i] for i in ordering)
        return new

    def _swap_ordering(self, dim0, dim1):
        assert dim0 != dim1
        dim0, dim1 = dim0 % self.ndim, dim1 % self.ndim
        ordering = list(range(self.ndim))
        ordering[dim0], ordering[dim1] = dim1, dim0
        return ordering

    def transpose_(self, dim0, dim1):
        return self.permute_(*self._swap_ordering(dim0, dim1))

    def transpose(self, dim0, dim1):
        return self.permute(*self._swap_ordering(dim0, dim1))

    def t(self):
        assert self.ndim == 2, "tensor isn't 2 dimensional, try x.transpose(dim1, dim2)"
        return self.transpose(0, 1)

    @property
    def T(self):
        return self.t()

    def _rekeyed(self, new_shape):
        """This tensor with its stored positions re-expressed in `new_shape` (same number of elements), built by ONE
        kernel that walks the slots, re-keys and inserts (dok_dok_rekey_insert); the table gets
        next_power_of_2(nnz) buckets like a tensor constructed from indices and values."""
        new_shape = tuple(int(x) for x in new_shape)
        hashmap = self._hashmap
        if hashmap._values is None:
            return SparseDOKTensor(size=new_shape, device=self.device, dtype=self.dtype)
        live = hashmap.count_live()
        out = CudaClosedHashmap(n_buckets=next_power_of_2(live), device=self.device)
        out._begin_bulk_insert((len(new_shape),), torch.long, (1,), self.dtype, live)
        if live:
            cnt = out._counters()
            old_sizes = (ctypes.c_int64 * len(self.shape))(*[int(x) for x in self.shape])
            new_sizes = (ctypes.c_int64 * len(new_shape))(*new_shape)
            with torch.cuda.device(self.device):
                L.check(L.lib().dok_dok_rekey_insert(hashmap._c_table(), hashmap._c_hash(), old_sizes, out._c_table(),
                                                     out._c_hash(), new_sizes, L.ptr(cnt), L.stream_ptr(self.device)),
                        "dok_dok_rekey_insert")
        return SparseDOKTensor.from_storage(out, size=new_shape)

    def flatten(self):
        """(sparse_dok_tensor.py:479-489)"""
        return self._rekeyed((int(np.prod(self.shape)),))

    def reshape(self, *new_shape):
        """(sparse_dok_tensor.py:491-514).  The reference builds the flattened tensor first and the reshaped one from
        it; here the slots are re-keyed straight into the new shape, and the random draws that the skipped
        intermediate table would have consumed are consumed all the same."""
        if len(new_shape) == 1 and isinstance(new_shape[0], (tuple, list, torch.Size)):
            new_shape = tuple(new_shape[0])
        assert np.prod(new_shape) == np.prod(self.shape)
        if len(new_shape) == 1:
            return self.flatten()
        if self._hashmap._values is not None:
            live = self._hashmap.count_live()
            util.consume_fresh_map_draws(next_power_of_2(live), 1, live)
        return self._rekeyed(new_shape)

    # ------------------------------------------------------------------ elementwise on stored values
    def _unary(self, name, *args, **kwargs):
        result = self.clone()
        getattr(result._values(), name)(*args, **kwargs)
        return result

    def abs(self):
        return self._unary("abs_")

    def sqrt(self):
        assert self.dtype in {torch.half, torch.float, torch.double}
        return self._unary("sqrt_")

    def ceil(self):
        assert self.dtype in {torch.half, torch.float, torch.double}
        return self._unary("ceil_")

    def floor(self):
        assert self.dtype in {torch.half, torch.float, torch.double}
        return self._unary("floor_")

    def round(self, decimals=0):
        assert self.dtype in {torch.half, torch.float, torch.double}
        return self._unary("round_", decimals=decimals)

    def index_select(self, dim, index):
        return self.to_sparse_coo().index_select(dim=dim, index=index)

    def select(self, dim, index):
        return self.to_sparse_coo().select(dim=dim, index=index)

    def __repr__(self) -> str:
        return (f"SparseDOKTensor(indices={self.indices()},\n                values={self.values()},\n"
                f"                size={self.size()}, nnz={self._nnz()}, sparsity={round(self.sparsity, 6)})")
