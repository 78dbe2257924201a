"""Selector normalisation for SparseDOKTensor indexing.

Restates what SparseDOKTensor._handle_selectors of the reference computes
(sparse_dok/components/sparse_dok_tensor.py:220-300): a tuple of selectors (ints, slices, lists, integer
or boolean tensors / arrays) becomes `ndim` int64 index tensors that are VIEWS broadcast to one common
shape, plus the positions of the scalar selectors.  Layout rule of the common shape: slice dims appear
in order; the block of broadcast index-tensor dims sits where the first index tensor appears.

Works on any device (the tests exercise it on CPU against fixtures generated from the reference).
Deliberate differences from the reference, all in places where the reference raises or misbehaves:
  * a bare int (`t[0]`) is accepted (the reference raises TypeError although its README shows it);
  * numpy arrays are accepted (the reference's ndarray branches call removed / invalid APIs);
  * negative slice bounds follow Python (the reference passes them to arange unchanged);
  * more selectors than dimensions raise IndexError.
Slice steps are ignored, as in the reference (:287-290).
"""
import numpy as np
import torch
from torch import Tensor

_INT_DTYPES = {torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8}


def normalise_selectors(selectors, shape, device):
    """Returns (index_tensors, scalar_positions).

    index_tensors: list of len(shape) int64 tensors, all broadcast (as views) to the common shape.
    scalar_positions: positions in the selector tuple that were scalars (int or 0-dim tensor).
    """
    ndim = len(shape)
    if isinstance(selectors, (Tensor, slice, np.ndarray, list, int, np.integer)):
        selectors = (selectors,)

    expanded = []
    for selector in selectors:
        if isinstance(selector, np.ndarray):
            selector = torch.from_numpy(selector)
        if isinstance(selector, Tensor) and selector.dtype == torch.bool:
            expanded += list(selector.to(device).nonzero(as_tuple=True))          # :226-228
        elif isinstance(selector, Tensor) and selector.dtype in _INT_DTYPES:
            expanded.append(selector.to(device).long())                           # :230-232
        elif isinstance(selector, (bool, np.bool_)):
            raise ValueError("boolean scalars are not valid selectors")
        elif isinstance(selector, (int, np.integer)):
            expanded.append(torch.tensor(int(selector), device=device, dtype=torch.long))   # :242-243
        elif isinstance(selector, slice):
            expanded.append(selector)                                             # :245-246
        elif isinstance(selector, (tuple, list)):
            expanded.append(torch.tensor(selector, device=device, dtype=torch.long))        # :248-250
        else:
            raise ValueError(f"unsupported selector of type {type(selector).__name__}")      # :252-253
    if len(expanded) > ndim:
        raise IndexError(f"too many indices: {len(expanded)} selectors for a {ndim}-dimensional tensor")
    expanded += [slice(None)] * (ndim - len(expanded))                            # :255

    scalar_positions = [i for i, s in enumerate(expanded) if isinstance(s, Tensor) and s.ndim == 0]   # :256
    tensor_shapes = [s.shape for s in expanded if isinstance(s, Tensor)]
    n_slices = sum(isinstance(s, slice) for s in expanded)
    block_shape = tuple(torch.broadcast_shapes(*tensor_shapes)) if tensor_shapes else ()             # :258-262
    out_ndim = len(block_shape) + n_slices                                        # :264
    first_tensor = next((i for i, s in enumerate(expanded) if isinstance(s, Tensor)), None)

    out = []
    axis = 0                       # next output axis for a slice
    block_placed = False
    for i, s in enumerate(expanded):
        if isinstance(s, Tensor):
            # the broadcast block occupies output axes [first_tensor, first_tensor + len(block_shape))   (:277-284)
            index = [None] * out_ndim
            for j in range(len(block_shape)):
                index[first_tensor + j] = slice(None)
            out.append(torch.broadcast_to(s, block_shape)[tuple(index)])          # a view: no index data is copied
            if not block_placed:
                axis += len(block_shape)
                block_placed = True
        else:
            start, stop, _ = _slice_bounds(s, int(shape[i]))                      # :286-290
            view_shape = [1] * out_ndim
            view_shape[axis] = stop - start
            out.append(torch.arange(start, stop, device=device).reshape(view_shape))
            axis += 1
    out = list(torch.broadcast_tensors(*out)) if out else []                      # :298-299
    return out, scalar_positions


def _slice_bounds(s, size):
    start = 0 if s.start is None else int(s.start)
    stop = size if s.stop is None else int(s.stop)
    if start < 0:
        start = max(start + size, 0)
    if stop < 0:
        stop = max(stop + size, 0)
    stop = max(min(stop, size), start)
    return start, stop, 1
