"""doksparse_b200: the batched GPU hash map and DOK sparse tensor of DeMoriarty/DOKSparse, written for
NVIDIA B200 (sm_100a).  `CudaClosedHashmap` and `SparseDOKTensor` keep the reference's Python API;
`ShardedClosedHashmap` spreads one logical map over the GPUs of a node."""
from .cuda_closed_hashmap import CudaClosedHashmap
from .sparse_dok_tensor import SparseDOKTensor

__all__ = ["CudaClosedHashmap", "SparseDOKTensor"]
