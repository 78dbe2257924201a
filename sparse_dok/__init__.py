"""Drop-in import name of the reference package: `from sparse_dok import SparseDOKTensor, CudaClosedHashmap`
(sparse_dok/__init__.py:1 of the reference) resolves to the B200 implementation."""
from doksparse_b200 import CudaClosedHashmap, SparseDOKTensor

__all__ = ["SparseDOKTensor", "CudaClosedHashmap"]
