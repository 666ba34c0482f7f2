"""clusternet_b200: B200-native dot / dotMPI / 8-bit codec / batch-allocator path of clusterNet.

The product is the C-ABI shared library built from clusternet_b200/csrc (include/clusternet_b200.h) and the
C++ facade in clusternet_b200/cpp.  This Python package is a thin harness over that ABI: it holds device
memory in torch tensors and passes raw pointers down.
"""
from . import _lib
from ._lib import CnError, Epilogue, load, check
from .api import Context, codebook_path, load_codebook, read_hdf5, read_sparse_hdf5, write_hdf5

__all__ = ["Context", "CnError", "Epilogue", "load", "check", "codebook_path", "load_codebook", "read_hdf5", "read_sparse_hdf5", "write_hdf5"]
