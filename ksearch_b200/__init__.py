"""ksearch_b200: a B200 (sm_100a) backend for the single-token decode path of ksearch.

The product is libksearch_cuda.so (C ABI in include/ksearch_cuda.h); this
package holds its sources, its build recipe and a thin host-side mirror of the
reference's op interface.  Importing the package does not load the library;
creating a ``CudaContext`` does, and fails loudly without an sm_100 GPU.
"""
from ._lib import F16, F32, Q4K, Q5K, Q6K, Q40  # noqa: F401
from .eng import Buffer, CudaContext, Eng, KsError, q40_nbytes, q40_row_bytes, q4k_nbytes, q6k_nbytes, write_meta  # noqa: F401

__all__ = ["Buffer", "CudaContext", "Eng", "KsError", "F32", "F16", "Q4K", "Q5K", "Q6K", "Q40",
           "q40_nbytes", "q40_row_bytes", "q4k_nbytes", "q6k_nbytes", "write_meta"]
