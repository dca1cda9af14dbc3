"""dataflow_lib_b200 -- sm_100a implementations of the native transformer ops of als244/dataflow_lib
(RMSNorm, RoPE, SwiGLU, softmax, cross entropy; forward and backward) behind that library's own
op-skeleton registry and Dataflow_Handle submit interface.

The product is the shared object lib/libdataflow_b200.so (C host layer + CUDA kernels, see
include/*.h). This Python package is a thin ctypes binding used by the tests and the benchmark:

    ops      -- the C-ABI kernel launchers on torch tensors (argument order of the reference kernels)
    handle   -- Dataflow_Handle: init / register_native_ops / submit_* / transfers, through the C API
    abi      -- ctypes mirrors of the ABI structs, DataflowDatatype
"""
from . import abi, _lib            # noqa: F401  (importing _lib fails loudly when the library is not built)
from .abi import DataflowDatatype  # noqa: F401
from . import ops, handle          # noqa: F401
from .handle import DataflowHandle  # noqa: F401
