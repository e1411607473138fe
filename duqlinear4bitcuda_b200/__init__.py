"""duqlinear4bitcuda_b200 -- a B200 (sm_100a) implementation of the DUQLinear4bitCUDA W4A4
linear layer behind that project's Python API.

    duqlinear4bitcuda_b200.nn      Linear4bit* / quantizer / quant-matmul modules
    duqlinear4bitcuda_b200.tools   functional wrappers (tensor_utils) and host-side packing helpers
    duqlinear4bitcuda_b200._CUDA   tensor-level operators (names of the reference's compiled module)
    duqlinear4bitcuda_b200.lib     ctypes binding of libduq4.so (C ABI in include/duq4.h)

`import qlinear4bit` (top-level alias package in this repository) resolves to these modules,
so code written against the reference imports unchanged.
"""
__version__ = "0.1.0"
