"""Kernel directory of the package: the ctypes binding of libbitween_b200.so (`_lib`) and
the `cuda_loader` module that exports `quantized_matmul_cuda`, the symbol the reference's
scripts import from `bitween.kernels.cuda_loader` (main.py:401)."""
