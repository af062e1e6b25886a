"""tab_b200 - B200 (sm_100a) implementation of TAB's ternary/binary quantise + popcount convolution.

Host-side mirror of the reference's PyTorch-extension interface (``TAB_GPU.cpp:34-65``): the same two
operators, the same positional arguments, the same error behaviour for non-CUDA / non-contiguous
inputs, implemented over the C ABI in ``include/tab_b200.h``.  torch is used for device memory and
streams only; all arithmetic happens in the library's CUDA kernels.
"""
from .ops import (Quantize, Conv2d, TAB_Quantize, TAB_Conv2d, Conv2dFused, conv2d_packed, conv_out_size,  # noqa: F401
                  residual_threshold)

__all__ = ["Quantize", "Conv2d", "TAB_Quantize", "TAB_Conv2d", "Conv2dFused", "conv2d_packed", "conv_out_size",
           "residual_threshold"]
