"""Host-side Python mirror of libh3q8's C interface (ctypes).

The library is CUDA-only: importing works anywhere, but every operator needs the
in-tree `libh3q8.so` and a B200; nothing here computes on the CPU.
"""
from .api import Gpu, Tensor, H3Error, LinearDesc, WeightStream, q8_blob, library, MODE_BF16, MODE_W8A16, MODE_W8A8, \
    ACT_NONE, ACT_GELU_TANH, ACT_SWIGLU, KERNEL_AUTO, KERNEL_PLAIN, KERNEL_TCGEN05, KERNEL_TCGEN05_M256, KERNEL_TCGEN05_N128, KERNEL_TCGEN05_PAIR, \
    KERNEL_TCGEN05_SPLITK, KERNEL_TCGEN05_SKINNY

__all__ = ["Gpu", "Tensor", "H3Error", "LinearDesc", "WeightStream", "q8_blob", "library", "MODE_BF16", "MODE_W8A16", "MODE_W8A8",
           "ACT_NONE", "ACT_GELU_TANH", "ACT_SWIGLU", "KERNEL_AUTO", "KERNEL_PLAIN", "KERNEL_TCGEN05", "KERNEL_TCGEN05_M256",
           "KERNEL_TCGEN05_N128", "KERNEL_TCGEN05_PAIR", "KERNEL_TCGEN05_SPLITK", "KERNEL_TCGEN05_SKINNY"]
