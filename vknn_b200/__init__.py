"""vknn_b200 — B200 (sm_100a) CUDA kernels for VKNN's transformer-attention / encoder hot path.

The product is `libvknn_cuda.so` (C-ABI in include/vknn_cuda.h) plus the C++17 `CudaBackend` plug-in in
vknn_b200/backend/ that sits behind VKNN's `vknn::Backend` / `vknn::Segment` interface. This Python package
is a thin ctypes binding of the same C-ABI, used by the tests and the benchmark; PyTorch only supplies device
memory, streams and the process group. There is no CPU or eager fallback: importing works without a GPU, but
every compute call needs the built library and a B200, and fails loudly otherwise.
"""
from .capi import (  # noqa: F401
    F32, F16, BF16, EPI_NONE, EPI_BIAS, EPI_GELU_ERF, EPI_RESIDUAL, B_KN, B_NK, IMPL_AUTO, IMPL_SIMT, IMPL_TCGEN05,
    VkcError, Context, lib_path, load_library, exported_symbols, declared_symbols,
)
