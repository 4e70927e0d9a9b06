"""B200-native BitLinear forward path behind the reference's operator API.

``cuda``      -- the bitnet-cuda crate's surface (CudaBackend, configs, errors)
``ops``       -- kernel-level operators on torch CUDA tensors
``bitlinear`` -- BitLinear / BitLinearLayer / FeedForwardNetwork
All of them call libbitnet_cuda_kernels.so (see include/bitnet_cuda.h); nothing here
computes on the CPU.
"""
from . import _lib  # noqa: F401

__all__ = ["_lib", "cuda", "ops", "bitlinear"]
__version__ = "0.1.0"
