"""B200-native BitLinear forward path behind the reference's operator API.

``cuda``      -- the bitnet-cuda crate's surface (CudaBackend, configs, errors)
``ops``       -- kernel-level operators on torch CUDA tensors (single calls, grouped calls, attention, sampler)
``bitlinear`` -- BitLinear / BitLinearLayer / FeedForwardNetwork
``pipeline``  -- ForwardPassPipeline / SamplingConfig / CudaInferenceBackend (the decode loop)
``parallel``  -- row sharding and the output-feature-split layer over several GPUs
All of them call libbitnet_cuda_kernels.so (see include/bitnet_cuda.h); nothing here
computes on the CPU.
"""
from . import _lib  # noqa: F401

__all__ = ["_lib", "cuda", "ops", "bitlinear", "pipeline", "parallel"]
__version__ = "0.1.0"
