"""Python face of the reference's ``bitnet-cuda`` crate: same names, argument meaning and
error behaviour as ``CudaBackend`` / ``CudaBackendConfig`` / ``W2A8GemvConfig`` /
``CudaMemoryManager`` / ``CudaError`` (bitnet-cuda/src/{backend,memory,stream,error}.rs,
kernels/w2a8_gemv.rs), implemented by libbitnet_cuda_kernels through ctypes.

torch is used for device memory and streams only; every computation is a call into the
shared library.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from enum import Enum

from . import _lib as L


class CudaError(Exception):
    """Base of the error family of bitnet-cuda/src/error.rs:7-56."""
    status = -1

    def __init__(self, message: str = "", status: int | None = None):
        super().__init__(message)
        if status is not None:
            self.status = status

    def is_recoverable(self) -> bool:      # error.rs:88-103
        return bool(L.load().bitnet_is_recoverable(self.status))


class CudaNotEnabled(CudaError): status = L.ERR_CUDA_NOT_ENABLED
class CudaDriver(CudaError): status = L.ERR_CUDA_DRIVER
class DeviceError(CudaError): status = L.ERR_DEVICE
class MemoryAllocation(CudaError): status = L.ERR_MEMORY_ALLOCATION
class KernelExecution(CudaError): status = L.ERR_KERNEL_EXECUTION
class InvalidConfig(CudaError): status = L.ERR_INVALID_CONFIG
class UnsupportedOperation(CudaError): status = L.ERR_UNSUPPORTED_OPERATION
class StreamSync(CudaError): status = L.ERR_STREAM_SYNC
class UnsupportedDataType(CudaError): status = L.ERR_UNSUPPORTED_DTYPE
class IncompatibleShapes(CudaError): status = L.ERR_INCOMPATIBLE_SHAPES
class PerformanceDegradation(CudaError): status = L.ERR_PERFORMANCE
class NullPointer(CudaError): status = L.ERR_NULL_POINTER
class WorkspaceError(CudaError): status = L.ERR_WORKSPACE


_BY_STATUS = {cls.status: cls for cls in (
    CudaNotEnabled, CudaDriver, DeviceError, MemoryAllocation, KernelExecution, InvalidConfig,
    UnsupportedOperation, StreamSync, UnsupportedDataType, IncompatibleShapes, PerformanceDegradation,
    NullPointer, WorkspaceError)}


def check(status: int) -> None:
    """Raise the CudaError that corresponds to a non-zero status."""
    if status != L.OK:
        raise _BY_STATUS.get(status, CudaError)(L.last_error(), status)


class GridStrategy(Enum):          # w2a8_gemv.rs:41-49
    Fixed = 0
    Dynamic = 1
    Occupancy = 2


class CoalescingLevel(Enum):       # w2a8_gemv.rs:52-60
    NoOptimization = 0
    Basic = 1
    Aggressive = 2


@dataclass
class W2A8GemvConfig:              # w2a8_gemv.rs:15-38
    block_size: int = 256
    grid_strategy: GridStrategy = GridStrategy.Dynamic
    grid_fixed: int = 0
    enable_weight_permutation: bool = True
    enable_dp4a: bool = True
    coalescing_level: CoalescingLevel = CoalescingLevel.Aggressive


@dataclass
class CudaBackendConfig:           # backend.rs:14-37
    device_id: int = 0
    memory_pool_size: int = 1024 * 1024 * 1024
    num_streams: int = 4
    enable_profiling: bool = False
    w2a8_config: W2A8GemvConfig = field(default_factory=W2A8GemvConfig)

    def _c(self) -> L.BackendConfig:
        w = self.w2a8_config
        return L.BackendConfig(self.device_id, self.memory_pool_size, self.num_streams, int(self.enable_profiling),
                               L.W2A8Config(w.block_size, w.grid_strategy.value, w.grid_fixed,
                                            int(w.enable_weight_permutation), int(w.enable_dp4a),
                                            w.coalescing_level.value))


@dataclass
class PerformanceStats:            # backend.rs:262-290
    total_w2a8_operations: int
    average_execution_time_us: float
    memory_utilization_percent: float
    peak_bandwidth_gbps: float

    def meets_performance_targets(self) -> bool:
        return self.memory_utilization_percent >= MEMORY_BANDWIDTH_TARGET

    def performance_ratio(self, baseline_time_us: float) -> float:
        return baseline_time_us / self.average_execution_time_us if self.average_execution_time_us > 0 else 0.0


# lib.rs:26-36
W2A8_SPEEDUP_MIN, W2A8_SPEEDUP_MAX = 1.27, 3.63
MEMORY_BANDWIDTH_TARGET, COMPUTE_UTILIZATION_TARGET = 85.0, 90.0


def _ptr(t) -> int:
    """Device (or host) address of a torch tensor / numpy array / int."""
    if t is None:
        return 0
    if isinstance(t, int):
        return t
    if hasattr(t, "data_ptr"):
        return t.data_ptr()
    return t.ctypes.data


def _numel(t) -> int:
    return t.numel() if hasattr(t, "numel") else t.size


class CudaMemoryManager:
    """CudaMemoryManager view of a backend (memory.rs:47-186)."""

    def __init__(self, backend: "CudaBackend"):
        self._b = backend

    def allocate(self, nbytes: int) -> int:
        out = C.c_void_p()
        check(L.load().bitnet_backend_allocate(self._b._h, nbytes, C.byref(out)))
        return out.value or 0

    def free(self, ptr: int) -> None:
        check(L.load().bitnet_backend_free(self._b._h, ptr))

    def copy_to_device(self, host_array) -> int:
        ptr = self.allocate(host_array.nbytes)
        check(L.load().bitnet_backend_copy_to_device(self._b._h, ptr, host_array.ctypes.data, host_array.nbytes))
        return ptr

    def copy_to_host(self, ptr: int, out_array) -> None:
        check(L.load().bitnet_backend_copy_to_host(self._b._h, out_array.ctypes.data, ptr, out_array.nbytes))

    def _usage(self):
        a, p = C.c_size_t(), C.c_size_t()
        check(L.load().bitnet_backend_memory_usage(self._b._h, C.byref(a), C.byref(p)))
        return a.value, p.value

    def utilization_percent(self) -> float:
        a, p = self._usage()
        return a / p * 100.0 if p else 0.0

    def available_bytes(self) -> int:
        a, p = self._usage()
        return max(p - a, 0)


class DeviceWeights:
    """A packed ternary weight matrix resident on the device (upload once, launch many)."""

    def __init__(self, backend: "CudaBackend", handle: int):
        self._b, self._h = backend, handle
        n, k, s, p = C.c_size_t(), C.c_size_t(), C.c_float(), C.c_void_p()
        check(L.load().bitnet_weights_info(handle, C.byref(n), C.byref(k), C.byref(s), C.byref(p)))
        self.out_features, self.in_features, self.scale, self.data_ptr = n.value, k.value, s.value, p.value

    def free(self) -> None:
        if self._h:
            check(L.load().bitnet_backend_free_weights(self._b._h, self._h))
            self._h = 0

    def __del__(self):
        try:
            if self._h and self._b._h:
                self.free()
        except Exception:
            pass


class CudaBackend:
    """CudaBackend (backend.rs:40-213)."""

    def __init__(self, config: CudaBackendConfig | None = None):
        self.config = config or CudaBackendConfig()
        self._h = None
        cfg = self.config._c()
        out = C.c_void_p()
        check(L.load().bitnet_backend_create(C.byref(cfg), C.byref(out)))
        self._h = out.value
        self._mm = CudaMemoryManager(self)

    @classmethod
    def new(cls, config: CudaBackendConfig) -> "CudaBackend":
        return cls(config)

    def close(self) -> None:
        if self._h:
            L.load().bitnet_backend_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def memory_manager(self) -> CudaMemoryManager:
        return self._mm

    def stream(self, index: int) -> int:
        out = C.c_void_p()
        check(L.load().bitnet_backend_stream(self._h, index, C.byref(out)))
        return out.value or 0

    def synchronize(self) -> None:
        check(L.load().bitnet_backend_synchronize(self._h))

    def get_performance_stats(self) -> PerformanceStats:
        s = L.PerformanceStats()
        check(L.load().bitnet_backend_get_performance_stats(self._h, C.byref(s)))
        return PerformanceStats(s.total_w2a8_operations, s.average_execution_time_us,
                                s.memory_utilization_percent, s.peak_bandwidth_gbps)

    def w2a8_gemv(self, weights, activations, output, m: int, k: int, stream_idx: int = 0) -> None:
        """CudaBackend::w2a8_gemv (backend.rs:129-157): uint8 packed weights, int8 activations,
        int32 output, all device tensors; m = output features, k = input features."""
        check(L.load().bitnet_backend_w2a8_gemv(self._h, _ptr(weights), _numel(weights), _ptr(activations),
                                                _numel(activations), _ptr(output), _numel(output), m, k, stream_idx))

    def upload_packed(self, packed_host, out_features: int, in_features: int, scale: float) -> DeviceWeights:
        import numpy as np
        packed_host = np.ascontiguousarray(packed_host, dtype=np.uint8).reshape(-1)
        if packed_host.size != (out_features * in_features + 3) // 4:
            raise IncompatibleShapes(f"packed buffer has {packed_host.size} bytes, expected "
                                     f"{(out_features * in_features + 3) // 4}")
        out = C.c_void_p()
        check(L.load().bitnet_backend_upload_packed(self._h, packed_host.ctypes.data, out_features, in_features,
                                                    scale, C.byref(out)))
        return DeviceWeights(self, out.value)

    def upload_ternary(self, ternary_host, scale: float) -> DeviceWeights:
        import numpy as np
        t = np.ascontiguousarray(ternary_host, dtype=np.int8)
        if t.ndim != 2:
            raise IncompatibleShapes("ternary weights must be [out_features, in_features]")
        out = C.c_void_p()
        check(L.load().bitnet_backend_upload_ternary(self._h, t.ctypes.data, t.shape[0], t.shape[1], scale, C.byref(out)))
        return DeviceWeights(self, out.value)

    def upload_f32(self, weights_host) -> DeviceWeights:
        """Full-precision [out_features, in_features] weights: absmean quantisation and packing on the device."""
        import numpy as np
        w = np.ascontiguousarray(weights_host, dtype=np.float32)
        if w.ndim != 2:
            raise IncompatibleShapes("weights must be [out_features, in_features]")
        out = C.c_void_p()
        check(L.load().bitnet_backend_upload_f32(self._h, w.ctypes.data, w.shape[0], w.shape[1], C.byref(out)))
        return DeviceWeights(self, out.value)

    def upload_gguf_ternary(self, tensor_bytes, out_features: int, in_features: int):
        """A GGUF ternary tensor (8 bytes of scale/offset metadata + 2-bit codes, gguf.rs:1089-1165);
        returns (weights, offset)."""
        import numpy as np
        t = np.frombuffer(bytes(tensor_bytes), dtype=np.uint8) if not isinstance(tensor_bytes, np.ndarray) else np.ascontiguousarray(tensor_bytes, dtype=np.uint8)
        out, off = C.c_void_p(), C.c_float()
        check(L.load().bitnet_backend_upload_gguf_ternary(self._h, t.ctypes.data, t.size, out_features, in_features, C.byref(off), C.byref(out)))
        return DeviceWeights(self, out.value), off.value

    def bitlinear_forward(self, w: DeviceWeights, x, y, opts: L.ForwardOpts | None = None, stream_idx: int = 0) -> None:
        """x [M,K] fp32 -> y [M,N] fp32, both device tensors."""
        M = _numel(x) // w.in_features
        check(L.load().bitnet_backend_bitlinear_forward(self._h, w._h, _ptr(x), _ptr(y), M,
                                                        C.byref(opts) if opts else None, stream_idx))

    def bitlinear_forward_host(self, w: DeviceWeights, x_host, opts: L.ForwardOpts | None = None, stream_idx: int = 0):
        """The end-to-end call: host fp32 [M,K] in, host fp32 [M,N] out."""
        import numpy as np
        x = np.ascontiguousarray(x_host, dtype=np.float32)
        if x.ndim != 2 or x.shape[1] != w.in_features:
            raise IncompatibleShapes(f"expected [M,{w.in_features}], got {list(x.shape)}")
        y = np.empty((x.shape[0], w.out_features), dtype=np.float32)
        check(L.load().bitnet_backend_bitlinear_forward_host(self._h, w._h, x.ctypes.data, y.ctypes.data, x.shape[0],
                                                             C.byref(opts) if opts else None, stream_idx))
        return y

    def ffn_forward_host(self, gate: DeviceWeights, up: DeviceWeights, down: DeviceWeights, x_host,
                         opts: L.ForwardOpts | None = None, stream_idx: int = 0, out=None):
        import numpy as np
        x = np.ascontiguousarray(x_host, dtype=np.float32)
        if x.ndim != 2 or x.shape[1] != gate.in_features:
            raise IncompatibleShapes(f"expected [M,{gate.in_features}], got {list(x.shape)}")
        y = out if out is not None else np.empty((x.shape[0], down.out_features), dtype=np.float32)
        check(L.load().bitnet_backend_ffn_forward_host(self._h, gate._h, up._h, down._h, x.ctypes.data, y.ctypes.data,
                                                       x.shape[0], C.byref(opts) if opts else None, stream_idx))
        return y

    def pin_host(self, array) -> None:
        """Page-locks a numpy array's memory so that host-buffer calls copy from/to it directly."""
        check(L.load().bitnet_backend_pin_host(self._h, array.ctypes.data, array.nbytes))

    def unpin_host(self, array) -> None:
        check(L.load().bitnet_backend_unpin_host(self._h, array.ctypes.data))

    def ffn_plan(self, calls, opts: L.ForwardOpts | None = None, n_lanes: int = 0) -> "FfnPlan":
        """`calls`: (gate, up, down, x_host, y_host) tuples; see FfnPlan."""
        return FfnPlan(self, calls, opts, n_lanes)

    def ffn_forward_host_async(self, gate: DeviceWeights, up: DeviceWeights, down: DeviceWeights, x_host, out,
                               opts: L.ForwardOpts | None = None, stream_idx: int = 0) -> None:
        """Queues the FFN block on stream `stream_idx` and returns; `out` (a C-contiguous float32 numpy
        array [M, hidden] that the caller keeps alive) is complete after `synchronize()` or after the next
        host-buffer call on the same stream (backend.rs:129-178: asynchronous launches, synchronize joins)."""
        import numpy as np
        x = np.ascontiguousarray(x_host, dtype=np.float32)
        if x.ndim != 2 or x.shape[1] != gate.in_features:
            raise IncompatibleShapes(f"expected [M,{gate.in_features}], got {list(x.shape)}")
        if out.dtype != np.float32 or not out.flags["C_CONTIGUOUS"] or out.shape != (x.shape[0], down.out_features):
            raise IncompatibleShapes(f"out must be a C-contiguous float32 array [{x.shape[0]},{down.out_features}]")
        check(L.load().bitnet_backend_ffn_forward_host_async(self._h, gate._h, up._h, down._h, x.ctypes.data, out.ctypes.data,
                                                             x.shape[0], C.byref(opts) if opts else None, stream_idx))


class FfnPlan:
    """A fixed batch of independent FFN blocks bound to host buffers, replayed as one unit
    (bitnet_backend_ffn_plan_*): the recorded form of a loop of asynchronous launches over the stream
    pool followed by CudaBackend::synchronize (backend.rs:129-178)."""

    def __init__(self, backend: "CudaBackend", calls, opts: L.ForwardOpts | None = None, n_lanes: int = 0):
        import numpy as np
        self._b, self._h = backend, None
        self._keep = []
        arr = (L.FfnCall * len(calls))()
        for i, (gate, up, down, x, y) in enumerate(calls):
            for name, a in (("x", x), ("y", y)):
                if a.dtype != np.float32 or not a.flags["C_CONTIGUOUS"] or a.ndim != 2 or a.shape[1] != gate.in_features:
                    raise IncompatibleShapes(f"call {i}: {name} must be a C-contiguous float32 array [M,{gate.in_features}]")
            if x.shape != y.shape:
                raise IncompatibleShapes(f"call {i}: x {x.shape} and y {y.shape} differ")
            arr[i] = L.FfnCall(gate._h, up._h, down._h, x.shape[0], x.ctypes.data, y.ctypes.data)
            self._keep.append((gate, up, down, x, y))
        out = C.c_void_p()
        check(L.load().bitnet_backend_ffn_plan_create(backend._h, arr, len(calls), C.byref(opts) if opts else None, n_lanes,
                                                      C.byref(out)))
        self._h = out.value

    def run(self) -> None:
        check(L.load().bitnet_backend_ffn_plan_run(self._h))

    def close(self) -> None:
        if self._h:
            L.load().bitnet_backend_ffn_plan_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            if self._b._h:
                self.close()
        except Exception:
            pass


def device_count() -> int:          # lib.rs:56-64
    n = C.c_int32()
    check(L.load().bitnet_device_count(C.byref(n)))
    return n.value


def is_cuda_available() -> bool:    # lib.rs:46-54
    n = C.c_int32()
    return L.load().bitnet_device_count(C.byref(n)) == L.OK and n.value > 0


def initialize() -> CudaBackend:    # lib.rs:40-43
    return CudaBackend(CudaBackendConfig())


def query_device(device_id: int = 0) -> L.DeviceInfo:
    info = L.DeviceInfo()
    check(L.load().bitnet_query_device(device_id, C.byref(info)))
    return info
