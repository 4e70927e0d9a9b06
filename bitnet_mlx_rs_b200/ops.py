"""Kernel-level operators on torch CUDA tensors: thin wrappers over the C ABI.

torch supplies device memory and the current stream; all arithmetic happens inside
libbitnet_cuda_kernels.  Every function raises a ``CudaError`` subclass on failure.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib as L
from .cuda import IncompatibleShapes, InvalidConfig, UnsupportedDataType, check

PATHS = {"auto": L.PATH_AUTO, "decode": L.PATH_DECODE, "prefill": L.PATH_PREFILL, "generic": L.PATH_GENERIC}
_workspaces: dict[tuple[int, int], torch.Tensor] = {}


def _stream(stream=None) -> int:
    return (stream or torch.cuda.current_stream()).cuda_stream


def _workspace(nbytes: int, device: torch.device, stream=None) -> torch.Tensor | None:
    """A scratch buffer per (device, stream the kernels are enqueued on), grown on demand and
    256-byte aligned: calls on different streams may overlap on the GPU and must not share one."""
    if nbytes == 0:
        return None
    key = (device.index or 0, _stream(stream))
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(nbytes + 256, dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def _aligned_ptr(ws: torch.Tensor | None) -> int:
    return 0 if ws is None else (ws.data_ptr() + 255) // 256 * 256


def _require(t: torch.Tensor, dtype: torch.dtype, name: str) -> torch.Tensor:
    if t.dtype != dtype:
        raise UnsupportedDataType(f"{name}: dtype {t.dtype} not supported on CUDA device (need {dtype})")
    if not t.is_cuda:
        raise IncompatibleShapes(f"{name} must be a CUDA tensor")
    return t.contiguous()


def packed_len(n_values: int) -> int:
    return (n_values + 3) // 4


def make_opts(path="auto", pdl=False, q_out=None, a_scale_out=None, acc_out=None, ldy=0, stages=0, y_peers=(),
              throughput=False) -> L.ForwardOpts:
    """``y_peers``: device addresses (ints) of the output slice in every GPU's full-width output."""
    if len(y_peers) > 8:
        raise InvalidConfig(f"at most 8 peer outputs (got {len(y_peers)})")
    peers = (C.c_void_p * 8)(*[C.c_void_p(int(p)) for p in y_peers])
    return L.ForwardOpts(PATHS[path] if isinstance(path, str) else path,
                         (L.FLAG_PDL if pdl else 0) | (L.FLAG_THROUGHPUT if throughput else 0),
                         q_out.data_ptr() if q_out is not None else None,
                         a_scale_out.data_ptr() if a_scale_out is not None else None,
                         acc_out.data_ptr() if acc_out is not None else None, ldy, stages, len(y_peers), peers)


def bitlinear_forward(wp: torch.Tensor, w_scale: float, x: torch.Tensor, out_features: int, *, path="auto",
                      pdl=False, debug=False, out: torch.Tensor | None = None, stages=0, stream=None, ldy=0, y_peers=(),
                      throughput=False):
    """y[M,N] = BitLinear(x[M,K]) with packed ternary weights ``wp`` (uint8, ceil(N*K/4) bytes).

    With ``debug=True`` also returns the int8 activations, per-token scales and int32
    accumulators as a dict (the parity tests compare those bit-exactly).
    """
    wp = _require(wp, torch.uint8, "weights")
    x = _require(x, torch.float32, "x")
    if x.dim() != 2:
        raise IncompatibleShapes(f"x must be [M,K], got {list(x.shape)}")
    M, K = x.shape
    N = out_features
    if wp.numel() != packed_len(N * K):
        raise IncompatibleShapes(f"Weight tensor size mismatch: expected {packed_len(N * K)} bytes for {N}x{K} matrix, "
                                 f"got {wp.numel()}")
    y = out if out is not None else torch.empty((M, N), dtype=torch.float32, device=x.device)
    dbg = {}
    if debug:
        dbg = {"q": torch.empty((M, K), dtype=torch.int8, device=x.device),
               "a_scale": torch.empty((M,), dtype=torch.float32, device=x.device),
               "acc": torch.empty((M, N), dtype=torch.int32, device=x.device)}
    opts = make_opts(path, pdl, dbg.get("q"), dbg.get("a_scale"), dbg.get("acc"), ldy, stages, y_peers, throughput)
    need = C.c_size_t()
    check(L.load().bitnet_bitlinear_workspace_size(M, K, N, opts.path, C.byref(need)))
    ws = _workspace(need.value, x.device, stream)
    check(L.load().bitnet_bitlinear_forward(wp.data_ptr(), w_scale, x.data_ptr(), y.data_ptr(), M, K, N, C.byref(opts),
                                            _aligned_ptr(ws), need.value, _stream(stream)))
    return (y, dbg) if debug else y


def w2a8_gemv(wp: torch.Tensor, a: torch.Tensor, n_out: int, out: torch.Tensor | None = None, stream=None):
    """Legacy single-token GEMV: int8 activations [K] -> int32 [n_out]."""
    wp = _require(wp, torch.uint8, "weights")
    a = _require(a, torch.int8, "activations")
    k = a.numel()
    if wp.numel() != packed_len(n_out * k):
        raise IncompatibleShapes(f"Weight tensor size mismatch: expected {packed_len(n_out * k)} bytes, got {wp.numel()}")
    y = out if out is not None else torch.empty((n_out,), dtype=torch.int32, device=a.device)
    check(L.load().bitnet_w2a8_gemv(wp.data_ptr(), a.data_ptr(), y.data_ptr(), n_out, k, _stream(stream)))
    return y


def quantize_activations(x: torch.Tensor, stream=None):
    """Per-token absmax int8 quantisation: returns (q int8 [M,K], a_scale fp32 [M])."""
    x = _require(x, torch.float32, "x")
    if x.dim() != 2:
        raise IncompatibleShapes(f"x must be [M,K], got {list(x.shape)}")
    M, K = x.shape
    q = torch.empty((M, K), dtype=torch.int8, device=x.device)
    s = torch.empty((M,), dtype=torch.float32, device=x.device)
    check(L.load().bitnet_quantize_activations(x.data_ptr(), M, K, q.data_ptr(), s.data_ptr(), _stream(stream)))
    return q, s


def ffn_forward(w_gate, s_gate, w_up, s_up, w_down, s_down, x: torch.Tensor, ffn: int, *, path="auto", pdl=False,
                out=None, h_out=None, stages=0, stream=None, throughput=False):
    """FFN block y = down(up(x) * relu(gate(x))^2); returns (y [M,hidden], h [M,ffn])."""
    x = _require(x, torch.float32, "x")
    M, hidden = x.shape
    for name, w, n, k in (("gate", w_gate, ffn, hidden), ("up", w_up, ffn, hidden), ("down", w_down, hidden, ffn)):
        _require(w, torch.uint8, name)
        if w.numel() != packed_len(n * k):
            raise IncompatibleShapes(f"{name}: expected {packed_len(n * k)} packed bytes, got {w.numel()}")
    y = out if out is not None else torch.empty((M, hidden), dtype=torch.float32, device=x.device)
    h = h_out if h_out is not None else torch.empty((M, ffn), dtype=torch.float32, device=x.device)
    opts = make_opts(path, pdl, stages=stages, throughput=throughput)
    need = C.c_size_t()
    check(L.load().bitnet_ffn_workspace_size(M, hidden, ffn, opts.path, C.byref(need)))
    ws = _workspace(need.value, x.device, stream)
    check(L.load().bitnet_ffn_forward(w_gate.data_ptr(), s_gate, w_up.data_ptr(), s_up, w_down.data_ptr(), s_down,
                                      x.data_ptr(), h.data_ptr(), y.data_ptr(), M, hidden, ffn, C.byref(opts),
                                      _aligned_ptr(ws), need.value, _stream(stream)))
    return y, h


def pack_ternary(w: torch.Tensor, stream=None) -> torch.Tensor:
    w = _require(w, torch.int8, "w")
    out = torch.empty((packed_len(w.numel()),), dtype=torch.uint8, device=w.device)
    check(L.load().bitnet_pack_ternary(w.data_ptr(), w.numel(), out.data_ptr(), _stream(stream)))
    return out


def unpack_ternary(packed: torch.Tensor, n_values: int, stream=None) -> torch.Tensor:
    packed = _require(packed, torch.uint8, "packed")
    if packed.numel() < packed_len(n_values):
        raise IncompatibleShapes(f"packed buffer too short for {n_values} values")
    out = torch.empty((n_values,), dtype=torch.int8, device=packed.device)
    check(L.load().bitnet_unpack_ternary(packed.data_ptr(), n_values, out.data_ptr(), _stream(stream)))
    return out


def device_error_flags() -> int:
    """Flags raised by bounded device-side waits since the last call (0 = none); synchronises."""
    v = C.c_uint32()
    check(L.load().bitnet_device_error_flags(C.byref(v)))
    return v.value


def sanitize_packed(packed: torch.Tensor, stream=None) -> int:
    """Rewrites the invalid code 3 to code 1 (weight 0) in place; returns how many were found."""
    packed = _require(packed, torch.uint8, "packed")
    count = torch.zeros((1,), dtype=torch.int64, device=packed.device)
    check(L.load().bitnet_sanitize_packed(packed.data_ptr(), packed.numel(), count.data_ptr(), _stream(stream)))
    return int(count.item())


def prepare_weights(packed: torch.Tensor, out_features: int, in_features: int, layout_id: int = 0, stream=None):
    """One-time preparation of a packed weight buffer (the reference's weight-permutation hook,
    bitnet-cuda/src/kernels/w2a8_gemv.rs:21, :259): removes code 3 in place and reports which fast
    kernels take the shape.  Returns (invalid codes found, {"decode": bool, "prefill": bool})."""
    packed = _require(packed, torch.uint8, "packed")
    if packed.numel() != packed_len(out_features * in_features):
        raise IncompatibleShapes(f"Weight tensor size mismatch: expected {packed_len(out_features * in_features)} bytes, "
                                 f"got {packed.numel()}")
    count = torch.zeros((1,), dtype=torch.int64, device=packed.device)
    mask = C.c_uint32(0)
    check(L.load().bitnet_prepare_weights(packed.data_ptr(), out_features, in_features, layout_id, count.data_ptr(),
                                          C.byref(mask), _stream(stream)))
    return int(count.item()), {"decode": bool(mask.value & 1), "prefill": bool(mask.value & 2)}
