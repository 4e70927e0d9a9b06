"""Kernel-level operators on torch CUDA tensors: thin wrappers over the C ABI.

torch supplies device memory and the current stream; all arithmetic happens inside
libbitnet_cuda_kernels.  Every function raises a ``CudaError`` subclass on failure.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib as L
from .cuda import IncompatibleShapes, InvalidConfig, UnsupportedDataType, check

PATHS = {"auto": L.PATH_AUTO, "decode": L.PATH_DECODE, "prefill": L.PATH_PREFILL, "generic": L.PATH_GENERIC,
         "cluster": L.PATH_CLUSTER}
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


# ---- decoder-layer glue and decode-step pieces -----------------------------------------------------------

def make_glue(residual=None, sum_out=None, norm_weight=None, norm_bias=None, eps=1e-5, normed_out=None) -> L.RowGlue:
    p = lambda t: t.data_ptr() if t is not None else None   # noqa: E731
    return L.RowGlue(p(residual), p(sum_out), p(norm_weight), p(norm_bias), eps, p(normed_out))


def bitlinear_forward_fused(wp_stacked: torch.Tensor, rows, scales, x: torch.Tensor, *, glue: L.RowGlue | None = None,
                            path="auto", pdl=False, out=None, debug=False, stream=None):
    """Up to three BitLinears that share x, weights stacked along the output features (`rows` features and one
    scale each), with optional row glue (residual add, SubLN) applied to x first.  Returns y [M, sum(rows)]."""
    wp_stacked = _require(wp_stacked, torch.uint8, "weights")
    x = _require(x, torch.float32, "x")
    M, K = x.shape
    N = int(sum(rows))
    if wp_stacked.numel() != packed_len(N * K):
        raise IncompatibleShapes(f"Weight tensor size mismatch: expected {packed_len(N * K)} bytes, got {wp_stacked.numel()}")
    st = L.Stack(len(rows), (C.c_size_t * 3)(*rows), (C.c_float * 3)(*scales))
    y = out if out is not None else torch.empty((M, N), dtype=torch.float32, device=x.device)
    dbg = {}
    if debug:
        dbg = {"q": torch.empty((M, K), dtype=torch.int8, device=x.device),
               "a_scale": torch.empty((M,), dtype=torch.float32, device=x.device),
               "acc": torch.empty((M, N), dtype=torch.int32, device=x.device)}
    opts = make_opts(path, pdl, dbg.get("q"), dbg.get("a_scale"), dbg.get("acc"))
    need = C.c_size_t()
    check(L.load().bitnet_bitlinear_fused_workspace_size(M, K, N, opts.path, C.byref(need)))
    ws = _workspace(need.value, x.device, stream)
    check(L.load().bitnet_bitlinear_forward_fused(wp_stacked.data_ptr(), C.byref(st), x.data_ptr(), C.byref(glue) if glue else None,
                                                  y.data_ptr(), M, K, C.byref(opts), _aligned_ptr(ws), need.value, _stream(stream)))
    return (y, dbg) if debug else y


def ffn_forward_fused(w_gate, s_gate, w_up, s_up, w_down, s_down, x: torch.Tensor, ffn: int, *, glue: L.RowGlue | None = None,
                      path="auto", pdl=False, out=None, h_out=None, stream=None):
    """FFN block with row glue in front of the gate and up projections; returns (y, h)."""
    x = _require(x, torch.float32, "x")
    M, hidden = x.shape
    y = out if out is not None else torch.empty((M, hidden), dtype=torch.float32, device=x.device)
    h = h_out if h_out is not None else torch.empty((M, ffn), dtype=torch.float32, device=x.device)
    opts = make_opts(path, pdl)
    need = C.c_size_t()
    check(L.load().bitnet_ffn_fused_workspace_size(M, hidden, ffn, opts.path, C.byref(need)))
    ws = _workspace(need.value, x.device, stream)
    check(L.load().bitnet_ffn_forward_fused(w_gate.data_ptr(), s_gate, w_up.data_ptr(), s_up, w_down.data_ptr(), s_down,
                                            x.data_ptr(), C.byref(glue) if glue else None, h.data_ptr(), y.data_ptr(), M, hidden,
                                            ffn, C.byref(opts), _aligned_ptr(ws), need.value, _stream(stream)))
    return y, h


class BitLinearGroup:
    """A group of independent BitLinear calls of one shape [N, K] (at most 16 tokens each) run as two launches for the
    whole group (bitnet_bitlinear_group_*).  members: (packed weights uint8, w_scale, x [M, K], y [M, N]); the tensors
    are bound at creation and kept alive by the group."""

    def __init__(self, members, N: int, K: int):
        self._keep = []
        arr = (L.BitLinearGroupMember * len(members))()
        for i, (w, s, x, y) in enumerate(members):
            x = _require(x, torch.float32, "x")
            y = _require(y, torch.float32, "y")
            if x.dim() != 2 or x.shape[1] != K or y.dim() != 2 or y.shape[0] != x.shape[0] or y.shape[1] != N:
                raise IncompatibleShapes(f"member {i}: x must be [M,{K}] and y [M,{N}], got {list(x.shape)} and {list(y.shape)}")
            if w.dtype != torch.uint8 or not w.is_contiguous() or w.numel() != packed_len(N * K):
                raise IncompatibleShapes(f"member {i}: packed weights must hold {packed_len(N * K)} bytes")
            arr[i] = L.BitLinearGroupMember(w.data_ptr(), s, x.data_ptr(), y.data_ptr(), x.shape[0], 0)
            self._keep.append((w, x, y))
        self._device = members[0][2].device if members else None
        handle = C.c_void_p()
        with torch.cuda.device(self._device):
            check(L.load().bitnet_bitlinear_group_create(arr, len(members), K, N, C.byref(handle)))
        self._handle = handle

    def run(self, stream=None) -> None:
        check(L.load().bitnet_bitlinear_group_run(self._handle, _stream(stream)))

    def close(self) -> None:
        if getattr(self, "_handle", None):
            L.load().bitnet_bitlinear_group_destroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class FfnGroup:
    """A group of independent FFN blocks of one shape (at most 16 tokens each) run as four launches for the whole group
    (bitnet_ffn_group_*).  members: (w_gate, s_gate, w_up, s_up, w_down, s_down, x [M, hidden], y [M, hidden]) with the
    packed weights as uint8 tensors; the tensors are bound at creation and kept alive by the group."""

    def __init__(self, members, hidden: int, ffn: int):
        self._keep = []
        arr = (L.FfnGroupMember * len(members))()
        for i, (wg, sg, wu, su, wd, sd, x, y) in enumerate(members):
            x = _require(x, torch.float32, "x")
            y = _require(y, torch.float32, "y")
            if x.dim() != 2 or x.shape[1] != hidden or y.shape != x.shape:
                raise IncompatibleShapes(f"member {i}: x and y must be [M,{hidden}], got {list(x.shape)} and {list(y.shape)}")
            for name, w, n, k in (("gate", wg, ffn, hidden), ("up", wu, ffn, hidden), ("down", wd, hidden, ffn)):
                if w.dtype != torch.uint8 or not w.is_contiguous() or w.numel() != n * k // 4:
                    raise IncompatibleShapes(f"member {i}: packed {name} weights must hold {n}x{k}/4 bytes")
            arr[i] = L.FfnGroupMember(wg.data_ptr(), wu.data_ptr(), wd.data_ptr(), sg, su, sd, x.data_ptr(), y.data_ptr(), x.shape[0])
            self._keep.append((wg, wu, wd, x, y))
        self._device = members[0][6].device if members else None
        handle = C.c_void_p()
        with torch.cuda.device(self._device):
            check(L.load().bitnet_ffn_group_create(arr, len(members), hidden, ffn, C.byref(handle)))
        self._handle = handle

    def run(self, stream=None) -> None:
        check(L.load().bitnet_ffn_group_run(self._handle, _stream(stream)))

    def close(self) -> None:
        if getattr(self, "_handle", None):
            L.load().bitnet_ffn_group_destroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def row_glue(x: torch.Tensor, glue: L.RowGlue, stream=None) -> None:
    """The glue alone: writes x + residual to glue.sum_out and SubLN(x + residual) to glue.normed_out."""
    x = _require(x, torch.float32, "x")
    check(L.load().bitnet_row_glue_forward(x.data_ptr(), x.shape[0], x.shape[1], C.byref(glue), _stream(stream)))


def attention_decode(qkv: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, pos: torch.Tensor, n_heads: int,
                     n_kv_heads: int, head_dim: int, *, n_splits: int = 0, stream=None) -> torch.Tensor:
    """One new token per sequence over bf16 caches [B, n_kv_heads, max_seq, head_dim]: qkv [B, (n_heads + 2 n_kv_heads) *
    head_dim] holds q, k, v side by side; the new k and v are stored at position pos[b], which is not advanced."""
    qkv = _require(qkv, torch.float32, "qkv")
    B = qkv.shape[0]
    qd, kd = n_heads * head_dim, n_kv_heads * head_dim
    if qkv.shape[1] != qd + 2 * kd:
        raise IncompatibleShapes(f"qkv must be [B,{qd + 2 * kd}], got {list(qkv.shape)}")
    for name, t in (("k_cache", k_cache), ("v_cache", v_cache)):
        if t.dtype != torch.bfloat16 or not t.is_contiguous() or t.dim() != 4 or t.shape[0] < B or t.shape[1] != n_kv_heads or t.shape[3] != head_dim:
            raise IncompatibleShapes(f"{name} must be a contiguous bf16 tensor [>=B,{n_kv_heads},max_seq,{head_dim}]")
    if pos.dtype != torch.int32:
        raise UnsupportedDataType("pos must be int32")
    max_seq = k_cache.shape[2]
    if n_splits <= 0:
        n_splits = L.load().bitnet_attention_splits(B, n_kv_heads, max_seq)
    need = C.c_size_t()
    check(L.load().bitnet_attention_scratch_size(B, n_heads, n_kv_heads, head_dim, n_splits, C.byref(need)))
    key = ("attn", qkv.device.index or 0, _stream(stream), need.value)
    scratch = _workspaces.get(key)
    if scratch is None:
        scratch = torch.zeros(need.value + 256, dtype=torch.uint8, device=qkv.device)   # the arrival counters start at zero
        _workspaces[key] = scratch
    out = torch.empty((B, qd), dtype=torch.float32, device=qkv.device)
    check(L.load().bitnet_attention_decode(qkv.data_ptr(), qd + 2 * kd, qd, qd + kd, k_cache.data_ptr(), v_cache.data_ptr(),
                                           pos.data_ptr(), out.data_ptr(), B, n_heads, n_kv_heads, head_dim, max_seq, n_splits,
                                           _aligned_ptr(scratch), need.value, _stream(stream)))
    return out


def sample_tokens(logits: torch.Tensor, rng_state: torch.Tensor | None = None, *, temperature=1.0, top_k=0, top_p=1.0,
                  deterministic=False, stream=None) -> torch.Tensor:
    """TokenSampler::sample for every row of logits [B, vocab]; rng_state: int64 [B] generator states (updated)."""
    logits = _require(logits, torch.float32, "logits")
    B, V = logits.shape
    cfg = L.SamplingConfig(temperature, top_k, top_p, 0, 1 if deterministic else 0)
    out = torch.empty((B,), dtype=torch.int32, device=logits.device)
    check(L.load().bitnet_sample_tokens(logits.data_ptr(), B, V, C.byref(cfg), rng_state.data_ptr() if rng_state is not None else None,
                                        out.data_ptr(), _stream(stream)))
    return out


def quantize_pack_weights(w: torch.Tensor, stream=None):
    """absmean ternary quantisation of fp32 weights and 2-bit packing on the device (weights.rs:807-857,
    packing.rs:352-388); returns (packed uint8 [ceil(n/4)], scale as a Python float)."""
    w = _require(w, torch.float32, "w")
    n = w.numel()
    packed = torch.empty((packed_len(n),), dtype=torch.uint8, device=w.device)
    scale = torch.empty((1,), dtype=torch.float32, device=w.device)
    need = C.c_size_t()
    check(L.load().bitnet_quantize_pack_weights_workspace_size(n, C.byref(need)))
    ws = _workspace(need.value, w.device, stream)
    check(L.load().bitnet_quantize_pack_weights(w.data_ptr(), n, packed.data_ptr(), scale.data_ptr(), _aligned_ptr(ws), need.value,
                                                _stream(stream)))
    return packed, float(scale.item())
