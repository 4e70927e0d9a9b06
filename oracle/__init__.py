"""ctypes/numpy front end of the CPU oracle (``bitlinear_oracle.c``).

TEST INFRASTRUCTURE ONLY: the oracle checks the CUDA path; the product package
never imports this module.  Fused-path status: PARITY UNPINNED (see the header of
``bitlinear_oracle.h``); the layout, unpack, scalar GEMV/GEMM, rounding and ReLU^2
pieces are pinned by the reference's known-answer tests.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB = None

CODE3_ZERO, CODE3_PLUS1, CODE3_PLUS2 = 0, 1, 2


def build(native: bool = False) -> Path:
    """Compile the oracle with the Makefile next to this file and return the library path."""
    target = "liboracle_native.so" if native else "liboracle.so"
    subprocess.run(["make", "-C", str(_HERE), target], check=True, capture_output=True)
    return _HERE / target


def _load(path: Path):
    lib = C.CDLL(str(path))
    sz, f32, u64, i32 = C.c_size_t, C.c_float, C.c_uint64, C.c_int
    vp = C.c_void_p
    sig = {
        "orc_packed_len": (sz, [sz]),
        "orc_pack_bits": (None, [vp, sz, C.c_uint, vp]),
        "orc_unpack_bits": (None, [vp, sz, C.c_uint, sz, vp]),
        "orc_pack_ternary": (None, [vp, sz, vp, C.POINTER(sz)]),
        "orc_unpack_ternary": (None, [vp, sz, vp, i32]),
        "orc_round_half_away": (f32, [f32]),
        "orc_round_clip": (f32, [f32, f32, f32]),
        "orc_relu2": (None, [vp, vp, sz]),
        "orc_ternary_gemv_f32": (None, [vp, vp, vp, sz, sz, f32]),
        "orc_ternary_gemm_f32": (None, [vp, vp, vp, sz, sz, sz, f32]),
        "orc_quantize_activations": (None, [vp, sz, sz, vp, vp, vp]),
        "orc_contract_i32": (None, [vp, vp, vp, sz, sz, sz]),
        "orc_dequantize": (None, [vp, vp, f32, vp, sz, sz]),
        "orc_bitlinear_forward": (None, [vp, f32, vp, sz, sz, sz, vp, vp, vp, vp]),
        "orc_bitlinear_forward_float_order": (None, [vp, f32, vp, sz, sz, sz, vp]),
        "orc_w2a8_gemv": (None, [vp, vp, vp, sz, sz]),
        "orc_gate_relu2": (None, [vp, vp, vp, sz]),
        "orc_ffn_forward": (None, [vp, f32, vp, f32, vp, f32, vp, sz, sz, sz, vp, vp]),
        "orc_absmean_quantize_weights": (f32, [vp, sz, vp]),
        "orc_max_threads": (i32, []),
        "orc_bitlinear_forward_mt": (None, [vp, f32, vp, sz, sz, sz, vp, i32]),
        "orc_splitmix64": (u64, [u64]),
        "orc_gen_ternary": (None, [u64, u64, sz, vp]),
        "orc_gen_ternary_packed": (None, [u64, u64, sz, vp]),
        "orc_gen_activations": (None, [u64, u64, sz, vp]),
        "orc_gen_weight_scale": (f32, [u64, u64, sz]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    return lib


def lib(native: bool = False):
    """The loaded oracle library; built on first use if the .so is absent."""
    global _LIB
    if native:
        path = _HERE / "liboracle_native.so"
        if not path.exists():
            build(native=True)
        return _load(path)
    if _LIB is None:
        path = _HERE / "liboracle.so"
        src_mtime = max((_HERE / n).stat().st_mtime for n in ("bitlinear_oracle.c", "bitlinear_oracle.h"))
        if not path.exists() or (path.stat().st_mtime < src_mtime and os.access(_HERE, os.W_OK)):
            build()
        _LIB = _load(path)
    return _LIB


def _p(a: np.ndarray | None):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dtype) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


# --- layout -----------------------------------------------------------------

def pack_ternary(w) -> tuple[np.ndarray, int]:
    """Row-major flattening of ``w`` ({-1,0,1}) -> packed bytes and the padding count."""
    w = _c(w, np.int8).reshape(-1)
    out = np.zeros((w.size + 3) // 4, dtype=np.uint8)
    pad = C.c_size_t(0)
    lib().orc_pack_ternary(_p(w), w.size, _p(out), C.byref(pad))
    return out, int(pad.value)


def unpack_ternary(packed, n_values: int, code3: int = CODE3_ZERO) -> np.ndarray:
    packed = _c(packed, np.uint8).reshape(-1)
    assert packed.size * 4 >= n_values
    out = np.empty(n_values, dtype=np.int8)
    lib().orc_unpack_ternary(_p(packed), n_values, _p(out), code3)
    return out


def pack_bits(values, bits: int) -> np.ndarray:
    values = _c(values, np.uint8).reshape(-1)
    per = 8 // bits if bits < 8 else 1
    out = np.zeros((values.size + per - 1) // per, dtype=np.uint8)
    lib().orc_pack_bits(_p(values), values.size, bits, _p(out))
    return out


def unpack_bits(packed, bits: int, n_values: int) -> np.ndarray:
    packed = _c(packed, np.uint8).reshape(-1)
    out = np.zeros(n_values, dtype=np.uint8)
    lib().orc_unpack_bits(_p(packed), packed.size, bits, n_values, _p(out))
    return out


# --- scalar pieces -----------------------------------------------------------

def round_clip(x: float, lo: float, hi: float) -> float:
    return float(lib().orc_round_clip(x, lo, hi))


def relu2(x) -> np.ndarray:
    x = _c(x, np.float32)
    y = np.empty_like(x)
    lib().orc_relu2(_p(x), _p(y), x.size)
    return y


def ternary_gemv_f32(a, x, scale: float = 1.0) -> np.ndarray:
    a = _c(a, np.int8)
    x = _c(x, np.float32)
    m, k = a.shape
    y = np.empty(m, dtype=np.float32)
    lib().orc_ternary_gemv_f32(_p(a), _p(x), _p(y), m, k, scale)
    return y


def ternary_gemm_f32(a, b, scale: float = 1.0) -> np.ndarray:
    a = _c(a, np.int8)
    b = _c(b, np.float32)
    m, k = a.shape
    n = b.shape[1]
    c = np.empty((m, n), dtype=np.float32)
    lib().orc_ternary_gemm_f32(_p(a), _p(b), _p(c), m, k, n, scale)
    return c


# --- the fused path ------------------------------------------------------------

def quantize_activations(x):
    """x [M,K] fp32 -> (q int8 [M,K], a_scale fp32 [M], fake-quantised fp32 [M,K])."""
    x = _c(x, np.float32)
    M, K = x.shape
    q = np.empty((M, K), dtype=np.int8)
    s = np.empty(M, dtype=np.float32)
    fq = np.empty((M, K), dtype=np.float32)
    lib().orc_quantize_activations(_p(x), M, K, _p(q), _p(s), _p(fq))
    return q, s, fq


def bitlinear_forward(wp, w_scale: float, x, N: int):
    """Packed weights + fp32 x [M,K] -> dict(y fp32 [M,N], q int8, a_scale, acc int32 [M,N])."""
    wp = _c(wp, np.uint8).reshape(-1)
    x = _c(x, np.float32)
    M, K = x.shape
    assert wp.size == (N * K + 3) // 4
    y = np.empty((M, N), dtype=np.float32)
    q = np.empty((M, K), dtype=np.int8)
    s = np.empty(M, dtype=np.float32)
    acc = np.empty((M, N), dtype=np.int32)
    lib().orc_bitlinear_forward(_p(wp), w_scale, _p(x), M, K, N, _p(y), _p(q), _p(s), _p(acc))
    return {"y": y, "q": q, "a_scale": s, "acc": acc}


def bitlinear_forward_float_order(wp, w_scale: float, x, N: int) -> np.ndarray:
    wp = _c(wp, np.uint8).reshape(-1)
    x = _c(x, np.float32)
    M, K = x.shape
    y = np.empty((M, N), dtype=np.float32)
    lib().orc_bitlinear_forward_float_order(_p(wp), w_scale, _p(x), M, K, N, _p(y))
    return y


def w2a8_gemv(wp, a, n_out: int) -> np.ndarray:
    wp = _c(wp, np.uint8).reshape(-1)
    a = _c(a, np.int8).reshape(-1)
    out = np.empty(n_out, dtype=np.int32)
    lib().orc_w2a8_gemv(_p(wp), _p(a), _p(out), n_out, a.size)
    return out


def ffn_forward(wp_gate, s_gate, wp_up, s_up, wp_down, s_down, x, ffn: int):
    """FFN block: returns (y [M,hidden], h [M,ffn])."""
    x = _c(x, np.float32)
    M, hidden = x.shape
    y = np.empty((M, hidden), dtype=np.float32)
    h = np.empty((M, ffn), dtype=np.float32)
    lib().orc_ffn_forward(_p(_c(wp_gate, np.uint8)), s_gate, _p(_c(wp_up, np.uint8)), s_up,
                          _p(_c(wp_down, np.uint8)), s_down, _p(x), M, hidden, ffn, _p(y), _p(h))
    return y, h


def absmean_quantize_weights(w):
    w = _c(w, np.float32)
    t = np.empty(w.shape, dtype=np.int8)
    scale = lib().orc_absmean_quantize_weights(_p(w), w.size, _p(t))
    return t, float(scale)


def bitlinear_forward_mt(wp, w_scale: float, x, N: int, threads: int, native: bool = False) -> np.ndarray:
    wp = _c(wp, np.uint8).reshape(-1)
    x = _c(x, np.float32)
    M, K = x.shape
    y = np.empty((M, N), dtype=np.float32)
    lib(native).orc_bitlinear_forward_mt(_p(wp), w_scale, _p(x), M, K, N, _p(y), threads)
    return y


def max_threads() -> int:
    return int(lib().orc_max_threads())


# --- seeded synthetic inputs -----------------------------------------------------

def gen_ternary(seed: int, tensor_id: int, n: int) -> np.ndarray:
    w = np.empty(n, dtype=np.int8)
    lib().orc_gen_ternary(seed, tensor_id, n, _p(w))
    return w


def gen_ternary_packed(seed: int, tensor_id: int, n: int) -> np.ndarray:
    out = np.empty((n + 3) // 4, dtype=np.uint8)
    lib().orc_gen_ternary_packed(seed, tensor_id, n, _p(out))
    return out


def gen_activations(seed: int, tensor_id: int, shape) -> np.ndarray:
    x = np.empty(shape, dtype=np.float32)
    lib().orc_gen_activations(seed, tensor_id, x.size, _p(x))
    return x


def gen_weight_scale(seed: int, tensor_id: int, K: int) -> float:
    return float(lib().orc_gen_weight_scale(seed, tensor_id, K))
