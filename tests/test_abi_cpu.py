"""CPU-only checks: the C-ABI library loads and exports every symbol the header declares,
its GPU-free entry points behave, the host-side mirror's logic is right, and the committed
golden fixtures agree with the oracle."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

import oracle
from bitnet_mlx_rs_b200 import _lib as L
from bitnet_mlx_rs_b200 import cuda
from bitnet_mlx_rs_b200.bitlinear import absmean_quantize_weights

ROOT = Path(__file__).resolve().parents[1]
GOLDEN = ROOT / "tests" / "golden"


def declared_functions():
    names = []
    for h in (ROOT / "include").glob("*.h"):
        text = re.sub(r"/\*.*?\*/", "", h.read_text(), flags=re.S)
        names += re.findall(r"\b(bitnet_\w+|launch_w2a8_gemv_optimized)\s*\(", text)
    return sorted(set(names))


def test_library_exports_every_declared_symbol():
    lib = L.load()
    names = declared_functions()
    assert len(names) >= 30
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/ but not exported"
    # and the ctypes table covers exactly the header
    assert set(L.SIGNATURES) == set(names)


def test_status_strings_and_recoverability():
    lib = L.load()
    assert lib.bitnet_status_string(0) == b"ok"
    # bitnet-cuda/src/error.rs:88-103
    rec = {L.ERR_MEMORY_ALLOCATION, L.ERR_KERNEL_EXECUTION, L.ERR_STREAM_SYNC, L.ERR_PERFORMANCE, L.ERR_CUDA_DRIVER}
    non = {L.ERR_CUDA_NOT_ENABLED, L.ERR_DEVICE, L.ERR_INVALID_CONFIG, L.ERR_UNSUPPORTED_OPERATION,
           L.ERR_UNSUPPORTED_DTYPE, L.ERR_INCOMPATIBLE_SHAPES}
    for s in rec:
        assert lib.bitnet_is_recoverable(s) == 1
    for s in non:
        assert lib.bitnet_is_recoverable(s) == 0
    assert cuda.IncompatibleShapes("x").is_recoverable() is False
    assert cuda.MemoryAllocation("x").is_recoverable() is True


def test_config_defaults_match_reference():
    cfg = L.BackendConfig()
    L.load().bitnet_backend_config_default(C.byref(cfg))
    # bitnet-cuda/src/backend.rs:27-37 and kernels/w2a8_gemv.rs:28-38
    assert (cfg.device_id, cfg.memory_pool_size, cfg.num_streams, cfg.enable_profiling) == (0, 1 << 30, 4, 0)
    w = cfg.w2a8_config
    assert (w.block_size, w.grid_strategy, w.enable_weight_permutation, w.enable_dp4a, w.coalescing_level) == \
        (256, 1, 1, 1, 2)
    d = cuda.CudaBackendConfig()
    assert (d.device_id, d.memory_pool_size, d.num_streams) == (0, 1 << 30, 4)
    assert cuda.MEMORY_BANDWIDTH_TARGET == 85.0 and cuda.W2A8_SPEEDUP_MAX == 3.63


def test_argument_errors_need_no_gpu():
    lib = L.load()
    assert lib.bitnet_bitlinear_forward(None, 1.0, None, None, 4, 64, 64, None, None, 0, None) == L.ERR_NULL_POINTER
    assert b"null" in lib.bitnet_last_error_string()
    assert lib.bitnet_bitlinear_forward(None, 1.0, None, None, 0, 64, 64, None, None, 0, None) == L.OK   # empty batch
    assert lib.bitnet_w2a8_gemv(None, None, None, 0, 64, None) == L.OK
    assert lib.bitnet_w2a8_gemv(None, None, None, 8, 64, None) == L.ERR_NULL_POINTER
    assert lib.bitnet_w2a8_gemv(1, 1, 1, 8, 0, None) == L.ERR_INCOMPATIBLE_SHAPES
    assert lib.bitnet_quantize_activations(1, 2, 0, 1, 1, None) == L.ERR_INCOMPATIBLE_SHAPES
    n = C.c_size_t(123)
    # decode path: room for the once-quantised activations (int8, fragment order) of 8 tokens
    assert lib.bitnet_bitlinear_workspace_size(8, 2560, 6912, L.PATH_AUTO, C.byref(n)) == L.OK
    assert 8 * 2560 <= n.value <= 64 * 1024 and n.value % 256 == 0
    assert lib.bitnet_bitlinear_workspace_size(3, 37, 29, L.PATH_AUTO, C.byref(n)) == L.OK and n.value >= 3 * 37 + 12
    assert lib.bitnet_bitlinear_workspace_size(8, 64, 64, 99, C.byref(n)) == L.ERR_INVALID_CONFIG
    with pytest.raises(cuda.NullPointer):
        cuda.check(L.ERR_NULL_POINTER)


def test_backend_without_gpu_reports_cuda_not_enabled():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    assert cuda.is_cuda_available() is False
    with pytest.raises(cuda.CudaNotEnabled):
        cuda.CudaBackend()


def test_host_absmean_quantiser_matches_oracle():
    rng = np.random.default_rng(1)
    w = rng.standard_normal((96, 160)).astype(np.float32)
    qw = absmean_quantize_weights(w)
    t, scale = oracle.absmean_quantize_weights(w)
    assert np.array_equal(qw.values, t)
    assert qw.scale == pytest.approx(scale, rel=1e-6)
    assert absmean_quantize_weights(np.zeros((4, 4), np.float32)).scale == 1.0   # weights.rs:554-556


@pytest.mark.parametrize("path", sorted(GOLDEN.glob("*.npz")), ids=lambda p: p.stem)
def test_oracle_reproduces_golden_fixtures(path):
    z = np.load(path)
    if "gate" in z:
        y, h = oracle.ffn_forward(z["gate"], float(z["s_gate"]), z["up"], float(z["s_up"]), z["down"],
                                  float(z["s_down"]), z["x"], int(z["ffn"]))
        assert np.array_equal(y, z["y"]) and np.array_equal(h, z["h"])
        return
    ref = oracle.bitlinear_forward(z["wp"], float(z["w_scale"]), z["x"], int(z["N"]))
    for key in ("q", "acc", "a_scale", "y"):
        assert np.array_equal(ref[key], z[key]), key
