"""The allocation-free entry point, bitnet_bitlinear_forward_static, against the regular one.

It serves callers that cannot allocate device memory or pass a workspace (a fixed memory
budget, a host that forbids allocation calls at that moment): its scratch is an array built
into the library.  The test calls it through the C ABI twice in a row with different shapes,
so that the second call meets the first call's leftovers in the shared array, and compares
each output with bitnet_bitlinear_forward on the same inputs and with the CPU oracle (bit for bit,
which is inside the 1e-5 relative tolerance the other parity tests use).  The shapes include
layers wide and ragged enough (many 16-row blocks per CTA, a K that does not divide evenly over
the warps) to reach the kernel plans that keep activations in registers and let the weight ring
grow over the staging area, where stale bytes of the shared array would show if anything read
them.  This file sorts last on purpose."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from bitnet_mlx_rs_b200 import _lib as L
from bitnet_mlx_rs_b200 import cuda, ops

pytestmark = pytest.mark.gpu


def test_static_scratch_forward_matches_regular_entry_point_twice():
    lib = L.load()
    stream = torch.cuda.current_stream().cuda_stream
    shapes = [(8, 6912, 2560), (3, 2560, 700), (1, 2560, 6912), (16, 1024, 144),
              (8, 7168, 16384), (1, 7168, 16384), (3, 8128, 16384), (8, 6912, 14400), (2, 64, 32)]
    for seed, (M, K, N) in enumerate(shapes):
        wp_h = oracle.gen_ternary_packed(40 + seed, 1, N * K)
        x_h = oracle.gen_activations(40 + seed, 2, (M, K))
        wp, x = torch.from_numpy(wp_h).cuda(), torch.from_numpy(x_h).cuda()
        ws = oracle.gen_weight_scale(40 + seed, 1, K)
        y_static = torch.full((M, N), float("nan"), device="cuda")
        cuda.check(lib.bitnet_bitlinear_forward_static(wp.data_ptr(), ws, x.data_ptr(), y_static.data_ptr(), M, K, N, stream))
        y_regular = ops.bitlinear_forward(wp, ws, x, N)
        torch.cuda.synchronize()
        np.testing.assert_allclose(y_static.cpu().numpy(), y_regular.cpu().numpy(), rtol=1e-5, atol=0)
        assert torch.equal(y_static, y_regular)
        ref = oracle.bitlinear_forward_mt(wp_h, ws, x_h, N, 8)
        np.testing.assert_allclose(y_static.cpu().numpy(), ref, rtol=1e-5, atol=0)
        assert np.array_equal(y_static.cpu().numpy(), ref)
    assert ops.device_error_flags() == 0


def test_static_scratch_forward_refuses_what_it_cannot_hold():
    lib = L.load()
    one = torch.zeros(16, dtype=torch.uint8, device="cuda").data_ptr()
    assert lib.bitnet_bitlinear_forward_static(one, 1.0, one, one, 17, 2560, 64, None) == L.ERR_UNSUPPORTED_OPERATION
    assert lib.bitnet_bitlinear_forward_static(one, 1.0, one, one, 4, 100, 64, None) == L.ERR_UNSUPPORTED_OPERATION
    assert b"decode shapes" in lib.bitnet_last_error_string()
    assert lib.bitnet_bitlinear_forward_static(None, 1.0, one, one, 4, 128, 64, None) == L.ERR_NULL_POINTER
    assert lib.bitnet_bitlinear_forward_static(one, 1.0, one, one, 0, 128, 64, None) == L.OK
