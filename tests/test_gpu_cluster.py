"""Parity of the cluster split-K tensor-core path (a few dozen tokens) with the CPU oracle, through the C ABI.
int8 activations, scales and int32 accumulators bit-exact; fp32 outputs within 1e-5 relative (bit-identical)."""
import numpy as np
import pytest
import torch

import oracle
from oracle import decoder as od
from bitnet_mlx_rs_b200 import ops

pytestmark = pytest.mark.gpu
RTOL = 1e-5


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def case(seed, M, K, N):
    return oracle.gen_ternary_packed(seed, 1, N * K), oracle.gen_weight_scale(seed, 1, K), oracle.gen_activations(seed, 2, (M, K))


SHAPES = [(17, 2560, 2560), (32, 2560, 640), (64, 2560, 2560), (128, 2560, 640), (64, 6912, 2560), (40, 2560, 6912),
          (20, 128, 8), (33, 384, 700), (1, 256, 130), (100, 1024, 513), (64, 2560, 3000), (16, 8192, 1024), (128, 8192, 256), (48, 12288, 300)]


@pytest.mark.parametrize("M,K,N", SHAPES)
def test_cluster_path_matches_oracle(M, K, N):
    wp, ws, x = case(700 + M + N, M, K, N)
    ref = oracle.bitlinear_forward(wp, ws, x, N)
    for _ in range(2):
        y, dbg = ops.bitlinear_forward(dev(wp), ws, dev(x), N, debug=True, path="cluster")
    assert ops.device_error_flags() == 0
    assert np.array_equal(dbg["q"].cpu().numpy(), ref["q"])
    assert np.array_equal(dbg["a_scale"].cpu().numpy(), ref["a_scale"])
    assert np.array_equal(dbg["acc"].cpu().numpy(), ref["acc"])
    np.testing.assert_allclose(y.cpu().numpy(), ref["y"], rtol=RTOL, atol=0)
    assert np.array_equal(y.cpu().numpy(), ref["y"])


def test_what_the_cluster_path_cannot_hold_goes_to_the_persistent_gemm():
    # 128 tokens x K = 16384: eight CTAs cannot hold a K slice each in shared and tensor memory
    M, K, N = 128, 16384, 256
    wp, ws, x = case(3, M, K, N)
    with pytest.raises(Exception):
        ops.bitlinear_forward(dev(wp), ws, dev(x), N, path="cluster")
    y = ops.bitlinear_forward(dev(wp), ws, dev(x), N)
    assert np.array_equal(y.cpu().numpy(), oracle.bitlinear_forward(wp, ws, x, N)["y"])


@pytest.mark.parametrize("M", [17, 64, 128])
def test_auto_dispatch_takes_the_cluster_path_between_the_other_two(M):
    K, N = 2560, 2560
    wp, ws, x = case(40 + M, M, K, N)
    y = ops.bitlinear_forward(dev(wp), ws, dev(x), N)
    assert np.array_equal(y.cpu().numpy(), oracle.bitlinear_forward(wp, ws, x, N)["y"])
    # and agrees with the persistent GEMM bit for bit
    assert torch.equal(y, ops.bitlinear_forward(dev(wp), ws, dev(x), N, path="prefill"))


@pytest.mark.parametrize("M", [24, 64])
def test_cluster_stack_and_glue(M):
    K, rows = 2560, (2560, 640, 640)
    x, r = oracle.gen_activations(5, 1, (M, K)), oracle.gen_activations(5, 2, (M, K))
    rng = np.random.default_rng(3)
    w, b = (1.0 + 0.1 * rng.standard_normal(K)).astype(np.float32), (0.05 * rng.standard_normal(K)).astype(np.float32)
    packs = [oracle.gen_ternary_packed(5, 10 + i, n * K) for i, n in enumerate(rows)]
    scales = [oracle.gen_weight_scale(5, 10 + i, K) for i in range(3)]
    xs, normed = dev(x), torch.empty(M, K, device="cuda")
    glue = ops.make_glue(dev(r), xs, dev(w), dev(b), 1e-5, normed)
    y, dbg = ops.bitlinear_forward_fused(dev(np.concatenate(packs)), rows, scales, xs, glue=glue, path="cluster", debug=True)
    assert ops.device_error_flags() == 0
    assert np.array_equal(xs.cpu().numpy(), x + r)
    n_gpu = normed.cpu().numpy()
    np.testing.assert_allclose(n_gpu, od.subln(x + r, w, b, 1e-5), rtol=1e-5, atol=2e-6)
    col = 0
    for pk, sc, n in zip(packs, scales, rows):
        ref = oracle.bitlinear_forward(pk, sc, n_gpu, n)
        assert np.array_equal(dbg["q"].cpu().numpy(), ref["q"])
        assert np.array_equal(dbg["acc"][:, col:col + n].cpu().numpy(), ref["acc"])
        assert np.array_equal(y[:, col:col + n].cpu().numpy(), ref["y"])
        col += n


@pytest.mark.parametrize("M,H,F", [(64, 2560, 6912), (32, 2560, 6912), (20, 256, 640), (128, 1024, 384)])
def test_cluster_ffn_pair(M, H, F):
    g, u, d = (oracle.gen_ternary_packed(6, i, F * H) for i in (1, 2, 3))
    sg, su, sd = (oracle.gen_weight_scale(6, i, k) for i, k in ((1, H), (2, H), (3, F)))
    x = oracle.gen_activations(6, 4, (M, H))
    ry, rh = oracle.ffn_forward(g, sg, u, su, d, sd, x, F)
    y, h = ops.ffn_forward(dev(g), sg, dev(u), su, dev(d), sd, dev(x), F)
    assert ops.device_error_flags() == 0
    assert np.array_equal(h.cpu().numpy(), rh)
    assert np.array_equal(y.cpu().numpy(), ry)
    y2, _ = ops.ffn_forward(dev(g), sg, dev(u), su, dev(d), sd, dev(x), F, path="cluster", pdl=True)
    assert np.array_equal(y2.cpu().numpy(), ry)
