"""Parity of the CUDA path with the CPU oracle, called through the C ABI.

Bar: int8 activations, per-token scales and int32 accumulators bit-exact; fp32 outputs
within 1e-5 relative (they are in fact bit-identical, which is also asserted where the
path promises it)."""
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle
from bitnet_mlx_rs_b200 import cuda, ops
from bitnet_mlx_rs_b200.bitlinear import BitLinear, BitLinearConfig, BitLinearLayer, FeedForwardNetwork, ShapeMismatch

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"
RTOL = 1e-5


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def case(seed, M, K, N):
    wp = oracle.gen_ternary_packed(seed, 1, N * K)
    x = oracle.gen_activations(seed, 2, (M, K))
    ws = oracle.gen_weight_scale(seed, 1, K)
    return wp, ws, x


def assert_parity(dbg, y, ref, M, N):
    assert np.array_equal(dbg["q"].cpu().numpy(), ref["q"]), "int8 activations differ"
    assert np.array_equal(dbg["a_scale"].cpu().numpy(), ref["a_scale"]), "activation scales differ"
    assert np.array_equal(dbg["acc"].cpu().numpy(), ref["acc"]), "int32 accumulators differ"
    yn = y.cpu().numpy()
    assert yn.shape == (M, N)
    np.testing.assert_allclose(yn, ref["y"], rtol=RTOL, atol=0)
    assert np.array_equal(yn, ref["y"]), "fp32 outputs are expected to be bit-identical"


# ---- activation quantiser -------------------------------------------------------------------

@pytest.mark.parametrize("M,K", [(1, 2560), (8, 6912), (3, 37), (5, 1), (2, 8192), (33, 130)])
def test_quantize_activations_bit_exact(M, K):
    x = oracle.gen_activations(1, 5, (M, K))
    q, s = ops.quantize_activations(dev(x))
    rq, rs, _ = oracle.quantize_activations(x)
    assert np.array_equal(q.cpu().numpy(), rq)
    assert np.array_equal(s.cpu().numpy(), rs)


def test_quantiser_rounding_ties_and_edges():
    # scale == 1 when absmax == 127: the quantiser then rounds the inputs themselves
    vals = [127.0]
    for n in range(-127, 127):
        h = np.float32(n) + np.float32(0.5)
        vals += [h, np.nextafter(h, np.float32(200)), np.nextafter(h, np.float32(-200))]
    vals += [0.49999997, -0.49999997, 0.0, -0.0, 1e-30, -1e-30]
    x = np.zeros((4, 1024), dtype=np.float32)
    x[0, : len(vals)] = vals
    x[1, :] = 0.0                                        # all-zero row: scale 1, a_scale 1
    x[2, :8] = [3.0e38, -3.0e38, 1.0, -1.0, 0.0, 1e20, -1e20, 5.0]
    x[3, 7] = 1e-38                                      # subnormal-range absmax
    q, s = ops.quantize_activations(dev(x))
    rq, rs, _ = oracle.quantize_activations(x)
    assert np.array_equal(q.cpu().numpy(), rq)
    assert np.array_equal(s.cpu().numpy(), rs)
    # and the same rows through the fused decode kernel
    wp, ws, _ = case(2, 4, 1024, 32)
    y, dbg = ops.bitlinear_forward(dev(wp), ws, dev(x), 32, debug=True, path="decode")
    assert_parity(dbg, y, oracle.bitlinear_forward(wp, ws, x, 32), 4, 32)


# ---- decode kernel ----------------------------------------------------------------------------

DECODE_SHAPES = [
    (1, 2560, 2560),      # config 1
    (1, 2560, 6912), (4, 2560, 6912), (8, 2560, 6912),      # config 2 gate/up
    (1, 6912, 2560), (4, 6912, 2560), (8, 6912, 2560),      # config 2 down
    (1, 64, 16), (2, 64, 1), (7, 128, 17), (8, 192, 250), (3, 320, 129),   # tails in N and few chunks
    (9, 256, 48), (16, 1024, 144), (13, 2560, 640),         # two token tiles
    (1, 8192, 3584), (16, 8192, 3584),                      # one 8-GPU slice of the oversized layer
]


@pytest.mark.parametrize("M,K,N", DECODE_SHAPES)
def test_decode_matches_oracle(M, K, N):
    wp, ws, x = case(100 + M, M, K, N)
    ref = oracle.bitlinear_forward(wp, ws, x, N)
    y, dbg = ops.bitlinear_forward(dev(wp), ws, dev(x), N, debug=True, path="decode")
    assert_parity(dbg, y, ref, M, N)


@pytest.mark.parametrize("stages", [1, 2, 3, 8])
@pytest.mark.parametrize("M,K,N", [(1, 2560, 6912), (8, 6912, 5200), (5, 512, 10400), (12, 1536, 7000), (8, 64, 4000),
                                   (2, 16384, 2400)])
def test_decode_every_ring_depth(stages, M, K, N):
    # several blocks per CTA, so that stages are reused and the ring wraps
    wp, ws, x = case(7 * stages + M, M, K, N)
    ref = oracle.bitlinear_forward(wp, ws, x, N)
    y, dbg = ops.bitlinear_forward(dev(wp), ws, dev(x), N, debug=True, path="decode", stages=stages)
    assert_parity(dbg, y, ref, M, N)
    assert ops.device_error_flags() == 0


@pytest.mark.parametrize("M,K,N", [(1, 7168, 16384), (8, 6912, 12000), (8, 7168, 16384), (3, 8128, 16384), (5, 7168, 14336),
                                   (1, 6912, 16000)])
def test_decode_ragged_k_slices_with_the_ring_over_the_staging_area(M, K, N):
    # Many blocks per CTA and a K that leaves some warps fewer chunks than their loop covers: the
    # plans that keep activations in registers let the weight ring grow over the staging area, and
    # the chunks past a warp's slice must still read zeros as weights.  The scratch buffer is filled
    # with 0xFF first, and a call of another shape runs before, so that stale bytes would show.
    wp, ws, x = case(400 + M + K // 64, M, K, N)
    ref = oracle.bitlinear_forward(wp, ws, x, N)
    dwp, dx = dev(wp), dev(x)
    ops.bitlinear_forward(dev(oracle.gen_ternary_packed(5, 5, 3000 * 1024)), 0.1, torch.full((16, 1024), 127.0, device="cuda"), 3000)
    for ws_buf in ops._workspaces.values():
        ws_buf.fill_(0xFF)
    for _ in range(2):
        y, dbg = ops.bitlinear_forward(dwp, ws, dx, N, debug=True, path="decode")
        assert_parity(dbg, y, ref, M, N)
    assert ops.device_error_flags() == 0


def test_decode_with_programmatic_dependent_launch_chain():
    # y1 = L1(x); y2 = L2(y1): the second launch may start before the first ends and must still see y1
    M, K, N = 8, 2560, 2560
    wp1, s1, x = case(31, M, K, N)
    wp2, s2, _ = case(32, M, N, K)
    d1, d2, dx = dev(wp1), dev(wp2), dev(x)
    for _ in range(3):
        y1 = ops.bitlinear_forward(d1, s1, dx, N, path="decode", pdl=True)
        y2 = ops.bitlinear_forward(d2, s2, y1, K, path="decode", pdl=True)
    r1 = oracle.bitlinear_forward(wp1, s1, x, N)["y"]
    r2 = oracle.bitlinear_forward(wp2, s2, r1, K)["y"]
    assert np.array_equal(y1.cpu().numpy(), r1)
    assert np.array_equal(y2.cpu().numpy(), r2)


@pytest.mark.parametrize("path", sorted(GOLDEN.glob("*.npz")), ids=lambda p: p.stem)
def test_golden_fixtures(path):
    z = np.load(path)
    if "gate" in z:
        y, h = ops.ffn_forward(dev(z["gate"]), float(z["s_gate"]), dev(z["up"]), float(z["s_up"]), dev(z["down"]),
                               float(z["s_down"]), dev(z["x"]), int(z["ffn"]))
        assert np.array_equal(h.cpu().numpy(), z["h"])
        np.testing.assert_allclose(y.cpu().numpy(), z["y"], rtol=RTOL, atol=0)
        return
    M, N = int(z["M"]), int(z["N"])
    y, dbg = ops.bitlinear_forward(dev(z["wp"]), float(z["w_scale"]), dev(z["x"]), N, debug=True)
    assert_parity(dbg, y, {k: z[k] for k in ("q", "a_scale", "acc", "y")}, M, N)


# ---- generic path: any shape, rows that start mid-byte ---------------------------------------------

@pytest.mark.parametrize("M,K,N", [(3, 37, 29), (1, 1, 1), (2, 5, 3), (20, 130, 33), (4, 2562, 10), (40, 64, 16)])
def test_generic_path_matches_oracle(M, K, N):
    wp, ws, x = case(200 + K, M, K, N)
    ref = oracle.bitlinear_forward(wp, ws, x, N)
    y, dbg = ops.bitlinear_forward(dev(wp), ws, dev(x), N, debug=True, path="generic")
    assert_parity(dbg, y, ref, M, N)
    y2 = ops.bitlinear_forward(dev(wp), ws, dev(x), N)          # auto dispatch lands on a correct kernel too
    assert np.array_equal(y2.cpu().numpy(), ref["y"])


def test_empty_batch_is_a_no_op():
    wp, ws, _ = case(1, 1, 64, 16)
    y = ops.bitlinear_forward(dev(wp), ws, torch.empty((0, 64), device="cuda"), 16)
    assert tuple(y.shape) == (0, 16)


# ---- legacy single-token GEMV -------------------------------------------------------------------------

@pytest.mark.parametrize("n_out,k", [(128, 512), (512, 2048), (2048, 8192), (2560, 2560), (3, 4), (17, 36), (100, 250)])
def test_w2a8_gemv_matches_oracle(n_out, k):
    # sizes of bitnet-cuda/examples/w2a8_gemv_demo.rs:45-51 plus ragged ones
    wp = oracle.gen_ternary_packed(5, n_out, n_out * k)
    a = np.random.default_rng(k).integers(-127, 128, size=k, dtype=np.int8)
    out = ops.w2a8_gemv(dev(wp), dev(a), n_out)
    assert np.array_equal(out.cpu().numpy(), oracle.w2a8_gemv(wp, a, n_out))


def test_w2a8_gemv_reference_pins():
    # bitnet-quant/src/simd/matrix.rs:531-558 through the packed integer path
    a = np.array([[1, -1, 0, 1], [0, 1, -1, 0], [-1, 0, 1, 1]], dtype=np.int8)
    packed, _ = oracle.pack_ternary(a)
    out = ops.w2a8_gemv(dev(packed), dev(np.array([2, 3, 1, -1], dtype=np.int8)), 3)
    assert out.cpu().tolist() == [-2, 2, -2]
    # bitnet-cuda/examples/w2a8_gemv_demo.rs:59-61: all codes 1 => all weights 0 => output 0
    n_out, k = 512, 2048
    wp = np.full(n_out * k // 4, 0x55, dtype=np.uint8)
    out = ops.w2a8_gemv(dev(wp), dev(np.ones(k, dtype=np.int8)), n_out)
    assert not out.any().item()


# ---- layout helpers ---------------------------------------------------------------------------------------

def test_pack_unpack_sanitize_on_device():
    for n in (3, 8, 32, 128 * 64 + 1):
        w = (np.arange(n) % 3 - 1).astype(np.int8)          # simd_unpacking_correctness_tests.rs:101-133
        packed = ops.pack_ternary(dev(w))
        assert np.array_equal(packed.cpu().numpy(), oracle.pack_ternary(w)[0])
        assert np.array_equal(ops.unpack_ternary(packed, n).cpu().numpy(), w)
    assert ops.unpack_ternary(dev(np.array([0b00100100], np.uint8)), 4).cpu().tolist() == [-1, 0, 1, -1]   # gguf.rs:2421
    assert ops.unpack_ternary(dev(np.array([0b11100100], np.uint8)), 4).cpu().tolist() == [-1, 0, 1, 0]    # weight_conversion.rs:478
    p = dev(np.array([0b11100100, 0xFF, 0x55, 0x00], np.uint8))
    assert ops.sanitize_packed(p) == 5
    assert p.cpu().tolist() == [0b01100100, 0x55, 0x55, 0x00]
    assert ops.sanitize_packed(p) == 0


# ---- FFN block ------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("M", [1, 4, 8])
def test_ffn_block_config2(M):
    H, F = 2560, 6912
    g, u, d = (oracle.gen_ternary_packed(9, i, F * H) for i in (1, 2, 3))
    sg, su, sd = (oracle.gen_weight_scale(9, i, k) for i, k in ((1, H), (2, H), (3, F)))
    x = oracle.gen_activations(9, 4, (M, H))
    ry, rh = oracle.ffn_forward(g, sg, u, su, d, sd, x, F)
    y, h = ops.ffn_forward(dev(g), sg, dev(u), su, dev(d), sd, dev(x), F)
    assert np.array_equal(h.cpu().numpy(), rh)
    np.testing.assert_allclose(y.cpu().numpy(), ry, rtol=RTOL, atol=0)
    assert np.array_equal(y.cpu().numpy(), ry)
    y2, _ = ops.ffn_forward(dev(g), sg, dev(u), su, dev(d), sd, dev(x), F, pdl=True)
    assert np.array_equal(y2.cpu().numpy(), ry)


def test_ffn_generic_path_small():
    M, H, F = 20, 96, 160
    g, u, d = (oracle.gen_ternary_packed(8, i, F * H) for i in (1, 2, 3))
    sg, su, sd = 0.1, 0.2, 0.3
    x = oracle.gen_activations(8, 4, (M, H))
    ry, rh = oracle.ffn_forward(g, sg, u, su, d, sd, x, F)
    y, h = ops.ffn_forward(dev(g), sg, dev(u), su, dev(d), sd, dev(x), F, path="generic")
    assert np.array_equal(h.cpu().numpy(), rh) and np.array_equal(y.cpu().numpy(), ry)


# ---- operator and backend mirrors --------------------------------------------------------------------------------

def test_bitlinear_operator_mirror():
    cfg = BitLinearConfig(in_features=512, out_features=1536)          # test_task_2_1_18...rs:69-110
    layer = BitLinear(cfg, "test_layer", seed=3)
    x = torch.randn(2, 16, 512, device="cuda")
    y = layer.forward(x)
    assert tuple(y.shape) == (2, 16, 1536) and torch.isfinite(y).all()
    assert layer.cache_misses == 1
    layer.forward(x)
    assert layer.cache_hits == 1                                        # layer.rs:236-294
    t, scale = oracle.absmean_quantize_weights(layer._weights.numpy())
    ref = oracle.bitlinear_forward(oracle.pack_ternary(t)[0], scale, x.reshape(-1, 512).cpu().numpy(), 1536)["y"]
    np.testing.assert_allclose(y.reshape(-1, 1536).cpu().numpy(), ref, rtol=RTOL, atol=1e-30)
    layer.update_weights(torch.zeros(1536, 512))                        # layer.rs:299-326
    assert not layer.forward(x).any().item() and layer.cache_misses == 2
    with pytest.raises(ShapeMismatch):
        layer.forward(torch.randn(2, 16, 500, device="cuda"))           # forward.rs:63-76


def test_feed_forward_network_mirror():
    H, F, M = 128, 320, 4
    z = np.load(GOLDEN / "ffn_m4_h128_f320.npz")
    ffn = FeedForwardNetwork(H, F, BitLinearLayer(H, F, packed=z["gate"], scale=float(z["s_gate"])),
                             BitLinearLayer(H, F, packed=z["up"], scale=float(z["s_up"])),
                             BitLinearLayer(F, H, packed=z["down"], scale=float(z["s_down"])))
    y = ffn.forward(dev(z["x"]).reshape(2, 2, H))
    assert np.array_equal(y.reshape(M, H).cpu().numpy(), z["y"])
    assert not BitLinearLayer(64, 16).forward(torch.randn(3, 64, device="cuda")).any().item()   # zero-init weights


def test_cuda_backend_mirror():
    b = cuda.CudaBackend(cuda.CudaBackendConfig(memory_pool_size=256 << 20, num_streams=2))
    m, k = 512, 2048
    wp = oracle.gen_ternary_packed(4, 1, m * k)
    a = np.random.default_rng(0).integers(-127, 128, size=k, dtype=np.int8)
    dw, da, out = dev(wp), dev(a), torch.zeros(m, dtype=torch.int32, device="cuda")
    b.w2a8_gemv(dw, da, out, m, k, 1)
    b.synchronize()
    assert np.array_equal(out.cpu().numpy(), oracle.w2a8_gemv(wp, a, m))
    with pytest.raises(cuda.IncompatibleShapes):                        # backend.rs:226-254
        b.w2a8_gemv(dw[:-1], da, out, m, k, 0)
    with pytest.raises(cuda.IncompatibleShapes):
        b.w2a8_gemv(dw, da[:-1], out, m, k, 0)
    with pytest.raises(cuda.IncompatibleShapes):
        b.w2a8_gemv(dw, da, out[:-1], m, k, 0)
    with pytest.raises(cuda.InvalidConfig):                             # backend.rs:112-117
        b.w2a8_gemv(dw, da, out, m, k, 2)
    st = b.get_performance_stats()
    assert st.total_w2a8_operations == 1 and st.average_execution_time_us > 0
    mm = b.memory_manager()
    p = mm.allocate(1 << 20)
    assert mm.utilization_percent() == pytest.approx(100.0 / 256, rel=1e-3)
    with pytest.raises(cuda.MemoryAllocation) as e:                     # memory.rs:83-89
        mm.allocate(256 << 20)
    assert e.value.is_recoverable()
    mm.free(p)
    host = np.arange(1000, dtype=np.float32)
    p = mm.copy_to_device(host)
    back = np.empty_like(host)
    mm.copy_to_host(p, back)
    assert np.array_equal(host, back)
    mm.free(p)
    with pytest.raises(cuda.InvalidConfig):
        cuda.CudaBackend(cuda.CudaBackendConfig(w2a8_config=cuda.W2A8GemvConfig(block_size=100)))
    with pytest.raises(cuda.DeviceError):
        cuda.CudaBackend(cuda.CudaBackendConfig(device_id=99))
    b.close()


@pytest.mark.parametrize("M,K,N", [(1, 2560, 2560), (8, 2560, 6912), (3, 37, 29)])
def test_backend_host_forward(M, K, N):
    b = cuda.initialize()
    wp, ws, x = case(300 + M, M, K, N)
    w = b.upload_packed(wp, N, K, ws)
    y = b.bitlinear_forward_host(w, x)
    assert np.array_equal(y, oracle.bitlinear_forward(wp, ws, x, N)["y"])
    t = oracle.unpack_ternary(wp, N * K).reshape(N, K)
    w2 = b.upload_ternary(t, ws)
    assert np.array_equal(b.bitlinear_forward_host(w2, x), y)
    w.free(); w2.free(); b.close()


def test_backend_host_ffn():
    z = np.load(GOLDEN / "ffn_m4_h128_f320.npz")
    H, F = int(z["hidden"]), int(z["ffn"])
    b = cuda.initialize()
    g, u, d = (b.upload_packed(z[k], n, kk, float(z[s])) for k, n, kk, s in
               (("gate", F, H, "s_gate"), ("up", F, H, "s_up"), ("down", H, F, "s_down")))
    assert np.array_equal(b.ffn_forward_host(g, u, d, z["x"]), z["y"])
    b.close()


# ---- full-size properties -------------------------------------------------------------------------------------

@pytest.mark.parametrize("M", [1, 16, 64, 256])
def test_oversized_layer_checksum_and_row_samples(M):
    # K=8192, N=28672 is too large for the oracle in seconds: check a size-independent identity
    # (sum_n acc[m,n] == q[m,:] . colsum(W)) with torch integer ops, and compare sampled row
    # ranges against the oracle exactly.
    K, N = 8192, 28672
    wp = oracle.gen_ternary_packed(0, 50, N * K)
    x = oracle.gen_activations(0, 51, (M, K))
    ws = oracle.gen_weight_scale(0, 50, K)
    dwp = dev(wp)
    y, dbg = ops.bitlinear_forward(dwp, ws, dev(x), N, debug=True)
    w = ops.unpack_ternary(dwp, N * K).reshape(N, K)
    colsum = w.sum(dim=0, dtype=torch.float64)      # |values| stay far below 2^53: exact in fp64
    assert torch.equal(dbg["acc"].sum(dim=1, dtype=torch.float64), dbg["q"].to(torch.float64) @ colsum)
    yn = y.cpu().numpy()
    for r0 in (0, 12345, N - 64):
        sl = wp[r0 * K // 4:(r0 + 64) * K // 4]
        ref = oracle.bitlinear_forward(sl, ws, x, 64)
        assert np.array_equal(dbg["acc"][:, r0:r0 + 64].cpu().numpy(), ref["acc"])
        np.testing.assert_allclose(yn[:, r0:r0 + 64], ref["y"], rtol=RTOL, atol=0)


def test_linearity_of_the_integer_path():
    # acc is linear in W's rows: a matrix whose second half repeats the first gives repeated outputs,
    # and negating every weight (code 0 <-> 2) negates the accumulators
    M, K, N = 8, 2560, 512
    wp, ws, x = case(77, M, K, N)
    w = oracle.unpack_ternary(wp, N * K).reshape(N, K)
    both = np.concatenate([w, -w], axis=0)
    p2, _ = oracle.pack_ternary(both)
    _, dbg = ops.bitlinear_forward(dev(p2), ws, dev(x), 2 * N, debug=True)
    acc = dbg["acc"].cpu().numpy()
    assert np.array_equal(acc[:, :N], -acc[:, N:])


def test_prepare_weights_hook():
    # canonical layout is the prepared layout: code 3 removed in place, fast-path mask reported
    wp = np.full(64 * 256 // 4, 0xFF, dtype=np.uint8)          # every code is 3
    t = dev(wp)
    n, paths = ops.prepare_weights(t, 64, 256)
    assert n == 64 * 256 and paths == {"decode": True, "prefill": True}
    assert np.array_equal(t.cpu().numpy(), np.full_like(wp, 0x55))
    n2, paths2 = ops.prepare_weights(dev(np.zeros(3 * 100 // 4, dtype=np.uint8)), 3, 100)
    assert n2 == 0 and paths2 == {"decode": False, "prefill": False}       # K % 64 != 0: generic kernel only
    with pytest.raises(Exception):
        ops.prepare_weights(t, 64, 256, layout_id=1)


def test_backend_host_ffn_async_streams():
    # asynchronous host-buffer calls spread over the backend's streams, joined by synchronize()
    hidden, ffn = 256, 640
    b = cuda.CudaBackend(cuda.CudaBackendConfig(num_streams=3))
    try:
        layers = []
        for l in range(5):
            packs = [oracle.gen_ternary_packed(7, 10 * l + i, ffn * hidden) for i in range(3)]
            scales = [oracle.gen_weight_scale(7, 10 * l + i, k) for i, k in ((0, hidden), (1, hidden), (2, ffn))]
            layers.append((packs, scales, (b.upload_packed(packs[0], ffn, hidden, scales[0]), b.upload_packed(packs[1], ffn, hidden, scales[1]),
                                           b.upload_packed(packs[2], hidden, ffn, scales[2]))))
        xs = [oracle.gen_activations(7, 100 + i, (1 + i % 4, hidden)) for i in range(12)]
        outs = [np.full((x.shape[0], hidden), np.nan, dtype=np.float32) for x in xs]
        for i, x in enumerate(xs):           # more calls than streams: a stream delivers its pending result before it is reused
            g, u, d = layers[i % 5][2]
            b.ffn_forward_host_async(g, u, d, x, outs[i], stream_idx=i % 3)
        b.synchronize()
        for i, x in enumerate(xs):
            packs, scales, _ = layers[i % 5]
            ref, _ = oracle.ffn_forward(packs[0], scales[0], packs[1], scales[1], packs[2], scales[2], x, ffn)
            assert np.array_equal(outs[i], ref), i
        # a synchronous call after asynchronous ones on the same stream
        g, u, d = layers[0][2]
        b.ffn_forward_host_async(g, u, d, xs[0], outs[0], stream_idx=0)
        y = b.ffn_forward_host(g, u, d, xs[1], stream_idx=0)
        packs, scales, _ = layers[0]
        assert np.array_equal(y, oracle.ffn_forward(packs[0], scales[0], packs[1], scales[1], packs[2], scales[2], xs[1], ffn)[0])
        assert np.array_equal(outs[0], oracle.ffn_forward(packs[0], scales[0], packs[1], scales[1], packs[2], scales[2], xs[0], ffn)[0])
    finally:
        b.close()


@pytest.mark.parametrize("shape", [(64, 128), (2560, 640), (37, 29), (1, 5), (700, 2561)])
def test_device_absmean_quantise_and_pack(shape):
    # weights.rs:807-857 + packing.rs:352-388 on the device: ternary codes exact, scale to fp32 rounding of double sums
    rng = np.random.default_rng(shape[0])
    w = rng.standard_normal(shape).astype(np.float32)
    w[0, 0] = 0.0
    packed, scale = ops.quantize_pack_weights(dev(w))
    t, ref_scale = oracle.absmean_quantize_weights(w)
    assert np.array_equal(packed.cpu().numpy(), oracle.pack_ternary(t.reshape(-1))[0])
    assert scale == pytest.approx(ref_scale, rel=1e-6)
    zero, s0 = ops.quantize_pack_weights(torch.zeros(8, 16, device="cuda"))          # all-zero weights: every code 1, scale 1
    assert s0 == 1.0 and bool((zero == 0x55).all())


def test_backend_ingests_full_precision_and_gguf_tensors():
    import struct
    N, K, M = 640, 2560, 4
    b = cuda.initialize()
    try:
        w = np.random.default_rng(2).standard_normal((N, K)).astype(np.float32)
        x = oracle.gen_activations(21, 1, (M, K))
        dw = b.upload_f32(w)
        t, ref_scale = oracle.absmean_quantize_weights(w)
        assert dw.scale == pytest.approx(ref_scale, rel=1e-6)
        ref = oracle.bitlinear_forward(oracle.pack_ternary(t.reshape(-1))[0], dw.scale, x, N)["y"]
        assert np.array_equal(b.bitlinear_forward_host(dw, x), ref)
        # gguf.rs:1089-1165: scale and offset as little-endian f32, then the codes; code 3 reads as weight 0
        wp = oracle.gen_ternary_packed(21, 2, N * K).copy()
        wp[::97] |= 0x03
        tensor = struct.pack("<ff", 0.0375, -1.5) + wp.tobytes()
        dg, offset = b.upload_gguf_ternary(tensor, N, K)
        assert dg.scale == np.float32(0.0375) and offset == -1.5
        clean = wp.copy()
        clean[::97] = (clean[::97] & 0xFC) | 0x01
        assert np.array_equal(b.bitlinear_forward_host(dg, x), oracle.bitlinear_forward(clean, float(np.float32(0.0375)), x, N)["y"])
        with pytest.raises(cuda.IncompatibleShapes):
            b.upload_gguf_ternary(tensor[:100], N, K)
    finally:
        b.close()


@pytest.mark.parametrize("n_lanes", [1, 3])
def test_backend_ffn_plan_replays_a_batch(n_lanes):
    # a fixed batch of FFN blocks bound to host buffers (some page-locked, some not), replayed twice
    # with refreshed inputs; every result equals the oracle's
    hidden, ffn = 256, 640
    b = cuda.CudaBackend(cuda.CudaBackendConfig(num_streams=2))
    try:
        layers = []
        for l in range(3):
            packs = [oracle.gen_ternary_packed(17, 10 * l + i, ffn * hidden) for i in range(3)]
            scales = [oracle.gen_weight_scale(17, 10 * l + i, k) for i, k in ((0, hidden), (1, hidden), (2, ffn))]
            layers.append((packs, scales, (b.upload_packed(packs[0], ffn, hidden, scales[0]), b.upload_packed(packs[1], ffn, hidden, scales[1]),
                                           b.upload_packed(packs[2], hidden, ffn, scales[2]))))
        Ms = [1, 4, 8, 2, 1, 16, 5]
        xs = [np.zeros((M, hidden), dtype=np.float32) for M in Ms]
        ys = [np.full((M, hidden), np.nan, dtype=np.float32) for M in Ms]
        for i in (0, 2, 5):
            b.pin_host(xs[i]); b.pin_host(ys[i])
        plan = b.ffn_plan([(*layers[i % 3][2], xs[i], ys[i]) for i in range(len(Ms))], n_lanes=n_lanes)
        for rnd in range(2):
            for i, M in enumerate(Ms):
                xs[i][...] = oracle.gen_activations(17, 100 + 10 * rnd + i, (M, hidden))
            plan.run()
            for i in range(len(Ms)):
                packs, scales, _ = layers[i % 3]
                ref, _ = oracle.ffn_forward(packs[0], scales[0], packs[1], scales[1], packs[2], scales[2], xs[i], ffn)
                assert np.array_equal(ys[i], ref), (rnd, i)
        plan.close()
        for i in (0, 2, 5):
            b.unpin_host(xs[i]); b.unpin_host(ys[i])
        assert ops.device_error_flags() == 0
    finally:
        b.close()


@pytest.mark.parametrize("token_counts", [[1 + (i * 3) % 8 for i in range(75)],      # three groups of 25 calls
                                          [4, 20, 1, 8]])                              # 20 tokens: per-call launches
def test_backend_ffn_plan_grouped_and_per_call_forms(token_counts):
    hidden, ffn = 128, 192
    b = cuda.CudaBackend(cuda.CudaBackendConfig(num_streams=2))
    try:
        packs = [oracle.gen_ternary_packed(19, i, ffn * hidden) for i in range(3)]
        scales = [oracle.gen_weight_scale(19, i, k) for i, k in ((0, hidden), (1, hidden), (2, ffn))]
        w = (b.upload_packed(packs[0], ffn, hidden, scales[0]), b.upload_packed(packs[1], ffn, hidden, scales[1]),
             b.upload_packed(packs[2], hidden, ffn, scales[2]))
        xs = [oracle.gen_activations(19, 50 + i, (M, hidden)) for i, M in enumerate(token_counts)]
        ys = [np.full((M, hidden), np.nan, dtype=np.float32) for M in token_counts]
        plan = b.ffn_plan([(*w, xs[i], ys[i]) for i in range(len(token_counts))], n_lanes=4)
        plan.run()
        for i in range(len(token_counts)):
            ref, _ = oracle.ffn_forward(packs[0], scales[0], packs[1], scales[1], packs[2], scales[2], xs[i], ffn)
            assert np.array_equal(ys[i], ref), i
        plan.close()
        assert ops.device_error_flags() == 0
    finally:
        b.close()


@pytest.mark.parametrize("M,K,N", [(1, 2560, 6912), (4, 6912, 2560), (8, 2560, 6912), (3, 320, 129), (16, 1024, 144), (1, 8192, 3584)])
def test_decode_throughput_flag_same_bits(M, K, N):
    # the small-CTA plan (four consumer warps) gives the same bits as the default plan
    wp, ws, x = case(11, M, K, N)
    y0, d0 = ops.bitlinear_forward(dev(wp), ws, dev(x), N, debug=True, path="decode")
    y1, d1 = ops.bitlinear_forward(dev(wp), ws, dev(x), N, debug=True, path="decode", throughput=True)
    assert torch.equal(y0, y1) and torch.equal(d0["acc"], d1["acc"]) and torch.equal(d0["q"], d1["q"])
    assert_parity(d1, y1, oracle.bitlinear_forward(wp, ws, x, N), M, N)


def test_ffn_throughput_flag_same_bits():
    z = np.load(GOLDEN / "ffn_m4_h128_f320.npz")
    H, F = int(z["hidden"]), int(z["ffn"])
    y, _ = ops.ffn_forward(dev(z["gate"]), float(z["s_gate"]), dev(z["up"]), float(z["s_up"]), dev(z["down"]), float(z["s_down"]),
                           dev(z["x"]), F, throughput=True)
    assert np.array_equal(y.cpu().numpy(), z["y"])
    for M in (1, 4, 8):
        wg, sg, x = case(12, M, 2560, 6912)
        wu, su, _ = case(13, M, 2560, 6912)
        wd, sd, _ = case(14, M, 6912, 2560)
        a, _ = ops.ffn_forward(dev(wg), sg, dev(wu), su, dev(wd), sd, dev(x), 6912)
        b, _ = ops.ffn_forward(dev(wg), sg, dev(wu), su, dev(wd), sd, dev(x), 6912, throughput=True)
        assert torch.equal(a, b)
